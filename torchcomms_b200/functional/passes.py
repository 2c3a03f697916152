"""FX graph passes for graphs that contain ``torch.ops.torchcomms_b200`` collectives.

``reinplace_pass``    rewrites ``y = all_reduce(x)`` / ``y = broadcast(x)`` (which copy ``x`` first)
                      into the in-place operators when nothing else reads ``x`` afterwards and ``x``
                      is produced inside the graph - one copy of the payload less per collective.
``strip_wait_pass``   removes ``wait_tensor`` nodes behind the synchronous operators: those return
                      finished tensors, so the node is a copy that only matters for graphs shared
                      with code that expects it.  Waits on the results of ``*_start`` operators stay.

Apply ``reinplace_pass`` first.  Both mutate the GraphModule and recompile it::

    gm = make_fx(fn, tracing_mode="fake")(*example_inputs)
    strip_wait_pass(reinplace_pass(gm))

Parity: comms/torchcomms/functional/passes.py (``reinplacement_pass``, which defers to Inductor's
re-inplacing, and ``strip_with_effects_pass``; this package's operators carry no effect tokens, the
removable wrapper here is ``wait_tensor``).
"""
from __future__ import annotations

import torch
from torch import fx

from . import NAMESPACE

_ops = getattr(torch.ops, NAMESPACE)

# functional overload -> in-place overload; argument 0 is the payload in both
_INPLACE = {
    _ops.all_reduce.default: _ops.all_reduce_.default,
    _ops.broadcast.default: _ops.broadcast_.default,
}


def _graph_positions(gm: fx.GraphModule):
    return {n: i for i, n in enumerate(gm.graph.nodes)}


def reinplace_pass(gm: fx.GraphModule, example_inputs=None) -> fx.GraphModule:
    """Functional collectives whose input dies at the call become in-place collectives."""
    pos = _graph_positions(gm)
    changed = 0
    for node in list(gm.graph.nodes):
        if node.op != "call_function" or node.target not in _INPLACE:
            continue
        src = node.args[0]
        if not isinstance(src, fx.Node) or src.op in ("placeholder", "get_attr"):
            continue                      # never write into the caller's tensors or into parameters
        if src.op == "call_function" and getattr(src.target, "_schema", None) is not None and any(
                a.alias_info is not None for a in src.target._schema.returns):
            continue                      # a view of something else: writing through it is not local
        if any(pos[user] > pos[node] for user in src.users if user is not node):
            continue                      # somebody still reads the un-reduced value afterwards
        if any(user is not node and pos[user] == pos[node] for user in src.users):
            continue
        node.target = _INPLACE[node.target]
        changed += 1
    if changed:
        gm.graph.lint()
        gm.recompile()
    return gm


def _is_started(node) -> bool:
    """True for the result of a ``*_start`` operator: the one kind of tensor that is not finished when it is made."""
    name = getattr(getattr(node, "target", None), "_schema", None)
    return isinstance(node, fx.Node) and node.op == "call_function" and name is not None and name.name.endswith("_start")


def strip_wait_pass(gm: fx.GraphModule, example_inputs=None) -> fx.GraphModule:
    """``wait_tensor(x)`` -> ``x``, except where ``x`` comes from a ``*_start`` operator (that wait is the only
    thing that orders the consumer behind the collective)."""
    changed = 0
    for node in list(gm.graph.nodes):
        if node.op == "call_function" and node.target is _ops.wait_tensor.default:
            if _is_started(node.args[0]):
                continue
            node.replace_all_uses_with(node.args[0])
            gm.graph.erase_node(node)
            changed += 1
    if changed:
        gm.graph.lint()
        gm.recompile()
    return gm


def count_ops(gm: fx.GraphModule) -> dict:
    """``{operator name: occurrences}`` of this package's operators in the graph (for tests and logs)."""
    out: dict = {}
    for node in gm.graph.nodes:
        if node.op == "call_function" and getattr(node.target, "namespace", None) == NAMESPACE:
            name = node.target._schema.name.split("::")[-1]
            out[name] = out.get(name, 0) + 1
    return out


# The reference's names (comms/torchcomms/functional/passes.py). Its second pass unwraps effect tokens, which the
# operators of this package do not carry; the wrapper that can be removed here is ``wait_tensor``.
reinplacement_pass = reinplace_pass
strip_with_effects_pass = strip_wait_pass

__all__ = ["reinplace_pass", "strip_wait_pass", "count_ops", "reinplacement_pass", "strip_with_effects_pass"]
