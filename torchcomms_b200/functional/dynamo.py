"""``torch.compile`` support for code that holds a ``TorchComm`` itself.

The traceable operators of this package take a communicator's *name*; code
written against the eager API calls methods of the communicator object, which
is a C++ object the tracer cannot look into.  After ``register_with_dynamo()``
the same code compiles with ``fullgraph=True``::

    from torchcomms_b200.functional.dynamo import register_with_dynamo
    register_with_dynamo()                     # once per process
    comm = torchcomms_b200.new_comm("b200", device, name="dp")

    @torch.compile(fullgraph=True)
    def step(x):
        comm.all_reduce(x, ReduceOp.SUM, False)            # recorded as torchcomms_b200::all_reduce + copy_
        work = comm.all_gather_single(out, x, True)        # ..._start now, wait_tensor at work.wait()
        ...
        work.wait()
        return out * comm.get_rank()                        # a constant of the graph

How: the bound class gets Python methods in front of its C++ ones.  Outside a
compiled region they call straight through.  Inside, the tracer inlines them
(they are plain Python), finds the communicator's traceable stand-in through
``id(comm)`` (which the tracer evaluates and guards on), and records the
functional operator followed by a ``copy_`` into the tensor the eager call
would have written; functionalisation turns that into data flow.  Reduce
operations are recognised the same way, by the identity of ``ReduceOp.SUM``
and friends.  Nothing inside the tracer is patched.

Counterpart in the reference: comms/torchcomms/functional/dynamo.py, which
registers the communicator as an opaque script object and replaces the tracer's
handling of its method calls (``TorchCommMethodVariable``); the effect for user
code - communicator methods usable in compiled regions, rank and size folded
to constants - is the same.
"""
from __future__ import annotations

import weakref
from typing import Dict, List, Optional, Sequence

import torch
from torch import Tensor

from .. import ReduceOp, TorchComm
from . import NAMESPACE

_ops = getattr(torch.ops, NAMESPACE)


class _Traceable:
    """What a compiled region knows of a communicator: three constants."""

    def __init__(self, comm: TorchComm, orig):
        self.name = _name_of(comm, orig)
        self.rank = orig["get_rank"](comm)
        self.size = orig["get_size"](comm)


def _name_of(comm: TorchComm, orig) -> str:
    from . import _comms as registry

    key = orig["get_name"](comm)
    registry.setdefault(key, comm)
    return key


_BY_ID: Dict[int, _Traceable] = {}
_REDUCE_BY_ID: Dict[int, str] = {}
_ORIG: Dict[str, object] = {}


class TracedCommWork:
    """Work handle of a communicator method called inside a compiled region.

    Synchronous calls are complete when they return.  For ``async_op=True`` the
    graph holds the started collective; ``wait()`` records ``wait_tensor`` and
    the copy into the caller's output."""

    def __init__(self, dsts: Optional[List[Tensor]] = None, pending: Optional[List[Tensor]] = None):
        self.dsts = dsts
        self.pending = pending

    def wait(self) -> bool:
        if self.pending is not None:
            for dst, src in zip(self.dsts, self.pending):
                dst.copy_(_ops.wait_tensor(src).view(dst.shape))
            self.pending = None
            self.dsts = None
        return True

    def is_completed(self) -> bool:
        return self.pending is None


def enable(comm: TorchComm) -> TorchComm:
    """Makes ``comm`` usable inside compiled regions (communicators created after
    ``register_with_dynamo()`` are enabled when they are created)."""
    orig = _ORIG if _ORIG else {n: getattr(TorchComm, n) for n in ("get_name", "get_rank", "get_size")}
    key = id(comm)
    if key not in _BY_ID:
        # The entry goes when the object does, so that a later object at the same address is not mistaken for it.
        weakref.finalize(comm, _BY_ID.pop, key, None)
    _BY_ID[key] = _Traceable(comm, orig)
    return comm


def _traceable(comm) -> _Traceable:
    # Evaluated by the tracer: id() of a Python object is a guarded constant there.
    return _BY_ID[id(comm)]


def _red(op) -> str:
    if isinstance(op, str):
        return op
    return _REDUCE_BY_ID[id(op)]


def register_reduce_op(op: ReduceOp, name: str) -> None:
    """Lets compiled regions recognise a reduce operation object other than the predefined ones
    (``name``: one of the operators' reduce names)."""
    _REDUCE_BY_ID[id(op)] = name


def _finish(dsts: Sequence[Tensor], results: Sequence[Tensor], async_op: bool, started: bool) -> TracedCommWork:
    if async_op and started:
        return TracedCommWork(list(dsts), list(results))
    for dst, src in zip(dsts, results):
        dst.copy_(src.view(dst.shape))
    return TracedCommWork()


# One function per communicator method.  Signatures follow the bound methods
# (tensor arguments, async_op, hints, timeout); hints and timeouts are per-call
# tuning of the eager path and are not recorded in the graph.


def _m_get_rank(self):
    if torch.compiler.is_compiling():
        return _traceable(self).rank
    return _ORIG["get_rank"](self)


def _m_get_size(self):
    if torch.compiler.is_compiling():
        return _traceable(self).size
    return _ORIG["get_size"](self)


def _m_get_name(self):
    if torch.compiler.is_compiling():
        return _traceable(self).name
    return _ORIG["get_name"](self)


def _m_all_reduce(self, tensor, op, async_op, hints=None, timeout=None):
    if torch.compiler.is_compiling():
        name = _traceable(self).name
        if async_op:
            return _finish([tensor], [_ops.all_reduce_start(tensor, _red(op), name)], True, True)
        return _finish([tensor], [_ops.all_reduce(tensor, _red(op), name)], False, False)
    return _ORIG["all_reduce"](self, tensor, op, async_op, hints, timeout)


def _m_broadcast(self, tensor, root, async_op, hints=None, timeout=None):
    if torch.compiler.is_compiling():
        return _finish([tensor], [_ops.broadcast(tensor, root, _traceable(self).name)], async_op, False)
    return _ORIG["broadcast"](self, tensor, root, async_op, hints, timeout)


def _m_reduce(self, tensor, root, op, async_op, hints=None, timeout=None):
    if torch.compiler.is_compiling():
        return _finish([tensor], [_ops.reduce(tensor, root, _red(op), _traceable(self).name)], async_op, False)
    return _ORIG["reduce"](self, tensor, root, op, async_op, hints, timeout)


def _m_all_gather_single(self, output, input, async_op, hints=None, timeout=None):
    if torch.compiler.is_compiling():
        name = _traceable(self).name
        flat = input.reshape(1, -1)
        if async_op:
            return _finish([output], [_ops.all_gather_single_start(flat, name)], True, True)
        return _finish([output], [_ops.all_gather_single(flat, name)], False, False)
    return _ORIG["all_gather_single"](self, output, input, async_op, hints, timeout)


def _m_reduce_scatter_single(self, output, input, op, async_op, hints=None, timeout=None):
    if torch.compiler.is_compiling():
        t = _traceable(self)
        rows = input.reshape(t.size, -1)
        if async_op:
            return _finish([output], [_ops.reduce_scatter_single_start(rows, _red(op), t.name)], True, True)
        return _finish([output], [_ops.reduce_scatter_single(rows, _red(op), t.name)], False, False)
    return _ORIG["reduce_scatter_single"](self, output, input, op, async_op, hints, timeout)


def _m_all_to_all_single(self, output, input, async_op, hints=None, timeout=None):
    if torch.compiler.is_compiling():
        t = _traceable(self)
        rows = input.reshape(t.size, -1)
        if async_op:
            return _finish([output], [_ops.all_to_all_single_start(rows, None, None, t.name)], True, True)
        return _finish([output], [_ops.all_to_all_single(rows, None, None, t.name)], False, False)
    return _ORIG["all_to_all_single"](self, output, input, async_op, hints, timeout)


def _m_all_to_all_v_single(self, output, input, output_split_sizes, input_split_sizes, async_op, hints=None, timeout=None):
    if torch.compiler.is_compiling():
        name = _traceable(self).name
        outs, ins = list(output_split_sizes), list(input_split_sizes)
        if async_op:
            return _finish([output], [_ops.all_to_all_single_start(input, outs, ins, name)], True, True)
        return _finish([output], [_ops.all_to_all_single(input, outs, ins, name)], False, False)
    return _ORIG["all_to_all_v_single"](self, output, input, output_split_sizes, input_split_sizes, async_op, hints, timeout)


def _m_all_gather(self, tensor_list, tensor, async_op, hints=None, timeout=None):
    if torch.compiler.is_compiling():
        return _finish(tensor_list, _ops.all_gather(tensor, _traceable(self).name), async_op, False)
    return _ORIG["all_gather"](self, tensor_list, tensor, async_op, hints, timeout)


def _m_reduce_scatter(self, output, input_list, op, async_op, hints=None, timeout=None):
    if torch.compiler.is_compiling():
        return _finish([output], [_ops.reduce_scatter(list(input_list), _red(op), _traceable(self).name)], async_op, False)
    return _ORIG["reduce_scatter"](self, output, input_list, op, async_op, hints, timeout)


def _m_reduce_scatter_v(self, output, input_list, op, async_op, hints=None, timeout=None):
    if torch.compiler.is_compiling():
        return _finish([output], [_ops.reduce_scatter_v(list(input_list), _red(op), _traceable(self).name)], async_op, False)
    return _ORIG["reduce_scatter_v"](self, output, input_list, op, async_op, hints, timeout)


def _m_all_to_all(self, output_tensor_list, input_tensor_list, async_op, hints=None, timeout=None):
    if torch.compiler.is_compiling():
        return _finish(output_tensor_list, _ops.all_to_all(list(input_tensor_list), _traceable(self).name), async_op, False)
    return _ORIG["all_to_all"](self, output_tensor_list, input_tensor_list, async_op, hints, timeout)


def _m_all_gather_v(self, tensor_list, tensor, async_op, hints=None, timeout=None):
    if torch.compiler.is_compiling():
        sizes = [t.shape[0] for t in tensor_list]
        return _finish(tensor_list, _ops.all_gather_v(tensor, sizes, _traceable(self).name), async_op, False)
    return _ORIG["all_gather_v"](self, tensor_list, tensor, async_op, hints, timeout)


def _m_gather_single(self, output, input, root, async_op, hints=None, timeout=None):
    if torch.compiler.is_compiling():
        t = _traceable(self)
        gathered = _ops.gather_single(input.reshape(1, -1), root, t.name)
        if t.rank == root:                       # elsewhere the output is left alone, as in the eager call
            output.copy_(gathered.view(output.shape))
        return TracedCommWork()
    return _ORIG["gather_single"](self, output, input, root, async_op, hints, timeout)


def _m_gather(self, output_tensor_list, input_tensor, root, async_op, hints=None, timeout=None):
    if torch.compiler.is_compiling():
        t = _traceable(self)
        gathered = _ops.gather_single(input_tensor.reshape(1, -1), root, t.name)
        if t.rank == root:
            for r, dst in enumerate(output_tensor_list):
                dst.copy_(gathered[r].view(dst.shape))
        return TracedCommWork()
    return _ORIG["gather"](self, output_tensor_list, input_tensor, root, async_op, hints, timeout)


def _m_scatter(self, output_tensor, input_tensor_list, root, async_op, hints=None, timeout=None):
    if torch.compiler.is_compiling():
        t = _traceable(self)
        if t.rank == root:
            stacked = torch.cat([x.reshape(1, -1) for x in input_tensor_list], dim=0)
        else:                                    # only the shape matters off the root
            stacked = output_tensor.new_empty((t.size, output_tensor.numel()))
        return _finish([output_tensor], [_ops.scatter(stacked, root, t.name)], async_op, False)
    return _ORIG["scatter"](self, output_tensor, input_tensor_list, root, async_op, hints, timeout)


# Persistent all-gather: the handle is made outside the compiled region (it registers the output once); inside,
# exec records an all-gather into that output.
_AGP_OUT: Dict[int, Tensor] = {}


def _m_all_gather_p_init(self, output, hints=None, timeout=None):
    handle = _ORIG["all_gather_p_init"](self, output, hints, timeout)
    _AGP_OUT[id(handle)] = output
    weakref.finalize(handle, _AGP_OUT.pop, id(handle), None)
    return handle


def _m_all_gather_p_exec(self, handle, input, async_op, hints=None, timeout=None):
    if torch.compiler.is_compiling():
        out = _AGP_OUT[id(handle)]
        name = _traceable(self).name
        flat = input.reshape(1, -1)
        if async_op:
            return _finish([out], [_ops.all_gather_single_start(flat, name)], True, True)
        return _finish([out], [_ops.all_gather_single(flat, name)], False, False)
    return _ORIG["all_gather_p_exec"](self, handle, input, async_op, hints, timeout)


def _m_send(self, tensor, dst, async_op, hints=None, timeout=None):
    if torch.compiler.is_compiling():
        _ops.send(tensor, dst, _traceable(self).name)
        return TracedCommWork()
    return _ORIG["send"](self, tensor, dst, async_op, hints, timeout)


def _m_recv(self, tensor, src, async_op, hints=None, timeout=None):
    if torch.compiler.is_compiling():
        return _finish([tensor], [_ops.recv(tensor, src, _traceable(self).name)], async_op, False)
    return _ORIG["recv"](self, tensor, src, async_op, hints, timeout)


def _m_barrier(self, async_op, hints=None, timeout=None):
    if torch.compiler.is_compiling():
        _ops.barrier(torch.zeros(()), _traceable(self).name)
        return TracedCommWork()
    return _ORIG["barrier"](self, async_op, hints, timeout)


class TracedBatch:
    """What ``comm.batch_op_create()`` gives inside a compiled region: it collects the sends and receives and
    records one ``batch_send_recv`` operator at ``issue()``, followed by the copies into the receive tensors."""

    def __init__(self, name: str):
        self.name = name
        self.sends: List[Tensor] = []
        self.dsts: List[int] = []
        self.recvs: List[Tensor] = []
        self.srcs: List[int] = []

    def send(self, tensor: Tensor, dst: int) -> None:
        self.sends.append(tensor)
        self.dsts.append(dst)

    def recv(self, tensor: Tensor, src: int) -> None:
        self.recvs.append(tensor)
        self.srcs.append(src)

    def issue(self, async_op: bool = False, options=None) -> TracedCommWork:
        got = _ops.batch_send_recv(self.sends, self.dsts, self.recvs, self.srcs, self.name)
        return _finish(self.recvs, got, async_op, False)


def _m_batch_op_create(self):
    if torch.compiler.is_compiling():
        return TracedBatch(_traceable(self).name)
    return _ORIG["batch_op_create"](self)


# ------------------------------------------------------------------ windows ---
# A window object's put / signal / wait_signal have no tensor results, so nothing in the data flow keeps them in
# program order. Each enabled window carries a token: every recorded window operator takes the window's current
# token and gives the next one, and ``get_tensor()`` inside a compiled region returns the window's contents ordered
# behind the last token (``window_read``).


class _WindowState:
    def __init__(self, name: str):
        self.name = name
        self.token = torch.empty(0)


_WIN_BY_ID: Dict[int, _WindowState] = {}
_WIN_ORIG: Dict[str, object] = {}
_win_counter = [0]


def enable_window(window, name: Optional[str] = None):
    """Makes a window's methods usable inside compiled regions (windows made by ``comm.new_window()`` after
    ``register_with_dynamo()`` are enabled when they are made)."""
    from .ext import register_window

    key = id(window)
    if key in _WIN_BY_ID:
        return window
    if name is None:
        _win_counter[0] += 1
        name = f"_traced_window_{_win_counter[0]}"
    register_window(name, weakref.proxy(window))     # the registry must not keep the window (and its tensor) alive
    _WIN_BY_ID[key] = _WindowState(name)
    weakref.finalize(window, _forget_window, key, name)
    return window


def _forget_window(key: int, name: str) -> None:
    from .ext import unregister_window

    _WIN_BY_ID.pop(key, None)
    unregister_window(name)


def _w_put(self, tensor, dst_rank, target_offset_nelems, async_op, hints=None, timeout=None):
    if torch.compiler.is_compiling():
        st = _WIN_BY_ID[id(self)]
        st.token = _ops.window_put(tensor, st.name, dst_rank, target_offset_nelems, st.token)
        return TracedCommWork()
    return _WIN_ORIG["put"](self, tensor, dst_rank, target_offset_nelems, async_op, hints, timeout)


def _w_signal(self, dst_rank, async_op, hints=None, timeout=None):
    if torch.compiler.is_compiling():
        st = _WIN_BY_ID[id(self)]
        st.token = _ops.window_signal(st.name, dst_rank, st.token)
        return TracedCommWork()
    return _WIN_ORIG["signal"](self, dst_rank, async_op, hints, timeout)


def _w_wait_signal(self, peer_rank, async_op, hints=None, timeout=None):
    if torch.compiler.is_compiling():
        st = _WIN_BY_ID[id(self)]
        st.token = _ops.window_wait_signal(st.name, peer_rank, st.token)
        return TracedCommWork()
    return _WIN_ORIG["wait_signal"](self, peer_rank, async_op, hints, timeout)


def _w_get_tensor(self):
    if torch.compiler.is_compiling():
        st = _WIN_BY_ID[id(self)]
        return _ops.window_read(st.name, st.token)
    return _WIN_ORIG["get_tensor"](self)


_WINDOW_METHODS = {"put": _w_put, "signal": _w_signal, "wait_signal": _w_wait_signal, "get_tensor": _w_get_tensor}


def _m_new_window(self, tensor=None):
    return enable_window(_ORIG["new_window"](self, tensor))


def _m_finalize(self):
    from . import _comms as registry

    t = _BY_ID.pop(id(self), None)
    if t is not None and registry.get(t.name) is self:
        registry.pop(t.name, None)        # the operator registry held the communicator for the traced operators
    return _ORIG["finalize"](self)


def _m_split(self, ranks, name, hints=None, timeout=None):
    child = _ORIG["split"](self, ranks, name, hints, timeout)
    if child is not None:
        enable(child)
    return child


_METHODS = {
    "get_rank": _m_get_rank, "get_size": _m_get_size, "get_name": _m_get_name,
    "all_reduce": _m_all_reduce, "broadcast": _m_broadcast, "reduce": _m_reduce,
    "all_gather_single": _m_all_gather_single, "reduce_scatter_single": _m_reduce_scatter_single,
    "all_to_all_single": _m_all_to_all_single, "all_to_all_v_single": _m_all_to_all_v_single,
    "all_gather": _m_all_gather, "reduce_scatter": _m_reduce_scatter, "all_to_all": _m_all_to_all,
    "all_gather_v": _m_all_gather_v, "reduce_scatter_v": _m_reduce_scatter_v,
    "all_gather_p_init": _m_all_gather_p_init, "all_gather_p_exec": _m_all_gather_p_exec, "gather_single": _m_gather_single, "gather": _m_gather, "scatter": _m_scatter,
    "send": _m_send, "recv": _m_recv, "barrier": _m_barrier, "batch_op_create": _m_batch_op_create,
    "finalize": _m_finalize, "split": _m_split, "new_window": _m_new_window,
}

def is_registered() -> bool:
    return bool(_ORIG)


def register_with_dynamo() -> None:
    """Puts the traceable methods in front of the communicator's bound methods (idempotent) and
    enables every communicator the operator registry already knows."""
    if _ORIG:
        return
    import torchcomms_b200 as pkg
    from . import _comms as registry
    from . import ext  # noqa: F401  (defines the *_start, list and window operators)
    from .inductor import mark_side_effects

    for name in _METHODS:
        _ORIG[name] = getattr(TorchComm, name)
    for name, fn in _METHODS.items():
        fn.__name__ = name
        fn.__qualname__ = f"TorchComm.{name}"
        fn.__doc__ = getattr(_ORIG[name], "__doc__", None)
        setattr(TorchComm, name, fn)
    from .. import TorchCommWindow

    for name, fn in _WINDOW_METHODS.items():
        _WIN_ORIG[name] = getattr(TorchCommWindow, name)
        fn.__name__ = name
        fn.__qualname__ = f"TorchCommWindow.{name}"
        setattr(TorchCommWindow, name, fn)
    for op_name, red in (("SUM", "sum"), ("AVG", "avg"), ("MAX", "max"), ("MIN", "min"), ("PRODUCT", "product")):
        _REDUCE_BY_ID[id(getattr(ReduceOp, op_name))] = red
    mark_side_effects()     # a barrier or send whose result nobody reads stays in the graph

    # Communicators made from now on are enabled as they are made.
    made = pkg.new_comm
    _ORIG["new_comm"] = made

    def new_comm(*args, **kwargs):
        return enable(made(*args, **kwargs))

    new_comm.__doc__ = made.__doc__
    pkg.new_comm = new_comm
    for comm in list(registry.values()):
        enable(comm)


def unregister_from_dynamo() -> None:
    """Restores the bound methods (for tests)."""
    if not _ORIG:
        return
    import torchcomms_b200 as pkg

    from .. import TorchCommWindow

    pkg.new_comm = _ORIG.pop("new_comm")
    for name, fn in list(_ORIG.items()):
        setattr(TorchComm, name, fn)
    for name, fn in list(_WIN_ORIG.items()):
        setattr(TorchCommWindow, name, fn)
    _ORIG.clear()
    _WIN_ORIG.clear()
    _BY_ID.clear()
    _REDUCE_BY_ID.clear()


__all__ = ["register_with_dynamo", "unregister_from_dynamo", "is_registered", "enable", "enable_window", "register_reduce_op",
           "TracedCommWork", "TracedBatch"]
