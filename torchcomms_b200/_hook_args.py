"""Typed per-operation views of the native hook record.

A pre-hook callback is called as ``cb(OpName, op_id, args)`` and a post-hook
callback as ``cb(op_id, args)``; ``args`` is one of the classes below, named
and shaped after ``comms/torchcomms/_comms.pyi:67-267`` in the reference
(``AllReducePreHookArgs.tensor``, ``AllGatherPreHookArgs.input/.output`` ...).
"""
from __future__ import annotations

from typing import Any, Callable, Dict, Tuple

from ._comms import OpName

__all__ = ["CollectivePostHookArgs", "PreHookArgs", "PostHookArgs"]


class _ArgsBase:
    __slots__ = ("_record",)

    def __init__(self, record: Any) -> None:
        self._record = record

    @property
    def record(self) -> Any:
        """The untyped native record (all fields of every operation)."""
        return self._record

    def __repr__(self) -> str:
        fields = ", ".join(f"{n}=..." for n in getattr(self, "_fields", ()))
        return f"{type(self).__name__}({fields})"


class CollectivePostHookArgs(_ArgsBase):
    """Post-hook view: the operation's work handle (``None`` once it died)."""

    __slots__ = ()

    @property
    def work(self) -> Any:
        return self._record.work


def _first(seq):
    return seq[0] if len(seq) else None


# field name -> extractor from the native record
_GETTERS: Dict[str, Callable[[Any], Any]] = {
    "tensor": lambda r: _first(r.inputs) if len(r.inputs) else _first(r.outputs),
    "input": lambda r: _first(r.inputs),
    "output": lambda r: _first(r.outputs),
    "input_list": lambda r: list(r.inputs),
    "output_list": lambda r: list(r.outputs),
    "peer": lambda r: r.root,
    "root": lambda r: r.root,
    "async_op": lambda r: r.async_op,
    "op": lambda r: r.red_op,
    "input_split_sizes": lambda r: list(r.in_splits),
    "output_split_sizes": lambda r: list(r.out_splits),
    "ops": lambda r: list(r.p2p_ops),
    "ranks": lambda r: list(r.ranks),
    "name": lambda r: r.name,
}

# op name -> (class prefix, pre-hook fields, field aliases)
_SPEC: Dict[str, Tuple[str, Tuple[str, ...], Dict[str, str]]] = {
    "send": ("Send", ("tensor", "peer", "async_op"), {}),
    "recv": ("Recv", ("tensor", "peer", "async_op"), {}),
    "broadcast": ("Broadcast", ("tensor", "root", "async_op"), {}),
    "all_reduce": ("AllReduce", ("tensor", "op", "async_op"), {}),
    "reduce": ("Reduce", ("tensor", "root", "op", "async_op"), {}),
    "all_gather": ("AllGather", ("input", "output", "async_op"), {"output": "output_list"}),
    "all_gather_v": ("AllGatherV", ("input", "output", "async_op"), {"output": "output_list"}),
    "all_gather_single": ("AllGatherSingle", ("input", "output", "async_op"), {}),
    "reduce_scatter": ("ReduceScatter", ("input", "output", "op", "async_op"), {"input": "input_list"}),
    "reduce_scatter_v": ("ReduceScatterV", ("input", "output", "op", "async_op"), {"input": "input_list"}),
    "reduce_scatter_single": ("ReduceScatterSingle", ("input", "output", "op", "async_op"), {}),
    "all_to_all_single": ("AllToAllSingle", ("input", "output", "async_op"), {}),
    "all_to_all_v_single": (
        "AllToAllVSingle",
        ("input", "output", "input_split_sizes", "output_split_sizes", "async_op"),
        {},
    ),
    "all_to_all": ("AllToAll", ("input", "output", "async_op"), {"input": "input_list", "output": "output_list"}),
    "barrier": ("Barrier", ("async_op",), {}),
    "scatter": ("Scatter", ("output", "input", "root", "async_op"), {"input": "input_list"}),
    "gather": ("Gather", ("input", "output", "root", "async_op"), {"output": "output_list"}),
    "gather_single": ("GatherSingle", ("input", "output", "root", "async_op"), {}),
    "split": ("Split", ("ranks", "name"), {}),
    "new_window": ("NewWindow", (), {}),
    "batch_op_issue": ("BatchOpIssue", ("ops", "async_op"), {}),
    "finalize": ("Finalize", (), {}),
}

_PRE: Dict[Any, type] = {}
_POST: Dict[Any, type] = {}


def _make_property(getter: Callable[[Any], Any]) -> property:
    return property(lambda self: getter(self._record))


for _opname, (_prefix, _fields, _alias) in _SPEC.items():
    _ns: Dict[str, Any] = {"__slots__": (), "_fields": _fields}
    for _f in _fields:
        _ns[_f] = _make_property(_GETTERS[_alias.get(_f, _f)])
    _pre_cls = type(f"{_prefix}PreHookArgs", (_ArgsBase,), _ns)
    _post_base = _ArgsBase if _opname in ("split", "new_window", "finalize") else CollectivePostHookArgs
    _post_cls = type(f"{_prefix}PostHookArgs", (_post_base,), {"__slots__": ()})
    globals()[_pre_cls.__name__] = _pre_cls
    globals()[_post_cls.__name__] = _post_cls
    __all__ += [_pre_cls.__name__, _post_cls.__name__]
    _PRE[getattr(OpName, _opname)] = _pre_cls
    _POST[getattr(OpName, _opname)] = _post_cls

PreHookArgs = tuple(_PRE.values())
PostHookArgs = tuple(_POST.values())


def _to_pre_args(record: Any) -> Any:
    return _PRE[record.op](record)


def _to_post_args(record: Any) -> Any:
    return _POST[record.op](record)
