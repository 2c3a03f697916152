"""Pre-hook that refuses to start a collective on tensors containing NaN.

A NaN that enters an all-reduce poisons every rank's copy; catching it at the
call site names the rank and the operation that produced it.  The check runs
on the caller's stream before the collective is enqueued.  On CUDA it is one
fused ``isnan().any()`` reduction per tensor followed by a host read, so it is
a debugging aid, not something to leave on in production.

Parity: comms/torchcomms/hooks/nan_check/nan_check.py:117-185 (the reference
calls ``torch.ops.c10d.check_for_nan``; that op exists only for NCCL builds of
c10d, so this implementation uses plain tensor ops).
"""
from __future__ import annotations

from typing import Any, Dict, Iterable, List, Optional, Tuple

import torch

from .._comms import OpName

# operation -> (attribute holding what is read, attribute holding what is written);
# an attribute may be one tensor or a list of tensors.  In-place operations read
# and write ``tensor``; receive-only operations have nothing to read.
_TENSOR_FIELDS: Dict[OpName, Tuple[Optional[str], Optional[str]]] = {
    OpName.send: ("tensor", None),
    OpName.recv: (None, "tensor"),
    OpName.broadcast: ("tensor", None),
    OpName.all_reduce: ("tensor", None),
    OpName.reduce: ("tensor", None),
}
for _op in (OpName.all_gather_single, OpName.reduce_scatter_single, OpName.all_to_all_single, OpName.all_to_all_v_single,
            OpName.gather_single, OpName.all_gather, OpName.all_gather_v, OpName.gather, OpName.reduce_scatter,
            OpName.reduce_scatter_v, OpName.scatter, OpName.all_to_all):
    _TENSOR_FIELDS[_op] = ("input", "output")


def _tensors(value: Any) -> Iterable[torch.Tensor]:
    if value is None:
        return ()
    if isinstance(value, torch.Tensor):
        return (value,)
    return tuple(t for t in value if isinstance(t, torch.Tensor))


def _has_nan(t: torch.Tensor) -> bool:
    if not t.is_floating_point() or t.numel() == 0:
        return False
    if t.dtype in (torch.float8_e4m3fn, torch.float8_e5m2):
        t = t.to(torch.bfloat16)
    return bool(torch.isnan(t).any())


class NanCheckHook:
    """``NanCheckHook(check_inputs=True, check_outputs=False).register_with_comm(comm)``."""

    def __init__(self, check_inputs: bool = True, check_outputs: bool = False):
        self._sides = (check_inputs, check_outputs)
        self._handles: List[Any] = []

    def register_with_comm(self, comm: Any) -> None:
        comm_name = comm.get_name() if hasattr(comm, "get_name") else "?"

        def inspect(op: OpName, op_id: int, args: Any) -> None:
            fields = _TENSOR_FIELDS.get(op)
            if fields is None:
                return
            for label, attr, enabled in zip(("input", "output"), fields, self._sides):
                if not enabled or attr is None:
                    continue
                for index, t in enumerate(_tensors(getattr(args, attr, None))):
                    if _has_nan(t):
                        raise RuntimeError(
                            f"NaN detected in {label} tensor {index} for '{op.name}' on comm '{comm_name}' (op id {op_id})")

        self._handles.append(comm.register_pre_hook(inspect))

    def unregister(self) -> None:
        while self._handles:
            self._handles.pop().remove()

    def is_enabled(self) -> bool:
        return bool(self._handles)
