"""Pre-hook that refuses to start a collective on tensors containing NaN.

A NaN that enters an all-reduce poisons every rank's copy; catching it at the
call site names the rank and the operation that produced it.  The check runs
on the caller's stream before the collective is enqueued.  On CUDA it is one
fused ``isnan().any()`` reduction per tensor followed by a host read, so it is
a debugging aid, not something to leave on in production.

Parity: comms/torchcomms/hooks/nan_check/nan_check.py:117-185 (the reference
calls ``torch.ops.c10d.check_for_nan``; that op exists only for NCCL builds of
c10d, so this implementation uses it when present and plain tensor ops
otherwise).
"""
from __future__ import annotations

from typing import Any, List

import torch

from .._comms import OpName

_IN_PLACE = {OpName.broadcast, OpName.all_reduce, OpName.reduce}
_SINGLE_SINGLE = {OpName.all_gather_single, OpName.reduce_scatter_single, OpName.all_to_all_single,
                  OpName.all_to_all_v_single, OpName.gather_single}
_SINGLE_LIST = {OpName.all_gather, OpName.all_gather_v, OpName.gather}
_LIST_SINGLE = {OpName.reduce_scatter, OpName.reduce_scatter_v, OpName.scatter}
_LIST_LIST = {OpName.all_to_all}


def _has_nan(t: torch.Tensor) -> bool:
    if not isinstance(t, torch.Tensor) or not t.is_floating_point() or t.numel() == 0:
        return False
    if t.dtype in (torch.float8_e4m3fn, torch.float8_e5m2):
        t = t.to(torch.bfloat16)
    return bool(torch.isnan(t).any())


def _check(tensors: Any, label: str, op: str, comm: str) -> None:
    if tensors is None:
        return
    if isinstance(tensors, torch.Tensor):
        tensors = [tensors]
    for i, t in enumerate(tensors):
        if _has_nan(t):
            raise RuntimeError(f"NaN detected in {label} tensor {i} for '{op}' on comm '{comm}'")


class NanCheckHook:
    def __init__(self, check_inputs: bool = True, check_outputs: bool = False):
        self._check_inputs = check_inputs
        self._check_outputs = check_outputs
        self._handles: List[Any] = []

    def register_with_comm(self, comm: Any) -> None:
        name = comm.get_name() if hasattr(comm, "get_name") else "?"

        def pre(op: OpName, op_id: int, args: Any) -> None:
            s = op.name
            if op == OpName.send:
                if self._check_inputs:
                    _check(args.tensor, "input", s, name)
            elif op == OpName.recv:
                if self._check_outputs:
                    _check(args.tensor, "output", s, name)
            elif op in _IN_PLACE:
                if self._check_inputs or self._check_outputs:
                    _check(args.tensor, "input", s, name)
            elif op in _SINGLE_SINGLE or op in _SINGLE_LIST or op in _LIST_SINGLE or op in _LIST_LIST:
                if self._check_inputs:
                    _check(args.input, "input", s, name)
                if self._check_outputs:
                    _check(args.output, "output", s, name)

        self._handles.append(comm.register_pre_hook(pre))

    def unregister(self) -> None:
        for h in self._handles:
            h.remove()
        self._handles.clear()

    def is_enabled(self) -> bool:
        return bool(self._handles)
