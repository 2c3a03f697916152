"""Fully sharded data parallelism driven by a communicator.

Each stage of a model becomes a ``ShardedUnit``: its parameters live as ONE
flat fp32 shard per rank (plus AdamW moments).  Before the stage runs, the
shards are all-gathered into a flat bf16 buffer the parameters are views of -
on the CUDA backend that is one kernel that casts fp32 -> bf16 while staging,
so only 16-bit values cross NVLink.  After backward the flat bf16 gradient is
reduce-scattered straight into an fp32 gradient shard (bf16 on the wire, fp32
accumulation, the 1/N average fused in), AdamW runs on the shard, and both
transient buffers are released.  Gathers and reductions are issued
asynchronously on the communicator's stream and overlap the neighbouring
stage's compute.

Parity: what the reference exercises through FSDP2 in
``comms/torchcomms/tests/integration/py/FSDPCommTest.py:16-66`` (parameter
``all_gather_into_tensor`` before forward/backward, gradient
``reduce_scatter_tensor`` after backward), here with the casts fused into the
collectives.
"""
from __future__ import annotations

from typing import List, Optional

import torch
import torch.nn as nn

from .. import ReduceOp, TorchComm
from ..ops import fused

_ALIGN = 8  # elements; keeps every parameter view 16-byte aligned in bf16

_CUDA_BACKENDS = ("b200", "nccl", "ncclx")


class ShardedUnit:
    def __init__(self, module: nn.Module, comm: TorchComm, param_dtype: torch.dtype = torch.bfloat16):
        self.module = module
        self.comm = comm
        self.world = comm.get_size()
        self.rank = comm.get_rank()
        self.param_dtype = param_dtype
        self.fused_casts = comm.get_backend() in _CUDA_BACKENDS
        params = [p for p in module.parameters()]
        self.params = params
        self.device = params[0].device
        self.offsets: List[int] = []
        off = 0
        for p in params:
            self.offsets.append(off)
            off += (p.numel() + _ALIGN - 1) // _ALIGN * _ALIGN
        quantum = self.world * 128
        self.total = (off + quantum - 1) // quantum * quantum
        self.shard_numel = self.total // self.world

        with torch.no_grad():
            lo = self.rank * self.shard_numel
            hi = lo + self.shard_numel
            self.shard = torch.zeros(self.shard_numel, dtype=torch.float32, device=self.device)
            for p, o in zip(params, self.offsets):
                a, b = max(o, lo), min(o + p.numel(), hi)
                if a < b:
                    self.shard[a - lo : b - lo] = p.detach().reshape(-1)[a - o : b - o].float()
        self.exp_avg = torch.zeros_like(self.shard)
        self.exp_avg_sq = torch.zeros_like(self.shard)

        # Parameters become views of one flat low-precision buffer whose
        # storage is only populated while the stage is in use.
        self.flat_param = torch.empty(self.total, dtype=param_dtype, device=self.device)
        for p, o in zip(params, self.offsets):
            p.data = self.flat_param[o : o + p.numel()].view(p.shape)
        self._param_bytes = self.flat_param.untyped_storage().nbytes()
        self.flat_param.untyped_storage().resize_(0)
        self.flat_grad: Optional[torch.Tensor] = None
        self.grad_shard: Optional[torch.Tensor] = None
        self._gather_work = None
        self._reduce_work = None
        self._resident = False

    # -- parameters ---------------------------------------------------------
    def gather(self, async_op: bool = True) -> None:
        """Starts materialising the full parameters (no-op if already there)."""
        if self._resident or self._gather_work is not None:
            return
        self.flat_param.untyped_storage().resize_(self._param_bytes)
        if self.fused_casts:
            src = self.shard
        else:
            src = self.shard.to(self.param_dtype)
        self._gather_work = self.comm.all_gather_single(self.flat_param, src, async_op)

    def wait_gather(self) -> None:
        if self._gather_work is not None:
            self._gather_work.wait()
            self._gather_work = None
            self._resident = True

    def release_params(self) -> None:
        if self._resident:
            self.flat_param.untyped_storage().resize_(0)
            self._resident = False

    # -- gradients ----------------------------------------------------------
    def prepare_grads(self) -> None:
        """Points every parameter's .grad at a slice of one zeroed flat buffer."""
        self.flat_grad = torch.zeros(self.total, dtype=self.param_dtype, device=self.device)
        for p, o in zip(self.params, self.offsets):
            p.grad = self.flat_grad[o : o + p.numel()].view(p.shape)

    def reduce_grads(self, async_op: bool = True) -> None:
        """Averages gradients over ranks into this rank's fp32 gradient shard."""
        assert self.flat_grad is not None
        for p in self.params:
            p.grad = None
        self.grad_shard = torch.empty(self.shard_numel, dtype=torch.float32, device=self.device)
        if self.fused_casts:
            self._reduce_work = self.comm.reduce_scatter_single(self.grad_shard, self.flat_grad, ReduceOp.AVG, async_op)
        else:
            wide = self.flat_grad.float()
            self._reduce_work = self.comm.reduce_scatter_single(self.grad_shard, wide, ReduceOp.AVG, async_op)

    def finish_step(self, *, lr: float, beta1: float, beta2: float, eps: float, weight_decay: float, step: int) -> None:
        """Waits for the reduction, applies AdamW to the shard, frees the transients."""
        if self._reduce_work is None:
            return
        self._reduce_work.wait()
        self._reduce_work = None
        fused.adamw_step_(
            self.shard, self.grad_shard, self.exp_avg, self.exp_avg_sq,
            lr=lr, beta1=beta1, beta2=beta2, eps=eps, weight_decay=weight_decay, step=step,
        )
        self.flat_grad = None
        self.grad_shard = None

    # -- checkpointing --------------------------------------------------------
    def state_dict(self) -> dict:
        return {"shard": self.shard, "exp_avg": self.exp_avg, "exp_avg_sq": self.exp_avg_sq}

    def load_state_dict(self, state: dict) -> None:
        self.shard.copy_(state["shard"])
        self.exp_avg.copy_(state["exp_avg"])
        self.exp_avg_sq.copy_(state["exp_avg_sq"])
