"""Fully sharded data parallelism driven by a communicator.

Each stage of a model becomes a ``ShardedUnit``: its parameters live as ONE
flat fp32 shard per rank (plus AdamW moments).  Before the stage runs, the
shards are all-gathered into a flat bf16 buffer the parameters are views of;
after backward the flat bf16 gradient is reduce-scattered into an fp32 gradient
shard (fp32 accumulation, the 1/N average fused in), AdamW runs on the shard,
and both transient buffers go back to their pool.  Gathers and reductions are
issued asynchronously and overlap the neighbouring stage's compute.

Three ways to move the data (``comm_mode``):

``"symm"`` (default on the CUDA backend)
    The flat parameter and gradient buffers are symmetric tensors of the
    communicator, taken from a small rotating pool.  The all-gather is one
    kernel that reads the fp32 shard, narrows it to bf16 in registers and
    stores it straight into every rank's parameter buffer (``multimem.st``
    through the switch where available); the reduce-scatter is one kernel that
    reads this rank's slice of every rank's gradient buffer
    (``multimem.ld_reduce``: the switch adds), scales and writes fp32.  Nothing
    is staged, every byte crosses NVLink once, and gathers and reductions use
    different channels of the communicator, so they run concurrently.
``"staged"``
    Ordinary buffers; the communicator's pipelined kernels stage through its
    heap with the casts fused into the copies.
``"nccl"``
    The stock path the reference's ``nccl`` backend would take: a separate
    fp32 -> bf16 cast, ``ncclAllGather``, ``ncclReduceScatter`` on bf16, and a
    separate cast + scale of the result.  Kept as the comparison arm.

Parity: what the reference exercises through FSDP2 in
``comms/torchcomms/tests/integration/py/FSDPCommTest.py:16-66`` (parameter
``all_gather_into_tensor`` before forward/backward, gradient
``reduce_scatter_tensor`` after backward), and its registered-buffer path
(``comms/torchcomms/ncclx/TorchCommNCCLXCCA.cpp:24-74``).
"""
from __future__ import annotations

import os
from typing import Dict, List, Optional, Tuple

import torch
import torch.nn as nn

from .. import ReduceOp, TorchComm, _comms
from ..mem import symm_empty
from ..ops import fused

_ALIGN = 8  # elements; keeps every parameter view 16-byte aligned in bf16

_CUDA_BACKENDS = ("b200", "nccl", "ncclx")


def _hints_from_env(var: str, default: Dict[str, str]) -> Dict[str, str]:
    raw = os.environ.get(var)
    if raw is None:
        return dict(default)
    return dict(kv.split("=", 1) for kv in raw.split(",") if "=" in kv)


class BufferPool:
    """Rotating flat buffers, one free list per (numel, dtype).

    With ``symmetric=True`` the buffers are symmetric tensors of ``comm``
    (allocation is collective: every rank must reserve in the same order).
    A stage takes a buffer for the time its parameters or gradients are
    materialised and gives it back afterwards; two per size class are enough
    for compute on one stage overlapped with communication for the next.
    """

    def __init__(self, comm: TorchComm, symmetric: bool):
        self.comm = comm
        self.symmetric = symmetric
        self._free: Dict[Tuple[int, torch.dtype], List[torch.Tensor]] = {}
        self._made: Dict[Tuple[int, torch.dtype], int] = {}
        self._users: Dict[Tuple[int, torch.dtype], int] = {}

    def add_user(self, numel: int, dtype: torch.dtype) -> None:
        """A stage announces its flat size. One stage of a size needs a parameter and a gradient buffer;
        several need two of each (compute on one stage while the next one's communication runs)."""
        key = (numel, dtype)
        self._users[key] = self._users.get(key, 0) + 1
        self.reserve(numel, dtype, 2 if self._users[key] == 1 else 4)

    def reserve(self, numel: int, dtype: torch.dtype, count: int) -> None:
        key = (numel, dtype)
        while self._made.get(key, 0) < count:
            if self.symmetric:
                buf = symm_empty(self.comm, (numel,), dtype)
            else:
                buf = torch.empty(numel, dtype=dtype, device=self.comm.get_device())
            self._free.setdefault(key, []).append(buf)
            self._made[key] = self._made.get(key, 0) + 1

    def acquire(self, numel: int, dtype: torch.dtype) -> torch.Tensor:
        free = self._free.get((numel, dtype))
        if not free:
            raise RuntimeError(f"buffer pool exhausted for {numel} x {dtype}: reserve more buffers")
        return free.pop()

    def release(self, buf: torch.Tensor) -> None:
        self._free[(buf.numel(), buf.dtype)].append(buf)

    def free_all(self) -> None:
        """Collective for symmetric pools: unmaps every buffer (all of them must have been released)."""
        from ..mem import symm_free

        for key in sorted(self._free, key=lambda k: (k[0], str(k[1]))):
            bufs = self._free[key]
            if len(bufs) != self._made.get(key, 0):
                raise RuntimeError("buffer pool: buffers are still in use")
            for b in bufs:
                if self.symmetric:
                    symm_free(self.comm, b)
        self._free.clear()
        self._made.clear()
        self._users.clear()

    def bytes_reserved(self) -> int:
        return sum(k[0] * torch.empty((), dtype=k[1]).element_size() * n for k, n in self._made.items())


class StepTimeline:
    """CUDA-event spans of one or more training steps, for a comm / compute breakdown.

    ``ag`` / ``rs``: time the all-gather / reduce-scatter kernels occupy their
    communication stream (from the moment their inputs are ready); ``wait``:
    time the compute stream sits blocked on a collective (the exposed part);
    ``opt``: the optimizer kernels.  Recording costs two events per span, so a
    timeline is attached for a few profiled steps only.
    """

    KINDS = ("ag", "rs", "wait", "opt")

    def __init__(self, comm: TorchComm, comm_mode: str):
        self.spans = {k: [] for k in self.KINDS}
        self._streams = {}
        if comm.get_backend() in _CUDA_BACKENDS and torch.cuda.is_available():
            impl = comm.get_backend_impl()
            chans = {"ag": 1, "rs": 2} if comm_mode == "symm" else {"ag": 0, "rs": 0}
            for kind, chan in chans.items():
                self._streams[kind] = torch.cuda.ExternalStream(impl.channel_stream(chan), device=comm.get_device())

    class _Span:
        def __init__(self, owner, kind, stream):
            self.owner, self.kind, self.stream = owner, kind, stream

        def __enter__(self):
            self.start = torch.cuda.Event(enable_timing=True)
            self.end = torch.cuda.Event(enable_timing=True)
            if self.stream is not None:
                # The collective's own dependency on the compute stream is taken
                # here already, so that the span starts when the inputs are ready.
                self.stream.wait_stream(torch.cuda.current_stream())
            self.start.record(self.stream)
            return self

        def __exit__(self, *exc):
            self.end.record(self.stream)
            self.owner.spans[self.kind].append((self.start, self.end))
            return False

    def span(self, kind: str):
        return self._Span(self, kind, self._streams.get(kind))

    def totals_ms(self) -> dict:
        torch.cuda.synchronize()
        return {k: sum(a.elapsed_time(b) for a, b in v) for k, v in self.spans.items()}


class _NoSpan:
    def __enter__(self):
        return self

    def __exit__(self, *exc):
        return False


_NO_SPAN = _NoSpan()


class ShardedUnit:
    def __init__(
        self,
        module: nn.Module,
        comm: TorchComm,
        param_dtype: torch.dtype = torch.bfloat16,
        comm_mode: Optional[str] = None,
        pool: Optional[BufferPool] = None,
    ):
        self.module = module
        self.comm = comm
        self.world = comm.get_size()
        self.rank = comm.get_rank()
        self.param_dtype = param_dtype
        on_cuda_backend = comm.get_backend() in _CUDA_BACKENDS
        if comm_mode is None:
            comm_mode = "symm" if on_cuda_backend else "plain"
        if comm_mode not in ("symm", "staged", "nccl", "plain"):
            raise ValueError(f"unknown comm_mode {comm_mode!r}")
        self.comm_mode = comm_mode
        self.fused_casts = on_cuda_backend and comm_mode in ("symm", "staged")
        self.pool = pool if pool is not None else BufferPool(comm, symmetric=comm_mode == "symm")
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

        # Parameters are views of one flat low-precision tensor whose storage
        # points at a pool buffer only while the stage is in use. Views (and
        # the tensors autograd saved for backward) follow the storage, so a
        # stage may get a different buffer for backward than it had in forward.
        self.flat_param = torch.empty(self.total, dtype=param_dtype, device=self.device)
        for p, o in zip(params, self.offsets):
            p.data = self.flat_param[o : o + p.numel()].view(p.shape)
        _comms.ops.rebind_storage_(self.flat_param, None)
        self.pool.add_user(self.total, param_dtype)
        self._param_buf: Optional[torch.Tensor] = None
        self.flat_grad: Optional[torch.Tensor] = None
        self.grad_shard: Optional[torch.Tensor] = None
        self._gather_work = None
        self._reduce_work = None
        self._resident = False
        self.timeline: Optional[StepTimeline] = None
        # The collectives of a training step run next to GEMMs, fully hidden behind them when they are
        # given time: small grids leave the SMs to the math (16 blocks measured best on 4 B200: 214 ms
        # per step against 216 with 24, 218 with 8 and 223 with 32 blocks), and the reduce-scatter takes
        # the switch's reduction (one load per 16 bytes instead of one per rank; peer loads would need
        # most of the SMs to reach link rate). B200COMMS_FSDP_AG_HINTS / _RS_HINTS ("k=v,k=v") override.
        self._ag_hints = self._rs_hints = None
        if comm_mode == "symm":
            has_mc = on_cuda_backend and self.world > 1 and bool(comm.get_backend_impl().has_multicast())
            self._ag_hints = _hints_from_env("B200COMMS_FSDP_AG_HINTS", {"symm_blocks": "16"})
            self._rs_hints = _hints_from_env(
                "B200COMMS_FSDP_RS_HINTS", {"symm_mc": "1", "symm_blocks": "16"} if has_mc else {"symm_blocks": "64"})

    def _span(self, kind: str):
        return self.timeline.span(kind) if self.timeline is not None and self.device.type == "cuda" else _NO_SPAN

    # -- parameters ---------------------------------------------------------
    def gather(self, async_op: bool = True) -> None:
        """Starts materialising the full parameters (no-op if already there)."""
        if self._resident or self._gather_work is not None:
            return
        self._param_buf = self.pool.acquire(self.total, self.param_dtype)
        _comms.ops.rebind_storage_(self.flat_param, self._param_buf)
        if self.comm_mode == "nccl":
            src = self.shard.to(self.param_dtype)
            with self._span("ag"):
                self._gather_work = self.comm.all_gather_single(self._param_buf, src, async_op, hints={"algo": "nccl"})
        elif self.fused_casts:
            with self._span("ag"):
                self._gather_work = self.comm.all_gather_single(self._param_buf, self.shard, async_op, hints=self._ag_hints)
        else:
            self._gather_work = self.comm.all_gather_single(self._param_buf, self.shard.to(self.param_dtype), async_op)

    def wait_gather(self) -> None:
        if self._gather_work is not None:
            with self._span("wait"):
                self._gather_work.wait()
            self._gather_work = None
            self._resident = True

    def release_params(self) -> None:
        if self._resident:
            _comms.ops.rebind_storage_(self.flat_param, None)
            self.pool.release(self._param_buf)
            self._param_buf = None
            self._resident = False

    # -- gradients ----------------------------------------------------------
    def prepare_grads(self) -> None:
        """Points every parameter's .grad at a slice of one zeroed flat buffer."""
        self.flat_grad = self.pool.acquire(self.total, self.param_dtype)
        self.flat_grad.zero_()
        for p, o in zip(self.params, self.offsets):
            p.grad = self.flat_grad[o : o + p.numel()].view(p.shape)

    def reduce_grads(self, async_op: bool = True) -> None:
        """Averages gradients over ranks into this rank's fp32 gradient shard."""
        assert self.flat_grad is not None
        for p in self.params:
            p.grad = None
        self.grad_shard = torch.empty(self.shard_numel, dtype=torch.float32, device=self.device)
        if self.comm_mode == "nccl":
            self._narrow = torch.empty(self.shard_numel, dtype=self.param_dtype, device=self.device)
            with self._span("rs"):
                self._reduce_work = self.comm.reduce_scatter_single(
                    self._narrow, self.flat_grad, ReduceOp.AVG, async_op, hints={"algo": "nccl"}
                )
        elif self.fused_casts:
            with self._span("rs"):
                self._reduce_work = self.comm.reduce_scatter_single(self.grad_shard, self.flat_grad, ReduceOp.AVG, async_op,
                                                                    hints=self._rs_hints)
        else:
            wide = self.flat_grad.float()
            self._reduce_work = self.comm.reduce_scatter_single(self.grad_shard, wide, ReduceOp.AVG, async_op)

    def finish_step(self, *, lr: float, beta1: float, beta2: float, eps: float, weight_decay: float, step: int) -> None:
        """Waits for the reduction, applies AdamW to the shard, frees the transients."""
        if self._reduce_work is None:
            return
        with self._span("wait"):
            self._reduce_work.wait()
        self._reduce_work = None
        with self._span("opt"):
            if self.comm_mode == "nccl":
                self.grad_shard.copy_(self._narrow)
                self._narrow = None
            fused.adamw_step_(
                self.shard, self.grad_shard, self.exp_avg, self.exp_avg_sq,
                lr=lr, beta1=beta1, beta2=beta2, eps=eps, weight_decay=weight_decay, step=step,
            )
        self.pool.release(self.flat_grad)
        self.flat_grad = None
        self.grad_shard = None

    # -- checkpointing --------------------------------------------------------
    def state_dict(self) -> dict:
        return {"shard": self.shard, "exp_avg": self.exp_avg, "exp_avg_sq": self.exp_avg_sq}

    def load_state_dict(self, state: dict) -> None:
        self.shard.copy_(state["shard"])
        self.exp_avg.copy_(state["exp_avg"])
        self.exp_avg_sq.copy_(state["exp_avg_sq"])
