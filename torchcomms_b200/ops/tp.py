"""Tensor-parallel layers whose collective runs inside the GEMM kernel.

Sequence-parallel MLP of a transformer block on ``tp`` ranks::

    up   = AllGatherGemm(comm, m_local=tokens // tp, k=hidden)     # column-parallel
    down = GemmReduceScatter(comm, m=tokens, n=hidden)              # row-parallel
    up.input.copy_(x_shard)                # or have the producer write into up.input
    gate_up = up(w_gate_up_shard)          # [tokens, 2*ffn/tp]; peers' rows arrive while the MMAs run
    h = swiglu(gate_up)
    y_shard = down(h, w_down_shard)        # [tokens // tp, hidden]; partial tiles leave from the epilogue

Both are one persistent tcgen05 kernel (TMA-fed, TMEM double-buffered
accumulators): in ``AllGatherGemm`` extra warps pull the peers' activation
rows over NVLink and the tile scheduler follows their arrival order; in
``GemmReduceScatter`` the epilogue stores bf16 partial tiles into the owning
rank's staging and the owner sums them in fp32 as flags arrive.

The reference has no counterpart: its tree contains no GEMM and no fused
compute+collective kernel; tensor parallelism is exercised there through
DTensor over NCCL all-gather / reduce-scatter plus cuBLAS
(comms/torchcomms/tests/integration/py/TPCommTest.py:71), which is the
baseline arm of ``benchmarks/tp_layer_perf.py``.  When the token shard is a
multiple of 256 rows the kernels run on CTA pairs (tcgen05 ``cta_group::2``).
``comm=None`` builds a single-rank layer on
the current device (no peers; tests and profiling).

``fp8=True`` runs the same kernels on e4m3 operands (``tcgen05.mma
kind::f8f6f4``, twice the tensor throughput and half the all-gather bytes):
activations carry one fp32 scale per token, weights one per output channel
(``quantize_rows``), and the product of the two scales the fp32 accumulator in
the epilogue, so the result is again bf16.  The partial tiles of the
reduce-scatter stay bf16.
"""
from __future__ import annotations

from typing import Optional, Tuple

import torch

from .. import TorchComm, _comms


FP8_MAX = 448.0


def _impl(comm: Optional[TorchComm]):
    return None if comm is None else comm.get_backend_impl()


def quantize_rows(x: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    """``(q, scale)`` with ``q`` e4m3 ``[rows, cols]`` and ``scale`` fp32 ``[rows]`` such that ``q * scale[:, None] ~ x``."""
    amax = x.float().abs().amax(dim=1).clamp_min(1e-8)
    scale = amax / FP8_MAX
    return (x.float() / scale.unsqueeze(1)).to(torch.float8_e4m3fn), scale


def gemm_e4m3_nt(a: torch.Tensor, b: torch.Tensor, scale_a: torch.Tensor, scale_b: torch.Tensor) -> torch.Tensor:
    """``(scale_a[:, None] * scale_b[None, :]) * (a @ b.T)`` for e4m3 ``a [m, k]``, ``b [n, k]``; bf16 result."""
    c, status = _comms.ops.gemm_e4m3_nt(a, b, scale_a, scale_b)
    return c


class AllGatherGemm:
    """``y = all_gather(x_shard, dim=0) @ w.T`` for bf16 ``x_shard [m_local, k]``, ``w [n, k]``."""

    def __init__(self, comm: Optional[TorchComm], m_local: int, k: int, wait_ms: float = 2000.0, fp8: bool = False):
        self.comm, self.m_local, self.k, self.fp8 = comm, m_local, k, fp8
        self._layer = _comms.TpLayer(_impl(comm), "ag_gemm", m_local, k, wait_ms, fp8)

    @property
    def input(self) -> torch.Tensor:
        """This rank's ``[m_local, k]`` shard in peer-readable memory (bf16, or e4m3 with ``fp8``)."""
        return self._layer.input()

    @property
    def input_scales(self) -> torch.Tensor:
        """``fp8``: this rank's ``[m_local]`` fp32 row scales, peer-readable; they travel with the rows."""
        return self._layer.input_scales()

    def __call__(self, w: torch.Tensor, x_shard: Optional[torch.Tensor] = None, scale_w: Optional[torch.Tensor] = None,
                 scale_x: Optional[torch.Tensor] = None) -> torch.Tensor:
        """``fp8``: ``w`` e4m3 with ``scale_w [n]``; ``x_shard`` e4m3 with ``scale_x [m_local]``, or bf16 (quantised here)."""
        if x_shard is not None:
            if self.fp8 and x_shard.dtype != torch.float8_e4m3fn:
                x_shard, scale_x = quantize_rows(x_shard)
            self.input.copy_(x_shard)
            if self.fp8:
                self.input_scales.copy_(scale_x)
        return self._layer.ag_gemm(w, scale_w)

    def status(self):
        return self._layer.status()


class GemmReduceScatter:
    """``out = reduce_scatter(h @ w.T, dim=0)`` for bf16 ``h [m, k_local]``, ``w [n, k_local]``."""

    def __init__(self, comm: Optional[TorchComm], m: int, n: int, wait_ms: float = 2000.0, fp8: bool = False):
        self.comm, self.m, self.n, self.fp8 = comm, m, n, fp8
        self._layer = _comms.TpLayer(_impl(comm), "gemm_rs", m, n, wait_ms, fp8)

    def __call__(self, h: torch.Tensor, w: torch.Tensor, scale_h: Optional[torch.Tensor] = None,
                 scale_w: Optional[torch.Tensor] = None) -> torch.Tensor:
        """``fp8``: ``w`` e4m3 with ``scale_w [n]``; ``h`` e4m3 with ``scale_h [m]``, or bf16 (quantised here)."""
        if self.fp8 and h.dtype != torch.float8_e4m3fn:
            h, scale_h = quantize_rows(h)
        return self._layer.gemm_rs(h, w, scale_h, scale_w)

    def status(self):
        return self._layer.status()
