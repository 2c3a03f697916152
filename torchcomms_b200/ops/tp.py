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
"""
from __future__ import annotations

from typing import Optional

import torch

from .. import TorchComm, _comms


def _impl(comm: Optional[TorchComm]):
    return None if comm is None else comm.get_backend_impl()


class AllGatherGemm:
    """``y = all_gather(x_shard, dim=0) @ w.T`` for bf16 ``x_shard [m_local, k]``, ``w [n, k]``."""

    def __init__(self, comm: Optional[TorchComm], m_local: int, k: int, wait_ms: float = 2000.0):
        self.comm, self.m_local, self.k = comm, m_local, k
        self._layer = _comms.TpLayer(_impl(comm), "ag_gemm", m_local, k, wait_ms)

    @property
    def input(self) -> torch.Tensor:
        """This rank's ``[m_local, k]`` shard in peer-readable memory."""
        return self._layer.input()

    def __call__(self, w: torch.Tensor, x_shard: Optional[torch.Tensor] = None) -> torch.Tensor:
        if x_shard is not None:
            self.input.copy_(x_shard)
        return self._layer.ag_gemm(w)

    def status(self):
        return self._layer.status()


class GemmReduceScatter:
    """``out = reduce_scatter(h @ w.T, dim=0)`` for bf16 ``h [m, k_local]``, ``w [n, k_local]``."""

    def __init__(self, comm: Optional[TorchComm], m: int, n: int, wait_ms: float = 2000.0):
        self.comm, self.m, self.n = comm, m, n
        self._layer = _comms.TpLayer(_impl(comm), "gemm_rs", m, n, wait_ms)

    def __call__(self, h: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
        return self._layer.gemm_rs(h, w)

    def status(self):
        return self._layer.status()
