"""Tensor / sequence parallel layers.

``ColumnParallelLinear`` and ``RowParallelLinear`` follow the Megatron
layout: the first shards the output features, the second the input features.
With ``sequence_parallel=True`` activations between blocks stay sharded along
the token dimension: the column layer all-gathers its input, the row layer
reduce-scatters its output (instead of identity / all-reduce).

Two execution paths share the same parameters:

* the differentiable path uses the functional collectives
  (``torchcomms_b200.functional``), so autograd produces the mirrored
  collective in backward; it runs on any backend (gloo on CPU in the tests);
* ``TensorParallelMLP.forward_fused`` (CUDA, bf16 or fp8 operands, sequence
  parallel) runs the two projections as the fused tcgen05 kernels of
  ``ops.tp``: the all-gather happens inside the up-projection GEMM and the
  reduce-scatter inside the down-projection's epilogue.

The reference exercises TP only through DTensor's ColwiseParallel /
RowwiseParallel over its process-group adapter
(comms/torchcomms/tests/integration/py/TPCommTest.py:71,
DPTPCommTest.py:23-81); those keep working through ``device_mesh``.
"""
from __future__ import annotations

import math
from typing import Optional

import torch
from torch import nn

from .. import TorchComm
from .. import functional as F


class ColumnParallelLinear(nn.Module):
    """y_local = x @ W_shard^T with W_shard = rows [r*out/n, (r+1)*out/n) of the full weight."""

    def __init__(self, in_features: int, out_features: int, comm: TorchComm, bias: bool = False,
                 sequence_parallel: bool = False, gather_output: bool = False, device=None, dtype=None):
        super().__init__()
        n = comm.get_size()
        if out_features % n != 0:
            raise ValueError("out_features must divide by the tensor-parallel size")
        self.comm, self.sequence_parallel, self.gather_output = comm, sequence_parallel, gather_output
        self.comm_name = F.register_comm(comm)
        self.weight = nn.Parameter(torch.empty(out_features // n, in_features, device=device, dtype=dtype))
        self.bias = nn.Parameter(torch.zeros(out_features // n, device=device, dtype=dtype)) if bias else None
        nn.init.kaiming_uniform_(self.weight, a=math.sqrt(5))

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        if self.sequence_parallel:
            x = F.all_gather_single(x, self.comm_name)            # tokens: [m/n, k] -> [m, k]
        else:
            x = _CopyToRegion.apply(x, self.comm_name)            # identity forward, all-reduce backward
        y = nn.functional.linear(x, self.weight, self.bias)
        if self.gather_output:
            parts = F.all_gather_single(y.transpose(0, -1).contiguous(), self.comm_name)
            y = parts.transpose(0, -1).contiguous()
        return y


class RowParallelLinear(nn.Module):
    """y = sum_r x_r @ W_r^T with W_r = columns [r*in/n, (r+1)*in/n) of the full weight."""

    def __init__(self, in_features: int, out_features: int, comm: TorchComm, bias: bool = False,
                 sequence_parallel: bool = False, device=None, dtype=None):
        super().__init__()
        n = comm.get_size()
        if in_features % n != 0:
            raise ValueError("in_features must divide by the tensor-parallel size")
        self.comm, self.sequence_parallel = comm, sequence_parallel
        self.comm_name = F.register_comm(comm)
        self.weight = nn.Parameter(torch.empty(out_features, in_features // n, device=device, dtype=dtype))
        self.bias = nn.Parameter(torch.zeros(out_features, device=device, dtype=dtype)) if bias else None
        nn.init.kaiming_uniform_(self.weight, a=math.sqrt(5))

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        y = nn.functional.linear(x, self.weight)
        if self.sequence_parallel:
            y = F.reduce_scatter_single(y, "sum", self.comm_name)  # [m, out] -> [m/n, out]
        else:
            y = F.all_reduce(y, "sum", self.comm_name)
        if self.bias is not None:
            y = y + self.bias
        return y


class _CopyToRegion(torch.autograd.Function):
    """Identity in forward; the gradients of the replicated input are summed over the ranks in backward."""

    @staticmethod
    def forward(ctx, x, comm_name):
        ctx.comm_name = comm_name
        return x

    @staticmethod
    def backward(ctx, grad):
        return F.all_reduce(grad.contiguous(), "sum", ctx.comm_name), None


class TensorParallelMLP(nn.Module):
    """SwiGLU MLP (gate/up column-parallel, down row-parallel), sequence parallel between blocks."""

    def __init__(self, hidden: int, ffn: int, comm: TorchComm, device=None, dtype=None):
        super().__init__()
        self.hidden, self.ffn, self.comm = hidden, ffn, comm
        self.n = comm.get_size()
        # One weight for gate and up: rows [0, ffn/n) gate, [ffn/n, 2 ffn/n) up, so one GEMM serves both.
        self.gate_up = ColumnParallelLinear(hidden, 2 * ffn, comm, sequence_parallel=True, device=device, dtype=dtype)
        self.down = RowParallelLinear(ffn, hidden, comm, sequence_parallel=True, device=device, dtype=dtype)
        self._fused = None
        self._fp8_weights = None

    def forward(self, x_shard: torch.Tensor) -> torch.Tensor:
        gu = self.gate_up(x_shard)
        g, u = gu.chunk(2, dim=-1)
        return self.down(nn.functional.silu(g) * u)

    @torch.no_grad()
    def forward_fused(self, x_shard: torch.Tensor, fp8: bool = False) -> torch.Tensor:
        """Forward only, CUDA: all-gather inside the up GEMM, reduce-scatter inside the down GEMM's epilogue.

        ``fp8``: both GEMMs run on e4m3 operands (activations quantised per token on the way in, weights per output
        channel once and cached until ``invalidate_fp8_weights()``); outputs stay bf16.
        """
        from ..ops import fused as fused_ops
        from ..ops.tp import AllGatherGemm, GemmReduceScatter, quantize_rows

        m_local = x_shard.shape[0]
        key = (m_local, fp8)
        if self._fused is None or self._fused[0] != key:
            self._fused = (key, AllGatherGemm(self.comm, m_local, self.hidden, fp8=fp8),
                           GemmReduceScatter(self.comm, m_local * self.n, self.hidden, fp8=fp8))
        _, up, down = self._fused
        if not fp8:
            gu = up(self.gate_up.weight, x_shard)
            return down(fused_ops.swiglu(gu).contiguous(), self.down.weight)
        if self._fp8_weights is None:
            self._fp8_weights = quantize_rows(self.gate_up.weight) + quantize_rows(self.down.weight)
        w_up, s_up, w_down, s_down = self._fp8_weights
        gu = up(w_up, x_shard, scale_w=s_up)
        return down(fused_ops.swiglu(gu).contiguous(), w_down, scale_w=s_down)

    def invalidate_fp8_weights(self) -> None:
        """Call after the weights changed: the next fp8 forward quantises them again."""
        self._fp8_weights = None
