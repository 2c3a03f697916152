"""MoE expert-parallel dispatch and combine over NVLink peer memory.

``Buffer`` owns symmetric receive / combine buffers sized for the worst case
(``nranks * max_tokens`` rows), so no call allocates and no call synchronises
with the host: the number of received rows is a device tensor.

    buf = Buffer(comm, max_tokens=4096, hidden=7168, num_experts=256, topk=8)
    recv = buf.dispatch(x, topk_idx, topk_weights)       # fp8 e4m3 rows + 1x128 scales
    n = recv.num_tokens                                  # 0-d int32 device tensor
    ...experts write their outputs into buf.combine_input[:n]...
    y = buf.combine()                                    # sum over destination ranks, bf16

Parity: ``comms/prims/collectives/link_ep/link_ep/buffer.py:76-660`` (Buffer,
get_dispatch_layout, dispatch, combine).  Differences by design: block-scaled
fp8 quantisation and the token permutation are fused into the dispatch
kernel, receive counts stay on the device, and combine is a pull: the token's
owner reads the expert outputs of every rank the token went to straight out of
that rank's ``combine_input`` and sums them with the weights applied (no ring
FIFOs, nothing staged, one pass over NVLink).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

import torch

from .. import TorchComm, _comms

FP8_MAX = 448.0


@dataclass
class Dispatched:
    x: torch.Tensor                 # [rows, hidden] float8_e4m3fn (or bf16), first num_tokens rows valid
    scales: Optional[torch.Tensor]  # [rows, hidden/128] float32 (fp8 only)
    topk_idx: torch.Tensor          # [rows, topk] int32: local expert id or -1
    topk_weights: torch.Tensor      # [rows, topk] float32
    src: torch.Tensor               # [rows] int32: src_rank * max_tokens + token
    num_tokens: torch.Tensor        # 0-d int32 on the device
    tokens_per_src: torch.Tensor    # [nranks] int32: rows are packed by source rank


def get_dispatch_layout(topk_idx: torch.Tensor, num_experts: int, nranks: int):
    """(tokens per rank, tokens per expert, is_token_in_rank[T, nranks]) as int32 device tensors."""
    return _comms.ep_layout(topk_idx.to(torch.int32).contiguous(), num_experts, nranks)


def per_token_cast_to_fp8(x: torch.Tensor):
    """Reference quantisation (plain PyTorch): e4m3 with one fp32 scale per 128 elements."""
    t, h = x.shape
    g = x.float().view(t, h // 128, 128)
    amax = g.abs().amax(dim=-1).clamp_min(1e-4)
    q = (g * (FP8_MAX / amax).unsqueeze(-1)).to(torch.float8_e4m3fn)
    return q.view(t, h), amax / FP8_MAX


class Buffer:
    def __init__(self, comm: TorchComm, max_tokens: int, hidden: int, num_experts: int, topk: int, fp8: bool = True):
        self.comm = comm
        self.nranks = comm.get_size()
        self.max_tokens, self.hidden, self.num_experts, self.topk, self.fp8 = max_tokens, hidden, num_experts, topk, fp8
        self._buf = _comms.EpBuffer(comm.get_backend_impl(), max_tokens, hidden, num_experts, topk, fp8)
        self._num_tokens = 0

    @property
    def combine_input(self) -> torch.Tensor:
        """[rows, hidden] bf16, peer-readable: expert outputs go here, row-aligned with the dispatched rows."""
        return self._buf.view(0, "combine_x")

    def dispatch(self, x: torch.Tensor, topk_idx: torch.Tensor, topk_weights: torch.Tensor) -> Dispatched:
        self._num_tokens = x.shape[0]
        self._buf.dispatch([x.contiguous()], [topk_idx.to(torch.int32).contiguous()], [topk_weights.float().contiguous()])
        info = self._buf.view(0, "recv_info")
        return Dispatched(
            x=self._buf.view(0, "recv_x"),
            scales=self._buf.view(0, "recv_scales") if self.fp8 else None,
            topk_idx=self._buf.view(0, "recv_topk_idx"),
            topk_weights=self._buf.view(0, "recv_topk_weights"),
            src=self._buf.view(0, "recv_src"),
            num_tokens=info[0],
            tokens_per_src=info[1:],
        )

    def combine(self, weights: Optional[torch.Tensor] = None, bias: Optional[torch.Tensor] = None,
                out: Optional[torch.Tensor] = None) -> torch.Tensor:
        """``out[t] = bias[t] + sum_d weights[t, d] * outputs_of_rank_d[row(t, d)]`` for the tokens of the last dispatch."""
        if out is None:
            out = torch.empty(self._num_tokens, self.hidden, dtype=torch.bfloat16, device=self.comm.get_device())
        self._buf.combine([out], [weights.float().contiguous()] if weights is not None else [],
                          [bias.contiguous()] if bias is not None else [])
        return out
