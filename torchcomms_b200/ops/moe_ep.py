"""MoE expert-parallel dispatch and combine over NVLink peer memory.

``Buffer`` owns symmetric receive / combine buffers sized for the worst case
(``nranks * max_tokens`` rows), so no call allocates and no call synchronises
with the host: the number of received rows is a device tensor.

    buf = Buffer(comm, max_tokens=4096, hidden=7168, num_experts=256, topk=8)
    recv = buf.dispatch(x, topk_idx, topk_weights)       # fp8 e4m3 rows + 1x128 scales
    n = recv.num_tokens                                  # 0-d int32 device tensor
    ...experts write their outputs into buf.combine_input[:n]...
    y = buf.combine()                                    # sum over destination ranks, bf16

Three more pieces serve training and decode:

* ``Dispatched.handle`` / ``Buffer.cached_dispatch`` / ``combine(handle=...)``:
  the layout of a dispatch kept for later calls (the gradient of a combine is
  a dispatch with the same layout, and the other way round);
* ``dispatch_autograd`` / ``combine_autograd``: differentiable forms (bf16
  rows) whose backward passes run on the same kernels;
* ``LowLatencyBuffer``: decode-sized batches, one row per (token, expert) pair
  in fixed slots, no layout exchange before the data moves.

Parity: ``comms/prims/collectives/link_ep/link_ep/buffer.py:76-660`` (Buffer,
get_dispatch_layout, dispatch, combine, low_latency_dispatch / combine).
Differences by design: block-scaled fp8 quantisation and the token permutation
are fused into the dispatch kernel, receive counts stay on the device, and
combine is a pull: the token's owner reads the expert outputs of every rank the
token went to straight out of that rank's ``combine_input`` and sums them with
the weights applied (no ring FIFOs, nothing staged, one pass over NVLink).
``ops/link_ep.py`` offers the reference's call signatures on top of this.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional, Tuple

import torch

from .. import TorchComm, _comms

FP8_MAX = 448.0


@dataclass
class Handle:
    """Layout of one dispatch: enough to repeat it (``cached_dispatch``) or undo it (``combine``) later."""

    send_slot: torch.Tensor   # [tokens, nranks] int32: row in each destination, -1 = not sent (source side)
    recv_src: torch.Tensor    # [rows] int32: src_rank * max_tokens + token (receiver side)
    num_recv: torch.Tensor    # 0-d int32 on the device: rows received
    num_tokens: int           # tokens of the source side


@dataclass
class Dispatched:
    x: torch.Tensor                 # [rows, hidden] float8_e4m3fn (or bf16), first num_tokens rows valid
    scales: Optional[torch.Tensor]  # [rows, hidden/128] float32 (fp8 only)
    topk_idx: torch.Tensor          # [rows, topk] int32: local expert id or -1
    topk_weights: torch.Tensor      # [rows, topk] float32
    src: torch.Tensor               # [rows] int32: src_rank * max_tokens + token
    num_tokens: torch.Tensor        # 0-d int32 on the device
    tokens_per_src: torch.Tensor    # [nranks] int32: rows are packed by source rank
    handle: Optional[Handle] = None


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

    @property
    def combine_topk_weights(self) -> torch.Tensor:
        """[rows, topk] fp32, peer-readable: per-expert weights (or their gradients) that ``combine`` carries back."""
        return self._buf.view(0, "combine_topk_weights")

    @property
    def dispatch_stage(self) -> torch.Tensor:
        """[max_tokens, hidden] bf16, peer-readable: the rows that ``cached_dispatch`` hands out."""
        return self._buf.view(0, "stage_x")

    def dispatch(self, x: torch.Tensor, topk_idx: torch.Tensor, topk_weights: torch.Tensor,
                 keep_handle: bool = False) -> Dispatched:
        """``keep_handle``: copy the layout out of the buffer so that it survives later dispatches."""
        self._num_tokens = x.shape[0]
        self._buf.dispatch([x.contiguous()], [topk_idx.to(torch.int32).contiguous()], [topk_weights.float().contiguous()])
        info = self._buf.view(0, "recv_info")
        out = Dispatched(
            x=self._buf.view(0, "recv_x"),
            scales=self._buf.view(0, "recv_scales") if self.fp8 else None,
            topk_idx=self._buf.view(0, "recv_topk_idx"),
            topk_weights=self._buf.view(0, "recv_topk_weights"),
            src=self._buf.view(0, "recv_src"),
            num_tokens=info[0],
            tokens_per_src=info[1:],
        )
        if keep_handle:
            out.handle = Handle(self._buf.view(0, "send_slot")[: x.shape[0]].clone(), out.src.clone(), info[0].clone(),
                                x.shape[0])
        return out

    def cached_dispatch(self, x: torch.Tensor, handle: Optional[Handle] = None, out: Optional[torch.Tensor] = None,
                        rows: Optional[int] = None) -> torch.Tensor:
        """Sends ``x`` (bf16, unquantised) along the layout of an earlier dispatch (``handle``; default: the last one).

        Returns ``[rows, hidden]`` bf16 with the first ``num_recv`` rows filled; ``rows`` defaults to the capacity.
        """
        self.dispatch_stage[: x.shape[0]].copy_(x)
        if out is None:
            out = torch.empty(self._buf.rows() if rows is None else rows, self.hidden, dtype=torch.bfloat16, device=x.device)
        if handle is None:
            self._buf.pull([out])
        else:
            self._buf.pull([out], [handle.recv_src], [handle.num_recv])
        return out

    def combine(self, weights: Optional[torch.Tensor] = None, bias: Optional[torch.Tensor] = None,
                out: Optional[torch.Tensor] = None, handle: Optional[Handle] = None,
                topk_weights_out: Optional[torch.Tensor] = None) -> torch.Tensor:
        """``out[t] = bias[t] + sum_d weights[t, d] * outputs_of_rank_d[row(t, d)]`` for the tokens of the last
        dispatch, or of the dispatch that produced ``handle``.  ``topk_weights_out`` ([tokens, topk] fp32), if given,
        receives the sum over destinations of their ``combine_topk_weights`` rows."""
        tokens = handle.num_tokens if handle is not None else self._num_tokens
        if out is None:
            out = torch.empty(tokens, self.hidden, dtype=torch.bfloat16, device=self.comm.get_device())
        self._buf.combine([out], [weights.float().contiguous()] if weights is not None else [],
                          [bias.contiguous()] if bias is not None else [],
                          [handle.send_slot] if handle is not None else [],
                          [topk_weights_out] if topk_weights_out is not None else [])
        return out


class _DispatchFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, buf: Buffer, x: torch.Tensor, topk_idx: torch.Tensor, topk_weights: torch.Tensor):
        if buf.fp8:
            raise ValueError("differentiable dispatch needs a bf16 buffer (fp8=False)")
        d = buf.dispatch(x.detach(), topk_idx, topk_weights.detach(), keep_handle=True)
        n = int(d.num_tokens)                      # host read: sizes everything downstream
        ctx.buf, ctx.handle, ctx.n = buf, d.handle, n
        local_idx = d.topk_idx[:n].clone()
        ctx.mark_non_differentiable(local_idx)
        ctx.set_materialize_grads(False)
        return d.x[:n].clone(), d.topk_weights[:n].clone(), local_idx, (d.handle, n)

    @staticmethod
    def backward(ctx, g_rows, g_weights, _g_idx, _g_meta):
        buf, n = ctx.buf, ctx.n
        # The gradient of a dispatch is a combine: every token sums what came back from the ranks it went to.
        if g_rows is None:
            buf.combine_input[:n].zero_()
        else:
            buf.combine_input[:n].copy_(g_rows)
        w_out = None
        if g_weights is not None:
            buf.combine_topk_weights[:n].copy_(g_weights)
            w_out = torch.empty(ctx.handle.num_tokens, buf.topk, dtype=torch.float32, device=buf.combine_input.device)
        gx = buf.combine(handle=ctx.handle, topk_weights_out=w_out)
        return None, gx if g_rows is not None else None, None, w_out


class _CombineFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, buf: Buffer, rows: torch.Tensor, handle: Handle, n: int):
        ctx.buf, ctx.handle, ctx.n = buf, handle, n
        buf.combine_input[:n].copy_(rows.detach())
        return buf.combine(handle=handle)

    @staticmethod
    def backward(ctx, g_out):
        # The gradient of a combine is a dispatch of the output gradients along the same layout.
        g = ctx.buf.cached_dispatch(g_out.contiguous().to(torch.bfloat16), ctx.handle, rows=ctx.n)
        return None, g, None, None


def dispatch_autograd(buf: Buffer, x: torch.Tensor, topk_idx: torch.Tensor,
                      topk_weights: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor, Tuple[Handle, int]]:
    """Differentiable dispatch (bf16 rows): ``(rows [n, hidden], weights [n, topk], local expert ids [n, topk], meta)``.

    Gradients reach ``x`` and ``topk_weights``; ``meta`` goes to ``combine_autograd``.
    """
    return _DispatchFn.apply(buf, x, topk_idx, topk_weights)


def combine_autograd(buf: Buffer, rows: torch.Tensor, meta: Tuple[Handle, int]) -> torch.Tensor:
    """Differentiable combine: ``y[t] = sum over the ranks token t went to of rows[row(t, rank)]`` (bf16)."""
    handle, n = meta
    return _CombineFn.apply(buf, rows, handle, n)


@dataclass
class LowLatencyRecv:
    x: torch.Tensor                 # [local experts, nranks * max_tokens, hidden] fp8 or bf16, packed per expert
    scales: Optional[torch.Tensor]  # [local experts, nranks * max_tokens, hidden / 128] fp32 (fp8 only)
    count: torch.Tensor             # [local experts] int32 rows per expert
    src_info: torch.Tensor          # [local experts, nranks * max_tokens] int32 token index at the source
    layout_range: torch.Tensor      # [local experts, nranks] int64: (first row << 32) | rows, per source rank
    send_slot: torch.Tensor         # source-side handle: [tokens, topk] row number per (token, expert) pair
    begin: torch.Tensor             # source-side handle: [num_experts] first packed row of this rank at each expert


class LowLatencyBuffer:
    """Decode-sized dispatch / combine: one row per (token, expert) pair into fixed slots.

        ll = LowLatencyBuffer(comm, max_tokens=128, hidden=7168, num_experts=256, topk=8)
        r = ll.dispatch(x, topk_idx)                  # r.x[e, :r.count[e]] are the rows of local expert e
        ll.expert_output[e, :count] = ...             # grouped GEMM writes here (peer-readable)
        y = ll.combine(topk_idx, topk_weights, r)     # weighted top-k sum at the token's owner

    Parity: ``link_ep/buffer.py:550-625`` (low_latency_dispatch / low_latency_combine,
    get_next_low_latency_combine_buffer), ``cpp/low_latency/kernels/{Dispatch,Combine}.cu``.
    """

    def __init__(self, comm: TorchComm, max_tokens: int, hidden: int, num_experts: int, topk: int, fp8: bool = True):
        self.comm = comm
        self.nranks = comm.get_size()
        self.max_tokens, self.hidden, self.num_experts, self.topk, self.fp8 = max_tokens, hidden, num_experts, topk, fp8
        self._buf = _comms.EpLlBuffer(comm.get_backend_impl(), max_tokens, hidden, num_experts, topk, fp8)

    @property
    def expert_output(self) -> torch.Tensor:
        """[local experts, nranks * max_tokens, hidden] bf16, peer-readable: where expert outputs must be for combine."""
        return self._buf.view(0, "out_x")

    def dispatch(self, x: torch.Tensor, topk_idx: torch.Tensor) -> LowLatencyRecv:
        px, ps, src, count, rng = self._buf.dispatch([x.contiguous()], [topk_idx.to(torch.int32).contiguous()])[0]
        t = x.shape[0]
        return LowLatencyRecv(px, ps if self.fp8 else None, count, src, rng,
                              self._buf.view(0, "send_slot")[:t].clone(), self._buf.view(0, "begin").clone())

    def combine(self, topk_idx: torch.Tensor, topk_weights: torch.Tensor, recv: Optional[LowLatencyRecv] = None,
                x: Optional[torch.Tensor] = None, out: Optional[torch.Tensor] = None) -> torch.Tensor:
        """``x`` (optional): expert outputs to copy into ``expert_output`` first; leave it out when the experts
        wrote there directly."""
        if x is not None:
            self.expert_output.copy_(x)
        if out is None:
            out = torch.empty(topk_idx.shape[0], self.hidden, dtype=torch.bfloat16, device=topk_idx.device)
        handles = ([recv.send_slot], [recv.begin]) if recv is not None else ([], [])
        self._buf.combine([out], [topk_idx.to(torch.int32).contiguous()], [topk_weights.float().contiguous()], *handles)
        return out
