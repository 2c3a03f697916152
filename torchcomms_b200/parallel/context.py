"""Context (sequence) parallel attention: ring attention and Ulysses.

Both shard the sequence over the ranks of a communicator.

* ``ring_attention``: K/V blocks travel around the ring in ``n - 1`` batched
  send/recv steps while each rank attends its local queries to the block it
  currently holds; partial results are merged with the running log-sum-exp,
  so the full score matrix never exists.  The transfer of step ``i + 1`` is
  issued before the math of step ``i`` (asynchronous batch on the
  communicator's side stream) and waited for afterwards.
  With ``layout="zigzag"`` (``zigzag_shard`` / ``zigzag_unshard``) causal attention is
  load-balanced over the ranks.  The backward pass sends the blocks round once
  more, each with an accumulator for its gradient.
* ``ulysses_attention``: one all-to-all turns sequence shards into head
  shards, attention runs locally over the full sequence for ``heads / n``
  heads, a second all-to-all turns the result back.  ``SeqHeadsExchange``
  runs those all-to-alls as one-pass kernels that also do the layout
  changes (CUDA backend, symmetric outputs).

The reference contains neither (its tree has no ring-attention / Ulysses /
context-parallel code); it provides the primitives they need - ``send`` /
``recv`` / ``BatchSendRecv`` rings and ``all_to_all_single``
(comms/torchcomms/TorchComm.hpp:50, TorchCommBatch.hpp:27-61).
"""
from __future__ import annotations

import math
from typing import Optional, Tuple

import torch

from .. import TorchComm


def _block_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, scale: float,
                     mask: Optional[torch.Tensor]) -> Tuple[torch.Tensor, torch.Tensor]:
    """softmax(q k^T) v for one K/V block plus the row log-sum-exp. q: [b, h, sq, d]; k, v: [b, h, sk, d]."""
    s = torch.matmul(q.float(), k.float().transpose(-1, -2)) * scale
    if mask is not None:
        s = s.masked_fill(~mask, float("-inf"))
    lse = torch.logsumexp(s, dim=-1)                     # [b, h, sq]; -inf where a row sees nothing
    p = torch.exp(s - lse.clamp_min(-1e30).unsqueeze(-1))
    p = torch.where(torch.isfinite(lse).unsqueeze(-1), p, torch.zeros_like(p))
    return torch.matmul(p, v.float()), lse


def _merge(o: torch.Tensor, lse: torch.Tensor, o2: torch.Tensor, lse2: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    new = torch.logaddexp(lse, lse2)
    w1 = torch.exp(lse - new).unsqueeze(-1)
    w2 = torch.exp(lse2 - new).unsqueeze(-1)
    w1 = torch.where(torch.isfinite(lse).unsqueeze(-1), w1, torch.zeros_like(w1))
    w2 = torch.where(torch.isfinite(lse2).unsqueeze(-1), w2, torch.zeros_like(w2))
    return o * w1 + o2 * w2, new


def shard_positions(rank: int, world: int, seq_local: int, layout: str = "contiguous", device=None) -> torch.Tensor:
    """Global sequence positions of the ``seq_local`` tokens rank ``rank`` holds.

    ``contiguous``: rank r holds ``[r * seq_local, (r + 1) * seq_local)``.
    ``zigzag``: the sequence is cut into ``2 * world`` chunks and rank r holds chunks ``r`` and
    ``2 * world - 1 - r`` - with a causal mask every rank then has the same amount of attention work,
    where the contiguous layout leaves rank 0 almost idle and the last rank with all of it.
    """
    if layout == "contiguous":
        return torch.arange(seq_local, device=device) + rank * seq_local
    if layout != "zigzag":
        raise ValueError(f"unknown layout '{layout}'")
    if seq_local % 2:
        raise ValueError("the zigzag layout needs an even number of local tokens")
    half = seq_local // 2
    lo = torch.arange(half, device=device) + rank * half
    hi = torch.arange(half, device=device) + (2 * world - 1 - rank) * half
    return torch.cat([lo, hi])


def zigzag_shard(x: torch.Tensor, rank: int, world: int, dim: int = -2) -> torch.Tensor:
    """This rank's part of a full-sequence tensor in the zigzag layout (sequence on ``dim``)."""
    chunks = x.chunk(2 * world, dim)
    return torch.cat([chunks[rank], chunks[2 * world - 1 - rank]], dim)


def zigzag_unshard(parts, dim: int = -2) -> torch.Tensor:
    """Inverse of ``zigzag_shard``: ``parts[r]`` is rank r's tensor; returns the full sequence."""
    world = len(parts)
    chunks = [None] * (2 * world)
    for r, p in enumerate(parts):
        lo, hi = p.chunk(2, dim)
        chunks[r], chunks[2 * world - 1 - r] = lo, hi
    return torch.cat(chunks, dim)


def _block_mask(rank: int, src: int, n: int, sq: int, layout: str, causal: bool, pos_q: torch.Tensor, device):
    """(skip, mask) for the local queries against the K/V block that rank ``src`` owns."""
    if not causal:
        return False, None
    if layout == "contiguous" and src > rank:
        return True, None                # that block lies entirely in the future
    if layout != "contiguous" or src == rank:
        pos_k = shard_positions(src, n, sq, layout, device)
        return False, pos_q.unsqueeze(-1) >= pos_k.unsqueeze(0)
    return False, None


def _ring_forward(q, k, v, comm: TorchComm, causal: bool, scale: float, layout: str) -> Tuple[torch.Tensor, torch.Tensor]:
    """fp32 output and row log-sum-exp of the local queries over the whole sequence."""
    n, rank = comm.get_size(), comm.get_rank()
    sq = q.shape[-2]
    nxt, prv = (rank + 1) % n, (rank - 1) % n
    kv = torch.stack([k, v]).contiguous()
    out = torch.zeros(q.shape, dtype=torch.float32, device=q.device)
    lse = torch.full(q.shape[:-1], float("-inf"), dtype=torch.float32, device=q.device)
    pos_q = shard_positions(rank, n, sq, layout, q.device)
    for step in range(n):
        src = (rank - step) % n          # whose K/V block we hold now
        work, incoming = None, None
        if step + 1 < n:
            incoming = torch.empty_like(kv)
            batch = comm.batch_op_create()
            batch.send(kv, nxt)
            batch.recv(incoming, prv)
            work = batch.issue(True)
        skip, mask = _block_mask(rank, src, n, sq, layout, causal, pos_q, q.device)
        if not skip:
            o2, l2 = _block_attention(q, kv[0], kv[1], scale, mask)
            out, lse = _merge(out, lse, o2, l2)
        if work is not None:
            work.wait()
            kv = incoming
    return out, lse


def _ring_backward(q, k, v, out, lse, dout, comm: TorchComm, causal: bool, scale: float, layout: str):
    """Gradients of the local q, k, v. The K/V blocks go round the ring once more, each with an accumulator for its
    gradient that every rank adds its queries' contribution to; one last hop brings the accumulator home."""
    n, rank = comm.get_size(), comm.get_rank()
    sq = q.shape[-2]
    nxt, prv = (rank + 1) % n, (rank - 1) % n
    qf, do = q.float(), dout.float()
    delta = (do * out).sum(-1)                                  # [b, h, sq]
    finite = torch.isfinite(lse).unsqueeze(-1)
    lse_safe = lse.clamp_min(-1e30).unsqueeze(-1)
    dq = torch.zeros_like(qf)
    kv = torch.stack([k, v]).contiguous()
    dkv = torch.zeros(kv.shape, dtype=torch.float32, device=q.device)
    pos_q = shard_positions(rank, n, sq, layout, q.device)
    for step in range(n):
        src = (rank - step) % n
        skip, mask = _block_mask(rank, src, n, sq, layout, causal, pos_q, q.device)
        if not skip:
            kf, vf = kv[0].float(), kv[1].float()
            s = torch.matmul(qf, kf.transpose(-1, -2)) * scale
            if mask is not None:
                s = s.masked_fill(~mask, float("-inf"))
            p = torch.where(finite, torch.exp(s - lse_safe), torch.zeros_like(s))
            dp = torch.matmul(do, vf.transpose(-1, -2))
            ds = p * (dp - delta.unsqueeze(-1))
            dq += torch.matmul(ds, kf) * scale
            dkv[0] += torch.matmul(ds.transpose(-1, -2), qf) * scale
            dkv[1] += torch.matmul(p.transpose(-1, -2), do)
        if n == 1:
            break
        batch = comm.batch_op_create()
        got_dkv = torch.empty_like(dkv)
        batch.send(dkv, nxt)
        batch.recv(got_dkv, prv)
        got_kv = None
        if step + 1 < n:
            got_kv = torch.empty_like(kv)
            batch.send(kv, nxt)
            batch.recv(got_kv, prv)
        batch.issue(False).wait()
        dkv = got_dkv
        if got_kv is not None:
            kv = got_kv
    return dq.to(q.dtype), dkv[0].to(k.dtype), dkv[1].to(v.dtype)


class _RingAttentionFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, k, v, comm, causal, scale, layout):
        out, lse = _ring_forward(q, k, v, comm, causal, scale, layout)
        ctx.save_for_backward(q, k, v, out, lse)
        ctx.comm, ctx.causal, ctx.scale, ctx.layout = comm, causal, scale, layout
        return out.to(q.dtype)

    @staticmethod
    def backward(ctx, dout):
        q, k, v, out, lse = ctx.saved_tensors
        dq, dk, dv = _ring_backward(q, k, v, out, lse, dout, ctx.comm, ctx.causal, ctx.scale, ctx.layout)
        return dq, dk, dv, None, None, None, None


def ring_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, comm: TorchComm, causal: bool = False,
                   scale: Optional[float] = None, layout: str = "contiguous") -> torch.Tensor:
    """q, k, v: [batch, heads, seq_local, head_dim]; which global positions the local tokens have is given by
    ``layout`` (see ``shard_positions``).  Differentiable: the backward pass is a second trip round the ring
    (every rank must run it, as it must the forward pass)."""
    scale = scale if scale is not None else 1.0 / math.sqrt(q.shape[-1])
    if torch.is_grad_enabled() and (q.requires_grad or k.requires_grad or v.requires_grad):
        return _RingAttentionFn.apply(q, k, v, comm, causal, scale, layout)
    return _ring_forward(q, k, v, comm, causal, scale, layout)[0].to(q.dtype)


def _all_to_all(send: torch.Tensor, comm: TorchComm) -> torch.Tensor:
    """Equal-split all-to-all along dim 0; through the differentiable operator when a gradient is wanted."""
    if send.requires_grad and torch.is_grad_enabled():
        from .. import functional as F

        return F.all_to_all_single(send, comm)
    recv = torch.empty_like(send)
    comm.all_to_all_single(recv, send, False)
    return recv


def _seq_to_heads(x: torch.Tensor, comm: TorchComm) -> torch.Tensor:
    """[b, h, s_local, d] -> [b, h/n, s_local*n, d]."""
    n = comm.get_size()
    b, h, s, d = x.shape
    send = x.reshape(b, n, h // n, s, d).permute(1, 0, 2, 3, 4).contiguous()   # [n(dest), b, h/n, s, d]
    recv = _all_to_all(send, comm)                                               # [n(src), b, h/n, s, d]
    return recv.permute(1, 2, 0, 3, 4).reshape(b, h // n, n * s, d)


def _heads_to_seq(x: torch.Tensor, comm: TorchComm) -> torch.Tensor:
    """[b, h/n, s_local*n, d] -> [b, h, s_local, d]."""
    n = comm.get_size()
    b, hn, sn, d = x.shape
    s = sn // n
    send = x.reshape(b, hn, n, s, d).permute(2, 0, 1, 3, 4).contiguous()        # [n(dest seq block), b, h/n, s, d]
    recv = _all_to_all(send, comm)                                               # [n(src head group), b, h/n, s, d]
    return recv.permute(1, 0, 2, 3, 4).reshape(b, n * hn, s, d)


class SeqHeadsExchange:
    """The two all-to-alls of Ulysses attention with their layout changes done inside the kernel (CUDA backend).

    ``to_heads``: ``[b, h, s_local, d]`` -> ``[b, h/n, n*s_local, d]``; ``to_seq``: the inverse.  Every ``[s_local, d]``
    slab goes from the caller's tensor straight to its place in the peer's output over NVLink, so the permuted
    copies that surround a plain ``all_to_all_single`` (one before, one after) disappear.  Outputs live in
    symmetric buffers that this object owns: one ring of ``slots`` buffers per (shape, dtype), allocated on first
    use (a collective call: every rank must use the object with the same sequence of shapes).  A result is valid
    until ``slots`` more exchanges of the same shape have been issued; when autograd records the call, or with
    ``keep=True``, the result is copied out of the ring.  Differentiable: the gradient of one direction is the
    other direction applied to the incoming gradient.

    On other backends, or with one rank, the calls fall back to ``all_to_all_single`` with explicit permutes.
    Counterpart in the reference tree: the scatter-gather collective of comms/ncclx/v2_31/contrib/pace
    (pace/sg/sgcomm.py), which fuses the same layout changes into its all-to-all.
    """

    def __init__(self, comm: TorchComm, slots: int = 4):
        self.comm = comm
        self.n = comm.get_size()
        self.slots = max(1, slots)
        impl = comm.get_backend_impl() if hasattr(comm, "get_backend_impl") else None
        self._impl = impl if impl is not None and hasattr(impl, "seq_heads_exchange") and self.n > 1 else None
        self._rings = {}

    @property
    def fused(self) -> bool:
        return self._impl is not None

    def _next(self, shape, dtype) -> torch.Tensor:
        key = (tuple(shape), dtype)
        ring = self._rings.get(key)
        if ring is None:
            ring = self._rings[key] = [[self._impl.symm_empty(list(shape), dtype) for _ in range(self.slots)], 0]
        buf = ring[0][ring[1] % self.slots]
        ring[1] += 1
        return buf

    def _run(self, x: torch.Tensor, to_heads: bool, keep: bool) -> torch.Tensor:
        b = x.shape[0]
        if to_heads:
            _, h, s, d = x.shape
            shape = (b, h // self.n, s * self.n, d)
        else:
            _, hn, sn, d = x.shape
            shape = (b, hn * self.n, sn // self.n, d)
        out = self._next(shape, x.dtype)
        self._impl.seq_heads_exchange(out, x.contiguous(), to_heads, False)
        return out.clone() if keep else out

    def to_heads(self, x: torch.Tensor, keep: bool = False) -> torch.Tensor:
        if x.shape[1] % self.n != 0:
            raise ValueError(f"heads ({x.shape[1]}) must divide by the number of ranks ({self.n})")
        if self._impl is None:
            return _seq_to_heads(x, self.comm) if self.n > 1 else x
        return _SeqHeadsFn.apply(x, self, True, keep)

    def to_seq(self, x: torch.Tensor, keep: bool = False) -> torch.Tensor:
        if x.shape[2] % self.n != 0:
            raise ValueError(f"sequence length ({x.shape[2]}) must divide by the number of ranks ({self.n})")
        if self._impl is None:
            return _heads_to_seq(x, self.comm) if self.n > 1 else x
        return _SeqHeadsFn.apply(x, self, False, keep)

    def close(self) -> None:
        """Gives the symmetric buffers back (collective)."""
        for ring in self._rings.values():
            for buf in ring[0]:
                self._impl.symm_free(buf)
        self._rings = {}


class _SeqHeadsFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, exchange, to_heads, keep):
        ctx.exchange, ctx.to_heads = exchange, to_heads
        return exchange._run(x, to_heads, keep or x.requires_grad)

    @staticmethod
    def backward(ctx, grad):
        return ctx.exchange._run(grad, not ctx.to_heads, True), None, None, None


def ulysses_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, comm: TorchComm, causal: bool = False,
                      scale: Optional[float] = None, exchange: Optional[SeqHeadsExchange] = None) -> torch.Tensor:
    """Same layout as ``ring_attention``; query heads and key / value heads (which may be fewer: grouped-query
    attention) must each divide by the communicator size.  With ``exchange`` (a ``SeqHeadsExchange`` of the same
    communicator) the four all-to-alls run as fused layout-changing kernels."""
    n = comm.get_size()
    for name, t in (("query", q), ("key / value", k)):
        if t.shape[1] % n != 0:
            raise ValueError(f"{name} heads ({t.shape[1]}) must divide by the number of ranks ({n})")
    grouped = q.shape[1] != k.shape[1]       # grouped-query attention: fewer key / value heads than query heads
    if exchange is not None:
        qh, kh, vh = (exchange.to_heads(t) for t in (q, k, v))
        o = torch.nn.functional.scaled_dot_product_attention(qh, kh, vh, is_causal=causal, scale=scale, enable_gqa=grouped)
        return exchange.to_seq(o)
    qh, kh, vh = (_seq_to_heads(t, comm) for t in (q, k, v))
    o = torch.nn.functional.scaled_dot_product_attention(qh, kh, vh, is_causal=causal, scale=scale, enable_gqa=grouped)
    return _heads_to_seq(o, comm)
