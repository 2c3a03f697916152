"""Context (sequence) parallel attention: ring attention and Ulysses.

Both shard the sequence over the ranks of a communicator.

* ``ring_attention``: K/V blocks travel around the ring in ``n - 1`` batched
  send/recv steps while each rank attends its local queries to the block it
  currently holds; partial results are merged with the running log-sum-exp,
  so the full score matrix never exists.  The transfer of step ``i + 1`` is
  issued before the math of step ``i`` (asynchronous batch on the
  communicator's side stream) and waited for afterwards.
  With ``layout="zigzag"`` (``zigzag_shard`` / ``zigzag_unshard``) causal attention is
  load-balanced over the ranks.
* ``ulysses_attention``: one all-to-all turns sequence shards into head
  shards, attention runs locally over the full sequence for ``heads / n``
  heads, a second all-to-all turns the result back.

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


def ring_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, comm: TorchComm, causal: bool = False,
                   scale: Optional[float] = None, layout: str = "contiguous") -> torch.Tensor:
    """q, k, v: [batch, heads, seq_local, head_dim]; which global positions the local tokens have is given by
    ``layout`` (see ``shard_positions``)."""
    n, rank = comm.get_size(), comm.get_rank()
    sq, d = q.shape[-2], q.shape[-1]
    scale = scale if scale is not None else 1.0 / math.sqrt(d)
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
        mask = None
        skip = False
        if causal:
            pos_k = shard_positions(src, n, sq, layout, q.device)
            if layout == "contiguous" and src > rank:
                skip = True              # that block lies entirely in the future
            elif layout != "contiguous" or src == rank:
                mask = pos_q.unsqueeze(-1) >= pos_k.unsqueeze(0)
        if not skip:
            o2, l2 = _block_attention(q, kv[0], kv[1], scale, mask)
            out, lse = _merge(out, lse, o2, l2)
        if work is not None:
            work.wait()
            kv = incoming
    return out.to(q.dtype)


def _seq_to_heads(x: torch.Tensor, comm: TorchComm) -> torch.Tensor:
    """[b, h, s_local, d] -> [b, h/n, s_local*n, d]."""
    n = comm.get_size()
    b, h, s, d = x.shape
    send = x.reshape(b, n, h // n, s, d).permute(1, 0, 2, 3, 4).contiguous()   # [n(dest), b, h/n, s, d]
    recv = torch.empty_like(send)
    comm.all_to_all_single(recv, send, False)                                    # [n(src), b, h/n, s, d]
    return recv.permute(1, 2, 0, 3, 4).reshape(b, h // n, n * s, d)


def _heads_to_seq(x: torch.Tensor, comm: TorchComm) -> torch.Tensor:
    """[b, h/n, s_local*n, d] -> [b, h, s_local, d]."""
    n = comm.get_size()
    b, hn, sn, d = x.shape
    s = sn // n
    send = x.reshape(b, hn, n, s, d).permute(2, 0, 1, 3, 4).contiguous()        # [n(dest seq block), b, h/n, s, d]
    recv = torch.empty_like(send)
    comm.all_to_all_single(recv, send, False)                                    # [n(src head group), b, h/n, s, d]
    return recv.permute(1, 0, 2, 3, 4).reshape(b, n * hn, s, d)


def ulysses_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, comm: TorchComm, causal: bool = False,
                      scale: Optional[float] = None) -> torch.Tensor:
    """Same layout as ``ring_attention``; ``heads`` must divide by the communicator size."""
    n = comm.get_size()
    if q.shape[1] % n != 0:
        raise ValueError(f"heads ({q.shape[1]}) must divide by the number of ranks ({n})")
    qh, kh, vh = (_seq_to_heads(t, comm) for t in (q, k, v))
    o = torch.nn.functional.scaled_dot_product_attention(qh, kh, vh, is_causal=causal, scale=scale)
    return _heads_to_seq(o, comm)
