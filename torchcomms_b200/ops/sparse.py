"""All-reduce of sparse blocks: every rank contributes a few fixed-length blocks of a large
vector (an embedding-gradient pattern) and every rank receives the dense sum.

    all_reduce_sparse_block(comm, send, recv_indices, block_length, recv)

``send`` holds ``len(recv_indices)`` blocks of ``block_length`` elements back to back;
``recv_indices[i]`` is the element offset of block ``i`` in the dense result ``recv``
(length ``recv_count``).  Blocks of different ranks may coincide (they are summed) and
positions nobody contributes to are zero.

Two routes, picked identically on all ranks from the exchanged block counts:

* ``gather``: all-gather the (index, block) pairs and scatter-add them locally - traffic is
  proportional to the number of blocks;
* ``dense``: scatter the blocks into a zeroed dense vector and all-reduce it - better once
  the blocks of all ranks together approach the dense size.

Parity: ``ncclAllReduceSparseBlock`` of the reference's NCCL fork
(comms/ncclx/v2_30/src/nccl.h.in:560-589, kernel all_reduce_sparse_block.cu); the example in
that header is the golden vector of this module's test.
"""
from __future__ import annotations

from typing import Optional

import torch

from .. import ReduceOp, TorchComm


def all_reduce_sparse_block(comm: TorchComm, send: torch.Tensor, recv_indices: torch.Tensor, block_length: int,
                            recv: torch.Tensor, mode: str = "auto") -> torch.Tensor:
    if mode not in ("auto", "gather", "dense"):
        raise ValueError(f"mode must be auto, gather or dense, got {mode}")
    n_blocks = int(recv_indices.numel())
    if send.numel() != n_blocks * block_length:
        raise ValueError(f"send has {send.numel()} elements, expected {n_blocks} blocks of {block_length}")
    if recv.dim() != 1 or not recv.is_contiguous():
        raise ValueError("recv must be a contiguous 1-D tensor")
    if n_blocks and (int(recv_indices.min()) < 0 or int(recv_indices.max()) + block_length > recv.numel()):
        raise ValueError("a block lies outside recv")
    world = comm.get_size()
    dev = recv.device
    idx = recv_indices.to(device=dev, dtype=torch.int64).contiguous()
    blocks = send.reshape(n_blocks, block_length).to(dev)

    counts = torch.zeros(world, dtype=torch.int64, device=dev)
    if world > 1:
        comm.all_gather_single(counts, torch.tensor([n_blocks], dtype=torch.int64, device=dev), False)
    else:
        counts[0] = n_blocks
    total = int(counts.sum())
    if mode == "auto":
        # gathered traffic per rank: every block plus its 8-byte index; dense traffic: 2 x the vector
        gathered = total * (block_length * recv.element_size() + 8)
        mode = "gather" if gathered < 2 * recv.numel() * recv.element_size() else "dense"

    offsets = (idx.unsqueeze(1) + torch.arange(block_length, device=dev).unsqueeze(0)).reshape(-1)
    if mode == "dense" or world == 1:
        recv.zero_()
        recv.index_add_(0, offsets, blocks.reshape(-1).to(recv.dtype))
        if world > 1:
            comm.all_reduce(recv, ReduceOp.SUM, False)
        return recv

    sizes = [int(c) for c in counts.tolist()]
    all_idx = [torch.empty(c, dtype=torch.int64, device=dev) for c in sizes]
    all_blk = [torch.empty(c * block_length, dtype=recv.dtype, device=dev) for c in sizes]
    comm.all_gather_v(all_idx, idx, False)
    comm.all_gather_v(all_blk, blocks.reshape(-1).to(recv.dtype).contiguous(), False)
    recv.zero_()
    span = torch.arange(block_length, device=dev).unsqueeze(0)
    for r in range(world):                                   # rank order: every rank rounds alike
        if sizes[r]:
            recv.index_add_(0, (all_idx[r].unsqueeze(1) + span).reshape(-1), all_blk[r])
    return recv


__all__ = ["all_reduce_sparse_block"]
