"""Redistribution of a tensor between two groups of ranks with different shardings.

A trainer group holds a tensor in one layout (say, sharded over 4 ranks along
dim 0), a generator group needs it in another (sharded over 2 ranks along dim 1,
each shard replicated twice).  ``reshard`` moves exactly the overlapping pieces
from the ranks that have them to the ranks that need them, in one batched
exchange, without gathering the tensor anywhere::

    from torchcomms_b200.ops.reshard import Mesh, Shard, REPLICATE, reshard

    src = Mesh(dims=(1, 4), start_rank=0, placement=(REPLICATE, Shard(0)))
    dst = Mesh(dims=(2, 2), start_rank=4, placement=(REPLICATE, Shard(1)))
    reshard(comm, src_local if rank < 4 else None, src, dst_local if rank >= 4 else None, dst)

A mesh is a 2-axis grid of consecutive ranks of the communicator; each axis
either replicates the tensor or shards one tensor dim evenly.  Every rank of the
communicator calls ``reshard`` with the same meshes (ranks in neither mesh pass
``None`` twice and take no part in the traffic).  Where a source tile exists in
several replicas, the readers are spread over them.  The groups may overlap: a
piece whose source and destination are the same rank is a local copy.

The transfer plan (``plan_transfers``) is a pure function of the meshes and the
global shape, so every rank derives the same list; pieces travel as one batch of
sends and receives on the communicator (grouped NCCL point-to-point on the CUDA
backend, pairs on gloo).

Counterpart in the reference tree: comms/ncclx/v2_31/contrib/nccl_m2n
(``ncclReshardWithWindow``: the same mesh / placement description, one-sided
through a registered window).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import List, Optional, Sequence, Tuple

import torch

from .. import TorchComm


@dataclass(frozen=True)
class Shard:
    """The mesh axis splits tensor dim ``dim`` evenly among its members."""

    dim: int


REPLICATE = None
Placement = Optional[Shard]


@dataclass(frozen=True)
class Mesh:
    """``dims[0] * dims[1]`` consecutive ranks from ``start_rank`` on, row-major; one placement per axis."""

    dims: Tuple[int, int]
    start_rank: int
    placement: Tuple[Placement, Placement]

    def __post_init__(self):
        if len(self.dims) != 2 or len(self.placement) != 2 or min(self.dims) < 1:
            raise ValueError("a mesh has two axes of at least one rank each")
        sharded = [p.dim for p in self.placement if p is not None]
        if len(set(sharded)) != len(sharded):
            raise ValueError("both mesh axes shard the same tensor dim")

    @property
    def size(self) -> int:
        return self.dims[0] * self.dims[1]

    def ranks(self) -> range:
        return range(self.start_rank, self.start_rank + self.size)

    def coords(self, rank: int) -> Tuple[int, int]:
        return divmod(rank - self.start_rank, self.dims[1])

    def shards(self, ndim: int) -> List[int]:
        """How many pieces each tensor dim is cut into."""
        out = [1] * ndim
        for axis, p in enumerate(self.placement):
            if p is not None:
                if not 0 <= p.dim < ndim:
                    raise ValueError(f"Shard({p.dim}) on a tensor with {ndim} dims")
                out[p.dim] = self.dims[axis]
        return out

    def tile_index(self, rank: int, ndim: int) -> List[int]:
        """Which piece of each tensor dim ``rank`` holds."""
        out = [0] * ndim
        c = self.coords(rank)
        for axis, p in enumerate(self.placement):
            if p is not None:
                out[p.dim] = c[axis]
        return out

    def replica_index(self, rank: int) -> int:
        """Position of ``rank`` among the ranks that hold the same tile."""
        idx = 0
        c = self.coords(rank)
        for axis, p in enumerate(self.placement):
            if p is None:
                idx = idx * self.dims[axis] + c[axis]
        return idx

    def holders(self, tile: Sequence[int]) -> List[int]:
        """Ranks that hold tile ``tile`` (one per replica), in replica order."""
        ndim = len(tile)
        return [r for r in self.ranks() if self.tile_index(r, ndim) == list(tile)]

    def local_shape(self, global_shape: Sequence[int]) -> Tuple[int, ...]:
        cuts = self.shards(len(global_shape))
        for d, (g, c) in enumerate(zip(global_shape, cuts)):
            if g % c != 0:
                raise ValueError(f"dim {d} of size {g} does not divide into {c} shards")
        return tuple(g // c for g, c in zip(global_shape, cuts))


@dataclass(frozen=True)
class Transfer:
    """One piece: ``src_slices`` of the source rank's tile go to ``dst_slices`` of the destination rank's tile."""

    src_rank: int
    dst_rank: int
    src_slices: Tuple[Tuple[int, int], ...]     # (start, stop) per dim, in the source tile's coordinates
    dst_slices: Tuple[Tuple[int, int], ...]

    @property
    def shape(self) -> Tuple[int, ...]:
        return tuple(b - a for a, b in self.src_slices)


def plan_transfers(global_shape: Sequence[int], src: Mesh, dst: Mesh) -> List[Transfer]:
    """Every piece that has to move, in an order that is the same on every rank."""
    ndim = len(global_shape)
    s_shape, d_shape = src.local_shape(global_shape), dst.local_shape(global_shape)
    s_cuts = src.shards(ndim)
    out: List[Transfer] = []
    for dst_rank in dst.ranks():
        d_tile = dst.tile_index(dst_rank, ndim)
        lo = [t * n for t, n in zip(d_tile, d_shape)]
        hi = [a + n for a, n in zip(lo, d_shape)]
        # source tiles that overlap [lo, hi) in every dim
        spans = [range(lo[d] // s_shape[d], (hi[d] - 1) // s_shape[d] + 1) for d in range(ndim)]
        tiles = [[]]
        for d in range(ndim):
            tiles = [t + [i] for t in tiles for i in spans[d] if i < s_cuts[d]]
        for k, tile in enumerate(tiles):
            holders = src.holders(tile)
            # the same rank if it has the tile (no traffic), else spread the readers over the replicas
            src_rank = dst_rank if dst_rank in holders else holders[(dst_rank - dst.start_rank + k) % len(holders)]
            s_lo = [t * n for t, n in zip(tile, s_shape)]
            a = [max(lo[d], s_lo[d]) for d in range(ndim)]
            b = [min(hi[d], s_lo[d] + s_shape[d]) for d in range(ndim)]
            out.append(Transfer(src_rank, dst_rank,
                                tuple((a[d] - s_lo[d], b[d] - s_lo[d]) for d in range(ndim)),
                                tuple((a[d] - lo[d], b[d] - lo[d]) for d in range(ndim))))
    return out


def _view(t: torch.Tensor, slices: Sequence[Tuple[int, int]]) -> torch.Tensor:
    return t[tuple(slice(a, b) for a, b in slices)]


def reshard(comm: TorchComm, src_local: Optional[torch.Tensor], src: Mesh, dst_local: Optional[torch.Tensor], dst: Mesh,
            global_shape: Optional[Sequence[int]] = None, async_op: bool = False):
    """Fills ``dst_local`` on the ranks of ``dst`` from the tiles ``src_local`` on the ranks of ``src``.

    ``global_shape`` may be omitted when this rank holds a tile (it follows from the tile and the mesh); ranks that
    hold none must pass it.  Returns ``None``, or with ``async_op=True`` an object whose ``wait()`` completes the
    receives and puts the pieces in place.
    """
    rank = comm.get_rank()
    in_src, in_dst = rank in src.ranks(), rank in dst.ranks()
    if in_src != (src_local is not None) or in_dst != (dst_local is not None):
        raise ValueError("pass a tile exactly on the ranks of the corresponding mesh")
    if src.start_rank < 0 or dst.start_rank < 0 or max(src.ranks()[-1], dst.ranks()[-1]) >= comm.get_size():
        raise ValueError("mesh ranks outside the communicator")
    if global_shape is None:
        if src_local is not None:
            global_shape = [n * c for n, c in zip(src_local.shape, src.shards(src_local.dim()))]
        elif dst_local is not None:
            global_shape = [n * c for n, c in zip(dst_local.shape, dst.shards(dst_local.dim()))]
        else:
            raise ValueError("a rank in neither mesh must be given global_shape")
    global_shape = list(global_shape)
    if src_local is not None and tuple(src_local.shape) != src.local_shape(global_shape):
        raise ValueError(f"source tile is {tuple(src_local.shape)}, the mesh implies {src.local_shape(global_shape)}")
    if dst_local is not None and tuple(dst_local.shape) != dst.local_shape(global_shape):
        raise ValueError(f"destination tile is {tuple(dst_local.shape)}, the mesh implies {dst.local_shape(global_shape)}")

    batch = comm.batch_op_create()
    landed: List[Tuple[torch.Tensor, torch.Tensor]] = []     # (received buffer, where it goes)
    keep: List[torch.Tensor] = []
    issued = False
    for t in plan_transfers(global_shape, src, dst):
        if t.src_rank == rank and t.dst_rank == rank:
            _view(dst_local, t.dst_slices).copy_(_view(src_local, t.src_slices))
        elif t.src_rank == rank:
            piece = _view(src_local, t.src_slices).contiguous()
            keep.append(piece)
            batch.send(piece, t.dst_rank)
            issued = True
        elif t.dst_rank == rank:
            where = _view(dst_local, t.dst_slices)
            buf = where if where.is_contiguous() else torch.empty(t.shape, dtype=dst_local.dtype, device=dst_local.device)
            if buf is not where:
                landed.append((buf, where))
            batch.recv(buf, t.src_rank)
            issued = True
    work = batch.issue(async_op) if issued else None
    done = _ReshardWork(work, landed, keep)
    if async_op:
        return done
    done.wait()
    return None


class _ReshardWork:
    def __init__(self, work, landed, keep):
        self._work, self._landed, self._keep = work, landed, keep

    def wait(self) -> bool:
        if self._work is not None:
            self._work.wait()
            self._work = None
        for buf, where in self._landed:
            where.copy_(buf)
        self._landed, self._keep = [], []
        return True


__all__ = ["Mesh", "Shard", "REPLICATE", "Transfer", "plan_transfers", "reshard"]
