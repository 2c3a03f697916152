"""Redistribution between rank groups with different shardings (ops.reshard): the transfer plan as a pure function,
and the exchange over gloo ranks against slices of a known global tensor.

Parity: the host-side plan tests and basic_api tests of comms/ncclx/v2_31/contrib/nccl_m2n/tests (same-dim and
cross-dim sharding, replicated sources and destinations).
"""
from datetime import timedelta

import pytest
import torch

from tests.mp_util import run_ranks
from torchcomms_b200.ops.reshard import REPLICATE, Mesh, Shard, plan_transfers


def _tile(full, mesh, rank):
    idx = mesh.tile_index(rank, full.dim())
    shape = mesh.local_shape(full.shape)
    return full[tuple(slice(i * n, (i + 1) * n) for i, n in zip(idx, shape))]


def test_plan_covers_every_destination_element_exactly_once():
    cases = [
        ((8, 12), Mesh((1, 4), 0, (REPLICATE, Shard(0))), Mesh((1, 2), 4, (REPLICATE, Shard(0)))),      # same dim, 4 -> 2
        ((8, 12), Mesh((1, 2), 0, (REPLICATE, Shard(0))), Mesh((1, 4), 2, (REPLICATE, Shard(0)))),      # same dim, 2 -> 4
        ((8, 12), Mesh((1, 4), 0, (REPLICATE, Shard(0))), Mesh((2, 3), 4, (REPLICATE, Shard(1)))),      # cross dim, replicated dst
        ((8, 12, 4), Mesh((2, 2), 0, (Shard(0), Shard(2))), Mesh((3, 1), 4, (Shard(1), REPLICATE))),    # two sharded dims
        ((6, 6), Mesh((2, 1), 0, (REPLICATE, REPLICATE)), Mesh((1, 3), 2, (REPLICATE, Shard(1)))),      # replicated source
    ]
    for shape, src, dst in cases:
        full = torch.arange(int(torch.tensor(shape).prod())).view(shape)
        plan = plan_transfers(shape, src, dst)
        got = {r: torch.full(dst.local_shape(shape), -1, dtype=torch.int64) for r in dst.ranks()}
        seen = {r: torch.zeros(dst.local_shape(shape), dtype=torch.int64) for r in dst.ranks()}
        for t in plan:
            assert t.src_rank in src.ranks() and t.dst_rank in dst.ranks()
            piece = _tile(full, src, t.src_rank)[tuple(slice(a, b) for a, b in t.src_slices)]
            where = tuple(slice(a, b) for a, b in t.dst_slices)
            got[t.dst_rank][where] = piece
            seen[t.dst_rank][where] += 1
        for r in dst.ranks():
            assert torch.equal(got[r], _tile(full, dst, r)), (shape, src, dst, r)
            assert bool((seen[r] == 1).all())
    # replicas of a source tile share the readers
    src, dst = Mesh((2, 1), 0, (REPLICATE, REPLICATE)), Mesh((1, 4), 2, (REPLICATE, Shard(0)))
    readers = [t.src_rank for t in plan_transfers((8, 4), src, dst)]
    assert sorted(set(readers)) == [0, 1] and readers.count(0) == readers.count(1)


def test_random_meshes_and_shapes_are_planned_correctly():
    """Seeded sweep over mesh sizes, placements and tensor ranks (1 to 3 dims), overlapping rank ranges included."""
    import random

    rng = random.Random(7)

    def random_mesh(ndim, start):
        dims = (rng.choice([1, 2, 3]), rng.choice([1, 2, 4]))
        free = list(range(ndim))
        rng.shuffle(free)
        placement = []
        for _ in range(2):
            if free and rng.random() < 0.6:
                placement.append(Shard(free.pop()))
            else:
                placement.append(REPLICATE)
        return Mesh(dims, start, tuple(placement))

    for _ in range(200):
        ndim = rng.choice([1, 2, 3])
        shape = tuple(rng.choice([12, 24]) for _ in range(ndim))
        src = random_mesh(ndim, 0)
        dst = random_mesh(ndim, rng.choice([0, src.size, max(0, src.size - 1)]))
        full = torch.arange(int(torch.tensor(shape).prod())).view(shape)
        seen = {r: torch.zeros(dst.local_shape(shape), dtype=torch.int64) for r in dst.ranks()}
        for t in plan_transfers(shape, src, dst):
            piece = _tile(full, src, t.src_rank)[tuple(slice(a, b) for a, b in t.src_slices)]
            where = tuple(slice(a, b) for a, b in t.dst_slices)
            assert torch.equal(piece, _tile(full, dst, t.dst_rank)[where]), (shape, src, dst, t)
            seen[t.dst_rank][where] += 1
            if t.dst_rank in src.holders(src.tile_index(t.src_rank, ndim)):
                assert t.src_rank == t.dst_rank          # a rank that has the tile itself does not fetch it
        assert all(bool((m == 1).all()) for m in seen.values()), (shape, src, dst)


def test_mesh_validation():
    with pytest.raises(ValueError):
        Mesh((2, 2), 0, (Shard(0), Shard(0)))
    with pytest.raises(ValueError):
        Mesh((1, 4), 0, (REPLICATE, Shard(0))).local_shape((6, 4))        # 6 rows do not divide into 4 shards
    with pytest.raises(ValueError):
        Mesh((1, 2), 0, (REPLICATE, Shard(3))).shards(2)


def _reshard_worker(rank, world):
    import torchcomms_b200 as tc
    from torchcomms_b200.ops.reshard import reshard

    comm = tc.new_comm("gloo", torch.device("cpu"), name="reshard", timeout=timedelta(seconds=60))
    full = torch.arange(8 * 12, dtype=torch.float32).view(8, 12)
    cases = [
        (Mesh((1, 4), 0, (REPLICATE, Shard(0))), Mesh((1, 2), 4, (REPLICATE, Shard(0)))),
        (Mesh((1, 4), 0, (REPLICATE, Shard(0))), Mesh((1, 2), 4, (REPLICATE, Shard(1)))),      # cross dim: strided pieces
        (Mesh((2, 2), 0, (REPLICATE, Shard(1))), Mesh((2, 1), 4, (Shard(0), REPLICATE))),      # replicated source
        (Mesh((1, 6), 0, (REPLICATE, Shard(1))), Mesh((2, 2), 1, (Shard(0), Shard(1)))),       # overlapping groups
    ]
    for i, (src, dst) in enumerate(cases):
        s_local = _tile(full, src, rank).clone() if rank in src.ranks() else None
        d_local = torch.full(dst.local_shape(full.shape), -1.0) if rank in dst.ranks() else None
        if i % 2 == 0:
            reshard(comm, s_local, src, d_local, dst, global_shape=full.shape)
        else:
            reshard(comm, s_local, src, d_local, dst, global_shape=full.shape, async_op=True).wait()
        if d_local is not None:
            assert torch.equal(d_local, _tile(full, dst, rank)), (i, rank)
    # the global shape follows from a tile; a rank without one has to be told
    src, dst = cases[0]
    if rank in src.ranks() or rank in dst.ranks():
        s_local = _tile(full, src, rank).clone() if rank in src.ranks() else None
        d_local = torch.empty(dst.local_shape(full.shape)) if rank in dst.ranks() else None
        reshard(comm, s_local, src, d_local, dst)
        if d_local is not None:
            assert torch.equal(d_local, _tile(full, dst, rank))
    with pytest.raises(ValueError):
        reshard(comm, torch.zeros(3, 3), Mesh((1, 1), (rank + 1) % world, (REPLICATE, REPLICATE)), None, dst, global_shape=(3, 3))
    comm.finalize()


def test_reshard_between_groups_over_gloo():
    run_ranks(_reshard_worker, 6, timeout=240)
