"""Less-travelled parts of the communicator API on gloo ranks: persistent all-gather,
gather / scatter / all_to_all lists, PREMUL_SUM and AVG, per-call timeouts and hints,
use after finalize.

Modelled on comms/torchcomms/tests/integration/py/AllGatherPTest.py, GatherTest.py,
ScatterTest.py, AllToAllTest.py, OptionsTest.py and FinalizeWarningTest.py.
"""
import os
from datetime import timedelta

import pytest
import torch

from tests.mp_util import run_ranks


def _worker(rank, world):
    import torchcomms_b200 as tc

    comm = tc.new_comm("gloo", torch.device("cpu"), name="corners", timeout=timedelta(seconds=60), hints={"note": "x"})
    assert comm.get_options().hints.get("note") == "x" and comm.get_options().timeout == timedelta(seconds=60)

    # persistent all-gather: the output is bound once, executed many times with fresh inputs
    out = torch.zeros(world * 4)
    handle = comm.all_gather_p_init(out)
    for it in range(3):
        w = comm.all_gather_p_exec(handle, torch.full((4,), float(10 * it + rank)), it % 2 == 1)
        w.wait()
        assert torch.equal(out, torch.tensor([float(10 * it + r) for r in range(world)]).repeat_interleave(4))
    comm.all_gather_p_free(handle)
    with pytest.raises(RuntimeError):
        comm.all_gather_p_exec(handle, torch.zeros(4), False)

    # gather / scatter with lists (only the root's lists matter), all_to_all with lists
    outs = [torch.zeros(2) for _ in range(world)] if rank == 1 else []
    comm.gather(outs, torch.full((2,), float(rank)), 1, False)
    if rank == 1:
        assert [o[0].item() for o in outs] == [float(r) for r in range(world)]
    got = torch.zeros(3)
    comm.scatter(got, [torch.full((3,), float(100 + r)) for r in range(world)] if rank == 0 else [], 0, False)
    assert torch.equal(got, torch.full((3,), float(100 + rank)))
    recv = [torch.zeros(1) for _ in range(world)]
    comm.all_to_all(recv, [torch.tensor([float(10 * rank + p)]) for p in range(world)], False)
    assert [t.item() for t in recv] == [float(10 * p + rank) for p in range(world)]
    gs = torch.zeros(world, 2) if rank == 0 else torch.zeros(0)
    comm.gather_single(gs, torch.full((1, 2), float(rank)), 0, False)
    if rank == 0:
        assert torch.equal(gs[:, 0], torch.arange(world, dtype=torch.float32))

    # PREMUL_SUM (host factor and tensor factor) and AVG
    t = torch.full((4,), float(rank + 1))
    comm.all_reduce(t, tc.ReduceOp.PREMUL_SUM(0.5), False)
    assert torch.equal(t, torch.full((4,), 0.5 * sum(range(1, world + 1))))
    t = torch.full((4,), float(rank + 1))
    comm.all_reduce(t, tc.ReduceOp.PREMUL_SUM(torch.tensor(2.0)), False)
    assert torch.equal(t, torch.full((4,), 2.0 * sum(range(1, world + 1))))
    t = torch.full((4,), float(rank + 1))
    comm.all_reduce(t, tc.ReduceOp.AVG, False)
    assert torch.allclose(t, torch.full((4,), sum(range(1, world + 1)) / world))
    ti = torch.full((4,), rank + 1, dtype=torch.int64)
    comm.all_reduce(ti, tc.ReduceOp.BOR, False)                # bitwise operators on integral types
    assert int(ti[0]) == (1 | 2 if world == 2 else int(ti[0]))

    # shape rules are checked before anything is sent
    with pytest.raises(RuntimeError):
        comm.all_gather_single(torch.zeros(world * 4 + 1), torch.zeros(4), False)
    with pytest.raises(RuntimeError):
        comm.reduce_scatter_single(torch.zeros(3), torch.zeros(3 * world + 1), tc.ReduceOp.SUM, False)
    with pytest.raises(RuntimeError):
        comm.all_reduce(torch.zeros(4, 4).t(), tc.ReduceOp.SUM, False)      # not contiguous
    with pytest.raises(RuntimeError):
        comm.send(torch.zeros(1), world, False)                             # rank out of range

    # per-call timeout and hints are accepted on every operation
    t = torch.ones(2)
    comm.all_reduce(t, tc.ReduceOp.SUM, False, hints={"algo": "auto"}, timeout=timedelta(seconds=5))
    comm.barrier(False, timeout=timedelta(seconds=5))

    # use after finalize, and double finalize, raise
    comm.finalize()
    with pytest.raises(RuntimeError):
        comm.all_reduce(torch.ones(1), tc.ReduceOp.SUM, False)
    with pytest.raises(RuntimeError):
        comm.finalize()


def test_api_corners_on_gloo():
    run_ranks(_worker, 2, timeout=120)


def _sparse_worker(rank, world):
    import torchcomms_b200 as tc
    from torchcomms_b200.ops.sparse import all_reduce_sparse_block

    comm = tc.new_comm("gloo", torch.device("cpu"), name="sparse", timeout=timedelta(seconds=60))
    # the worked example of comms/ncclx/v2_30/src/nccl.h.in:574-584 (block length 2, 14 elements)
    contrib = {
        0: ([1, 2, 3, 6, 7], [0, 2, 4, 10, 12]),
        1: ([2, 3, 5, 6], [2, 4, 8, 10]),
        2: ([1, 3, 4, 6], [0, 4, 6, 10]),
        3: ([1, 2, 3, 4, 5, 6, 7], [0, 2, 4, 6, 8, 10, 12]),
    }
    vals, idx = contrib[rank]
    send = torch.tensor(vals, dtype=torch.float32).repeat_interleave(2)
    expect = torch.tensor([3, 3, 6, 6, 12, 12, 8, 8, 10, 10, 24, 24, 14, 14], dtype=torch.float32)
    for mode in ("gather", "dense", "auto"):
        recv = torch.full((14,), -1.0)
        all_reduce_sparse_block(comm, send, torch.tensor(idx), 2, recv, mode=mode)
        assert torch.equal(recv, expect), (mode, recv)
    # a rank with nothing to contribute, and a sparse case where the gather route is chosen
    big = torch.full((4096,), -1.0)
    mine = torch.tensor([128 * rank]) if rank % 2 == 0 else torch.empty(0, dtype=torch.int64)
    all_reduce_sparse_block(comm, torch.ones(mine.numel() * 4), mine, 4, big)
    ref = torch.zeros(4096)
    for r in range(0, world, 2):
        ref[128 * r:128 * r + 4] = 1
    assert torch.equal(big, ref)
    with pytest.raises(ValueError):
        all_reduce_sparse_block(comm, torch.ones(4), torch.tensor([4094]), 4, big)
    comm.finalize()


def test_all_reduce_sparse_block():
    run_ranks(_sparse_worker, 4, timeout=120)


def _options_worker(rank, world):
    """Every operation takes ``hints=`` and ``timeout=`` (OptionsTest.py of the reference)."""
    import torchcomms_b200 as tc

    comm = tc.new_comm("gloo", torch.device("cpu"), name="opts", timeout=timedelta(seconds=60))
    kw = {"hints": {"example": "1"}, "timeout": timedelta(seconds=600)}
    peer = 1 - rank
    t = torch.full((4,), float(rank))
    if rank == 0:
        comm.send(t, peer, False, **kw)
        comm.recv(t, peer, False, **kw)
    else:
        got = torch.empty(4)
        comm.recv(got, peer, False, **kw)
        comm.send(got + 1, peer, False, **kw)
    comm.broadcast(t, 0, False, **kw)
    comm.all_reduce(t, tc.ReduceOp.SUM, False, **kw)
    comm.reduce(t, 0, tc.ReduceOp.SUM, False, **kw)
    out = torch.empty(world * 4)
    comm.all_gather_single(out, t, False, **kw)
    comm.all_gather([torch.empty(4) for _ in range(world)], t, False, **kw)
    comm.all_gather_v([torch.empty(4) for _ in range(world)], t, False, **kw)
    comm.gather([torch.empty(4) for _ in range(world)] if rank == 0 else [], t, 0, False, **kw)
    comm.gather_single(torch.empty(world * 4) if rank == 0 else torch.empty(0), t, 0, False, **kw)
    rs = torch.empty(2)
    comm.reduce_scatter_single(rs, torch.ones(2 * world), tc.ReduceOp.SUM, False, **kw)
    comm.reduce_scatter(rs, [torch.ones(2) for _ in range(world)], tc.ReduceOp.SUM, False, **kw)
    comm.reduce_scatter_v(rs, [torch.ones(2) for _ in range(world)], tc.ReduceOp.SUM, False, **kw)
    comm.scatter(rs, [torch.ones(2) for _ in range(world)] if rank == 0 else [], 0, False, **kw)
    comm.all_to_all([torch.empty(1) for _ in range(world)], [torch.ones(1) for _ in range(world)], False, **kw)
    a2a = torch.empty(world)
    comm.all_to_all_single(a2a, torch.ones(world), False, **kw)
    comm.all_to_all_v_single(a2a, torch.ones(world), [1] * world, [1] * world, False, **kw)
    comm.barrier(False, **kw)
    batch = comm.batch_op_create()
    box = torch.empty(1)
    batch.send(torch.ones(1), peer)
    batch.recv(box, peer)
    bo = tc.BatchP2POptions()
    bo.hints = {"example": "1"}
    bo.timeout = timedelta(seconds=600)
    batch.issue(False, bo).wait()
    sub = comm.split(list(range(world)), "sub", **kw)
    assert sub.get_size() == world
    handle = comm.all_gather_p_init(out, **kw)
    comm.all_gather_p_exec(handle, t, False, **kw).wait()
    comm.all_gather_p_free(handle)
    # a per-call timeout that is too short for an absent peer is the call's own error, not the communicator's default
    sub.finalize()
    comm.finalize()


def test_every_operation_accepts_hints_and_timeout():
    run_ranks(_options_worker, 2, timeout=120)


def _split_worker(rank, world):
    """SplitTest.py and MultiCommTest.py of the reference: non-contiguous groups, invalid rank lists,
    splits of splits, communicators on separate and shared stores."""
    import torch.distributed as dist

    import torchcomms_b200 as tc

    comm = tc.new_comm("gloo", torch.device("cpu"), name="split_world", timeout=timedelta(seconds=60))
    # non-contiguous: even and odd ranks; the child's ranks are global ranks, its rank is the index in the list
    evens, odds = [0, 2], [1, 3]
    mine = evens if rank % 2 == 0 else odds
    child = None
    for group in (evens, odds):
        c = comm.split(group if rank in group else [], "parity")
        child = c if c is not None else child
    assert child.get_size() == 2 and child.get_rank() == mine.index(rank) and list(child.get_ranks()) == mine
    t = torch.tensor([float(rank)])
    child.all_reduce(t, tc.ReduceOp.SUM, False)
    assert t.item() == float(sum(mine))
    # invalid lists are refused before anything is exchanged
    with pytest.raises(RuntimeError):
        comm.split([0, 0, 1], "dup")
    with pytest.raises(RuntimeError):
        comm.split([(rank + 1) % world], "not_me")
    with pytest.raises(RuntimeError):
        comm.split([0, world], "out_of_range")
    # multi-level: split the child again into singletons
    leaf = None
    for i in range(2):
        c = child.split([i] if child.get_rank() == i else [], "leaf")
        leaf = c if c is not None else leaf
    assert leaf.get_size() == 1 and list(leaf.get_ranks()) == [rank]
    u = torch.tensor([5.0])
    leaf.all_reduce(u, tc.ReduceOp.SUM, False)
    assert u.item() == 5.0
    # the parent still works while children exist, in any interleaving
    w1 = comm.all_reduce(torch.ones(2), tc.ReduceOp.SUM, True)
    w2 = child.all_reduce(torch.ones(2), tc.ReduceOp.SUM, True)
    w2.wait()
    w1.wait()
    # communicators with their own stores and with a shared one, side by side
    port = int(os.environ["MASTER_PORT"])
    own = dist.TCPStore("127.0.0.1", port + 7, world, rank == 0, timeout=timedelta(seconds=60))
    shared = dist.PrefixStore("shared", own)
    a = tc.new_comm("gloo", torch.device("cpu"), name="store_a", store=own, timeout=timedelta(seconds=60))
    b = tc.new_comm("gloo", torch.device("cpu"), name="store_b", store=shared, timeout=timedelta(seconds=60))
    c3 = tc.new_comm("gloo", torch.device("cpu"), name="store_c", timeout=timedelta(seconds=60))     # default store
    for i, x in enumerate((a, b, c3)):
        v = torch.tensor([float(i + 1)])
        x.all_reduce(v, tc.ReduceOp.SUM, False)
        assert v.item() == float((i + 1) * world)
    for x in (c3, b, a, leaf, child, comm):
        x.finalize()


def test_split_cases_and_communicators_on_several_stores():
    run_ranks(_split_worker, 4, timeout=150)


def _variants_worker(rank, world):
    """The per-operation variants of the reference's integration tests (AllReduceTest.py:22-110): synchronous
    with and without keeping the work, asynchronous wait, work dropped early, input deleted before wait."""
    import gc

    import torchcomms_b200 as tc

    comm = tc.new_comm("gloo", torch.device("cpu"), name="variants", timeout=timedelta(seconds=60))
    total = float(sum(range(1, world + 1)))
    nxt, prv = (rank + 1) % world, (rank - 1) % world

    def fresh():
        return torch.full((64,), float(rank + 1))

    # synchronous, keeping the work / ignoring it
    t = fresh()
    w = comm.all_reduce(t, tc.ReduceOp.SUM, False)
    w.wait()
    assert torch.equal(t, torch.full((64,), total))
    t = fresh()
    comm.all_reduce(t, tc.ReduceOp.SUM, False)
    assert torch.equal(t, torch.full((64,), total))
    # asynchronous + wait
    t = fresh()
    comm.all_reduce(t, tc.ReduceOp.SUM, True).wait()
    assert torch.equal(t, torch.full((64,), total))
    # asynchronous, the work dropped before it was waited on: the operation still completes
    t = fresh()
    w = comm.all_reduce(t, tc.ReduceOp.SUM, True)
    w = None
    gc.collect()
    comm.barrier(False)
    assert torch.equal(t, torch.full((64,), total))
    # input deleted before the wait: the work keeps what it reads alive
    out = torch.empty(world * 64)
    src = fresh()
    w = comm.all_gather_single(out, src, True)
    del src
    gc.collect()
    w.wait()
    assert torch.equal(out.view(world, 64)[:, 0], torch.arange(1, world + 1, dtype=torch.float32))
    # the same five variants for a batch of send + recv around the ring
    for variant in ("sync", "sync_no_work", "async", "async_dropped", "input_deleted"):
        got = torch.zeros(8)
        payload = torch.full((8,), float(rank))
        batch = comm.batch_op_create()
        batch.send(payload, nxt)
        batch.recv(got, prv)
        if variant == "sync":
            batch.issue(False).wait()
        elif variant == "sync_no_work":
            batch.issue(False)
        elif variant == "async":
            batch.issue(True).wait()
        elif variant == "async_dropped":
            batch.issue(True)
            gc.collect()
            comm.barrier(False)
        else:
            w = batch.issue(True)
            del payload, batch
            gc.collect()
            w.wait()
        assert torch.equal(got, torch.full((8,), float(prv))), variant
    comm.finalize()


def test_operation_variants_sync_async_dropped_and_deleted_inputs():
    run_ranks(_variants_worker, 3, timeout=120)


def _matrix_worker(rank, world):
    from datetime import timedelta

    import torch
    import torchcomms_b200 as tc
    from tests.variant_matrix import VARIANTS_CPU, run_matrix

    comm = tc.new_comm("gloo", torch.device("cpu"), name="matrix", timeout=timedelta(seconds=60))
    ran = run_matrix(comm, tc, torch.device("cpu"), VARIANTS_CPU)
    assert ran == 16 * len(VARIANTS_CPU), ran
    comm.finalize()


def test_every_operation_in_every_calling_variant_on_gloo():
    """16 operations x (sync, sync without the work, async, async with the work dropped, inputs deleted)."""
    run_ranks(_matrix_worker, 3, timeout=180)
