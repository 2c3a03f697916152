"""Behaviour of the c10d adapter and of communicator lifetime on gloo ranks: aliased all-gather
outputs, shutdown / destroy more than once, several communicators side by side,
``wait_blocking``, init handles, DDP-style dropped works.

Modelled on comms/torchcomms/tests/integration/py/BackendWrapperAllGatherAliasedTest.py,
BackendWrapperShutdownTest.py, MultiCommTest.py, WaitBlockingTest.py and GetInitHandleTest.py.
"""
from datetime import timedelta

import torch

from tests.mp_util import run_ranks


def _worker(rank, world):
    import torch.distributed as dist

    import torchcomms_b200 as tc
    from torchcomms_b200.device_mesh import init_device_mesh

    comm = tc.new_comm("gloo", torch.device("cpu"), name="wrap", timeout=timedelta(seconds=60))
    pg = init_device_mesh(mesh_dim_comms=(comm,), mesh_dim_names=("w",)).get_group("w")

    # distinct outputs: per-rank inputs in rank order
    outs = [torch.empty(1) for _ in range(world)]
    dist.all_gather(outs, torch.tensor([float(rank)]), group=pg)
    assert [o.item() for o in outs] == [float(r) for r in range(world)]
    # aliased outputs ([buf] * N): no race, the last rank's value wins, and the next call is clean
    shared = torch.full((1,), -1.0)
    dist.all_gather([shared] * world, torch.tensor([float(rank)]), group=pg)
    assert shared.item() == float(world - 1)
    outs = [torch.empty(1) for _ in range(world)]
    dist.all_gather(outs, torch.tensor([float(rank) + 10]), group=pg)
    assert [o.item() for o in outs] == [float(r) + 10 for r in range(world)]

    # a caller that keeps only the future (what DistributedDataParallel's reducer does)
    t = torch.full((3,), float(rank + 1))
    fut = dist.all_reduce(t, group=pg, async_op=True).get_future()
    fut.wait()
    assert torch.equal(t, torch.full((3,), float(world * (world + 1) // 2)))
    # ... and one that waits on both the work and the future
    t = torch.ones(3)
    w = dist.all_reduce(t, group=pg, async_op=True)
    f = w.get_future()
    w.wait()
    f.wait()
    assert torch.equal(t, torch.full((3,), float(world)))

    # several communicators side by side, interleaved operations, independent lifetimes
    a = tc.new_comm("gloo", torch.device("cpu"), name="multi_a", timeout=timedelta(seconds=60))
    b = tc.new_comm("gloo", torch.device("cpu"), name="multi_b", timeout=timedelta(seconds=60))
    ta, tb = torch.full((4,), 1.0), torch.full((4,), 2.0)
    wa = a.all_reduce(ta, tc.ReduceOp.SUM, True)
    wb = b.all_reduce(tb, tc.ReduceOp.SUM, True)
    wb.wait()
    wa.wait()
    assert torch.equal(ta, torch.full((4,), float(world))) and torch.equal(tb, torch.full((4,), 2.0 * world))
    a.finalize()
    tb.fill_(1.0)
    b.all_reduce(tb, tc.ReduceOp.MAX, False)                   # b is untouched by a's finalize
    assert torch.equal(tb, torch.ones(4))

    # wait_blocking blocks the host until the result is there
    tw = torch.full((2,), float(rank))
    work = b.all_reduce(tw, tc.ReduceOp.SUM, True)
    work.wait_blocking()
    assert work.is_completed() and torch.equal(tw, torch.full((2,), float(sum(range(world)))))
    b.finalize()

    # init handles: "<backend>:<rank>:<uuid>:<address>", distinct per rank and per communicator
    from torchcomms_b200.utils.store import create_prefix_store

    store = create_prefix_store("handles", timedelta(seconds=30))
    r1 = tc.new_comm("gloo", torch.device("cpu"), name="h1", store=store, enable_reconfigure=True, timeout=timedelta(seconds=30))
    r2 = tc.new_comm("gloo", torch.device("cpu"), name="h2", store=store, enable_reconfigure=True, timeout=timedelta(seconds=30))
    h1, h2 = r1.get_init_handle(), r2.get_init_handle()
    parts = h1.split(":")
    assert h1 != h2 and parts[0] == "gloo" and int(parts[1]) == rank and len(parts) >= 4

    # shutdown through the c10d wrapper finalizes the communicator; doing it again is harmless
    backend = pg._get_backend(torch.device("cpu"))
    backend.shutdown()
    backend.shutdown()
    import pytest

    with pytest.raises(RuntimeError):
        comm.all_reduce(torch.ones(1), tc.ReduceOp.SUM, False)


def test_c10d_wrapper_and_lifetime_behaviour():
    run_ranks(_worker, 2, timeout=120)


def _reduce_ops_worker(rank, world):
    """Every torch.distributed reduction operator through the adapter (C10dTorchCommTest.py), PREMUL_SUM included."""
    import math

    import torch.distributed as dist

    import torchcomms_b200 as tc
    from torchcomms_b200.device_mesh import init_device_mesh

    comm = tc.new_comm("gloo", torch.device("cpu"), name="redops", timeout=timedelta(seconds=60))
    pg = init_device_mesh(mesh_dim_comms=(comm,), mesh_dim_names=("w",)).get_group("w")
    total = sum(range(1, world + 1))
    expect = {dist.ReduceOp.SUM: float(total), dist.ReduceOp.AVG: total / world, dist.ReduceOp.MIN: 1.0,
              dist.ReduceOp.MAX: float(world), dist.ReduceOp.PRODUCT: float(math.factorial(world))}
    for op, want in expect.items():
        t = torch.tensor([float(rank + 1)])
        dist.all_reduce(t, op=op, group=pg)
        assert abs(t.item() - want) < 1e-6, (op, t.item(), want)
        r = torch.tensor([float(rank + 1)])
        dist.reduce(r, dst=0, op=op, group=pg)
        if rank == 0:
            assert abs(r.item() - want) < 1e-6, (op, r.item(), want)
    ti = torch.tensor([rank + 1])
    dist.all_reduce(ti, op=dist.ReduceOp.BOR, group=pg)
    bits = 0
    for r in range(1, world + 1):
        bits |= r
    assert ti.item() == bits
    rs = torch.empty(1)
    dist.reduce_scatter_tensor(rs, torch.arange(float(world)), op=dist.ReduceOp.MAX, group=pg)
    assert rs.item() == float(rank)
    comm.finalize()


def test_every_c10d_reduce_op_through_the_adapter():
    run_ranks(_reduce_ops_worker, 3, timeout=120)


def _no_finalize_worker(rank, world):
    import torchcomms_b200 as tc

    comm = tc.new_comm("gloo", torch.device("cpu"), name="nofinal", timeout=timedelta(seconds=60))
    t = torch.ones(4)
    comm.all_reduce(t, tc.ReduceOp.SUM, False)
    assert torch.equal(t, torch.full((4,), float(world)))
    sub = comm.split(list(range(world)), "child")
    sub.barrier(False)
    # no finalize(): the destructors warn and clean up; the process must exit normally


def test_destruction_without_finalize_does_not_abort():
    """FinalizeWarningTest.py of the reference."""
    assert run_ranks(_no_finalize_worker, 2, timeout=120) == [0, 0]


def _hooks_through_wrapper_worker(rank, world):
    """Hooks registered on the communicator fire for operations issued through torch.distributed
    (test_backend_wrapper.py of the reference), with correlated, increasing operation ids."""
    import torch.distributed as dist

    import torchcomms_b200 as tc
    from torchcomms_b200.device_mesh import init_device_mesh

    comm = tc.new_comm("gloo", torch.device("cpu"), name="hookwrap", timeout=timedelta(seconds=60))
    pg = init_device_mesh(mesh_dim_comms=(comm,), mesh_dim_names=("w",)).get_group("w")
    pre, post = [], []
    h1 = comm.register_pre_hook(lambda op, op_id, args: pre.append((op.name, op_id)))
    h2 = comm.register_post_hook(lambda op_id, args: post.append(op_id))
    t = torch.ones(4)
    dist.all_reduce(t, group=pg)
    out = torch.empty(world * 4)
    dist.all_gather_into_tensor(out, t, group=pg)
    dist.broadcast(t, src=0, group=pg)
    assert [n for n, _ in pre] == ["all_reduce", "all_gather_single", "broadcast"]
    ids = [i for _, i in pre]
    assert ids == post and ids == sorted(ids) and len(set(ids)) == 3
    h1.remove()
    h2.remove()
    dist.all_reduce(t, group=pg)
    assert len(pre) == 3 and len(post) == 3
    # a pre-hook that raises stops the operation on every rank alike (nothing was sent)
    import pytest

    def veto(op, op_id, args):
        raise ValueError("vetoed by the hook")

    h3 = comm.register_pre_hook(veto)
    with pytest.raises((RuntimeError, ValueError), match="vetoed"):
        comm.all_reduce(torch.ones(2), tc.ReduceOp.SUM, False)
    h3.remove()
    u = torch.ones(2)
    comm.all_reduce(u, tc.ReduceOp.SUM, False)                 # the communicator is still usable
    assert torch.equal(u, torch.full((2,), float(world)))
    comm.finalize()


def test_hooks_fire_through_the_c10d_adapter():
    run_ranks(_hooks_through_wrapper_worker, 2, timeout=120)
