"""Python framework layers on CPU: the torch.distributed-shaped wrapper,
hooks, functional ops and the parallelism helpers (gloo ranks)."""
from datetime import timedelta

import pytest
import torch

from tests.mp_util import run_ranks


def _distwrap_worker(rank, world):
    from torchcomms_b200 import distwrap as dist

    dist.init_process_group(backend="gloo", use_torchcomms=True, timeout=timedelta(seconds=60))
    assert dist.torchcomms_is_enabled() and dist.is_initialized()
    assert dist.get_rank() == rank and dist.get_world_size() == world
    t = torch.full((8,), float(rank + 1))
    dist.all_reduce(t)
    assert torch.equal(t, torch.full((8,), float(sum(range(1, world + 1)))))
    w = dist.all_reduce(t, op=dist.ReduceOp.MAX, async_op=True)
    w.wait()
    out = torch.empty(world * 4)
    dist.all_gather_into_tensor(out, torch.full((4,), float(rank)))
    assert torch.equal(out.view(world, 4)[:, 0], torch.arange(world, dtype=torch.float32))
    rs = torch.empty(2)
    dist.reduce_scatter_tensor(rs, torch.arange(2 * world, dtype=torch.float32))
    assert torch.equal(rs, torch.arange(2 * world, dtype=torch.float32).view(world, 2)[rank] * world)
    b = torch.full((3,), float(rank))
    dist.broadcast(b, src=1)
    assert torch.equal(b, torch.ones(3))
    a2a = torch.empty(world)
    dist.all_to_all_single(a2a, torch.full((world,), float(rank)))
    assert torch.equal(a2a, torch.arange(world, dtype=torch.float32))
    # point to point ring + batch
    nxt, prv = (rank + 1) % world, (rank - 1) % world
    got = torch.empty(2)
    ops = [dist.P2POp(dist.isend, torch.full((2,), float(rank)), nxt), dist.P2POp(dist.irecv, got, prv)]
    for wk in dist.batch_isend_irecv(ops):
        wk.wait()
    assert torch.equal(got, torch.full((2,), float(prv)))
    # objects
    objs = [None] * world
    dist.all_gather_object(objs, {"r": rank})
    assert [o["r"] for o in objs] == list(range(world))
    lst = [{"k": 7}] if rank == 0 else [None]
    dist.broadcast_object_list(lst, src=0)
    assert lst[0] == {"k": 7}
    # sub-groups by split; new_group is refused
    with pytest.raises(AssertionError):
        dist.new_group([0, 1])
    halves = [list(range(0, world // 2)), list(range(world // 2, world))]
    sub = dist.split_group(split_ranks=halves, group_desc="half")
    assert dist.get_world_size(sub) == world // 2
    s = torch.ones(2)
    dist.all_reduce(s, group=sub)
    assert torch.equal(s, torch.full((2,), float(world // 2)))
    dist.broadcast(s, src=halves[rank // (world // 2)][0], group=sub)
    # plain torch.distributed calls land on the same communicator
    import torch.distributed as td

    u = torch.ones(2)
    td.all_reduce(u)
    assert torch.equal(u, torch.full((2,), float(world)))
    dist.barrier()
    dist.destroy_process_group()
    assert not dist.torchcomms_is_enabled()


def test_distwrap_over_gloo():
    run_ranks(_distwrap_worker, 4, timeout=120)


def test_distwrap_backend_parsing():
    from torchcomms_b200.distwrap import _parse_backend

    assert _parse_backend("gloo") == {"cpu": "gloo"}
    assert _parse_backend("nccl") == {"cuda": "b200"}
    assert _parse_backend("cpu:gloo,cuda:ncclx") == {"cpu": "gloo", "cuda": "b200"}


def test_nan_check_hook():
    import torchcomms_b200 as tc
    from torchcomms_b200.hooks import NanCheckHook

    c = tc.new_comm("fake", torch.device("cpu"), name="nan")
    h = NanCheckHook()
    h.register_with_comm(c)
    t = torch.ones(4)
    c.all_reduce(t, tc.ReduceOp.SUM, False)
    t[1] = float("nan")
    with pytest.raises(RuntimeError, match="NaN detected in input"):
        c.all_reduce(t, tc.ReduceOp.SUM, False)
    with pytest.raises(RuntimeError, match="all_gather_single"):
        c.all_gather_single(torch.empty(4), t, False)
    h.unregister()
    c.all_reduce(t, tc.ReduceOp.SUM, False)
    c.finalize()


def test_profiler_span_and_health_handler():
    import torchcomms_b200 as tc
    from torch._C._distributed_c10d import _get_handler_names
    from torch.profiler import ProfilerActivity, profile

    assert "torchcomms_health_check" in _get_handler_names()
    c = tc.new_comm("fake", torch.device("cpu"), name="prof")
    with profile(activities=[ProfilerActivity.CPU]) as prof:
        c.all_reduce(torch.ones(4), tc.ReduceOp.SUM, False)
    assert any(e.name == "torchcomms_b200::all_reduce" for e in prof.events())
    c.finalize()


def _functional_worker(rank, world):
    import torchcomms_b200 as tc
    from torchcomms_b200 import functional as F

    comm = tc.new_comm("gloo", torch.device("cpu"), name="fn", timeout=timedelta(seconds=60))
    F.register_comm(comm)
    x = torch.full((4, 3), float(rank + 1), requires_grad=True)
    y = F.all_reduce(x, "sum", comm)
    assert torch.equal(y, torch.full((4, 3), float(sum(range(1, world + 1)))))
    assert torch.equal(x.detach(), torch.full((4, 3), float(rank + 1)))  # out of place
    # d/dx sum_ranks(loss_r) with loss_r = (r+1) * sum(y): every rank's grad is the all-reduced upstream grad
    (y.sum() * (rank + 1)).backward()
    assert torch.equal(x.grad, torch.full((4, 3), float(sum(range(1, world + 1)))))

    # all_gather <-> reduce_scatter
    s = torch.full((2, 3), float(rank), requires_grad=True)
    g = F.all_gather_single(s, comm)
    assert g.shape == (2 * world, 3) and torch.equal(g[2 * rank], torch.full((3,), float(rank)))
    (g * torch.arange(2 * world, dtype=torch.float32).view(-1, 1)).sum().backward()
    expect = torch.arange(2 * world, dtype=torch.float32).view(world, 2)[rank] * world
    assert torch.equal(s.grad, expect.view(2, 1).expand(2, 3))

    r = torch.ones(2 * world, 3, requires_grad=True)
    rs = F.reduce_scatter_single(r, "sum", comm)
    assert rs.shape == (2, 3) and torch.equal(rs, torch.full((2, 3), float(world)))
    rs.sum().backward()
    assert torch.equal(r.grad, torch.ones(2 * world, 3))

    a = torch.arange(world, dtype=torch.float32) + 10 * rank
    assert torch.equal(F.all_to_all_single(a, comm), torch.tensor([10.0 * p + rank for p in range(world)]))
    b = F.broadcast(torch.full((2,), float(rank)), 1, comm)
    assert torch.equal(b, torch.ones(2))
    t = torch.ones(3)
    F.all_reduce_(t, "max", comm)
    F.barrier(comm)

    # traced with fake tensors: shapes only, no collective runs
    from torch.fx.experimental.proxy_tensor import make_fx

    def f(v):
        return F.wait_tensor(F.reduce_scatter_single(F.all_gather_single(v, "fn"), "sum", "fn")) * 2

    gm = make_fx(f, tracing_mode="fake")(torch.ones(2, 3))
    names = [n.target.__name__ if hasattr(n.target, "__name__") else str(n.target) for n in gm.graph.nodes if n.op == "call_function"]
    assert any("all_gather_single" in n for n in names) and any("reduce_scatter_single" in n for n in names)
    compiled = torch.compile(f, backend="aot_eager", fullgraph=True)
    out = compiled(torch.full((2, 3), float(rank)))
    assert torch.equal(out, torch.full((2, 3), float(rank) * world * 2))
    comm.finalize()


def test_functional_ops_over_gloo():
    run_ranks(_functional_worker, 2, timeout=240)
