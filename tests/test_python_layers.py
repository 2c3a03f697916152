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
    # list collectives, rooted collectives, blocking point-to-point, object gather / scatter
    lst_out = [torch.empty(2) for _ in range(world)]
    dist.all_gather(lst_out, torch.full((2,), float(rank)))
    assert [t[0].item() for t in lst_out] == [float(r) for r in range(world)]
    a2a_out = [torch.empty(1) for _ in range(world)]
    dist.all_to_all(a2a_out, [torch.tensor([float(10 * rank + p)]) for p in range(world)])
    assert [t.item() for t in a2a_out] == [float(10 * p + rank) for p in range(world)]
    red = torch.full((2,), float(rank + 1))
    dist.reduce(red, dst=2)
    if rank == 2:
        assert torch.equal(red, torch.full((2,), float(sum(range(1, world + 1)))))
    rs_out = torch.empty(2)
    dist.reduce_scatter(rs_out, [torch.full((2,), float(p)) for p in range(world)])
    assert torch.equal(rs_out, torch.full((2,), float(rank * world)))
    gathered = [torch.empty(1) for _ in range(world)] if rank == 0 else None
    dist.gather(torch.tensor([float(rank)]), gathered, dst=0)
    if rank == 0:
        assert [t.item() for t in gathered] == [float(r) for r in range(world)]
    sc = torch.empty(1)
    dist.scatter(sc, [torch.tensor([float(100 + p)]) for p in range(world)] if rank == 1 else None, src=1)
    assert sc.item() == float(100 + rank)
    if rank == 0:
        dist.send(torch.tensor([42.0]), dst=1)
    elif rank == 1:
        box = torch.empty(1)
        dist.recv(box, src=0)
        assert box.item() == 42.0
    og = [None] * world if rank == 3 else None
    dist.gather_object({"from": rank}, og, dst=3)
    if rank == 3:
        assert [o["from"] for o in og] == list(range(world))
    so = [None]
    dist.scatter_object_list(so, [f"for{p}" for p in range(world)] if rank == 0 else None, src=0)
    assert so[0] == f"for{rank}"
    assert dist.get_torchcomms_instance().get_size() == world

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

    # differentiable point-to-point: a two-stage "pipeline" y = (x * 2 on rank 0) -> (* 3 on rank 1)
    if rank == 0:
        p = torch.full((2, 2), 1.5, requires_grad=True)
        sent = F.send(p * 2, 1, comm)
        sent.sum().mul(0).backward()                     # the gradient of what was sent comes back from rank 1
        assert torch.equal(p.grad, torch.full((2, 2), 6.0))
    elif rank == 1:
        got = F.recv(torch.empty(2, 2), 0, comm)
        got.requires_grad_()
        assert torch.equal(got, torch.full((2, 2), 3.0))
        (got * 3).sum().backward()
        F.send(got.grad, 0, comm)                        # what _bw_recv does when recv is inside a graph
    # gather <-> scatter
    gs = torch.full((1, 2), float(rank + 1), requires_grad=True)
    gathered = F.gather_single(gs, 0, comm)
    if rank == 0:
        assert torch.equal(gathered, torch.tensor([[float(r + 1)] * 2 for r in range(world)]))
    (gathered * (torch.arange(world, dtype=torch.float32).view(-1, 1) + 1)).sum().backward()
    assert torch.equal(gs.grad, torch.full((1, 2), float(rank + 1)))   # the root's upstream gradient, scattered back
    sc = F.scatter(torch.arange(2.0 * world).view(world, 2) if rank == 0 else torch.zeros(world, 2), 0, comm)
    assert torch.equal(sc, torch.tensor([[2.0 * rank, 2.0 * rank + 1]]))

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

    # graph passes: a collective whose input dies at the call runs in place, wait_tensor goes away
    from torchcomms_b200.functional.passes import count_ops, reinplace_pass, strip_wait_pass

    def g(v):
        a = F.all_reduce(v * 2, "sum", "fn")            # v * 2 is dead after the call: re-inplaced
        b = F.all_reduce(v, "sum", "fn")                # v is a graph input: stays functional
        k = v + 1
        c = F.all_reduce(k, "sum", "fn")                # k is read again below: stays functional
        return F.wait_tensor(a) + b + c + k

    gm2 = make_fx(g, tracing_mode="fake")(torch.ones(2, 3))
    assert count_ops(gm2) == {"all_reduce": 3, "wait_tensor": 1}
    strip_wait_pass(reinplace_pass(gm2))
    assert count_ops(gm2) == {"all_reduce_": 1, "all_reduce": 2}
    x = torch.full((2, 3), float(rank + 1))
    keep = x.clone()
    total = float(sum(range(1, world + 1)))
    torch.testing.assert_close(gm2(x), torch.full((2, 3), 4 * total + world) + keep + 1)
    assert torch.equal(x, keep)                         # the caller's tensor was not written

    # the wait behind a started collective is the only thing that orders its consumer: it stays
    def started(v):
        h = F.all_reduce_async(v * 3, "sum", "fn")
        return h.wait() + F.wait_tensor(F.all_reduce(v, "sum", "fn"))

    gm3 = make_fx(started, tracing_mode="fake")(torch.ones(2, 3))
    assert count_ops(gm3) == {"all_reduce_start": 1, "wait_tensor": 2, "all_reduce": 1}
    strip_wait_pass(gm3)
    assert count_ops(gm3) == {"all_reduce_start": 1, "wait_tensor": 1, "all_reduce": 1}
    torch.testing.assert_close(gm3(x), torch.full((2, 3), 4 * total))
    comm.finalize()


def test_functional_ops_over_gloo():
    run_ranks(_functional_worker, 2, timeout=240)


def _pipeline_worker(rank, world, schedule):
    import torchcomms_b200 as tc
    from torchcomms_b200.parallel.pipeline import PipelineStage, run_gpipe

    comm = tc.new_comm("gloo", torch.device("cpu"), name="pp", timeout=timedelta(seconds=60))
    torch.manual_seed(0)
    layers = [torch.nn.Sequential(torch.nn.Linear(16, 16), torch.nn.Tanh()) for _ in range(world)]  # same on every rank
    micro = [torch.randn(4, 16) for _ in range(6)]
    targets = [torch.randn(4, 16) for _ in range(6)]
    # reference: the whole model in this process
    ref_layers = [torch.nn.Sequential(torch.nn.Linear(16, 16), torch.nn.Tanh()) for _ in range(world)]
    for a, b in zip(ref_layers, layers):
        a.load_state_dict(b.state_dict())
    ref_losses = []
    for x, t in zip(micro, targets):
        y = x
        for l in ref_layers:
            y = l(y)
        loss = ((y - t) ** 2).mean()
        loss.backward()
        ref_losses.append(loss.detach())
    stage = PipelineStage(layers[rank], comm, input_like=None if rank == 0 else torch.empty(4, 16))
    loss_fn = lambda y, i: ((y - targets[i]) ** 2).mean()
    losses = stage.run_1f1b(micro, loss_fn) if schedule == "1f1b" else run_gpipe(stage, micro, loss_fn)
    for p, q in zip(layers[rank].parameters(), ref_layers[rank].parameters()):
        torch.testing.assert_close(p.grad, q.grad, rtol=1e-5, atol=1e-6)
    if rank == world - 1:
        torch.testing.assert_close(torch.stack(losses), torch.stack(ref_losses))
    comm.finalize()


@pytest.mark.parametrize("schedule", ["1f1b", "gpipe"])
def test_pipeline_schedules_match_single_process(schedule):
    run_ranks(_pipeline_worker, 3, args=(schedule,), timeout=120)


def _context_worker(rank, world):
    import torchcomms_b200 as tc
    from torchcomms_b200.parallel.context import (ring_attention, shard_positions, ulysses_attention, zigzag_shard,
                                                   zigzag_unshard)

    comm = tc.new_comm("gloo", torch.device("cpu"), name="cp", timeout=timedelta(seconds=60))
    torch.manual_seed(1)
    b, h, s, d = 2, 4, 8 * world, 16
    q, k, v = (torch.randn(b, h, s, d) for _ in range(3))
    sl = slice(rank * s // world, (rank + 1) * s // world)
    for causal in (False, True):
        ref = torch.nn.functional.scaled_dot_product_attention(q, k, v, is_causal=causal)[:, :, sl]
        got = ring_attention(q[:, :, sl].contiguous(), k[:, :, sl].contiguous(), v[:, :, sl].contiguous(), comm, causal=causal)
        torch.testing.assert_close(got, ref, rtol=1e-4, atol=1e-5)
        got = ulysses_attention(q[:, :, sl].contiguous(), k[:, :, sl].contiguous(), v[:, :, sl].contiguous(), comm, causal=causal)
        torch.testing.assert_close(got, ref, rtol=1e-4, atol=1e-5)
        # zigzag layout: rank r holds chunks r and 2*world-1-r of the sequence
        full = torch.nn.functional.scaled_dot_product_attention(q, k, v, is_causal=causal)
        zq, zk, zv = (zigzag_shard(t, rank, world).contiguous() for t in (q, k, v))
        got = ring_attention(zq, zk, zv, comm, causal=causal, layout="zigzag")
        torch.testing.assert_close(got, zigzag_shard(full, rank, world), rtol=1e-4, atol=1e-5)
    pos = [shard_positions(r, world, s // world, "zigzag") for r in range(world)]
    assert sorted(torch.cat(pos).tolist()) == list(range(s))
    # the causal work (visible key count) is the same on every rank, unlike the contiguous layout
    assert len({int((p + 1).sum()) for p in pos}) == 1
    assert len({int((shard_positions(r, world, s // world) + 1).sum()) for r in range(world)}) == world
    parts = [zigzag_shard(q, r, world) for r in range(world)]
    assert torch.equal(zigzag_unshard(parts), q)
    # Ulysses attention is differentiable: gradients of the sequence shards equal those of full attention
    # (same q / k / v on every rank, so the full-sequence loss is the sum of the ranks' losses)
    from torchcomms_b200.parallel.context import SeqHeadsExchange

    fq, fk, fv = (t.clone().requires_grad_(True) for t in (q, k, v))
    full = torch.nn.functional.scaled_dot_product_attention(fq, fk, fv, is_causal=True)
    gq, gk, gv = torch.autograd.grad(full.square().sum(), (fq, fk, fv))
    lq, lk, lv = (t[:, :, sl].clone().requires_grad_(True) for t in (q, k, v))
    out = ulysses_attention(lq, lk, lv, comm, causal=True)
    grads = torch.autograd.grad(out.square().sum(), (lq, lk, lv))
    for got_g, ref_g in zip(grads, (gq, gk, gv)):
        torch.testing.assert_close(got_g, ref_g[:, :, sl], rtol=1e-4, atol=1e-5)
    # ring attention is differentiable too (a second trip round the ring), in both layouts
    for layout in ("contiguous", "zigzag"):
        take = (lambda t: t[:, :, sl]) if layout == "contiguous" else (lambda t: zigzag_shard(t, rank, world))
        rq, rk, rv = (take(t).clone().requires_grad_(True) for t in (q, k, v))
        r_out = ring_attention(rq, rk, rv, comm, causal=True, layout=layout)
        torch.testing.assert_close(r_out, take(full.detach()), rtol=1e-4, atol=1e-5)
        r_grads = torch.autograd.grad(r_out.square().sum(), (rq, rk, rv))
        for got_g, ref_g in zip(r_grads, (gq, gk, gv)):
            torch.testing.assert_close(got_g, take(ref_g), rtol=1e-4, atol=1e-5)
    rq, rk, rv = (t[:, :, sl].clone().requires_grad_(True) for t in (q, k, v))
    nc_full = torch.nn.functional.scaled_dot_product_attention(fq, fk, fv, is_causal=False)
    nc_ref = torch.autograd.grad(nc_full.square().sum(), (fq, fk, fv))
    nc_grads = torch.autograd.grad(ring_attention(rq, rk, rv, comm, causal=False).square().sum(), (rq, rk, rv))
    for got_g, ref_g in zip(nc_grads, nc_ref):
        torch.testing.assert_close(got_g, ref_g[:, :, sl], rtol=1e-4, atol=1e-5)
    # grouped-query attention: 8 query heads share 4 key / value heads (head groups stay together on a rank)
    gq, gk2, gv2 = torch.randn(b, 8, s, d), torch.randn(b, 4, s, d), torch.randn(b, 4, s, d)
    ref = torch.nn.functional.scaled_dot_product_attention(gq, gk2, gv2, is_causal=True, enable_gqa=True)[:, :, sl]
    got = ulysses_attention(gq[:, :, sl].contiguous(), gk2[:, :, sl].contiguous(), gv2[:, :, sl].contiguous(), comm, causal=True)
    torch.testing.assert_close(got, ref, rtol=1e-4, atol=1e-5)
    # the exchange object falls back to the same all-to-all on backends without the fused kernel
    ex = SeqHeadsExchange(comm)
    assert not ex.fused
    out2 = ulysses_attention(lq, lk, lv, comm, causal=True, exchange=ex)
    torch.testing.assert_close(out2, out)
    torch.testing.assert_close(ex.to_seq(ex.to_heads(lq.detach())), lq.detach())
    comm.finalize()


def test_ring_and_ulysses_attention():
    run_ranks(_context_worker, 4, timeout=120)


def _tensor_parallel_worker(rank, world):
    import torchcomms_b200 as tc
    from torchcomms_b200.parallel.tensor import ColumnParallelLinear, RowParallelLinear, TensorParallelMLP

    comm = tc.new_comm("gloo", torch.device("cpu"), name="tp", timeout=timedelta(seconds=60))
    torch.manual_seed(2)
    hidden, ffn, tokens = 16, 32, 8
    w_gu = torch.randn(2 * ffn, hidden) * 0.2   # rows: [gate | up]
    w_dn = torch.randn(hidden, ffn) * 0.2
    x = torch.randn(tokens, hidden)
    # unsharded reference
    xr = x.clone().requires_grad_(True)
    wg, wd = w_gu.clone().requires_grad_(True), w_dn.clone().requires_grad_(True)
    g, u = (xr @ wg.t()).chunk(2, dim=-1)
    ref = (torch.nn.functional.silu(g) * u) @ wd.t()
    ref.square().sum().backward()

    mlp = TensorParallelMLP(hidden, ffn, comm)
    fl = ffn // world
    with torch.no_grad():
        mlp.gate_up.weight.copy_(torch.cat([w_gu[:ffn][rank * fl:(rank + 1) * fl], w_gu[ffn:][rank * fl:(rank + 1) * fl]]))
        mlp.down.weight.copy_(w_dn[:, rank * fl:(rank + 1) * fl])
    tl = tokens // world
    xs = x[rank * tl:(rank + 1) * tl].clone().requires_grad_(True)
    y = mlp(xs)
    torch.testing.assert_close(y, ref[rank * tl:(rank + 1) * tl].detach(), rtol=1e-4, atol=1e-5)
    # each rank's loss covers its token shard; the sum over ranks is the reference loss
    y.square().sum().backward()
    torch.testing.assert_close(xs.grad, xr.grad[rank * tl:(rank + 1) * tl], rtol=1e-4, atol=1e-5)
    torch.testing.assert_close(mlp.down.weight.grad, wd.grad[:, rank * fl:(rank + 1) * fl], rtol=1e-4, atol=1e-5)
    torch.testing.assert_close(mlp.gate_up.weight.grad[:fl], wg.grad[:ffn][rank * fl:(rank + 1) * fl], rtol=1e-4, atol=1e-5)

    # replicated-activation variant: identity in, all-reduce out
    col = ColumnParallelLinear(hidden, ffn, comm)
    row = RowParallelLinear(ffn, hidden, comm)
    with torch.no_grad():
        col.weight.copy_(w_gu[:ffn][rank * fl:(rank + 1) * fl])
        row.weight.copy_(w_dn[:, rank * fl:(rank + 1) * fl])
    x2 = x.clone().requires_grad_(True)
    y2 = row(torch.relu(col(x2)))
    x3 = x.clone().requires_grad_(True)
    ref2 = torch.relu(x3 @ w_gu[:ffn].t()) @ w_dn.t()
    torch.testing.assert_close(y2, ref2.detach(), rtol=1e-4, atol=1e-5)
    y2.sum().backward()
    ref2.sum().backward()
    # The differentiated objective is the SUM of the ranks' losses; here every rank holds the same loss.
    torch.testing.assert_close(x2.grad, x3.grad * world, rtol=1e-4, atol=1e-5)
    comm.finalize()


def test_tensor_parallel_layers():
    run_ranks(_tensor_parallel_worker, 2, timeout=120)


def _lazy_worker(rank, world):
    import torchcomms_b200 as tc
    from torchcomms_b200 import _comms

    comm = tc.new_comm("gloo-lazy", torch.device("cpu"), name="lazy", timeout=timedelta(seconds=60))
    impl = comm.get_backend_impl()
    assert comm.get_backend() == "gloo-lazy" and _comms._lazy_pair_count(impl) == 0
    # collectives run on the primary and create no pair
    t = torch.full((4,), float(rank))
    comm.all_reduce(t, tc.ReduceOp.SUM, False)
    assert _comms._lazy_pair_count(impl) == 0
    # ring: each rank talks to two peers -> two pair communicators (one when world == 2)
    nxt, prv = (rank + 1) % world, (rank - 1) % world
    got = torch.empty(4)
    if rank % 2 == 0:
        comm.send(torch.full((4,), float(rank)), nxt, False)
        comm.recv(got, prv, False)
    else:
        comm.recv(got, prv, False)
        comm.send(torch.full((4,), float(rank)), nxt, False)
    assert torch.equal(got, torch.full((4,), float(prv)))
    assert _comms._lazy_pair_count(impl) == len({nxt, prv})
    # the same pair is reused
    if rank % 2 == 0:
        comm.send(torch.ones(2), nxt, False)
    else:
        comm.recv(torch.empty(2), prv, False)
    assert _comms._lazy_pair_count(impl) == len({nxt, prv})
    # batches stay on the primary
    b = comm.batch_op_create()
    r2 = torch.empty(3)
    b.send(torch.full((3,), float(rank)), nxt)
    b.recv(r2, prv)
    b.issue(False)
    assert torch.equal(r2, torch.full((3,), float(prv)))
    comm.barrier(False)
    comm.finalize()


def test_lazy_backend_pair_comms():
    run_ranks(_lazy_worker, 4, timeout=120)


def test_distwrap_turns_pg_options_into_hints():
    import torch.distributed as td

    from torchcomms_b200.distwrap import _pg_options_to_hints

    assert _pg_options_to_hints(None) == ({}, None)
    if not hasattr(td, "ProcessGroupNCCL"):
        pytest.skip("torch without the NCCL process group")
    opts = td.ProcessGroupNCCL.Options(is_high_priority_stream=True)
    opts.config.min_ctas, opts.config.max_ctas = 4, 16
    hints, high_priority = _pg_options_to_hints(opts)
    assert high_priority is True and hints["min_ctas"] == "4" and hints["max_ctas"] == "16"
    assert all(isinstance(v, str) for v in hints.values()) and "is_high_priority_stream" not in hints


def test_distwrap_requires_a_backend():
    from torchcomms_b200 import distwrap

    with pytest.raises(ValueError, match="backend must be specified"):
        distwrap.init_process_group(backend=None)


def test_reference_import_name():
    import torchcomms_b200

    torchcomms_b200.install_alias()
    import torchcomms
    from torchcomms import distwrap, objcol  # noqa: F401
    from torchcomms.device_mesh import init_device_mesh  # noqa: F401
    from torchcomms.hooks import NanCheckHook  # noqa: F401

    from torchcomms._comms import AllReducePreHookArgs, OpName, RemovableHandle, _BackendWrapper  # noqa: F401

    c = torchcomms.new_comm("fake", torch.device("cpu"), name="alias")
    assert c.get_size() == 1 and torchcomms.ReduceOp.SUM is not None
    seen = []
    handle = c.register_pre_hook(lambda op, op_id, args: seen.append((op, type(args))))
    assert isinstance(handle, RemovableHandle)
    c.all_reduce(torch.ones(2), torchcomms.ReduceOp.SUM, False)
    assert seen == [(OpName.all_reduce, AllReducePreHookArgs)]
    handle.remove()
    from torchcomms.distwrap.collectives import all_reduce, register_mem_pool  # noqa: F401
    from torchcomms.distwrap.collectives_extension import new_window, reduce_scatter_quantized  # noqa: F401

    assert all_reduce is distwrap.all_reduce and new_window is distwrap.new_window
    from torchcomms._comms_fake import TorchCommFake
    from torchcomms._comms_gloo import TorchCommGloo  # noqa: F401
    from torchcomms._comms_ncclx import TorchCommNCCLX, comm_dump_all  # noqa: F401

    assert isinstance(c.get_backend_impl(), TorchCommFake)
    c.finalize()


def test_trace_to_perfetto(tmp_path):
    import json

    from torchcomms_b200.utils.trace_to_perfetto import (flight_recorder_events, phase_summary, phase_trace_events,
                                                          write_trace)

    trace = torch.zeros(4, 16, dtype=torch.long)          # nanoseconds of the device timer
    trace[0, :4] = torch.tensor([1000, 2000, 3000, 5000])
    trace[2, :3] = torch.tensor([1100, 2100, 2110])
    ev = phase_trace_events(trace, rank=3, phases=("copy-in", "barrier", "reduce"))
    slices = [e for e in ev if e["ph"] == "X"]
    assert len(slices) == 5 and slices[0]["name"] == "copy-in" and abs(slices[0]["dur"] - 1.0) < 1e-6
    assert abs(slices[3]["ts"] - 0.1) < 1e-6 and {e["tid"] for e in slices} == {0, 2}
    text = phase_summary(trace, ("copy-in", "barrier", "reduce"))
    assert text[0].startswith("2 blocks") and "barrier" in text[3] and text[3].split()[1] == "2"
    assert float(text[4].split()[-1]) == 4.0            # the reduce phase of block 0 ends 4 us after the first mark
    fr = {"rank": 3, "entries": [
        {"profiling_name": "all_reduce", "time_created_ns": 5_000, "time_discovered_started_ns": 6_000,
         "time_discovered_completed_ns": 16_000, "collective_seq_id": 1, "state": "completed"},
        {"profiling_name": "barrier", "time_created_ns": 20_000, "duration_ms": 0.002},
    ]}
    fe = [e for e in flight_recorder_events(fr) if e["ph"] == "X"]
    assert fe[0]["dur"] == 10.0 and fe[1]["dur"] == 2.0 and fe[0]["pid"] == 3
    write_trace(str(tmp_path / "t.json"), ev + fe)
    assert len(json.load(open(tmp_path / "t.json"))["traceEvents"]) == len(ev) + len(fe)


def test_tuning_crossovers():
    from torchcomms_b200.utils.tuning import best_config, crossovers, hint_sweep

    rows = []
    for b, k, n in [(1024, 12.0, 25.0), (2048, 12.5, 25.1), (1 << 20, 36.0, 28.0), (1 << 24, 90.0, 97.0)]:
        rows.append({"op": "all_reduce", "dtype": "bf16", "bytes": b, "algo": "kernel", "us": k})
        rows.append({"op": "all_reduce", "dtype": "bf16", "bytes": b, "algo": "nccl", "us": n})
    assert best_config(rows)[("all_reduce", "bf16", 1 << 20)]["algo"] == "nccl"
    assert crossovers(rows)[("all_reduce", "bf16")] == [(1024, 2048, "kernel"), (1 << 20, 1 << 20, "nccl"), (1 << 24, 1 << 24, "kernel")]
    hs = hint_sweep({"steps=8": [r for r in rows if r["algo"] == "kernel"],
                     "steps=2": [dict(r, us=r["us"] * (0.5 if r["bytes"] > 4096 else 2)) for r in rows if r["algo"] == "kernel"]})
    assert hs[("all_reduce", "bf16", 1 << 24)]["hints"] == "steps=2" and hs[("all_reduce", "bf16", 1024)]["hints"] == "steps=8"
    # rows of the bench sweep (arm / avg_us) are read as well; a margin keeps near ties with the kernels
    from torchcomms_b200.utils.tuning import tuner_file_lines

    sweep = []
    for b, k, n in [(1 << 20, 12.0, 20.0), (1 << 21, 33.0, 29.0), (1 << 22, 35.0, 34.5), (1 << 24, 50.0, 58.0)]:
        sweep.append({"op": "all_to_all_v", "dtype": "bf16", "bytes": b, "arm": "own", "avg_us": k, "p50_us": k})
        sweep.append({"op": "all_to_all_v", "dtype": "bf16", "bytes": b, "arm": "nccl", "avg_us": n, "p50_us": n})
    assert [a for _, _, a in crossovers(sweep)[("all_to_all_v", "bf16")]] == ["kernel", "nccl", "kernel"]
    assert crossovers(sweep, margin=0.05)[("all_to_all_v", "bf16")] == [
        (1 << 20, 1 << 20, "kernel"), (1 << 21, 1 << 21, "nccl"), (1 << 22, 1 << 24, "kernel")]
    assert tuner_file_lines(sweep, margin=0.05)[1:] == [
        f"all_to_all_v {1 << 20} kernel", f"all_to_all_v {1 << 21} nccl", "all_to_all_v inf kernel"]


def _data_parallel_worker(rank, world):
    import torchcomms_b200 as tc
    from torchcomms_b200.parallel.data import DataParallel

    comm = tc.new_comm("gloo", torch.device("cpu"), name="dp", timeout=timedelta(seconds=60))
    torch.manual_seed(100 + rank)  # different initial weights: the wrapper broadcasts rank 0's
    model = torch.nn.Sequential(torch.nn.Linear(8, 16), torch.nn.ReLU(), torch.nn.Linear(16, 4))
    dp = DataParallel(model, comm, bucket_mb=0.0003)  # tiny buckets -> several all-reduces
    assert len(dp._buckets) > 1
    torch.manual_seed(0)
    ref = torch.nn.Sequential(torch.nn.Linear(8, 16), torch.nn.ReLU(), torch.nn.Linear(16, 4))
    torch.manual_seed(100)
    ref0 = torch.nn.Sequential(torch.nn.Linear(8, 16), torch.nn.ReLU(), torch.nn.Linear(16, 4))
    for p, q in zip(model.parameters(), ref0.parameters()):
        assert torch.equal(p, q)  # rank 0's weights everywhere
    g = torch.Generator().manual_seed(7)
    xs = [torch.randn(5, 8, generator=g) for _ in range(world)]
    ys = [torch.randn(5, 4, generator=g) for _ in range(world)]
    for step in range(2):
        model.zero_grad()
        ((dp(xs[rank]) - ys[rank]) ** 2).mean().backward()
        dp.finish()
        ref0.zero_grad()
        sum(((ref0(x) - y) ** 2).mean() for x, y in zip(xs, ys)).div(world).backward()
        for p, q in zip(model.parameters(), ref0.parameters()):
            torch.testing.assert_close(p.grad, q.grad, rtol=1e-5, atol=1e-6)
    comm.finalize()


def test_data_parallel_bucketed_all_reduce():
    run_ranks(_data_parallel_worker, 2, timeout=120)


def _chaos_worker(rank, world):
    import time

    import torchcomms_b200 as tc
    from torchcomms_b200 import objcol
    from torchcomms_b200.hooks import ChecksumHook, DelayInjectionHook

    comm = tc.new_comm("gloo", torch.device("cpu"), name="chaos")
    delay = DelayInjectionHook(max_ms=20, seed=rank, probability=0.7, ops=["all_reduce", tc.OpName.broadcast], ranks=[0, 1])
    delay.register_with_comm(comm)
    chk = ChecksumHook(ops=["all_reduce", "broadcast", "all_gather_single"])
    chk.register_with_comm(comm)
    # with ranks arriving in a different order every time the results stay right
    for step in range(6):
        t = torch.full((257,), float(rank + step))
        comm.all_reduce(t, tc.ReduceOp.SUM, step % 2 == 1).wait()
        assert torch.equal(t, torch.full((257,), float(sum(r + step for r in range(world)))))
    b = torch.arange(5.0) if rank == 1 else torch.zeros(5)
    comm.broadcast(b, 1, False)
    out = torch.empty(world * 3)
    comm.all_gather_single(out, torch.full((3,), float(rank)), False)
    comm.barrier(False)                                         # not recorded: filtered out
    assert delay.is_enabled() and len(delay.injected) >= 1 and all(name in ("all_reduce", "broadcast") for _, name, _ in delay.injected)
    deadline = time.time() + 5
    while time.time() < deadline and len(chk.records()) < 8:
        time.sleep(0.01)
    mine = chk.records()
    assert [r["op"] for r in mine] == ["all_reduce"] * 6 + ["broadcast", "all_gather_single"]
    chk.unregister()
    delay.unregister()
    everyone = [None] * world
    objcol.all_gather_object(comm, everyone, mine)
    assert ChecksumHook.divergence(everyone) is None
    # inputs differ between ranks, outputs of replicating operations do not
    assert len({r[0]["in"] for r in everyone}) == world and len({r[0]["out"] for r in everyone}) == 1
    # a replica that silently diverged is named by sequence number
    broken = [list(map(dict, r)) for r in everyone]
    broken[1][3]["out"] ^= 1
    bad = ChecksumHook.divergence(broken)
    assert bad["seq"] == 3 and bad["reason"] == "output mismatch" and bad["op"] == "all_reduce"
    assert ChecksumHook.divergence([everyone[0], everyone[1][:-1]])["reason"] == "operation count mismatch"
    comm.finalize()


def test_delay_injection_and_checksum_hooks():
    run_ranks(_chaos_worker, 2, timeout=120)


def _moe_unfused_worker(rank, world):
    import torchcomms_b200 as tc
    from torchcomms_b200.parallel.expert import ExpertParallelMoEUnfused

    comm = tc.new_comm("gloo", torch.device("cpu"), name="moe", timeout=timedelta(seconds=60))
    hidden, num_experts, topk, tokens = 8, 4, 2, 6
    local = num_experts // world

    def make_expert(e):
        torch.manual_seed(100 + e)
        return torch.nn.Linear(hidden, hidden)

    def make_router():
        torch.manual_seed(7)
        return torch.nn.Linear(hidden, num_experts)

    def inputs(r):
        g = torch.Generator().manual_seed(1000 + r)
        return torch.randn(tokens, hidden, generator=g)

    layer = ExpertParallelMoEUnfused(comm, hidden, num_experts, topk, [make_expert(rank * local + i) for i in range(local)],
                                     make_router())
    x = inputs(rank).requires_grad_()
    y = layer(x)
    (y * (rank + 1)).sum().backward()

    # single-process reference over the tokens of all ranks, every expert local
    experts, router = [make_expert(e) for e in range(num_experts)], make_router()
    xs = [inputs(r).requires_grad_() for r in range(world)]
    total = 0
    ys = []
    for r in range(world):
        gates, idx = torch.softmax(router(xs[r]).float(), -1).topk(topk, -1)
        out = torch.zeros(tokens, hidden)
        for t in range(tokens):
            for k in range(topk):
                out[t] = out[t] + gates[t, k] * experts[int(idx[t, k])](xs[r][t])
        ys.append(out)
        total = total + (out * (r + 1)).sum()
    total.backward()
    torch.testing.assert_close(y, ys[rank], rtol=1e-5, atol=1e-6)
    torch.testing.assert_close(x.grad, xs[rank].grad, rtol=1e-5, atol=1e-6)
    for i in range(local):                                     # an expert's gradient comes from the tokens of every rank
        ref = experts[rank * local + i]
        torch.testing.assert_close(layer.experts[i].weight.grad, ref.weight.grad, rtol=1e-5, atol=1e-6)
        torch.testing.assert_close(layer.experts[i].bias.grad, ref.bias.grad, rtol=1e-5, atol=1e-6)
    g = layer.router.weight.grad.clone()                       # the router is replicated: its gradient is summed over ranks
    comm.all_reduce(g, tc.ReduceOp.SUM, False)
    torch.testing.assert_close(g, router.weight.grad, rtol=1e-5, atol=1e-6)
    comm.finalize()


def test_unfused_expert_parallel_moe_trains():
    run_ranks(_moe_unfused_worker, 2, timeout=120)


def _distwrap_passthrough_worker(rank, world):
    """use_torchcomms=False: calls go to torch.distributed, groups are still registered, and what gloo
    lacks (all-to-all, group splitting) is built from what it has."""
    from torchcomms_b200 import distwrap as dist
    from torchcomms_b200.distwrap import pginfo

    dist.init_process_group(backend="gloo", timeout=timedelta(seconds=60))
    assert not dist.torchcomms_is_enabled() and dist.is_initialized()
    world_pg = dist.GroupMember.WORLD
    assert pginfo.pg_info_get_global_ranks(world_pg) == list(range(world))
    assert pginfo.pg_info_get_rank_map(world_pg) == {r: r for r in range(world)}
    assert dist.get_backend_for_device(None, "cpu") == "gloo"
    t = torch.full((4,), float(rank + 1))
    dist.all_reduce(t)
    assert torch.equal(t, torch.full((4,), float(sum(range(1, world + 1)))))
    # all-to-all on gloo: batched point to point underneath
    outs = [torch.empty(2) for _ in range(world)]
    dist.all_to_all(outs, [torch.full((2,), float(rank * world + d)) for d in range(world)])
    assert [float(o[0]) for o in outs] == [float(s * world + rank) for s in range(world)]
    out = torch.empty(world * 3)
    w = dist.all_to_all_single(out, torch.arange(world * 3, dtype=torch.float32) + 100 * rank, async_op=True)
    w.wait()
    assert torch.equal(out.view(world, 3)[:, 0], torch.tensor([100.0 * s + 3 * rank for s in range(world)]))
    # uneven splits
    ins = [r + 1 for r in range(world)]
    outsz = [rank + 1] * world
    dst = torch.empty(sum(outsz))
    src = torch.cat([torch.full((d + 1,), float(rank * 10 + d)) for d in range(world)])
    dist.all_to_all_single(dst, src, outsz, ins)
    assert torch.equal(dst, torch.cat([torch.full((rank + 1,), float(s * 10 + rank)) for s in range(world)]))
    # splitting a gloo group: partitions are created with new_group, every rank takes part in each
    halves = [[r for r in range(world) if r % 2 == 0], [r for r in range(world) if r % 2 == 1]]
    sub = dist.split_group(split_ranks=halves, group_desc="parity")
    mine = halves[rank % 2]
    assert pginfo.pg_info_get_global_ranks(sub) == mine and pginfo.pg_info_get_group_desc(sub) == "parity"
    t = torch.full((2,), float(rank + 1))
    dist.all_reduce(t, group=sub)
    assert torch.equal(t, torch.full((2,), float(sum(m + 1 for m in mine))))
    g = dist.new_group(ranks=list(range(world)), backend="gloo", group_desc="again")
    assert pginfo.pg_info_get_group_desc(g) == "again"
    dist.destroy_process_group()
    assert pginfo.pg_info_get(world_pg) is None


def test_distwrap_passthrough_registry_and_fallbacks():
    run_ranks(_distwrap_passthrough_worker, 4, timeout=180)
