"""Communicator objects inside ``torch.compile(fullgraph=True)`` regions: methods of a ``TorchComm`` are
recorded as this package's operators, rank / size / name fold to constants, asynchronous calls keep their
start / wait structure in the graph, and the eager behaviour of the same methods is unchanged.

Parity: comms/torchcomms/tests/integration/py/FullgraphCompileTest.py (communicator methods called on the
object inside a compiled function) and the unit tests of comms/torchcomms/functional/dynamo.py.
"""
from datetime import timedelta

import pytest

import torch

from tests.mp_util import run_ranks


def _graph_ops(fn, *args):
    """Runs ``fn`` under torch.compile with a backend that records the operator names of the traced graph."""
    seen = []

    def backend(gm, example_inputs):
        for n in gm.graph.nodes:
            if n.op == "call_function":
                seen.append(getattr(n.target, "__name__", str(n.target)))
        return gm.forward

    out = torch.compile(fn, fullgraph=True, backend=backend)(*args)
    return out, seen


def _dynamo_worker(rank, world):
    import torchcomms_b200 as tc
    from torchcomms_b200 import ReduceOp
    from torchcomms_b200.functional import dynamo as D

    D.register_with_dynamo()
    D.register_with_dynamo()                      # idempotent
    comm = tc.new_comm("gloo", torch.device("cpu"), name="dyn", timeout=timedelta(seconds=60))
    tri = world * (world + 1) // 2

    # eager calls go straight through the original methods
    t = torch.full((4,), float(rank + 1))
    assert comm.all_reduce(t, ReduceOp.SUM, False) is not None and torch.equal(t, torch.full((4,), float(tri)))
    assert comm.get_rank() == rank and comm.get_size() == world and comm.get_name() == "dyn"

    def step(x, out_g, out_s):
        y = x * 2
        comm.all_reduce(y, ReduceOp.SUM, False)                                 # in place on an intermediate
        w = comm.all_gather_single(out_g, x, True)                              # asynchronous, into a graph input
        z = y + comm.get_rank() + 10 * comm.get_size()                          # constants of the graph
        comm.reduce_scatter_single(out_s, z.repeat(comm.get_size()), ReduceOp.AVG, False)
        w.wait()
        comm.barrier(False)
        return z, out_g.sum() + out_s.sum()

    x = torch.full((4,), float(rank + 1))
    out_g, out_s = torch.zeros(world * 4), torch.zeros(4)
    (z, total), seen = _graph_ops(step, x, out_g, out_s)
    exp_z = torch.full((4,), 2.0 * tri + rank + 10 * world)
    assert torch.equal(z, exp_z)
    assert torch.equal(out_g, torch.arange(1, world + 1, dtype=torch.float32).repeat_interleave(4))   # written through
    exp_s = torch.full((4,), 2.0 * tri + 10 * world + (world - 1) / 2)
    assert torch.allclose(out_s, exp_s)
    assert torch.allclose(total, out_g.sum() + out_s.sum())
    joined = " ".join(seen)
    for name in ("all_reduce", "all_gather_single_start", "wait_tensor", "reduce_scatter_single", "barrier"):
        assert name in joined, (name, seen)
    first = lambda part: next(i for i, s in enumerate(seen) if part in s)  # noqa: E731
    assert first("all_gather_single_start") < first("reduce_scatter_single") < first("wait_tensor")   # the wait stays where it was called

    # the same function through AOT autograd (functionalisation of the copies into inputs and intermediates)
    out_g2, out_s2 = torch.zeros(world * 4), torch.zeros(4)
    z2, total2 = torch.compile(step, fullgraph=True, backend="aot_eager")(x, out_g2, out_s2)
    assert torch.equal(z2, exp_z) and torch.equal(out_g2, out_g) and torch.allclose(out_s2, exp_s)
    assert torch.allclose(total2, total)

    # list forms, broadcast, all-to-all and point-to-point in one region
    nxt, prv = (rank + 1) % world, (rank - 1) % world

    def more(x):
        parts = [torch.empty_like(x) for _ in range(comm.get_size())]
        comm.all_gather(parts, x, False)
        b = x.clone()
        comm.broadcast(b, 0, False)
        a = torch.empty(comm.get_size() * 2)
        comm.all_to_all_single(a, torch.arange(comm.get_size() * 2.0) + 100 * comm.get_rank(), False)
        got = torch.empty_like(x)
        if comm.get_rank() % 2 == 0:
            comm.send(x, nxt, False)
            comm.recv(got, prv, False)
        else:
            comm.recv(got, prv, False)
            comm.send(x, nxt, False)
        return torch.stack(parts).sum(0), b, a, got

    s, b, a, got = torch.compile(more, fullgraph=True, backend="aot_eager")(x)
    assert torch.equal(s, torch.full((4,), float(tri))) and torch.equal(b, torch.full((4,), 1.0))
    assert torch.equal(a, torch.cat([torch.arange(2.0) + 2 * rank + 100 * src for src in range(world)]))
    assert torch.equal(got, torch.full((4,), float(prv + 1)))

    # rooted and variable-size forms
    def rooted(x):
        g = torch.zeros(comm.get_size() * 4)
        comm.gather_single(g, x, 1, False)
        parts = [torch.zeros(4) for _ in range(comm.get_size())]
        comm.gather(parts, x * 2, 0, False)
        sc = torch.empty(4)
        comm.scatter(sc, [x + 10 * r for r in range(comm.get_size())] if comm.get_rank() == 0 else [], 0, False)
        vs = [torch.empty(r + 1, 2) for r in range(comm.get_size())]
        comm.all_gather_v(vs, torch.full((comm.get_rank() + 1, 2), float(comm.get_rank())), False)
        rv = torch.empty(comm.get_rank() + 1, 2)
        comm.reduce_scatter_v(rv, [torch.full((r + 1, 2), 1.0 + comm.get_rank()) for r in range(comm.get_size())],
                              ReduceOp.SUM, False)
        return g, torch.stack(parts), sc, vs[-1], rv

    g, parts, sc, last, rv = torch.compile(rooted, fullgraph=True, backend="aot_eager")(x)
    assert torch.equal(rv, torch.full((rank + 1, 2), float(tri)))
    every = torch.arange(1, world + 1, dtype=torch.float32).repeat_interleave(4)
    assert torch.equal(g, every if rank == 1 else torch.zeros(world * 4))          # only the root's output is written
    assert torch.equal(parts.flatten(), 2 * every if rank == 0 else torch.zeros(world * 4))
    assert torch.equal(sc, torch.full((4,), 1.0 + 10 * rank))                         # rank 0's x is all ones
    assert last.shape == (world, 2) and float(last[0, 0]) == world - 1

    # a batch of sends and receives becomes one operator
    def ring(x):
        batch = comm.batch_op_create()
        got = torch.empty_like(x)
        batch.send(x * 3, nxt)
        batch.recv(got, prv)
        batch.issue(False).wait()
        return got + 1

    (out_ring), seen_ring = _graph_ops(ring, x)
    assert torch.equal(out_ring, torch.full((4,), 3.0 * (prv + 1) + 1))
    assert sum("batch_send_recv" in s for s in seen_ring) == 1

    # persistent all-gather: the handle comes from outside the region, exec is recorded inside
    agp_out = torch.zeros(world * 4)
    handle = comm.all_gather_p_init(agp_out)

    def persistent(x):
        comm.all_gather_p_exec(handle, x + 1, True).wait()
        return agp_out.sum()

    total_p = torch.compile(persistent, fullgraph=True, backend="aot_eager")(x)
    assert torch.equal(agp_out, torch.arange(2, world + 2, dtype=torch.float32).repeat_interleave(4))
    assert float(total_p) == float(agp_out.sum())
    comm.all_gather_p_free(handle)

    # gradients flow through communicator methods called inside a compiled region (the recorded operators carry
    # autograd formulas): all-reduce of the upstream gradient, reduce-scatter for an all-gather
    def loss_fn(w, inp):
        y = inp * w
        comm.all_reduce(y, ReduceOp.SUM, False)
        g = torch.empty(comm.get_size() * 4)
        comm.all_gather_single(g, y * (comm.get_rank() + 1), False)
        return (g * g).sum()

    w = torch.full((4,), 0.5, requires_grad=True)
    inp = torch.full((4,), float(rank + 1))
    loss = torch.compile(loss_fn, fullgraph=True, backend="aot_eager")(w, inp)
    loss.backward()
    # the same computation written with the differentiable operators of the functional module, uncompiled
    from torchcomms_b200 import functional as F

    w2 = torch.full((4,), 0.5, requires_grad=True)
    y2 = F.all_reduce(inp * w2, "sum", comm)
    g2 = F.all_gather_single((y2 * (rank + 1)).reshape(1, -1), comm).reshape(-1)
    loss2 = (g2 * g2).sum()
    loss2.backward()
    assert torch.allclose(loss, loss2) and torch.allclose(w.grad, w2.grad) and float(w.grad.abs().sum()) > 0

    # a split communicator is enabled as it is made
    sub = comm.split(list(range(world)), "dyn_sub")

    def on_sub(x):
        y = x.clone()
        sub.all_reduce(y, ReduceOp.MAX, False)
        return y * sub.get_size()

    assert torch.equal(torch.compile(on_sub, fullgraph=True, backend="aot_eager")(x), torch.full((4,), float(world * world)))
    sub.finalize()
    comm.finalize()
    D.unregister_from_dynamo()
    assert not D.is_registered() and type(tc.TorchComm.get_rank).__name__ != "function"


def test_communicator_methods_compile_fullgraph_over_gloo():
    run_ranks(_dynamo_worker, 2, timeout=300)


def test_unknown_communicator_or_reduce_op_is_reported_at_trace_time():
    import os

    import pytest

    os.environ.update(RANK="0", WORLD_SIZE="1")
    import torchcomms_b200 as tc
    from torchcomms_b200 import ReduceOp
    from torchcomms_b200.functional import dynamo as D

    made_before = tc.new_comm("fake", torch.device("cpu"), name="dyn_before")
    D.register_with_dynamo()
    try:
        def f(x, c, op):
            y = x.clone()
            c.all_reduce(y, op, False)
            return y

        with pytest.raises(Exception):
            torch.compile(f, fullgraph=True, backend="eager")(torch.ones(2), made_before, ReduceOp.SUM)   # never enabled
        D.enable(made_before)
        torch._dynamo.reset()
        assert torch.equal(torch.compile(f, fullgraph=True, backend="eager")(torch.ones(2), made_before, ReduceOp.SUM), torch.ones(2))
        mine = ReduceOp(tc.RedOpType.MAX)                                                                   # not the predefined object
        with pytest.raises(Exception):
            torch.compile(f, fullgraph=True, backend="eager")(torch.ones(2), made_before, mine)
        D.register_reduce_op(mine, "max")
        torch._dynamo.reset()
        torch.compile(f, fullgraph=True, backend="eager")(torch.ones(2), made_before, mine)
    finally:
        made_before.finalize()
        D.unregister_from_dynamo()


def test_inductor_lowerings_are_registered():
    from torch._inductor.lowering import lowerings

    from torchcomms_b200.functional import inductor as I

    assert I.register_with_inductor() and I.register_with_inductor()
    for op in I.lowered_ops():
        assert op in lowerings, op
    import torch.fx.node as fx_node

    for name in ("barrier", "gather_single", "all_reduce", "send"):
        assert getattr(torch.ops.torchcomms_b200, name).default in fx_node._side_effectful_functions


def test_patch_for_compile_variable_registers_on_import():
    """TORCHCOMMS_PATCH_FOR_COMPILE=1 (the reference's gate) makes importing the functional package enough."""
    import subprocess
    import sys

    code = (
        "import os; os.environ.update(RANK='0', WORLD_SIZE='1')\n"
        "import sys, torch, torchcomms_b200 as tc\n"
        "assert ('torchcomms_b200.functional' in sys.modules) == (os.environ.get('TORCHCOMMS_PATCH_FOR_COMPILE') == '1')\n"
        "from torchcomms_b200.functional import dynamo as D\n"
        "assert D.is_registered() == (os.environ.get('TORCHCOMMS_PATCH_FOR_COMPILE') == '1')\n"
        "if D.is_registered():\n"
        "    c = tc.new_comm('fake', torch.device('cpu'), name='gate')\n"
        "    f = torch.compile(lambda x: x * (c.get_size() + 1), fullgraph=True, backend='eager')\n"
        "    assert float(f(torch.ones(1))) == 2.0\n"
        "    c.finalize()\n"
        "print('ok')\n"
    )
    import os

    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    for flag in ("1", "0"):
        env = dict(os.environ, TORCHCOMMS_PATCH_FOR_COMPILE=flag, PYTHONPATH=root)
        out = subprocess.run([sys.executable, "-c", code], env=env, capture_output=True, text=True, timeout=300)
        assert out.returncode == 0 and out.stdout.strip().endswith("ok"), out.stderr[-2000:]


def test_window_methods_are_traced_in_program_order():
    """put / signal / wait_signal of a window object inside a compiled region: recorded as the window operators,
    chained by the window's token, and get_tensor() reads behind the last of them."""
    import os

    os.environ.update(RANK="0", WORLD_SIZE="1")
    import torchcomms_b200 as tc
    from torchcomms_b200.functional import dynamo as D

    D.register_with_dynamo()
    try:
        comm = tc.new_comm("fake", torch.device("cpu"), name="dyn_win")
        win = comm.new_window()
        buf = torch.zeros(8)
        win.tensor_register(buf)

        def fn(src):
            win.put(src, 0, 2, False)
            win.signal(0, False)
            win.wait_signal(0, False)
            return win.get_tensor() * 2

        expect = torch.tensor([0, 0, 2, 4, 6, 0, 0, 0], dtype=torch.float32)
        assert torch.equal(fn(torch.tensor([1.0, 2.0, 3.0])), expect)          # eager: the bound methods
        buf.zero_()
        out, seen = _graph_ops(fn, torch.tensor([1.0, 2.0, 3.0]))
        assert torch.equal(out, expect)
        ops = [s.split(".")[0] for s in seen if s.startswith("window_")]
        assert ops == ["window_put", "window_signal", "window_wait_signal", "window_read"], seen
        buf.zero_()
        assert torch.equal(torch.compile(fn, fullgraph=True, backend="aot_eager")(torch.tensor([1.0, 2.0, 3.0])), expect)
        win.tensor_deregister()
        # the registration goes with the window object
        import gc

        from torchcomms_b200.functional import ext

        name = D._WIN_BY_ID[id(win)].name
        assert name in ext._windows
        del win
        gc.collect()
        assert name not in ext._windows and not D._WIN_BY_ID
        comm.finalize()
    finally:
        D.unregister_from_dynamo()
