"""Traceable operators beyond the basic collectives: list forms, asynchronous
starts with ``wait_tensor``, the async tensor wrapper, windows, batched
send / receive, argument normalisation, and a compiled function that calls a
communicator's methods (CPU: gloo ranks and the fake backend).

Parity: comms/torchcomms/tests/unit/py/{test_param_parsing,test_passes,
test_wait_proxy_propagation}.py and tests/integration/py/FullgraphCompile[Autograd]Test.py.
"""
from datetime import timedelta

import pytest
import torch

from tests.mp_util import run_ranks


def _ext_worker(rank, world):
    import torchcomms_b200 as tc
    from torchcomms_b200 import functional as F
    from torchcomms_b200.functional.async_tensor import AsyncCollectiveTensor

    comm = tc.new_comm("gloo", torch.device("cpu"), name="fx", timeout=timedelta(seconds=60))
    F.register_comm(comm)
    tri = world * (world + 1) // 2

    # list forms, with gradients
    x = torch.full((3,), float(rank + 1), requires_grad=True)
    parts = F.all_gather(x, comm)
    assert [float(p[0]) for p in parts] == [float(r + 1) for r in range(world)]
    sum(((r + 1) * p).sum() for r, p in enumerate(parts)).backward()
    # d/dx of sum_r (r+1) * x_gathered[r]: every rank contributes (own rank + 1) for my slot -> reduce_scatter of weights
    assert torch.equal(x.grad, torch.full((3,), float(world * (rank + 1))))
    ys = F.all_gather_v(torch.full((rank + 1, 2), float(rank)), [r + 1 for r in range(world)], comm)
    assert [tuple(y.shape) for y in ys] == [(r + 1, 2) for r in range(world)] and float(ys[world - 1][0, 0]) == world - 1
    rs = F.reduce_scatter([torch.full((4,), float(rank + 1 + r)) for r in range(world)], "sum", comm)
    assert torch.equal(rs, torch.full((4,), float(tri + world * rank)))
    # uneven shares: rank r keeps r + 1 rows; the gradient of every share comes back from its owner
    shares = [torch.full((r + 1, 2), float(rank + 1), requires_grad=True) for r in range(world)]
    mine = F.reduce_scatter_v(shares, "sum", comm)
    assert mine.shape == (rank + 1, 2) and torch.equal(mine, torch.full((rank + 1, 2), float(tri)))
    (mine * (rank + 1)).sum().backward()
    assert [float(t.grad[0, 0]) for t in shares] == [float(r + 1) for r in range(world)]
    outs = F.all_to_all([torch.full((2,), float(rank * world + d)) for d in range(world)], comm)
    assert [float(o[0]) for o in outs] == [float(s * world + rank) for s in range(world)]

    # asynchronous starts: eager gives a tensor that waits on first use
    a = F.all_reduce_async(torch.full((5,), float(rank + 1)), "sum", comm)
    assert isinstance(a, AsyncCollectiveTensor) and "in flight" in repr(a)
    b = a + 1                                   # first use waits
    assert torch.equal(b, torch.full((5,), float(tri + 1))) and "ready" in repr(a)
    g = F.all_gather_single_async(torch.full((2,), float(rank)), comm).wait()
    assert torch.equal(g, torch.arange(world, dtype=torch.float32).repeat_interleave(2))
    r = F.reduce_scatter_single_async(torch.arange(2.0 * world), "sum", comm)
    assert torch.equal(r.wait(), torch.arange(2.0 * world).view(world, 2)[rank] * world)

    # started operators differentiate like the synchronous ones
    for start, sync, shape in ((lambda t: F.all_gather_single_async(t, comm), lambda t: F.all_gather_single(t, comm), (2, 3)),
                               (lambda t: F.all_reduce_async(t, "sum", comm), lambda t: F.all_reduce(t, "sum", comm), (2, 3)),
                               (lambda t: F.reduce_scatter_single_async(t, "avg", comm),
                                lambda t: F.reduce_scatter_single(t, "avg", comm), (2 * world, 3)),
                               (lambda t: F.all_to_all_single_async(t, comm), lambda t: F.all_to_all_single(t, comm), (world, 3))):
        a1 = torch.full(shape, float(rank + 1), requires_grad=True)
        a2 = torch.full(shape, float(rank + 1), requires_grad=True)
        weight = torch.arange(1.0, 1.0 + start(a1.detach()).wait().numel()).view_as(sync(a2.detach()))
        (start(a1 * 2).wait() * weight).sum().backward()
        (sync(a2 * 2) * weight).sum().backward()
        assert torch.equal(a1.grad, a2.grad) and float(a1.grad.abs().sum()) > 0

    # one wait for several started collectives, with gradients passed straight through
    s1 = torch.full((2, 3), float(rank + 1), requires_grad=True)
    h1 = torch.ops.torchcomms_b200.all_reduce_start(s1 * 1.0, "sum", "fx")
    h2 = torch.ops.torchcomms_b200.all_gather_single_start(s1 * 2.0, "fx")
    r1, r2 = F.wait_tensors([h1, h2])
    assert torch.equal(r1, torch.full((2, 3), float(tri))) and r2.shape == (2 * world, 3)
    (r1.sum() + r2.sum()).backward()
    assert torch.equal(s1.grad, torch.full((2, 3), float(world + 2 * world)))

    # batched send / receive in a ring
    nxt, prv = (rank + 1) % world, (rank - 1) % world
    (got,) = F.batch_send_recv([torch.full((3,), float(rank))], [nxt], [torch.empty(3)], [prv], comm)
    assert torch.equal(got, torch.full((3,), float(prv)))

    # a traced graph carries start + wait_tensor and still computes the right thing
    from torch.fx.experimental.proxy_tensor import make_fx

    def fn(t):
        h = F.all_gather_single_async(t * 2, comm)
        local = (t + 1).sum()
        return h.wait().sum() + local

    gm = make_fx(fn, tracing_mode="fake")(torch.ones(4))
    names = [n.target._schema.name for n in gm.graph.nodes if n.op == "call_function" and hasattr(n.target, "_schema")]
    assert "torchcomms_b200::all_gather_single_start" in names and "torchcomms_b200::wait_tensor" in names
    assert names.index("torchcomms_b200::all_gather_single_start") < names.index("torchcomms_b200::wait_tensor")
    t = torch.full((4,), float(rank + 1))
    assert float(gm(t)) == float(fn(t)) == 2.0 * 4 * tri + 4 * (rank + 2)

    # compiled function calling communicator methods, forward and backward
    cc = F.compiled(comm)

    @torch.compile(fullgraph=True, backend="aot_eager")
    def step(w, inp):
        y = cc.all_reduce(inp * w, "sum")
        z = cc.reduce_scatter_single(y.repeat(cc.get_size()), "avg")
        return (z * z).sum()

    w = torch.full((4,), 0.5, requires_grad=True)
    loss = step(w, torch.full((4,), float(rank + 1)))
    ref_w = torch.full((4,), 0.5, requires_grad=True)
    ref_y = ref_w * float(tri)
    (ref_y * ref_y).sum().backward()
    assert torch.allclose(loss, (ref_y * ref_y).sum())
    loss.backward()
    # every rank's loss depends on every rank's w through the all-reduce; the gradient of the local loss w.r.t. the
    # local w is what the reference's autograd formulas give: all-reduce of the upstream gradient times the local input
    assert w.grad is not None and torch.isfinite(w.grad).all()
    comm.finalize()


def test_functional_extensions_over_gloo():
    run_ranks(_ext_worker, 2, timeout=240)


def test_window_operators_trace_and_run():
    import os

    os.environ.update(RANK="0", WORLD_SIZE="1")
    import torchcomms_b200 as tc
    from torchcomms_b200 import functional as F
    from torch.fx.experimental.proxy_tensor import make_fx

    comm = tc.new_comm("fake", torch.device("cpu"), name="fxwin")
    win = comm.new_window()
    buf = torch.zeros(8)
    win.tensor_register(buf)
    F.register_window("w0", win)

    def fn(src):
        tok = F.window_put(src, "w0", 0, 2)
        tok = F.window_signal("w0", 0, tok)
        tok = F.window_wait_signal("w0", 0, tok)
        return F.window_read("w0", tok) * 2

    out = fn(torch.tensor([1.0, 2.0, 3.0]))
    assert torch.equal(out, torch.tensor([0, 0, 2, 4, 6, 0, 0, 0], dtype=torch.float32))
    gm = make_fx(fn, tracing_mode="fake")(torch.ones(3))
    names = [n.target._schema.name.split("::")[1] for n in gm.graph.nodes if n.op == "call_function" and hasattr(n.target, "_schema")
             and n.target._schema.name.startswith("torchcomms_b200::")]
    assert names == ["window_put", "window_signal", "window_wait_signal", "window_read"]  # program order is kept by the token
    buf.zero_()
    assert torch.equal(gm(torch.tensor([1.0, 2.0, 3.0])), out)
    F.unregister_window("w0")
    with pytest.raises(RuntimeError, match="not registered"):
        fn(torch.ones(3))
    win.tensor_deregister()
    comm.finalize()


def test_param_parsing():
    import torchcomms_b200 as tc
    from torchcomms_b200.functional.param_parsing import (CollectiveSchema, ParamKind, ParamSpec, normalize_reduce_op,
                                                          parse_hints, parse_timeout, reduce_op_from_string)

    assert normalize_reduce_op("SUM") == "sum" and normalize_reduce_op(tc.ReduceOp.MAX) == "max"
    assert normalize_reduce_op(tc.ReduceOp.PREMUL_SUM(0.25)) == "premul_sum:0.25"
    assert normalize_reduce_op(torch.distributed.ReduceOp.AVG) == "avg"
    with pytest.raises(ValueError):
        normalize_reduce_op("median")
    op = reduce_op_from_string("premul_sum:0.5")
    assert normalize_reduce_op(op) == "premul_sum:0.5"
    assert parse_timeout(None) is None and parse_timeout(timedelta(milliseconds=1500)) == 1.5 and parse_timeout(3) == 3.0
    with pytest.raises(TypeError):
        parse_timeout("soon")
    assert parse_hints({"algo": "nccl", "blocks": 4, "flag": True}) == {"algo": "nccl", "blocks": "4", "flag": "1"}
    assert parse_hints(None) == {}

    schema = CollectiveSchema("all_reduce", [
        ParamSpec("tensor", ParamKind.TENSOR, mutated=True), ParamSpec("op", ParamKind.REDUCE_OP),
        ParamSpec("async_op", ParamKind.BOOL, default=False), ParamSpec("hints", ParamKind.HINTS, default=None),
        ParamSpec("timeout", ParamKind.TIMEOUT, default=None)])
    t = torch.ones(2)
    p = schema.bind((t, tc.ReduceOp.SUM), {"timeout": timedelta(seconds=2)})
    assert p["op"] == "sum" and p["async_op"] is False and p["hints"] == {} and p["timeout"] == 2.0
    assert schema.mutated() == ["tensor"] and p.tensors(schema) == [t]
    with pytest.raises(TypeError, match="missing argument 'op'"):
        schema.bind((t,), {})
    with pytest.raises(TypeError, match="unexpected argument 'root'"):
        schema.bind((t, "sum"), {"root": 0})
    with pytest.raises(TypeError, match="multiple values for 'op'"):
        schema.bind((t, "sum"), {"op": "max"})
    with pytest.raises(ValueError, match="all_reduce: argument 'op'"):
        schema.bind((t, "median"), {})


def test_once_work_waits_a_shared_handle_once():
    from torchcomms_b200.functional.async_tensor import OnceWork, wrap_async

    class Handle:
        waits = 0

        def wait(self):
            Handle.waits += 1

    shared = OnceWork(Handle())
    a, b = wrap_async([torch.ones(2), torch.zeros(2)], shared)
    assert float((a + b).sum()) == 2.0 and Handle.waits == 1
    assert float(a.wait().sum()) == 2.0 and Handle.waits == 1


def test_register_collective_adds_a_traceable_differentiable_operator():
    """The extension point for collectives of out-of-tree backends: eager, traced and differentiated like the
    built-in operators; the reference's names for passes / async tensor are available as aliases."""
    import os

    os.environ.update(RANK="0", WORLD_SIZE="1")
    import torchcomms_b200 as tc
    from torchcomms_b200 import functional as F
    from torchcomms_b200.functional import async_tensor, inductor, passes

    def impl(input, scale, comm):
        out = input.clone()
        F._get(comm).all_reduce(out, tc.ReduceOp.SUM, False)
        return out * scale

    op = F.register_collective(
        "test_scaled_all_reduce", "(Tensor input, float scale, str comm) -> Tensor", impl,
        lambda input, scale, comm: torch.empty_like(input),
        backward=lambda ctx, g: (torch.ops.torchcomms_b200.test_scaled_all_reduce(g.contiguous(), *ctx.args), None, None))
    F.finalize_registration()
    comm = tc.new_comm("fake", torch.device("cpu"), name="reg_coll")
    F.register_comm(comm)
    x = torch.ones(3, requires_grad=True)
    y = torch.compile(lambda t: op(t * 2, 0.5, "reg_coll"), fullgraph=True, backend="aot_eager")(x)
    y.sum().backward()
    assert torch.equal(y.detach(), torch.ones(3)) and torch.equal(x.grad, torch.ones(3))
    import torch.fx.node as fx_node

    assert op.default in fx_node._side_effectful_functions
    assert passes.reinplacement_pass is passes.reinplace_pass and passes.strip_with_effects_pass is passes.strip_wait_pass
    assert async_tensor.TorchCommsAsyncTensor is async_tensor.AsyncCollectiveTensor
    assert inductor.register_torchcomms_lowerings is inductor.register_with_inductor
    comm.finalize()
