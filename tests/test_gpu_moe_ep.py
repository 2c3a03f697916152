"""MoE expert-parallel dispatch / combine: emulated ranks on one GPU checked
against a PyTorch reference, then the real multi-process path."""
import os
from datetime import timedelta

import pytest
import torch

from tests.mp_util import run_ranks

pytestmark = pytest.mark.gpu


def _route(tokens, num_experts, topk, seed):
    g = torch.Generator(device="cuda").manual_seed(seed)
    logits = torch.randn(tokens, num_experts, generator=g, device="cuda")
    w, idx = torch.softmax(logits, dim=-1).topk(topk, dim=-1)
    return idx.to(torch.int32).contiguous(), w.float().contiguous()


def _check_dispatch(r, nranks, epr, topk, max_tokens, xs, idxs, ws, view, fp8):
    from torchcomms_b200.ops.moe_ep import per_token_cast_to_fp8

    info = view(r, "recv_info").cpu()
    n = int(info[0])
    src = view(r, "recv_src")[:n].cpu()
    # expected set of (src_rank, token) pairs, packed by source rank
    expect = []
    for s in range(nranks):
        hit = ((idxs[s] // epr) == r).any(dim=1).nonzero().flatten().cpu().tolist()
        assert int(info[1 + s]) == len(hit), (r, s, int(info[1 + s]), len(hit))
        expect += [s * max_tokens + t for t in hit]
    assert n == len(expect)
    assert sorted(src.tolist()) == sorted(expect)
    # rows of one source are contiguous
    bounds = torch.tensor([0] + [int(v) for v in info[1:].tolist()]).cumsum(0)
    for s in range(nranks):
        seg = src[bounds[s] : bounds[s + 1]]
        assert ((seg // max_tokens) == s).all()
    rx = view(r, "recv_x")[:n]
    tidx = view(r, "recv_topk_idx")[:n].cpu()
    tw = view(r, "recv_topk_weights")[:n].cpu()
    for row in range(0, n, max(1, n // 40)):
        s, t = int(src[row]) // max_tokens, int(src[row]) % max_tokens
        x_ref = xs[s][t].float()
        if fp8:
            scales = view(r, "recv_scales")[row]
            deq = rx[row].float().view(-1, 128) * scales.unsqueeze(-1)
            torch.testing.assert_close(deq.view(-1), x_ref, rtol=0.07, atol=0.02)
            q_ref, s_ref = per_token_cast_to_fp8(xs[s][t : t + 1])
            torch.testing.assert_close(scales, s_ref[0], rtol=1e-5, atol=1e-8)
            # identical bits to the reference quantisation except for ties
            assert (rx[row].view(torch.uint8) == q_ref[0].view(torch.uint8)).float().mean() > 0.95
        else:
            assert torch.equal(rx[row].float(), x_ref)
        gi, gw = idxs[s][t].cpu(), ws[s][t].cpu()
        here = (gi // epr) == r
        assert torch.equal(tidx[row], torch.where(here, gi - r * epr, torch.full_like(gi, -1)))
        assert torch.equal(tw[row], torch.where(here, gw, torch.zeros_like(gw)))
    return n


@pytest.mark.parametrize("nranks,fp8", [(2, True), (4, True), (8, True), (4, False)])
def test_dispatch_combine_emulated(nranks, fp8):
    from torchcomms_b200 import _comms

    tokens, hidden, topk = 96, 1024, 4
    num_experts = nranks * 4
    epr = num_experts // nranks
    buf = _comms.EpBuffer.emulated(nranks, 128, hidden, num_experts, topk, fp8, 2000.0)
    torch.manual_seed(1234 + nranks)
    for it in range(2):  # second round: counters, flags and slots are reusable
        xs = [(torch.randn(tokens, hidden, device="cuda") * (1 + r)).to(torch.bfloat16) for r in range(nranks)]
        routes = [_route(tokens, num_experts, topk, 10 * it + r) for r in range(nranks)]
        idxs, ws = [a for a, _ in routes], [b for _, b in routes]
        idxs[0][0, 0] = -1  # an unrouted slot
        buf.dispatch(xs, idxs, ws)
        torch.cuda.synchronize()
        assert buf.status()[0] == 0
        counts = [_check_dispatch(r, nranks, epr, topk, 128, xs, idxs, ws, buf.view, fp8) for r in range(nranks)]
        # "experts": every rank scales the rows it received by (rank + 1) and writes them to its combine buffer
        for r in range(nranks):
            rx = buf.view(r, "recv_x")[: counts[r]].float()
            if fp8:
                sc = buf.view(r, "recv_scales")[: counts[r]]
                rx = (rx.view(counts[r], -1, 128) * sc.unsqueeze(-1)).view(counts[r], hidden)
            buf.view(r, "combine_x")[: counts[r]] = (rx * (r + 1)).to(torch.bfloat16)
        outs = [torch.empty(tokens, hidden, dtype=torch.bfloat16, device="cuda") for _ in range(nranks)]
        wts = [torch.rand(tokens, nranks, device="cuda") for _ in range(nranks)]
        bias = [torch.randn(tokens, hidden, device="cuda").to(torch.bfloat16) for _ in range(nranks)]
        buf.combine(outs, wts, bias)
        torch.cuda.synchronize()
        assert buf.status()[0] == 0
        for s in range(nranks):
            in_rank = torch.stack([((idxs[s] // epr) == d).any(dim=1) & True for d in range(nranks)], dim=1)
            valid = idxs[s] >= 0
            in_rank = torch.stack([(((idxs[s] // epr) == d) & valid).any(dim=1) for d in range(nranks)], dim=1).float()
            coef = (in_rank * wts[s] * torch.arange(1, nranks + 1, device="cuda")).sum(dim=1, keepdim=True)
            ref = bias[s].float() + coef * xs[s].float()
            torch.testing.assert_close(outs[s].float(), ref, rtol=0.08, atol=0.15 * nranks)
        # per-expert weights travel back through the combine (handles given explicitly, as a later call would)
        handles = [buf.view(r, "send_slot").clone() for r in range(nranks)]
        for r in range(nranks):
            buf.view(r, "combine_topk_weights")[: counts[r]] = buf.view(r, "recv_topk_weights")[: counts[r]]
        w_back = [torch.full((tokens, topk), -1.0, device="cuda") for _ in range(nranks)]
        buf.combine(outs, [], [], handles, w_back)
        torch.cuda.synchronize()
        for s in range(nranks):
            torch.testing.assert_close(w_back[s], torch.where(idxs[s] >= 0, ws[s], torch.zeros_like(ws[s])))
        # cached dispatch: the receivers pull the same rows again, this time bf16 rows out of the sources' staging
        fresh = [(torch.randn(tokens, hidden, device="cuda") * (1 + r)).to(torch.bfloat16) for r in range(nranks)]
        for r in range(nranks):
            buf.view(r, "stage_x")[:tokens] = fresh[r]
        srcs = [buf.view(r, "recv_src").clone() for r in range(nranks)]
        nums = [buf.view(r, "recv_info")[0].clone() for r in range(nranks)]
        pulled = [torch.zeros(128 * nranks, hidden, dtype=torch.bfloat16, device="cuda") for _ in range(nranks)]
        buf.pull(pulled, srcs, nums)
        torch.cuda.synchronize()
        assert buf.status()[0] == 0
        for r in range(nranks):
            src = srcs[r][: counts[r]].long()
            want = torch.stack([fresh[int(v) // 128][int(v) % 128] for v in src.tolist()]) if counts[r] else pulled[r][:0]
            assert torch.equal(pulled[r][: counts[r]], want)
            assert not pulled[r][counts[r]:].any()


def test_layout_kernel():
    from torchcomms_b200.ops.moe_ep import get_dispatch_layout

    idx, _ = _route(500, 32, 4, 3)
    per_rank, per_expert, in_rank = get_dispatch_layout(idx, 32, 8)
    ref_expert = torch.bincount(idx.flatten().long(), minlength=32).int()
    assert torch.equal(per_expert, ref_expert)
    ref_in = torch.stack([((idx // 4) == r).any(dim=1) for r in range(8)], dim=1).int()
    assert torch.equal(in_rank, ref_in)
    assert torch.equal(per_rank, ref_in.sum(0).int())


def _ep_worker(rank, world):
    import torchcomms_b200 as tc
    from torchcomms_b200.ops.moe_ep import Buffer

    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    comm = tc.new_comm("b200", dev, name="ep", timeout=timedelta(seconds=60), abort_process_on_timeout_or_error=False)
    tokens, hidden, topk, experts = 200, 1024, 4, world * 4
    epr = experts // world
    buf = Buffer(comm, max_tokens=256, hidden=hidden, num_experts=experts, topk=topk, fp8=True)
    for it in range(3):
        g = torch.Generator(device=dev).manual_seed(100 * it + rank)
        x = torch.randn(tokens, hidden, generator=g, device=dev).to(torch.bfloat16)
        logits = torch.randn(tokens, experts, generator=g, device=dev)
        w, idx = torch.softmax(logits, -1).topk(topk, -1)
        d = buf.dispatch(x, idx, w)
        n = int(d.num_tokens)
        assert n == int(d.tokens_per_src.sum())
        # every received row really is routed to one of this rank's experts
        assert bool(((d.topk_idx[:n] >= 0) & (d.topk_idx[:n] < epr)).any(dim=1).all())
        # identity experts: combine must give (number of destination ranks) * x
        deq = (d.x[:n].float().view(n, -1, 128) * d.scales[:n].unsqueeze(-1)).view(n, hidden)
        buf.combine_input[:n] = deq.to(torch.bfloat16)
        y = buf.combine()
        torch.cuda.synchronize()
        fanout = torch.stack([((idx // epr) == r).any(dim=1) for r in range(world)], 1).sum(1, keepdim=True).float()
        torch.testing.assert_close(y.float(), fanout * x.float(), rtol=0.08, atol=0.3)
    comm.finalize()


def test_dispatch_combine_multi_gpu():
    world = min(torch.cuda.device_count(), int(os.environ.get("B200COMMS_TEST_WORLD", "2")))
    if world < 2:
        pytest.skip("needs 2 GPUs")
    run_ranks(_ep_worker, world, timeout=150)


@pytest.mark.parametrize("nranks,fp8,topk", [(2, True, 4), (4, True, 8), (8, True, 8), (4, False, 2)])
def test_low_latency_emulated(nranks, fp8, topk):
    """Fixed-slot dispatch and pull combine with virtual ranks on one GPU, three calls (both buffer parities)."""
    from torchcomms_b200 import _comms
    from torchcomms_b200.ops.moe_ep import per_token_cast_to_fp8

    tokens, max_tokens, hidden = 24, 32, 1024
    num_experts = nranks * 4
    le_n = num_experts // nranks
    buf = _comms.EpLlBuffer.emulated(nranks, max_tokens, hidden, num_experts, topk, fp8, 2000.0)
    torch.manual_seed(4321 + nranks)
    for it in range(3):
        xs = [(torch.randn(tokens, hidden, device="cuda") * (1 + r)).to(torch.bfloat16) for r in range(nranks)]
        routes = [_route(tokens, num_experts, topk, 50 * it + r) for r in range(nranks)]
        idxs, ws = [a for a, _ in routes], [b for _, b in routes]
        idxs[0][0, 0] = -1  # an unrouted pair
        outs = buf.dispatch(xs, idxs)
        torch.cuda.synchronize()
        assert buf.status()[0] == 0
        for r in range(nranks):
            px, ps, src, count, rng = outs[r]
            for le in range(le_n):
                ex = r * le_n + le
                want_rows = [(s, t) for s in range(nranks) for t in (idxs[s] == ex).any(dim=1).nonzero().flatten().tolist()]
                n = int(count[le])
                assert n == len(want_rows), (it, r, le, n, len(want_rows))
                # sources in rank order, ranges consistent with the counts
                begins = [int(v) >> 32 for v in rng[le].tolist()]
                lens = [int(v) & 0xFFFFFFFF for v in rng[le].tolist()]
                assert sum(lens) == n and begins == [sum(lens[:s]) for s in range(nranks)]
                got = []
                for s in range(nranks):
                    got += [(s, int(t)) for t in src[le, begins[s] : begins[s] + lens[s]].tolist()]
                assert sorted(got) == sorted(want_rows)
                for j, (s, t) in enumerate(got[: 6]):
                    if fp8:
                        deq = px[le, j].float().view(-1, 128) * ps[le, j].unsqueeze(-1)
                        torch.testing.assert_close(deq.view(-1), xs[s][t].float(), rtol=0.07, atol=0.02)
                        _, s_ref = per_token_cast_to_fp8(xs[s][t : t + 1])
                        torch.testing.assert_close(ps[le, j], s_ref[0], rtol=1e-5, atol=1e-8)
                    else:
                        assert torch.equal(px[le, j], xs[s][t])
        # "experts": expert e multiplies its rows by (e + 1)
        for r in range(nranks):
            px, ps, src, count, rng = outs[r]
            rows = px.float()
            if fp8:
                rows = (rows.view(le_n, -1, hidden // 128, 128) * ps.unsqueeze(-1)).view(le_n, -1, hidden)
            scale = torch.arange(r * le_n + 1, (r + 1) * le_n + 1, device="cuda").view(le_n, 1, 1)
            buf.view(r, "out_x").copy_((rows * scale).to(torch.bfloat16))
        ys = [torch.empty(tokens, hidden, dtype=torch.bfloat16, device="cuda") for _ in range(nranks)]
        handles = [buf.view(r, "send_slot").clone() for r in range(nranks)], [buf.view(r, "begin").clone() for r in range(nranks)]
        buf.combine(ys, idxs, ws, *handles)
        torch.cuda.synchronize()
        assert buf.status()[0] == 0
        for s in range(nranks):
            valid = (idxs[s] >= 0).float()
            coef = (ws[s] * (idxs[s] + 1).float() * valid).sum(dim=1, keepdim=True)
            torch.testing.assert_close(ys[s].float(), coef * xs[s].float(), rtol=0.08, atol=0.05 * num_experts)


def _ep_train_worker(rank, world):
    """The fused trainable layer against the all-to-all layer: same outputs, same gradients."""
    import copy

    import torchcomms_b200 as tc
    from torchcomms_b200.parallel.expert import ExpertParallelMoETrain, ExpertParallelMoEUnfused

    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    comm = tc.new_comm("b200", dev, name="ept", timeout=timedelta(seconds=60), abort_process_on_timeout_or_error=False)
    tokens, hidden, topk, experts = 64, 512, 2, world * 2
    torch.manual_seed(7 + rank)
    local = [torch.nn.Sequential(torch.nn.Linear(hidden, hidden, bias=False), torch.nn.Tanh()).to(dev).to(torch.bfloat16)
             for _ in range(experts // world)]
    torch.manual_seed(3)
    router = torch.nn.Linear(hidden, experts, bias=False).to(dev).to(torch.bfloat16)
    fused = ExpertParallelMoETrain(comm, hidden, experts, topk, 128, copy.deepcopy(local), copy.deepcopy(router))
    plain = ExpertParallelMoEUnfused(comm, hidden, experts, topk, copy.deepcopy(local), copy.deepcopy(router))
    for it in range(2):
        g = torch.Generator(device=dev).manual_seed(11 * it + rank)
        x1 = torch.randn(tokens, hidden, generator=g, device=dev).to(torch.bfloat16).requires_grad_()
        x2 = x1.detach().clone().requires_grad_()
        target = torch.randn(tokens, hidden, generator=g, device=dev)
        y1, y2 = fused(x1), plain(x2)
        torch.testing.assert_close(y1.float(), y2.float(), rtol=0.05, atol=0.05)
        ((y1.float() - target) ** 2).sum().div(tokens).backward()
        ((y2.float() - target) ** 2).sum().div(tokens).backward()
        torch.cuda.synchronize()

        def rel(a, b):
            return float((a.float() - b.float()).norm() / b.float().norm().clamp_min(1e-12))

        assert rel(x1.grad, x2.grad) < 0.03, rel(x1.grad, x2.grad)
        for (name, p1), p2 in zip(fused.named_parameters(), plain.parameters()):
            assert p1.grad is not None and p2.grad is not None, name
            assert rel(p1.grad, p2.grad) < 0.03, (name, rel(p1.grad, p2.grad))
        fused.zero_grad()
        plain.zero_grad()
    comm.finalize()


def _link_ep_worker(rank, world):
    """The reference's call sequence (layout -> dispatch -> combine, cached dispatch, low-latency pair)."""
    import torchcomms_b200 as tc
    from torchcomms_b200.ops.link_ep import Buffer, EventOverlap

    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    comm = tc.new_comm("b200", dev, name="lep", timeout=timedelta(seconds=60), abort_process_on_timeout_or_error=False)
    tokens, hidden, topk, experts = 100, 1024, 4, world * 4
    epr = experts // world
    buffer = Buffer(comm, hidden=hidden, num_experts=experts, num_topk=topk, num_max_tokens=128,
                    low_latency_mode=True, num_max_dispatch_tokens_per_rank=128, low_latency_fp8=False)
    g = torch.Generator(device=dev).manual_seed(5 + rank)
    x = torch.randn(tokens, hidden, generator=g, device=dev).to(torch.bfloat16)
    w, idx = torch.softmax(torch.randn(tokens, experts, generator=g, device=dev), -1).topk(topk, -1)
    ntpr, none, ntpe, in_rank, ev = buffer.get_dispatch_layout(idx, experts)
    assert none is None and in_rank.dtype == torch.bool and int(ntpe.sum()) == tokens * topk
    assert torch.equal(ntpr.long(), in_rank.sum(0))
    recv_x, recv_idx, recv_w, counts, handle, ev = buffer.dispatch(
        x, num_tokens_per_rank=ntpr, is_token_in_rank=in_rank, num_tokens_per_expert=ntpe, topk_idx=idx, topk_weights=w,
        async_finish=True)
    assert isinstance(ev, EventOverlap) and ev.event is not None
    ev.current_stream_wait()
    n = recv_x.shape[0]
    assert len(counts) == epr and sum(counts) == int((recv_idx >= 0).sum()) and recv_idx.dtype == idx.dtype
    fan = in_rank.sum(1, keepdim=True).float()
    y, w_back, ev = buffer.combine(recv_x, handle, topk_weights=recv_w)
    torch.cuda.synchronize()
    torch.testing.assert_close(y.float(), fan * x.float(), rtol=0.02, atol=0.1)
    torch.testing.assert_close(w_back, w.float())
    # cached dispatch: other rows along the same layout
    x2 = (x.float() * 2).to(torch.bfloat16)
    again, a, b, c, handle2, _ = buffer.dispatch(x2, handle=handle)
    assert a is None and b is None and c == [] and again.shape[0] == n
    torch.cuda.synchronize()
    assert torch.equal(again.float(), recv_x.float() * 2)
    # low-latency pair: identity experts scaled by the gate weights
    t2 = 32
    xr, count, h, ev, hook = buffer.low_latency_dispatch(x[:t2], idx[:t2], 128, experts, use_fp8=False)
    assert xr.shape == (epr, world * 128, hidden) and hook is None
    out_buf = buffer.get_next_low_latency_combine_buffer(h)
    out_buf.copy_(xr)
    y2, ev, hook = buffer.low_latency_combine(out_buf, idx[:t2], w[:t2], h, zero_copy=True)
    torch.cuda.synchronize()
    torch.testing.assert_close(y2.float(), w[:t2].sum(1, keepdim=True) * x[:t2].float(), rtol=0.02, atol=0.05)
    comm.finalize()


@pytest.mark.parametrize("worker", [_ep_train_worker, _link_ep_worker])
def test_fused_training_and_link_ep_surface_multi_gpu(worker):
    world = min(torch.cuda.device_count(), int(os.environ.get("B200COMMS_TEST_WORLD", "2")))
    if world < 2:
        pytest.skip("needs 2 GPUs")
    run_ranks(worker, world, timeout=150)
