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
            assert (rx[row].view(torch.uint8) == q_ref[0].view(torch.uint8)).float().mean() > 0.98
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
