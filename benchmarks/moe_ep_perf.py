"""MoE expert-parallel dispatch / combine latency.

    torchrun --nproc-per-node 8 benchmarks/moe_ep_perf.py \
        [--tokens 4096] [--hidden 7168] [--experts 256] [--topk 8] [--warmup 10] [--iters 50]

Router logits ~N(0,1), softmax, top-k; x ~N(0,1) bf16.  Arms:

  * ``fused``  - ops.moe_ep.Buffer: one kernel does routing counts, block-scaled
                 fp8 (e4m3, 1x128) quantisation, token permutation and the peer
                 stores; combine pulls and applies the weighted top-k sum.
  * ``nccl``   - the unfused pipeline the reference's users run: per-destination
                 token gather, fp8 quantisation in PyTorch, split exchange,
                 ``all_to_all_v_single`` of payload and scales through NCCL;
                 combine: ``all_to_all_v_single`` back in bf16 + index_add.

Device-timed per call (CUDA events), maximum over ranks; the reported
bandwidth counts the payload bytes a rank receives (dispatch) or sends back
(combine).
"""
from __future__ import annotations

import argparse
import json
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import torch  # noqa: E402

import torchcomms_b200 as tc  # noqa: E402
from torchcomms_b200.ops.moe_ep import Buffer, per_token_cast_to_fp8  # noqa: E402


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--tokens", type=int, default=4096)
    ap.add_argument("--hidden", type=int, default=7168)
    ap.add_argument("--experts", type=int, default=256)
    ap.add_argument("--topk", type=int, default=8)
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--iters", type=int, default=50)
    ap.add_argument("--json", default="")
    args = ap.parse_args()

    os.environ.setdefault("RANK", "0")
    os.environ.setdefault("WORLD_SIZE", "1")
    os.environ.setdefault("LOCAL_RANK", os.environ["RANK"])
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    os.environ.setdefault("MASTER_PORT", "29575")
    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    comm = tc.new_comm("b200", dev, name="ep_perf")
    T, H, E, K = args.tokens, args.hidden, args.experts, args.topk
    epr = E // world
    g = torch.Generator(device=dev).manual_seed(1234 + rank)
    x = torch.randn(T, H, generator=g, device=dev).to(torch.bfloat16)
    logits = torch.randn(T, E, generator=g, device=dev)
    w, idx = torch.softmax(logits, -1).topk(K, -1)
    idx = idx.to(torch.int32).contiguous()
    w = w.float().contiguous()
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)

    def time_it(fn):
        for _ in range(args.warmup):
            fn()
        comm.barrier(False)
        torch.cuda.synchronize()
        total = 0.0
        for _ in range(args.iters):
            flush.zero_()
            comm.barrier(False)
            s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            s.record()
            fn()
            e.record()
            e.synchronize()
            total += s.elapsed_time(e)
        t = torch.tensor([total * 1000.0 / args.iters], device=dev)
        comm.all_reduce(t, tc.ReduceOp.MAX, False)
        return float(t.item())

    rows = []

    def report(phase, arm, us, nbytes):
        row = {"phase": phase, "arm": arm, "us": round(us, 1), "gbs": round(nbytes / us / 1e3, 1), "world": world,
               "tokens": T, "hidden": H, "experts": E, "topk": K}
        rows.append(row)
        if rank == 0:
            print(f"{phase:9s} {arm:6s} {us:10.1f} us {row['gbs']:8.1f} GB/s", flush=True)

    # ---------------- fused
    buf = Buffer(comm, max_tokens=T, hidden=H, num_experts=E, topk=K, fp8=True)
    d = buf.dispatch(x, idx, w)
    torch.cuda.synchronize()
    n_recv = int(d.num_tokens)
    recv_bytes = n_recv * (H + H // 128 * 4)
    comb_bytes = n_recv * H * 2
    if rank == 0:
        print(f"# world={world} tokens/rank={T} hidden={H} experts={E} topk={K}: rank 0 receives {n_recv} rows")
    report("dispatch", "fused", time_it(lambda: buf.dispatch(x, idx, w)), recv_bytes)
    buf.combine_input[:n_recv].normal_()
    out = torch.empty(T, H, dtype=torch.bfloat16, device=dev)
    report("combine", "fused", time_it(lambda: buf.combine(out=out)), comb_bytes)

    # ---------------- unfused pipeline over NCCL
    if world > 1:
        hint = {"algo": "nccl"}
        in_rank = torch.stack([((idx // epr) == r).any(dim=1) for r in range(world)], dim=0)  # [world, T]
        state = {}

        def nccl_dispatch():
            sel = [in_rank[r].nonzero().flatten() for r in range(world)]
            counts = torch.tensor([s.numel() for s in sel], dtype=torch.int64, device=dev)  # one sync, as users pay
            order = torch.cat(sel)
            q, sc = per_token_cast_to_fp8(x[order])
            recv_counts = torch.empty_like(counts)
            comm.all_to_all_single(recv_counts, counts, False, hints=hint)
            ins, outs = counts.tolist(), recv_counts.tolist()
            n = sum(outs)
            rq = torch.empty(n, H, dtype=torch.uint8, device=dev)
            rs = torch.empty(n, H // 128, dtype=torch.float32, device=dev)
            comm.all_to_all_v_single(rq, q.view(torch.uint8), outs, ins, False, hints=hint)
            comm.all_to_all_v_single(rs, sc.contiguous(), outs, ins, False, hints=hint)
            state.update(order=order, ins=ins, outs=outs, n=n)
            return rq, rs

        nccl_dispatch()
        torch.cuda.synchronize()
        report("dispatch", "nccl", time_it(nccl_dispatch), state["n"] * (H + H // 128 * 4))
        y_exp = torch.randn(state["n"], H, device=dev).to(torch.bfloat16)

        def nccl_combine():
            back = torch.empty(len(state["order"]), H, dtype=torch.bfloat16, device=dev)
            comm.all_to_all_v_single(back, y_exp, state["ins"], state["outs"], False, hints=hint)
            res = torch.zeros(T, H, dtype=torch.float32, device=dev)
            res.index_add_(0, state["order"], back.float())
            return res.to(torch.bfloat16)

        report("combine", "nccl", time_it(nccl_combine), state["n"] * H * 2)
    torch.cuda.synchronize()
    del buf
    comm.finalize()
    if rank == 0 and args.json:
        with open(args.json, "w") as f:
            json.dump(rows, f)


if __name__ == "__main__":
    main()
