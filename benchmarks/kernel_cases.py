"""Small single-GPU cases of the hot kernels, for timing and for profiler captures.

    python benchmarks/kernel_cases.py --case gemm            # persistent tcgen05 GEMM, 8192 x 4096 x 4096
    python benchmarks/kernel_cases.py --case ag_gemm         # fused all-gather -> GEMM kernel, single rank
    python benchmarks/kernel_cases.py --case gemm_rs         # fused GEMM -> reduce-scatter kernel, single rank
    python benchmarks/kernel_cases.py --case ar_oneshot      # one-shot all-reduce, 8 virtual ranks in one launch
    python benchmarks/kernel_cases.py --case ar_pipe         # pipelined all-reduce, 8 virtual ranks, 32 MB each
    python benchmarks/kernel_cases.py --case rs_cast         # reduce-scatter fp32 -> bf16 wire -> fp32, 8 virtual ranks
    python benchmarks/kernel_cases.py --case ep              # MoE dispatch + combine, 8 virtual ranks
    python benchmarks/kernel_cases.py --case ar_norm         # fused all-reduce + residual + RMSNorm, 8 virtual ranks
    python benchmarks/kernel_cases.py --case model           # RMSNorm, SwiGLU, cross-entropy, AdamW
    python benchmarks/kernel_cases.py --case gemm_fp8        # e4m3 GEMM with row / channel scales, 8192 x 4096 x 4096
    python benchmarks/kernel_cases.py --case gemm_rs_fp8     # fused GEMM -> reduce-scatter kernel on e4m3 operands, single rank
    python benchmarks/kernel_cases.py --case symm            # one-pass all-gather / reduce-scatter / all-reduce, 8 virtual ranks, 32 MB
    python benchmarks/kernel_cases.py --case lamport         # flag-less small all-reduce, 8 virtual ranks, 16 KB
    python benchmarks/kernel_cases.py --case ep_ll           # low-latency MoE dispatch + combine, 8 virtual ranks x 128 tokens

Each case runs ``--warmup`` untimed and ``--iters`` timed launches (CUDA events,
L2-sized scratch write between launches) and prints one line per kernel with
the achieved rate.  Collective kernels run all virtual ranks as one cooperative
launch on one GPU, so their numbers measure the kernel's memory path, not
NVLink.  Inputs are larger than L2 where that matters and stay below a few GB.
"""
from __future__ import annotations

import argparse
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import torch  # noqa: E402

from torchcomms_b200 import _comms  # noqa: E402


def timed(fn, warmup, iters, flush):
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    total = 0.0
    for _ in range(iters):
        flush.zero_()
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record()
        fn()
        e.record()
        e.synchronize()
        total += s.elapsed_time(e)
    return total * 1000.0 / iters  # us


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--case", required=True)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--iters", type=int, default=10)
    args = ap.parse_args()
    torch.cuda.set_device(0)
    dev = torch.device("cuda", 0)
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    bf = torch.bfloat16

    def rnd(*shape, scale=1.0, dtype=bf):
        return (torch.randn(*shape, device=dev) * scale).to(dtype)

    if args.case == "gemm":
        m, n, k = 8192, 4096, 4096
        a, b = rnd(m, k, scale=0.5), rnd(n, k, scale=0.05)
        us = timed(lambda: _comms.ops.gemm_bf16_nt(a, b), args.warmup, args.iters, flush)
        us2 = timed(lambda: _comms.ops.gemm_bf16_nt_pair(a, b), args.warmup, args.iters, flush)
        ref = timed(lambda: torch.matmul(a, b.t()), args.warmup, args.iters, flush)
        fl = 2.0 * m * n * k / 1e6
        print(f"gemm tcgen05 {m}x{n}x{k}: one CTA per tile {us:.1f} us {fl / us:.1f} TFLOP/s; CTA pairs {us2:.1f} us {fl / us2:.1f} TFLOP/s; "
              f"cuBLAS {ref:.1f} us {fl / ref:.1f} TFLOP/s")
    elif args.case in ("ag_gemm", "gemm_rs"):
        from torchcomms_b200.ops.tp import AllGatherGemm, GemmReduceScatter

        m, n, k = 8192, 4096, 4096
        if args.case == "ag_gemm":
            layer = AllGatherGemm(None, m, k)
            layer.input.copy_(rnd(m, k, scale=0.5))
            w = rnd(n, k, scale=0.05)
            us = timed(lambda: layer(w), args.warmup, args.iters, flush)
        else:
            layer = GemmReduceScatter(None, m, n)
            h, w = rnd(m, k, scale=0.5), rnd(n, k, scale=0.05)
            us = timed(lambda: layer(h, w), args.warmup, args.iters, flush)
        print(f"{args.case} single rank {m}x{n}x{k}: {us:.1f} us {2.0 * m * n * k / us / 1e6:.1f} TFLOP/s status {layer.status()[:1]}")
    elif args.case in ("ar_oneshot", "ar_pipe", "rs_cast"):
        nranks = 8
        w = _comms._EmuWorld(nranks, 64 << 20, 2000.0)
        if args.case == "ar_oneshot":
            count = 64 * 1024  # 128 KB bf16 per rank
            ins = [rnd(count) for _ in range(nranks)]
            outs = [torch.empty_like(t) for t in ins]
            us = timed(lambda: w.all_reduce(ins, outs, 0, 1.0, 0, 32, 0), args.warmup, args.iters, flush)
            print(f"all_reduce one-shot, {nranks} virtual ranks x {count * 2} B: {us:.1f} us")
        elif args.case == "ar_pipe":
            count = 16 * 1024 * 1024  # 32 MB bf16 per rank
            ins = [rnd(count) for _ in range(nranks)]
            outs = [torch.empty_like(t) for t in ins]
            us = timed(lambda: w.all_reduce(ins, outs, 0, 1.0, 1, 18, 64 * 1024), args.warmup, args.iters, flush)
            moved = nranks * count * 2 * 4  # copy-in, reduce reads, broadcast writes, copy-out (per rank x ranks)
            print(f"all_reduce pipelined, {nranks} virtual ranks x {count * 2 >> 20} MB: {us:.1f} us (~{moved / us / 1e3:.0f} GB/s of local traffic)")
        else:
            count = 2 * 1024 * 1024  # fp32 in: 8 x 8 MB per rank
            ins = [rnd(nranks * count, dtype=torch.float32) for _ in range(nranks)]
            outs = [torch.empty(count, dtype=torch.float32, device=dev) for _ in range(nranks)]
            us = timed(lambda: w.reduce_scatter(ins, outs, "bf16", 0, 1.0, 18, 32 * 1024), args.warmup, args.iters, flush)
            print(f"reduce_scatter fp32->bf16 wire->fp32, {nranks} virtual ranks x {nranks * count * 4 >> 20} MB in: {us:.1f} us")
        print("status", w.status()[:1])
    elif args.case == "ar_norm":
        nranks, rows, hidden = 8, 32, 8192
        w = _comms._EmuWorld(nranks, 8 << 20, 2000.0)
        xs = [rnd(rows, hidden) for _ in range(nranks)]
        res = [rnd(rows, hidden) for _ in range(nranks)]
        outs = [torch.empty_like(t) for t in xs]
        wn = rnd(hidden)
        us = timed(lambda: w.all_reduce_rmsnorm(xs, res, wn, outs, 1e-5), args.warmup, args.iters, flush)
        flat_in = [t.view(-1) for t in xs]
        flat_out = [torch.empty_like(t) for t in flat_in]

        def unfused():
            w.all_reduce(flat_in, flat_out, 0, 1.0, 0, 32, 0)
            for r in range(nranks):
                res[r].add_(flat_out[r].view(rows, hidden))
                _comms.ops.rmsnorm_fwd(res[r], wn, 1e-5)

        us2 = timed(unfused, args.warmup, args.iters, flush)
        print(f"all_reduce + residual + rmsnorm, {nranks} virtual ranks x [{rows}, {hidden}] bf16: fused {us:.1f} us; "
              f"one-shot all-reduce + add + rmsnorm kernels {us2:.1f} us (both include the emulation launch's host sync)")
        print("status", w.status()[:1])
    elif args.case == "ep":
        nranks, tokens, hidden, experts, topk = 8, 512, 7168, 256, 8
        buf = _comms.EpBuffer.emulated(nranks, tokens, hidden, experts, topk, True, 2000.0)
        xs = [rnd(tokens, hidden) for _ in range(nranks)]
        routes = [torch.softmax(torch.randn(tokens, experts, device=dev), -1).topk(topk, -1) for _ in range(nranks)]
        ws = [r[0].float().contiguous() for r in routes]
        idxs = [r[1].to(torch.int32).contiguous() for r in routes]
        us_d = timed(lambda: buf.dispatch(xs, idxs, ws), args.warmup, args.iters, flush)
        outs = [torch.empty(tokens, hidden, dtype=bf, device=dev) for _ in range(nranks)]
        us_c = timed(lambda: buf.combine(outs), args.warmup, args.iters, flush)
        rows = sum(int(buf.view(r, "recv_info")[0]) for r in range(nranks))
        print(f"ep dispatch, {nranks} virtual ranks x {tokens} tokens: {us_d:.1f} us ({rows} rows, fp8 + scales {rows * (hidden + hidden // 128 * 4) / us_d / 1e3:.0f} GB/s)")
        print(f"ep combine: {us_c:.1f} us ({rows * hidden * 2 / us_c / 1e3:.0f} GB/s) status {buf.status()[:1]}")
    elif args.case == "gemm_fp8":
        from torchcomms_b200.ops.tp import gemm_e4m3_nt, quantize_rows

        m, n, k = 8192, 4096, 4096
        (qa, sa), (qb, sb) = quantize_rows(rnd(m, k, scale=0.5)), quantize_rows(rnd(n, k, scale=0.05))
        us = timed(lambda: gemm_e4m3_nt(qa, qb, sa, sb), args.warmup, args.iters, flush)
        ref = timed(lambda: torch._scaled_mm(qa, qb.t(), scale_a=sa.unsqueeze(1), scale_b=sb.unsqueeze(0), out_dtype=bf),
                    args.warmup, args.iters, flush)
        fl = 2.0 * m * n * k / 1e6
        print(f"gemm e4m3 tcgen05 {m}x{n}x{k}: {us:.1f} us {fl / us:.1f} TFLOP/s; torch._scaled_mm {ref:.1f} us {fl / ref:.1f} TFLOP/s")
    elif args.case == "gemm_rs_fp8":
        from torchcomms_b200.ops.tp import GemmReduceScatter, quantize_rows

        m, n, k = 8192, 4096, 4096
        layer = GemmReduceScatter(None, m, n, fp8=True)
        (qh, sh), (qw, sw) = quantize_rows(rnd(m, k, scale=0.5)), quantize_rows(rnd(n, k, scale=0.05))
        us = timed(lambda: layer(qh, qw, sh, sw), args.warmup, args.iters, flush)
        print(f"gemm_rs e4m3 single rank {m}x{n}x{k}: {us:.1f} us {2.0 * m * n * k / us / 1e6:.1f} TFLOP/s status {layer.status()[:1]}")
    elif args.case == "symm":
        nranks, count = 8, 2 * 1024 * 1024  # 4 MB bf16 per rank part, 32 MB gathered
        w = _comms._EmuWorld(nranks, 8 << 20, 2000.0)
        parts = [rnd(count) for _ in range(nranks)]
        full = [rnd(nranks * count) for _ in range(nranks)]
        outs = [torch.empty(count, dtype=bf, device=dev) for _ in range(nranks)]
        us = timed(lambda: w.symm_all_gather(parts, full, False, 16), args.warmup, args.iters, flush)
        print(f"symm all_gather, {nranks} virtual ranks x {count * 2 >> 20} MB: {us:.1f} us ({nranks * nranks * count * 2 / us / 1e3:.0f} GB/s of stores)")
        us = timed(lambda: w.symm_reduce_scatter(full, outs, 1.0, 16), args.warmup, args.iters, flush)
        print(f"symm reduce_scatter, {nranks} virtual ranks x {nranks * count * 2 >> 20} MB in: {us:.1f} us ({nranks * nranks * count * 2 / us / 1e3:.0f} GB/s of loads)")
        us = timed(lambda: w.symm_all_reduce(full, 1.0 / nranks, 16), args.warmup, args.iters, flush)
        print(f"symm all_reduce in place, {nranks} virtual ranks x {nranks * count * 2 >> 20} MB: {us:.1f} us")
        print("status", w.status()[:1])
    elif args.case == "lamport":
        nranks, count = 8, 8 * 1024  # 16 KB bf16 per rank
        w = _comms._EmuWorld(nranks, 8 << 20, 2000.0)
        ins = [rnd(count) for _ in range(nranks)]
        outs = [torch.empty_like(t) for t in ins]
        us = timed(lambda: w.all_reduce_lamport(ins, outs, 1.0), args.warmup, args.iters, flush)
        print(f"all_reduce flag-less, {nranks} virtual ranks x {count * 2} B: {us:.1f} us (includes the emulation launch's host sync) status {w.status()[:1]}")
    elif args.case == "ep_ll":
        nranks, tokens, hidden, experts, topk = 8, 128, 7168, 256, 8
        buf = _comms.EpLlBuffer.emulated(nranks, tokens, hidden, experts, topk, True, 2000.0)
        xs = [rnd(tokens, hidden) for _ in range(nranks)]
        routes = [torch.softmax(torch.randn(tokens, experts, device=dev), -1).topk(topk, -1) for _ in range(nranks)]
        ws = [r[0].float().contiguous() for r in routes]
        idxs = [r[1].to(torch.int32).contiguous() for r in routes]
        us_d = timed(lambda: buf.dispatch(xs, idxs), args.warmup, args.iters, flush)
        outs = [torch.empty(tokens, hidden, dtype=bf, device=dev) for _ in range(nranks)]
        us_c = timed(lambda: buf.combine(outs, idxs, ws), args.warmup, args.iters, flush)
        pairs = nranks * tokens * topk
        print(f"ep low-latency dispatch, {nranks} virtual ranks x {tokens} tokens: {us_d:.1f} us ({pairs} rows)")
        print(f"ep low-latency combine: {us_c:.1f} us status {buf.status()[:1]}")
    elif args.case == "model":
        rows, cols, vocab, ffn = 8192, 4096, 128256, 14336
        x, wn = rnd(rows, cols), rnd(cols)
        us = timed(lambda: _comms.ops.rmsnorm_fwd(x, wn, 1e-5), args.warmup, args.iters, flush)
        print(f"rmsnorm_fwd {rows}x{cols}: {us:.1f} us {rows * cols * 4 / us / 1e3:.0f} GB/s")
        y, rstd = _comms.ops.rmsnorm_fwd(x, wn, 1e-5)
        us = timed(lambda: _comms.ops.rmsnorm_bwd(y, x, wn, rstd), args.warmup, args.iters, flush)
        print(f"rmsnorm_bwd {rows}x{cols}: {us:.1f} us {rows * cols * 6 / us / 1e3:.0f} GB/s")
        gu = rnd(rows, 2 * ffn)
        us = timed(lambda: _comms.ops.swiglu_fwd(gu), args.warmup, args.iters, flush)
        print(f"swiglu_fwd {rows}x{ffn}: {us:.1f} us {rows * ffn * 6 / us / 1e3:.0f} GB/s")
        logits = rnd(2048, vocab)
        tg = torch.randint(0, vocab, (2048,), device=dev)
        us = timed(lambda: _comms.ops.cross_entropy_fwd_bwd_(logits, tg, 1.0), args.warmup, args.iters, flush)
        print(f"cross_entropy_fwd_bwd 2048x{vocab}: {us:.1f} us {2048 * vocab * 4 / us / 1e3:.0f} GB/s")
        n = 64 * 1024 * 1024
        p, g, m_, v_ = (torch.zeros(n, device=dev) for _ in range(4))
        us = timed(lambda: _comms.ops.adamw_step_(p, g, m_, v_, 1e-3, 0.9, 0.95, 1e-8, 0.1, 1, 1.0), args.warmup, args.iters, flush)
        print(f"adamw {n} params: {us:.1f} us {n * 28 / us / 1e3:.0f} GB/s")
    else:
        raise SystemExit(f"unknown case {args.case}")
    torch.cuda.synchronize()


if __name__ == "__main__":
    main()
