"""Tensor-parallel MLP layers: fused kernels versus GEMM + collective.

    python benchmarks/tp_layer_perf.py                       # 1 GPU: GEMM kernels only
    torchrun --nproc-per-node N benchmarks/tp_layer_perf.py  # fused layers on N ranks

Default shape: the MLP of Llama-3-70B (hidden 8192, ffn 28672) on ``tokens``
rows, sharded over the N ranks.  Timed per call on the device with CUDA
events (median of the calls), an L2-sized scratch write and a barrier before
each call, maximum over ranks.

Arms:
  * ``fused``   - ops.tp.AllGatherGemm / GemmReduceScatter (one kernel each)
  * ``unfused`` - this framework's all-gather / reduce-scatter collective
                  followed / preceded by ``torch.matmul`` (cuBLAS)
  * ``nccl``    - the same with the collective routed through NCCL
  * ``nccl-ovl``- NCCL and cuBLAS overlapped by hand: the rows are cut into ``--chunks`` pieces, the
                  collective of one piece runs on the communicator's stream while cuBLAS works on its
                  neighbour (the strongest baseline that needs no fused kernel)
  * ``cublas`` / ``tcgen05`` / ``tcgen05x2`` - the local GEMM alone (cuBLAS, this framework's
                  kernel with one CTA per tile, and on CTA pairs): the lower bound of any arm
  * ``*-fp8``   - the same with e4m3 operands and per-row / per-channel fp32 scales
                  (``cublas-fp8`` is ``torch._scaled_mm``); TFLOP/s counts the same 2mnk
"""
from __future__ import annotations

import argparse
import json
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import torch  # noqa: E402

import torchcomms_b200 as tc  # noqa: E402
from torchcomms_b200 import _comms  # noqa: E402
from torchcomms_b200.ops.tp import AllGatherGemm, GemmReduceScatter, gemm_e4m3_nt, quantize_rows  # noqa: E402


PHASES = ["start", "loads issued", "MMAs committed", "tiles stored", "copy / forward warps done", "first own tile complete",
          "reduce warps done", "CTA done", "closing barrier passed"]


def phase_timeline(comm, dev, path, calls):
    """One traced call of each fused kernel: when each phase ended on each CTA, relative to the earliest CTA start
    on this GPU (the kernels stamp the GPU's nanosecond timer). Written by every rank into one text file each."""
    impl = comm.get_backend_impl()
    lines = []
    for name, fn in calls.items():
        for _ in range(2):
            fn()
        comm.barrier(False)
        torch.cuda.synchronize()
        trace = impl.enable_trace()
        fn()
        torch.cuda.synchronize()
        impl.disable_trace()
        t = trace.cpu()
        used = t[:, 0] > 0
        t0 = int(t[used, 0].min())
        lines.append(f"## {name}: rank {comm.get_rank()} of {comm.get_size()}, {int(used.sum())} CTAs; microseconds after the first CTA started")
        lines.append(f"{'phase':28s} {'CTAs':>5s} {'min':>9s} {'median':>9s} {'max':>9s}")
        for slot, label in enumerate(PHASES):
            col = t[used, slot]
            col = col[col > 0]
            if col.numel() == 0:
                continue
            us = (col - t0).double() / 1000.0
            lines.append(f"{label:28s} {col.numel():5d} {float(us.min()):9.1f} {float(us.median()):9.1f} {float(us.max()):9.1f}")
        lines.append("")
    with open(f"{path}.rank{comm.get_rank()}", "w") as f:
        f.write("\n".join(lines))
    if comm.get_rank() == 0:
        print("\n".join(lines), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--tokens", type=int, default=8192)
    ap.add_argument("--hidden", type=int, default=8192)
    ap.add_argument("--ffn", type=int, default=28672)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--chunks", type=int, default=4)
    ap.add_argument("--no-fp8", action="store_true")
    ap.add_argument("--trace", default="", help="write the fused kernels' per-CTA phase timeline (text) to this file")
    ap.add_argument("--json", default="")
    args = ap.parse_args()

    os.environ.setdefault("RANK", "0")
    os.environ.setdefault("WORLD_SIZE", "1")
    os.environ.setdefault("LOCAL_RANK", os.environ["RANK"])
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    os.environ.setdefault("MASTER_PORT", "29573")
    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    comm = tc.new_comm("b200", dev, name="tp_perf")
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)

    def time_it(fn):
        """Median device time of one call (microseconds), maximum over ranks; the ranks start each call together."""
        for _ in range(args.warmup):
            fn()
        per = []
        for _ in range(args.iters):
            flush.zero_()
            comm.barrier(False)        # aligned start: a fused kernel would otherwise be billed for the peer's lag
            s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            s.record()
            fn()
            e.record()
            e.synchronize()
            per.append(s.elapsed_time(e) * 1000.0)
        per.sort()
        t = torch.tensor([per[len(per) // 2]], device=dev)
        comm.all_reduce(t, tc.ReduceOp.MAX, False)
        return float(t.item())

    m, hid = args.tokens, args.hidden
    m_local = m // world
    n_up = 2 * args.ffn // world        # gate and up projections of this rank
    k_down = args.ffn // world
    bf = torch.bfloat16
    x_shard = (torch.randn(m_local, hid, device=dev) * 0.5).to(bf)
    w_up = (torch.randn(n_up, hid, device=dev) * 0.02).to(bf)
    h = (torch.randn(m, k_down, device=dev) * 0.5).to(bf)
    w_down = (torch.randn(hid, k_down, device=dev) * 0.02).to(bf)
    x_full = torch.empty(m, hid, dtype=bf, device=dev)
    y_part = torch.empty(m, hid, dtype=bf, device=dev)
    out = torch.empty(m_local, hid, dtype=bf, device=dev)

    up = AllGatherGemm(comm, m_local, hid)
    down = GemmReduceScatter(comm, m, hid)
    up.input.copy_(x_shard)

    rows = []

    def report(layer, arm, us, flops):
        row = {"layer": layer, "arm": arm, "us": round(us, 1), "tflops": round(flops / us / 1e6, 1), "world": world,
               "tokens": m, "hidden": hid, "ffn": args.ffn}
        rows.append(row)
        if rank == 0:
            print(f"{layer:10s} {arm:8s} {us:10.1f} us {row['tflops']:8.1f} TFLOP/s/GPU", flush=True)

    f_up = 2.0 * m * n_up * hid
    f_down = 2.0 * m * hid * k_down
    if rank == 0:
        print(f"# world={world} tokens={m} hidden={hid} ffn={args.ffn} (per rank: up n={n_up}, down k={k_down})")

    # local GEMMs alone
    x_all = (torch.randn(m, hid, device=dev) * 0.5).to(bf)
    report("up", "cublas", time_it(lambda: torch.matmul(x_all, w_up.t())), f_up)
    report("up", "tcgen05", time_it(lambda: _comms.ops.gemm_bf16_nt(x_all, w_up)), f_up)
    report("up", "tcgen05x2", time_it(lambda: _comms.ops.gemm_bf16_nt_pair(x_all, w_up)), f_up)
    report("down", "cublas", time_it(lambda: torch.matmul(h, w_down.t())), f_down)
    report("down", "tcgen05", time_it(lambda: _comms.ops.gemm_bf16_nt(h, w_down)), f_down)
    report("down", "tcgen05x2", time_it(lambda: _comms.ops.gemm_bf16_nt_pair(h, w_down)), f_down)

    report("up", "fused", time_it(lambda: up(w_up)), f_up)
    report("down", "fused", time_it(lambda: down(h, w_down)), f_down)
    if args.trace:
        phase_timeline(comm, dev, args.trace, {"up (all-gather -> GEMM)": lambda: up(w_up),
                                               "down (GEMM -> reduce-scatter)": lambda: down(h, w_down)})
    if world > 1:
        for arm, algo in (("unfused", "auto"), ("nccl", "nccl")):
            hint = {"algo": algo}

            def up_unfused():
                comm.all_gather_single(x_full, x_shard, False, hints=hint)
                return torch.matmul(x_full, w_up.t())

            def down_unfused():
                torch.matmul(h, w_down.t(), out=y_part)
                comm.reduce_scatter_single(out, y_part, tc.ReduceOp.SUM, False, hints=hint)

            report("up", arm, time_it(up_unfused), f_up)
            report("down", arm, time_it(down_unfused), f_down)
        # NCCL and cuBLAS overlapped by hand, piece by piece
        nccl = {"algo": "nccl"}
        C = args.chunks
        if m_local % C == 0 and (m // C) % world == 0:
            piece = m_local // C
            x_pieces = [torch.empty(world * piece, hid, dtype=bf, device=dev) for _ in range(C)]
            y_pieces = [torch.empty(world * piece, n_up, dtype=bf, device=dev) for _ in range(C)]

            def up_overlapped():
                works = [comm.all_gather_single(x_pieces[c], x_shard[c * piece:(c + 1) * piece], True, hints=nccl)
                         for c in range(C)]
                for c in range(C):
                    works[c].wait()                      # the current stream waits for piece c only
                    torch.matmul(x_pieces[c], w_up.t(), out=y_pieces[c])

            rows_c = m // C
            part_pieces = [torch.empty(rows_c, hid, dtype=bf, device=dev) for _ in range(C)]
            out_pieces = [torch.empty(rows_c // world, hid, dtype=bf, device=dev) for _ in range(C)]

            def down_overlapped():
                works = []
                for c in range(C):
                    torch.matmul(h[c * rows_c:(c + 1) * rows_c], w_down.t(), out=part_pieces[c])
                    works.append(comm.reduce_scatter_single(out_pieces[c], part_pieces[c], tc.ReduceOp.SUM, True, hints=nccl))
                for w in works:
                    w.wait()

            report("up", "nccl-ovl", time_it(up_overlapped), f_up)
            report("down", "nccl-ovl", time_it(down_overlapped), f_down)

    if not args.no_fp8:
        qx_all, sx_all = quantize_rows(x_all)
        qw_up, sw_up = quantize_rows(w_up)
        qh, sh = quantize_rows(h)
        qw_down, sw_down = quantize_rows(w_down)
        try:
            report("up", "cublas-fp8", time_it(lambda: torch._scaled_mm(
                qx_all, qw_up.t(), scale_a=sx_all.unsqueeze(1), scale_b=sw_up.unsqueeze(0), out_dtype=bf)), f_up)
            report("down", "cublas-fp8", time_it(lambda: torch._scaled_mm(
                qh, qw_down.t(), scale_a=sh.unsqueeze(1), scale_b=sw_down.unsqueeze(0), out_dtype=bf)), f_down)
        except Exception as e:  # noqa: BLE001
            if rank == 0:
                print(f"# cublas-fp8 arm skipped: {type(e).__name__}: {str(e)[:120]}")
        report("up", "tcgen05-fp8", time_it(lambda: gemm_e4m3_nt(qx_all, qw_up, sx_all, sw_up)), f_up)
        report("down", "tcgen05-fp8", time_it(lambda: gemm_e4m3_nt(qh, qw_down, sh, sw_down)), f_down)
        up8 = AllGatherGemm(comm, m_local, hid, fp8=True)
        down8 = GemmReduceScatter(comm, m, hid, fp8=True)
        qx_shard, sx_shard = quantize_rows(x_shard)
        up8.input.copy_(qx_shard)
        up8.input_scales.copy_(sx_shard)
        report("up", "fused-fp8", time_it(lambda: up8(qw_up, scale_w=sw_up)), f_up)
        report("down", "fused-fp8", time_it(lambda: down8(qh, qw_down, sh, sw_down)), f_down)
        torch.cuda.synchronize()
        del up8, down8
    torch.cuda.synchronize()
    st = up.status()
    del up, down
    comm.finalize()
    if rank == 0:
        if args.json:
            with open(args.json, "w") as f:
                json.dump(rows, f)
        print("status", st)


if __name__ == "__main__":
    main()
