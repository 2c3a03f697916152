"""Tensor-parallel MLP layers: fused kernels versus GEMM + collective.

    python benchmarks/tp_layer_perf.py                       # 1 GPU: GEMM kernels only
    torchrun --nproc-per-node N benchmarks/tp_layer_perf.py  # fused layers on N ranks

Default shape: the MLP of Llama-3-70B (hidden 8192, ffn 28672) on ``tokens``
rows, sharded over the N ranks.  Timed per call on the device with CUDA
events, an L2-sized scratch write between calls, maximum over ranks.

Arms:
  * ``fused``   - ops.tp.AllGatherGemm / GemmReduceScatter (one kernel each)
  * ``unfused`` - this framework's all-gather / reduce-scatter collective
                  followed / preceded by ``torch.matmul`` (cuBLAS)
  * ``nccl``    - the same with the collective routed through NCCL
  * ``cublas`` / ``tcgen05`` / ``tcgen05x2`` - the local GEMM alone (cuBLAS, this framework's
                  kernel with one CTA per tile, and on CTA pairs): the lower bound of any arm
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
from torchcomms_b200.ops.tp import AllGatherGemm, GemmReduceScatter  # noqa: E402


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--tokens", type=int, default=8192)
    ap.add_argument("--hidden", type=int, default=8192)
    ap.add_argument("--ffn", type=int, default=28672)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--iters", type=int, default=20)
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
        for _ in range(args.warmup):
            fn()
        comm.barrier(False)
        torch.cuda.synchronize()
        total = 0.0
        for _ in range(args.iters):
            flush.zero_()
            s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            s.record()
            fn()
            e.record()
            e.synchronize()
            total += s.elapsed_time(e)
        t = torch.tensor([total * 1000.0 / args.iters], device=dev)
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
