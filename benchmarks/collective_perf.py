"""Collective sweep: bus bandwidth and latency versus message size.

    torchrun --nproc-per-node N benchmarks/collective_perf.py \
        [--ops all_reduce,all_gather,reduce_scatter,all_to_all] [--dtypes bf16,fp32] \
        [--min-bytes 1024] [--max-bytes 1073741824] [--algos auto,nccl] [--warmup 20] [--iters 100]

Protocol: per (op, dtype, size, algorithm) ``warmup`` untimed and ``iters`` timed
back-to-back calls on buffers ~U[-1, 1], timed on the device with CUDA events
bracketed by a barrier and a synchronize, maximum over ranks.  ``algo=kernel`` is
this framework's peer-memory kernel family (one-shot / two-shot / NVLS picked by
size), ``algo=nccl`` routes the same call through NCCL (the reference backend's
data path) and ``algo=auto`` is the default routing between the two by measured
cross-over sizes.  Bus bandwidth uses the
usual factors: 2(n-1)/n for all-reduce, (n-1)/n for the others.

Parity: comms/torchcomms/tests/perf/py/collective_perf_test.py and
perf_test_helpers.py:22-36 (host-timed there).
"""
from __future__ import annotations

import argparse
import json
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import torch  # noqa: E402

import torchcomms_b200 as tc  # noqa: E402

DTYPES = {"bf16": torch.bfloat16, "fp32": torch.float32, "fp16": torch.float16}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--ops", default="all_reduce,all_gather,reduce_scatter")
    ap.add_argument("--dtypes", default="bf16")
    ap.add_argument("--algos", default="auto,kernel,nccl")
    ap.add_argument("--min-bytes", type=int, default=1024)
    ap.add_argument("--max-bytes", type=int, default=1 << 30)
    ap.add_argument("--warmup", type=int, default=20)
    ap.add_argument("--iters", type=int, default=100)
    ap.add_argument("--json", default="")
    ap.add_argument("--hints", default="", help="k=v,k=v passed to new_comm")
    args = ap.parse_args()

    os.environ.setdefault("RANK", "0")
    os.environ.setdefault("WORLD_SIZE", "1")
    os.environ.setdefault("LOCAL_RANK", os.environ["RANK"])
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    os.environ.setdefault("MASTER_PORT", "29571")
    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    hints = dict(kv.split("=") for kv in args.hints.split(",") if kv)
    comm = tc.new_comm("b200", dev, name="perf", hints=hints)
    results = []
    sizes = []
    b = args.min_bytes
    while b <= args.max_bytes:
        sizes.append(b)
        b *= 2

    def time_it(fn, iters):
        for _ in range(args.warmup):
            fn()
        comm.barrier(False)
        torch.cuda.synchronize()
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record()
        for _ in range(iters):
            fn()
        e.record()
        torch.cuda.synchronize()
        t = torch.tensor([s.elapsed_time(e) * 1000.0 / iters], device=dev)
        comm.all_reduce(t, tc.ReduceOp.MAX, False)
        return float(t.item())

    if rank == 0:
        print(f"# world={world} multicast={comm.get_backend_impl().has_multicast()}")
        print(f"{'op':16s} {'dtype':5s} {'bytes':>11s} {'algo':6s} {'us':>10s} {'algbw GB/s':>11s} {'busbw GB/s':>11s}")
    for op in args.ops.split(","):
        for dname in args.dtypes.split(","):
            dt = DTYPES[dname]
            esz = torch.empty(0, dtype=dt).element_size()
            for nbytes in sizes:
                n = max(world, nbytes // esz // world * world)
                for algo in args.algos.split(","):
                    if algo == "nccl" and world == 1:
                        continue
                    h = {"algo": algo}
                    if op == "all_reduce":
                        buf = (torch.rand(n, device=dev) * 2 - 1).to(dt)
                        fn = lambda: comm.all_reduce(buf, tc.ReduceOp.SUM, False, hints=h)
                        factor = 2 * (world - 1) / world
                    elif op == "all_gather":
                        src = (torch.rand(n // world, device=dev) * 2 - 1).to(dt)
                        dst = torch.empty(n, dtype=dt, device=dev)
                        fn = lambda: comm.all_gather_single(dst, src, False, hints=h)
                        factor = (world - 1) / world
                    elif op == "reduce_scatter":
                        src = (torch.rand(n, device=dev) * 2 - 1).to(dt)
                        dst = torch.empty(n // world, dtype=dt, device=dev)
                        fn = lambda: comm.reduce_scatter_single(dst, src, tc.ReduceOp.SUM, False, hints=h)
                        factor = (world - 1) / world
                    elif op == "all_to_all":
                        src = (torch.rand(n, device=dev) * 2 - 1).to(dt)
                        dst = torch.empty(n, dtype=dt, device=dev)
                        fn = lambda: comm.all_to_all_single(dst, src, False, hints=h)
                        factor = (world - 1) / world
                    else:
                        raise SystemExit(f"unknown op {op}")
                    iters = args.iters if nbytes <= (64 << 20) else max(10, args.iters // 5)
                    us = time_it(fn, iters)
                    total = n * esz
                    algbw = total / us / 1e3
                    row = {"op": op, "dtype": dname, "bytes": total, "algo": algo, "us": round(us, 2),
                           "algbw_gbs": round(algbw, 2), "busbw_gbs": round(algbw * factor, 2), "world": world}
                    results.append(row)
                    if rank == 0:
                        print(f"{op:16s} {dname:5s} {total:11d} {algo:6s} {us:10.2f} {algbw:11.2f} {algbw * factor:11.2f}", flush=True)
    torch.cuda.synchronize()
    comm.finalize()
    if rank == 0 and args.json:
        with open(args.json, "w") as f:
            json.dump(results, f)


if __name__ == "__main__":
    main()
