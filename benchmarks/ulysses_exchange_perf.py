"""Sequence <-> heads exchange of Ulysses attention: fused layout-changing kernel versus all-to-all with permutes.

    torchrun --nproc-per-node N --master-addr 127.0.0.1 benchmarks/ulysses_exchange_perf.py

Default shape: 32 heads of 128, 8192 positions per rank, bf16 (the q / k / v of one Llama-3-8B layer on a
sequence of N * 8192).  Timed per call on the device with CUDA events (median of the calls), an L2-sized
scratch write and a barrier before each call, maximum over ranks.

Arms (both directions):
  * ``fused``        - parallel.context.SeqHeadsExchange: one kernel, every [s, d] slab goes from the caller's
                       tensor to its place in the peer's tensor
  * ``own a2a``      - permute + contiguous, this framework's all_to_all_single into a symmetric buffer, permute +
                       contiguous (what ulysses_attention does without an exchange object)
  * ``nccl a2a``     - the same with the all-to-all routed through NCCL
"""
from __future__ import annotations

import argparse
import json
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import torch  # noqa: E402

import torchcomms_b200 as tc  # noqa: E402
from torchcomms_b200.parallel.context import SeqHeadsExchange  # noqa: E402


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--batch", type=int, default=1)
    ap.add_argument("--heads", type=int, default=32)
    ap.add_argument("--seq", type=int, default=8192, help="positions per rank")
    ap.add_argument("--dim", type=int, default=128)
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--json", default="")
    args = ap.parse_args()

    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", str(rank)))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    comm = tc.new_comm("b200", dev, name="ulysses_perf", abort_process_on_timeout_or_error=False)
    n = comm.get_size()
    b, h, s, d = args.batch, args.heads, args.seq, args.dim
    x = torch.randn(b, h, s, d, device=dev).to(torch.bfloat16)
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)

    def time_it(fn):
        for _ in range(args.warmup):
            fn()
        per = []
        for _ in range(args.iters):
            flush.zero_()
            comm.barrier(False)
            st, en = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            st.record()
            fn()
            en.record()
            en.synchronize()
            per.append(st.elapsed_time(en) * 1000.0)
        per.sort()
        t = torch.tensor([per[len(per) // 2]], device=dev)
        comm.all_reduce(t, tc.ReduceOp.MAX, False)
        return float(t.item())

    ex = SeqHeadsExchange(comm)
    recv = comm.symm_empty((n, b, h // n, s, d), torch.bfloat16) if n > 1 else torch.empty(n, b, h // n, s, d, dtype=torch.bfloat16, device=dev)

    def a2a_to_heads(t, hints):
        send = t.reshape(b, n, h // n, s, d).permute(1, 0, 2, 3, 4).contiguous()
        comm.all_to_all_single(recv, send, False, hints=hints)
        return recv.permute(1, 2, 0, 3, 4).reshape(b, h // n, n * s, d)      # the reshape copies

    def a2a_to_seq(t, hints):
        send = t.reshape(b, h // n, n, s, d).permute(2, 0, 1, 3, 4).contiguous()
        comm.all_to_all_single(recv, send, False, hints=hints)
        return recv.permute(1, 0, 2, 3, 4).reshape(b, h, s, d)

    heads = ex.to_heads(x, keep=True)
    assert torch.equal(heads, a2a_to_heads(x, None)) and torch.equal(ex.to_seq(heads), x)
    rows = []
    moved = x.nbytes * (n - 1) / n      # bytes that cross NVLink per rank and direction
    for name, fn in (("to_heads fused", lambda: ex.to_heads(x)), ("to_heads own a2a", lambda: a2a_to_heads(x, None)),
                     ("to_heads nccl a2a", lambda: a2a_to_heads(x, {"algo": "nccl"})),
                     ("to_seq fused", lambda: ex.to_seq(heads)), ("to_seq own a2a", lambda: a2a_to_seq(heads, None)),
                     ("to_seq nccl a2a", lambda: a2a_to_seq(heads, {"algo": "nccl"}))):
        if n == 1 and "nccl" in name:
            continue
        us = time_it(fn)
        rows.append({"arm": name, "us": round(us, 1), "nvlink_gbs": round(moved / us / 1e3, 1), "world": n,
                     "shape": [b, h, s, d], "bytes": x.nbytes})
        if rank == 0:
            print(f"{name:20s} {us:9.1f} us   {moved / us / 1e3:7.1f} GB/s over NVLink per rank", flush=True)
    if rank == 0 and args.json:
        with open(args.json, "w") as f:
            json.dump(rows, f, indent=1)
    torch.cuda.synchronize()
    ex.close()
    comm.finalize()


if __name__ == "__main__":
    main()
