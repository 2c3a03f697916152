"""MoE expert-parallel dispatch / combine latency.

    torchrun --nproc-per-node 8 benchmarks/moe_ep_perf.py \
        [--tokens 4096] [--hidden 7168] [--experts 256] [--topk 8] [--ll-tokens 128] [--warmup 10] [--iters 50]

Router logits ~N(0,1), softmax, top-k; x ~N(0,1) bf16.  Phases and arms
(``torchcomms_b200.utils.perf.moe_ep_latency`` does the work; ``bench.py`` reports the same rows):

  * ``dispatch`` / ``combine``, arm ``fused`` - ops.moe_ep.Buffer: one kernel does routing counts,
    block-scaled fp8 (e4m3, 1x128) quantisation, token permutation and the peer stores; combine
    pulls the expert outputs and applies the weighted sum.
  * the same phases, arm ``nccl`` - the unfused pipeline the reference's users run: per-destination
    token gather, fp8 quantisation in PyTorch, split exchange, ``all_to_all_v_single`` of payload
    and scales through NCCL; combine: ``all_to_all_v_single`` back in bf16 + index_add.
  * ``ll_dispatch`` / ``ll_combine`` - ops.moe_ep.LowLatencyBuffer on ``--ll-tokens`` tokens per rank
    (decode batch): one row per (token, expert) pair into fixed slots, counts as arrival flags.

Device-timed per call (CUDA events, L2 flushed between calls), maximum over ranks; the reported
bandwidth counts the payload bytes a rank receives (dispatch) or sends back (combine).
"""
from __future__ import annotations

import argparse
import json
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import torch  # noqa: E402

import torchcomms_b200 as tc  # noqa: E402
from torchcomms_b200.utils.perf import moe_ep_latency  # noqa: E402


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--tokens", type=int, default=4096)
    ap.add_argument("--hidden", type=int, default=7168)
    ap.add_argument("--experts", type=int, default=256)
    ap.add_argument("--topk", type=int, default=8)
    ap.add_argument("--ll-tokens", type=int, default=128)
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--iters", type=int, default=50)
    ap.add_argument("--no-nccl", action="store_true")
    ap.add_argument("--json", default="")
    args = ap.parse_args()

    os.environ.setdefault("RANK", "0")
    os.environ.setdefault("WORLD_SIZE", "1")
    os.environ.setdefault("LOCAL_RANK", os.environ["RANK"])
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    os.environ.setdefault("MASTER_PORT", "29575")
    rank, local = int(os.environ["RANK"]), int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    comm = tc.new_comm("b200", dev, name="ep_perf")
    rows = moe_ep_latency(comm, dev, tokens=args.tokens, hidden=args.hidden, experts=args.experts, topk=args.topk,
                          warmup=args.warmup, iters=args.iters, with_nccl=not args.no_nccl, ll_tokens=args.ll_tokens)
    if rank == 0:
        print(f"# world={comm.get_size()} hidden={args.hidden} experts={args.experts} topk={args.topk}")
        for r in rows:
            print(f"{r['phase']:12s} {r['arm']:6s} tokens {r['tokens']:6d}  avg {r['avg_us']:9.1f} us  p50 {r['p50_us']:9.1f} us  "
                  f"{r['gbs']:7.1f} GB/s", flush=True)
        if args.json:
            with open(args.json, "w") as f:
                json.dump(rows, f)
    comm.finalize()


if __name__ == "__main__":
    main()
