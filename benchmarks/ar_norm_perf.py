"""All-reduce + residual add + RMSNorm latency for tensor-parallel decode batches.

    torchrun --nproc-per-node 8 benchmarks/ar_norm_perf.py [--hidden 8192] [--rows 1,8,32,128] [--iters 200]

For each token count the row-parallel partial ``[rows, hidden]`` bf16 is reduced
over the ranks, added to the residual stream and normalised.  Arms:

  * ``fused``   - ``ops.ar_norm.AllReduceRMSNorm``: one kernel, one cross-GPU barrier;
  * ``kernels`` - this framework's one-shot all-reduce kernel, then the residual
                  add and the stand-alone RMSNorm kernel (three launches);
  * ``nccl``    - the same three steps with the all-reduce routed to NCCL
                  (what a user of the reference runs: ``all_reduce`` + PyTorch ops).

Device-timed per call with CUDA events on the launching stream, L2 flushed
between calls, maximum over ranks.
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
from torchcomms_b200.ops.ar_norm import AllReduceRMSNorm  # noqa: E402


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--hidden", type=int, default=8192)
    ap.add_argument("--rows", default="1,8,32,128")
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--iters", type=int, default=100)
    ap.add_argument("--json", default="")
    args = ap.parse_args()

    os.environ.setdefault("RANK", "0")
    os.environ.setdefault("WORLD_SIZE", "1")
    os.environ.setdefault("LOCAL_RANK", os.environ["RANK"])
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    os.environ.setdefault("MASTER_PORT", "29577")
    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    comm = tc.new_comm("b200", dev, name="ar_norm_perf")
    hidden = args.hidden
    fused = AllReduceRMSNorm(comm, hidden)
    weight = (1.0 + 0.1 * torch.randn(hidden, device=dev)).to(torch.bfloat16)
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

    out_rows = []
    for rows in [int(r) for r in args.rows.split(",")]:
        x = torch.randn(rows, hidden, device=dev).to(torch.bfloat16)
        res = torch.randn(rows, hidden, device=dev).to(torch.bfloat16)
        scratch = torch.empty_like(x)

        def three_step(algo):
            scratch.copy_(x)
            comm.all_reduce(scratch, tc.ReduceOp.SUM, False, hints={"algo": algo})
            res.add_(scratch)
            return _comms.ops.rmsnorm_fwd(res, weight, 1e-5)[0]

        timings = {
            "fused": time_it(lambda: fused(x, weight, residual=res)),
            "kernels": time_it(lambda: three_step("kernel")),
            "nccl": time_it(lambda: three_step("nccl")),
        }
        for arm, us in timings.items():
            out_rows.append({"rows": rows, "hidden": hidden, "world": world, "arm": arm, "us": round(us, 2)})
        if rank == 0:
            print(f"rows {rows:4d} hidden {hidden}: fused {timings['fused']:.1f} us, kernels {timings['kernels']:.1f} us, "
                  f"nccl {timings['nccl']:.1f} us", flush=True)
    if rank == 0 and args.json:
        with open(args.json, "w") as f:
            json.dump(out_rows, f, indent=1)
    comm.finalize()


if __name__ == "__main__":
    main()
