"""Headline benchmark: one Llama-3-8B sharded-data-parallel training step.

    python bench.py --gpus N --steps K --warmup W        (N > 1: launched with torchrun, one rank per GPU)

Config (from the benchmark set): Llama-3-8B architecture (32 layers, hidden
4096, 32 heads / 8 KV heads, FFN 14336, vocab 128256, RMSNorm, RoPE), random
init, sequence 4096, micro-batch 1 per GPU, token ids uniform over the
vocabulary; parameters all-gathered before each stage's forward and backward
and gradients reduce-scattered behind backward through this framework's
communicator; bf16 compute, fp32 master weights and AdamW state.

Prints ONE JSON line on rank 0.  ``value`` is whole-job tokens/s timed on the
device with CUDA events (max over ranks) over exactly K steps after W warm-up
steps; ``e2e`` repeats the measurement with the per-step host->device copy of
the token ids from pinned memory and a device->host read of the loss inside
the timed region.  With N > 1 the line also carries bus bandwidth of this
framework's all_reduce / all_gather / reduce_scatter kernels next to NCCL's.

``--impl reference`` would run the unmodified reference package from
``baseline/_ref``; it cannot be installed offline here (its CMake build
downloads third-party sources), so that arm reports itself unavailable.
"""
from __future__ import annotations

import argparse
import json
import os
import sys
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)


def parse_args():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--model", default="llama3_8b", choices=["llama3_8b", "llama_1b", "tiny"])
    ap.add_argument("--seq-len", type=int, default=4096)
    ap.add_argument("--micro-batch", type=int, default=1)
    ap.add_argument("--recompute-blocks", type=int, default=0)
    ap.add_argument("--skip-collectives", action="store_true")
    return ap.parse_args()


def reference_arm():
    print(json.dumps({
        "impl": "reference",
        "unavailable": "torchcomms cannot be installed offline: its CMake build fetches nlohmann_json and gloo "
                       "from GitHub (FetchContent) and no network is available",
    }))


def model_config(name):
    from torchcomms_b200.models.llama import LlamaConfig

    if name == "llama3_8b":
        return LlamaConfig.llama3_8b()
    if name == "llama_1b":
        return LlamaConfig(dim=2048, n_layers=16, n_heads=32, n_kv_heads=8, ffn_dim=8192, vocab_size=128256)
    return LlamaConfig.tiny()


def max_over_ranks(comm, value, device):
    import torch

    import torchcomms_b200 as tc

    t = torch.tensor([value], dtype=torch.float32, device=device)
    comm.all_reduce(t, tc.ReduceOp.MAX, False)
    return float(t.item())


def bench_collectives(comm, device, world):
    """Bus bandwidth (GB/s) of AR / AG / RS: this framework's kernels and NCCL, bf16."""
    import torch

    import torchcomms_b200 as tc

    out = {}
    sizes = [64 * 1024, 1 << 20, 16 << 20, 256 << 20]
    for algo in ("auto", "kernel", "nccl"):
        for op in ("all_reduce", "all_gather", "reduce_scatter"):
            for nbytes in sizes:
                n = nbytes // 2
                hints = {"algo": algo}
                if op == "all_reduce":
                    buf = torch.zeros(n, dtype=torch.bfloat16, device=device)
                    fn = lambda: comm.all_reduce(buf, tc.ReduceOp.SUM, False, hints=hints)
                    factor = 2 * (world - 1) / world
                elif op == "all_gather":
                    src = torch.zeros(n // world, dtype=torch.bfloat16, device=device)
                    dst = torch.empty(n // world * world, dtype=torch.bfloat16, device=device)
                    fn = lambda: comm.all_gather_single(dst, src, False, hints=hints)
                    factor = (world - 1) / world
                else:
                    src = torch.zeros(n // world * world, dtype=torch.bfloat16, device=device)
                    dst = torch.empty(n // world, dtype=torch.bfloat16, device=device)
                    fn = lambda: comm.reduce_scatter_single(dst, src, tc.ReduceOp.SUM, False, hints=hints)
                    factor = (world - 1) / world
                iters = 20 if nbytes >= (16 << 20) else 50
                for _ in range(5):
                    fn()
                comm.barrier(False)
                torch.cuda.synchronize()
                start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                start.record()
                for _ in range(iters):
                    fn()
                end.record()
                torch.cuda.synchronize()
                us = max_over_ranks(comm, start.elapsed_time(end) * 1000.0 / iters, device)
                out[f"{op}/{algo}/{nbytes}"] = {"us": round(us, 2), "busbw_gbs": round(nbytes * factor / us / 1e3, 1)}
    return out


def main():
    args = parse_args()
    if args.impl == "reference":
        reference_arm()
        return
    os.environ.setdefault("RANK", "0")
    os.environ.setdefault("LOCAL_RANK", os.environ["RANK"])
    os.environ.setdefault("WORLD_SIZE", "1")
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    os.environ.setdefault("MASTER_PORT", "29555")
    import torch

    import torchcomms_b200 as tc
    from torchcomms_b200.ops import fused
    from torchcomms_b200.parallel.engine import TrainEngine
    from torchcomms_b200.utils.clocks import ClockSampler

    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    local = int(os.environ["LOCAL_RANK"])
    assert world == args.gpus, f"--gpus {args.gpus} but WORLD_SIZE={world} (launch with torchrun for N > 1)"
    torch.cuda.set_device(local)
    device = torch.device("cuda", local)
    comm = tc.new_comm("b200", device, name="bench")
    cfg = model_config(args.model)
    cfg.max_seq_len = max(cfg.max_seq_len, args.seq_len)
    engine = TrainEngine(cfg, comm, lr=3e-4, seed=0, recompute_blocks=args.recompute_blocks)
    mb, seq = args.micro_batch, args.seq_len
    tokens_per_step = world * mb * seq
    total_steps = args.warmup + 2 * args.steps

    g = torch.Generator().manual_seed(1234 + rank)
    host_tokens = torch.randint(0, cfg.vocab_size, (total_steps, mb, seq + 1), generator=g).pin_memory()
    dev_tokens = host_tokens.to(device)
    h2d_bytes = mb * (seq + 1) * host_tokens.element_size()

    def device_step(i):
        t = dev_tokens[i]
        return engine.step(t[:, :-1].contiguous(), t[:, 1:].contiguous())

    def e2e_step(i):
        t = host_tokens[i].to(device, non_blocking=True)
        loss = engine.step(t[:, :-1].contiguous(), t[:, 1:].contiguous())
        return float(loss.item())  # device -> host read of the step's result

    for i in range(args.warmup):
        device_step(i)

    def timed(fn, first):
        comm.barrier(False)
        torch.cuda.synchronize()
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        launches0 = fused.kernel_launch_count()
        with ClockSampler(local) as clocks:
            start.record()
            last = None
            for i in range(first, first + args.steps):
                last = fn(i)
            end.record()
            comm.barrier(False)
            torch.cuda.synchronize()
        ms = max_over_ranks(comm, start.elapsed_time(end), device)
        return ms, fused.kernel_launch_count() - launches0, clocks.summary(), last

    ms, launches, clocks, last_loss = timed(device_step, args.warmup)
    ms_e2e, _, _, last_e2e = timed(e2e_step, args.warmup + args.steps)
    peak_gb = torch.cuda.max_memory_allocated() / 2**30

    collectives = None
    if world > 1 and not args.skip_collectives:
        collectives = bench_collectives(comm, device, world)

    value = tokens_per_step * args.steps / (ms / 1000.0)
    e2e_value = tokens_per_step * args.steps / (ms_e2e / 1000.0)
    flops = cfg.flops_per_token(seq) * value
    line = {
        "metric": "llama3_8b_fsdp_train_tokens_per_s",
        "value": round(value, 1),
        "unit": "tokens/s",
        "n_gpus": world,
        "steps": args.steps,
        "warmup": args.warmup,
        "ms_per_step": round(ms / args.steps, 3),
        "higher_is_better": True,
        "scaling": "weak",
        "vs_baseline": None,
        "dtype": "bf16",
        "data": "synthetic (token ids uniform over the vocabulary, random-init weights)",
        "config": {
            "model": {"llama3_8b": "Llama-3-8B", "llama_1b": "Llama-1B (reduced, not the headline config)",
                      "tiny": "tiny (smoke only)"}[args.model],
            "global_batch": world * mb,
            "seq_len": seq,
            "parallelism": f"fsdp{world}",
            "params": cfg.param_count(),
            "optimizer": "AdamW, fp32 master weights and moments",
            "recompute_blocks": args.recompute_blocks,
            "l2": "every step streams >100 GB of parameters, activations and optimizer state: inputs are larger than L2",
        },
        "e2e": {
            "value": round(e2e_value, 1),
            "unit": "tokens/s",
            "ms_per_step": round(ms_e2e / args.steps, 3),
            "h2d_bytes_per_step": h2d_bytes,
            "d2h_bytes_per_step": 4,
        },
        "gpu_launches": int(launches),
        "clocks": {k: clocks[k] for k in ("sm_mhz", "sm_max_mhz", "reasons")},
        "model_tflops_per_gpu": round(flops / world / 1e12, 1),
        "peak_mem_gb": round(peak_gb, 1),
        "final_loss": round(float(last_loss), 4),
        "impl": "ours",
    }
    if collectives is not None:
        line["collectives_bf16"] = collectives
    torch.cuda.synchronize()
    comm.finalize()
    if rank == 0:
        print(json.dumps(line))


if __name__ == "__main__":
    main()
