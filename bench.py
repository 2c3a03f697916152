"""Headline benchmark.

    python bench.py --gpus N --steps K --warmup W        (N > 1: launched with torchrun, one rank per GPU)

What it measures, on synthetic data of the named shapes with random-init weights:

1. **Training step** (``value``): one Llama-3-8B sharded-data-parallel step
   (32 layers, hidden 4096, 32 heads / 8 KV heads, FFN 14336, vocab 128256,
   RMSNorm, RoPE; sequence 4096, micro-batch 1 per GPU; token ids uniform over
   the vocabulary; bf16 compute, fp32 master weights and AdamW state).
   Parameters are all-gathered before each stage's forward and backward and
   gradients reduce-scattered behind backward through this framework's
   communicator.  Whole-job tokens/s over exactly K steps after W warm-up
   steps, timed on the device with CUDA events, max over ranks.  ``e2e``
   repeats it with the per-step host->device copy of the token ids from pinned
   memory and a device->host read of the loss inside the timed region.
   With N > 1 the same engine is timed a second time with its parameter gathers
   and gradient reductions on NCCL (``step_nccl_arm``: separate cast kernels +
   ``ncclAllGather`` / ``ncclReduceScatter`` in bf16, the path the reference's
   ``nccl`` backend takes), and a profiled pass reports how long the
   communication kernels run, how long compute sits blocked on them, and the
   optimizer time (``step_breakdown``).
2. **Collective sweep** (``collectives``; N > 1): bus bandwidth, average and p50
   latency of all_reduce / all_gather / reduce_scatter / all_to_all_v on bf16 and
   fp32 buffers ~U[-1,1], 1 KB - 1 GB in powers of two, 20 warm-up + 100 timed
   calls per point: this framework's kernels next to NCCL.
3. **MoE dispatch / combine latency** (``moe_ep``; N > 1): 4096 tokens per rank,
   hidden 7168, 256 experts, top-8, fp8 (e4m3, 1x128 scales) dispatch and bf16
   weighted combine: the fused kernels next to the unfused NCCL pipeline.

Rank 0 prints ONE JSON line.  ``--impl reference`` would run the unmodified
reference package from ``baseline/_ref``; it cannot be built offline here (see
the message it prints), so that arm reports itself unavailable.
"""
from __future__ import annotations

import argparse
import gc
import json
import os
import sys

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
    ap.add_argument("--comm", default="symm", choices=["symm", "staged", "nccl"],
                    help="how the step's all-gathers / reduce-scatters move data (the headline arm)")
    ap.add_argument("--skip-nccl-arm", action="store_true", help="do not time the step a second time on NCCL")
    ap.add_argument("--skip-collectives", action="store_true")
    ap.add_argument("--skip-ep", action="store_true")
    ap.add_argument("--sweep-max-bytes", type=int, default=1 << 30)
    ap.add_argument("--sweep-iters", type=int, default=100)
    ap.add_argument("--sweep-warmup", type=int, default=20)
    ap.add_argument("--sweep-json", default="", help="also write every sweep row to this file")
    return ap.parse_args()


def reference_arm():
    if int(os.environ.get("RANK", "0")) != 0:     # under torchrun every rank gets here: one line, from rank 0
        return
    print(json.dumps({
        "impl": "reference",
        "unavailable": "torchcomms cannot be built offline: its CMake configure step needs nlohmann_json, gflags, glog "
                       "and gloo as CMake packages (FetchContent downloads them otherwise) and none of them is in the "
                       "image; no network is available",
    }))


def model_config(name):
    from torchcomms_b200.models.llama import LlamaConfig

    if name == "llama3_8b":
        return LlamaConfig.llama3_8b()
    if name == "llama_1b":
        return LlamaConfig(dim=2048, n_layers=16, n_heads=32, n_kv_heads=8, ffn_dim=8192, vocab_size=128256)
    return LlamaConfig.tiny()


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
    from torchcomms_b200.utils import perf
    from torchcomms_b200.utils.clocks import ClockSampler

    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    local = int(os.environ["LOCAL_RANK"])
    assert world == args.gpus, f"--gpus {args.gpus} but WORLD_SIZE={world} (launch with torchrun for N > 1)"
    torch.cuda.set_device(local)
    device = torch.device("cuda", local)
    # Communication kernels get a high-priority stream: their (few) blocks are placed as soon as an SM
    # has room instead of queueing behind the GEMMs' waves.
    comm = tc.new_comm("b200", device, name="bench",
                       is_high_priority_stream=os.environ.get("B200COMMS_BENCH_HIGH_PRIORITY", "1") != "0")
    cfg = model_config(args.model)
    cfg.max_seq_len = max(cfg.max_seq_len, args.seq_len)
    mb, seq = args.micro_batch, args.seq_len
    tokens_per_step = world * mb * seq
    total_steps = args.warmup + 2 * args.steps + 3

    g = torch.Generator().manual_seed(1234 + rank)
    host_tokens = torch.randint(0, cfg.vocab_size, (total_steps, mb, seq + 1), generator=g).pin_memory()
    dev_tokens = host_tokens.to(device)
    h2d_bytes = mb * (seq + 1) * host_tokens.element_size()

    def log(msg):
        if rank == 0:
            print(msg, file=sys.stderr, flush=True)

    def run_arm(comm_mode, with_e2e, with_breakdown):
        """Builds the engine, warms it up, times K steps (and K more end to end), tears it down."""
        engine = TrainEngine(cfg, comm, lr=3e-4, seed=0, recompute_blocks=args.recompute_blocks, comm_mode=comm_mode)

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
            (ms,) = perf.max_over_ranks(comm, [start.elapsed_time(end)], device)
            return ms, fused.kernel_launch_count() - launches0, clocks.summary(), last

        out = {}
        ms, launches, clocks, last_loss = timed(device_step, args.warmup)
        out.update(ms=ms, launches=launches, clocks=clocks, loss=float(last_loss))
        if with_e2e:
            ms_e2e, _, clocks_e2e, _ = timed(e2e_step, args.warmup + args.steps)
            out.update(ms_e2e=ms_e2e, clocks_e2e=clocks_e2e)
        if with_breakdown:
            n_prof = 3
            tl = engine.attach_timeline()
            comm.barrier(False)
            torch.cuda.synchronize()
            s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            s.record()
            for i in range(n_prof):
                device_step(args.warmup + 2 * args.steps + i)
            e.record()
            torch.cuda.synchronize()
            tot = tl.totals_ms()
            engine.detach_timeline()
            vals = perf.max_over_ranks(comm, [s.elapsed_time(e)] + [tot[k] for k in ("ag", "rs", "wait", "opt")], device)
            out["breakdown"] = {
                "profiled_steps": n_prof,
                "ms_per_step": round(vals[0] / n_prof, 2),
                "all_gather_kernels_ms": round(vals[1] / n_prof, 2),
                "reduce_scatter_kernels_ms": round(vals[2] / n_prof, 2),
                "compute_blocked_on_comm_ms": round(vals[3] / n_prof, 2),
                "optimizer_ms": round(vals[4] / n_prof, 2),
                "note": "max over ranks of each quantity; kernel times run from the moment a collective's inputs are "
                        "ready, so they include waiting for the slowest rank to arrive",
            }
        out["peak_mem_gb"] = torch.cuda.max_memory_allocated() / 2**30
        engine.close()
        del engine
        gc.collect()
        torch.cuda.empty_cache()
        return out

    log(f"[bench] step arm '{args.comm}' on {world} GPU(s)")
    main_arm = run_arm(args.comm if world > 1 else "symm", with_e2e=True, with_breakdown=True)
    nccl_arm, side_errors = None, {}
    if world > 1 and not args.skip_nccl_arm and args.comm != "nccl":
        log("[bench] step arm 'nccl'")
        try:
            nccl_arm = run_arm("nccl", with_e2e=False, with_breakdown=True)
        except Exception as exc:  # noqa: BLE001 - the headline number above must still be reported
            side_errors["step_nccl_arm"] = f"{type(exc).__name__}: {exc}"

    sweep_rows, sweep_summary, ep_rows = None, None, None
    if world > 1 and not args.skip_collectives:
        log("[bench] collective sweep")
        try:
            sweep_rows = perf.sweep_collectives(
                comm, device, max_bytes=args.sweep_max_bytes, warmup=args.sweep_warmup, iters=args.sweep_iters, log=log)
            sweep_summary = perf.summarize_sweep(sweep_rows)
            if rank == 0 and args.sweep_json:
                with open(args.sweep_json, "w") as f:
                    json.dump(sweep_rows, f)
        except Exception as exc:  # noqa: BLE001
            sweep_rows, sweep_summary = None, None
            side_errors["collectives"] = f"{type(exc).__name__}: {exc}"
    if world > 1 and not args.skip_ep and 256 % world == 0:
        log("[bench] MoE dispatch / combine")
        try:
            ep_rows = perf.moe_ep_latency(comm, device)
        except Exception as exc:  # noqa: BLE001 - the step and sweep numbers must still be reported
            ep_rows = [{"error": f"{type(exc).__name__}: {exc}"}]

    ms, ms_e2e = main_arm["ms"], main_arm["ms_e2e"]
    value = tokens_per_step * args.steps / (ms / 1000.0)
    e2e_value = tokens_per_step * args.steps / (ms_e2e / 1000.0)
    flops = cfg.flops_per_token(seq) * value
    clocks = main_arm["clocks"]
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
            "comm": args.comm if world > 1 else "none (one rank)",
            "l2": "training step: every step streams >100 GB of parameters, activations and optimizer state, inputs "
                  "are larger than L2; collective sweep: back-to-back calls as in nccl-tests, no flush (messages up "
                  "to 64 MB are L2-resident for both arms); MoE: a 256 MB buffer is rewritten between calls",
        },
        "e2e": {
            "value": round(e2e_value, 1),
            "unit": "tokens/s",
            "ms_per_step": round(ms_e2e / args.steps, 3),
            "h2d_bytes_per_step": h2d_bytes,
            "d2h_bytes_per_step": 4,
        },
        "gpu_launches": int(main_arm["launches"]),
        "clocks": {k: clocks[k] for k in ("sm_mhz", "sm_max_mhz", "reasons")},
        "ms_per_step_x_sm_ghz": round(ms / args.steps * (clocks["sm_mhz"] or 0) / 1000.0, 2),
        "timed_regions_ms_per_step": [round(ms / args.steps, 3), round(ms_e2e / args.steps, 3)],
        "model_tflops_per_gpu": round(flops / world / 1e12, 1),
        "peak_mem_gb": round(main_arm["peak_mem_gb"], 1),
        "final_loss": round(main_arm["loss"], 4),
        "step_breakdown": main_arm.get("breakdown"),
        "impl": "ours",
    }
    if nccl_arm is not None:
        nv = tokens_per_step * args.steps / (nccl_arm["ms"] / 1000.0)
        line["step_nccl_arm"] = {
            "what": "same engine, parameter all-gather and gradient reduce-scatter on NCCL (bf16) with separate cast kernels",
            "value": round(nv, 1),
            "unit": "tokens/s",
            "ms_per_step": round(nccl_arm["ms"] / args.steps, 3),
            "clocks": {k: nccl_arm["clocks"][k] for k in ("sm_mhz", "sm_max_mhz", "reasons")},
            "own_over_nccl": round(value / nv, 3),
            "step_breakdown": nccl_arm.get("breakdown"),
        }
    if sweep_summary is not None:
        line["collectives"] = {
            "protocol": f"{args.sweep_warmup} warm-up + {args.sweep_iters} timed calls per point, device-timed, max over "
                        "ranks; own = kernels on symmetric tensors, nccl = NCCL on ordinary tensors",
            "summary": sweep_summary,
            "rows": [[r["op"], r["dtype"], r["bytes"], r["arm"], r["avg_us"], r["p50_us"], r["busbw_gbs"]] for r in sweep_rows],
            "row_fields": ["op", "dtype", "bytes", "arm", "avg_us", "p50_us", "busbw_gbs"],
        }
    if ep_rows is not None:
        line["moe_ep"] = ep_rows
    if side_errors:
        line["side_measurement_errors"] = side_errors
    if rank == 0:
        print(json.dumps(line), flush=True)      # before the teardown: a failed side measurement may have broken it
    try:
        torch.cuda.synchronize()
        comm.finalize()
    except Exception as exc:  # noqa: BLE001
        log(f"[bench] teardown: {type(exc).__name__}: {exc}")


if __name__ == "__main__":
    main()
