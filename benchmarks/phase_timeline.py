"""Per-block phase timelines of the multi-GPU kernels, from the stamps the kernels write themselves.

    torchrun --nproc-per-node N benchmarks/phase_timeline.py [--bytes 268435456] [--out timeline.txt]

For each kernel: two warm-up calls, a barrier, then ONE traced call (`enable_trace`: every block stamps the GPU's
nanosecond timer at its phase boundaries). Printed per phase: minimum / median / maximum duration over the blocks and
when the last block left the phase; for the transfer phases also the bytes this rank moved over NVLink divided by the
time from the first block entering to the last block leaving. Rank 0 prints; every rank writes `<out>.rank<r>`.

Kernels: one-pass all-gather, reduce-scatter, all-reduce and all-to-all on symmetric tensors (`coll_symm.cu`), MoE
dispatch and pull combine (`moe_ep.cu`). The fused tensor-parallel GEMM kernels have their own timeline in
`tp_layer_perf.py --trace`.
"""
from __future__ import annotations

import argparse
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import torch  # noqa: E402

import torchcomms_b200 as tc  # noqa: E402
from torchcomms_b200.utils.trace_to_perfetto import phase_summary  # noqa: E402

BARRIERED = ("opening barrier (peers ready)", "transfer", "closing barrier (all data landed)")


def traced(comm, impl, fn):
    for _ in range(2):
        fn()
    comm.barrier(False)
    torch.cuda.synchronize()
    trace = impl.enable_trace()
    fn()
    torch.cuda.synchronize()
    impl.disable_trace()
    return trace.cpu()


def span_us(trace, first_mark, last_mark):
    rows = [r for r in trace.tolist() if r[first_mark] and r[last_mark]]
    if not rows:
        return 0.0
    return (max(r[last_mark] for r in rows) - min(r[first_mark] for r in rows)) / 1e3


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--bytes", type=int, default=256 << 20)
    ap.add_argument("--tokens", type=int, default=4096)
    ap.add_argument("--out", default="")
    args = ap.parse_args()
    os.environ.setdefault("RANK", "0")
    os.environ.setdefault("WORLD_SIZE", "1")
    os.environ.setdefault("LOCAL_RANK", os.environ["RANK"])
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    os.environ.setdefault("MASTER_PORT", "29577")
    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    comm = tc.new_comm("b200", dev, name="timeline")
    impl = comm.get_backend_impl()
    impl.enable_trace()          # first use allocates the trace buffer: keep that out of the first timeline
    impl.disable_trace()
    lines = []

    def section(title, trace, phases, nvlink_bytes=None, transfer=(1, 2)):
        lines.append(f"## {title}: rank {rank} of {world}")
        lines.extend(phase_summary(trace, phases))
        if nvlink_bytes is not None:
            us = span_us(trace, *transfer)
            if us > 0:
                lines.append(f"transfer: {nvlink_bytes / 1e6:.1f} MB over NVLink per rank in {us:.1f} us = {nvlink_bytes / us / 1e3:.0f} GB/s per direction")
        lines.append("")

    n = args.bytes // 2 // world * world                      # bf16 elements of the whole buffer
    part = n // world
    full = comm.symm_empty((n,), torch.bfloat16)
    full.normal_()
    shard = torch.randn(part, device=dev).to(torch.bfloat16)
    out_part = torch.empty(part, dtype=torch.bfloat16, device=dev)
    moved = (world - 1) * part * 2
    section(f"all_gather_single, {n * 2 >> 20} MB gathered", traced(comm, impl, lambda: comm.all_gather_single(full, shard, False)),
            BARRIERED, moved)
    section(f"reduce_scatter_single, {n * 2 >> 20} MB in", traced(comm, impl, lambda: comm.reduce_scatter_single(out_part, full, tc.ReduceOp.SUM, False)),
            BARRIERED, moved)
    section(f"all_reduce in place, {n * 2 >> 20} MB", traced(comm, impl, lambda: comm.all_reduce(full, tc.ReduceOp.AVG, False)),
            BARRIERED, 2 * moved if not impl.has_multicast() or world < 4 else (world + 1) * part * 2)
    src = torch.randn(n, device=dev).to(torch.bfloat16)
    section(f"all_to_all_single, {n * 2 >> 20} MB", traced(comm, impl, lambda: comm.all_to_all_single(full, src, False)), BARRIERED, moved)
    comm.symm_free(full)

    if world > 1 and 256 % world == 0:
        from torchcomms_b200.ops.moe_ep import Buffer

        T, H, E, K = args.tokens, 7168, 256, 8
        g = torch.Generator(device=dev).manual_seed(1234 + rank)
        x = torch.randn(T, H, generator=g, device=dev).to(torch.bfloat16)
        w, idx = torch.softmax(torch.randn(T, E, generator=g, device=dev), -1).topk(K, -1)
        idx, w = idx.to(torch.int32).contiguous(), w.float().contiguous()
        buf = Buffer(comm, max_tokens=T, hidden=H, num_experts=E, topk=K, fp8=True)
        d = buf.dispatch(x, idx, w)
        torch.cuda.synchronize()
        rows = int(d.num_tokens)
        epr = E // world
        remote_rows = int(torch.stack([((idx // epr) == r).any(dim=1) for r in range(world) if r != rank]).sum())
        section(f"MoE dispatch, {T} tokens (fp8 rows + scales)", traced(comm, impl, lambda: buf.dispatch(x, idx, w)),
                ("count destinations", "exchange counts (cross-GPU)", "quantise + store rows", "closing sync (block 0: cross-GPU)"),
                remote_rows * (H + H // 128 * 4), transfer=(2, 3))
        buf.combine_input[:rows].normal_()
        out = torch.empty(T, H, dtype=torch.bfloat16, device=dev)
        section(f"MoE combine (pull), {T} tokens", traced(comm, impl, lambda: buf.combine(out=out)),
                ("opening barrier (outputs complete)", "pull rows + weighted sum", "closing barrier (reads done)"),
                remote_rows * H * 2)
        del buf
        from torchcomms_b200.ops.moe_ep import LowLatencyBuffer

        t2 = 128
        ll = LowLatencyBuffer(comm, max_tokens=t2, hidden=H, num_experts=E, topk=K, fp8=True)
        x2, idx2, w2 = x[:t2].contiguous(), idx[:t2].contiguous(), w[:t2].contiguous()
        r = ll.dispatch(x2, idx2)
        section(f"MoE low-latency dispatch, {t2} tokens", traced(comm, impl, lambda: ll.dispatch(x2, idx2)),
                ("number rows per expert + grid sync", "publish counts", "quantise + store rows",
                 "wait for peers' counts", "pack rows as they arrive"))
        ll.expert_output.normal_()
        out2 = torch.empty(t2, H, dtype=torch.bfloat16, device=dev)
        section(f"MoE low-latency combine, {t2} tokens", traced(comm, impl, lambda: ll.combine(idx2, w2, r, out=out2)),
                ("opening barrier (outputs complete)", "pull rows + weighted sum", "closing barrier (reads done)"))
        del ll
    text = "\n".join(lines)
    if args.out:
        with open(f"{args.out}.rank{rank}", "w") as f:
            f.write(text)
    if rank == 0:
        print(text, flush=True)
    comm.finalize()


if __name__ == "__main__":
    main()
