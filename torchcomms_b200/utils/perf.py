"""Device-timed measurement helpers shared by ``bench.py`` and ``benchmarks/``.

Everything here times on the device with CUDA events on the launching stream,
after warm-up calls, bracketed by a communicator barrier and a synchronize, and
reports the maximum over ranks.

* ``time_calls``         - back-to-back calls of one function: average and p50
* ``sweep_collectives``  - bus bandwidth and latency versus message size for
  all-reduce, all-gather, reduce-scatter and all-to-all-v, this framework's
  kernels (symmetric tensors, the way a user of ``comm.symm_empty`` runs them)
  next to NCCL on ordinary tensors
* ``moe_ep_latency``     - MoE dispatch / combine latency, fused kernels next to
  the unfused NCCL pipeline

Parity: ``comms/torchcomms/tests/perf/py/perf_test_helpers.py:22-36`` and
``all_reduce_perf.py:66-70`` (bus-bandwidth factors; host-timed there).
"""
from __future__ import annotations

import statistics
from typing import Callable, Dict, Iterable, List, Optional

import torch

from .. import ReduceOp

DTYPES = {"bf16": torch.bfloat16, "fp32": torch.float32, "fp16": torch.float16}


def max_over_ranks(comm, values: List[float], device) -> List[float]:
    t = torch.tensor(values, dtype=torch.float32, device=device)
    comm.all_reduce(t, ReduceOp.MAX, False)
    return [float(v) for v in t.tolist()]


def time_calls(comm, fn: Callable[[], object], warmup: int, iters: int, device, batch: int = 10) -> Dict[str, float]:
    """Average and median device time (microseconds) of one call of ``fn``, issued back to back.

    The average spans all ``iters`` calls between two events. The median is
    taken over batches of ``batch`` calls (an event after every call would cost
    about as much as a small collective and hold the stream back).
    """
    for _ in range(warmup):
        fn()
    comm.barrier(False)
    torch.cuda.synchronize()
    batch = max(1, min(batch, iters))
    nb = (iters + batch - 1) // batch
    marks = [torch.cuda.Event(enable_timing=True) for _ in range(nb + 1)]
    marks[0].record()
    done = 0
    sizes = []
    for b in range(nb):
        k = min(batch, iters - done)
        for _ in range(k):
            fn()
        done += k
        sizes.append(k)
        marks[b + 1].record()
    torch.cuda.synchronize()
    per_call = [marks[b].elapsed_time(marks[b + 1]) * 1000.0 / sizes[b] for b in range(nb)]
    avg = marks[0].elapsed_time(marks[-1]) * 1000.0 / iters
    avg, p50 = max_over_ranks(comm, [avg, statistics.median(per_call)], device)
    return {"avg_us": avg, "p50_us": p50}


def a2av_splits(rank: int, world: int, rows: int) -> tuple:
    """Uneven but globally consistent row counts: what ``rank`` sends to / receives from each peer.

    Peer p gets ``base + s(rank, p) * base // 4`` rows with s = +1 for the
    next world/2 - 1 ranks, -1 for the previous ones, 0 otherwise, so every
    rank's rows still add up to ``rows`` on both sides.
    """
    base = rows // world

    def s(a, b):
        d = (b - a) % world
        if d == 0 or 2 * d == world:
            return 0
        return 1 if 2 * d < world else -1

    send = [base + s(rank, p) * (base // 4) for p in range(world)]
    recv = [base + s(p, rank) * (base // 4) for p in range(world)]
    return send, recv


def sweep_collectives(
    comm,
    device,
    *,
    ops: Iterable[str] = ("all_reduce", "all_gather", "reduce_scatter", "all_to_all_v"),
    dtypes: Iterable[str] = ("bf16", "fp32"),
    min_bytes: int = 1024,
    max_bytes: int = 1 << 30,
    warmup: int = 20,
    iters: int = 100,
    arms: Iterable[str] = ("own", "nccl"),
    log: Optional[Callable[[str], None]] = None,
    small_recv_bytes: int = 1 << 20,
) -> List[dict]:
    """Rows of {op, dtype, bytes, arm, avg_us, p50_us, algbw_gbs, busbw_gbs}.

    ``bytes`` is the size of the whole reduced / gathered / scattered /
    exchanged buffer on one rank, as in nccl-tests. The ``own`` arm runs the
    operation on a symmetric tensor (one-pass kernels; messages in the latency
    class of all-reduce take the flag-less kernel), the ``nccl`` arm routes the
    same call through NCCL on ordinary tensors.
    """
    world = comm.get_size()
    if world < 2:
        return []
    sizes = []
    b = min_bytes
    while b <= max_bytes:
        sizes.append(b)
        b *= 2
    top = sizes[-1]
    # One symmetric and two ordinary buffers serve every case as views.
    symm_raw = comm.symm_empty((top,), torch.uint8)
    plain_a = torch.empty(top, dtype=torch.uint8, device=device)
    plain_b = torch.empty(top, dtype=torch.uint8, device=device)
    rows = []
    for op in ops:
        for dname in dtypes:
            dt = DTYPES[dname]
            esz = torch.empty(0, dtype=dt).element_size()
            for t in (symm_raw, plain_a, plain_b):
                t.view(dt).uniform_(-1.0, 1.0)
            for nbytes in sizes:
                # element counts that keep every rank's part a whole number of 16-byte vectors
                n = max(world * (16 // esz), nbytes // esz // (world * (16 // esz)) * (world * (16 // esz)))
                total = n * esz
                for arm in arms:
                    own_small = None
                    hints = {"algo": "nccl"} if arm == "nccl" else None
                    sym = symm_raw[:total].view(dt)
                    pa = plain_a[:total].view(dt)
                    pb = plain_b[:total].view(dt)
                    if op == "all_reduce":
                        buf = sym if arm == "own" else pa
                        fn = lambda buf=buf: comm.all_reduce(buf, ReduceOp.AVG, False, hints=hints)  # AVG keeps values bounded
                        factor = 2 * (world - 1) / world
                    elif op == "all_gather":
                        src = pb[: n // world]
                        dst = sym if arm == "own" else pa
                        fn = lambda src=src, dst=dst: comm.all_gather_single(dst, src, False, hints=hints)
                        factor = (world - 1) / world
                    elif op == "reduce_scatter":
                        src = sym if arm == "own" else pa
                        dst = pb[: n // world]
                        fn = lambda src=src, dst=dst: comm.reduce_scatter_single(dst, src, ReduceOp.SUM, False, hints=hints)
                        factor = (world - 1) / world
                    elif op == "all_to_all_v":
                        row = 16 // esz  # rows of 16 bytes
                        send, recv = a2av_splits(comm.get_rank(), world, n // row)
                        src = pb.view(-1, row)
                        if arm == "own" and total <= small_recv_bytes:
                            # A receive buffer of the message's own size, as a caller with small messages allocates
                            # it: its size bounds every part on every rank, which lets the backend take the
                            # flag-less exchange. (The other points share one large symmetric buffer.)
                            own_small = comm.symm_empty((total,), torch.uint8)
                            dst = own_small.view(dt).view(-1, row)
                        else:
                            dst = (sym if arm == "own" else pa).view(-1, row)
                        fn = lambda src=src, dst=dst, send=send, recv=recv: comm.all_to_all_v_single(
                            dst, src, recv, send, False, hints=hints)
                        factor = (world - 1) / world
                    else:
                        raise ValueError(f"unknown op {op}")
                    t = time_calls(comm, fn, warmup, iters, device)
                    if own_small is not None:
                        torch.cuda.synchronize()
                        comm.symm_free(own_small)
                        own_small = None
                    algbw = total / t["avg_us"] / 1e3
                    r = {
                        "op": op, "dtype": dname, "bytes": total, "arm": arm,
                        "avg_us": round(t["avg_us"], 2), "p50_us": round(t["p50_us"], 2),
                        "algbw_gbs": round(algbw, 1), "busbw_gbs": round(algbw * factor, 1),
                    }
                    rows.append(r)
                    if log is not None:
                        log(f"{op:15s} {dname:5s} {total:11d} {arm:5s} avg {r['avg_us']:10.2f} us  p50 {r['p50_us']:10.2f} us  "
                            f"busbw {r['busbw_gbs']:8.1f} GB/s")
    torch.cuda.synchronize()
    comm.symm_free(symm_raw)
    return rows


def summarize_sweep(rows: List[dict]) -> dict:
    """Compact view for a one-line report: per op and dtype, busbw at 1 MB / 64 MB / the largest size and
    p50 latency at the smallest / 64 KB, both arms, plus how many sizes >= 1 MB the own arm wins."""
    out: dict = {}
    keys = sorted({(r["op"], r["dtype"]) for r in rows})
    for op, dt in keys:
        mine = {r["bytes"]: r for r in rows if r["op"] == op and r["dtype"] == dt and r["arm"] == "own"}
        ref = {r["bytes"]: r for r in rows if r["op"] == op and r["dtype"] == dt and r["arm"] == "nccl"}
        sizes = sorted(mine)
        if not sizes:
            continue

        def near(target):
            return min(sizes, key=lambda s: abs(s - target))

        entry = {}
        for label, target in (("1MB", 1 << 20), ("64MB", 64 << 20), ("max", sizes[-1])):
            s = near(target)
            entry[f"busbw_{label}"] = {"bytes": s, "own": mine[s]["busbw_gbs"], "nccl": ref.get(s, {}).get("busbw_gbs")}
        for label, target in (("min", sizes[0]), ("64KB", 64 << 10)):
            s = near(target)
            entry[f"p50_us_{label}"] = {"bytes": s, "own": mine[s]["p50_us"], "nccl": ref.get(s, {}).get("p50_us")}
        big = [s for s in sizes if s >= (1 << 20) and s in ref]
        entry["sizes_ge_1MB_own_faster"] = f"{sum(1 for s in big if mine[s]['avg_us'] <= ref[s]['avg_us'])}/{len(big)}"
        out[f"{op}/{dt}"] = entry
    return out


def moe_ep_latency(
    comm,
    device,
    *,
    tokens: int = 4096,
    hidden: int = 7168,
    experts: int = 256,
    topk: int = 8,
    warmup: int = 10,
    iters: int = 50,
    with_nccl: bool = True,
    ll_tokens: int = 128,
) -> List[dict]:
    """Dispatch / combine latency (microseconds, max over ranks), L2 flushed between calls.

    ``ll_tokens`` > 0 adds the low-latency pair (``ll_dispatch`` / ``ll_combine``, arm ``fused``) on that many
    tokens per rank: one row per (token, expert) pair into fixed slots, pull combine.

    Router logits ~N(0,1), softmax, top-k; x ~N(0,1) bf16. ``fused``: one kernel
    does routing counts, block-scaled fp8 (e4m3, 1x128) quantisation, token
    permutation and the peer stores; combine applies the weighted top-k sum.
    ``nccl``: per-destination gather, quantisation in PyTorch, split exchange
    and ``all_to_all_v_single`` through NCCL; combine = exchange back + index_add.
    """
    from ..ops.moe_ep import Buffer, per_token_cast_to_fp8

    world, rank = comm.get_size(), comm.get_rank()
    T, H, E, K = tokens, hidden, experts, topk
    epr = E // world
    g = torch.Generator(device=device).manual_seed(1234 + rank)
    x = torch.randn(T, H, generator=g, device=device).to(torch.bfloat16)
    logits = torch.randn(T, E, generator=g, device=device)
    w, idx = torch.softmax(logits, -1).topk(K, -1)
    idx = idx.to(torch.int32).contiguous()
    w = w.float().contiguous()
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=device)

    def time_it(fn):
        for _ in range(warmup):
            fn()
        comm.barrier(False)
        torch.cuda.synchronize()
        per = []
        for _ in range(iters):
            flush.zero_()
            comm.barrier(False)
            s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            s.record()
            fn()
            e.record()
            e.synchronize()
            per.append(s.elapsed_time(e) * 1000.0)
        avg, p50 = max_over_ranks(comm, [sum(per) / len(per), statistics.median(per)], device)
        return avg, p50

    rows = []

    def report(phase, arm, t, nbytes):
        rows.append({"phase": phase, "arm": arm, "avg_us": round(t[0], 1), "p50_us": round(t[1], 1),
                     "gbs": round(nbytes / t[0] / 1e3, 1), "world": world, "tokens": T, "hidden": H, "experts": E, "topk": K})

    buf = Buffer(comm, max_tokens=T, hidden=H, num_experts=E, topk=K, fp8=True)
    d = buf.dispatch(x, idx, w)
    torch.cuda.synchronize()
    n_recv = int(d.num_tokens)
    report("dispatch", "fused", time_it(lambda: buf.dispatch(x, idx, w)), n_recv * (H + H // 128 * 4))
    buf.combine_input[:n_recv].normal_()
    out = torch.empty(T, H, dtype=torch.bfloat16, device=device)
    report("combine", "fused", time_it(lambda: buf.combine(out=out)), n_recv * H * 2)

    if with_nccl and world > 1:
        hint = {"algo": "nccl"}
        in_rank = torch.stack([((idx // epr) == r).any(dim=1) for r in range(world)], dim=0)
        state = {}

        def nccl_dispatch():
            sel = [in_rank[r].nonzero().flatten() for r in range(world)]
            counts = torch.tensor([s.numel() for s in sel], dtype=torch.int64, device=device)  # one host sync, as users pay
            order = torch.cat(sel)
            q, sc = per_token_cast_to_fp8(x[order])
            recv_counts = torch.empty_like(counts)
            comm.all_to_all_single(recv_counts, counts, False, hints=hint)
            ins, outs = counts.tolist(), recv_counts.tolist()
            n = sum(outs)
            rq = torch.empty(n, H, dtype=torch.uint8, device=device)
            rs = torch.empty(n, H // 128, dtype=torch.float32, device=device)
            comm.all_to_all_v_single(rq, q.view(torch.uint8), outs, ins, False, hints=hint)
            comm.all_to_all_v_single(rs, sc.contiguous(), outs, ins, False, hints=hint)
            state.update(order=order, ins=ins, outs=outs, n=n)
            return rq, rs

        nccl_dispatch()
        torch.cuda.synchronize()
        report("dispatch", "nccl", time_it(nccl_dispatch), state["n"] * (H + H // 128 * 4))
        y_exp = torch.randn(state["n"], H, device=device).to(torch.bfloat16)

        def nccl_combine():
            back = torch.empty(len(state["order"]), H, dtype=torch.bfloat16, device=device)
            comm.all_to_all_v_single(back, y_exp, state["ins"], state["outs"], False, hints=hint)
            res = torch.zeros(T, H, dtype=torch.float32, device=device)
            res.index_add_(0, state["order"], back.float())
            return res.to(torch.bfloat16)

        report("combine", "nccl", time_it(nccl_combine), state["n"] * H * 2)
    torch.cuda.synchronize()
    del buf
    if ll_tokens > 0:
        from ..ops.moe_ep import LowLatencyBuffer

        t2 = min(ll_tokens, T)
        ll = LowLatencyBuffer(comm, max_tokens=t2, hidden=H, num_experts=E, topk=K, fp8=True)
        x2, idx2, w2 = x[:t2].contiguous(), idx[:t2].contiguous(), w[:t2].contiguous()
        r = ll.dispatch(x2, idx2)
        torch.cuda.synchronize()
        pairs = int((idx2 >= 0).sum())

        def ll_report(phase, t, nbytes):
            rows.append({"phase": phase, "arm": "fused", "avg_us": round(t[0], 1), "p50_us": round(t[1], 1),
                         "gbs": round(nbytes / t[0] / 1e3, 1), "world": world, "tokens": t2, "hidden": H, "experts": E, "topk": K})

        ll_report("ll_dispatch", time_it(lambda: ll.dispatch(x2, idx2)), pairs * (H + H // 128 * 4))
        ll.expert_output.normal_()
        out2 = torch.empty(t2, H, dtype=torch.bfloat16, device=device)
        ll_report("ll_combine", time_it(lambda: ll.combine(idx2, w2, r, out=out2)), pairs * H * 2)
        # Back to back (no flush, no barrier, 100 calls between two events): what a decode loop sees once the
        # launch path of the host is hidden behind the previous call.
        for phase, fn, nbytes in (("ll_dispatch_b2b", lambda: ll.dispatch(x2, idx2), pairs * (H + H // 128 * 4)),
                                  ("ll_combine_b2b", lambda: ll.combine(idx2, w2, r, out=out2), pairs * H * 2)):
            t = time_calls(comm, fn, warmup, 100, device)
            ll_report(phase, (t["avg_us"], t["p50_us"]), nbytes)
        torch.cuda.synchronize()
        del ll
    return rows
