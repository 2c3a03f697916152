"""Every collective of a communicator in every calling variant.

The table below describes each operation once (how to build its buffers, how
to start it, what the result must be); ``run_matrix`` then drives every entry
through the variants of the reference's per-operation integration tests
(comms/torchcomms/tests/integration/py/AllReduceTest.py:22-110 and its
siblings: ``_sync_*``, ``_sync_*_no_work``, ``_async_*``,
``_async_*_early_reset``, ``_*_input_deleted``, ``_graph_*``):

* ``sync``            synchronous call, work waited for
* ``sync_no_work``    synchronous call, returned work ignored
* ``async``           asynchronous call, then ``wait()``
* ``early_reset``     asynchronous call whose work is dropped at once; a later
                      barrier on the same communicator orders the check
* ``input_deleted``   asynchronous call, the caller's references to the inputs
                      are dropped before ``wait()``
* ``graph``           (CUDA only) the call captured into a CUDA graph that is
                      replayed three times with fresh inputs

Used by the gloo test (CPU) and by the two-rank GPU battery.
"""
from __future__ import annotations

import gc
from typing import Callable, Dict, List, Tuple

import torch

VARIANTS_CPU = ("sync", "sync_no_work", "async", "early_reset", "input_deleted")
VARIANTS_GPU = VARIANTS_CPU + ("graph",)

N = 96  # elements per rank-sized piece


class Case:
    """One operation: ``make()`` builds fresh buffers, ``start(bufs, async_op)`` issues it and returns the work,
    ``check(bufs)`` asserts the outcome.  ``inputs`` names the entries of ``bufs`` that are read only."""

    def __init__(self, name: str, make: Callable[[], Dict[str, object]], start: Callable[[Dict[str, object], bool], object],
                 check: Callable[[Dict[str, object]], None], inputs: Tuple[str, ...] = (), refill: Callable = None):
        self.name, self.make, self.start, self.check, self.inputs, self.refill = name, make, start, check, inputs, refill


def build_cases(comm, tc, dev: torch.device, dtype=torch.float32) -> List[Case]:
    rank, world = comm.get_rank(), comm.get_size()
    tri = float(world * (world + 1) // 2)
    root = world - 1

    def val(r, n=N):
        return torch.full((n,), float(r + 1), dtype=dtype, device=dev)

    def empty(n=N):
        return torch.zeros(n, dtype=dtype, device=dev)

    def eq(t, expect):
        assert torch.equal(t.float().cpu(), expect.float().cpu()), (t.flatten()[:4], expect.flatten()[:4])

    ranks_col = torch.arange(1, world + 1, dtype=torch.float32).repeat_interleave(N)
    cases: List[Case] = []

    cases.append(Case(
        "all_reduce", lambda: {"t": val(rank)},
        lambda b, a: comm.all_reduce(b["t"], tc.ReduceOp.SUM, a),
        lambda b: eq(b["t"], torch.full((N,), tri))))
    cases.append(Case(
        "reduce", lambda: {"t": val(rank)},
        lambda b, a: comm.reduce(b["t"], root, tc.ReduceOp.SUM, a),
        lambda b: eq(b["t"], torch.full((N,), tri)) if rank == root else None))
    cases.append(Case(
        "broadcast", lambda: {"t": val(rank)},
        lambda b, a: comm.broadcast(b["t"], root, a),
        lambda b: eq(b["t"], torch.full((N,), float(root + 1)))))
    cases.append(Case(
        "all_gather_single", lambda: {"out": empty(world * N), "in": val(rank)},
        lambda b, a: comm.all_gather_single(b["out"], b["in"], a),
        lambda b: eq(b["out"], ranks_col), inputs=("in",)))
    cases.append(Case(
        "all_gather", lambda: {"outs": [empty() for _ in range(world)], "in": val(rank)},
        lambda b, a: comm.all_gather(b["outs"], b["in"], a),
        lambda b: eq(torch.cat(b["outs"]), ranks_col), inputs=("in",)))
    cases.append(Case(
        "all_gather_v", lambda: {"outs": [empty(8 * (r + 1)) for r in range(world)], "in": val(rank, 8 * (rank + 1))},
        lambda b, a: comm.all_gather_v(b["outs"], b["in"], a),
        lambda b: eq(torch.cat(b["outs"]), torch.cat([torch.full((8 * (r + 1),), float(r + 1)) for r in range(world)])),
        inputs=("in",)))
    cases.append(Case(
        "reduce_scatter_single", lambda: {"out": empty(), "in": val(rank, world * N)},
        lambda b, a: comm.reduce_scatter_single(b["out"], b["in"], tc.ReduceOp.SUM, a),
        lambda b: eq(b["out"], torch.full((N,), tri)), inputs=("in",)))
    cases.append(Case(
        "reduce_scatter", lambda: {"out": empty(), "ins": [val(rank) * (d + 1) for d in range(world)]},
        lambda b, a: comm.reduce_scatter(b["out"], b["ins"], tc.ReduceOp.SUM, a),
        lambda b: eq(b["out"], torch.full((N,), tri * (rank + 1))), inputs=("ins",)))
    cases.append(Case(
        "reduce_scatter_v", lambda: {"out": empty(8 * (rank + 1)), "ins": [val(rank, 8 * (d + 1)) for d in range(world)]},
        lambda b, a: comm.reduce_scatter_v(b["out"], b["ins"], tc.ReduceOp.SUM, a),
        lambda b: eq(b["out"], torch.full((8 * (rank + 1),), tri)), inputs=("ins",)))
    cases.append(Case(
        "all_to_all_single",
        lambda: {"out": empty(world * N), "in": torch.cat([torch.full((N,), float(rank * world + d), dtype=dtype, device=dev) for d in range(world)])},
        lambda b, a: comm.all_to_all_single(b["out"], b["in"], a),
        lambda b: eq(b["out"], torch.cat([torch.full((N,), float(s * world + rank)) for s in range(world)])), inputs=("in",)))
    in_splits = [d + 1 for d in range(world)]
    out_splits = [rank + 1] * world
    cases.append(Case(
        "all_to_all_v_single",
        lambda: {"out": empty(sum(out_splits)),
                 "in": torch.cat([torch.full((d + 1,), float(rank * 10 + d), dtype=dtype, device=dev) for d in range(world)])},
        lambda b, a: comm.all_to_all_v_single(b["out"], b["in"], out_splits, in_splits, a),
        lambda b: eq(b["out"], torch.cat([torch.full((rank + 1,), float(s * 10 + rank)) for s in range(world)])), inputs=("in",)))
    cases.append(Case(
        "all_to_all",
        lambda: {"outs": [empty(16) for _ in range(world)],
                 "ins": [torch.full((16,), float(rank * world + d), dtype=dtype, device=dev) for d in range(world)]},
        lambda b, a: comm.all_to_all(b["outs"], b["ins"], a),
        lambda b: eq(torch.cat(b["outs"]), torch.cat([torch.full((16,), float(s * world + rank)) for s in range(world)])),
        inputs=("ins",)))
    cases.append(Case(
        "scatter",
        lambda: {"out": empty(), "ins": [val(d) for d in range(world)] if rank == root else []},
        lambda b, a: comm.scatter(b["out"], b["ins"], root, a),
        lambda b: eq(b["out"], torch.full((N,), float(rank + 1))), inputs=("ins",)))
    cases.append(Case(
        "gather",
        lambda: {"outs": [empty() for _ in range(world)] if rank == root else [], "in": val(rank)},
        lambda b, a: comm.gather(b["outs"], b["in"], root, a),
        lambda b: eq(torch.cat(b["outs"]), ranks_col) if rank == root else None, inputs=("in",)))
    cases.append(Case("barrier", lambda: {}, lambda b, a: comm.barrier(a), lambda b: None))

    nxt, prv = (rank + 1) % world, (rank - 1) % world

    def start_ring(b, a):
        batch = comm.batch_op_create()
        batch.send(b["payload"], nxt)
        batch.recv(b["got"], prv)
        return batch.issue(a)

    cases.append(Case(
        "batch_send_recv", lambda: {"payload": val(rank, 32), "got": empty(32)}, start_ring,
        lambda b: eq(b["got"], torch.full((32,), float(prv + 1))), inputs=("payload",)))
    return cases


def _sync(dev: torch.device) -> None:
    if dev.type == "cuda":
        torch.cuda.synchronize(dev)


def run_matrix(comm, tc, dev: torch.device, variants=VARIANTS_CPU, skip: Tuple[str, ...] = (), dtype=torch.float32) -> int:
    """Runs every case in every variant; returns the number of (case, variant) pairs that ran."""
    ran = 0
    for case in build_cases(comm, tc, dev, dtype):
        if case.name in skip:
            continue
        for variant in variants:
            bufs = case.make()
            if variant == "sync":
                w = case.start(bufs, False)
                w.wait()
            elif variant == "sync_no_work":
                case.start(bufs, False)
            elif variant == "async":
                case.start(bufs, True).wait()
            elif variant == "early_reset":
                w = case.start(bufs, True)
                w = None
                gc.collect()
                comm.barrier(False)       # issued after the dropped work on the same communicator
            elif variant == "input_deleted":
                w = case.start(bufs, True)
                for key in case.inputs:   # the work keeps what it still reads alive
                    bufs[key] = None
                gc.collect()
                w.wait()
            elif variant == "graph":
                if case.name in ("batch_send_recv",):
                    continue              # point-to-point inside a capture is covered by the backend battery
                stream = torch.cuda.Stream(dev)
                stream.wait_stream(torch.cuda.current_stream(dev))
                graph = torch.cuda.CUDAGraph()
                with torch.cuda.stream(stream):
                    with torch.cuda.graph(graph, stream=stream):
                        case.start(bufs, False)
                    fresh = case.make()
                    for _ in range(3):
                        for key, value in fresh.items():   # same values again: a replay must recompute the result
                            _copy_into(bufs[key], value)
                        graph.replay()
                        stream.synchronize()
                        case.check(bufs)
                torch.cuda.current_stream(dev).wait_stream(stream)
                del graph
                ran += 1
                continue
            else:
                raise ValueError(variant)
            _sync(dev)
            try:
                case.check(bufs)
            except AssertionError as e:
                raise AssertionError(f"{case.name} / {variant}: {e}") from e
            ran += 1
    return ran


def _copy_into(dst, src) -> None:
    if isinstance(dst, list):
        for d, s in zip(dst, src):
            d.copy_(s)
    elif dst is not None:
        dst.copy_(src)
