"""Turns the in-kernel phase trace and flight-recorder dumps into a Chrome / Perfetto trace.

    tr = comm.get_backend_impl().enable_trace()      # [blocks, 16] int64, device nanosecond timer per phase mark of each block
    ... run ONE collective ...
    events = phase_trace_events(tr.cpu(), rank=comm.get_rank(),
                                phases=("copy-in", "barrier", "reduce", "barrier", "copy-out"))
    write_trace("ar.json", events + flight_recorder_events(json.load(open("fr_dump.json"))))

Open the file in ui.perfetto.dev or chrome://tracing: one process per rank, one
track per block, one slice per phase, plus one track of collective entries.

Parity: comms/pipes/scripts/pipestrace_to_perfetto.py (PipesTrace event log ->
Perfetto JSON) and the fr_trace-style dumps of comms/torchcomms/hooks/fr.
"""
from __future__ import annotations

import json
from typing import Any, Dict, Iterable, List, Optional, Sequence


def phase_trace_events(trace: Any, rank: int = 0, phases: Optional[Sequence[str]] = None,
                       name: str = "collective") -> List[Dict[str, Any]]:
    """``trace[b, s]`` = the GPU's nanosecond timer at mark ``s`` of block ``b`` (0 = mark not reached)."""
    rows = trace.tolist() if hasattr(trace, "tolist") else list(trace)
    starts = [r[0] for r in rows if r and r[0] != 0]
    if not starts:
        return []
    t0 = min(starts)
    to_us = 1e-3  # nanoseconds -> microseconds
    events: List[Dict[str, Any]] = [
        {"ph": "M", "pid": rank, "name": "process_name", "args": {"name": f"rank {rank} ({name})"}},
    ]
    for b, marks in enumerate(rows):
        if not marks or marks[0] == 0:
            continue
        events.append({"ph": "M", "pid": rank, "tid": b, "name": "thread_name", "args": {"name": f"block {b}"}})
        for s in range(len(marks) - 1):
            a, z = marks[s], marks[s + 1]
            if a == 0 or z == 0 or z < a:
                break
            label = phases[s] if phases is not None and s < len(phases) else f"phase {s}"
            events.append({"ph": "X", "pid": rank, "tid": b, "name": label, "cat": name,
                           "ts": (a - t0) * to_us, "dur": (z - a) * to_us})
    return events


def phase_summary(trace: Any, phases: Sequence[str]) -> List[str]:
    """Text table of a phase trace: for each phase (mark ``s`` to mark ``s + 1``) the minimum / median / maximum
    duration over the blocks that reached both marks, and when the last block left it (microseconds after the
    first block's first mark)."""
    rows = trace.tolist() if hasattr(trace, "tolist") else list(trace)
    rows = [r for r in rows if r and r[0] != 0]
    if not rows:
        return ["(no block stamped the trace)"]
    t0 = min(r[0] for r in rows)
    out = [f"{len(rows)} blocks; microseconds", f"{'phase':34s} {'blocks':>6s} {'min':>8s} {'median':>8s} {'max':>8s} {'last end':>9s}"]
    for s, label in enumerate(phases):
        durs = sorted((r[s + 1] - r[s]) / 1e3 for r in rows if s + 1 < len(r) and r[s] and r[s + 1] and r[s + 1] >= r[s])
        if not durs:
            continue
        last = max((r[s + 1] - t0) / 1e3 for r in rows if s + 1 < len(r) and r[s] and r[s + 1])
        out.append(f"{label:34s} {len(durs):6d} {durs[0]:8.1f} {durs[len(durs) // 2]:8.1f} {durs[-1]:8.1f} {last:9.1f}")
    return out


def flight_recorder_events(dump: Dict[str, Any], rank: Optional[int] = None) -> List[Dict[str, Any]]:
    """Entries of a flight-recorder JSON dump (``entries`` with ``profiling_name``, ``time_created_ns``,
    ``time_discovered_started_ns`` / ``time_discovered_completed_ns`` or ``duration_ms``) as slices."""
    entries: Iterable[Dict[str, Any]] = dump.get("entries", [])
    pid = rank if rank is not None else int(dump.get("rank", 0))
    out: List[Dict[str, Any]] = [
        {"ph": "M", "pid": pid, "tid": 100000, "name": "thread_name", "args": {"name": "collectives (flight recorder)"}},
    ]
    base = None
    for e in entries:
        start = e.get("time_discovered_started_ns") or e.get("time_created_ns")
        if start is None:
            continue
        base = start if base is None else min(base, start)
    for e in entries:
        start = e.get("time_discovered_started_ns") or e.get("time_created_ns")
        if start is None:
            continue
        end = e.get("time_discovered_completed_ns")
        if end is None and e.get("duration_ms") is not None:
            end = start + float(e["duration_ms"]) * 1e6
        dur_us = max(0.0, ((end or start) - start) / 1e3)
        out.append({"ph": "X", "pid": pid, "tid": 100000, "name": str(e.get("profiling_name", e.get("op", "op"))),
                    "cat": "fr", "ts": (start - base) / 1e3, "dur": dur_us,
                    "args": {k: e[k] for k in ("collective_seq_id", "state", "input_sizes", "output_sizes") if k in e}})
    return out


def write_trace(path: str, events: List[Dict[str, Any]]) -> None:
    with open(path, "w") as f:
        json.dump({"traceEvents": events, "displayTimeUnit": "ns"}, f)
