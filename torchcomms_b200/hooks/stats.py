"""Per-operation counters of a communicator, exportable as a dict.

    stats = CommStatsHook(); stats.register_with_comm(comm)
    ... training ...
    stats.snapshot()
    # {"all_reduce": {"calls": 120, "bytes": 503316480, "async_calls": 120, "completed": 120,
    #                 "busy_ms": 18.4, "max_ms": 0.31, "gbps": 27.3, "size_histogram": {"4MiB": 120}}, ...}

``calls`` / ``bytes`` / ``size_histogram`` are counted in the pre-hook (bytes =
what the operation moves on this rank: the larger of its input and output).
``busy_ms`` sums, per operation, the host-clock time from the work's start hook
to its end hook (for stream-ordered backends that is the watchdog's view of the
device: resolution is its polling interval, so use it to rank operations and
spot stragglers, not as a kernel timer); ``gbps`` = bytes of completed
operations / busy time.

Parity: the reference keeps such counters inside NCCLX (``CollectiveStats`` and
the GPU collstats histograms, comms/utils/cvars/nccl_cvars.yaml:21-60); here
they are a hook any backend gets.
"""
from __future__ import annotations

import threading
import time
from typing import Any, Dict, List

import torch

from .._comms import OpName


def _nbytes(value: Any) -> int:
    if value is None:
        return 0
    if isinstance(value, torch.Tensor):
        return value.nbytes
    return sum(t.nbytes for t in value if isinstance(t, torch.Tensor))


def _bucket(nbytes: int) -> str:
    """Power-of-two size class: "0B", "4KiB", "2MiB", ..."""
    if nbytes <= 0:
        return "0B"
    b = 1 << (nbytes - 1).bit_length()
    for unit, shift in (("GiB", 30), ("MiB", 20), ("KiB", 10)):
        if b >= 1 << shift:
            return f"{b >> shift}{unit}"
    return f"{b}B"


class _OpStats:
    __slots__ = ("calls", "bytes", "async_calls", "completed", "completed_bytes", "busy_s", "max_s", "hist")

    def __init__(self) -> None:
        self.calls = self.bytes = self.async_calls = self.completed = self.completed_bytes = 0
        self.busy_s = self.max_s = 0.0
        self.hist: Dict[str, int] = {}


class CommStatsHook:
    """Counts calls, bytes and busy time per operation of the communicators it is registered with."""

    def __init__(self) -> None:
        self._lock = threading.Lock()
        self._ops: Dict[str, _OpStats] = {}
        self._pending: Dict[int, tuple] = {}     # op id -> (op name, bytes)
        self._handles: List[Any] = []

    # ------------------------------------------------------------------ registration
    def register_with_comm(self, comm: Any) -> None:
        self._handles.append(comm.register_pre_hook(self._pre))
        self._handles.append(comm.register_post_hook(self._post))

    def unregister(self) -> None:
        while self._handles:
            self._handles.pop().remove()

    def is_enabled(self) -> bool:
        return bool(self._handles)

    # ------------------------------------------------------------------ hooks
    def _pre(self, op: OpName, op_id: int, args: Any) -> None:
        rec = args.record
        nbytes = max(_nbytes(list(rec.inputs)), _nbytes(list(rec.outputs)))
        with self._lock:
            st = self._ops.setdefault(op.name, _OpStats())
            st.calls += 1
            st.bytes += nbytes
            st.async_calls += 1 if rec.async_op else 0
            b = _bucket(nbytes)
            st.hist[b] = st.hist.get(b, 0) + 1
            self._pending[op_id] = (op.name, nbytes)
            if len(self._pending) > 4096:                 # operations that raised never reach the post-hook
                for stale in sorted(self._pending)[:2048]:
                    del self._pending[stale]

    def _post(self, op_id: int, args: Any) -> None:
        with self._lock:
            entry = self._pending.pop(op_id, None)
        work = args.work
        if entry is None or work is None:
            return
        name, nbytes = entry
        started: List[float] = []

        def on_start() -> None:
            started.append(time.perf_counter())

        def on_end() -> None:
            now = time.perf_counter()
            dt = now - started[0] if started else 0.0
            with self._lock:
                st = self._ops.setdefault(name, _OpStats())
                st.completed += 1
                st.completed_bytes += nbytes
                st.busy_s += dt
                st.max_s = max(st.max_s, dt)

        work.register_start_hook(on_start)
        work.register_end_hook(on_end)

    # ------------------------------------------------------------------ export
    def snapshot(self) -> Dict[str, Dict[str, Any]]:
        out: Dict[str, Dict[str, Any]] = {}
        with self._lock:
            for name, st in self._ops.items():
                out[name] = {
                    "calls": st.calls,
                    "bytes": st.bytes,
                    "async_calls": st.async_calls,
                    "completed": st.completed,
                    "busy_ms": st.busy_s * 1e3,
                    "max_ms": st.max_s * 1e3,
                    "gbps": (st.completed_bytes / st.busy_s / 1e9) if st.busy_s > 0 else 0.0,
                    "size_histogram": dict(st.hist),
                }
        return out

    def reset(self) -> None:
        with self._lock:
            self._ops.clear()
            self._pending.clear()

    def report(self) -> str:
        """A fixed-width table of ``snapshot()``, largest byte count first."""
        snap = self.snapshot()
        lines = [f"{'operation':<24}{'calls':>8}{'MiB':>12}{'busy ms':>10}{'max ms':>9}{'GB/s':>8}"]
        for name, s in sorted(snap.items(), key=lambda kv: -kv[1]["bytes"]):
            lines.append(f"{name:<24}{s['calls']:>8}{s['bytes'] / 2**20:>12.1f}{s['busy_ms']:>10.2f}{s['max_ms']:>9.2f}{s['gbps']:>8.1f}")
        return "\n".join(lines)
