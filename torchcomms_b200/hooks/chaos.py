"""Debugging hooks that shake out ordering bugs and replica divergence.

``DelayInjectionHook`` sleeps a pseudo-random time on the host before selected
operations of selected ranks, so that ranks arrive at collectives in a
different order every run; a protocol that only works when the ranks are in
lock step (a flag consumed from the wrong epoch, a staging slot overwritten
early) then fails in a test instead of once a week in production::

    DelayInjectionHook(max_ms=5, seed=rank, probability=0.3).register_with_comm(comm)

``ChecksumHook`` records a checksum of what every operation read and, once the
operation completed, of what it wrote.  After a replicating collective
(all-reduce, broadcast, all-gather) every rank must hold the same output, so
comparing the records of the ranks (``records()`` through
``objcol.all_gather_object``, or ``divergence(all_records)``) names the first
operation whose result differs::

    chk = ChecksumHook(); chk.register_with_comm(comm)
    ...
    bad = ChecksumHook.divergence(objcol_all_gather(chk.records()))

Both are host-side: nothing is injected into kernels.  Parity: the reference has
no sanitizer integration; its aids are device checksums inside ctran
(comms/ctran/algos/common/Checksum.cuh) and sleeps in test ranks
(comms/torchcomms/tests/integration/py/TimeoutTest.py:24-90).
"""
from __future__ import annotations

import random
import threading
import time
from typing import Any, Dict, Iterable, List, Optional, Sequence, Tuple

import torch

from .._comms import OpName

# Operations after which every rank holds identical output.
REPLICATING = frozenset({"all_reduce", "broadcast", "all_gather", "all_gather_single", "all_gather_v"})


def _names(ops: Optional[Iterable[Any]]) -> Optional[frozenset]:
    if ops is None:
        return None
    return frozenset(o.name if isinstance(o, OpName) else str(o) for o in ops)


class DelayInjectionHook:
    """Sleeps up to ``max_ms`` before an operation with the given probability."""

    def __init__(self, max_ms: float = 2.0, seed: int = 0, probability: float = 1.0,
                 ops: Optional[Iterable[Any]] = None, ranks: Optional[Sequence[int]] = None):
        self._max_s = max_ms / 1e3
        self._rng = random.Random(seed)
        self._p = probability
        self._ops = _names(ops)
        self._ranks = None if ranks is None else frozenset(ranks)
        self._handles: List[Any] = []
        self._lock = threading.Lock()
        self.injected: List[Tuple[int, str, float]] = []      # (op id, operation, seconds slept)

    def register_with_comm(self, comm: Any) -> None:
        if self._ranks is not None and comm.get_rank() not in self._ranks:
            return

        def delay(op: OpName, op_id: int, args: Any) -> None:
            if self._ops is not None and op.name not in self._ops:
                return
            with self._lock:
                if self._rng.random() >= self._p:
                    return
                dt = self._rng.random() * self._max_s
                self.injected.append((op_id, op.name, dt))
            time.sleep(dt)

        self._handles.append(comm.register_pre_hook(delay))

    def unregister(self) -> None:
        while self._handles:
            self._handles.pop().remove()

    def is_enabled(self) -> bool:
        return bool(self._handles)


def _checksum(tensors: Iterable[torch.Tensor]) -> int:
    """Order-dependent 64-bit checksum of the tensors' bytes (reads them back to the host)."""
    total = 0
    for t in tensors:
        if not isinstance(t, torch.Tensor) or t.numel() == 0:
            continue
        raw = t.detach().contiguous().view(torch.uint8).to("cpu", torch.int64)
        weights = (torch.arange(raw.numel(), dtype=torch.int64) % 251) + 1
        total = (total * 1000003 + int((raw * weights).sum())) & 0xFFFFFFFFFFFFFFFF
    return total


class ChecksumHook:
    """Records ``(sequence number, operation, input checksum, output checksum)`` per operation."""

    def __init__(self, ops: Optional[Iterable[Any]] = None):
        self._ops = _names(ops)
        self._lock = threading.Lock()
        self._records: List[Dict[str, Any]] = []
        self._pending: Dict[int, Dict[str, Any]] = {}
        self._handles: List[Any] = []

    def register_with_comm(self, comm: Any) -> None:
        self._handles.append(comm.register_pre_hook(self._pre))
        self._handles.append(comm.register_post_hook(self._post))

    def unregister(self) -> None:
        while self._handles:
            self._handles.pop().remove()

    def is_enabled(self) -> bool:
        return bool(self._handles)

    def _pre(self, op: OpName, op_id: int, args: Any) -> None:
        if self._ops is not None and op.name not in self._ops:
            return
        rec = args.record
        outputs = list(rec.outputs) or list(rec.inputs)        # in-place operations write their input
        entry = {"seq": None, "op": op.name, "in": _checksum(list(rec.inputs)), "out": None, "_outputs": outputs}
        with self._lock:
            entry["seq"] = len(self._records)
            self._records.append(entry)
            self._pending[op_id] = entry

    def _post(self, op_id: int, args: Any) -> None:
        with self._lock:
            entry = self._pending.pop(op_id, None)
        work = args.work
        if entry is None:
            return

        def finish() -> None:
            outputs = entry.pop("_outputs", [])
            if any(t.is_cuda for t in outputs):
                torch.cuda.synchronize()                        # the end hook fires from the watchdog thread
            entry["out"] = _checksum(outputs)

        if work is None:
            finish()
        else:
            work.register_end_hook(finish)

    def records(self) -> List[Dict[str, Any]]:
        """Completed records, in issue order (picklable)."""
        with self._lock:
            return [{k: v for k, v in r.items() if not k.startswith("_")} for r in self._records if r["out"] is not None]

    @staticmethod
    def divergence(per_rank: Sequence[List[Dict[str, Any]]]) -> Optional[Dict[str, Any]]:
        """First replicating operation whose output checksum differs between ranks, or whose sequence
        of operations differs; ``None`` when all ranks agree."""
        if not per_rank:
            return None
        for seq in range(min(len(r) for r in per_rank)):
            ops = {r[seq]["op"] for r in per_rank}
            if len(ops) > 1:
                return {"seq": seq, "reason": "operation mismatch", "ops": sorted(ops)}
            op = next(iter(ops))
            outs = [r[seq]["out"] for r in per_rank]
            if op in REPLICATING and len(set(outs)) > 1:
                return {"seq": seq, "reason": "output mismatch", "op": op, "checksums": outs}
        lengths = {len(r) for r in per_rank}
        if len(lengths) > 1:
            return {"seq": min(lengths), "reason": "operation count mismatch", "counts": [len(r) for r in per_rank]}
        return None
