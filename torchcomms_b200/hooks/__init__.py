"""Hooks that attach to a communicator: flight recorder, collective log, NaN check, per-operation counters.

    from torchcomms_b200.hooks import NanCheckHook, fr, clog
    NanCheckHook().register_with_comm(comm)
    rec = fr.FlightRecorderHook(); rec.register_with_comm(comm)

``python -m torchcomms_b200.hooks.fr_analyze <dump files>`` lines the ranks' recorder dumps up and names
the first collective on which they disagree.  ``fr`` and ``clog`` are the native recorders (ring buffer in the c10d
flight-recorder JSON layout; pipe-delimited collective log with graph
capture / replay lines).  Parity: comms/torchcomms/hooks/__init__.py,
hooks/fr/FlightRecorderHook.hpp:43-146, hooks/clog/ClogHook.hpp:118-279,
hooks/nan_check/nan_check.py:117-185.
"""
from .._comms import hooks as _native
from .nan_check import NanCheckHook
from .chaos import ChecksumHook, DelayInjectionHook
from .stats import CommStatsHook

fr = _native.fr
FlightRecorderHook = _native.fr.FlightRecorderHook
ClogHook = _native.clog.ClogHook


class _Clog:
    """``hooks.clog``: the namespace of the native collective log (``clog.ClogHook(path)``), and - the reference's
    spelling - a constructor: ``clog(output="/tmp/clog.log", events=["ALL"])``.  Every event kind is always
    written (queued, started, ended, waited, graph capture and replay lines), so ``events`` and ``verbose`` only
    have to be well-formed; a reader that wants fewer kinds filters on the first column."""

    ClogHook = _native.clog.ClogHook
    EVENTS = ("ALL", "Q", "S", "E", "W", "G")

    def __call__(self, output: str = "", events=("ALL",), verbose=()):
        bad = [e for e in events if str(e).upper() not in self.EVENTS]
        if bad:
            raise ValueError(f"unknown clog events {bad} (expected some of {list(self.EVENTS)})")
        return _native.clog.ClogHook(output)

    def __getattr__(self, name):
        return getattr(_native.clog, name)


clog = _Clog()

__all__ = ["NanCheckHook", "CommStatsHook", "DelayInjectionHook", "ChecksumHook", "FlightRecorderHook", "ClogHook", "fr", "clog"]
