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
clog = _native.clog

__all__ = ["NanCheckHook", "CommStatsHook", "DelayInjectionHook", "ChecksumHook", "fr", "clog"]
