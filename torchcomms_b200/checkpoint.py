"""Communicator-aware process checkpoints.

A process that is to be checkpointed and restored as a whole (CUDA checkpoint
plus CRIU, or a move to another box) must hold no GPU state that it shares with
other processes: no peer mappings, no multicast bindings, no NCCL communicator.
``checkpoint_prepare`` takes those down for the given communicators and keeps
what identifies them (rank, size, name, options, hooks); ``checkpoint_restore``
builds them again among the same members, so the application carries on with
the communicator objects it had::

    from torchcomms_b200.checkpoint import checkpoint_prepare, checkpoint_restore

    checkpoint_prepare([dp_comm, tp_comm])      # collective, same order on every rank
    ...                                          # lock / checkpoint / dump / restore / unlock the process
    checkpoint_restore([dp_comm, tp_comm])      # collective

Tensors from ``symm_empty``, windows and fused layers hold symmetric memory of
the old mappings and must be created again after the restore, as after
``reconfigure``.  Backends without cross-process GPU state (gloo, fake) are left
alone.  The store that the communicators were created with must still be
reachable at restore time (it carries the new rendezvous).

Counterpart in the reference tree: comms/ncclx/v2_31/contrib/nccl_checkpoint
(``nccl_checkpoint.checkpoint_prepare`` / ``checkpoint_restore``), a preloaded
shim that records every NCCL set-up call and replays it after the restore; here
the backend owns its set-up and can simply run it again.
"""
from __future__ import annotations

from typing import Iterable, List

from . import TorchComm


def _suspendable(comm: TorchComm):
    impl = comm.get_backend_impl()
    return impl if hasattr(impl, "suspend") and hasattr(impl, "resume") else None


def checkpoint_prepare(comms: Iterable[TorchComm]) -> List[TorchComm]:
    """Suspends every communicator of ``comms`` that holds cross-process GPU state; returns those it suspended."""
    done = []
    for comm in comms:
        impl = _suspendable(comm)
        if impl is not None and not impl.is_suspended():
            impl.suspend()
            done.append(comm)
    return done


def checkpoint_restore(comms: Iterable[TorchComm]) -> List[TorchComm]:
    """Resumes every suspended communicator of ``comms``; returns those it resumed."""
    done = []
    for comm in comms:
        impl = _suspendable(comm)
        if impl is not None and impl.is_suspended():
            impl.resume()
            done.append(comm)
    return done


__all__ = ["checkpoint_prepare", "checkpoint_restore"]
