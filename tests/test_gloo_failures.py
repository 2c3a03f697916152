"""Failure detection and elastic recovery on CPU (gloo) ranks: every failure is
made on the host - a rank that joins late, a rank that leaves between steps -
and nothing here touches a GPU.

Modelled on comms/torchcomms/tests/integration/py/TimeoutTest.py:24-90,
AbortTest.py and ReconfigureTest.py (which re-execute themselves in
sub-processes; here every rank already is a child process).
"""
import os
import time
from datetime import timedelta

import pytest
import torch

from tests.mp_util import run_ranks


def _leave():
    import sys

    sys.stdout.flush()
    sys.stderr.flush()
    os._exit(0)


def _late_rank_worker(rank, world):
    import torchcomms_b200 as tc

    comm = tc.new_comm("gloo", torch.device("cpu"), name="late", timeout=timedelta(seconds=60),
                       abort_process_on_timeout_or_error=False)
    aborted = []
    comm.register_abort_hook(lambda: aborted.append(True))
    t = torch.ones(4)
    comm.all_reduce(t, tc.ReduceOp.SUM, False)          # everybody is here: fine
    assert tc.healthy()
    if rank == 0:
        time.sleep(6.0)                                  # the straggler: joins long after the others gave up
        with pytest.raises(RuntimeError):
            comm.all_reduce(torch.ones(4), tc.ReduceOp.SUM, False, timeout=timedelta(seconds=2))
    else:
        t0 = time.time()
        with pytest.raises(RuntimeError, match="(?i)time|abort|fail"):
            comm.all_reduce(torch.ones(4), tc.ReduceOp.SUM, False, timeout=timedelta(seconds=2))
        waited = time.time() - t0
        assert 1.0 < waited < 30.0, waited                # bounded by the per-call timeout, not by the straggler
        assert not tc.healthy()                          # the process-wide flag the health endpoint reports
        # the communicator refuses further work instead of hanging on a half-broken group
        with pytest.raises(RuntimeError):
            comm.all_reduce(torch.ones(4), tc.ReduceOp.SUM, False)
    # A failed communicator is not finalized. Its transport threads may still sit in the collective
    # that never completed and cannot be cancelled, so the rank ends the way a trainer would after a
    # fatal communication error: abort, then leave without running static destructors under them.
    comm.abort()
    _leave()


def test_late_rank_times_out_without_hanging():
    run_ranks(_late_rank_worker, 3, timeout=120)


def _async_timeout_worker(rank, world):
    import torchcomms_b200 as tc

    comm = tc.new_comm("gloo", torch.device("cpu"), name="async_to", timeout=timedelta(seconds=60),
                       abort_process_on_timeout_or_error=False)
    if rank == 0:
        time.sleep(5.0)
        _leave()
    w = comm.all_reduce(torch.ones(2), tc.ReduceOp.SUM, True, timeout=timedelta(seconds=1))
    with pytest.raises(RuntimeError):
        w.wait()
    assert w.status() in (tc.WorkStatus.TIMEDOUT, tc.WorkStatus.ERROR)
    comm.abort()
    _leave()


def test_async_work_reports_timeout():
    run_ranks(_async_timeout_worker, 2, timeout=120)


def _elastic_worker(rank, world):
    """Three candidates share a store; the first membership is all three, then rank 2 leaves between
    steps (cleanly, nothing in flight) and the survivors reconfigure to a world of two."""
    import torch.distributed as dist

    import torchcomms_b200 as tc

    store = dist.TCPStore("127.0.0.1", int(os.environ["MASTER_PORT"]) + 1, world, rank == 0,
                          timeout=timedelta(seconds=60))
    comm = tc.new_comm("gloo", torch.device("cpu"), name="elastic", store=store, enable_reconfigure=True,
                       timeout=timedelta(seconds=30), abort_process_on_timeout_or_error=False)
    me = comm.get_init_handle()
    store.set(f"handle/{rank}", me)
    handles = [store.get(f"handle/{r}").decode() for r in range(world)]
    comm.reconfigure(1, handles, timeout=timedelta(seconds=30))
    assert comm.get_size() == world and comm.get_rank() == rank
    t = torch.full((4,), float(rank + 1))
    comm.all_reduce(t, tc.ReduceOp.SUM, False)
    assert torch.equal(t, torch.full((4,), 6.0))
    if rank == 2:
        store.set("left/2", "1")                         # tells the others on the host, then goes away
        return
    store.wait(["left/2"])
    comm.reconfigure(2, handles[:2], timeout=timedelta(seconds=30))
    assert comm.get_size() == 2 and comm.get_rank() == rank
    t = torch.full((4,), float(rank + 1))
    comm.all_reduce(t, tc.ReduceOp.SUM, False)
    assert torch.equal(t, torch.full((4,), 3.0))
    # a set of handles (no order given) sorts them: both survivors agree without exchanging ranks
    comm.reconfigure(3, set(handles[:2]), timeout=timedelta(seconds=30))
    assert comm.get_size() == 2
    got = torch.empty(2)
    comm.all_gather_single(got, torch.full((1,), float(comm.get_rank())), False)
    assert torch.equal(got, torch.tensor([0.0, 1.0]))
    comm.finalize()


def test_elastic_reconfigure_after_a_rank_leaves():
    run_ranks(_elastic_worker, 3, timeout=120)


def _abort_worker(rank, world):
    import torchcomms_b200 as tc

    comm = tc.new_comm("gloo", torch.device("cpu"), name="abort", timeout=timedelta(seconds=30),
                       abort_process_on_timeout_or_error=False)
    fired = []
    comm.register_abort_hook(lambda: fired.append("abort"))
    comm.barrier(False)
    assert comm.is_abort_supported() and not comm.is_aborted()
    comm.abort()
    assert comm.is_aborted() and fired == ["abort"]
    with pytest.raises(RuntimeError, match="abort"):
        comm.all_reduce(torch.ones(2), tc.ReduceOp.SUM, False)


def test_abort_runs_hooks_and_blocks_further_work():
    run_ranks(_abort_worker, 2, timeout=120)
