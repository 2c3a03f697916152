"""Elastic membership on the CUDA backend: the communicator is created without a membership,
formed by ``reconfigure``, used, re-formed under a new id (everything bootstrap created is
released and built again: symmetric heap, peer mappings, flags, streams, watchdog), used again.
One member on a single GPU; with two GPUs a member leaves between steps, the other carries on
alone, and both re-form with swapped ranks.
Modelled on comms/torchcomms/tests/integration/py/ReconfigureTest.py (fresh init, identity,
shrink and grow cases); failures of a member are covered on the gloo backend in
test_gloo_failures.py."""
from datetime import timedelta

import pytest
import torch

pytestmark = pytest.mark.gpu


def test_single_member_reconfigure_cycles():
    import torch.distributed as dist

    import torchcomms_b200 as tc

    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    store = dist.HashStore()
    comm = tc.new_comm("b200", dev, name="elastic_single", store=store, enable_reconfigure=True,
                       timeout=timedelta(seconds=30), abort_process_on_timeout_or_error=False, hints={"use_nccl": "0"})
    handle = comm.get_init_handle()
    parts = handle.split(":")
    assert parts[0] == "b200" and len(parts) >= 4
    with pytest.raises(RuntimeError):
        comm.all_reduce(torch.ones(4, device=dev), tc.ReduceOp.SUM, False)      # no membership yet
    with pytest.raises(RuntimeError):
        comm.reconfigure(1, ["b200:0:someone:else:1"], timeout=timedelta(seconds=5))
    for uuid, handles in ((1, [handle]), (2, {handle}), (3, [handle])):
        comm.reconfigure(uuid, handles, timeout=timedelta(seconds=30))
        assert comm.get_size() == 1 and comm.get_rank() == 0
        t = torch.full((4096,), float(uuid), device=dev)
        comm.all_reduce(t, tc.ReduceOp.SUM, False)
        out = torch.empty(4096, device=dev)
        comm.all_gather_single(out, t, True).wait()
        comm.barrier(False)
        torch.cuda.synchronize()
        assert torch.equal(t, torch.full((4096,), float(uuid), device=dev)) and torch.equal(out, t)
        assert comm.comm_dump()["size"] == "1"
    comm.finalize()
    with pytest.raises(RuntimeError):
        comm.reconfigure(4, [handle])


def test_unformed_communicator_finalizes_cleanly():
    import torch.distributed as dist

    import torchcomms_b200 as tc

    comm = tc.new_comm("b200", torch.device("cuda", 0), name="elastic_unformed", store=dist.HashStore(),
                       enable_reconfigure=True, timeout=timedelta(seconds=10), abort_process_on_timeout_or_error=False)
    assert comm.get_init_handle().startswith("b200:")
    comm.finalize()


def _shrink_grow_worker(rank, world):
    """Two members form a communicator; rank 1 leaves between steps (nothing of its own in flight, the others told
    through the store); rank 0 re-forms alone, works, and then both re-form together under a new id."""
    import os

    import torch.distributed as dist

    import torchcomms_b200 as tc

    dev = torch.device("cuda", rank)
    torch.cuda.set_device(dev)
    store = dist.TCPStore("127.0.0.1", int(os.environ["MASTER_PORT"]) + 1, world, rank == 0, timeout=timedelta(seconds=60))
    # Plain peer loads and stores only: no multicast binding and no NCCL communicator that a leaving rank could strand.
    comm = tc.new_comm("b200", dev, name="elastic2", store=store, enable_reconfigure=True, timeout=timedelta(seconds=30),
                       abort_process_on_timeout_or_error=False, hints={"use_multicast": "0", "use_nccl": "0"})
    store.set(f"h/{rank}", comm.get_init_handle())
    handles = [store.get(f"h/{r}").decode() for r in range(world)]

    def check_sum(expected):
        t = torch.full((4096,), float(rank + 1), device=dev)
        comm.all_reduce(t, tc.ReduceOp.SUM, False)
        out = torch.empty(4096 * comm.get_size(), device=dev)
        comm.all_gather_single(out, t, False)
        torch.cuda.synchronize()
        assert torch.equal(t, torch.full((4096,), expected, device=dev))
        assert torch.equal(out, torch.full((4096 * comm.get_size(),), expected, device=dev))

    comm.reconfigure(1, handles, timeout=timedelta(seconds=30))
    assert comm.get_size() == 2 and comm.get_rank() == rank
    check_sum(3.0)
    if rank == 1:
        store.set("left", "1")                       # leaves between steps
        store.wait(["rejoin"], timedelta(seconds=60))
    else:
        store.wait(["left"], timedelta(seconds=60))
        comm.reconfigure(2, handles[:1], timeout=timedelta(seconds=30))
        assert comm.get_size() == 1 and comm.get_rank() == 0
        check_sum(1.0)
        store.set("rejoin", "1")
    comm.reconfigure(3, list(reversed(handles)), timeout=timedelta(seconds=30))   # ranks follow the list: swapped
    assert comm.get_size() == 2 and comm.get_rank() == 1 - rank
    check_sum(3.0)
    comm.finalize()


def test_two_members_shrink_and_grow():
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    from tests.mp_util import run_ranks

    run_ranks(_shrink_grow_worker, 2, timeout=150, extra_env={"NCCL_NVLS_ENABLE": "0", "B200COMMS_NVLS": "0"})
