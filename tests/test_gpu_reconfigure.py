"""Elastic membership on the CUDA backend, single member: the communicator is created without
a membership, formed by ``reconfigure``, used, re-formed under a new id (everything bootstrap
created is released and built again: symmetric heap, flags, streams, watchdog), used again.
Modelled on comms/torchcomms/tests/integration/py/ReconfigureTest.py (fresh init and identity
cases); leaving and joining ranks are covered on the gloo backend in test_gloo_failures.py."""
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
