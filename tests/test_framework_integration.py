"""PyTorch's own parallel wrappers running over this framework's communicators (gloo ranks
on CPU): DistributedDataParallel, FSDP2 ``fully_shard`` and DTensor tensor parallelism on a
DeviceMesh built from communicators.

Modelled on comms/torchcomms/tests/integration/py/DDPCommTest.py, FSDPCommTest.py:16-66,
TPCommTest.py:71 and DPTPCommTest.py (2-D mesh).
"""
from datetime import timedelta

import torch

from tests.mp_util import run_ranks


def _mlp(seed):
    torch.manual_seed(seed)
    return torch.nn.Sequential(torch.nn.Linear(16, 32), torch.nn.ReLU(), torch.nn.Linear(32, 8))


def _single_process_reference(world, steps, lr):
    """The same training on one process over the concatenated batch (mean loss over ranks)."""
    model = _mlp(0)
    opt = torch.optim.SGD(model.parameters(), lr=lr)
    for step in range(steps):
        opt.zero_grad()
        loss = sum(model(_batch(r, step)).pow(2).mean() for r in range(world)) / world
        loss.backward()
        opt.step()
    return [p.detach().clone() for p in model.parameters()]


def _batch(rank, step):
    g = torch.Generator().manual_seed(100 * step + rank)
    return torch.randn(4, 16, generator=g)


def _ddp_worker(rank, world):
    from torch.nn.parallel import DistributedDataParallel as DDP

    import torchcomms_b200 as tc
    from torchcomms_b200.device_mesh import init_device_mesh

    comm = tc.new_comm("gloo", torch.device("cpu"), name="ddp", timeout=timedelta(seconds=60))
    mesh = init_device_mesh(mesh_dim_comms=(comm,), mesh_dim_names=("dp",))
    model = DDP(_mlp(rank), process_group=mesh.get_group("dp"), bucket_cap_mb=0.001)   # rank 0's weights are broadcast
    opt = torch.optim.SGD(model.parameters(), lr=0.1)
    for step in range(3):
        opt.zero_grad()
        model(_batch(rank, step)).pow(2).mean().backward()
        opt.step()
    for p, ref in zip(model.module.parameters(), _single_process_reference(world, 3, 0.1)):
        torch.testing.assert_close(p.detach(), ref, rtol=1e-5, atol=1e-6)
    comm.finalize()


def test_ddp_over_device_mesh_process_group():
    run_ranks(_ddp_worker, 2, timeout=90)


def _fsdp_worker(rank, world):
    from torch.distributed.fsdp import fully_shard

    import torchcomms_b200 as tc
    from torchcomms_b200.device_mesh import init_device_mesh

    comm = tc.new_comm("gloo", torch.device("cpu"), name="fsdp", timeout=timedelta(seconds=60))
    mesh = init_device_mesh(mesh_dim_comms=(comm,), mesh_dim_names=("dp",))
    model = _mlp(0)
    for layer in model:
        if isinstance(layer, torch.nn.Linear):
            fully_shard(layer, mesh=mesh)
    fully_shard(model, mesh=mesh)
    opt = torch.optim.SGD(model.parameters(), lr=0.1)
    for step in range(3):
        opt.zero_grad()
        model(_batch(rank, step)).pow(2).mean().backward()
        opt.step()
    for p, ref in zip(model.parameters(), _single_process_reference(world, 3, 0.1)):
        torch.testing.assert_close(p.full_tensor().detach(), ref, rtol=1e-5, atol=1e-6)
    comm.finalize()


def test_fsdp2_fully_shard_over_device_mesh():
    run_ranks(_fsdp_worker, 2, timeout=90)


def _tp_worker(rank, world):
    from torch.distributed.tensor.parallel import ColwiseParallel, RowwiseParallel, parallelize_module

    import torchcomms_b200 as tc
    from torchcomms_b200.device_mesh import init_device_mesh

    comm = tc.new_comm("gloo", torch.device("cpu"), name="tp", timeout=timedelta(seconds=60))
    mesh = init_device_mesh(mesh_dim_comms=(comm,), mesh_dim_names=("tp",))
    ref_model = _mlp(0)
    model = _mlp(0)
    parallelize_module(model, mesh, {"0": ColwiseParallel(), "2": RowwiseParallel()})
    x = _batch(0, 0)                                           # replicated input
    out = model(x)
    torch.testing.assert_close(out, ref_model(x), rtol=1e-5, atol=1e-5)
    out.pow(2).mean().backward()
    ref_model(x).pow(2).mean().backward()
    got = model[0].weight.grad.full_tensor()
    torch.testing.assert_close(got, ref_model[0].weight.grad, rtol=1e-5, atol=1e-6)
    comm.finalize()


def test_dtensor_tensor_parallel_over_device_mesh():
    run_ranks(_tp_worker, 2, timeout=90)


def _dp_tp_worker(rank, world):
    """2-D mesh: dp = 2 x tp = 2 from two communicators obtained by split."""
    from torch.distributed.tensor.parallel import ColwiseParallel, RowwiseParallel, parallelize_module
    from torch.nn.parallel import DistributedDataParallel as DDP

    import torchcomms_b200 as tc
    from torchcomms_b200.device_mesh import init_device_mesh

    comm = tc.new_comm("gloo", torch.device("cpu"), name="world", timeout=timedelta(seconds=60))
    dp_idx, tp_idx = rank // 2, rank % 2
    tp_comm = None
    for d in range(2):                                         # every rank takes part in every split
        c = comm.split([2 * d, 2 * d + 1] if d == dp_idx else [], f"tp{d}")
        tp_comm = c if c is not None else tp_comm
    dp_comm = None
    for t in range(2):
        c = comm.split([t, t + 2] if t == tp_idx else [], f"dp{t}")
        dp_comm = c if c is not None else dp_comm
    assert tp_comm.get_size() == 2 and dp_comm.get_size() == 2
    mesh = init_device_mesh(mesh_dim_comms=(dp_comm, tp_comm), mesh_dim_names=("dp", "tp"), _global_comm=comm)
    assert mesh.get_local_rank("dp") == dp_idx and mesh.get_local_rank("tp") == tp_idx
    model = _mlp(0)
    parallelize_module(model, mesh["tp"], {"0": ColwiseParallel(), "2": RowwiseParallel()})
    x = _batch(dp_idx, 0)                                      # each data-parallel replica sees its own batch
    out = model(x)
    torch.testing.assert_close(out, _mlp(0)(x), rtol=1e-5, atol=1e-5)
    # gradients averaged over the data-parallel dimension by hand through the mesh's group
    out.pow(2).mean().backward()
    import torch.distributed as dist

    g = model[2].bias.grad
    g = g.full_tensor() if hasattr(g, "full_tensor") else g
    g = g.clone()
    dist.all_reduce(g, group=mesh.get_group("dp"))
    ref = _mlp(0)
    (sum(ref(_batch(d, 0)).pow(2).mean() for d in range(2))).backward()
    torch.testing.assert_close(g, ref[2].bias.grad, rtol=1e-5, atol=1e-6)
    # the two dimensions flattened onto the world communicator give a 1-D mesh whose group spans all ranks
    from torchcomms_b200.device_mesh import _flatten_with_comm

    flat = _flatten_with_comm(mesh, "dp_tp", comm, list(range(world)))
    assert flat.ndim == 1 and flat.size() == world
    t = torch.full((2,), float(rank))
    dist.all_reduce(t, group=flat.get_group("dp_tp"))
    assert torch.equal(t, torch.full((2,), float(sum(range(world)))))
    for c in (tp_comm, dp_comm, comm):
        c.finalize()


def test_two_dimensional_mesh_dp_by_tp():
    run_ranks(_dp_tp_worker, 4, timeout=120)


def _dcp_worker(rank, world, path):
    """torch.distributed.checkpoint over the adapter: sharded save, load into a fresh model."""
    import torch.distributed.checkpoint as dcp
    from torch.distributed.fsdp import fully_shard

    import torchcomms_b200 as tc
    from torchcomms_b200.device_mesh import init_device_mesh

    comm = tc.new_comm("gloo", torch.device("cpu"), name="dcp", timeout=timedelta(seconds=60))
    mesh = init_device_mesh(mesh_dim_comms=(comm,), mesh_dim_names=("dp",))
    pg = mesh.get_group("dp")
    model = _mlp(0)
    fully_shard(model, mesh=mesh)
    dcp.save({"model": model.state_dict(), "step": torch.tensor(7)}, checkpoint_id=path, process_group=pg)
    fresh = _mlp(1)
    fully_shard(fresh, mesh=mesh)
    state = {"model": fresh.state_dict(), "step": torch.tensor(0)}
    dcp.load(state, checkpoint_id=path, process_group=pg)
    fresh.load_state_dict(state["model"])
    for a, b in zip(model.parameters(), fresh.parameters()):
        assert torch.equal(a.full_tensor(), b.full_tensor())
    assert int(state["step"]) == 7
    comm.finalize()


def test_distributed_checkpoint_save_and_load(tmp_path):
    run_ranks(_dcp_worker, 2, args=(str(tmp_path / "ckpt"),), timeout=120)


def _split_mesh_worker(rank, world):
    import torch.distributed as dist

    import torchcomms_b200 as tc
    from torchcomms_b200.parallel.mesh import device_mesh_from_world, mesh_coordinates, mesh_groups, split_mesh

    assert mesh_groups((2, 2), 0) == [[0, 2], [1, 3]] and mesh_groups((2, 2), 1) == [[0, 1], [2, 3]]
    assert mesh_coordinates(3, (2, 2)) == [1, 1]
    comm = tc.new_comm("gloo", torch.device("cpu"), name="world", timeout=timedelta(seconds=60))
    comms = split_mesh(comm, (2, 2), ("dp", "tp"))
    dp_idx, tp_idx = mesh_coordinates(rank, (2, 2))
    assert comms["dp"].get_size() == 2 and comms["dp"].get_rank() == dp_idx
    assert comms["tp"].get_size() == 2 and comms["tp"].get_rank() == tp_idx
    t = torch.tensor([float(rank)])
    comms["tp"].all_reduce(t, tc.ReduceOp.SUM, False)          # ranks {0,1} and {2,3}
    assert t.item() == float(4 * dp_idx + 1)
    t = torch.tensor([float(rank)])
    comms["dp"].all_reduce(t, tc.ReduceOp.SUM, False)          # ranks {0,2} and {1,3}
    assert t.item() == float(2 * tp_idx + 2)
    for c in comms.values():
        c.finalize()
    mesh = device_mesh_from_world(comm, (2, 2), ("dp", "tp"))
    assert mesh.get_local_rank("dp") == dp_idx and mesh.get_local_rank("tp") == tp_idx
    u = torch.tensor([1.0])
    dist.all_reduce(u, group=mesh.get_group("tp"))
    assert u.item() == 2.0
    import pytest

    with pytest.raises(ValueError):
        split_mesh(comm, (3, 2), ("a", "b"))
    for c in mesh._b200c_comms.values():
        c.finalize()
    comm.finalize()


def test_split_mesh_helpers():
    run_ranks(_split_mesh_worker, 4, timeout=120)
