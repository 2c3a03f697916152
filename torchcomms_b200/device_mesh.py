"""Builds a ``torch.distributed.DeviceMesh`` whose dimensions are communicators.

Each mesh dimension gets a bare ``ProcessGroup`` whose only backend is the
c10d adapter around one ``TorchComm``; the group is entered into the c10d world
tables so ``fully_shard``, DTensor, ``ColwiseParallel`` and plain
``torch.distributed`` calls (including the object collectives that
state-dict / checkpoint code uses) run on the communicator without changes.

Parity: ``comms/torchcomms/device_mesh.py:38-97`` (group registration),
``:100-173`` (``init_device_mesh``), ``:176-245`` (``_flatten_with_comm``).
"""
from __future__ import annotations

import math
from typing import Dict, Optional, Sequence

import torch
import torch.distributed as dist
from torch.distributed import distributed_c10d as c10d

from . import TorchComm, _BackendWrapper, new_comm

BACKEND_TAG = "torchcomm"

_wrappers: Dict[str, _BackendWrapper] = {}


def _ensure_backend_tag() -> None:
    if BACKEND_TAG.upper() not in dist.Backend.backend_list and BACKEND_TAG not in dist.Backend.backend_list:
        dist.Backend.register_backend(BACKEND_TAG, new_comm)


def wrap_comm_as_process_group(
    comm: TorchComm,
    group_name: str,
    global_to_group_rank: Optional[Dict[int, int]] = None,
) -> dist.ProcessGroup:
    """Registers ``comm`` with torch.distributed under ``group_name``.

    ``global_to_group_rank`` maps world ranks to ranks inside this group; by
    default the communicator is taken to span ranks ``0..size-1``.
    """
    _ensure_backend_tag()
    world = c10d._world
    adapter = _BackendWrapper(comm)
    # The communicator does its own bootstrap; the group's store only has to
    # satisfy the ProcessGroup constructor.
    placeholder_store = dist.HashStore()
    pg = dist.ProcessGroup(placeholder_store, comm.get_rank(), comm.get_size())
    pg._register_backend(comm.get_device(), dist.ProcessGroup.BackendType.CUSTOM, adapter)
    if comm.get_device().type != "cpu":
        # Object collectives stage through CPU tensors; serve them with the same adapter.
        pg._register_backend(torch.device("cpu"), dist.ProcessGroup.BackendType.CUSTOM, adapter)
    pg._set_group_name(group_name)
    pg._set_default_backend(dist.ProcessGroup.BackendType.CUSTOM)

    ranks = global_to_group_rank or {r: r for r in range(comm.get_size())}
    world.pg_map[pg] = (BACKEND_TAG, placeholder_store)
    world.pg_names[pg] = group_name
    world.pg_backend_config[pg] = str(dist.BackendConfig(dist.Backend(BACKEND_TAG)))
    world.pg_group_ranks[pg] = dict(ranks)
    tag = f"ptd:{group_name}"
    world.tags_to_pg.setdefault(tag, []).append(pg)
    world.pg_to_tag[pg] = tag
    c10d._register_process_group(group_name, pg)
    _wrappers[group_name] = adapter
    return pg


def _members_along(mesh: torch.Tensor, dim: int, global_rank: int) -> list[int]:
    """World ranks that share every coordinate with ``global_rank`` except ``dim``."""
    lines = mesh.movedim(dim, -1).reshape(-1, mesh.size(dim))
    row = (lines == global_rank).any(dim=1).nonzero()[0, 0]
    return [int(x) for x in lines[row].tolist()]


def init_device_mesh(
    mesh_dim_comms: Sequence[TorchComm],
    mesh_dim_names: Sequence[str],
    _global_comm: Optional[TorchComm] = None,
) -> dist.DeviceMesh:
    """One communicator per mesh dimension (row-major rank layout).

    With more than one dimension a communicator over all ranks must be given as
    ``_global_comm``; it becomes the default (WORLD) group.
    """
    if len(mesh_dim_comms) != len(mesh_dim_names):
        raise ValueError("mesh_dim_comms and mesh_dim_names must have the same length")
    if len(mesh_dim_comms) > 1 and _global_comm is None:
        raise RuntimeError(
            "a multi-dimensional mesh needs a communicator spanning all ranks (_global_comm)"
        )
    shape = tuple(c.get_size() for c in mesh_dim_comms)
    mesh = torch.arange(math.prod(shape), dtype=torch.int).view(shape)
    coords = tuple(c.get_rank() for c in mesh_dim_comms)
    global_rank = int(mesh[coords].item())

    world_pg = None
    if _global_comm is not None:
        world_pg = wrap_comm_as_process_group(_global_comm, _global_comm.get_name())

    names = []
    for dim, (comm, dim_name) in enumerate(zip(mesh_dim_comms, mesh_dim_names)):
        members = _members_along(mesh, dim, global_rank)
        pg = wrap_comm_as_process_group(comm, dim_name, {g: i for i, g in enumerate(members)})
        if world_pg is None and dim == 0:
            world_pg = pg
        names.append(dim_name)

    c10d.GroupMember.WORLD = world_pg
    dm = dist.DeviceMesh(
        device_type=mesh_dim_comms[0].get_device().type,
        mesh=mesh,
        mesh_dim_names=tuple(mesh_dim_names),
        _init_backend=False,
        _rank=global_rank,
    )
    dm._dim_group_names = list(names)
    return dm


def _flatten_with_comm(
    device_mesh: dist.DeviceMesh,
    mesh_dim_name: str,
    comm: TorchComm,
    global_ranks: Sequence[int],
) -> dist.DeviceMesh:
    """Registers ``comm`` as the group of a flattened mesh dimension.

    ``global_ranks`` lists the world ranks of ``comm``'s members in group order.
    Returns a one-dimensional mesh named ``mesh_dim_name`` over those ranks.
    """
    wrap_comm_as_process_group(comm, mesh_dim_name, {g: i for i, g in enumerate(global_ranks)})
    flat = dist.DeviceMesh(
        device_type=device_mesh.device_type,
        mesh=torch.tensor(list(global_ranks), dtype=torch.int),
        mesh_dim_names=(mesh_dim_name,),
        _init_backend=False,
        _rank=device_mesh.get_rank() if hasattr(device_mesh, "get_rank") else None,
    )
    flat._dim_group_names = [mesh_dim_name]
    return flat
