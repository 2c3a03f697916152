"""Multi-dimensional parallel layouts from one world communicator.

    comms = split_mesh(world, shape=(2, 4), names=("dp", "tp"))     # {"dp": comm of size 2, "tp": comm of size 4}
    mesh = device_mesh_from_world(world, shape=(2, 4), names=("dp", "tp"))   # torch DeviceMesh over the same comms

Ranks are laid out row-major over ``shape`` (the last dimension varies fastest, so with
``("dp", "tp")`` the ranks of one tensor-parallel group are consecutive - on one NVSwitch box
every placement has the same bandwidth, consecutive ranks just read best in logs).  Every rank
of ``world`` must call these functions with the same arguments: each sub-communicator is made
with ``world.split``, which is collective over the world.

Parity: the 2-D setups of comms/torchcomms/tests/integration/py/DPTPCommTest.py and
DeviceMeshTest.py, which build the per-dimension communicators by hand.
"""
from __future__ import annotations

import itertools
import math
from typing import Dict, List, Sequence

from .. import TorchComm


def mesh_coordinates(rank: int, shape: Sequence[int]) -> List[int]:
    """Row-major coordinates of ``rank`` in a mesh of ``shape``."""
    coords = []
    for extent in reversed(shape):
        coords.append(rank % extent)
        rank //= extent
    return coords[::-1]


def mesh_groups(shape: Sequence[int], dim: int) -> List[List[int]]:
    """All groups of ranks along ``dim``: one group per setting of the other coordinates."""
    strides = [math.prod(shape[i + 1:]) for i in range(len(shape))]
    others = [range(e) for i, e in enumerate(shape) if i != dim]
    groups = []
    for fixed in itertools.product(*others):
        it = iter(fixed)
        base = sum((next(it) if i != dim else 0) * strides[i] for i in range(len(shape)))
        groups.append([base + k * strides[dim] for k in range(shape[dim])])
    return groups


def split_mesh(world: TorchComm, shape: Sequence[int], names: Sequence[str]) -> Dict[str, TorchComm]:
    """One communicator per mesh dimension for the calling rank."""
    if len(shape) != len(names) or len(set(names)) != len(names):
        raise ValueError("shape and names must have the same length and names must be distinct")
    if math.prod(shape) != world.get_size():
        raise ValueError(f"mesh {tuple(shape)} has {math.prod(shape)} ranks, the communicator has {world.get_size()}")
    rank = world.get_rank()
    out: Dict[str, TorchComm] = {}
    for dim, name in enumerate(names):
        for index, group in enumerate(mesh_groups(shape, dim)):
            sub = world.split(group if rank in group else [], f"{name}{index}")
            if sub is not None:
                out[name] = sub
    return out


def device_mesh_from_world(world: TorchComm, shape: Sequence[int], names: Sequence[str]):
    """A ``torch.distributed.DeviceMesh`` whose dimension groups are communicators split from ``world``.
    The communicators stay reachable as ``mesh._b200c_comms`` (finalize them before ``world``)."""
    from ..device_mesh import init_device_mesh

    comms = split_mesh(world, shape, names)
    mesh = init_device_mesh(mesh_dim_comms=tuple(comms[n] for n in names), mesh_dim_names=tuple(names),
                            _global_comm=world if len(shape) > 1 else None)
    mesh._b200c_comms = comms
    return mesh


__all__ = ["mesh_coordinates", "mesh_groups", "split_mesh", "device_mesh_from_world"]
