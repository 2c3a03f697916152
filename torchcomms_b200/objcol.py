"""Collectives over arbitrary picklable Python objects.

Every function serialises on the host, exchanges byte lengths first and the
padded payloads second, both through ordinary tensor collectives of the given
communicator (payloads live on the communicator's device).  This is what
state-dict / checkpoint planning code uses to exchange metadata.

Serialisation is ``torch.save`` / ``torch.load`` by default (``weights_only``
honoured) or ``pickle`` when ``TORCHCOMMS_SERIALIZATION=pickle``.

Parity: ``comms/torchcomms/objcol.py:15-36`` (serialisation switch), ``:67``
(all_gather_object), ``:170`` (gather_object), ``:297`` / ``:384``
(send/recv_object_list), ``:473`` (broadcast_object_list), ``:587``
(scatter_object_list).  Signatures match the reference.
"""
from __future__ import annotations

import io
import os
import pickle
from datetime import timedelta
from typing import Any, List, Optional

import torch

from . import TorchComm

__all__ = [
    "all_gather_object",
    "gather_object",
    "send_object_list",
    "recv_object_list",
    "broadcast_object_list",
    "scatter_object_list",
]


def _use_pickle() -> bool:
    return os.environ.get("TORCHCOMMS_SERIALIZATION", "torch").lower() == "pickle"


def _encode(obj: Any, device: torch.device) -> torch.Tensor:
    if _use_pickle():
        raw = pickle.dumps(obj)
    else:
        buf = io.BytesIO()
        torch.save(obj, buf)
        raw = buf.getvalue()
    t = torch.frombuffer(bytearray(raw), dtype=torch.uint8)
    return t.to(device) if device.type != "cpu" else t


def _decode(payload: torch.Tensor, nbytes: int, weights_only: bool) -> Any:
    raw = payload[:nbytes].cpu().numpy().tobytes()
    if _use_pickle():
        return pickle.loads(raw)
    return torch.load(io.BytesIO(raw), weights_only=weights_only)


def _len_tensor(n: int, device: torch.device) -> torch.Tensor:
    return torch.tensor([n], dtype=torch.int64, device=device)


def _kw(timeout: Optional[timedelta]) -> dict:
    return {} if timeout is None else {"timeout": timeout}


def all_gather_object(
    comm: TorchComm,
    object_list: List[Any],
    obj: Any,
    timeout: Optional[timedelta] = None,
    weights_only: bool = False,
) -> List[Any]:
    """Fills ``object_list[r]`` with rank ``r``'s ``obj`` on every rank."""
    world, dev = comm.get_size(), comm.get_device()
    if len(object_list) != world:
        raise ValueError(f"object_list must have {world} entries")
    mine = _encode(obj, dev)
    lens = torch.zeros(world, dtype=torch.int64, device=dev)
    comm.all_gather_single(lens, _len_tensor(mine.numel(), dev), False, **_kw(timeout))
    lens_host = lens.cpu().tolist()
    width = max(lens_host)
    padded = torch.zeros(width, dtype=torch.uint8, device=dev)
    padded[: mine.numel()] = mine
    gathered = torch.empty(world * width, dtype=torch.uint8, device=dev)
    comm.all_gather_single(gathered, padded, False, **_kw(timeout))
    if dev.type != "cpu":
        torch.cuda.current_stream(dev).synchronize()
    rows = gathered.view(world, width)
    for r in range(world):
        object_list[r] = _decode(rows[r], lens_host[r], weights_only)
    return object_list


def gather_object(
    comm: TorchComm,
    obj: Any,
    root: int,
    object_gather_list: Optional[List[Any]] = None,
    timeout: Optional[timedelta] = None,
    weights_only: bool = False,
) -> Optional[List[Any]]:
    """Collects every rank's ``obj`` into ``object_gather_list`` on ``root``."""
    world, rank, dev = comm.get_size(), comm.get_rank(), comm.get_device()
    mine = _encode(obj, dev)
    lens = torch.zeros(world, dtype=torch.int64, device=dev)
    comm.all_gather_single(lens, _len_tensor(mine.numel(), dev), False, **_kw(timeout))
    lens_host = lens.cpu().tolist()
    width = max(lens_host)
    padded = torch.zeros(width, dtype=torch.uint8, device=dev)
    padded[: mine.numel()] = mine
    sink = torch.empty(world * width if rank == root else 0, dtype=torch.uint8, device=dev)
    comm.gather_single(sink, padded, root, False, **_kw(timeout))
    if rank != root:
        return None
    if dev.type != "cpu":
        torch.cuda.current_stream(dev).synchronize()
    if object_gather_list is None:
        object_gather_list = [None] * world
    if len(object_gather_list) != world:
        raise ValueError(f"object_gather_list must have {world} entries")
    rows = sink.view(world, width)
    for r in range(world):
        object_gather_list[r] = _decode(rows[r], lens_host[r], weights_only)
    return object_gather_list


def send_object_list(
    comm: TorchComm,
    object_list: List[Any],
    dst: int,
    timeout: Optional[timedelta] = None,
) -> None:
    """Sends the objects to ``dst`` (pair with ``recv_object_list``)."""
    dev = comm.get_device()
    blobs = [_encode(o, dev) for o in object_list]
    lens = torch.tensor([b.numel() for b in blobs], dtype=torch.int64, device=dev)
    comm.send(lens, dst, False, **_kw(timeout))
    if blobs:
        comm.send(torch.cat(blobs), dst, False, **_kw(timeout))


def recv_object_list(
    comm: TorchComm,
    object_list: List[Any],
    src: int,
    timeout: Optional[timedelta] = None,
    weights_only: bool = False,
) -> List[Any]:
    """Receives ``len(object_list)`` objects from ``src`` in place."""
    dev = comm.get_device()
    lens = torch.zeros(len(object_list), dtype=torch.int64, device=dev)
    comm.recv(lens, src, False, **_kw(timeout))
    lens_host = lens.cpu().tolist()
    if not lens_host:
        return object_list
    payload = torch.empty(sum(lens_host), dtype=torch.uint8, device=dev)
    comm.recv(payload, src, False, **_kw(timeout))
    if dev.type != "cpu":
        torch.cuda.current_stream(dev).synchronize()
    off = 0
    for i, n in enumerate(lens_host):
        object_list[i] = _decode(payload[off : off + n], n, weights_only)
        off += n
    return object_list


def broadcast_object_list(
    comm: TorchComm,
    object_list: List[Any],
    root: int,
    timeout: Optional[timedelta] = None,
    weights_only: bool = False,
) -> List[Any]:
    """Replaces ``object_list`` on every rank with ``root``'s objects."""
    dev, rank = comm.get_device(), comm.get_rank()
    if rank == root:
        blobs = [_encode(o, dev) for o in object_list]
        lens = torch.tensor([b.numel() for b in blobs], dtype=torch.int64, device=dev)
    else:
        blobs = []
        lens = torch.zeros(len(object_list), dtype=torch.int64, device=dev)
    comm.broadcast(lens, root, False, **_kw(timeout))
    lens_host = lens.cpu().tolist()
    total = sum(lens_host)
    if total == 0:
        return object_list
    payload = torch.cat(blobs) if rank == root else torch.empty(total, dtype=torch.uint8, device=dev)
    comm.broadcast(payload, root, False, **_kw(timeout))
    if rank != root:
        if dev.type != "cpu":
            torch.cuda.current_stream(dev).synchronize()
        off = 0
        for i, n in enumerate(lens_host):
            object_list[i] = _decode(payload[off : off + n], n, weights_only)
            off += n
    return object_list


def scatter_object_list(
    comm: TorchComm,
    root: int,
    scatter_object_output_list: List[Any],
    scatter_object_input_list: Optional[List[Any]] = None,
    timeout: Optional[timedelta] = None,
    weights_only: bool = False,
) -> List[Any]:
    """Rank ``r`` receives ``scatter_object_input_list[r]`` of ``root`` in
    ``scatter_object_output_list[0]``."""
    world, rank, dev = comm.get_size(), comm.get_rank(), comm.get_device()
    if not scatter_object_output_list:
        raise ValueError("scatter_object_output_list needs at least one slot")
    if rank == root:
        if scatter_object_input_list is None or len(scatter_object_input_list) != world:
            raise ValueError(f"the root must pass {world} objects")
        blobs = [_encode(o, dev) for o in scatter_object_input_list]
        width = max(b.numel() for b in blobs)
        meta = torch.tensor([width] + [b.numel() for b in blobs], dtype=torch.int64, device=dev)
    else:
        blobs, width = [], 0
        meta = torch.zeros(world + 1, dtype=torch.int64, device=dev)
    comm.broadcast(meta, root, False, **_kw(timeout))
    meta_host = meta.cpu().tolist()
    width = meta_host[0]
    rows = []
    if rank == root:
        for b in blobs:
            row = torch.zeros(width, dtype=torch.uint8, device=dev)
            row[: b.numel()] = b
            rows.append(row)
    mine = torch.empty(width, dtype=torch.uint8, device=dev)
    comm.scatter(mine, rows, root, False, **_kw(timeout))
    if dev.type != "cpu":
        torch.cuda.current_stream(dev).synchronize()
    scatter_object_output_list[0] = _decode(mine, meta_host[1 + rank], weights_only)
    return scatter_object_output_list
