"""One-sided point-to-point transfers between processes of one box, and a
tensor publisher built on them (weight sync, checkpoint hand-over).

Transport::

    # owner                                  # initiator
    mem = TransportMemory(weights)           tr = P2pTransport(torch.device("cuda", 0))
    tr = P2pTransport(weights.device)        url = tr.bind();  ... exchange urls ...
    url = tr.bind(); ... exchange urls ...   tr.connect(owner_url)
    tr.connect(initiator_url)                dst = TransportMemory(torch.empty_like(weights))
    send(mem.to_remote_buffer())             tr.read(dst.to_mutable_view(), remote_buffer)   # owner makes no call

Device memory on both sides moves as one NVLink peer copy issued by the
initiator (the access key carries a CUDA IPC handle); host memory, or
``B200COMMS_TRANSPORT_STAGED=1``, goes through the connection's socket and the
owner's service thread.  ``write`` / ``read`` return a status (``OK`` = 0),
``write_async`` / ``read_async`` a future.

Publisher::

    pub = TensorPublisher(model.state_dict())        # owner: registers, binds
    manifest = pub.manifest()                        # picklable; ship it by any channel
    fetch_tensors(manifest, into=replica.state_dict())   # any process on the box, any number of them

Parity: comms/torchcomms/transport/_transport.pyi (``RdmaTransport``,
``RdmaMemory``, ``RdmaMemoryView``, ``RdmaRemoteBuffer``; the same names are
exported here as aliases) and the weight-transfer use of comms/uniflow
(publish segments once, let consumers pull them).
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, Iterable, List, Mapping, Optional, Tuple

import torch

from . import _comms

_t = _comms.transport

P2pTransport = _t.P2pTransport
TransportMemory = _t.TransportMemory
MemoryView = _t.MemoryView
RemoteBuffer = _t.RemoteBuffer
TransportFuture = _t.TransportFuture
strerror = _t.strerror

OK = _t.OK
BAD_KEY = _t.BAD_KEY
OUT_OF_RANGE = _t.OUT_OF_RANGE
NOT_CONNECTED = _t.NOT_CONNECTED
IO_ERROR = _t.IO_ERROR
CUDA_ERROR = _t.CUDA_ERROR
TIMEOUT = _t.TIMEOUT
CLOSED = _t.CLOSED
SIZE_MISMATCH = _t.SIZE_MISMATCH

# The reference's names for the same objects.
RdmaTransport = P2pTransport
RdmaMemory = TransportMemory
RdmaMemoryView = MemoryView
RdmaMemoryMutableView = MemoryView
RdmaRemoteBuffer = RemoteBuffer


def init_caching_allocator_hook() -> None:
    """Registers every segment of PyTorch's CUDA caching allocator, present and future, with the
    transport, so that ``TransportMemory(tensor)`` reuses the segment's registration (one export
    per segment instead of one per tensor; ``reused_registration()`` is then true).  Needs no
    communicator.  Parity: ``init_caching_allocator_hook`` of the reference's NCCLX module
    (comms/torchcomms/ncclx/TorchCommNCCLXPy.cpp:187-204) and its transport CCA hook
    (comms/torchcomms/transport/RdmaTransportCCA.cpp)."""
    torch.cuda.init()
    _t.init_caching_allocator_hook()


attach_rdma_memory_hook = init_caching_allocator_hook   # the reference's name (transport/cca_hook)
register_segment = _t.register_segment
unregister_segment = _t.unregister_segment
segment_count = _t.segment_count


class TransportError(RuntimeError):
    def __init__(self, status: int, what: str):
        super().__init__(f"{what}: {strerror(status)} (status {status})")
        self.status = status


def _check(status: int, what: str) -> None:
    if status != OK:
        raise TransportError(status, what)


@dataclass
class TensorEntry:
    """One published tensor: where it lives and what it is."""

    name: str
    remote: RemoteBuffer
    dtype: torch.dtype
    shape: Tuple[int, ...]


@dataclass
class Manifest:
    """Everything a consumer needs to pull a published set of tensors."""

    url: bytes
    entries: List[TensorEntry] = field(default_factory=list)

    def names(self) -> List[str]:
        return [e.name for e in self.entries]

    def nbytes(self) -> int:
        return sum(e.remote.len for e in self.entries)


class TensorPublisher:
    """Registers a set of tensors and serves them to any number of consumers.

    The owner makes no call per transfer: consumers connect to ``manifest().url``
    and read.  Tensors must stay alive and unmodified in place for as long as
    consumers may read them (the publisher holds references); call ``close()``
    to stop serving.
    """

    def __init__(self, tensors: Mapping[str, torch.Tensor], device: Optional[torch.device] = None):
        tensors = dict(tensors)
        if not tensors:
            raise ValueError("nothing to publish")
        if device is None:
            device = next(iter(tensors.values())).device
        self._transport = P2pTransport(device)
        self._url = self._transport.bind()
        self._mems: Dict[str, TransportMemory] = {}
        self._entries: List[TensorEntry] = []
        for name, t in tensors.items():
            if not t.is_contiguous():
                raise ValueError(f"{name}: published tensors must be contiguous")
            if t.numel() == 0:
                continue
            mem = TransportMemory(t.detach())
            self._mems[name] = mem
            self._entries.append(TensorEntry(name, mem.to_remote_buffer(), t.dtype, tuple(t.shape)))

    def manifest(self) -> Manifest:
        return Manifest(self._url, list(self._entries))

    def counters(self) -> dict:
        return self._transport.counters()

    def close(self) -> None:
        self._transport.close()
        self._mems.clear()

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.close()


def fetch_tensors(
    manifest: Manifest,
    into: Optional[Mapping[str, torch.Tensor]] = None,
    device: Optional[torch.device] = None,
    names: Optional[Iterable[str]] = None,
    max_in_flight: int = 16,
) -> Dict[str, torch.Tensor]:
    """Pulls published tensors into ``into`` (same names, dtypes and shapes) or into new
    tensors on ``device``.  Returns the filled tensors by name."""
    wanted = set(names) if names is not None else None
    if device is None:
        device = next(iter(into.values())).device if into else torch.device("cpu")
    tr = P2pTransport(device)
    try:
        tr.bind()
        _check(tr.connect(manifest.url), "connect to the publisher")
        out: Dict[str, torch.Tensor] = {}
        pending: List[Tuple[str, TransportFuture, TransportMemory]] = []

        def drain(limit: int) -> None:
            while len(pending) > limit:
                name, fut, _mem = pending.pop(0)
                _check(fut.wait(), f"read of {name}")

        for e in manifest.entries:
            if wanted is not None and e.name not in wanted:
                continue
            if into is not None:
                if e.name not in into:
                    raise KeyError(f"{e.name} is published but missing from the destination")
                dst = into[e.name]
                if dst.dtype != e.dtype or tuple(dst.shape) != e.shape or not dst.is_contiguous():
                    raise ValueError(f"{e.name}: destination is {dst.dtype} {tuple(dst.shape)}, published {e.dtype} {e.shape}")
            else:
                dst = torch.empty(e.shape, dtype=e.dtype, device=device)
            mem = TransportMemory(dst.detach())
            pending.append((e.name, tr.read_async(mem.to_mutable_view(), e.remote), mem))
            out[e.name] = dst
            drain(max_in_flight)
        drain(0)
        return out
    finally:
        tr.close()


__all__ = [
    "P2pTransport", "TransportMemory", "MemoryView", "RemoteBuffer", "TransportFuture", "TransportError",
    "RdmaTransport", "RdmaMemory", "RdmaMemoryView", "RdmaMemoryMutableView", "RdmaRemoteBuffer",
    "TensorPublisher", "Manifest", "TensorEntry", "fetch_tensors", "strerror",
    "init_caching_allocator_hook", "attach_rdma_memory_hook", "register_segment", "unregister_segment", "segment_count",
    "OK", "BAD_KEY", "OUT_OF_RANGE", "NOT_CONNECTED", "IO_ERROR", "CUDA_ERROR", "TIMEOUT", "CLOSED", "SIZE_MISMATCH",
]
