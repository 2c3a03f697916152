"""Peer-exportable device memory.

``get_mem_allocator(backend)`` returns an allocator object for
``torch.cuda.MemPool``; tensors created inside
``torch.cuda.use_mem_pool(pool)`` live in CUDA virtual-memory allocations with
POSIX-fd shareable handles, so a window can map them into every peer
(zero-copy one-sided access and NVLS multicast binding).

Parity: ``comm.mem_allocator`` / ``get_mem_allocator`` of the reference
(``comms/torchcomms/ncclx/TorchCommNCCLX.cpp:2343-2382``, a
CUDAPluggableAllocator over ncclMemAlloc / ncclMemFree).
"""
from __future__ import annotations

import os

_allocators = {}


def _library_path() -> str:
    return os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "_comms.so")


def get_mem_allocator(backend: str):
    """Allocator handle for ``torch.cuda.MemPool`` (CUDA backends only)."""
    if backend not in ("b200", "nccl", "ncclx"):
        raise RuntimeError(f"backend '{backend}' has no device memory allocator")
    if "cuda" not in _allocators:
        from torch.cuda.memory import CUDAPluggableAllocator

        pluggable = CUDAPluggableAllocator(_library_path(), "b200c_symm_alloc", "b200c_symm_free")
        _allocators["cuda"] = (pluggable, pluggable.allocator())
    return _allocators["cuda"][1]


def symmetric_empty(comm, shape, dtype):
    """A tensor in peer-exportable memory, ready for ``comm.new_window``."""
    import torch

    pool = torch.cuda.MemPool(get_mem_allocator(comm.get_backend()))
    with torch.cuda.use_mem_pool(pool):
        t = torch.empty(shape, dtype=dtype, device=comm.get_device())
    t._b200c_pool = pool  # the pool must outlive the tensor
    return t
