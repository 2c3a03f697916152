"""Peer-exportable device memory.

``get_mem_allocator(backend)`` returns an allocator object for
``torch.cuda.MemPool``; tensors created inside
``torch.cuda.use_mem_pool(pool)`` live in CUDA virtual-memory allocations with
POSIX-fd shareable handles, so a window can map them into every peer
(zero-copy one-sided access and NVLS multicast binding).

``symm_empty(comm, shape, dtype)`` goes one step further: a collective call
that returns a tensor in memory every rank of ``comm`` has already mapped
(bound to the NVLS multicast object where the box allows).  Collectives whose
output (all-gather, all-to-all), input (reduce-scatter) or in-place buffer
(all-reduce) is such a tensor run as one-pass kernels with no staging copies.
Tensors made inside a ``MemPool`` of ``get_mem_allocator`` get the same
treatment after ``comm.tensor_register(tensor)``.

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


_CUDA_BACKENDS = ("b200", "nccl", "ncclx")


def symm_empty(comm, shape, dtype):
    """Collective: a tensor of ``shape`` in symmetric memory of ``comm``.

    Every rank calls this in the same order with the same shape.  The memory
    stays mapped until ``symm_free(comm, tensor)`` or ``comm.finalize()``;
    the tensor must not be used afterwards.  Backends without peer memory
    (gloo, fake) return an ordinary tensor.
    """
    import torch

    if isinstance(shape, int):
        shape = (shape,)
    if comm.get_backend() in _CUDA_BACKENDS:
        return comm.get_backend_impl().symm_empty([int(d) for d in shape], dtype)
    return torch.empty(tuple(shape), dtype=dtype, device=comm.get_device())


def symm_free(comm, tensor) -> None:
    """Collective: unmaps a tensor made by ``symm_empty``."""
    if comm.get_backend() in _CUDA_BACKENDS:
        comm.get_backend_impl().symm_free(tensor)


def is_symmetric(comm, tensor) -> bool:
    """True when collectives of ``comm`` on ``tensor`` take the one-pass kernels."""
    if comm.get_backend() in _CUDA_BACKENDS:
        return bool(comm.get_backend_impl().is_symmetric(tensor))
    return False
