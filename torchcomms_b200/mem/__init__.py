"""Peer-exportable memory: allocator handles for ``comm.mem_allocator``."""


def get_mem_allocator(backend: str):
    raise NotImplementedError("filled in by the CUDA backend")
