"""Data parallel gradient averaging with bucketed, overlapped all-reduce.

``DataParallel(module, comm)`` registers post-accumulate-grad hooks; gradients
are packed into flat buckets in reverse parameter order (the order in which
backward produces them), each full bucket starts one asynchronous
``all_reduce(AVG)`` on the communicator's side stream while backward keeps
running, and ``finish()`` (call it before the optimizer step) waits for the
buckets and scatters the averaged values back into ``param.grad``.

On the CUDA backend a bucket of up to 512 KiB takes the one-shot kernel and a
larger one the NVLS two-shot kernel, with the 1/n scale fused into the
reduction.  ``torch.nn.parallel.DistributedDataParallel`` over the c10d adapter
(``device_mesh.init_device_mesh``) keeps working as in the reference
(comms/torchcomms/tests/integration/py/DDPCommTest.py); this class is the
dependency-free equivalent used by the examples.
"""
from __future__ import annotations

from typing import List, Tuple

import torch
from torch import nn

from .. import ReduceOp, TorchComm


class DataParallel:
    def __init__(self, module: nn.Module, comm: TorchComm, bucket_mb: float = 25.0, broadcast_parameters: bool = True):
        self.module, self.comm = module, comm
        self.bucket_bytes = int(bucket_mb * (1 << 20))
        self.params: List[nn.Parameter] = [p for p in module.parameters() if p.requires_grad]
        if broadcast_parameters:
            for p in self.params:
                comm.broadcast(p.data, 0, False)
        # bucket layout in reverse order: backward reaches the last layers first
        self._buckets: List[List[nn.Parameter]] = [[]]
        size = 0
        for p in reversed(self.params):
            nbytes = p.numel() * p.element_size()
            if self._buckets[-1] and (size + nbytes > self.bucket_bytes or self._buckets[-1][0].dtype != p.dtype):
                self._buckets.append([])
                size = 0
            self._buckets[-1].append(p)
            size += nbytes
        self._bucket_of = {id(p): i for i, b in enumerate(self._buckets) for p in b}
        self._pending = [0] * len(self._buckets)
        self._inflight: List[Tuple[int, torch.Tensor, object]] = []
        self._hooks = [p.register_post_accumulate_grad_hook(self._on_grad) for p in self.params]
        self._reset()

    def _reset(self) -> None:
        self._pending = [len(b) for b in self._buckets]
        self._inflight = []

    def _on_grad(self, p: nn.Parameter) -> None:
        i = self._bucket_of[id(p)]
        self._pending[i] -= 1
        if self._pending[i] == 0:
            flat = torch.cat([q.grad.reshape(-1) for q in self._buckets[i]])
            work = self.comm.all_reduce(flat, ReduceOp.AVG, True)
            self._inflight.append((i, flat, work))

    def finish(self) -> None:
        """Waits for every bucket and writes the averaged gradients back."""
        launched = {i for i, _, _ in self._inflight}
        for i, bucket in enumerate(self._buckets):  # parameters that received no gradient this step
            if i not in launched and any(q.grad is not None for q in bucket):
                flat = torch.cat([(q.grad if q.grad is not None else torch.zeros_like(q)).reshape(-1) for q in bucket])
                self._inflight.append((i, flat, self.comm.all_reduce(flat, ReduceOp.AVG, True)))
        for i, flat, work in self._inflight:
            work.wait()
            off = 0
            for q in self._buckets[i]:
                n = q.numel()
                if q.grad is None:
                    q.grad = torch.empty_like(q)
                q.grad.copy_(flat[off:off + n].view_as(q))
                off += n
        self._reset()

    def __call__(self, *args, **kwargs):
        return self.module(*args, **kwargs)

    def remove_hooks(self) -> None:
        for h in self._hooks:
            h.remove()
        self._hooks = []
