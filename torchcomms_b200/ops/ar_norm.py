"""All-reduce + residual add + RMSNorm as one kernel (tensor-parallel decode).

After a row-parallel projection every rank holds a partial ``[tokens, hidden]``;
the next layer needs ``rmsnorm(sum of partials + residual)`` on every rank::

    fused = AllReduceRMSNorm(comm, hidden=4096)
    normed = fused(partial, weight, residual=resid)      # resid <- all_reduce(partial) + resid, in place

One block per token row stages the row in peer-visible memory, meets its peers
at one barrier, sums the row from all peers in fp32, adds the residual, and
normalises it in registers: the all-reduced activations are never written and
re-read on their own.  Up to ``MAX_ROWS`` (128) tokens and ``MAX_HIDDEN`` (8192)
features per call, bf16; larger batches fall back to the communicator's
all-reduce followed by the stand-alone RMSNorm kernel (two launches).

Parity: NVIDIA's ``nccl_ubx`` in the reference's vendored contrib tree
(comms/ncclx/v2_31/contrib/nccl_ubx) fuses the same three steps; the
reference's own API has no counterpart.  ``comm=None`` builds a single-rank
layer on the current device.
"""
from __future__ import annotations

from typing import Optional

import torch

from .. import ReduceOp, TorchComm, _comms

MAX_ROWS = _comms.AR_NORM_MAX_ROWS
MAX_HIDDEN = _comms.AR_NORM_MAX_HIDDEN


class AllReduceRMSNorm:
    def __init__(self, comm: Optional[TorchComm], hidden: int, eps: float = 1e-5, wait_ms: float = 2000.0):
        self.comm, self.hidden, self.eps = comm, hidden, eps
        impl = None if comm is None else comm.get_backend_impl()
        self._native = comm is None or isinstance(impl, _comms.CudaBackend)
        fused = self._native and hidden <= MAX_HIDDEN and hidden % 8 == 0 and torch.cuda.is_available()
        self._layer = _comms.ArNormLayer(impl, hidden, wait_ms) if fused else None

    def __call__(self, x: torch.Tensor, weight: torch.Tensor, residual: Optional[torch.Tensor] = None) -> torch.Tensor:
        if self._layer is not None and x.is_cuda and x.dtype == torch.bfloat16 and x.dim() == 2 and x.shape[0] <= MAX_ROWS:
            return self._layer.forward(x, residual, weight, self.eps)
        return self._unfused(x, weight, residual)

    def _unfused(self, x, weight, residual):
        total = x.clone()
        if self.comm is not None and self.comm.get_size() > 1:
            self.comm.all_reduce(total, ReduceOp.SUM, False)
        if residual is not None:
            residual.add_(total)
            total = residual
        if total.is_cuda and total.dtype == torch.bfloat16 and weight.dtype == torch.bfloat16:
            return _comms.ops.rmsnorm_fwd(total.reshape(-1, total.shape[-1]), weight, self.eps)[0].reshape(total.shape)
        t = total.float()
        return (t * torch.rsqrt(t.pow(2).mean(-1, keepdim=True) + self.eps) * weight.float()).to(x.dtype)

    def status(self):
        return self._layer.status() if self._layer is not None else []
