"""Pipeline parallelism over a communicator's point-to-point operations.

One rank = one stage.  Activations travel forward and gradients backward with
``send`` / ``recv``; the 1F1B schedule keeps at most ``num_stages - stage``
micro-batches alive per stage.  Where a stage both sends and receives in the
same step the two transfers are issued as one ``BatchSendRecv`` so that
neither side blocks the other (on the CUDA backend they become one grouped
NCCL call on the communicator's side stream).

The reference ships the primitives (BatchSendRecv, send/recv, per-peer lazy
communicators: comms/torchcomms/TorchCommBatch.hpp:27-61,
lazy/LazyBackend.hpp:29-86) and leaves the schedule to the trainer; this
module is that schedule.
"""
from __future__ import annotations

from typing import Callable, List, Optional, Sequence

import torch

from .. import TorchComm


class PipelineStage:
    """``module`` is this rank's slice of the model; ``input_like`` describes the activation it receives."""

    def __init__(self, module: torch.nn.Module, comm: TorchComm, input_like: Optional[torch.Tensor] = None):
        self.module = module
        self.comm = comm
        self.stage = comm.get_rank()
        self.num_stages = comm.get_size()
        self.input_like = input_like
        if not self.is_first and input_like is None:
            raise ValueError("stages after the first need input_like (shape/dtype/device of the incoming activation)")

    @property
    def is_first(self) -> bool:
        return self.stage == 0

    @property
    def is_last(self) -> bool:
        return self.stage == self.num_stages - 1

    # -- transfers ---------------------------------------------------------
    def _recv_activation(self) -> torch.Tensor:
        buf = torch.empty_like(self.input_like)
        self.comm.recv(buf, self.stage - 1, False)
        return buf.requires_grad_(True)

    def _send_activation(self, y: torch.Tensor) -> None:
        self.comm.send(y.detach().contiguous(), self.stage + 1, False)

    def _send_grad(self, g: torch.Tensor) -> None:
        self.comm.send(g.contiguous(), self.stage - 1, False)

    def _recv_grad(self, like: torch.Tensor) -> torch.Tensor:
        buf = torch.empty_like(like)
        self.comm.recv(buf, self.stage + 1, False)
        return buf

    def _send_act_recv_grad(self, y: torch.Tensor, like: torch.Tensor) -> torch.Tensor:
        """Steady state of 1F1B: push this micro-batch's activation, pull the gradient of an older one."""
        g = torch.empty_like(like)
        batch = self.comm.batch_op_create()
        batch.send(y.detach().contiguous(), self.stage + 1)
        batch.recv(g, self.stage + 1)
        batch.issue(False)
        return g

    # -- schedule ----------------------------------------------------------
    def run_1f1b(self, microbatches: Sequence[torch.Tensor], loss_fn: Optional[Callable[[torch.Tensor, int], torch.Tensor]] = None,
                 ) -> List[torch.Tensor]:
        """One training step.  ``microbatches``: the first stage's inputs (ignored elsewhere, only its
        length counts).  ``loss_fn(output, microbatch_index)`` runs on the last stage.  Parameter
        gradients accumulate in ``module``; the last stage returns the per-micro-batch losses."""
        m = len(microbatches)
        warmup = min(self.num_stages - self.stage - 1, m)
        inputs: List[Optional[torch.Tensor]] = []
        outputs: List[torch.Tensor] = []
        losses: List[torch.Tensor] = []
        fwd = bwd = 0

        def forward_one() -> torch.Tensor:
            nonlocal fwd
            x = microbatches[fwd] if self.is_first else self._recv_activation()
            y = self.module(x)
            inputs.append(None if self.is_first else x)
            if self.is_last:
                if loss_fn is None:
                    raise ValueError("the last stage needs loss_fn")
                y = loss_fn(y, fwd)
                losses.append(y.detach())
            outputs.append(y)
            fwd += 1
            return y

        def backward_one(grad: Optional[torch.Tensor]) -> None:
            nonlocal bwd
            y, x = outputs[bwd], inputs[bwd]
            if self.is_last:
                y.backward()
            else:
                y.backward(grad)
            outputs[bwd] = None  # free the graph
            if x is not None:
                self._send_grad(x.grad)
                inputs[bwd] = None
            bwd += 1

        for _ in range(warmup):
            self._send_activation(forward_one())
        for _ in range(m - warmup):
            y = forward_one()
            if self.is_last:
                backward_one(None)
            else:
                backward_one(self._send_act_recv_grad(y, outputs[bwd]))
        while bwd < m:
            backward_one(self._recv_grad(outputs[bwd]))
        return losses


def run_gpipe(stage: PipelineStage, microbatches: Sequence[torch.Tensor],
              loss_fn: Optional[Callable[[torch.Tensor, int], torch.Tensor]] = None) -> List[torch.Tensor]:
    """All forwards, then all backwards (simplest schedule; peak activation memory = all micro-batches)."""
    xs, ys, losses = [], [], []
    for i in range(len(microbatches)):
        x = microbatches[i] if stage.is_first else stage._recv_activation()
        y = stage.module(x)
        if stage.is_last:
            y = loss_fn(y, i)
            losses.append(y.detach())
        else:
            stage._send_activation(y)
        xs.append(None if stage.is_first else x)
        ys.append(y)
    for i in range(len(microbatches)):
        if stage.is_last:
            ys[i].backward()
        else:
            ys[i].backward(stage._recv_grad(ys[i]))
        if xs[i] is not None:
            stage._send_grad(xs[i].grad)
    return losses
