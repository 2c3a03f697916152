"""Training engine: Llama-style decoder, sharded data parallel over one
communicator, stage-at-a-time execution.

One step = forward over the stages (embedding, blocks, head) with the next
stage's parameter gather in flight on the communicator's stream; backward in
reverse with the previous stage's gather and the just-finished stage's
gradient reduce-scatter in flight; AdamW on each shard as soon as its
reduction lands.  Stage boundaries are detached tensors, so each stage's
autograd graph is released as soon as its backward ran.
"""
from __future__ import annotations

from typing import List, Optional

import torch

from .. import TorchComm
from ..models.llama import Block, Embedding, Head, LlamaConfig
from ..ops import fused
from .fsdp import BufferPool, ShardedUnit, StepTimeline


class TrainEngine:
    def __init__(
        self,
        cfg: LlamaConfig,
        comm: TorchComm,
        *,
        lr: float = 3e-4,
        beta1: float = 0.9,
        beta2: float = 0.95,
        eps: float = 1e-8,
        weight_decay: float = 0.1,
        seed: int = 0,
        param_dtype: torch.dtype = torch.bfloat16,
        recompute_blocks: int = 0,
        comm_mode: Optional[str] = None,
    ):
        self.cfg = cfg
        self.comm = comm
        self.device = comm.get_device()
        self.hp = dict(lr=lr, beta1=beta1, beta2=beta2, eps=eps, weight_decay=weight_decay)
        self.step_count = 0
        self.recompute_blocks = recompute_blocks
        self.units: List[ShardedUnit] = []
        if comm_mode is None:
            comm_mode = "symm" if comm.get_backend() in ("b200", "nccl", "ncclx") else "plain"
        self.comm_mode = comm_mode
        # One pool for all stages: stages of the same size share its rotating buffers.
        self.pool = BufferPool(comm, symmetric=comm_mode == "symm")
        # Stages are created one at a time on the device and immediately
        # reduced to their shard, so the full fp32 model never exists.
        makers = [lambda: Embedding(cfg)] + [lambda: Block(cfg) for _ in range(cfg.n_layers)] + [lambda: Head(cfg)]
        for i, make in enumerate(makers):
            torch.manual_seed(seed * 100003 + i)
            with torch.device(self.device):
                stage = make()
            self.units.append(ShardedUnit(stage, comm, param_dtype, comm_mode=comm_mode, pool=self.pool))
        self.cos_t, self.sin_t = fused.rope_tables(cfg.max_seq_len, cfg.head_dim, cfg.rope_theta, self.device)

    def attach_timeline(self) -> StepTimeline:
        """Starts recording comm / wait / optimizer spans of the following steps."""
        tl = StepTimeline(self.comm, self.comm_mode)
        for u in self.units:
            u.timeline = tl
        return tl

    def detach_timeline(self) -> None:
        for u in self.units:
            u.timeline = None

    def close(self) -> None:
        """Gives the pool's symmetric buffers back (collective). The engine is unusable afterwards."""
        for u in self.units:
            u.release_params()
        if self.pool.symmetric:
            self.pool.free_all()
        self.units = []

    @property
    def num_parameters(self) -> int:
        return self.cfg.param_count()

    def _run_stage(self, i: int, x, pos, targets):
        unit = self.units[i]
        if i == 0:
            return unit.module(x)
        if i == len(self.units) - 1:
            return unit.module(x, targets)
        return unit.module(x, pos, self.cos_t, self.sin_t)

    def step(self, tokens: torch.Tensor, targets: torch.Tensor) -> torch.Tensor:
        """One optimizer step on this rank's micro-batch; returns the loss (a 0-d device tensor)."""
        units = self.units
        n = len(units)
        b, s = tokens.shape
        pos = torch.arange(s, dtype=torch.int32, device=self.device).repeat(b)
        self.step_count += 1

        # ---- forward
        inputs: List[Optional[torch.Tensor]] = [None] * n
        outputs: List[Optional[torch.Tensor]] = [None] * n
        units[0].gather()
        x = tokens
        for i in range(n):
            if i + 1 < n:
                units[i + 1].gather()  # prefetch while this stage computes
            units[i].wait_gather()
            recompute = 1 <= i < n - 1 and (i - 1) < self.recompute_blocks
            if i > 0:
                x = x.detach().requires_grad_(True)
            inputs[i] = x
            if recompute:
                with torch.no_grad():
                    y = self._run_stage(i, x, pos, targets)
            else:
                y = self._run_stage(i, x, pos, targets)
                outputs[i] = y
            if i < n - 1:
                units[i].release_params()
            x = y
        loss = x

        # ---- backward (the head's parameters are still resident)
        grad = None
        for i in range(n - 1, -1, -1):
            if i - 1 >= 0:
                units[i - 1].gather()  # prefetch for the next backward stage
            units[i].wait_gather()
            units[i].prepare_grads()
            y = outputs[i]
            if y is None:  # recomputed stage
                y = self._run_stage(i, inputs[i], pos, targets)
            if i == n - 1:
                y.backward()
            else:
                y.backward(grad)
            grad = inputs[i].grad if i > 0 else None
            outputs[i] = None
            inputs[i] = None
            units[i].release_params()
            units[i].reduce_grads()
            # The stage that finished one iteration ago has had a whole
            # backward stage of compute to hide its reduction behind.
            if i + 1 < n:
                units[i + 1].finish_step(step=self.step_count, **self.hp)
        units[0].finish_step(step=self.step_count, **self.hp)
        return loss.detach()

    def state_dict(self) -> dict:
        return {"step": self.step_count, "units": [u.state_dict() for u in self.units]}

    def load_state_dict(self, state: dict) -> None:
        self.step_count = int(state["step"])
        for u, s in zip(self.units, state["units"]):
            u.load_state_dict(s)
