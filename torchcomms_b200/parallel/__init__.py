"""Parallelism strategies built on a communicator.

* ``data``               - replicated data parallel: bucketed, overlapped gradient all-reduce
* ``engine`` / ``fsdp``  - sharded data parallel (ZeRO-3 style) training engine
* ``tensor``             - column / row parallel layers, sequence parallel, fused TP MLP
* ``pipeline``           - 1F1B and GPipe schedules over send / recv
* ``context``            - ring attention and Ulysses (sequence sharded attention)
* ``expert``             - MoE layer on the fused dispatch / combine kernels
"""
from .engine import TrainEngine  # noqa: F401
from .fsdp import ShardedUnit  # noqa: F401
