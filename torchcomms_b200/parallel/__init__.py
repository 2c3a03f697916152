"""Parallelism strategies built on a communicator: sharded data parallel (FSDP), tensor, pipeline, expert and sequence parallel helpers."""
from .engine import TrainEngine  # noqa: F401
from .fsdp import ShardedUnit  # noqa: F401
