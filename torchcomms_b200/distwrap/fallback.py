"""Software versions of operations a ``torch.distributed`` backend lacks, built
from operations it has.  Used on the pass-through path (``use_torchcomms=False``):
gloo has no all-to-all and cannot split a group.

* ``split_group_via_new_group``  every member learns all partitions (object
  all-gather from each partition's lowest rank) and calls ``new_group`` for
  each of them in the same order
* ``all_to_all_via_p2p`` / ``all_to_all_single_via_p2p``  one batched
  exchange of point-to-point operations
* ``all_gather_via_all_to_all``  all-gather as an all-to-all that sends the
  same tensor to everybody

Parity: comms/torchcomms/distwrap/fallback.py:19-176.
"""
from __future__ import annotations

from datetime import timedelta
from typing import Any, List, Optional, Sequence

import torch
import torch.distributed as dist


def split_group_via_new_group(parent_pg: Any, my_ranks: Optional[Sequence[int]], timeout: Optional[timedelta] = None,
                              pg_options: Any = None, group_desc: Optional[str] = None) -> Any:
    """Collective over ``parent_pg``. ``my_ranks``: global ranks of the caller's partition (None = in none)."""
    me = dist.get_rank()
    announce = list(my_ranks) if my_ranks is not None and me == min(my_ranks) else None
    everyone: List[Optional[List[int]]] = [None] * dist.get_world_size(parent_pg)
    dist.all_gather_object(everyone, announce, group=parent_pg)
    mine = None
    for ranks in sorted((r for r in everyone if r is not None), key=min):
        pg = dist.new_group(ranks=ranks, timeout=timeout, pg_options=pg_options, group_desc=group_desc)
        if me in ranks:
            mine = pg
    if my_ranks is not None and mine is None:
        raise RuntimeError("split_group: no process group was created for this rank's partition")
    return mine


def _exchange(pairs_recv, pairs_send, pg: Any, async_op: bool):
    ops = [dist.P2POp(dist.irecv, t, dist.get_global_rank(pg, p) if pg is not None else p, pg) for t, p in pairs_recv]
    ops += [dist.P2POp(dist.isend, t, dist.get_global_rank(pg, p) if pg is not None else p, pg) for t, p in pairs_send]
    if not ops:
        return None
    works = dist.batch_isend_irecv(ops)
    if async_op:
        return _All(works)
    for w in works:
        w.wait()
    return None


class _All:
    """One handle over several works."""

    def __init__(self, works):
        self._works = list(works)

    def wait(self, timeout=None):
        for w in self._works:
            w.wait()
        return True

    def is_completed(self):
        return all(w.is_completed() for w in self._works)


def all_to_all_via_p2p(outputs: List[torch.Tensor], inputs: List[torch.Tensor], pg: Any = None, async_op: bool = False):
    me, n = dist.get_rank(pg), dist.get_world_size(pg)
    outputs[me].copy_(inputs[me])
    return _exchange([(outputs[p], p) for p in range(n) if p != me], [(inputs[p], p) for p in range(n) if p != me], pg, async_op)


def all_to_all_single_via_p2p(output: torch.Tensor, input: torch.Tensor, output_split_sizes: Optional[List[int]] = None,
                              input_split_sizes: Optional[List[int]] = None, pg: Any = None, async_op: bool = False):
    n = dist.get_world_size(pg)
    ins = list(input.split(input_split_sizes if input_split_sizes else input.shape[0] // n, dim=0))
    outs = list(output.split(output_split_sizes if output_split_sizes else output.shape[0] // n, dim=0))
    return all_to_all_via_p2p(outs, ins, pg, async_op)


def all_gather_via_all_to_all(outputs: List[torch.Tensor], tensor: torch.Tensor, pg: Any = None, async_op: bool = False):
    return all_to_all_via_p2p(outputs, [tensor] * len(outputs), pg, async_op)


__all__ = ["split_group_via_new_group", "all_to_all_via_p2p", "all_to_all_single_via_p2p", "all_gather_via_all_to_all"]
