"""``torch.distributed``-shaped module whose collectives run on communicators.

    from torchcomms_b200 import distwrap as dist
    dist.init_process_group(backend="cpu:gloo,cuda:b200", use_torchcomms=True)
    dist.all_reduce(t)                     # -> TorchComm.all_reduce of the comm for t's device
    sub = dist.split_group(split_ranks=[[0, 1], [2, 3]], group_desc="tp")
    dist.all_gather_into_tensor(out, t, group=sub)

With ``use_torchcomms=False`` every call is forwarded to ``torch.distributed``
unchanged.  With it, one communicator per device type is created and a
``ProcessGroup`` served by the c10d adapter is installed as the WORLD group, so
``dist.get_rank()``, DeviceMesh and code that still calls ``torch.distributed``
directly keep working *and* land on the same communicators (the reference
blocks such direct calls because its process groups are native NCCL ones that
would bypass torchcomms; here they cannot bypass it).  Sub-groups come from
``split_group`` (communicator split); ``new_group`` is refused as in the
reference.

Parity: comms/torchcomms/distwrap/{__init__,new_comm,collectives,
collectives_extension,pginfo,utils}.py and distwrap/README.md.
"""
from __future__ import annotations

import os
from dataclasses import dataclass, field
from datetime import timedelta
from typing import Any, Dict, List, Optional, Sequence, Tuple

import torch
import torch.distributed as _td
from torch.distributed import (  # noqa: F401  (re-exports)
    GroupMember,
    HashStore,
    ProcessGroup,
    Store,
    Work,
    get_process_group_ranks,
    group,
    is_available,
)

# Backend classes of torch.distributed that code written against it names (options objects, isinstance checks);
# absent in torch builds without the corresponding backend.
ProcessGroupGloo = getattr(_td, "ProcessGroupGloo", None)
ProcessGroupNCCL = getattr(_td, "ProcessGroupNCCL", None)

from .. import ReduceOp as _TcReduceOp  # noqa: E402
from .. import TorchComm, new_comm, objcol
from ..device_mesh import wrap_comm_as_process_group
from ..mem import get_mem_allocator as _tc_get_mem_allocator

ReduceOp = _td.ReduceOp

_CUDA_NAMES = {"nccl", "ncclx", "b200", "cuda"}


from . import fallback  # noqa: E402
from .pginfo import PgInfo as _PgInfo  # noqa: E402
from .pginfo import _REGISTRY  # noqa: E402
from .pginfo import (  # noqa: E402,F401
    pg_info_assert_registered, pg_info_create, pg_info_destroy, pg_info_get, pg_info_get_data, pg_info_get_global_ranks,
    pg_info_get_group_desc, pg_info_get_rank_map, pg_info_set_data,
)

_enabled = False
_split_seq = 0


def torchcomms_is_enabled() -> bool:
    return _enabled


def _pg_options_to_hints(pg_options: Any) -> Tuple[Dict[str, str], Optional[bool]]:
    """What a ``ProcessGroupNCCL.Options``-like object says, as communicator hints: the scalar fields of its
    ``config`` (NCCL configuration: ``min_ctas``, ``max_ctas``, ``cga_cluster_size``, ``net_name``, ... - the CUDA
    backend hands those to ``ncclCommInitRankConfig``) and its own scalar fields, each as a string; the stream
    priority flag is returned separately.  Parity: ``_pg_options_to_hints`` of
    comms/torchcomms/distwrap/utils.py."""
    hints: Dict[str, str] = {}
    if pg_options is None:
        return hints, None

    def scalars(obj, skip=()):
        for attr in dir(obj):
            if attr.startswith("_") or attr in skip:
                continue
            try:
                value = getattr(obj, attr)
            except Exception:
                continue
            if isinstance(value, (bool, int, float, str)) and value != -2147483648 and value != "":
                yield attr, value        # -2**31 is NCCL's "not set"

    config = getattr(pg_options, "config", None)
    if config is not None:
        for attr, value in scalars(config):
            hints[attr] = str(int(value) if isinstance(value, bool) else value)
    high_priority = None
    for attr, value in scalars(pg_options, skip=("config",)):
        if attr == "is_high_priority_stream":
            high_priority = bool(value)
        else:
            hints[attr] = str(int(value) if isinstance(value, bool) else value)
    return hints, high_priority


def _parse_backend(backend: Optional[str]) -> Dict[str, str]:
    """'gloo' | 'nccl' | 'b200' | 'cpu:gloo,cuda:nccl' -> {device type: communicator backend}."""
    if backend is None:
        out = {"cpu": "gloo"}
        if torch.cuda.is_available():
            out["cuda"] = "b200"
        return out
    out: Dict[str, str] = {}
    for part in str(backend).lower().split(","):
        if ":" in part:
            dev, name = part.split(":", 1)
        else:
            name = part
            dev = "cuda" if name in _CUDA_NAMES else "cpu"
        out[dev.strip()] = "b200" if name.strip() in _CUDA_NAMES else name.strip()
    return out


def _device_for(dev_type: str) -> torch.device:
    if dev_type == "cuda":
        return torch.device("cuda", int(os.environ.get("LOCAL_RANK", "0")))
    return torch.device(dev_type)


def _info(pg: Any) -> _PgInfo:
    pg = pg if pg is not None else GroupMember.WORLD
    if pg not in _REGISTRY:
        raise ValueError("this process group was not created through distwrap")
    return _REGISTRY[pg]


def get_torchcomms_instance(pg: Any = None, tensor: Optional[torch.Tensor] = None, device_type: Optional[str] = None) -> TorchComm:
    comms: Dict[str, TorchComm] = _info(pg).data["torchcomms"]
    want = device_type or (tensor.device.type if tensor is not None else None)
    if want is None or want not in comms:
        if want is not None and len(comms) > 1:
            raise ValueError(f"no communicator for device type '{want}' in this group (have {list(comms)})")
        return next(iter(comms.values()))
    return comms[want]


# ------------------------------------------------------------------ groups ---


def init_process_group(backend: Optional[str] = None, init_method: Optional[str] = None,
                       timeout: Optional[timedelta] = None, world_size: int = -1, rank: int = -1,
                       store: Optional[Store] = None, group_name: str = "", pg_options: Any = None,
                       device_id: Any = None, use_torchcomms: bool = False, **kwargs: Any) -> None:
    global _enabled
    if backend is None:
        raise ValueError("backend must be specified")     # as the reference: no silent default in either mode
    if not use_torchcomms:
        _td.init_process_group(backend=backend, init_method=init_method, timeout=timeout, world_size=world_size,
                               rank=rank, store=store, group_name=group_name, pg_options=pg_options,
                               device_id=device_id)
        # Pass-through groups are registered too, so that rank maps, descriptions and the
        # backend per device type can be looked up the same way in both modes.
        info = pg_info_create(GroupMember.WORLD, list(range(_td.get_world_size())), group_name or "world")
        info.data["device_backends"] = _parse_backend(backend or _td.get_backend())
        return
    if _enabled:
        raise RuntimeError("distwrap is already initialised")
    if rank >= 0:
        os.environ.setdefault("RANK", str(rank))
    if world_size > 0:
        os.environ.setdefault("WORLD_SIZE", str(world_size))
    backends = _parse_backend(backend)
    comms: Dict[str, TorchComm] = {}
    for dev_type, name in backends.items():
        kw: Dict[str, Any] = {}
        if timeout is not None:
            kw["timeout"] = timeout
        if store is not None:
            kw["store"] = _td.PrefixStore(f"distwrap_{dev_type}", store)
        if dev_type == "cuda" and pg_options is not None:
            opt_hints, high_priority = _pg_options_to_hints(pg_options)
            if opt_hints:
                kw["hints"] = opt_hints
            if high_priority is not None:
                kw["is_high_priority_stream"] = high_priority
        comms[dev_type] = new_comm(name, _device_for(dev_type), name=f"{group_name or 'world'}_{dev_type}", **kw)
    first = next(iter(comms.values()))
    # The WORLD group is served by the communicator of the accelerator when there is one.
    main = comms.get("cuda", first)
    pg = wrap_comm_as_process_group(main, group_name or "distwrap_world")
    GroupMember.WORLD = pg
    n = first.get_size()
    _REGISTRY[pg] = _PgInfo(list(range(n)), group_name or "world", {r: r for r in range(n)},
                            {"torchcomms": comms, "device_backends": backends})
    _enabled = True


def _forget_group(pg: Any) -> None:
    """Removes one of our groups from torch.distributed's world tables (other groups stay untouched)."""
    from torch.distributed import distributed_c10d as c10d

    world = c10d._world
    tag = world.pg_to_tag.pop(pg, None)
    if tag is not None and pg in world.tags_to_pg.get(tag, []):
        world.tags_to_pg[tag].remove(pg)
    for table in (world.pg_map, world.pg_names, world.pg_group_ranks, world.pg_backend_config):
        table.pop(pg, None)
    if GroupMember.WORLD is pg:
        GroupMember.WORLD = None


def destroy_process_group(group: Any = None) -> None:
    global _enabled
    if not _enabled:
        for pg in ([group] if group is not None and group is not GroupMember.WORLD else list(_REGISTRY)):
            pg_info_destroy(pg)
        _td.destroy_process_group(group)
        return
    targets = [group] if group is not None and group is not GroupMember.WORLD else list(_REGISTRY)
    for pg in targets:
        info = _REGISTRY.pop(pg, None)
        if info is None:
            continue
        for comm in info.data["torchcomms"].values():
            try:
                comm.finalize()
            except RuntimeError:
                pass
        _forget_group(pg)
    if not _REGISTRY:
        _enabled = False


def new_group(*args: Any, **kwargs: Any) -> Any:
    if _enabled:
        raise AssertionError("new_group() is not available with use_torchcomms=True: use split_group() "
                             "(communicators are split from an existing one)")
    pg = _td.new_group(*args, **kwargs)
    ranks = kwargs.get("ranks", args[0] if args else None)
    ranks = list(ranks) if ranks is not None else list(range(_td.get_world_size()))
    if pg is not None and pg is not GroupMember.NON_GROUP_MEMBER and pg_info_get(pg) is None:
        info = pg_info_create(pg, ranks, kwargs.get("group_desc"))
        info.data["device_backends"] = _parse_backend(kwargs.get("backend") or _td.get_backend())
    return pg


def split_group(parent_pg: Any = None, split_ranks: Optional[Sequence[Sequence[int]]] = None,
                timeout: Optional[timedelta] = None, pg_options: Any = None, group_desc: Optional[str] = None) -> Any:
    """Collective over ``parent_pg``: every member passes the same partition; returns the caller's sub-group (or None)."""
    global _split_seq
    if not _enabled:
        parent = parent_pg if parent_pg is not None else GroupMember.WORLD
        me = _td.get_rank()
        mine = next((list(r) for r in (split_ranks or []) if me in r), None)
        try:
            pg = _td.split_group(parent_pg, split_ranks, timeout, pg_options, group_desc)
        except (RuntimeError, ValueError, AssertionError, NotImplementedError):
            # The backend cannot split (gloo): build the partitions with new_group instead.
            pg = fallback.split_group_via_new_group(parent, mine, timeout, pg_options, group_desc)
        if pg is not None and mine is not None and pg_info_get(pg) is None:
            info = pg_info_create(pg, mine, group_desc)
            info.data["device_backends"] = dict(pg_info_get_data(parent, "device_backends", {}) or {})
        return pg
    parent = _info(parent_pg)
    if not split_ranks:
        raise ValueError("split_ranks is required")
    me_global = parent.global_ranks[next(iter(parent.data["torchcomms"].values())).get_rank()]
    mine: Optional[List[int]] = None
    for ranks in split_ranks:
        if me_global in ranks:
            mine = list(ranks)
    _split_seq += 1
    name = group_desc or f"split{_split_seq}"
    comms: Dict[str, TorchComm] = {}
    for dev_type, comm in parent.data["torchcomms"].items():
        local = [parent.rank_to_group_rank[g] for g in mine] if mine is not None else []
        sub = comm.split(local, f"{name}_{dev_type}")
        if sub is not None:
            comms[dev_type] = sub
    if mine is None or not comms:
        return None
    main = comms.get("cuda", next(iter(comms.values())))
    mapping = {g: i for i, g in enumerate(mine)}
    pg = wrap_comm_as_process_group(main, f"distwrap_{name}_{_split_seq}", mapping)
    _REGISTRY[pg] = _PgInfo(mine, name, mapping, {"torchcomms": comms, "device_backends": parent.data["device_backends"]})
    return pg


def get_rank(group: Any = None) -> int:
    if not _enabled:
        return _td.get_rank(group)
    return next(iter(_info(group).data["torchcomms"].values())).get_rank()


def get_world_size(group: Any = None) -> int:
    if not _enabled:
        return _td.get_world_size(group)
    return next(iter(_info(group).data["torchcomms"].values())).get_size()


def is_initialized() -> bool:
    return _enabled or _td.is_initialized()


def _group_rank(group: Any, global_rank: int) -> int:
    return _info(group).rank_to_group_rank[global_rank]


# ------------------------------------------------------------- collectives ---

_RED = {
    ReduceOp.SUM: _TcReduceOp.SUM, ReduceOp.PRODUCT: _TcReduceOp.PRODUCT, ReduceOp.MIN: _TcReduceOp.MIN,
    ReduceOp.MAX: _TcReduceOp.MAX, ReduceOp.AVG: _TcReduceOp.AVG, ReduceOp.BAND: _TcReduceOp.BAND,
    ReduceOp.BOR: _TcReduceOp.BOR, ReduceOp.BXOR: _TcReduceOp.BXOR,
}


def _red(op: Any) -> Any:
    if isinstance(op, _TcReduceOp):
        return op
    for k, v in _RED.items():
        if op == k:
            return v
    raise NotImplementedError(f"reduce op {op!r}: build PREMUL_SUM with distwrap._make_nccl_premul_sum(factor)")


def _make_nccl_premul_sum(factor: Any) -> Any:
    if _enabled:
        return _TcReduceOp.PREMUL_SUM(factor)
    return _td._make_nccl_premul_sum(factor)


def _ret(work: Any, async_op: bool) -> Any:
    return work if async_op else None


def all_reduce(tensor: torch.Tensor, op: Any = ReduceOp.SUM, group: Any = None, async_op: bool = False) -> Any:
    if not _enabled:
        return _td.all_reduce(tensor, op, group, async_op)
    return _ret(get_torchcomms_instance(group, tensor).all_reduce(tensor, _red(op), async_op), async_op)


def broadcast(tensor: torch.Tensor, src: Optional[int] = None, group: Any = None, async_op: bool = False,
              group_src: Optional[int] = None) -> Any:
    if not _enabled:
        return _td.broadcast(tensor, src=src, group=group, async_op=async_op, group_src=group_src)
    root = group_src if group_src is not None else _group_rank(group, src or 0)
    return _ret(get_torchcomms_instance(group, tensor).broadcast(tensor, root, async_op), async_op)


def reduce(tensor: torch.Tensor, dst: Optional[int] = None, op: Any = ReduceOp.SUM, group: Any = None,
           async_op: bool = False, group_dst: Optional[int] = None) -> Any:
    if not _enabled:
        return _td.reduce(tensor, dst=dst, op=op, group=group, async_op=async_op, group_dst=group_dst)
    root = group_dst if group_dst is not None else _group_rank(group, dst or 0)
    return _ret(get_torchcomms_instance(group, tensor).reduce(tensor, root, _red(op), async_op), async_op)


def all_gather(tensor_list: List[torch.Tensor], tensor: torch.Tensor, group: Any = None, async_op: bool = False) -> Any:
    if not _enabled:
        return _td.all_gather(tensor_list, tensor, group, async_op)
    return _ret(get_torchcomms_instance(group, tensor).all_gather(tensor_list, tensor, async_op), async_op)


def all_gather_into_tensor(output_tensor: torch.Tensor, input_tensor: torch.Tensor, group: Any = None,
                           async_op: bool = False) -> Any:
    if not _enabled:
        return _td.all_gather_into_tensor(output_tensor, input_tensor, group, async_op)
    return _ret(get_torchcomms_instance(group, input_tensor).all_gather_single(output_tensor, input_tensor, async_op), async_op)


def reduce_scatter(output: torch.Tensor, input_list: List[torch.Tensor], op: Any = ReduceOp.SUM, group: Any = None,
                   async_op: bool = False) -> Any:
    if not _enabled:
        return _td.reduce_scatter(output, input_list, op, group, async_op)
    return _ret(get_torchcomms_instance(group, output).reduce_scatter(output, input_list, _red(op), async_op), async_op)


def reduce_scatter_tensor(output: torch.Tensor, input: torch.Tensor, op: Any = ReduceOp.SUM, group: Any = None,
                          async_op: bool = False) -> Any:
    if not _enabled:
        return _td.reduce_scatter_tensor(output, input, op, group, async_op)
    return _ret(get_torchcomms_instance(group, input).reduce_scatter_single(output, input, _red(op), async_op), async_op)


def get_backend_for_device(group: Any = None, device_type: str = "cpu") -> str:
    """Name of the backend that serves tensors of ``device_type`` in ``group`` (both modes)."""
    pg = group if group is not None else GroupMember.WORLD
    backends = pg_info_get_data(pg, "device_backends", {}) or {}
    if device_type in backends:
        return backends[device_type]
    if not _enabled:
        return str(_td.get_backend(pg))
    raise ValueError(f"no backend for device type '{device_type}' in this group (have {list(backends)})")


def _lacks_all_to_all(group: Any, tensor: torch.Tensor) -> bool:
    """Pass-through mode: gloo implements no all-to-all."""
    try:
        return get_backend_for_device(group, tensor.device.type) == "gloo"
    except ValueError:
        return False


def all_to_all(output_tensor_list: List[torch.Tensor], input_tensor_list: List[torch.Tensor], group: Any = None,
               async_op: bool = False) -> Any:
    if not _enabled:
        if _lacks_all_to_all(group, input_tensor_list[0]):
            return fallback.all_to_all_via_p2p(output_tensor_list, input_tensor_list, group, async_op)
        return _td.all_to_all(output_tensor_list, input_tensor_list, group, async_op)
    comm = get_torchcomms_instance(group, input_tensor_list[0])
    return _ret(comm.all_to_all(output_tensor_list, input_tensor_list, async_op), async_op)


def all_to_all_single(output: torch.Tensor, input: torch.Tensor, output_split_sizes: Optional[List[int]] = None,
                      input_split_sizes: Optional[List[int]] = None, group: Any = None, async_op: bool = False) -> Any:
    if not _enabled:
        if _lacks_all_to_all(group, input):
            return fallback.all_to_all_single_via_p2p(output, input, output_split_sizes, input_split_sizes, group, async_op)
        return _td.all_to_all_single(output, input, output_split_sizes, input_split_sizes, group, async_op)
    comm = get_torchcomms_instance(group, input)
    if not output_split_sizes and not input_split_sizes:
        return _ret(comm.all_to_all_single(output, input, async_op), async_op)
    n = comm.get_size()
    outs = list(output_split_sizes) if output_split_sizes else [output.size(0) // n] * n
    ins = list(input_split_sizes) if input_split_sizes else [input.size(0) // n] * n
    return _ret(comm.all_to_all_v_single(output, input, outs, ins, async_op), async_op)


def scatter(tensor: torch.Tensor, scatter_list: Optional[List[torch.Tensor]] = None, src: Optional[int] = None,
            group: Any = None, async_op: bool = False, group_src: Optional[int] = None) -> Any:
    if not _enabled:
        return _td.scatter(tensor, scatter_list, src=src, group=group, async_op=async_op, group_src=group_src)
    root = group_src if group_src is not None else _group_rank(group, src or 0)
    return _ret(get_torchcomms_instance(group, tensor).scatter(tensor, scatter_list or [], root, async_op), async_op)


def gather(tensor: torch.Tensor, gather_list: Optional[List[torch.Tensor]] = None, dst: Optional[int] = None,
           group: Any = None, async_op: bool = False, group_dst: Optional[int] = None) -> Any:
    if not _enabled:
        return _td.gather(tensor, gather_list, dst=dst, group=group, async_op=async_op, group_dst=group_dst)
    root = group_dst if group_dst is not None else _group_rank(group, dst or 0)
    return _ret(get_torchcomms_instance(group, tensor).gather(gather_list or [], tensor, root, async_op), async_op)


def barrier(group: Any = None, async_op: bool = False, device_ids: Any = None) -> Any:
    if not _enabled:
        return _td.barrier(group, async_op, device_ids)
    info = _info(group)
    comm = info.data["torchcomms"].get("cuda") or next(iter(info.data["torchcomms"].values()))
    return _ret(comm.barrier(async_op), async_op)


# ---------------------------------------------------------- point to point ---


def send(tensor: torch.Tensor, dst: Optional[int] = None, group: Any = None, tag: int = 0,
         group_dst: Optional[int] = None) -> None:
    if not _enabled:
        return _td.send(tensor, dst=dst, group=group, tag=tag, group_dst=group_dst)
    peer = group_dst if group_dst is not None else _group_rank(group, dst)
    get_torchcomms_instance(group, tensor).send(tensor, peer, False)


def recv(tensor: torch.Tensor, src: Optional[int] = None, group: Any = None, tag: int = 0,
         group_src: Optional[int] = None) -> int:
    if not _enabled:
        return _td.recv(tensor, src=src, group=group, tag=tag, group_src=group_src)
    if src is None and group_src is None:
        raise NotImplementedError("recv from any source is not available on communicators")
    peer = group_src if group_src is not None else _group_rank(group, src)
    get_torchcomms_instance(group, tensor).recv(tensor, peer, False)
    return src if src is not None else _info(group).global_ranks[peer]


def isend(tensor: torch.Tensor, dst: Optional[int] = None, group: Any = None, tag: int = 0,
          group_dst: Optional[int] = None) -> Any:
    if not _enabled:
        return _td.isend(tensor, dst=dst, group=group, tag=tag, group_dst=group_dst)
    peer = group_dst if group_dst is not None else _group_rank(group, dst)
    return get_torchcomms_instance(group, tensor).send(tensor, peer, True)


def irecv(tensor: torch.Tensor, src: Optional[int] = None, group: Any = None, tag: int = 0,
          group_src: Optional[int] = None) -> Any:
    if not _enabled:
        return _td.irecv(tensor, src=src, group=group, tag=tag, group_src=group_src)
    peer = group_src if group_src is not None else _group_rank(group, src)
    return get_torchcomms_instance(group, tensor).recv(tensor, peer, True)


class P2POp:
    """``P2POp(dist.isend | dist.irecv, tensor, peer, group)`` for ``batch_isend_irecv``."""

    def __init__(self, op: Any, tensor: torch.Tensor, peer: Optional[int] = None, group: Any = None, tag: int = 0,
                 group_peer: Optional[int] = None):
        self.op, self.tensor, self.peer, self.group, self.tag, self.group_peer = op, tensor, peer, group, tag, group_peer
        self._p2p_op = None
        if not _enabled:
            native = {isend: _td.isend, irecv: _td.irecv}.get(op, op)
            self._p2p_op = _td.P2POp(native, tensor, peer, group, tag, group_peer)

    def __repr__(self) -> str:
        return repr(self._p2p_op) if self._p2p_op is not None else f"P2POp({self.op.__name__}, peer={self.peer})"


def batch_isend_irecv(p2p_op_list: List[P2POp]) -> List[Any]:
    if not _enabled:
        return _td.batch_isend_irecv([p._p2p_op for p in p2p_op_list])
    if not p2p_op_list:
        return []
    grp = p2p_op_list[0].group
    comm = get_torchcomms_instance(grp, p2p_op_list[0].tensor)
    batch = comm.batch_op_create()
    for p in p2p_op_list:
        peer = p.group_peer if p.group_peer is not None else _group_rank(p.group, p.peer)
        if p.op in (isend, _td.isend):
            batch.send(p.tensor, peer)
        else:
            batch.recv(p.tensor, peer)
    return [batch.issue(True)]


# ------------------------------------------------------ object collectives ---


def all_gather_object(object_list: List[Any], obj: Any, group: Any = None) -> None:
    if not _enabled:
        return _td.all_gather_object(object_list, obj, group)
    objcol.all_gather_object(get_torchcomms_instance(group), object_list, obj)


def gather_object(obj: Any, object_gather_list: Optional[List[Any]] = None, dst: Optional[int] = None, group: Any = None,
                  group_dst: Optional[int] = None) -> None:
    if not _enabled:
        return _td.gather_object(obj, object_gather_list, dst=dst, group=group, group_dst=group_dst)
    root = group_dst if group_dst is not None else _group_rank(group, dst or 0)
    objcol.gather_object(get_torchcomms_instance(group), obj, root, object_gather_list=object_gather_list)


def broadcast_object_list(object_list: List[Any], src: Optional[int] = None, group: Any = None, device: Any = None,
                          group_src: Optional[int] = None) -> None:
    if not _enabled:
        return _td.broadcast_object_list(object_list, src=src, group=group, device=device, group_src=group_src)
    root = group_src if group_src is not None else _group_rank(group, src or 0)
    objcol.broadcast_object_list(get_torchcomms_instance(group), object_list, root)


def scatter_object_list(scatter_object_output_list: List[Any], scatter_object_input_list: Optional[List[Any]] = None,
                        src: Optional[int] = None, group: Any = None, group_src: Optional[int] = None) -> None:
    if not _enabled:
        return _td.scatter_object_list(scatter_object_output_list, scatter_object_input_list, src=src, group=group,
                                       group_src=group_src)
    root = group_src if group_src is not None else _group_rank(group, src or 0)
    objcol.scatter_object_list(get_torchcomms_instance(group), root, scatter_object_output_list,
                               scatter_object_input_list=scatter_object_input_list)


# -------------------------------------------------------------- extensions ---


def new_window(group: Any = None, device_type: str = "cuda") -> Any:
    """One-sided window on the group's communicator (communicator-only extension)."""
    if not _enabled:
        raise NotImplementedError("new_window needs init_process_group(use_torchcomms=True)")
    return get_torchcomms_instance(group, device_type=device_type).new_window()


def reduce_scatter_quantized(output: torch.Tensor, input: torch.Tensor, op: Any = ReduceOp.SUM, seed: int = 0,
                             group: Any = None, async_op: bool = False) -> Any:
    """fp32 reduce-scatter whose wire format is bf16 (communicator-only extension)."""
    if not _enabled:
        raise NotImplementedError("reduce_scatter_quantized needs init_process_group(use_torchcomms=True)")
    comm = get_torchcomms_instance(group, input)
    return _ret(comm.get_backend_impl().reduce_scatter_quantized(output, input, _red(op), seed=seed, async_op=async_op), async_op)


def get_mem_allocator(group: Any = None, device: Any = None) -> Any:
    if not _enabled:
        raise NotImplementedError("get_mem_allocator needs init_process_group(use_torchcomms=True)")
    return _tc_get_mem_allocator(_info(group).data["device_backends"].get("cuda", "b200"))


def register_mem_pool(pool: Any, group: Any = None) -> None:
    """Memory from the communicator's allocator is peer-mapped when it is allocated; nothing to do per pool."""
    return None


def __getattr__(name: str) -> Any:
    # Anything not wrapped here (ProcessGroupGloo, TCPStore, ...) comes from torch.distributed.
    return getattr(_td, name)
