"""Registry of the process groups this module created: global ranks, the
global -> group rank map, a description, and a free-form data dict (the
communicators per device type, the backend per device type).

Parity: comms/torchcomms/distwrap/pginfo.py:15-92.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional


@dataclass
class PgInfo:
    global_ranks: List[int]
    group_desc: str
    rank_to_group_rank: Dict[int, int]
    data: Dict[str, Any] = field(default_factory=dict)


_REGISTRY: Dict[Any, PgInfo] = {}


def pg_info_create(pg: Any, global_ranks: List[int], group_desc: Optional[str] = None) -> PgInfo:
    if pg in _REGISTRY:
        raise ValueError("process group is already registered")
    info = PgInfo(list(global_ranks), group_desc or "", {g: i for i, g in enumerate(global_ranks)})
    _REGISTRY[pg] = info
    return info


def pg_info_destroy(pg: Any) -> Optional[PgInfo]:
    return _REGISTRY.pop(pg, None)


def pg_info_get(pg: Any) -> Optional[PgInfo]:
    return _REGISTRY.get(pg)


def pg_info_assert_registered(pg: Any) -> PgInfo:
    info = _REGISTRY.get(pg)
    if info is None:
        raise ValueError("this process group was not created through distwrap")
    return info


def pg_info_get_global_ranks(pg: Any) -> List[int]:
    return list(pg_info_assert_registered(pg).global_ranks)


def pg_info_get_rank_map(pg: Any) -> Dict[int, int]:
    return dict(pg_info_assert_registered(pg).rank_to_group_rank)


def pg_info_get_group_desc(pg: Any) -> str:
    return pg_info_assert_registered(pg).group_desc


def pg_info_set_data(pg: Any, key: str, value: Any) -> None:
    pg_info_assert_registered(pg).data[key] = value


def pg_info_get_data(pg: Any, key: str, default: Any = None) -> Any:
    return pg_info_assert_registered(pg).data.get(key, default)


def registered_groups() -> List[Any]:
    return list(_REGISTRY)


__all__ = ["PgInfo", "pg_info_create", "pg_info_destroy", "pg_info_get", "pg_info_assert_registered",
           "pg_info_get_global_ranks", "pg_info_get_rank_map", "pg_info_get_group_desc", "pg_info_set_data",
           "pg_info_get_data", "registered_groups"]
