"""Turns the loosely typed arguments callers pass to collectives into the plain
values operator schemas can carry (strings, ints, lists of ints).

* reduce operations: ``ReduceOp`` members, their names in any case, c10d's
  ``ReduceOp``, and ``PREMUL_SUM`` with its factor (``"premul_sum:0.5"``)
* timeouts: ``timedelta``, seconds as a number, or ``None``
* hints: any mapping, stringified; ``None`` becomes an empty dict

``CollectiveSchema`` binds positional and keyword arguments of a call to the
parameter list of an operator, applies those conversions and reports mistakes
with the operator's name.

Parity: comms/torchcomms/functional/param_parsing.py (``ParamKind``,
``ParamSpec``, ``ParsedArgs``, ``CollectiveParamSchema``).
"""
from __future__ import annotations

from dataclasses import dataclass, field
from datetime import timedelta
from enum import Enum
from typing import Any, Dict, List, Mapping, Optional, Sequence, Tuple

import torch

_NAMES = {"sum", "avg", "max", "min", "product", "band", "bor", "bxor"}


def normalize_reduce_op(op: Any) -> str:
    """Canonical lower-case name; PREMUL_SUM carries its factor: ``"premul_sum:<factor>"``."""
    if isinstance(op, str):
        low = op.lower()
        if low in _NAMES:
            return low
        if low.startswith("premul_sum:"):
            float(low.split(":", 1)[1])  # raises on a malformed factor
            return low
        raise ValueError(f"unknown reduce op '{op}'")
    name = getattr(op, "name", None)
    if callable(name):
        name = name()
    if name is None:
        name = str(op).split(".")[-1]
    low = str(name).lower()
    if low == "premul_sum":
        factor = getattr(op, "factor", None)
        factor = factor() if callable(factor) else factor
        if isinstance(factor, torch.Tensor):
            factor = float(factor.item())
        if factor is None:
            raise ValueError("PREMUL_SUM needs a factor")
        return f"premul_sum:{float(factor)}"
    if low in _NAMES:
        return low
    raise ValueError(f"unknown reduce op '{op}'")


def reduce_op_from_string(name: str):
    """The communicator's ``ReduceOp`` for a canonical name."""
    from .. import ReduceOp

    low = normalize_reduce_op(name)
    if low.startswith("premul_sum:"):
        return ReduceOp.PREMUL_SUM(float(low.split(":", 1)[1]))
    return {"sum": ReduceOp.SUM, "avg": ReduceOp.AVG, "max": ReduceOp.MAX, "min": ReduceOp.MIN, "product": ReduceOp.PRODUCT,
            "band": ReduceOp.BAND, "bor": ReduceOp.BOR, "bxor": ReduceOp.BXOR}[low]


def parse_timeout(t: Any) -> Optional[float]:
    """Seconds as a float, or None for the communicator's default."""
    if t is None:
        return None
    if isinstance(t, timedelta):
        return t.total_seconds()
    if isinstance(t, (int, float)) and not isinstance(t, bool):
        if t < 0:
            raise ValueError("timeout must not be negative")
        return float(t)
    raise TypeError(f"timeout must be a timedelta or a number of seconds, got {type(t).__name__}")


def parse_hints(h: Optional[Mapping[Any, Any]]) -> Dict[str, str]:
    if h is None:
        return {}
    if not isinstance(h, Mapping):
        raise TypeError(f"hints must be a mapping, got {type(h).__name__}")
    return {str(k): ("1" if v is True else "0" if v is False else str(v)) for k, v in h.items()}


class ParamKind(Enum):
    TENSOR = "tensor"
    TENSOR_LIST = "tensor_list"
    INT = "int"
    INT_LIST = "int_list"
    BOOL = "bool"
    REDUCE_OP = "reduce_op"
    COMM = "comm"
    TIMEOUT = "timeout"
    HINTS = "hints"


@dataclass
class ParamSpec:
    name: str
    kind: ParamKind
    default: Any = field(default_factory=lambda: ParamSpec.REQUIRED)
    mutated: bool = False   # written by the in-place form of the operator

    REQUIRED = object()

    @property
    def required(self) -> bool:
        return self.default is ParamSpec.REQUIRED


@dataclass
class ParsedArgs:
    values: Dict[str, Any]

    def __getitem__(self, key: str) -> Any:
        return self.values[key]

    def tensors(self, schema: "CollectiveSchema") -> List[torch.Tensor]:
        out: List[torch.Tensor] = []
        for p in schema.params:
            v = self.values[p.name]
            if p.kind is ParamKind.TENSOR and v is not None:
                out.append(v)
            elif p.kind is ParamKind.TENSOR_LIST:
                out.extend(v)
        return out


class CollectiveSchema:
    def __init__(self, op_name: str, params: Sequence[ParamSpec]):
        self.op_name = op_name
        self.params = list(params)
        seen = set()
        for p in self.params:
            if p.name in seen:
                raise ValueError(f"{op_name}: duplicate parameter '{p.name}'")
            seen.add(p.name)

    def mutated(self) -> List[str]:
        return [p.name for p in self.params if p.mutated]

    def bind(self, args: Tuple[Any, ...], kwargs: Mapping[str, Any]) -> ParsedArgs:
        if len(args) > len(self.params):
            raise TypeError(f"{self.op_name}: takes at most {len(self.params)} arguments, got {len(args)}")
        values: Dict[str, Any] = {}
        for p, v in zip(self.params, args):
            values[p.name] = v
        for k, v in kwargs.items():
            if k in values:
                raise TypeError(f"{self.op_name}: got multiple values for '{k}'")
            if all(p.name != k for p in self.params):
                raise TypeError(f"{self.op_name}: unexpected argument '{k}'")
            values[k] = v
        for p in self.params:
            if p.name not in values:
                if p.required:
                    raise TypeError(f"{self.op_name}: missing argument '{p.name}'")
                values[p.name] = p.default
            values[p.name] = self._convert(p, values[p.name])
        return ParsedArgs(values)

    def _convert(self, p: ParamSpec, v: Any) -> Any:
        k = p.kind
        try:
            if k is ParamKind.TENSOR:
                if v is not None and not isinstance(v, torch.Tensor):
                    raise TypeError("expected a tensor")
                return v
            if k is ParamKind.TENSOR_LIST:
                v = list(v)
                if not all(isinstance(t, torch.Tensor) for t in v):
                    raise TypeError("expected a list of tensors")
                return v
            if k is ParamKind.INT:
                if isinstance(v, bool) or not isinstance(v, int):
                    raise TypeError("expected an int")
                return v
            if k is ParamKind.INT_LIST:
                return None if v is None else [int(x) for x in v]
            if k is ParamKind.BOOL:
                return bool(v)
            if k is ParamKind.REDUCE_OP:
                return normalize_reduce_op(v)
            if k is ParamKind.COMM:
                return v if isinstance(v, str) else v.get_name()
            if k is ParamKind.TIMEOUT:
                return parse_timeout(v)
            if k is ParamKind.HINTS:
                return parse_hints(v)
        except (TypeError, ValueError) as exc:
            raise type(exc)(f"{self.op_name}: argument '{p.name}': {exc}") from None
        return v


__all__ = ["normalize_reduce_op", "reduce_op_from_string", "parse_timeout", "parse_hints", "ParamKind", "ParamSpec",
           "ParsedArgs", "CollectiveSchema"]
