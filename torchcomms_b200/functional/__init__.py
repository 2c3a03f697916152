"""Functional (traceable, differentiable) collectives as ``torch.ops.torchcomms_b200.*``.

Communicators are opaque to the tracer, so the ops take the communicator's
*name* and look it up in a process-wide registry::

    from torchcomms_b200 import functional as F
    F.register_comm(comm)                              # once per communicator
    y = F.all_reduce(x, "sum", comm)                   # out-of-place, differentiable
    g = F.all_gather_single(x_shard, comm)             # [n*rows, ...]
    s = F.reduce_scatter_single(x, "sum", comm)        # [rows/n, ...]
    F.all_reduce_(x, "sum", comm)                      # in-place variant

Every op is a ``torch.library`` custom op with a fake (meta) implementation,
so ``torch.compile`` / ``make_fx`` / ``torch.export`` trace through them
without running a collective, and an autograd formula (all-reduce <->
all-reduce, all-gather <-> reduce-scatter, all-to-all <-> all-to-all with the
splits swapped, broadcast -> reduce to root).  The ops run synchronously with
respect to the caller's stream (stream-ordered ``wait``), so no separate
``wait_tensor`` is needed; one is provided as an identity for code written
against functional-collective APIs.

Code that calls methods of the communicator object itself compiles after
``functional.dynamo.register_with_dynamo()``; ``functional.inductor.
register_with_inductor()`` adds Inductor lowerings (in-place all-reduce and
broadcast kernels, start / wait kernels that keep a started collective's
input alive).  Without the latter the operators run as opaque functional calls
inside compiled graphs, which is correct but copies more.

Parity: comms/torchcomms/functional/{registry,collectives,async_tensor,
param_parsing,dynamo,inductor_lowering,passes}.py.  Overlap in this framework
comes from CUDA streams and graphs rather than from a tracing compiler, so the
compile path is kept correct and cheap, not tuned.
"""
from __future__ import annotations

import os
from typing import Dict, List, Optional, Union

import torch
from torch import Tensor

from .. import ReduceOp, TorchComm

NAMESPACE = "torchcomms_b200"
MIN_PYTORCH_VERSION_FOR_COMPILE = "2.4.0"

_comms: Dict[str, TorchComm] = {}


def is_torch_compile_supported(min_version: str = MIN_PYTORCH_VERSION_FOR_COMPILE, _current_version: Optional[str] = None) -> bool:
    from packaging import version

    cur = _current_version or torch.__version__
    if os.environ.get("TORCHCOMMS_COMPILE_IGNORE_PYTORCH_VERSION_REQUIREMENT") == "1":
        return True
    return version.parse(cur.split("+")[0]) >= version.parse(min_version)


def is_torch_compile_supported_and_enabled(min_version: str = MIN_PYTORCH_VERSION_FOR_COMPILE,
                                           _current_version: Optional[str] = None) -> bool:
    return is_torch_compile_supported(min_version, _current_version) and os.environ.get("TORCHCOMMS_PATCH_FOR_COMPILE") == "1"


def register_comm(comm: TorchComm, name: Optional[str] = None) -> str:
    key = name or comm.get_name()
    _comms[key] = comm
    return key


def unregister_comm(comm_or_name: Union[TorchComm, str]) -> None:
    key = comm_or_name if isinstance(comm_or_name, str) else comm_or_name.get_name()
    _comms.pop(key, None)


def _name(comm: Union[TorchComm, str]) -> str:
    if isinstance(comm, str):
        return comm
    key = comm.get_name()
    if key not in _comms:
        _comms[key] = comm
    return key


def _get(name: str) -> TorchComm:
    try:
        return _comms[name]
    except KeyError:
        raise RuntimeError(f"communicator '{name}' is not registered: call functional.register_comm(comm)") from None


_REDS = {"sum": ReduceOp.SUM, "avg": ReduceOp.AVG, "max": ReduceOp.MAX, "min": ReduceOp.MIN, "product": ReduceOp.PRODUCT}


def _red(op: str) -> ReduceOp:
    try:
        return _REDS[op.lower()]
    except KeyError:
        raise ValueError(f"unknown reduce op '{op}' (expected one of {sorted(_REDS)})") from None


# ------------------------------------------------------------ op definitions ---

_lib = torch.library.Library(NAMESPACE, "FRAGMENT")  # keeps the definitions alive
_lib.define("all_reduce(Tensor input, str op, str comm) -> Tensor")
_lib.define("all_reduce_(Tensor(a!) input, str op, str comm) -> Tensor(a!)")
_lib.define("all_gather_single(Tensor input, str comm) -> Tensor")
_lib.define("reduce_scatter_single(Tensor input, str op, str comm) -> Tensor")
_lib.define("all_to_all_single(Tensor input, int[]? output_split_sizes, int[]? input_split_sizes, str comm) -> Tensor")
_lib.define("broadcast(Tensor input, int root, str comm) -> Tensor")
_lib.define("broadcast_(Tensor(a!) input, int root, str comm) -> Tensor(a!)")
_lib.define("reduce(Tensor input, int root, str op, str comm) -> Tensor")
_lib.define("barrier(Tensor token, str comm) -> Tensor")
_lib.define("wait_tensor(Tensor input) -> Tensor")


def _size(name: str) -> int:
    return _get(name).get_size()


def _impl_all_reduce(input: Tensor, op: str, comm: str) -> Tensor:
    out = input.contiguous().clone()
    _get(comm).all_reduce(out, _red(op), False)
    return out


def _impl_all_reduce_(input: Tensor, op: str, comm: str) -> Tensor:
    _get(comm).all_reduce(input, _red(op), False)
    return input


def _impl_all_gather_single(input: Tensor, comm: str) -> Tensor:
    c = _get(comm)
    x = input.contiguous()
    out = x.new_empty((x.shape[0] * c.get_size(),) + tuple(x.shape[1:]))
    c.all_gather_single(out, x, False)
    return out


def _impl_reduce_scatter_single(input: Tensor, op: str, comm: str) -> Tensor:
    c = _get(comm)
    x = input.contiguous()
    out = x.new_empty((x.shape[0] // c.get_size(),) + tuple(x.shape[1:]))
    c.reduce_scatter_single(out, x, _red(op), False)
    return out


def _impl_all_to_all_single(input: Tensor, output_split_sizes: Optional[List[int]], input_split_sizes: Optional[List[int]],
                            comm: str) -> Tensor:
    c = _get(comm)
    x = input.contiguous()
    if not output_split_sizes and not input_split_sizes:
        out = torch.empty_like(x)
        c.all_to_all_single(out, x, False)
        return out
    n = c.get_size()
    ins = list(input_split_sizes) if input_split_sizes else [x.shape[0] // n] * n
    outs = list(output_split_sizes) if output_split_sizes else [x.shape[0] // n] * n
    out = x.new_empty((sum(outs),) + tuple(x.shape[1:]))
    c.all_to_all_v_single(out, x, outs, ins, False)
    return out


def _impl_broadcast(input: Tensor, root: int, comm: str) -> Tensor:
    out = input.contiguous().clone()
    _get(comm).broadcast(out, root, False)
    return out


def _impl_broadcast_(input: Tensor, root: int, comm: str) -> Tensor:
    _get(comm).broadcast(input, root, False)
    return input


def _impl_reduce(input: Tensor, root: int, op: str, comm: str) -> Tensor:
    out = input.contiguous().clone()
    _get(comm).reduce(out, root, _red(op), False)
    return out


def _impl_barrier(token: Tensor, comm: str) -> Tensor:
    _get(comm).barrier(False)
    return token.clone()


def _impl_wait_tensor(input: Tensor) -> Tensor:
    # Results of the *_start operators carry a work handle until somebody waits for them.
    from .ext import wait_pending

    wait_pending(input)
    return input.clone()


for _op, _fn in (("all_reduce", _impl_all_reduce), ("all_reduce_", _impl_all_reduce_),
                 ("all_gather_single", _impl_all_gather_single), ("reduce_scatter_single", _impl_reduce_scatter_single),
                 ("all_to_all_single", _impl_all_to_all_single), ("broadcast", _impl_broadcast),
                 ("broadcast_", _impl_broadcast_), ("reduce", _impl_reduce), ("barrier", _impl_barrier),
                 ("wait_tensor", _impl_wait_tensor)):
    _lib.impl(_op, _fn, "CompositeExplicitAutograd")


# ------------------------------------------------------- fake implementations ---


@torch.library.register_fake(f"{NAMESPACE}::all_reduce")
def _fake_all_reduce(input, op, comm):
    return torch.empty_like(input, memory_format=torch.contiguous_format)


@torch.library.register_fake(f"{NAMESPACE}::all_reduce_")
def _fake_all_reduce_(input, op, comm):
    return input


@torch.library.register_fake(f"{NAMESPACE}::all_gather_single")
def _fake_all_gather_single(input, comm):
    return input.new_empty((input.shape[0] * _size(comm),) + tuple(input.shape[1:]))


@torch.library.register_fake(f"{NAMESPACE}::reduce_scatter_single")
def _fake_reduce_scatter_single(input, op, comm):
    return input.new_empty((input.shape[0] // _size(comm),) + tuple(input.shape[1:]))


@torch.library.register_fake(f"{NAMESPACE}::all_to_all_single")
def _fake_all_to_all_single(input, output_split_sizes, input_split_sizes, comm):
    if output_split_sizes:
        return input.new_empty((sum(output_split_sizes),) + tuple(input.shape[1:]))
    return torch.empty_like(input, memory_format=torch.contiguous_format)


@torch.library.register_fake(f"{NAMESPACE}::broadcast")
def _fake_broadcast(input, root, comm):
    return torch.empty_like(input, memory_format=torch.contiguous_format)


@torch.library.register_fake(f"{NAMESPACE}::broadcast_")
def _fake_broadcast_(input, root, comm):
    return input


@torch.library.register_fake(f"{NAMESPACE}::reduce")
def _fake_reduce(input, root, op, comm):
    return torch.empty_like(input, memory_format=torch.contiguous_format)


@torch.library.register_fake(f"{NAMESPACE}::barrier")
def _fake_barrier(token, comm):
    return torch.empty_like(token)


@torch.library.register_fake(f"{NAMESPACE}::wait_tensor")
def _fake_wait_tensor(input):
    return torch.empty_like(input)


# ------------------------------------------------------------------ autograd ---

_ops = getattr(torch.ops, NAMESPACE)


def _setup(ctx, inputs, output):
    ctx.args = inputs[1:]


def _bw_all_reduce(ctx, grad):
    op, comm = ctx.args
    if op.lower() not in ("sum", "avg"):
        raise RuntimeError(f"all_reduce with op '{op}' is not differentiable")
    return _ops.all_reduce(grad.contiguous(), op, comm), None, None


def _bw_all_gather_single(ctx, grad):
    (comm,) = ctx.args
    return _ops.reduce_scatter_single(grad.contiguous(), "sum", comm), None


def _bw_reduce_scatter_single(ctx, grad):
    op, comm = ctx.args
    g = _ops.all_gather_single(grad.contiguous(), comm)
    if op.lower() == "avg":
        g = g / _size(comm)
    elif op.lower() != "sum":
        raise RuntimeError(f"reduce_scatter_single with op '{op}' is not differentiable")
    return g, None, None


def _bw_all_to_all_single(ctx, grad):
    outs, ins, comm = ctx.args
    return _ops.all_to_all_single(grad.contiguous(), ins, outs, comm), None, None, None


def _bw_broadcast(ctx, grad):
    root, comm = ctx.args
    g = _ops.reduce(grad.contiguous(), root, "sum", comm)
    if _get(comm).get_rank() != root:
        g = torch.zeros_like(g)
    return g, None, None


def _bw_reduce(ctx, grad):
    root, op, comm = ctx.args
    return _ops.broadcast(grad.contiguous(), root, comm), None, None, None


def _bw_identity(ctx, grad):
    return (grad,) + (None,) * len(ctx.args)


torch.library.register_autograd(f"{NAMESPACE}::all_reduce", _bw_all_reduce, setup_context=_setup)
torch.library.register_autograd(f"{NAMESPACE}::all_gather_single", _bw_all_gather_single, setup_context=_setup)
torch.library.register_autograd(f"{NAMESPACE}::reduce_scatter_single", _bw_reduce_scatter_single, setup_context=_setup)
torch.library.register_autograd(f"{NAMESPACE}::all_to_all_single", _bw_all_to_all_single, setup_context=_setup)
torch.library.register_autograd(f"{NAMESPACE}::broadcast", _bw_broadcast, setup_context=_setup)
torch.library.register_autograd(f"{NAMESPACE}::reduce", _bw_reduce, setup_context=_setup)
torch.library.register_autograd(f"{NAMESPACE}::wait_tensor", _bw_identity, setup_context=_setup)


# ------------------------------------------------------------- Python surface ---


def all_reduce(x: Tensor, op: str, comm: Union[TorchComm, str]) -> Tensor:
    return _ops.all_reduce(x, op, _name(comm))


def all_reduce_(x: Tensor, op: str, comm: Union[TorchComm, str]) -> Tensor:
    return _ops.all_reduce_(x, op, _name(comm))


def all_gather_single(x: Tensor, comm: Union[TorchComm, str]) -> Tensor:
    return _ops.all_gather_single(x, _name(comm))


def reduce_scatter_single(x: Tensor, op: str, comm: Union[TorchComm, str]) -> Tensor:
    return _ops.reduce_scatter_single(x, op, _name(comm))


def all_to_all_single(x: Tensor, comm: Union[TorchComm, str], output_split_sizes: Optional[List[int]] = None,
                      input_split_sizes: Optional[List[int]] = None) -> Tensor:
    return _ops.all_to_all_single(x, output_split_sizes, input_split_sizes, _name(comm))


def broadcast(x: Tensor, root: int, comm: Union[TorchComm, str]) -> Tensor:
    return _ops.broadcast(x, root, _name(comm))


def broadcast_(x: Tensor, root: int, comm: Union[TorchComm, str]) -> Tensor:
    return _ops.broadcast_(x, root, _name(comm))


def reduce(x: Tensor, root: int, op: str, comm: Union[TorchComm, str]) -> Tensor:
    return _ops.reduce(x, root, op, _name(comm))


def barrier(comm: Union[TorchComm, str], token: Optional[Tensor] = None) -> Tensor:
    return _ops.barrier(token if token is not None else torch.zeros(()), _name(comm))


def wait_tensor(x: Tensor) -> Tensor:
    return _ops.wait_tensor(x)


# ------------------------------------------------- point-to-point, gather, scatter ---
# Registered after the collectives above with the same three parts (implementation,
# fake, autograd).  `send` returns its input so that the call has a result the
# graph can depend on; its gradient is received from the destination.  `recv`
# takes a tensor that only gives shape and dtype; its gradient is sent back to
# the source.  Pairs of ranks must issue matching calls in the same order in the
# backward pass as they did (mirrored) in the forward pass.

_lib.define("send(Tensor input, int dst, str comm) -> Tensor")
_lib.define("recv(Tensor like, int src, str comm) -> Tensor")
_lib.define("gather_single(Tensor input, int root, str comm) -> Tensor")
_lib.define("scatter(Tensor input, int root, str comm) -> Tensor")


def _impl_send(input: Tensor, dst: int, comm: str) -> Tensor:
    x = input.contiguous()
    _get(comm).send(x, dst, False)
    return x.clone()


def _impl_recv(like: Tensor, src: int, comm: str) -> Tensor:
    out = torch.empty_like(like, memory_format=torch.contiguous_format)
    _get(comm).recv(out, src, False)
    return out


def _impl_gather_single(input: Tensor, root: int, comm: str) -> Tensor:
    c = _get(comm)
    x = input.contiguous()
    out = x.new_zeros((x.shape[0] * c.get_size(),) + tuple(x.shape[1:]))   # meaningful on the root only
    c.gather_single(out, x, root, False)
    return out


def _impl_scatter(input: Tensor, root: int, comm: str) -> Tensor:
    c = _get(comm)
    n = c.get_size()
    x = input.contiguous()
    out = x.new_empty((x.shape[0] // n,) + tuple(x.shape[1:]))
    c.scatter(out, list(x.chunk(n, 0)) if c.get_rank() == root else [], root, False)
    return out


for _op, _fn in (("send", _impl_send), ("recv", _impl_recv), ("gather_single", _impl_gather_single), ("scatter", _impl_scatter)):
    _lib.impl(_op, _fn, "CompositeExplicitAutograd")


@torch.library.register_fake(f"{NAMESPACE}::send")
def _fake_send(input, dst, comm):
    return torch.empty_like(input, memory_format=torch.contiguous_format)


@torch.library.register_fake(f"{NAMESPACE}::recv")
def _fake_recv(like, src, comm):
    return torch.empty_like(like, memory_format=torch.contiguous_format)


@torch.library.register_fake(f"{NAMESPACE}::gather_single")
def _fake_gather_single(input, root, comm):
    return input.new_empty((input.shape[0] * _size(comm),) + tuple(input.shape[1:]))


@torch.library.register_fake(f"{NAMESPACE}::scatter")
def _fake_scatter(input, root, comm):
    return input.new_empty((input.shape[0] // _size(comm),) + tuple(input.shape[1:]))


def _bw_send(ctx, grad):
    dst, comm = ctx.args
    return _ops.recv(grad.contiguous(), dst, comm), None, None


def _bw_recv(ctx, grad):
    src, comm = ctx.args
    _ops.send(grad.contiguous(), src, comm)
    return None, None, None


def _bw_gather_single(ctx, grad):
    root, comm = ctx.args
    return _ops.scatter(grad.contiguous(), root, comm), None, None


def _bw_scatter(ctx, grad):
    root, comm = ctx.args
    return _ops.gather_single(grad.contiguous(), root, comm), None, None


torch.library.register_autograd(f"{NAMESPACE}::send", _bw_send, setup_context=_setup)
torch.library.register_autograd(f"{NAMESPACE}::recv", _bw_recv, setup_context=_setup)
torch.library.register_autograd(f"{NAMESPACE}::gather_single", _bw_gather_single, setup_context=_setup)
torch.library.register_autograd(f"{NAMESPACE}::scatter", _bw_scatter, setup_context=_setup)


def send(x: Tensor, dst: int, comm: Union[TorchComm, str]) -> Tensor:
    """Sends ``x`` to ``dst``; returns a copy of ``x`` whose gradient arrives from ``dst``."""
    return _ops.send(x, dst, _name(comm))


def recv(like: Tensor, src: int, comm: Union[TorchComm, str]) -> Tensor:
    """Receives a tensor shaped like ``like`` from ``src``; its gradient is sent back to ``src``."""
    return _ops.recv(like, src, _name(comm))


def gather_single(x: Tensor, root: int, comm: Union[TorchComm, str]) -> Tensor:
    """``[n0, ...] -> [world * n0, ...]`` on ``root`` (zeros elsewhere)."""
    return _ops.gather_single(x, root, _name(comm))


def scatter(x: Tensor, root: int, comm: Union[TorchComm, str]) -> Tensor:
    """``[world * n0, ...]`` on ``root`` ``-> [n0, ...]`` on every rank."""
    return _ops.scatter(x, root, _name(comm))


def register_collective(name: str, schema: str, impl, fake, backward=None, setup_context=None) -> object:
    """Adds an operator ``torch.ops.torchcomms_b200.<name>`` for a collective of an out-of-tree backend or of user
    code, with everything the built-in operators have: an eager implementation, a fake implementation for tracing,
    optionally an autograd formula, and the mark that keeps it in traced graphs on ranks that ignore its result.

        register_collective("my_gather", "(Tensor input, int root, str comm) -> Tensor",
                            impl=lambda input, root, comm: ..., fake=lambda input, root, comm: ...)

    ``impl`` gets the communicator's registered name (look it up with ``functional._get(name)``).  Returns the
    operator.  Counterpart in the reference: ``register_collective`` / ``finalize_registration`` of
    comms/torchcomms/functional/registry.py (driven by parameter specs of communicator methods there)."""
    _lib.define(f"{name}{schema}")
    _lib.impl(name, impl, "CompositeExplicitAutograd")
    torch.library.register_fake(f"{NAMESPACE}::{name}")(fake)
    if backward is not None:
        torch.library.register_autograd(f"{NAMESPACE}::{name}", backward, setup_context=setup_context or _setup)
    op = getattr(_ops, name)
    torch.fx.node.has_side_effect(op.default)
    return op


def finalize_registration(lib=None) -> None:
    """Nothing to do: operators are complete when ``register_collective`` returns (kept for code written against
    the reference, where registration is a two-step affair)."""


from .async_tensor import AsyncCollectiveTensor, OnceWork, TracedWork, wrap_async  # noqa: E402
from .ext import (  # noqa: E402
    CompiledComm, all_gather, all_gather_single_async, all_gather_v, all_reduce_async, all_to_all, all_to_all_single_async,
    batch_send_recv, compiled, reduce_scatter, reduce_scatter_single_async, reduce_scatter_v, wait_tensors, register_window, unregister_window,
    window_put, window_read, window_signal, window_token, window_wait_signal,
)
from .param_parsing import normalize_reduce_op, parse_hints, parse_timeout  # noqa: E402
from .inductor import mark_side_effects as _mark_side_effects  # noqa: E402

# A collective whose result is unused on one rank (a gather off the root, a barrier) must not be eliminated from
# that rank's traced graph: the peers make the matching call and would wait for it.
_mark_side_effects()

if is_torch_compile_supported_and_enabled():
    # TORCHCOMMS_PATCH_FOR_COMPILE=1, as in the reference: communicator methods become traceable and the Inductor
    # lowerings are registered as soon as this package is imported.
    from .dynamo import register_with_dynamo as _register_with_dynamo  # noqa: E402
    from .inductor import register_with_inductor as _register_with_inductor  # noqa: E402

    _register_with_dynamo()
    _register_with_inductor()

__all__ = [
    "AsyncCollectiveTensor", "OnceWork", "TracedWork", "wrap_async", "CompiledComm", "compiled",
    "all_gather", "all_gather_v", "reduce_scatter", "reduce_scatter_v", "all_to_all", "all_reduce_async", "all_gather_single_async",
    "reduce_scatter_single_async", "all_to_all_single_async", "batch_send_recv", "register_window", "unregister_window",
    "window_put", "window_read", "window_signal", "window_token", "window_wait_signal",
    "normalize_reduce_op", "parse_hints", "parse_timeout",
    "send", "recv", "gather_single", "scatter",
    "register_comm", "unregister_comm", "register_collective", "finalize_registration", "is_torch_compile_supported", "is_torch_compile_supported_and_enabled",
    "all_reduce", "all_reduce_", "all_gather_single", "reduce_scatter_single", "all_to_all_single", "broadcast",
    "broadcast_", "reduce", "barrier", "wait_tensor", "wait_tensors",
]
