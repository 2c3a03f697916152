"""The rest of the communicator surface as traceable operators: list-form
collectives, asynchronous starts with ``wait_tensor``, one-sided windows and
batched send / receive, plus ``CompiledComm``, a pure-Python stand-in for a
communicator whose methods a tracing compiler can inline.

    cc = functional.compiled(comm)                      # plain attributes only: name, rank, size

    @torch.compile(fullgraph=True)
    def step(x):
        y = cc.all_reduce(x * 2, "sum")                 # torch.ops.torchcomms_b200.all_reduce
        h = cc.all_gather_single_async(y)               # start ...
        z = (y + 1).sum()
        return h.wait().sum() + z                       # ... wait_tensor in the graph

Asynchronous starts keep their work handle in a table keyed by the result
tensor; ``wait_tensor`` looks it up, orders the caller behind the collective
and hands the data on.  In eager mode the start functions return an
``AsyncCollectiveTensor`` instead, which waits on first use.

Parity: comms/torchcomms/functional/registry.py:40-90,247-725 (every TorchComm,
Window and BatchSendRecv method as an operator with functional and in-place
forms), collectives.py, async_tensor.py:252-320 and dynamo.py (method calls on
the communicator inside compiled code; here through ``CompiledComm``).
"""
from __future__ import annotations

from typing import Dict, List, Optional, Sequence, Union

import torch
from torch import Tensor

from .. import TorchComm
from . import NAMESPACE, _get, _lib, _name, _red, _size
from .async_tensor import TracedWork, is_tracing, wrap_async

_ops = getattr(torch.ops, NAMESPACE)

# ------------------------------------------------------------- list forms ----

_lib.define("all_gather(Tensor input, str comm) -> Tensor[]")
_lib.define("all_gather_v(Tensor input, int[] sizes, str comm) -> Tensor[]")
_lib.define("reduce_scatter(Tensor[] inputs, str op, str comm) -> Tensor")
_lib.define("all_to_all(Tensor[] inputs, str comm) -> Tensor[]")
_lib.define("reduce_scatter_v(Tensor[] inputs, str op, str comm) -> Tensor")


def _impl_all_gather(input: Tensor, comm: str) -> List[Tensor]:
    c = _get(comm)
    outs = [torch.empty_like(input, memory_format=torch.contiguous_format) for _ in range(c.get_size())]
    c.all_gather(outs, input.contiguous(), False)
    return outs


def _impl_all_gather_v(input: Tensor, sizes: List[int], comm: str) -> List[Tensor]:
    c = _get(comm)
    outs = [input.new_empty((n,) + tuple(input.shape[1:])) for n in sizes]
    c.all_gather_v(outs, input.contiguous(), False)
    return outs


def _impl_reduce_scatter(inputs: List[Tensor], op: str, comm: str) -> Tensor:
    c = _get(comm)
    out = torch.empty_like(inputs[c.get_rank()], memory_format=torch.contiguous_format)
    c.reduce_scatter(out, [t.contiguous() for t in inputs], _red(op), False)
    return out


def _impl_reduce_scatter_v(inputs: List[Tensor], op: str, comm: str) -> Tensor:
    c = _get(comm)
    out = torch.empty_like(inputs[c.get_rank()], memory_format=torch.contiguous_format)
    c.reduce_scatter_v(out, [t.contiguous() for t in inputs], _red(op), False)
    return out


def _impl_all_to_all(inputs: List[Tensor], comm: str) -> List[Tensor]:
    c = _get(comm)
    outs = [torch.empty_like(t, memory_format=torch.contiguous_format) for t in inputs]
    c.all_to_all(outs, [t.contiguous() for t in inputs], False)
    return outs


for _op, _fn in (("all_gather", _impl_all_gather), ("all_gather_v", _impl_all_gather_v),
                 ("reduce_scatter", _impl_reduce_scatter), ("all_to_all", _impl_all_to_all),
                 ("reduce_scatter_v", _impl_reduce_scatter_v)):
    _lib.impl(_op, _fn, "CompositeExplicitAutograd")


@torch.library.register_fake(f"{NAMESPACE}::all_gather")
def _fake_all_gather(input, comm):
    return [torch.empty_like(input, memory_format=torch.contiguous_format) for _ in range(_size(comm))]


@torch.library.register_fake(f"{NAMESPACE}::all_gather_v")
def _fake_all_gather_v(input, sizes, comm):
    return [input.new_empty((n,) + tuple(input.shape[1:])) for n in sizes]


@torch.library.register_fake(f"{NAMESPACE}::reduce_scatter")
def _fake_reduce_scatter(inputs, op, comm):
    return torch.empty_like(inputs[0], memory_format=torch.contiguous_format)


@torch.library.register_fake(f"{NAMESPACE}::reduce_scatter_v")
def _fake_reduce_scatter_v(inputs, op, comm):
    return torch.empty_like(inputs[_get(comm).get_rank()], memory_format=torch.contiguous_format)   # shares differ per rank


@torch.library.register_fake(f"{NAMESPACE}::all_to_all")
def _fake_all_to_all(inputs, comm):
    return [torch.empty_like(t, memory_format=torch.contiguous_format) for t in inputs]


def _setup(ctx, inputs, output):
    ctx.args = inputs[1:]


def _bw_all_gather(ctx, grads):
    (comm,) = ctx.args
    return _ops.reduce_scatter([g.contiguous() for g in grads], "sum", comm), None


def _bw_reduce_scatter(ctx, grad):
    op, comm = ctx.args
    if op.lower() not in ("sum", "avg"):
        raise RuntimeError(f"reduce_scatter: no gradient for op '{op}'")
    gs = _ops.all_gather(grad.contiguous(), comm)
    if op.lower() == "avg":
        gs = [g / _size(comm) for g in gs]
    return gs, None, None


def _setup_reduce_scatter_v(ctx, inputs, output):
    ctx.args = inputs[1:]
    ctx.sizes = [t.shape[0] for t in inputs[0]]


def _bw_reduce_scatter_v(ctx, grad):
    op, comm = ctx.args
    if op.lower() not in ("sum", "avg"):
        raise RuntimeError(f"reduce_scatter_v: no gradient for op '{op}'")
    gs = _ops.all_gather_v(grad.contiguous(), ctx.sizes, comm)
    if op.lower() == "avg":
        gs = [g / _size(comm) for g in gs]
    return gs, None, None


def _bw_all_to_all(ctx, grads):
    (comm,) = ctx.args
    return _ops.all_to_all([g.contiguous() for g in grads], comm), None


torch.library.register_autograd(f"{NAMESPACE}::all_gather", _bw_all_gather, setup_context=_setup)
torch.library.register_autograd(f"{NAMESPACE}::reduce_scatter", _bw_reduce_scatter, setup_context=_setup)
torch.library.register_autograd(f"{NAMESPACE}::all_to_all", _bw_all_to_all, setup_context=_setup)
torch.library.register_autograd(f"{NAMESPACE}::reduce_scatter_v", _bw_reduce_scatter_v, setup_context=_setup_reduce_scatter_v)


def all_gather(x: Tensor, comm: Union[TorchComm, str]) -> List[Tensor]:
    """One tensor per rank, each shaped like ``x``."""
    return _ops.all_gather(x, _name(comm))


def all_gather_v(x: Tensor, sizes: Sequence[int], comm: Union[TorchComm, str]) -> List[Tensor]:
    """One tensor per rank with ``sizes[r]`` rows (``x`` has ``sizes[own rank]`` rows)."""
    return _ops.all_gather_v(x, list(sizes), _name(comm))


def reduce_scatter(xs: Sequence[Tensor], op: str, comm: Union[TorchComm, str]) -> Tensor:
    """Reduction over ranks of ``xs[own rank]``."""
    return _ops.reduce_scatter(list(xs), op, _name(comm))


def reduce_scatter_v(xs: Sequence[Tensor], op: str, comm: Union[TorchComm, str]) -> Tensor:
    """Reduction over ranks of ``xs[own rank]``; the shares may have different numbers of rows."""
    return _ops.reduce_scatter_v(list(xs), op, _name(comm))


def all_to_all(xs: Sequence[Tensor], comm: Union[TorchComm, str]) -> List[Tensor]:
    """``out[r]`` is what rank ``r`` passed as ``xs[own rank]`` (shapes mirror ``xs``)."""
    return _ops.all_to_all(list(xs), _name(comm))


# ------------------------------------------------------ asynchronous starts ----

# Work handles of collectives started but not yet waited for, by the result's storage address.
_pending: Dict[int, object] = {}

_lib.define("all_reduce_start(Tensor input, str op, str comm) -> Tensor")
_lib.define("all_gather_single_start(Tensor input, str comm) -> Tensor")
_lib.define("reduce_scatter_single_start(Tensor input, str op, str comm) -> Tensor")
_lib.define("all_to_all_single_start(Tensor input, int[]? output_split_sizes, int[]? input_split_sizes, str comm) -> Tensor")


def _remember(out: Tensor, work) -> Tensor:
    _pending[out.untyped_storage().data_ptr()] = work
    return out


def wait_pending(t: Tensor) -> None:
    """Orders the caller behind the collective that produces ``t``, if one is still registered."""
    work = _pending.pop(t.untyped_storage().data_ptr(), None)
    if work is not None:
        work.wait()


def _impl_all_reduce_start(input: Tensor, op: str, comm: str) -> Tensor:
    out = input.contiguous().clone()
    return _remember(out, _get(comm).all_reduce(out, _red(op), True))


def _impl_all_gather_single_start(input: Tensor, comm: str) -> Tensor:
    c = _get(comm)
    out = input.new_empty((input.shape[0] * c.get_size(),) + tuple(input.shape[1:]))
    return _remember(out, c.all_gather_single(out, input.contiguous(), True))


def _impl_reduce_scatter_single_start(input: Tensor, op: str, comm: str) -> Tensor:
    c = _get(comm)
    out = input.new_empty((input.shape[0] // c.get_size(),) + tuple(input.shape[1:]))
    return _remember(out, c.reduce_scatter_single(out, input.contiguous(), _red(op), True))


def _impl_all_to_all_single_start(input: Tensor, output_split_sizes: Optional[List[int]],
                                  input_split_sizes: Optional[List[int]], comm: str) -> Tensor:
    c = _get(comm)
    if output_split_sizes:
        out = input.new_empty((sum(output_split_sizes),) + tuple(input.shape[1:]))
        work = c.all_to_all_v_single(out, input.contiguous(), list(output_split_sizes), list(input_split_sizes or []), True)
    else:
        out = torch.empty_like(input, memory_format=torch.contiguous_format)
        work = c.all_to_all_single(out, input.contiguous(), True)
    return _remember(out, work)


for _op, _fn in (("all_reduce_start", _impl_all_reduce_start), ("all_gather_single_start", _impl_all_gather_single_start),
                 ("reduce_scatter_single_start", _impl_reduce_scatter_single_start),
                 ("all_to_all_single_start", _impl_all_to_all_single_start)):
    _lib.impl(_op, _fn, "CompositeExplicitAutograd")


@torch.library.register_fake(f"{NAMESPACE}::all_reduce_start")
def _fake_all_reduce_start(input, op, comm):
    return torch.empty_like(input, memory_format=torch.contiguous_format)


@torch.library.register_fake(f"{NAMESPACE}::all_gather_single_start")
def _fake_all_gather_single_start(input, comm):
    return input.new_empty((input.shape[0] * _size(comm),) + tuple(input.shape[1:]))


@torch.library.register_fake(f"{NAMESPACE}::reduce_scatter_single_start")
def _fake_reduce_scatter_single_start(input, op, comm):
    return input.new_empty((input.shape[0] // _size(comm),) + tuple(input.shape[1:]))


@torch.library.register_fake(f"{NAMESPACE}::all_to_all_single_start")
def _fake_all_to_all_single_start(input, output_split_sizes, input_split_sizes, comm):
    if output_split_sizes:
        return input.new_empty((sum(output_split_sizes),) + tuple(input.shape[1:]))
    return torch.empty_like(input, memory_format=torch.contiguous_format)


# The started operators differentiate like their synchronous counterparts (the gradient itself is computed with
# the synchronous operators: nothing in a backward graph waits for it).
def _register_start_autograd() -> None:
    from . import _bw_all_gather_single, _bw_all_reduce, _bw_all_to_all_single, _bw_reduce_scatter_single
    from . import _setup as _setup_sync

    for name, fn in (("all_reduce_start", _bw_all_reduce), ("all_gather_single_start", _bw_all_gather_single),
                     ("reduce_scatter_single_start", _bw_reduce_scatter_single),
                     ("all_to_all_single_start", _bw_all_to_all_single)):
        torch.library.register_autograd(f"{NAMESPACE}::{name}", fn, setup_context=_setup_sync)


_register_start_autograd()


# The list form of ``wait_tensor`` under the name the reference gives it (``torchcomm_wait_tensors``): one wait for
# the results of several started collectives.
_lib.define("torchcomm_wait_tensors(Tensor[] inputs) -> Tensor[]")


def _impl_wait_tensors(inputs: List[Tensor]) -> List[Tensor]:
    for t in inputs:
        wait_pending(t)
    return [t.clone() for t in inputs]


_lib.impl("torchcomm_wait_tensors", _impl_wait_tensors, "CompositeExplicitAutograd")


@torch.library.register_fake(f"{NAMESPACE}::torchcomm_wait_tensors")
def _fake_wait_tensors(inputs):
    return [torch.empty_like(t) for t in inputs]


torch.library.register_autograd(f"{NAMESPACE}::torchcomm_wait_tensors", lambda ctx, grads: (list(grads),),
                                setup_context=lambda ctx, inputs, output: None)


def wait_tensors(xs: Sequence[Tensor]) -> List[Tensor]:
    """``wait_tensor`` for several results at once."""
    return _ops.torchcomm_wait_tensors(list(xs))


def _start(op, *args):
    """Eager: an AsyncCollectiveTensor. Tracing: the start operator's result with a TracedWork."""
    out = op(*args)
    if is_tracing():
        return TracedWork(out)
    work = _pending.pop(out.untyped_storage().data_ptr(), None)
    return wrap_async(out, work)


def all_reduce_async(x: Tensor, op: str, comm: Union[TorchComm, str]):
    return _start(_ops.all_reduce_start, x, op, _name(comm))


def all_gather_single_async(x: Tensor, comm: Union[TorchComm, str]):
    return _start(_ops.all_gather_single_start, x, _name(comm))


def reduce_scatter_single_async(x: Tensor, op: str, comm: Union[TorchComm, str]):
    return _start(_ops.reduce_scatter_single_start, x, op, _name(comm))


def all_to_all_single_async(x: Tensor, comm: Union[TorchComm, str], output_split_sizes: Optional[List[int]] = None,
                            input_split_sizes: Optional[List[int]] = None):
    return _start(_ops.all_to_all_single_start, x, output_split_sizes, input_split_sizes, _name(comm))


# ------------------------------------------------------------------ windows ----

_windows: Dict[str, object] = {}


def register_window(name: str, window) -> str:
    """Makes a window (with its tensor registered) addressable from traced code."""
    _windows[name] = window
    return name


def unregister_window(name: str) -> None:
    _windows.pop(name, None)


def _window(name: str):
    try:
        return _windows[name]
    except KeyError:
        raise RuntimeError(f"window '{name}' is not registered: call functional.register_window(name, window)") from None


# Every window operator threads a token (an empty tensor) so that a graph keeps them in program order.
_lib.define("window_put(Tensor src, str window, int dst_rank, int target_offset_nelems, Tensor token) -> Tensor")
_lib.define("window_signal(str window, int peer, Tensor token) -> Tensor")
_lib.define("window_wait_signal(str window, int peer, Tensor token) -> Tensor")
_lib.define("window_read(str window, Tensor token) -> Tensor")


def _impl_window_put(src: Tensor, window: str, dst_rank: int, target_offset_nelems: int, token: Tensor) -> Tensor:
    _window(window).put(src.contiguous(), dst_rank, target_offset_nelems, False)
    return token.clone()


def _impl_window_signal(window: str, peer: int, token: Tensor) -> Tensor:
    _window(window).signal(peer, False)
    return token.clone()


def _impl_window_wait_signal(window: str, peer: int, token: Tensor) -> Tensor:
    _window(window).wait_signal(peer, False)
    return token.clone()


def _impl_window_read(window: str, token: Tensor) -> Tensor:
    return _window(window).get_tensor().clone()


for _op, _fn in (("window_put", _impl_window_put), ("window_signal", _impl_window_signal),
                 ("window_wait_signal", _impl_window_wait_signal), ("window_read", _impl_window_read)):
    _lib.impl(_op, _fn, "CompositeExplicitAutograd")


@torch.library.register_fake(f"{NAMESPACE}::window_put")
def _fake_window_put(src, window, dst_rank, target_offset_nelems, token):
    return torch.empty_like(token)


@torch.library.register_fake(f"{NAMESPACE}::window_signal")
def _fake_window_signal(window, peer, token):
    return torch.empty_like(token)


@torch.library.register_fake(f"{NAMESPACE}::window_wait_signal")
def _fake_window_wait_signal(window, peer, token):
    return torch.empty_like(token)


@torch.library.register_fake(f"{NAMESPACE}::window_read")
def _fake_window_read(window, token):
    w = _window(window)
    return torch.empty(list(w.shape), dtype=w.dtype, device=token.device)


def window_token(device=None) -> Tensor:
    return torch.empty(0, device=device)


def window_put(src: Tensor, window: str, dst_rank: int, target_offset_nelems: int = 0, token: Optional[Tensor] = None) -> Tensor:
    return _ops.window_put(src, window, dst_rank, target_offset_nelems, token if token is not None else window_token(src.device))


def window_signal(window: str, peer: int, token: Tensor) -> Tensor:
    return _ops.window_signal(window, peer, token)


def window_wait_signal(window: str, peer: int, token: Tensor) -> Tensor:
    return _ops.window_wait_signal(window, peer, token)


def window_read(window: str, token: Tensor) -> Tensor:
    """A copy of the local window contents, ordered behind ``token``."""
    return _ops.window_read(window, token)


# ---------------------------------------------------------- batched p2p ----

_lib.define("batch_send_recv(Tensor[] sends, int[] dsts, Tensor[] recv_like, int[] srcs, str comm) -> Tensor[]")


def _impl_batch_send_recv(sends: List[Tensor], dsts: List[int], recv_like: List[Tensor], srcs: List[int], comm: str) -> List[Tensor]:
    c = _get(comm)
    outs = [torch.empty_like(t, memory_format=torch.contiguous_format) for t in recv_like]
    batch = c.batch_op_create()
    for t, d in zip(sends, dsts):
        batch.send(t.contiguous(), d)
    for t, s in zip(outs, srcs):
        batch.recv(t, s)
    batch.issue(False).wait()
    return outs


_lib.impl("batch_send_recv", _impl_batch_send_recv, "CompositeExplicitAutograd")


@torch.library.register_fake(f"{NAMESPACE}::batch_send_recv")
def _fake_batch_send_recv(sends, dsts, recv_like, srcs, comm):
    return [torch.empty_like(t, memory_format=torch.contiguous_format) for t in recv_like]


def batch_send_recv(sends: Sequence[Tensor], dsts: Sequence[int], recv_like: Sequence[Tensor], srcs: Sequence[int],
                    comm: Union[TorchComm, str]) -> List[Tensor]:
    """One grouped exchange: ``sends[i]`` goes to ``dsts[i]``; returns tensors shaped like ``recv_like[j]`` from ``srcs[j]``."""
    return _ops.batch_send_recv(list(sends), list(dsts), list(recv_like), list(srcs), _name(comm))


# ------------------------------------------------------ compiled communicator ----


class CompiledComm:
    """What traced code holds instead of a ``TorchComm``: the registered name and a few integers.

    Methods mirror the communicator's but are functional: they return the result
    instead of writing into an output argument. ``*_async`` methods return a
    handle whose ``wait()`` gives the result.
    """

    def __init__(self, comm: TorchComm):
        self.name = _name(comm)
        self.rank = comm.get_rank()
        self.size = comm.get_size()

    def get_rank(self) -> int:
        return self.rank

    def get_size(self) -> int:
        return self.size

    def all_reduce(self, x: Tensor, op: str = "sum") -> Tensor:
        return _ops.all_reduce(x, op, self.name)

    def all_gather_single(self, x: Tensor) -> Tensor:
        return _ops.all_gather_single(x, self.name)

    def reduce_scatter_single(self, x: Tensor, op: str = "sum") -> Tensor:
        return _ops.reduce_scatter_single(x, op, self.name)

    def all_to_all_single(self, x: Tensor, output_split_sizes=None, input_split_sizes=None) -> Tensor:
        return _ops.all_to_all_single(x, output_split_sizes, input_split_sizes, self.name)

    def broadcast(self, x: Tensor, root: int) -> Tensor:
        return _ops.broadcast(x, root, self.name)

    def all_gather(self, x: Tensor) -> List[Tensor]:
        return _ops.all_gather(x, self.name)

    def reduce_scatter(self, xs: Sequence[Tensor], op: str = "sum") -> Tensor:
        return _ops.reduce_scatter(list(xs), op, self.name)

    def all_to_all(self, xs: Sequence[Tensor]) -> List[Tensor]:
        return _ops.all_to_all(list(xs), self.name)

    def all_reduce_async(self, x: Tensor, op: str = "sum"):
        return all_reduce_async(x, op, self.name)

    def all_gather_single_async(self, x: Tensor):
        return all_gather_single_async(x, self.name)

    def reduce_scatter_single_async(self, x: Tensor, op: str = "sum"):
        return reduce_scatter_single_async(x, op, self.name)


def compiled(comm: TorchComm) -> CompiledComm:
    return CompiledComm(comm)


__all__ = [
    "all_gather", "all_gather_v", "reduce_scatter", "all_to_all",
    "all_reduce_async", "all_gather_single_async", "reduce_scatter_single_async", "all_to_all_single_async", "wait_pending",
    "register_window", "unregister_window", "window_token", "window_put", "window_signal", "window_wait_signal", "window_read",
    "batch_send_recv", "CompiledComm", "compiled",
]
