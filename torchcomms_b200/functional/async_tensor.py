"""Asynchronous results of functional collectives.

``AsyncCollectiveTensor`` wraps the output buffer of a collective that is still
in flight together with its work handle.  The first operation that touches the
tensor (or an explicit ``wait()``) orders the caller behind the collective and
from then on the wrapper behaves like the plain tensor.  Several tensors that
came out of ONE collective share a ``OnceWork`` so that the handle is waited
for a single time.  While a graph is being traced the same interface is served
by ``TracedWork``, whose ``wait()`` emits ``wait_tensor`` operators so that the
dependency is part of the graph.

Parity: comms/torchcomms/functional/async_tensor.py (``_OnceWaitWork``,
``FakeWork``, ``TorchCommsAsyncTensor``, ``_maybe_wrap_tensor``).
"""
from __future__ import annotations

from typing import Any, List, Optional, Sequence, Union

import torch
from torch import Tensor
from torch.utils import _pytree as pytree


class OnceWork:
    """Waits for the underlying handle the first time only."""

    __slots__ = ("_work", "_done")

    def __init__(self, work: Any):
        self._work = work
        self._done = work is None

    def wait(self) -> None:
        if not self._done:
            self._done = True
            self._work.wait()

    @property
    def done(self) -> bool:
        return self._done


def is_tracing() -> bool:
    """True while dynamo, make_fx or export is building a graph."""
    if torch.compiler.is_compiling():
        return True
    mode = torch._C._get_dispatch_mode(torch._C._TorchDispatchModeKey.PROXY) if hasattr(torch._C, "_get_dispatch_mode") else None
    return mode is not None


class TracedWork:
    """Work handle of a collective recorded in a graph: ``wait()`` returns the results passed through
    ``wait_tensor`` (same nesting as they were given), once."""

    __slots__ = ("_result", "_waited")

    def __init__(self, result: Union[Tensor, Sequence[Tensor]]):
        self._result = result
        self._waited = None

    def wait(self):
        if self._waited is None:
            from . import wait_tensor

            self._waited = pytree.tree_map(lambda t: wait_tensor(t) if isinstance(t, Tensor) else t, self._result)
        return self._waited


class AsyncCollectiveTensor(Tensor):
    """A tensor whose contents are still being produced by a collective."""

    elem: Tensor
    work: Optional[OnceWork]

    __slots__ = ("elem", "work")

    @staticmethod
    def __new__(cls, elem: Tensor, work: Optional[OnceWork]):
        r = Tensor._make_wrapper_subclass(
            cls, elem.size(), strides=elem.stride(), storage_offset=elem.storage_offset(), dtype=elem.dtype,
            layout=elem.layout, device=elem.device, requires_grad=elem.requires_grad,
        )
        r.elem = elem
        r.work = work
        return r

    def __repr__(self) -> str:  # type: ignore[override]
        state = "ready" if self.work is None or self.work.done else "in flight"
        return f"AsyncCollectiveTensor({state}, shape={tuple(self.shape)}, dtype={self.dtype})"

    def wait(self) -> Tensor:
        """Orders the caller behind the collective and returns the plain tensor."""
        if self.work is not None:
            self.work.wait()
        return self.elem

    trigger_wait = wait

    def tolist(self):
        return self.wait().tolist()

    def numpy(self):
        return self.wait().numpy()

    def __tensor_flatten__(self):
        return ["elem"], None

    @staticmethod
    def __tensor_unflatten__(inner, meta, outer_size, outer_stride):
        return AsyncCollectiveTensor(inner["elem"], None)

    @classmethod
    def __torch_dispatch__(cls, func, types, args=(), kwargs=None):  # type: ignore[override]
        def unwrap(x):
            return x.wait() if isinstance(x, AsyncCollectiveTensor) else x

        return func(*pytree.tree_map(unwrap, args), **pytree.tree_map(unwrap, kwargs or {}))


def wrap_async(result: Union[Tensor, List[Tensor]], work: Any):
    """Eager: the result(s) as ``AsyncCollectiveTensor`` sharing one handle. Tracing: the result(s) unchanged."""
    if is_tracing() or work is None:
        return result
    shared = work if isinstance(work, OnceWork) else OnceWork(work)
    if isinstance(result, Tensor):
        return AsyncCollectiveTensor(result, shared)
    return [AsyncCollectiveTensor(t, shared) for t in result]


# The reference's names for the same things (comms/torchcomms/functional/async_tensor.py).
TorchCommsAsyncTensor = AsyncCollectiveTensor
FakeWork = TracedWork

__all__ = ["OnceWork", "TracedWork", "AsyncCollectiveTensor", "wrap_async", "is_tracing", "TorchCommsAsyncTensor", "FakeWork"]
