"""Inductor lowerings of the ``torchcomms_b200`` operators.

Without them Inductor treats every operator of this package as an opaque
functional call, which is correct for the synchronous ones but costs a copy per
all-reduce / broadcast (the functional form clones its input) and says nothing
about the lifetime of the input of a started, not yet awaited collective.
``register_with_inductor()`` gives Inductor what it has for its own functional
collectives:

* ``all_reduce`` / ``broadcast`` lower to a clone followed by an in-place
  kernel (``all_reduce_inplace`` / ``broadcast_inplace``) on it; Inductor's
  buffer reuse drops the clone whenever the input dies at the call.
  ``all_reduce_`` / ``broadcast_`` lower to the in-place kernel directly.
* ``*_start`` lower to out-of-place collective kernels and ``wait_tensor`` to a
  wait kernel that acts in place on the started result, so that the scheduler
  keeps the input of the collective alive and untouched until the wait, and
  no copy is made at the wait.
* every operator that other ranks take part in is marked as having side
  effects, so that dead-code elimination cannot drop a call whose result is
  unused on one rank (a gather off the root, a barrier, a send) while the
  peers still make theirs.

Everything else (all-gather, reduce-scatter, all-to-all, list forms, windows)
stays with Inductor's default handling of custom operators.

Counterpart in the reference: comms/torchcomms/functional/inductor_lowering.py
(in-place and functional lowerings per registered collective, registration with
the re-inplacing pass, ``wait_tensors`` lowering).  Here the re-inplacing is
left to Inductor's buffer reuse, as Inductor does for its own all-reduce.
"""
from __future__ import annotations

import torch

from . import NAMESPACE, _get, _lib, _red
from . import ext  # noqa: F401  (defines the *_start operators)

_ops = getattr(torch.ops, NAMESPACE)
_registered = False

# The kernels the lowerings emit. Inductor's extern-kernel node accepts a mutating custom operator only if
# none of its results aliases an input, so these write in place and return nothing (the public in-place
# operators return their argument, as the in-place operators of torch do).
_lib.define("all_reduce_inplace(Tensor(a!) input, str op, str comm) -> ()")
_lib.define("broadcast_inplace(Tensor(a!) input, int root, str comm) -> ()")


def _impl_all_reduce_inplace(input: torch.Tensor, op: str, comm: str) -> None:
    _get(comm).all_reduce(input, _red(op), False)


def _impl_broadcast_inplace(input: torch.Tensor, root: int, comm: str) -> None:
    _get(comm).broadcast(input, root, False)


_lib.impl("all_reduce_inplace", _impl_all_reduce_inplace, "CompositeExplicitAutograd")
_lib.impl("broadcast_inplace", _impl_broadcast_inplace, "CompositeExplicitAutograd")


@torch.library.register_fake(f"{NAMESPACE}::all_reduce_inplace")
def _fake_all_reduce_inplace(input, op, comm):
    return None


@torch.library.register_fake(f"{NAMESPACE}::broadcast_inplace")
def _fake_broadcast_inplace(input, root, comm):
    return None


# Every operator that talks to other ranks has to stay in the graph even where its result goes unused on this rank
# (a gather off the root, a barrier, a send): the peers make the matching call and would wait for this one.
_SIDE_EFFECTS = (
    "all_reduce", "all_reduce_", "all_gather_single", "reduce_scatter_single", "all_to_all_single", "broadcast",
    "broadcast_", "reduce", "barrier", "send", "recv", "gather_single", "scatter", "all_gather", "all_gather_v",
    "reduce_scatter", "reduce_scatter_v", "all_to_all", "all_reduce_start", "all_gather_single_start", "reduce_scatter_single_start",
    "all_to_all_single_start", "all_reduce_inplace", "broadcast_inplace", "window_put", "window_signal",
    "window_wait_signal", "batch_send_recv",
)
_STARTS = ("all_reduce_start", "all_gather_single_start", "reduce_scatter_single_start", "all_to_all_single_start")


def mark_side_effects() -> None:
    """Keeps every call that other ranks take part in in traced graphs, whether or not its result is read here."""
    for name in _SIDE_EFFECTS:
        packet = getattr(_ops, name, None)
        if packet is not None:
            torch.fx.node.has_side_effect(packet.default)


def lowered_ops():
    """The operator overloads that ``register_with_inductor`` gives a lowering."""
    names = ("all_reduce", "all_reduce_", "broadcast", "broadcast_", "wait_tensor") + _STARTS
    return [getattr(_ops, n).default for n in names]


def register_with_inductor() -> bool:
    """Registers the lowerings (idempotent). False when this torch build has no Inductor."""
    global _registered
    if _registered:
        return True
    try:
        from torch._inductor import ir
        from torch._inductor.lowering import add_layout_constraint, clone, constrain_to_fx_strides, register_lowering
    except ImportError:
        return False
    mark_side_effects()

    def lowering(op):
        add_layout_constraint(op, constrain_to_fx_strides)
        return register_lowering(op)

    def in_place(kernel, functional):
        def lower(inp, *args):
            if functional:
                inp = clone(inp)              # dropped by buffer reuse when the input dies here
            inp = ir.ExternKernel.require_contiguous(inp)
            ir._CollectiveKernel.create_inplace(kernel, inp, *args)
            return inp

        return lower

    lowering(_ops.all_reduce.default)(in_place(_ops.all_reduce_inplace.default, True))
    lowering(_ops.all_reduce_.default)(in_place(_ops.all_reduce_inplace.default, False))
    lowering(_ops.broadcast.default)(in_place(_ops.broadcast_inplace.default, True))
    lowering(_ops.broadcast_.default)(in_place(_ops.broadcast_inplace.default, False))

    def out_of_place(kernel):
        def lower(inp, *args):
            node = ir._CollectiveKernel.create_out_of_place(kernel, inp, *args)
            return ir.TensorBox.create(node)

        return lower

    for name in _STARTS:
        op = getattr(_ops, name).default
        lowering(op)(out_of_place(op))

    @lowering(_ops.wait_tensor.default)
    def _wait(inp):
        ir._WaitKernel.create_wait(_ops.wait_tensor.default, inp)
        return inp

    _registered = True
    return True


register_torchcomms_lowerings = register_with_inductor     # the reference's name

__all__ = ["register_with_inductor", "register_torchcomms_lowerings", "mark_side_effects", "lowered_ops"]
