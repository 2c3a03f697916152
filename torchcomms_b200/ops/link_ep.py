"""The reference's ``link_ep.Buffer`` call signatures on the fused kernels of ``ops/moe_ep.py``.

Code written against ``link_ep`` (``get_dispatch_layout`` -> ``dispatch`` ->
experts -> ``combine``, the cached-handle forms, the low-latency pair and the
``EventOverlap`` hand-off between streams) runs unchanged:

    buffer = Buffer(comm, hidden=7168, num_experts=256, num_topk=8, num_max_tokens=4096)
    ntpr, _, ntpe, in_rank, ev = buffer.get_dispatch_layout(topk_idx, num_experts)
    recv_x, recv_idx, recv_w, counts, handle, ev = buffer.dispatch(
        x, num_tokens_per_rank=ntpr, is_token_in_rank=in_rank, num_tokens_per_expert=ntpe,
        topk_idx=topk_idx, topk_weights=topk_w)
    combined, combined_w, ev = buffer.combine(expert_out, handle, topk_weights=recv_w)

What differs from the reference, by design: the layout tensors passed to
``dispatch`` are accepted and not needed (the kernel derives the layout from
``topk_idx``); ``x`` given as bf16 is returned as bf16, and as an ``(fp8,
scales)`` pair when the buffer was built with ``fp8=True`` (quantisation happens
inside the dispatch kernel, so a pre-quantised pair is not accepted); the sizes
that the reference passes as byte counts (``num_nvl_bytes``) are given as
``num_max_tokens``; ``num_worst_tokens > 0`` returns the whole fixed-size
buffers without reading the receive count on the host.

Parity: ``comms/prims/collectives/link_ep/link_ep/buffer.py:76-660``,
``link_ep/utils.py:38-74`` (``EventOverlap``).
"""
from __future__ import annotations

from typing import Any, Callable, List, Optional, Tuple, Union

import torch

from .. import TorchComm
from . import moe_ep


class EventOverlap:
    """A CUDA event (or none) plus tensors kept alive until the event has been waited for."""

    def __init__(self, event: Optional[torch.cuda.Event] = None, extra_tensors: Optional[Tuple[torch.Tensor, ...]] = None):
        self.event = event
        self.extra_tensors = extra_tensors

    def current_stream_wait(self) -> None:
        if self.event is None:
            raise RuntimeError("EventOverlap.current_stream_wait called with no event")
        torch.cuda.current_stream().wait_event(self.event)

    def __enter__(self) -> "EventOverlap":
        return self

    def __exit__(self, exc_type: Any, exc_val: Any, exc_tb: Any) -> None:
        if self.event is not None:
            torch.cuda.current_stream().wait_event(self.event)


class Config:
    """Tuning record of the reference (SM count, chunk sizes); kept for signature compatibility, only ``num_sms`` is read."""

    def __init__(self, num_sms: int = 0, *chunks: int):
        self.num_sms = num_sms
        self.chunks = chunks


class Buffer:
    num_sms: int = 0   # 0 = every SM (the kernels are cooperative and size their own grid)

    def __init__(self, comm: TorchComm, hidden: int, num_experts: int, num_topk: int, num_max_tokens: int,
                 fp8: bool = False, low_latency_mode: bool = False, num_max_dispatch_tokens_per_rank: int = 128,
                 low_latency_fp8: bool = True):
        self.comm = comm
        self.rank, self.group_size = comm.get_rank(), comm.get_size()
        self.hidden, self.num_experts, self.num_topk = hidden, num_experts, num_topk
        self._normal = moe_ep.Buffer(comm, num_max_tokens, hidden, num_experts, num_topk, fp8=fp8)
        self._ll: Optional[moe_ep.LowLatencyBuffer] = None
        self._ll_fp8 = low_latency_fp8
        if low_latency_mode:
            self._ll = moe_ep.LowLatencyBuffer(comm, num_max_dispatch_tokens_per_rank, hidden, num_experts, num_topk,
                                               fp8=low_latency_fp8)
        self._comm_stream = torch.cuda.Stream(device=comm.get_device())

    def destroy(self) -> None:
        self._normal = None
        self._ll = None

    # ---- static helpers of the reference

    @staticmethod
    def is_sm90_compiled() -> bool:
        return False   # sm_100a only

    @staticmethod
    def set_num_sms(new_num_sms: int) -> None:
        Buffer.num_sms = new_num_sms

    @staticmethod
    def capture() -> EventOverlap:
        ev = torch.cuda.Event()
        ev.record()
        return EventOverlap(ev)

    @staticmethod
    def get_dispatch_config(num_ranks: int) -> Config:
        return Config(Buffer.num_sms)

    @staticmethod
    def get_combine_config(num_ranks: int) -> Config:
        return Config(Buffer.num_sms)

    @staticmethod
    def get_low_latency_rdma_size_hint(num_max_dispatch_tokens_per_rank: int, hidden: int, num_ranks: int,
                                       num_experts: int) -> int:
        """Bytes of symmetric memory that ``low_latency_mode`` takes per rank (bf16 rows, both parities, plus outputs)."""
        slots = 2 * num_experts * num_max_dispatch_tokens_per_rank
        return slots * (hidden * 2 + hidden // 128 * 4 + 4) + slots // 2 * hidden * 2 + 2 * num_experts * num_ranks * 8

    # ---- stream hand-off shared by all calls

    def _run(self, fn: Callable[[], Any], previous_event: Optional[EventOverlap], async_finish: bool,
             extra: Tuple[torch.Tensor, ...] = ()):
        """Runs ``fn`` after ``previous_event``; with ``async_finish`` on the buffer's own stream, returning an event."""
        if not async_finish:
            if previous_event is not None and previous_event.event is not None:
                previous_event.current_stream_wait()
            return fn(), EventOverlap(None)
        cur = torch.cuda.current_stream()
        if previous_event is not None and previous_event.event is not None:
            self._comm_stream.wait_event(previous_event.event)
        else:
            self._comm_stream.wait_stream(cur)
        with torch.cuda.stream(self._comm_stream):
            out = fn()
            ev = torch.cuda.Event()
            ev.record(self._comm_stream)
        return out, EventOverlap(ev, extra)

    # ---- normal mode

    def get_dispatch_layout(self, topk_idx: torch.Tensor, num_experts: int, previous_event: Optional[EventOverlap] = None,
                            async_finish: bool = False, allocate_on_comm_stream: bool = False):
        """``(num_tokens_per_rank, None, num_tokens_per_expert, is_token_in_rank, event)``; the mask is boolean."""
        def fn():
            per_rank, per_expert, in_rank = moe_ep.get_dispatch_layout(topk_idx, num_experts, self.group_size)
            return per_rank, per_expert, in_rank.bool()

        (per_rank, per_expert, in_rank), ev = self._run(fn, previous_event, async_finish, (topk_idx,))
        return per_rank, None, per_expert, in_rank, ev

    def dispatch(self, x: Union[torch.Tensor, Tuple[torch.Tensor, torch.Tensor]], handle: Optional[tuple] = None,
                 num_tokens_per_rank: Optional[torch.Tensor] = None, num_tokens_per_rdma_rank: Optional[torch.Tensor] = None,
                 is_token_in_rank: Optional[torch.Tensor] = None, num_tokens_per_expert: Optional[torch.Tensor] = None,
                 topk_idx: Optional[torch.Tensor] = None, topk_weights: Optional[torch.Tensor] = None,
                 expert_alignment: int = 1, num_worst_tokens: int = 0, config: Optional[Config] = None,
                 previous_event: Optional[EventOverlap] = None, async_finish: bool = False,
                 allocate_on_comm_stream: bool = False):
        """``(recv_x, recv_topk_idx, recv_topk_weights, num_recv_tokens_per_expert_list, handle, event)``.

        With ``handle`` (from an earlier call) the rows of ``x`` travel along that call's layout and the second to
        fourth results are ``None`` / empty, as in the reference.
        """
        if isinstance(x, tuple):
            raise ValueError("pass bf16 rows: quantisation to fp8 happens inside the dispatch kernel (Buffer(fp8=True))")
        buf = self._normal
        if handle is not None:
            inner: moe_ep.Handle = handle[0]

            def cached():
                if num_worst_tokens > 0:
                    return buf.cached_dispatch(x, inner, rows=num_worst_tokens)
                return buf.cached_dispatch(x, inner, rows=int(inner.num_recv))

            rows, ev = self._run(cached, previous_event, async_finish, (x,))
            return rows, None, None, [], handle, ev
        if topk_idx is None or topk_weights is None:
            raise ValueError("dispatch without a handle needs topk_idx and topk_weights")

        def fn():
            d = buf.dispatch(x, topk_idx, topk_weights, keep_handle=True)
            if num_worst_tokens > 0:        # fixed-size results, no host read
                n = min(num_worst_tokens, d.x.shape[0])
                counts: List[int] = []
            else:
                n = int(d.num_tokens)
                local = d.topk_idx[:n]
                per_expert = torch.bincount(local[local >= 0].long(), minlength=self.num_experts // self.group_size)
                counts = [(c + expert_alignment - 1) // expert_alignment * expert_alignment for c in per_expert.tolist()]
            rx = d.x[:n].clone()
            recv_x = (rx, d.scales[:n].clone()) if d.scales is not None else rx
            return recv_x, d.topk_idx[:n].to(topk_idx.dtype), d.topk_weights[:n].clone(), counts, d.handle

        (recv_x, ridx, rw, counts, inner), ev = self._run(fn, previous_event, async_finish, (x, topk_idx, topk_weights))
        # Shaped like the reference's 6-tuple; entry 0 carries the layout, entry 4 the mask the caller passed in.
        out_handle = (inner, None, None, inner.recv_src, is_token_in_rank, inner.send_slot)
        return recv_x, ridx, rw, counts, out_handle, ev

    def combine(self, x: torch.Tensor, handle: tuple, topk_weights: Optional[torch.Tensor] = None,
                bias: Union[torch.Tensor, Tuple[torch.Tensor, torch.Tensor], None] = None, config: Optional[Config] = None,
                previous_event: Optional[EventOverlap] = None, async_finish: bool = False,
                allocate_on_comm_stream: bool = False):
        """``(combined_x, combined_topk_weights, event)``: the sum of ``x``'s rows over the ranks each token went to,
        plus the bias(es); ``topk_weights`` ([rows, topk], receiver side) come back summed per token."""
        buf = self._normal
        inner: moe_ep.Handle = handle[0]
        b0, b1 = bias if isinstance(bias, tuple) else (bias, None)
        total_bias = b0 if b1 is None else (b0 + b1 if b0 is not None else b1)

        def fn():
            n = x.shape[0]
            buf.combine_input[:n].copy_(x)
            w_out = None
            if topk_weights is not None:
                buf.combine_topk_weights[:n].copy_(topk_weights)
                w_out = torch.empty(inner.num_tokens, self.num_topk, dtype=torch.float32, device=x.device)
            y = buf.combine(bias=total_bias.to(torch.bfloat16) if total_bias is not None else None, handle=inner,
                            topk_weights_out=w_out)
            return y, w_out

        (y, w_out), ev = self._run(fn, previous_event, async_finish, (x,))
        return y, w_out, ev

    # ---- low-latency mode

    def _need_ll(self) -> moe_ep.LowLatencyBuffer:
        if self._ll is None:
            raise RuntimeError("construct the Buffer with low_latency_mode=True")
        return self._ll

    def clean_low_latency_buffer(self, num_max_dispatch_tokens_per_rank: int, hidden: int, num_experts: int) -> None:
        """Nothing to clean: counts carry the call number, and slots are rewritten before they are read."""

    def low_latency_dispatch(self, x: torch.Tensor, topk_idx: torch.Tensor, num_max_dispatch_tokens_per_rank: int,
                             num_experts: int, use_fp8: bool = False, round_scale: bool = False, use_ue8m0: bool = False,
                             async_finish: bool = False, return_recv_hook: bool = False,
                             cumulative_local_expert_recv_stats: Optional[torch.Tensor] = None,
                             dispatch_wait_recv_cost_stats: Optional[torch.Tensor] = None):
        """``(packed_recv_x | (packed_recv_x, scales), packed_recv_count, handle, event, hook)``."""
        ll = self._need_ll()
        if use_fp8 != ll.fp8:
            raise ValueError(f"this buffer was built with low_latency_fp8={ll.fp8}")
        if round_scale or use_ue8m0:
            raise NotImplementedError("power-of-two scales are not offered; scales are fp32")
        if num_max_dispatch_tokens_per_rank != ll.max_tokens or num_experts != ll.num_experts:
            raise ValueError("sizes differ from the ones the buffer was built with")
        r, ev = self._run(lambda: ll.dispatch(x, topk_idx), None, async_finish, (x, topk_idx))
        if cumulative_local_expert_recv_stats is not None:
            cumulative_local_expert_recv_stats.add_(r.count.to(cumulative_local_expert_recv_stats.dtype))
        handle = (r.src_info, r.layout_range, num_max_dispatch_tokens_per_rank, self.hidden, num_experts, r)
        recv = (r.x, r.scales) if ll.fp8 else r.x
        return recv, r.count, handle, ev, (lambda: None) if return_recv_hook else None

    def get_next_low_latency_combine_buffer(self, handle: tuple) -> torch.Tensor:
        """The peer-readable expert-output tensor: write there and pass ``zero_copy=True`` to skip one copy."""
        return self._need_ll().expert_output

    def low_latency_combine(self, x: torch.Tensor, topk_idx: torch.Tensor, topk_weights: torch.Tensor, handle: tuple,
                            use_logfmt: bool = False, async_finish: bool = False, return_recv_hook: bool = False,
                            zero_copy: bool = False, out: Optional[torch.Tensor] = None,
                            combine_wait_recv_cost_stats: Optional[torch.Tensor] = None):
        """``(combined_x, event, hook)``"""
        ll = self._need_ll()
        if use_logfmt:
            raise NotImplementedError("rows travel as bf16")
        r: moe_ep.LowLatencyRecv = handle[5]
        y, ev = self._run(lambda: ll.combine(topk_idx, topk_weights, r, None if zero_copy else x, out), None,
                          async_finish, (x, topk_idx, topk_weights))
        return y, ev, (lambda: None) if return_recv_hook else None


__all__ = ["Buffer", "Config", "EventOverlap"]
