"""Expert-parallel MoE layer on the fused dispatch / combine kernels.

Each rank owns ``num_experts / n`` experts.  ``forward``:

1. router: softmax over expert logits, top-k;
2. ``Buffer.dispatch``: one kernel counts, quantises to block-scaled fp8
   (e4m3, 1x128), permutes and stores every token into the ranks that own its
   experts (rows arrive packed by source rank);
3. local experts run on the received rows (grouped by expert with one sort);
   a row selected by several local experts accumulates their weighted outputs;
4. ``Buffer.combine``: the token's owner pulls its rows back and sums them.

Gate weights are applied on the expert side (step 3), so combine is a plain
sum over destination ranks.  ``ExpertParallelMoE`` is forward only (inference /
evaluation, fp8 rows).  ``ExpertParallelMoETrain`` trains through the same
kernels with bf16 rows: the backward of the combine is a dispatch of the output
gradients along the saved layout, the backward of the dispatch a combine of the
row gradients, and the gate gradients travel back with them, so experts, router
and inputs all receive gradients.  ``ExpertParallelMoEUnfused`` is the same
computation through the functional all-to-all (whose backward is the reverse
all-to-all), gates applied at the token's owner; it runs on any backend,
including gloo, and is the reference the fused layer is tested against.

Parity: the usage pattern of comms/prims/collectives/link_ep (Buffer.dispatch
-> experts -> Buffer.combine, link_ep/buffer.py:76-660).
"""
from __future__ import annotations

from typing import Callable, List, Sequence

import torch
from torch import nn

from .. import TorchComm
from .. import functional as F
from ..ops.moe_ep import Buffer, combine_autograd, dispatch_autograd


class ExpertParallelMoE(nn.Module):
    def __init__(self, comm: TorchComm, hidden: int, num_experts: int, topk: int, max_tokens: int,
                 experts: List[Callable[[torch.Tensor], torch.Tensor]], router: nn.Module, fp8: bool = True):
        super().__init__()
        n = comm.get_size()
        if num_experts % n != 0 or len(experts) != num_experts // n:
            raise ValueError("give exactly num_experts / nranks local experts")
        self.comm, self.hidden, self.num_experts, self.topk = comm, hidden, num_experts, topk
        self.local = num_experts // n
        self.experts = nn.ModuleList(experts) if all(isinstance(e, nn.Module) for e in experts) else experts
        self.router = router
        self.buffer = Buffer(comm, max_tokens=max_tokens, hidden=hidden, num_experts=num_experts, topk=topk, fp8=fp8)

    @torch.no_grad()
    def forward(self, x: torch.Tensor) -> torch.Tensor:
        w, idx = torch.softmax(self.router(x).float(), dim=-1).topk(self.topk, dim=-1)
        d = self.buffer.dispatch(x, idx.to(torch.int32), w)
        n = int(d.num_tokens)                      # the one host read: sizes the expert GEMMs
        if d.scales is not None:
            rows = (d.x[:n].float().view(n, -1, 128) * d.scales[:n].unsqueeze(-1)).view(n, self.hidden).to(torch.bfloat16)
        else:
            rows = d.x[:n]
        out = torch.zeros(n, self.hidden, dtype=torch.float32, device=x.device)
        tidx, tw = d.topk_idx[:n], d.topk_weights[:n]
        for e in range(self.local):
            hit = (tidx == e)
            sel = hit.any(dim=1).nonzero().flatten()
            if sel.numel() == 0:
                continue
            gate = (tw[sel] * hit[sel]).sum(dim=1, keepdim=True)
            out.index_add_(0, sel, self.experts[e](rows[sel]).float() * gate)
        self.buffer.combine_input[:n] = out.to(torch.bfloat16)
        return self.buffer.combine()


class ExpertParallelMoETrain(nn.Module):
    """Differentiable expert-parallel MoE on the fused dispatch / combine kernels (bf16 rows).

    ``y[token] = sum_k gate[token, k] * expert_k(x[token])``; gradients flow to the experts, to the router
    (the gates ride with the rows and their gradients ride back) and to ``x``.
    """

    def __init__(self, comm: TorchComm, hidden: int, num_experts: int, topk: int, max_tokens: int,
                 experts: Sequence[nn.Module], router: nn.Module):
        super().__init__()
        n = comm.get_size()
        if num_experts % n != 0 or len(experts) != num_experts // n:
            raise ValueError("give exactly num_experts / nranks local experts")
        self.comm, self.hidden, self.num_experts, self.topk = comm, hidden, num_experts, topk
        self.local = num_experts // n
        self.experts = nn.ModuleList(experts)
        self.router = router
        self.buffer = Buffer(comm, max_tokens=max_tokens, hidden=hidden, num_experts=num_experts, topk=topk, fp8=False)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        gates, idx = torch.softmax(self.router(x).float(), dim=-1).topk(self.topk, dim=-1)
        rows, w, local_idx, meta = dispatch_autograd(self.buffer, x.to(torch.bfloat16), idx.to(torch.int32), gates)
        out = torch.zeros(rows.shape[0], self.hidden, dtype=torch.float32, device=x.device)
        for e in range(self.local):
            hit = local_idx == e
            sel = hit.any(dim=1).nonzero().flatten()
            if sel.numel() == 0:
                continue
            gate = (w[sel] * hit[sel]).sum(dim=1, keepdim=True)
            out = out.index_add(0, sel, self.experts[e](rows[sel]).float() * gate)
        return combine_autograd(self.buffer, out.to(torch.bfloat16), meta).to(x.dtype)


class ExpertParallelMoEUnfused(nn.Module):
    """Differentiable expert-parallel MoE over functional all-to-all collectives.

    Every (token, expert) pair travels as one row to the rank that owns the expert and comes back
    after the expert ran; ``y[token] = sum_k gate[token, k] * expert_k(x[token])``.  Gradients flow
    to the experts (through the reverse all-to-all), to the router (through the gates) and to ``x``.
    """

    def __init__(self, comm: TorchComm, hidden: int, num_experts: int, topk: int, experts: Sequence[nn.Module],
                 router: nn.Module):
        super().__init__()
        n = comm.get_size()
        if num_experts % n != 0 or len(experts) != num_experts // n:
            raise ValueError("give exactly num_experts / nranks local experts")
        self.comm, self.hidden, self.num_experts, self.topk = comm, hidden, num_experts, topk
        self.local = num_experts // n
        self.experts = nn.ModuleList(experts)
        self.router = router
        self._name = F.register_comm(comm)

    def _exchange_int(self, values: torch.Tensor, send_counts: List[int], recv_counts: List[int]) -> torch.Tensor:
        out = values.new_empty(sum(recv_counts))
        self.comm.all_to_all_v_single(out, values.contiguous(), recv_counts, send_counts, False)
        return out

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        n, rank = self.comm.get_size(), self.comm.get_rank()
        tokens = x.shape[0]
        gates, idx = torch.softmax(self.router(x).float(), dim=-1).topk(self.topk, dim=-1)
        pair_expert = idx.reshape(-1)                                  # [tokens * topk]
        pair_token = torch.arange(tokens, device=x.device).repeat_interleave(self.topk)
        order = torch.argsort(pair_expert // self.local, stable=True)   # pairs grouped by destination rank
        dest = (pair_expert // self.local)[order]
        send_counts = torch.bincount(dest, minlength=n).tolist()
        counts = torch.tensor(send_counts, dtype=torch.int64, device=x.device)
        got = torch.empty_like(counts)
        if n > 1:
            self.comm.all_to_all_single(got, counts, False)
        else:
            got.copy_(counts)
        recv_counts = got.tolist()

        rows = x[pair_token[order]]
        local_expert = (pair_expert[order] % self.local).to(torch.int64)
        if n > 1:
            rows = F.all_to_all_single(rows.contiguous(), self._name, output_split_sizes=recv_counts, input_split_sizes=send_counts)
            local_expert = self._exchange_int(local_expert, send_counts, recv_counts)
        out = torch.zeros_like(rows)
        for e in range(self.local):
            sel = (local_expert == e).nonzero().flatten()
            if sel.numel():
                out = out.index_add(0, sel, self.experts[e](rows[sel]).to(out.dtype))
        if n > 1:
            out = F.all_to_all_single(out.contiguous(), self._name, output_split_sizes=send_counts, input_split_sizes=recv_counts)
        # back at the owner: undo the grouping, apply the gates, sum the top-k contributions per token
        per_pair = torch.empty_like(out).index_copy(0, order, out)     # pair order again: [tokens * topk, hidden]
        weighted = per_pair.view(tokens, self.topk, -1).float() * gates.unsqueeze(-1)
        return weighted.sum(dim=1).to(x.dtype)
