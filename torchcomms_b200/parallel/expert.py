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
sum over destination ranks.  Forward only (inference / evaluation); training
through the kernels would need the mirrored dispatch of gradients.

Parity: the usage pattern of comms/prims/collectives/link_ep (Buffer.dispatch
-> experts -> Buffer.combine, link_ep/buffer.py:76-660).
"""
from __future__ import annotations

from typing import Callable, List

import torch
from torch import nn

from .. import TorchComm
from ..ops.moe_ep import Buffer


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
