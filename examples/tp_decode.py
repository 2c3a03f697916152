"""Tensor-parallel decode step tail: the row-parallel projection's partial sums are all-reduced,
added to the residual stream and RMS-normalised by ONE kernel (one cross-GPU barrier) instead of
an all-reduce followed by two elementwise kernels."""
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import torchcomms_b200 as tc  # noqa: E402
from torchcomms_b200.ops.ar_norm import AllReduceRMSNorm  # noqa: E402


def main():
    local = int(os.environ.get("LOCAL_RANK", "0"))
    dev = torch.device("cuda", local)
    torch.cuda.set_device(dev)
    comm = tc.new_comm("b200", dev, name="decode")
    n, hidden, k_local, batch = comm.get_size(), 8192, 28672 // comm.get_size(), 16
    torch.manual_seed(comm.get_rank())
    w_down = (torch.randn(hidden, k_local, device=dev) * 0.02).to(torch.bfloat16)     # this rank's columns
    norm_w = torch.ones(hidden, device=dev, dtype=torch.bfloat16)
    fused = AllReduceRMSNorm(comm, hidden)
    act = torch.randn(batch, k_local, device=dev).to(torch.bfloat16)
    residual = torch.zeros(batch, hidden, device=dev, dtype=torch.bfloat16)
    check = residual.clone()
    partial = act @ w_down.t()                       # [batch, hidden], partial over the ranks
    normed = fused(partial, norm_w, residual=residual)            # residual <- sum(partial) + residual
    expect = fused._unfused(partial, norm_w, check)               # all_reduce, add, rmsnorm as separate steps
    torch.cuda.synchronize()
    if comm.get_rank() == 0:
        print(f"{n} ranks: max |fused - three steps| = {(normed.float() - expect.float()).abs().max().item():.4f}")
    comm.finalize()


if __name__ == "__main__":
    main()
