"""Sequence-parallel SwiGLU MLP: the all-gather runs inside the up-projection GEMM and the
reduce-scatter inside the down-projection's epilogue (bf16 and fp8, tcgen05)."""
import os

import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import torchcomms_b200 as tc  # noqa: E402
from torchcomms_b200.parallel.tensor import TensorParallelMLP


def main():
    local = int(os.environ.get("LOCAL_RANK", "0"))
    dev = torch.device("cuda", local)
    torch.cuda.set_device(dev)
    comm = tc.new_comm("b200", dev, name="tp")
    n = comm.get_size()
    hidden, ffn, tokens = 8192, 28672, 8192
    mlp = TensorParallelMLP(hidden, ffn, comm, device=dev, dtype=torch.bfloat16)
    x_shard = torch.randn(tokens // n, hidden, device=dev, dtype=torch.bfloat16)   # tokens sharded over the ranks
    y_fused = mlp.forward_fused(x_shard)            # two fused kernels + SwiGLU
    y_fp8 = mlp.forward_fused(x_shard, fp8=True)    # the same on e4m3 operands (per-token / per-channel scales)
    y_ref = mlp(x_shard)                            # functional collectives + cuBLAS, differentiable
    torch.cuda.synchronize()
    if comm.get_rank() == 0:
        print("max |fused - unfused| =", (y_fused.float() - y_ref.float()).abs().max().item())
        rel = (y_fp8.float() - y_ref.float()).norm() / y_ref.float().norm()
        print("relative error of the fp8 path =", rel.item())
    comm.finalize()


if __name__ == "__main__":
    main()
