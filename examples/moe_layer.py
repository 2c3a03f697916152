"""Expert-parallel MoE layer: dispatch quantises to block-scaled fp8 and permutes inside the kernel that
stores the rows into the expert ranks; combine returns and sums the expert outputs."""
import os

import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import torchcomms_b200 as tc  # noqa: E402
from torchcomms_b200.parallel.expert import ExpertParallelMoE


def main():
    local = int(os.environ.get("LOCAL_RANK", "0"))
    dev = torch.device("cuda", local)
    torch.cuda.set_device(dev)
    comm = tc.new_comm("b200", dev, name="ep")
    n = comm.get_size()
    hidden, experts, topk, tokens = 2048, 8 * n, 2, 1024
    make = lambda: torch.nn.Sequential(torch.nn.Linear(hidden, 4 * hidden), torch.nn.GELU(),
                                       torch.nn.Linear(4 * hidden, hidden)).to(dev, torch.bfloat16)
    router = torch.nn.Linear(hidden, experts, bias=False).to(dev, torch.bfloat16)
    comm.broadcast(router.weight.data, 0, False)   # every rank must route alike
    moe = ExpertParallelMoE(comm, hidden, experts, topk, max_tokens=tokens, experts=[make() for _ in range(experts // n)],
                            router=router)
    y = moe(torch.randn(tokens, hidden, device=dev, dtype=torch.bfloat16))
    torch.cuda.synchronize()
    if comm.get_rank() == 0:
        print("output", tuple(y.shape), y.dtype)
    del moe
    comm.finalize()


if __name__ == "__main__":
    main()
