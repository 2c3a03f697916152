"""PyTorch FSDP2 (``fully_shard``) and DistributedDataParallel over communicators of this package.

    torchrun --nproc-per-node 2 --master-addr 127.0.0.1 examples/fsdp_device_mesh.py            # gloo, CPU
    torchrun --nproc-per-node 8 --master-addr 127.0.0.1 examples/fsdp_device_mesh.py --cuda     # b200 backend

``init_device_mesh`` turns one communicator per mesh dimension into a ``torch.distributed.DeviceMesh``;
everything PyTorch builds on process groups (FSDP2, DDP, DTensor, distributed checkpoint) then runs on
the communicator's collectives.
"""
import argparse
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import torchcomms_b200 as tc  # noqa: E402
from torchcomms_b200.device_mesh import init_device_mesh  # noqa: E402


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--cuda", action="store_true")
    ap.add_argument("--steps", type=int, default=5)
    args = ap.parse_args()
    local = int(os.environ.get("LOCAL_RANK", "0"))
    dev = torch.device("cuda", local) if args.cuda else torch.device("cpu")
    if args.cuda:
        torch.cuda.set_device(dev)
    comm = tc.new_comm("b200" if args.cuda else "gloo", dev, name="dp")
    mesh = init_device_mesh(mesh_dim_comms=(comm,), mesh_dim_names=("dp",))

    from torch.distributed.fsdp import fully_shard

    torch.manual_seed(0)
    model = torch.nn.Sequential(torch.nn.Linear(256, 1024), torch.nn.GELU(), torch.nn.Linear(1024, 256)).to(dev)
    for layer in model:
        if isinstance(layer, torch.nn.Linear):
            fully_shard(layer, mesh=mesh)
    fully_shard(model, mesh=mesh)
    opt = torch.optim.AdamW(model.parameters(), lr=1e-3)
    g = torch.Generator(device="cpu").manual_seed(comm.get_rank())
    for step in range(args.steps):
        x = torch.randn(32, 256, generator=g).to(dev)
        loss = (model(x) - x).pow(2).mean()
        opt.zero_grad()
        loss.backward()
        opt.step()
        if comm.get_rank() == 0:
            print(f"step {step}: loss {loss.item():.4f}")
    comm.finalize()


if __name__ == "__main__":
    main()
