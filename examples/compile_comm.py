"""Communicator methods inside `torch.compile(fullgraph=True)`. Runs on GPUs (`b200`) or on CPU with `--backend gloo`
(there the `aot_eager` backend of torch.compile is used, which needs no C++ toolchain)."""
import argparse
import os
import sys
from datetime import timedelta

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import torchcomms_b200 as tc  # noqa: E402
from torchcomms_b200.functional.dynamo import register_with_dynamo  # noqa: E402
from torchcomms_b200.functional.inductor import register_with_inductor  # noqa: E402


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--backend", default="b200")
    args = ap.parse_args()
    local = int(os.environ.get("LOCAL_RANK", "0"))
    dev = torch.device("cuda", local) if args.backend != "gloo" else torch.device("cpu")
    if dev.type == "cuda":
        torch.cuda.set_device(dev)
    register_with_dynamo()          # communicator methods become traceable (or: TORCHCOMMS_PATCH_FOR_COMPILE=1)
    register_with_inductor()        # Inductor lowerings: in-place all-reduce, start / wait kernels
    comm = tc.new_comm(args.backend, dev, name="world", timeout=timedelta(seconds=60))
    rank, size = comm.get_rank(), comm.get_size()

    def step(w, x, gathered):
        y = x * w
        comm.all_reduce(y, tc.ReduceOp.SUM, False)                 # recorded as an operator + copy_, differentiable
        work = comm.all_gather_single(gathered, y, True)           # start now ...
        z = torch.relu(y) * comm.get_size() + comm.get_rank()      # ... rank and size are constants of the graph
        work.wait()                                                # ... wait_tensor here
        return z.sum() + gathered.sum()

    compiled = torch.compile(step, fullgraph=True, backend="inductor" if dev.type == "cuda" else "aot_eager")
    w = torch.full((1024,), 0.5, device=dev, requires_grad=True)
    x = torch.full((1024,), float(rank + 1), device=dev)
    gathered = torch.zeros(size * 1024, device=dev)
    loss = compiled(w, x, gathered)
    loss.backward()
    expect = step(w.detach(), x, torch.zeros_like(gathered))
    if rank == 0:
        print(f"compiled {loss.item():.1f}  eager {expect.item():.1f}  |grad| {w.grad.abs().sum().item():.1f}")
    comm.finalize()


if __name__ == "__main__":
    main()
