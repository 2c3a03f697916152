"""Communicator basics. Runs on GPUs (`b200` backend) or on CPU with `--backend gloo`."""
import argparse
import os
from datetime import timedelta

import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import torchcomms_b200 as tc  # noqa: E402
from torchcomms_b200.hooks import NanCheckHook, fr


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--backend", default="b200")
    args = ap.parse_args()
    local = int(os.environ.get("LOCAL_RANK", "0"))
    dev = torch.device("cuda", local) if args.backend != "gloo" else torch.device("cpu")
    if dev.type == "cuda":
        torch.cuda.set_device(dev)
    comm = tc.new_comm(args.backend, dev, name="world", timeout=timedelta(seconds=60))
    rank, size = comm.get_rank(), comm.get_size()
    NanCheckHook().register_with_comm(comm)
    recorder = fr.FlightRecorderHook()
    recorder.register_with_comm(comm)

    t = torch.full((1 << 20,), float(rank + 1), device=dev)
    comm.all_reduce(t, tc.ReduceOp.SUM, False)                       # synchronous with respect to the current stream
    work = comm.all_reduce(t, tc.ReduceOp.AVG, True)                 # asynchronous on the communicator's stream
    work.wait()                                                      # the current stream now waits for it
    gathered = torch.empty(size * 4, device=dev)
    comm.all_gather_single(gathered, torch.full((4,), float(rank), device=dev), False)
    shard = torch.empty(1 << 18, device=dev)
    comm.reduce_scatter_single(shard, torch.ones(size << 18, device=dev), tc.ReduceOp.SUM, False)

    if size >= 2:
        nxt, prv = (rank + 1) % size, (rank - 1) % size
        got = torch.empty(8, device=dev)
        batch = comm.batch_op_create()
        batch.send(torch.full((8,), float(rank), device=dev), nxt)
        batch.recv(got, prv)
        batch.issue(False)
        half = comm.split(list(range(size // 2)) if rank < size // 2 else list(range(size // 2, size)), "half")
        if half is not None:
            half.barrier(False)
            half.finalize()
    if rank == 0:
        print(f"{size} ranks on '{comm.get_backend()}': all_reduce -> {t[0].item():.1f}, gathered {gathered[::4].tolist()}")
    comm.finalize()


if __name__ == "__main__":
    main()
