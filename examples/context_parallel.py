"""Sequence-sharded attention (ring and Ulysses, with gradients) and redistribution of a tensor between two rank
groups. Runs on GPUs (`b200`) or on CPU with `--backend gloo`; needs an even number of ranks (2 or more)."""
import argparse
import os
import sys
from datetime import timedelta

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import torchcomms_b200 as tc  # noqa: E402
from torchcomms_b200.ops.reshard import REPLICATE, Mesh, Shard, reshard  # noqa: E402
from torchcomms_b200.parallel.context import SeqHeadsExchange, ring_attention, ulysses_attention, zigzag_shard  # noqa: E402


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--backend", default="b200")
    args = ap.parse_args()
    local = int(os.environ.get("LOCAL_RANK", "0"))
    dev = torch.device("cuda", local) if args.backend != "gloo" else torch.device("cpu")
    if dev.type == "cuda":
        torch.cuda.set_device(dev)
    comm = tc.new_comm(args.backend, dev, name="cp", timeout=timedelta(seconds=60))
    rank, n = comm.get_rank(), comm.get_size()

    torch.manual_seed(0)                                   # every rank builds the same full tensors, then keeps its part
    b, h, s, d = 1, 2 * n, 64 * n, 32
    q, k, v = (torch.randn(b, h, s, d, device=dev) for _ in range(3))
    full = torch.nn.functional.scaled_dot_product_attention(q, k, v, is_causal=True)

    # ring attention, load-balanced zigzag layout, with its backward pass
    zq, zk, zv = (zigzag_shard(t, rank, n).contiguous().requires_grad_(True) for t in (q, k, v))
    out = ring_attention(zq, zk, zv, comm, causal=True, layout="zigzag")
    out.square().sum().backward()
    err_ring = (out.detach() - zigzag_shard(full, rank, n)).abs().max()

    # Ulysses: sequence shards <-> head shards; the fused exchange kernel where the backend has it
    sl = slice(rank * s // n, (rank + 1) * s // n)
    ex = SeqHeadsExchange(comm)
    o2 = ulysses_attention(q[:, :, sl].contiguous(), k[:, :, sl].contiguous(), v[:, :, sl].contiguous(), comm, causal=True,
                           exchange=ex)
    err_uly = (o2 - full[:, :, sl]).abs().max()
    ex.close()

    # the first half of the ranks holds a weight sharded by rows, the second half wants it sharded by columns
    half = n // 2
    weight = torch.arange(8 * half * 4 * half, dtype=torch.float32, device=dev).view(8 * half, 4 * half)
    src = Mesh((1, half), 0, (REPLICATE, Shard(0)))
    dst = Mesh((1, half), half, (REPLICATE, Shard(1)))
    mine = weight.chunk(half, 0)[rank].contiguous() if rank < half else None
    want = torch.empty(8 * half, 4, device=dev) if rank >= half else None
    reshard(comm, mine, src, want, dst, global_shape=weight.shape)
    ok = want is None or torch.equal(want, weight.chunk(half, 1)[rank - half])

    print(f"rank {rank}: ring |err| {float(err_ring):.2e}, ulysses |err| {float(err_uly):.2e} (fused exchange: {ex.fused}), "
          f"reshard {'ok' if ok else 'MISMATCH'}")
    comm.finalize()


if __name__ == "__main__":
    main()
