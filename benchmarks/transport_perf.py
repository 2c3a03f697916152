"""Bandwidth and latency of the one-sided point-to-point transport between two processes.

    python benchmarks/transport_perf.py                 # host memory over the socket path
    python benchmarks/transport_perf.py --cuda          # device memory: CUDA IPC peer copies (GPU 0 -> GPU 1 if present)
    python benchmarks/transport_perf.py --cuda --staged # device memory through the socket + bounce-buffer path

The owner process registers one buffer and then only waits; the initiator times ``write`` and ``read`` of
growing sizes (host clock around the blocking call, which returns when the bytes are in place).
"""
import argparse
import multiprocessing as mp
import os
import pickle
import sys
import time

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import torch  # noqa: E402


def _device(cuda, index):
    if not cuda:
        return torch.device("cpu")
    return torch.device("cuda", index % max(torch.cuda.device_count(), 1))


def owner(conn, cuda, nbytes):
    from torchcomms_b200 import transport as T

    dev = _device(cuda, 1)
    buf = torch.zeros(nbytes, dtype=torch.uint8, device=dev)
    tr = T.P2pTransport(dev)
    mem = T.TransportMemory(buf)
    conn.send((tr.bind(), pickle.dumps(mem.to_remote_buffer())))
    tr.connect(conn.recv())
    conn.recv()                                   # the initiator says it is done
    print("owner counters:", tr.counters(), flush=True)
    tr.close()


def initiator(conn, cuda, nbytes, iters):
    from torchcomms_b200 import transport as T

    dev = _device(cuda, 0)
    tr = T.P2pTransport(dev)
    url, remote = conn.recv()
    remote = pickle.loads(remote)
    conn.send(tr.bind())
    assert tr.connect(url) == T.OK
    local = torch.ones(nbytes, dtype=torch.uint8, device=dev)
    mem = T.TransportMemory(local)
    size = 4096
    print(f"{'bytes':>12} {'write us':>10} {'GB/s':>8} {'read us':>10} {'GB/s':>8}")
    while size <= nbytes:
        n = max(3, min(iters, (256 << 20) // size))
        row = []
        for op, view in ((tr.write, mem.to_view(0, size)), (tr.read, mem.to_mutable_view(0, size))):
            assert op(view, remote.slice(0, size)) == T.OK          # warm-up (first use maps / validates)
            t0 = time.perf_counter()
            for _ in range(n):
                op(view, remote.slice(0, size))
            dt = (time.perf_counter() - t0) / n
            row += [dt * 1e6, size / dt / 1e9]
        print(f"{size:>12} {row[0]:>10.1f} {row[1]:>8.2f} {row[2]:>10.1f} {row[3]:>8.2f}", flush=True)
        size *= 8
    print("initiator counters:", tr.counters(), flush=True)
    conn.send("done")
    tr.close()


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--cuda", action="store_true")
    ap.add_argument("--staged", action="store_true")
    ap.add_argument("--max-mb", type=int, default=128)
    ap.add_argument("--iters", type=int, default=50)
    args = ap.parse_args()
    if args.staged:
        os.environ["B200COMMS_TRANSPORT_STAGED"] = "1"
    ctx = mp.get_context("spawn")
    a, b = ctx.Pipe()
    nbytes = args.max_mb << 20
    procs = [ctx.Process(target=owner, args=(a, args.cuda, nbytes)),
             ctx.Process(target=initiator, args=(b, args.cuda, nbytes, args.iters))]
    for p in procs:
        p.start()
    for p in procs:
        p.join(600)
    sys.exit(0 if all(p.exitcode == 0 for p in procs) else 1)
