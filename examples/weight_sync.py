"""Weight hand-over between two processes with the one-sided transport.

    python examples/weight_sync.py            # host memory; add --cuda on a GPU box

The trainer process publishes its parameters once; the replica process pulls
them with one-sided reads (the trainer makes no call per transfer).  With
``--cuda`` both sides keep the tensors on GPU 0 and every read is one device
copy through a CUDA IPC mapping.
"""
import argparse
import multiprocessing as mp
import os
import pickle
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import torch  # noqa: E402


def trainer(conn, cuda):
    from torchcomms_b200.transport import TensorPublisher

    dev = torch.device("cuda", 0) if cuda else torch.device("cpu")
    torch.manual_seed(0)
    params = {f"layers.{i}.weight": torch.randn(1024, 1024, device=dev) for i in range(8)}
    with TensorPublisher(params) as pub:
        conn.send(pickle.dumps(pub.manifest()))
        checks = conn.recv()                     # the replica reports what it got
        for name, total in checks.items():
            assert abs(float(params[name].sum()) - total) < 1e-2, name
        print(f"trainer: served {pub.counters()['served_ops']} socket requests, "
              f"{len(checks)} tensors verified")


def replica(conn, cuda):
    from torchcomms_b200.transport import fetch_tensors

    dev = torch.device("cuda", 0) if cuda else torch.device("cpu")
    manifest = pickle.loads(conn.recv())
    got = fetch_tensors(manifest, device=dev)
    print(f"replica: pulled {len(got)} tensors, {manifest.nbytes() >> 20} MB")
    conn.send({k: float(v.sum()) for k, v in got.items()})


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--cuda", action="store_true")
    args = ap.parse_args()
    ctx = mp.get_context("spawn")
    a, b = ctx.Pipe()
    procs = [ctx.Process(target=trainer, args=(a, args.cuda)), ctx.Process(target=replica, args=(b, args.cuda))]
    for p in procs:
        p.start()
    for p in procs:
        p.join(120)
    sys.exit(0 if all(p.exitcode == 0 for p in procs) else 1)
