"""One-sided transport on device memory: the CUDA IPC peer-copy path between two
processes, the staged (socket + pinned bounce buffer) path, and mixed host /
device transfers.  Both processes use GPU 0, so one GPU is enough; the copies
are ordinary stream-ordered memcpys, nothing waits on another process's kernel.
"""
import os
import pickle
from datetime import timedelta

import pytest
import torch

from tests.mp_util import run_ranks

pytestmark = pytest.mark.gpu


def test_same_process_device_copy_and_mixed_paths():
    from torchcomms_b200 import transport as T

    dev = torch.device("cuda", 0)
    a, b = T.P2pTransport(dev), T.P2pTransport(dev)
    ua, ub = a.bind(), b.bind()
    assert a.connect(ub) == T.OK and b.connect(ua) == T.OK
    src = torch.randn(3 << 20, device=dev)
    dst = torch.zeros_like(src)
    msrc, mdst = T.TransportMemory(src), T.TransportMemory(dst)
    assert a.write(msrc.to_view(), mdst.to_remote_buffer()) == T.OK
    assert torch.equal(dst, src)
    assert a.counters()["peer_copy_ops"] == 1 and a.counters()["socket_ops"] == 0
    # host view -> device memory goes through the owner's service thread (9 MB + 4: three bounce pieces)
    host = torch.randint(0, 255, ((9 << 20) + 4,), dtype=torch.uint8)
    dev_dst = torch.zeros((9 << 20) + 4, dtype=torch.uint8, device=dev)
    mh, md = T.TransportMemory(host), T.TransportMemory(dev_dst)
    assert a.write(mh.to_view(), md.to_remote_buffer()) == T.OK
    assert torch.equal(dev_dst.cpu(), host)
    # device view <- host memory
    back = torch.zeros((9 << 20) + 4, dtype=torch.uint8, device=dev)
    mb = T.TransportMemory(back)
    assert a.read(mb.to_mutable_view(), mh.to_remote_buffer()) == T.OK
    assert torch.equal(back.cpu(), host)
    assert a.counters()["socket_ops"] == 2
    a.close()
    b.close()


def _ipc_worker(rank, world, staged):
    import torch.distributed as dist

    from torchcomms_b200 import transport as T

    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    store = dist.TCPStore("127.0.0.1", int(os.environ["MASTER_PORT"]), world, rank == 0, timeout=timedelta(seconds=60))
    tr = T.P2pTransport(dev)
    store.set(f"url/{rank}", tr.bind())
    peer = 1 - rank
    assert tr.connect(store.get(f"url/{peer}")) == T.OK
    n = (5 << 20) + 8                                       # floats: 20 MB + 32 B
    if rank == 0:
        table = torch.arange(n, dtype=torch.float32, device=dev)
        inbox = torch.zeros(4096, dtype=torch.float32, device=dev)
        torch.cuda.synchronize()
        mt, mi = T.TransportMemory(table), T.TransportMemory(inbox)
        store.set("table", pickle.dumps(mt.to_remote_buffer()))
        store.set("inbox", pickle.dumps(mi.to_remote_buffer().slice(1024 * 4, 2048 * 4)))
        store.wait(["done"])
        expect = torch.zeros(4096, dtype=torch.float32)
        expect[1024:3072] = torch.arange(2048, dtype=torch.float32) + 0.5
        assert torch.equal(inbox.cpu(), expect)
        c = tr.counters()
        assert c["served_ops"] == (2 if staged else 0) and c["rejected"] == 1
    else:
        table = pickle.loads(store.get("table"))
        inbox = pickle.loads(store.get("inbox"))
        got = torch.empty(n, dtype=torch.float32, device=dev)
        mg = T.TransportMemory(got)
        assert tr.read(mg.to_mutable_view(), table) == T.OK
        assert torch.equal(got, torch.arange(n, dtype=torch.float32, device=dev))
        out = torch.arange(2048, dtype=torch.float32, device=dev) + 0.5
        torch.cuda.synchronize()
        assert tr.write(T.TransportMemory(out).to_view(), inbox) == T.OK
        # a range outside the owner's registration is refused by the owner on either path
        assert tr.write(T.TransportMemory(out).to_view(), T.RemoteBuffer(inbox.ptr + 4096 * 4, inbox.len, inbox.access_key)) == T.OUT_OF_RANGE
        c = tr.counters()
        if staged:
            assert c["socket_ops"] == 2 and c["peer_copy_ops"] == 0
        else:
            assert c["peer_copy_ops"] == 2 and c["peer_copy_bytes"] == n * 4 + 2048 * 4 and c["socket_ops"] == 0
        store.set("done", "1")
    store.set(f"bye/{rank}", "1")
    store.wait([f"bye/{peer}"])
    tr.close()


def test_two_processes_peer_copy_over_ipc():
    run_ranks(_ipc_worker, 2, args=(False,), timeout=150)


def test_two_processes_staged():
    run_ranks(_ipc_worker, 2, args=(True,), timeout=150, extra_env={"B200COMMS_TRANSPORT_STAGED": "1"})


def test_caching_allocator_hook_shares_segment_registrations():
    from torchcomms_b200 import transport as T

    dev = torch.device("cuda", 0)
    warm = torch.zeros(1 << 20, device=dev)                     # a segment that exists before the hook
    T.init_caching_allocator_hook()
    T.init_caching_allocator_hook()                             # idempotent
    assert T.segment_count() >= 1
    m0 = T.TransportMemory(warm)
    assert m0.reused_registration()
    torch.cuda.empty_cache()                                    # no cached block can serve the next allocation
    before = T.segment_count()
    big = torch.empty(96 << 20, dtype=torch.uint8, device=dev)  # forces a new segment
    assert T.segment_count() == before + 1
    x, y = big[: 1 << 20], big[(8 << 20): (9 << 20)]
    mx, my = T.TransportMemory(x), T.TransportMemory(y)
    assert mx.reused_registration() and my.reused_registration() and mx.access_key == my.access_key
    a, b = T.P2pTransport(dev), T.P2pTransport(dev)
    ua, ub = a.bind(), b.bind()
    assert a.connect(ub) == T.OK and b.connect(ua) == T.OK
    x.copy_(torch.randint(0, 255, (1 << 20,), dtype=torch.uint8, device=dev))
    torch.cuda.synchronize()
    assert a.write(mx.to_view(), my.to_remote_buffer()) == T.OK
    assert torch.equal(x, y)
    a.close()
    b.close()
    del mx, my, x, y, big
    torch.cuda.empty_cache()
    assert T.segment_count() <= before
