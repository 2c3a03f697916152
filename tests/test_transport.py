"""One-sided point-to-point transport on host memory: in-process pairs, two
processes, refused requests, and the tensor publisher.

Modelled on comms/torchcomms/transport/tests (write / read between two
transports, views, remote buffers that pickle, registration reuse).
"""
import os
import pickle
import time
from datetime import timedelta

import pytest
import torch

from tests.mp_util import run_ranks


def _pair(device=None):
    from torchcomms_b200 import transport as T

    a, b = T.P2pTransport(device), T.P2pTransport(device)
    ua, ub = a.bind(), b.bind()
    assert ua.startswith(b"b200p2p://") and a.bind() == ua   # bind is idempotent
    assert not a.connected()
    assert a.connect(ub) == T.OK and b.connect(ua) == T.OK
    assert a.connected() and b.connected()
    return a, b


def test_write_and_read_between_two_transports():
    from torchcomms_b200 import transport as T

    assert T.P2pTransport.supported()
    a, b = _pair()
    src = torch.arange(1 << 20, dtype=torch.float32)           # 4 MB: several socket segments
    dst = torch.zeros_like(src)
    msrc, mdst = T.TransportMemory(src), T.TransportMemory(dst)
    assert msrc.size() == src.nbytes and not msrc.reused_registration()
    assert a.write(msrc.to_view(), mdst.to_remote_buffer()) == T.OK
    assert torch.equal(dst, src)
    # the owner of `src` makes no call while b reads it
    back = torch.empty_like(src)
    mback = T.TransportMemory(back)
    assert b.read(mback.to_mutable_view(), msrc.to_remote_buffer()) == T.OK
    assert torch.equal(back, src)
    ca, cb = a.counters(), b.counters()
    assert ca["socket_ops"] == 1 and ca["socket_bytes"] == src.nbytes and ca["peer_copy_ops"] == 0
    assert cb["served_ops"] == 1 and ca["served_ops"] == 1 and ca["rejected"] == 0
    a.close()
    b.close()
    assert not a.connected()


def test_views_slices_and_async_futures():
    from torchcomms_b200 import transport as T

    a, b = _pair()
    src = torch.arange(4096, dtype=torch.uint8)
    dst = torch.zeros(4096, dtype=torch.uint8)
    msrc, mdst = T.TransportMemory(src), T.TransportMemory(dst)
    view = msrc.to_view(1024, 512)
    assert view.size() == 512 and not view.mutable and msrc.to_mutable_view().mutable
    remote = mdst.to_remote_buffer().slice(2048, 512)
    futs = [a.write_async(view, remote), a.write_async(msrc.to_view(0, 16), mdst.to_remote_buffer().slice(0, 16))]
    assert [f.wait(10_000) for f in futs] == [T.OK, T.OK] and all(f.done() for f in futs)
    assert torch.equal(dst[2048:2560], src[1024:1536]) and torch.equal(dst[:16], src[:16])
    assert int(dst[16:2048].sum()) == 0 and int(dst[2560:].sum()) == 0
    with pytest.raises(RuntimeError, match="mutable"):
        b.read(msrc.to_view(), mdst.to_remote_buffer())
    with pytest.raises(RuntimeError, match="outside"):
        msrc.to_view(4000, 200)
    a.close()
    b.close()


def test_refused_requests_move_no_bytes():
    from torchcomms_b200 import transport as T

    a, b = _pair()
    src = torch.ones(256, dtype=torch.float32)
    dst = torch.zeros(256, dtype=torch.float32)
    msrc, mdst = T.TransportMemory(src), T.TransportMemory(dst)
    good = mdst.to_remote_buffer()
    # a range that leaves the registration
    assert a.write(msrc.to_view(), T.RemoteBuffer(good.ptr + 512, good.len, good.access_key)) == T.OUT_OF_RANGE
    # a forged nonce
    parts = good.access_key.split(":")
    parts[3] = "deadbeef"
    assert a.write(msrc.to_view(), T.RemoteBuffer(good.ptr, good.len, ":".join(parts))) == T.BAD_KEY
    assert a.write(msrc.to_view(), T.RemoteBuffer(good.ptr, good.len, "nonsense")) == T.BAD_KEY
    # a remote buffer smaller than the local view
    assert a.write(msrc.to_view(), good.slice(0, 16)) == T.SIZE_MISMATCH
    assert int(dst.sum()) == 0 and b.counters()["rejected"] == 2
    # a registration that went away
    del mdst
    assert a.write(msrc.to_view(), good) == T.BAD_KEY
    # the connection survives refusals
    dst2 = torch.zeros(256, dtype=torch.float32)
    mdst2 = T.TransportMemory(dst2)
    assert a.write(msrc.to_view(), mdst2.to_remote_buffer()) == T.OK and torch.equal(dst2, src)
    assert "key" in T.strerror(T.BAD_KEY)
    a.close()
    b.close()


def test_registration_reuse_pickle_and_unconnected():
    from torchcomms_b200 import transport as T

    t = torch.zeros(64)
    m1 = T.TransportMemory(t)
    m2 = T.TransportMemory(t)
    assert not m1.reused_registration() and m2.reused_registration() and m1.access_key == m2.access_key
    rb = pickle.loads(pickle.dumps(m1.to_remote_buffer()))
    assert (rb.ptr, rb.len, rb.access_key) == (t.data_ptr(), t.nbytes, m1.access_key)
    assert T.RdmaTransport is T.P2pTransport and T.RdmaMemory is T.TransportMemory
    lone = T.P2pTransport()
    assert lone.write(m1.to_view(), rb) == T.NOT_CONNECTED
    assert lone.connect(b"tcp://nowhere") == T.NOT_CONNECTED
    lone.close()
    assert lone.write(m1.to_view(), rb) == T.CLOSED
    with pytest.raises(RuntimeError, match="contiguous"):
        T.TransportMemory(torch.zeros(4, 4).t())


def test_peer_that_went_away_is_an_error_not_a_hang():
    from torchcomms_b200 import transport as T

    a, b = _pair()
    src, dst = torch.ones(16), torch.zeros(16)
    msrc, mdst = T.TransportMemory(src), T.TransportMemory(dst)
    remote = mdst.to_remote_buffer()
    b.close()
    assert a.write(msrc.to_view(), remote) in (T.IO_ERROR, T.TIMEOUT)
    assert not a.connected()
    assert a.write(msrc.to_view(), remote) == T.NOT_CONNECTED
    a.close()


def _two_process_worker(rank, world):
    import torch.distributed as dist

    from torchcomms_b200 import transport as T

    store = dist.TCPStore("127.0.0.1", int(os.environ["MASTER_PORT"]), world, rank == 0, timeout=timedelta(seconds=60))
    tr = T.P2pTransport()
    store.set(f"url/{rank}", tr.bind())
    peer = 1 - rank
    assert tr.connect(store.get(f"url/{peer}")) == T.OK
    if rank == 0:
        # owner: registers, publishes the remote buffer, then only waits
        table = torch.arange(1 << 18, dtype=torch.int64)
        inbox = torch.zeros(1024, dtype=torch.int64)
        mt, mi = T.TransportMemory(table), T.TransportMemory(inbox)
        store.set("table", pickle.dumps(mt.to_remote_buffer()))
        store.set("inbox", pickle.dumps(mi.to_remote_buffer()))
        store.wait(["done"])
        assert torch.equal(inbox, torch.arange(1024, dtype=torch.int64) * 3)
        deadline = time.time() + 5           # the service thread counts an operation after it has answered it
        while tr.counters()["served_ops"] < 2 and time.time() < deadline:
            time.sleep(0.01)
        assert tr.counters()["served_ops"] == 2
    else:
        table = pickle.loads(store.get("table"))
        inbox = pickle.loads(store.get("inbox"))
        got = torch.empty(1 << 18, dtype=torch.int64)
        mg = T.TransportMemory(got)
        assert tr.read(mg.to_mutable_view(), table) == T.OK
        assert torch.equal(got, torch.arange(1 << 18, dtype=torch.int64))
        out = torch.arange(1024, dtype=torch.int64) * 3
        assert tr.write(T.TransportMemory(out).to_view(), inbox) == T.OK
        store.set("done", "1")
    store.set(f"bye/{rank}", "1")
    store.wait([f"bye/{peer}"])
    tr.close()


def test_two_processes_one_sided():
    run_ranks(_two_process_worker, 2, timeout=120)


def _publisher_worker(rank, world):
    import torch.distributed as dist

    from torchcomms_b200 import transport as T

    store = dist.TCPStore("127.0.0.1", int(os.environ["MASTER_PORT"]), world, rank == 0, timeout=timedelta(seconds=60))
    torch.manual_seed(0)
    weights = {"layer.w": torch.randn(128, 64), "layer.b": torch.randn(64).to(torch.bfloat16), "empty": torch.empty(0)}
    if rank == 0:
        with T.TensorPublisher(weights) as pub:
            man = pub.manifest()
            assert man.names() == ["layer.w", "layer.b"] and man.nbytes() == 128 * 64 * 4 + 64 * 2
            store.set("manifest", pickle.dumps(man))
            store.wait([f"got/{r}" for r in range(1, world)])
            assert pub.counters()["served_ops"] == 2 * (world - 1) + 1
    else:
        man = pickle.loads(store.get("manifest"))
        if rank == 1:
            into = {"layer.w": torch.zeros(128, 64), "layer.b": torch.zeros(64, dtype=torch.bfloat16)}
            got = T.fetch_tensors(man, into=into)
            assert got["layer.w"] is into["layer.w"]
            with pytest.raises(ValueError, match="destination"):
                T.fetch_tensors(man, into={"layer.w": torch.zeros(64, 128), "layer.b": into["layer.b"]})
            only = T.fetch_tensors(man, names=["layer.b"])
            assert list(only) == ["layer.b"] and torch.equal(only["layer.b"], weights["layer.b"])
        else:
            got = T.fetch_tensors(man)
            store.wait(["got/1"])                            # rank 1 makes one extra read; keep the count exact
        assert torch.equal(got["layer.w"], weights["layer.w"]) and torch.equal(got["layer.b"], weights["layer.b"])
        store.set(f"got/{rank}", "1")


def test_publisher_serves_several_consumers():
    run_ranks(_publisher_worker, 3, timeout=120)


def test_segment_registration_is_shared_by_ranges_inside_it():
    """What the caching-allocator hook does for device segments, driven by hand on host memory."""
    from torchcomms_b200 import transport as T

    a, b = _pair()
    arena = torch.zeros(1 << 16, dtype=torch.uint8)              # stands for one allocator segment
    before = T.segment_count()
    T.register_segment(arena.data_ptr(), arena.nbytes, -1)
    assert T.segment_count() == before + 1
    t1, t2 = arena[1024:2048], arena[8192:8192 + 4096]           # two "tensors" carved from it
    m1, m2 = T.TransportMemory(t1), T.TransportMemory(t2)
    assert m1.reused_registration() and m2.reused_registration() and m1.access_key == m2.access_key
    src = torch.arange(1024, dtype=torch.int32).view(torch.uint8)[:1024].clone()
    assert a.write(T.TransportMemory(src).to_view(), m1.to_remote_buffer()) == T.OK
    assert torch.equal(arena[1024:2048], src) and int(arena[:1024].sum()) == 0 and int(arena[2048:].sum()) == 0
    # a range outside the segment is a registration of its own
    outside = torch.zeros(64, dtype=torch.uint8)
    assert not T.TransportMemory(outside).reused_registration()
    # once the segment is gone its key stops validating, also for views made earlier
    remote = m2.to_remote_buffer()
    T.unregister_segment(arena.data_ptr())
    assert T.segment_count() == before
    assert a.write(T.TransportMemory(src).to_view(0, 512), remote.slice(0, 512)) == T.BAD_KEY
    a.close()
    b.close()
