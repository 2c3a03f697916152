"""The CUDA backend end to end: one rank per GPU (two by default, more with
B200COMMS_TEST_WORLD), and a single-rank communicator when there is only one GPU.

Per-operation matrix after the reference's integration tests
(comms/torchcomms/tests/integration/py/AllReduceTest.py:22-110): synchronous,
asynchronous with wait, and CUDA-graph capture with replays; expected values
are closed-form from ``ones * (rank + 1)``.
"""
import os
from datetime import timedelta

import pytest
import torch

from tests.mp_util import run_ranks

pytestmark = pytest.mark.gpu


def _battery(rank, world, backend_name="b200"):
    import torchcomms_b200 as tc

    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    comm = tc.new_comm(backend_name, dev, name="battery", timeout=timedelta(seconds=60),
                       abort_process_on_timeout_or_error=False)
    assert comm.get_rank() == rank and comm.get_size() == world
    impl = comm.get_backend_impl()
    tri = world * (world + 1) // 2

    def ones(n, dtype=torch.float32):
        return torch.ones(n, dtype=dtype, device=dev) * (rank + 1)

    # all_reduce: sizes on both sides of the one-shot / two-shot switch, dtypes, ops
    for dtype in (torch.float32, torch.bfloat16, torch.float16):
        for n in (1, 1000, 100_000, 3_000_000):
            for async_op in (False, True):
                t = ones(n, dtype)
                w = comm.all_reduce(t, tc.ReduceOp.SUM, async_op)
                w.wait()
                torch.cuda.current_stream().synchronize()
                assert torch.equal(t, torch.full((n,), float(tri), dtype=dtype, device=dev)), (dtype, n, async_op)
    t = ones(5000); comm.all_reduce(t, tc.ReduceOp.AVG, False)
    torch.testing.assert_close(t, torch.full((5000,), tri / world, device=dev))
    t = ones(5000); comm.all_reduce(t, tc.ReduceOp.MAX, False)
    assert torch.equal(t, torch.full((5000,), float(world), device=dev))
    t = ones(5000); comm.all_reduce(t, tc.ReduceOp.MIN, False)
    assert torch.equal(t, torch.ones(5000, device=dev))
    t = ones(5000); comm.all_reduce(t, tc.ReduceOp.PREMUL_SUM(0.5), False)
    torch.testing.assert_close(t, torch.full((5000,), tri * 0.5, device=dev))
    for algo in ("oneshot", "twoshot") + (("nccl",) if world > 1 else ()):
        t = ones(30_000); comm.all_reduce(t, tc.ReduceOp.SUM, False, hints={"algo": algo})
        assert torch.equal(t, torch.full((30_000,), float(tri), device=dev)), algo
    if world > 1:
        ti = torch.full((64,), rank + 1, dtype=torch.int64, device=dev)
        comm.all_reduce(ti, tc.ReduceOp.SUM, False)  # integer dtypes ride on NCCL
        assert torch.equal(ti, torch.full((64,), tri, dtype=torch.int64, device=dev))

    # all_gather_single (+ fused fp32 -> bf16 cast), list form, uneven form
    for n in (7, 4096, 1_000_001):
        out = torch.empty(world * n, device=dev)
        comm.all_gather_single(out, ones(n), True).wait()
        assert torch.equal(out, torch.arange(1, world + 1, device=dev).repeat_interleave(n).float())
    out16 = torch.empty(world * 5000, dtype=torch.bfloat16, device=dev)
    comm.all_gather_single(out16, ones(5000), False)
    assert torch.equal(out16.float(), torch.arange(1, world + 1, device=dev).repeat_interleave(5000).float())
    outs = [torch.empty(33, device=dev) for _ in range(world)]
    comm.all_gather(outs, ones(33), False)
    for r in range(world):
        assert torch.equal(outs[r], torch.full((33,), float(r + 1), device=dev))
    outs = [torch.empty(r + 1, device=dev) for r in range(world)]
    comm.all_gather_v(outs, ones(rank + 1), False)
    for r in range(world):
        assert torch.equal(outs[r], torch.full((r + 1,), float(r + 1), device=dev))

    # reduce_scatter_single: plain, mixed precision, bf16 on the wire; list and uneven forms
    for n in (5, 4096, 500_001):
        out = torch.empty(n, device=dev)
        comm.reduce_scatter_single(out, ones(world * n), tc.ReduceOp.SUM, True).wait()
        assert torch.equal(out, torch.full((n,), float(tri), device=dev))
    out = torch.empty(4096, device=dev)
    comm.reduce_scatter_single(out, ones(world * 4096, torch.bfloat16), tc.ReduceOp.AVG, False)
    torch.testing.assert_close(out, torch.full((4096,), tri / world, device=dev), rtol=1e-2, atol=1e-2)
    out = torch.empty(4096, device=dev)
    impl.reduce_scatter_quantized(out, ones(world * 4096), tc.ReduceOp.SUM, seed=1, async_op=False)
    torch.testing.assert_close(out, torch.full((4096,), float(tri), device=dev), rtol=1e-2, atol=1e-2)
    out = torch.empty(17, device=dev)
    comm.reduce_scatter(out, [ones(17) for _ in range(world)], tc.ReduceOp.SUM, False)
    assert torch.equal(out, torch.full((17,), float(tri), device=dev))
    out = torch.empty(rank + 1, device=dev)
    comm.reduce_scatter_v(out, [ones(r + 1) for r in range(world)], tc.ReduceOp.SUM, False)
    assert torch.equal(out, torch.full((rank + 1,), float(tri), device=dev))

    # all_to_all family
    n = 1024
    src = torch.cat([torch.full((n,), float(rank * world + d), device=dev) for d in range(world)])
    dst = torch.empty_like(src)
    comm.all_to_all_single(dst, src, False)
    assert torch.equal(dst, torch.cat([torch.full((n,), float(s * world + rank), device=dev) for s in range(world)]))
    in_splits = [d + 1 for d in range(world)]
    out_splits = [rank + 1] * world
    src = torch.cat([torch.full((d + 1, 3), float(rank * 10 + d), device=dev) for d in range(world)])
    dst = torch.empty(sum(out_splits), 3, device=dev)
    comm.all_to_all_v_single(dst, src, out_splits, in_splits, True).wait()
    assert torch.equal(dst, torch.cat([torch.full((rank + 1, 3), float(s * 10 + rank), device=dev) for s in range(world)]))
    dst.zero_()
    impl.device_alltoallv_single(dst, src, torch.tensor(out_splits, device=dev), torch.tensor(in_splits, device=dev), False)
    assert torch.equal(dst, torch.cat([torch.full((rank + 1, 3), float(s * 10 + rank), device=dev) for s in range(world)]))
    outs = [torch.empty(9, device=dev) for _ in range(world)]
    comm.all_to_all(outs, [torch.full((9,), float(rank * world + d), device=dev) for d in range(world)], False)
    for s in range(world):
        assert torch.equal(outs[s], torch.full((9,), float(s * world + rank), device=dev))

    # rooted operations
    root = world - 1
    b = ones(100_000); comm.broadcast(b, root, False)
    assert torch.equal(b, torch.full((100_000,), float(root + 1), device=dev))
    t = ones(1000); comm.reduce(t, 0, tc.ReduceOp.SUM, False)
    assert torch.equal(t, torch.full((1000,), float(tri if rank == 0 else rank + 1), device=dev))
    # bandwidth-class reduce: reduce-scatter + gather to the root; non-root inputs stay untouched
    n_big = world * 8 * 40_000
    t = ones(n_big); comm.reduce(t, root, tc.ReduceOp.SUM, False)
    torch.cuda.synchronize()
    assert torch.equal(t, torch.full((n_big,), float(tri if rank == root else rank + 1), device=dev))
    t = ones(n_big, torch.bfloat16); comm.reduce(t, 0, tc.ReduceOp.AVG, True).wait()
    torch.cuda.synchronize()
    torch.testing.assert_close(t.float(), torch.full((n_big,), tri / world if rank == 0 else float(rank + 1), device=dev),
                               rtol=1e-2, atol=1e-2)
    # uneven reduce-scatter with sizeable shares (padded reduce-scatter) and with one dominating share (all-reduce)
    shares = [10_000 + 7 * r for r in range(world)]
    out = torch.empty(shares[rank], device=dev)
    comm.reduce_scatter_v(out, [ones(s) for s in shares], tc.ReduceOp.SUM, False)
    torch.cuda.synchronize()
    assert torch.equal(out, torch.full((shares[rank],), float(tri), device=dev))
    shares = [90_000 if world < 3 else 50_000] + [3] * (world - 1)
    out = torch.empty(shares[rank], device=dev)
    comm.reduce_scatter_v(out, [ones(s) for s in shares], tc.ReduceOp.SUM, True).wait()
    torch.cuda.synchronize()
    assert torch.equal(out, torch.full((shares[rank],), float(tri), device=dev))
    got = torch.empty(5, device=dev)
    comm.scatter(got, [torch.full((5,), float(r), device=dev) for r in range(world)] if rank == root else [], root, False)
    assert torch.equal(got, torch.full((5,), float(rank), device=dev))
    outs = [torch.empty(5, device=dev) for _ in range(world)] if rank == 0 else []
    comm.gather(outs, ones(5), 0, False)
    if rank == 0:
        for r in range(world):
            assert torch.equal(outs[r], torch.full((5,), float(r + 1), device=dev))
    comm.barrier(False)
    comm.barrier(True).wait()

    # point to point (NCCL) in a ring, single and batched
    if world > 1:
        nxt, prv = (rank + 1) % world, (rank - 1) % world
        got = torch.empty(1000, device=dev)
        batch = comm.batch_op_create()
        batch.send(ones(1000), nxt)
        batch.recv(got, prv)
        batch.issue(True).wait()
        assert torch.equal(got, torch.full((1000,), float(prv + 1), device=dev))
        if rank % 2 == 0:
            comm.send(ones(10), nxt, False)
            comm.recv(got[:10], prv, False)
        else:
            tmp = torch.empty(10, device=dev)
            comm.recv(tmp, prv, False)
            comm.send(ones(10), nxt, False)
            assert torch.equal(tmp, torch.full((10,), float(prv + 1), device=dev))

    # CUDA graph: capture an all_reduce and replay it 4 times
    static = ones(20_000)
    graph = torch.cuda.CUDAGraph()
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        with torch.cuda.graph(graph, stream=side):
            comm.all_reduce(static, tc.ReduceOp.SUM, False)
    for i in range(4):
        static.fill_(rank + 1)
        graph.replay()
        torch.cuda.synchronize()
        assert torch.equal(static, torch.full((20_000,), float(tri), device=dev)), i

    # split: even / odd halves
    members = [r for r in range(world) if r % 2 == rank % 2]
    sub = comm.split(members, "parity")
    assert sub.get_size() == len(members) and sub.get_ranks() == members
    t = ones(100); sub.all_reduce(t, tc.ReduceOp.SUM, False)
    assert torch.equal(t, torch.full((100,), float(sum(m + 1 for m in members)), device=dev))
    sub.finalize()

    # one-sided window over peer-exportable memory, then over ordinary memory
    from torchcomms_b200.mem import symmetric_empty

    for make in (lambda: symmetric_empty(comm, (world, 256), torch.float32), lambda: torch.empty(world, 256, device=dev)):
        buf = make()
        buf.zero_()
        win = comm.new_window()
        win.tensor_register(buf)
        assert win.get_size() == buf.nbytes and win.shape == [world, 256]
        comm.barrier(False)
        dst_rank = (rank + 1) % world
        win.put(ones(256), dst_rank, rank * 256, False)
        win.signal(dst_rank, False)
        win.wait_signal((rank - 1) % world, False)
        torch.cuda.synchronize()
        left = (rank - 1) % world
        assert torch.equal(buf[left], torch.full((256,), float(left + 1), device=dev))
        remote = win.map_remote_tensor(dst_rank)
        assert remote.shape == buf.shape
        comm.barrier(False)
        torch.cuda.synchronize()
        assert torch.equal(remote[rank], ones(256))
        assert win.get_attr(dst_rank).access_type == tc.TorchCommWinAccessType.WIN_ACCESS_TYPE_UNIFIED
        assert win.get_device_window() != 0
        del remote
        win.tensor_deregister()

    dump = impl.comm_dump()
    assert dump["rank"] == str(rank) and int(dump["ops_issued"]) > 50
    want = "count/all_reduce/oneshot" if os.environ.get("B200COMMS_AUTO_NCCL") == "0" or world >= 4 else "count/all_reduce/"
    assert any(k.startswith(want) for k in dump)
    torch.cuda.synchronize()
    comm.finalize()


def _world_size():
    return max(1, min(torch.cuda.device_count(), int(os.environ.get("B200COMMS_TEST_WORLD", "2"))))


def test_cuda_backend_battery():
    world = _world_size()
    # NVLS is exercised by default; it is available whenever the box grants multicast.
    run_ranks(_battery, world, timeout=240, extra_env={"B200COMMS_AUTO_NCCL": "0"})


def test_cuda_backend_battery_without_multicast():
    if _world_size() < 2:
        pytest.skip("needs 2 GPUs")
    run_ranks(_battery, 2, timeout=240, extra_env={"B200COMMS_NVLS": "0", "NCCL_NVLS_ENABLE": "0", "B200COMMS_AUTO_NCCL": "0"})


def _variant_matrix(rank, world):
    from datetime import timedelta

    import torchcomms_b200 as tc
    from tests.variant_matrix import VARIANTS_GPU, run_matrix

    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    comm = tc.new_comm("b200", dev, name="matrix", timeout=timedelta(seconds=60), abort_process_on_timeout_or_error=False)
    for dtype in (torch.float32, torch.bfloat16):
        ran = run_matrix(comm, tc, dev, VARIANTS_GPU, dtype=dtype)
        assert ran == 16 * len(VARIANTS_GPU) - 1, ran     # no graph variant for the point-to-point batch
    torch.cuda.synchronize()
    comm.finalize()


def test_every_operation_in_every_calling_variant():
    """16 operations x (sync, sync without the work, async, work dropped early, inputs deleted, CUDA graph)."""
    world = _world_size()
    if world < 2:
        pytest.skip("needs 2 GPUs")
    run_ranks(_variant_matrix, world, timeout=240)


def test_timestamp_ring_single_gpu():
    """GPU-written start / end stamps per operation (`colltrace` hint), read from mapped host memory."""
    import torchcomms_b200 as tc

    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    os.environ.setdefault("MASTER_PORT", "29641")
    os.environ["RANK"], os.environ["WORLD_SIZE"] = "0", "1"
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(0)
    comm = tc.new_comm("b200", dev, name="ring", hints={"colltrace": "8"}, abort_process_on_timeout_or_error=False)
    impl = comm.get_backend_impl()
    t = torch.ones(1 << 20, device=dev)
    for i in range(5):
        comm.all_reduce(t, tc.ReduceOp.SUM, i % 2 == 1).wait()
    torch.cuda.synchronize()
    entries = impl.colltrace_dump()
    assert [e["seq"] for e in entries] == list(range(5))
    for e in entries:
        assert e["op"].startswith("all_reduce") and 0 < e["start_ns"] <= e["end_ns"], e
    assert all(a["end_ns"] <= b["start_ns"] for a, b in zip(entries, entries[1:]))   # one stream order per channel
    comm.finalize()


def test_seq_heads_exchange_single_rank_is_a_copy():
    """With one rank both layouts coincide: the backend call copies, checks shapes and dtypes, and the exchange
    object of the context-parallel layer passes tensors through."""
    import torchcomms_b200 as tc
    from torchcomms_b200.parallel.context import SeqHeadsExchange

    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    os.environ.setdefault("MASTER_PORT", "29643")
    os.environ["RANK"], os.environ["WORLD_SIZE"] = "0", "1"
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(0)
    comm = tc.new_comm("b200", dev, name="sh1", abort_process_on_timeout_or_error=False)
    impl = comm.get_backend_impl()
    x = torch.randn(2, 4, 16, 8, device=dev, dtype=torch.bfloat16)
    out = torch.zeros_like(x)
    impl.seq_heads_exchange(out, x, True, False)
    torch.cuda.synchronize()
    assert torch.equal(out, x)
    with pytest.raises(RuntimeError):
        impl.seq_heads_exchange(torch.zeros(2, 4, 8, 8, device=dev, dtype=torch.bfloat16), x, True, False)   # wrong shape
    with pytest.raises(RuntimeError):
        impl.seq_heads_exchange(out.float(), x, True, False)                                                  # dtype mismatch
    ex = SeqHeadsExchange(comm)
    assert not ex.fused and ex.to_heads(x) is x and ex.to_seq(x) is x
    comm.finalize()


def _stalled_peer(rank, world):
    """Rank 1 never joins an all-reduce: rank 0's kernel gives up after its
    device-side wait budget and the next call raises; no GPU hangs or faults."""
    import time

    import torchcomms_b200 as tc

    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    comm = tc.new_comm("b200", dev, name="stall", timeout=timedelta(seconds=20),
                       abort_process_on_timeout_or_error=False,
                       hints={"device_wait_ms": "500", "use_multicast": "0", "use_nccl": "0"})
    t = torch.ones(1024, device=dev)
    comm.all_reduce(t, tc.ReduceOp.SUM, False)  # both ranks: fine
    torch.cuda.synchronize()
    fired = []
    comm.register_abort_hook(lambda: fired.append(True))
    if rank == 0:
        comm.all_reduce(t, tc.ReduceOp.SUM, False)  # peer is absent: bounded wait runs out
        torch.cuda.synchronize()                    # returns: the kernel exited by itself
        deadline = time.time() + 10
        while tc.healthy() and time.time() < deadline:
            time.sleep(0.05)
        assert not tc.healthy()
        assert fired, "abort hook must have run"
        with pytest.raises(RuntimeError, match="unusable after a failure"):
            comm.all_reduce(t, tc.ReduceOp.SUM, False)
        assert comm.is_aborted()
        # the CUDA context is intact
        assert float(torch.ones(8, device=dev).sum()) == 8.0
    else:
        time.sleep(3.0)  # between steps, nothing in flight
    try:
        comm.finalize()
    except RuntimeError:
        pass


def test_absent_peer_is_detected_without_hanging():
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    run_ranks(_stalled_peer, 2, timeout=180, extra_env={"NCCL_NVLS_ENABLE": "0", "B200COMMS_NVLS": "0"})
