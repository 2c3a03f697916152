"""Collectives on symmetric tensors through the CUDA backend: one rank per GPU
(two by default, more with B200COMMS_TEST_WORLD; a single rank when there is
one GPU).  Checks that the one-pass kernels are the ones that run (per-route
counters of ``comm_dump``), their numerics against closed-form expectations,
asynchronous operations on different channels in flight together, CUDA-graph
capture with release of the bookkeeping when the graph is destroyed, and
registration of allocator memory.
"""
import os
import time
from datetime import timedelta

import pytest
import torch

from tests.mp_util import run_ranks

pytestmark = pytest.mark.gpu


def _symm_battery(rank, world):
    import torchcomms_b200 as tc
    from torchcomms_b200.mem import is_symmetric, symmetric_empty

    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    comm = tc.new_comm("b200", dev, name="symm", timeout=timedelta(seconds=60), abort_process_on_timeout_or_error=False)
    impl = comm.get_backend_impl()
    tri = world * (world + 1) // 2

    def ones(n, dtype=torch.float32):
        return torch.ones(n, dtype=dtype, device=dev) * (rank + 1)

    def count(key):
        return int(impl.comm_dump().get("count/" + key, "0"))

    # ---- all-gather into a symmetric output (plain and with the fp32 -> bf16 cast)
    for n in (8, 4096, 1_000_000):
        out = comm.symm_empty((world * n,), torch.bfloat16)
        assert is_symmetric(comm, out)
        out.zero_()
        for async_op in (False, True):
            comm.all_gather_single(out, ones(n, torch.bfloat16), async_op).wait()
            torch.cuda.synchronize()
            assert torch.equal(out.float(), torch.arange(1, world + 1, device=dev).repeat_interleave(n).float())
        comm.all_gather_single(out, ones(n, torch.float32) * 0.5, False)
        torch.cuda.synchronize()
        assert torch.equal(out.float(), torch.arange(1, world + 1, device=dev).repeat_interleave(n).float() * 0.5)
        comm.symm_free(out)
    if world > 1:
        # the two small sizes take the flag-less exchange, the large one the one-pass kernel
        assert count("all_gather/symm") >= 2 and count("all_gather/lamport") >= 4 and count("all_gather/symm+cast") >= 3

    # ---- reduce-scatter from a symmetric input: bf16 -> bf16, bf16 -> fp32 with AVG, fp32 -> fp32
    for n in (8, 4096, 1_500_000):
        src = comm.symm_empty((world * n,), torch.bfloat16)
        src.copy_(ones(world * n, torch.bfloat16))
        out = torch.empty(n, dtype=torch.bfloat16, device=dev)
        comm.reduce_scatter_single(out, src, tc.ReduceOp.SUM, True).wait()
        torch.cuda.synchronize()
        assert torch.equal(out.float(), torch.full((n,), float(tri), device=dev))
        out32 = torch.empty(n, device=dev)
        comm.reduce_scatter_single(out32, src, tc.ReduceOp.AVG, False)
        torch.cuda.synchronize()
        torch.testing.assert_close(out32, torch.full((n,), tri / world, device=dev), rtol=1e-2, atol=1e-2)
        comm.symm_free(src)
        src32 = comm.symm_empty((world * n,), torch.float32)
        src32.copy_(ones(world * n))
        comm.reduce_scatter_single(out32, src32, tc.ReduceOp.SUM, False)
        torch.cuda.synchronize()
        assert torch.equal(out32, torch.full((n,), float(tri), device=dev))
        comm.symm_free(src32)
    if world > 1:
        assert count("reduce_scatter/symm") >= 5 and count("reduce_scatter/lamport") >= 4

    # ---- all-reduce in place on a symmetric tensor; small sizes take the flag-less kernel
    for dtype in (torch.float32, torch.bfloat16):
        for n in (1, 1000, 16_384, 600_000, 3_000_000):
            t = comm.symm_empty((n,), dtype)
            for it in range(3):
                t.copy_(ones(n, dtype))
                comm.all_reduce(t, tc.ReduceOp.SUM, it == 1).wait()
                torch.cuda.synchronize()
                assert torch.equal(t, torch.full((n,), float(tri), dtype=dtype, device=dev)), (dtype, n, it)
            comm.symm_free(t)
    t = comm.symm_empty((200_000,), torch.float32)
    t.copy_(ones(200_000))
    comm.all_reduce(t, tc.ReduceOp.AVG, False)
    torch.cuda.synchronize()
    torch.testing.assert_close(t, torch.full((200_000,), tri / world, device=dev))
    comm.symm_free(t)
    # plain tensors: latency class on the flag-less kernel, back to back, changing sizes
    for it in range(20):
        n = (1, 300, 8192, 32_000)[it % 4]
        p = ones(n, torch.bfloat16)
        comm.all_reduce(p, tc.ReduceOp.SUM, False)
        assert torch.equal(p.float(), torch.full((n,), float(tri), device=dev)), it
    if world > 1:
        assert count("all_reduce/symm") >= 7 and count("all_reduce/lamport") >= 20

    # ---- all-to-all family into a symmetric output
    for n in (4096, 300_000):   # flag-less exchange, then the one-pass push
        src = torch.cat([torch.full((n,), float(rank * world + d), device=dev) for d in range(world)])
        dst = comm.symm_empty((world * n,), torch.float32)
        comm.all_to_all_single(dst, src, False)
        torch.cuda.synchronize()
        assert torch.equal(dst, torch.cat([torch.full((n,), float(s * world + rank), device=dev) for s in range(world)]))
        comm.symm_free(dst)
    in_splits = [d + 1 for d in range(world)]
    out_splits = [rank + 1] * world
    src = torch.cat([torch.full((d + 1, 3), float(rank * 10 + d), device=dev) for d in range(world)])
    want = torch.cat([torch.full((rank + 1, 3), float(s * 10 + rank), device=dev) for s in range(world)])
    # a small symmetric receive buffer: the flag-less exchange (12-byte rows: parts are not whole 16-byte vectors)
    dst = comm.symm_empty((world * world, 3), torch.float32)  # same size everywhere, used up to sum(out_splits)
    for it in range(3):
        dst.zero_()
        comm.all_to_all_v_single(dst[: sum(out_splits)], src, out_splits, in_splits, it == 1).wait()
        torch.cuda.synchronize()
        assert torch.equal(dst[: sum(out_splits)], want), it
    comm.symm_free(dst)
    # ordinary tensors with a bound on the parts given by the caller: the flag-less exchange as well
    plain = torch.zeros(sum(out_splits), 3, device=dev)
    comm.all_to_all_v_single(plain, src, out_splits, in_splits, False, hints={"max_part_bytes": "4096"})
    torch.cuda.synchronize()
    assert torch.equal(plain, want)
    # a large one: the one-pass push, with host splits and with splits that live on the device
    dst = comm.symm_empty((400_000 + world * world, 3), torch.float32)
    dst.zero_()
    comm.all_to_all_v_single(dst[: sum(out_splits)], src, out_splits, in_splits, True).wait()
    torch.cuda.synchronize()
    assert torch.equal(dst[: sum(out_splits)], want)
    dst.zero_()
    impl.device_alltoallv_single(dst, src, torch.tensor(out_splits, device=dev), torch.tensor(in_splits, device=dev), False)
    torch.cuda.synchronize()
    assert torch.equal(dst[: sum(out_splits)], want)
    comm.symm_free(dst)
    if world > 1:
        assert count("all_to_all_single/symm") >= 1 and count("all_to_all_single/lamport") >= 1
        assert count("all_to_all_v_single/lamport") >= 4 and count("all_to_all_v_single/symm") >= 1
        assert count("device_alltoallv/symm") >= 1

    # ---- operations of different channels in flight together
    big = 8_000_000
    ag_out = comm.symm_empty((world * big,), torch.bfloat16)
    rs_in = comm.symm_empty((world * big,), torch.bfloat16)
    rs_in.copy_(ones(world * big, torch.bfloat16))
    rs_out = torch.empty(big, device=dev)
    ar = comm.symm_empty((big,), torch.float32)
    ar.copy_(ones(big))
    torch.cuda.synchronize()
    w1 = comm.all_gather_single(ag_out, ones(big, torch.bfloat16), True)
    w2 = comm.reduce_scatter_single(rs_out, rs_in, tc.ReduceOp.SUM, True)
    w3 = comm.all_reduce(ar, tc.ReduceOp.SUM, True)
    for w in (w1, w2, w3):
        w.wait()
    torch.cuda.synchronize()
    assert torch.equal(ag_out.float(), torch.arange(1, world + 1, device=dev).repeat_interleave(big).float())
    assert torch.equal(rs_out, torch.full((big,), float(tri), device=dev))
    assert torch.equal(ar, torch.full((big,), float(tri), device=dev))
    if world > 1:
        streams = {impl.channel_stream(c) for c in range(4)}
        assert len(streams) == 4  # each channel has a stream of its own
    for t in (ag_out, rs_in, ar):
        comm.symm_free(t)

    # ---- CUDA graph: symmetric all-reduce + flag-less all-reduce captured together, replayed,
    #      and the bookkeeping released once the graph is gone
    static = comm.symm_empty((50_000,), torch.float32)
    small = ones(512)
    graph = torch.cuda.CUDAGraph()
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        with torch.cuda.graph(graph, stream=side):
            comm.all_reduce(static, tc.ReduceOp.SUM, False)
            w = comm.all_reduce(small, tc.ReduceOp.SUM, True)
            w.wait()
    for i in range(4):
        static.fill_(rank + 1)
        small.fill_(rank + 1)
        graph.replay()
        torch.cuda.synchronize()
        assert torch.equal(static, torch.full((50_000,), float(tri), device=dev)), i
        assert torch.equal(small, torch.full((512,), float(tri), device=dev)), i
    assert int(impl.comm_dump()["graph_entries"]) == 2
    del graph
    deadline = time.time() + 10
    while int(impl.comm_dump()["graph_entries"]) != 0 and time.time() < deadline:
        time.sleep(0.05)
    assert int(impl.comm_dump()["graph_entries"]) == 0, "entries of a destroyed graph must be released"
    comm.symm_free(static)

    # ---- allocator memory: registered once, then zero-copy for every tensor inside it
    buf = symmetric_empty(comm, (world * 1_048_576,), torch.bfloat16)
    assert not is_symmetric(comm, buf)
    comm.tensor_register(buf)
    assert is_symmetric(comm, buf)
    before = count("all_gather/symm")
    comm.all_gather_single(buf, ones(1_048_576, torch.bfloat16), False)
    torch.cuda.synchronize()
    assert torch.equal(buf.float(), torch.arange(1, world + 1, device=dev).repeat_interleave(1_048_576).float())
    if world > 1:
        assert count("all_gather/symm") == before + 1
    comm.tensor_deregister(buf)
    assert not is_symmetric(comm, buf)

    torch.cuda.synchronize()
    comm.finalize()


def _world_size():
    return max(1, min(torch.cuda.device_count(), int(os.environ.get("B200COMMS_TEST_WORLD", "2"))))


def test_symmetric_collectives():
    run_ranks(_symm_battery, _world_size(), timeout=300)


def test_symmetric_collectives_without_multicast():
    if _world_size() < 2:
        pytest.skip("needs 2 GPUs")
    run_ranks(_symm_battery, 2, timeout=300, extra_env={"B200COMMS_NVLS": "0", "NCCL_NVLS_ENABLE": "0"})


def _ulysses_worker(rank, world):
    """Fused sequence <-> heads exchange against the all-to-all with explicit permutes: values, the attention built
    on it, gradients, reuse of the buffer ring, the route counter."""
    import torchcomms_b200 as tc
    from torchcomms_b200.parallel.context import SeqHeadsExchange, _heads_to_seq, _seq_to_heads, ulysses_attention

    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    comm = tc.new_comm("b200", dev, name="uly", timeout=timedelta(seconds=60), abort_process_on_timeout_or_error=False)
    impl = comm.get_backend_impl()
    ex = SeqHeadsExchange(comm, slots=3)
    assert ex.fused == (world > 1)
    b, h, s, d = 2, 4 * world, 96, 64
    g = torch.Generator(device=dev).manual_seed(100 + rank)
    for dtype in (torch.bfloat16, torch.float32):
        x = torch.randn(b, h, s, d, device=dev, generator=g).to(dtype)
        ref = _seq_to_heads(x, comm)
        got = ex.to_heads(x)
        assert got.shape == ref.shape and torch.equal(got, ref)
        assert torch.equal(ex.to_seq(got), x) and torch.equal(_heads_to_seq(ref, comm), x)
    if world > 1:
        assert int(impl.comm_dump().get("count/seq_heads_exchange/symm", "0")) == 4
    # the ring: a result stays valid for `slots` - 1 further exchanges of its shape, keep=True copies it out
    first = ex.to_heads(x)
    kept = ex.to_heads(x * 2, keep=True)
    for i in range(3):
        ex.to_heads(x * (3 + i))
    assert torch.equal(kept, _seq_to_heads(x * 2, comm))
    if world > 1:
        assert not torch.equal(first, _seq_to_heads(x, comm))          # overwritten by the fourth call after it

    # attention and its gradients
    q, k, v = (torch.randn(b, h, s, d, device=dev, generator=g, dtype=torch.float32, requires_grad=True) for _ in range(3))
    o_ref = ulysses_attention(q, k, v, comm, causal=True)
    gr = torch.autograd.grad(o_ref.square().sum(), (q, k, v))
    o = ulysses_attention(q, k, v, comm, causal=True, exchange=ex)
    gf = torch.autograd.grad(o.square().sum(), (q, k, v))
    assert torch.allclose(o, o_ref, atol=1e-5, rtol=1e-5)
    for a, r in zip(gf, gr):
        assert torch.allclose(a, r, atol=1e-4, rtol=1e-4)
    torch.cuda.synchronize()
    ex.close()
    comm.finalize()


def test_fused_sequence_heads_exchange_and_ulysses_attention():
    run_ranks(_ulysses_worker, _world_size(), timeout=300)
