"""Fused tensor-parallel layers (all-gather -> GEMM, GEMM -> reduce-scatter):
single-rank numerics on one GPU, then the real multi-process path, both
against an fp32 PyTorch reference."""
import os
from datetime import timedelta

import pytest
import torch

from tests.mp_util import run_ranks

pytestmark = pytest.mark.gpu


def _rand(shape, seed, dev="cuda", scale=1.0):
    g = torch.Generator(device=dev).manual_seed(seed)
    return (torch.randn(*shape, generator=g, device=dev) * scale).to(torch.bfloat16)


@pytest.mark.parametrize("m,n,k", [(128, 256, 64), (512, 512, 1024), (1024, 1792, 2048), (128 * 37, 256 * 5, 512)])
def test_ag_gemm_single_rank(m, n, k):
    from torchcomms_b200.ops.tp import AllGatherGemm

    layer = AllGatherGemm(None, m, k)
    for it in range(3):  # repeated calls exercise the device-side epoch
        x, w = _rand((m, k), 10 + it), _rand((n, k), 20 + it, scale=0.05)
        y = layer(w, x)
        torch.cuda.synchronize()
        assert layer.status()[0] == 0
        ref = x.float() @ w.float().t()
        torch.testing.assert_close(y.float(), ref, rtol=2e-2, atol=2e-2)


@pytest.mark.parametrize("m,n,k", [(128, 256, 64), (512, 512, 1024), (2048, 1024, 1536)])
def test_gemm_rs_single_rank(m, n, k):
    from torchcomms_b200.ops.tp import GemmReduceScatter

    layer = GemmReduceScatter(None, m, n)
    for it in range(3):
        h, w = _rand((m, k), 30 + it), _rand((n, k), 40 + it, scale=0.05)
        out = layer(h, w)
        torch.cuda.synchronize()
        assert layer.status()[0] == 0
        ref = h.float() @ w.float().t()
        torch.testing.assert_close(out.float(), ref, rtol=2e-2, atol=2e-2)


@pytest.mark.parametrize("nranks,m_local,n,k", [(2, 128, 256, 64), (2, 256, 512, 1024), (4, 128, 768, 512), (4, 384, 256, 2048)])
def test_ag_gemm_emulated_ranks(nranks, m_local, n, k):
    """The fused all-gather -> GEMM protocol (copy warps, arrival counters, opening and closing barrier) with
    2 and 4 ranks on one GPU, every rank on its share of the SMs, against fp32 PyTorch."""
    from torchcomms_b200 import _comms

    world = _comms.TpEmuWorld(nranks, "ag_gemm", m_local, k, 5000.0)
    for it in range(3):
        xs = [_rand((m_local, k), 100 * it + r) for r in range(nranks)]
        ws = [_rand((n, k), 100 * it + 50 + r, scale=0.05) for r in range(nranks)]
        for r in range(nranks):
            world.input(r).copy_(xs[r])
        ys = world.ag_gemm(ws)
        torch.cuda.synchronize()
        assert world.status()[0] == 0, world.status()
        full = torch.cat(xs).float()
        for r in range(nranks):
            torch.testing.assert_close(ys[r].float(), full @ ws[r].float().t(), rtol=2e-2, atol=2e-2)


@pytest.mark.parametrize("nranks,m,n,k_local", [(2, 256, 256, 64), (2, 512, 512, 1024), (4, 512, 768, 512), (4, 1536, 256, 1024)])
def test_gemm_rs_emulated_ranks(nranks, m, n, k_local):
    """The fused GEMM -> reduce-scatter protocol (partial tiles stored into the owner's staging, per-tile flags, the
    owner's sum) with 2 and 4 ranks on one GPU, against fp32 PyTorch."""
    from torchcomms_b200 import _comms

    world = _comms.TpEmuWorld(nranks, "gemm_rs", m, n, 5000.0)
    for it in range(3):
        hs = [_rand((m, k_local), 200 * it + r) for r in range(nranks)]
        ws = [_rand((n, k_local), 200 * it + 50 + r, scale=0.05) for r in range(nranks)]
        outs = world.gemm_rs(hs, ws)
        torch.cuda.synchronize()
        assert world.status()[0] == 0, world.status()
        total = sum(h.float() @ w.float().t() for h, w in zip(hs, ws))
        rows = m // nranks
        for r in range(nranks):
            torch.testing.assert_close(outs[r].float(), total[r * rows : (r + 1) * rows], rtol=2e-2, atol=3e-2)


def _fp8_ref(q_a, s_a, q_b, s_b):
    """fp32 reference of the fp8 product computed from the SAME quantised operands."""
    return (q_a.float() * s_a.unsqueeze(1)) @ (q_b.float() * s_b.unsqueeze(1)).t()


@pytest.mark.parametrize("m,n,k", [(128, 256, 128), (300, 264, 256), (1024, 1792, 2048), (128 * 9, 256 * 5, 1024)])
def test_gemm_e4m3_rowwise_scales(m, n, k):
    from torchcomms_b200.ops.tp import gemm_e4m3_nt, quantize_rows

    a, b = _rand((m, k), 1), _rand((n, k), 2, scale=0.05)
    (qa, sa), (qb, sb) = quantize_rows(a), quantize_rows(b)
    c = gemm_e4m3_nt(qa, qb, sa, sb)
    torch.cuda.synchronize()
    ref = _fp8_ref(qa, sa, qb, sb)
    # the kernel multiplies exact e4m3 products in fp32: only the bf16 rounding of the result separates the two
    torch.testing.assert_close(c.float(), ref, rtol=1e-2, atol=1e-2)
    # and the quantisation itself stays within fp8's precision of the bf16 product
    full = a.float() @ b.float().t()
    assert float((c.float() - full).norm() / full.norm()) < 0.06


@pytest.mark.parametrize("nranks", [1, 2, 4])
def test_fp8_fused_layers_emulated_ranks(nranks):
    """e4m3 all-gather -> GEMM (row scales travel with the rows) and GEMM -> reduce-scatter on 1, 2 and 4 ranks."""
    from torchcomms_b200 import _comms
    from torchcomms_b200.ops.tp import quantize_rows

    m_local, n, k = 256, 512, 1024
    world = _comms.TpEmuWorld(nranks, "ag_gemm", m_local, k, 5000.0, True)
    for it in range(2):
        xs = [quantize_rows(_rand((m_local, k), 300 * it + r)) for r in range(nranks)]
        ws = [quantize_rows(_rand((n, k), 300 * it + 50 + r, scale=0.05)) for r in range(nranks)]
        for r in range(nranks):
            world.input(r).copy_(xs[r][0])
            world.input_scales(r).copy_(xs[r][1])
        ys = world.ag_gemm([w for w, _ in ws], [s for _, s in ws])
        torch.cuda.synchronize()
        assert world.status()[0] == 0, world.status()
        qx, sx = torch.cat([q for q, _ in xs]), torch.cat([s for _, s in xs])
        for r in range(nranks):
            torch.testing.assert_close(ys[r].float(), _fp8_ref(qx, sx, ws[r][0], ws[r][1]), rtol=1e-2, atol=2e-2)
    m = 128 * nranks * 2
    world = _comms.TpEmuWorld(nranks, "gemm_rs", m, n, 5000.0, True)
    for it in range(2):
        hs = [quantize_rows(_rand((m, k), 400 * it + r)) for r in range(nranks)]
        ws = [quantize_rows(_rand((n, k), 400 * it + 50 + r, scale=0.05)) for r in range(nranks)]
        outs = world.gemm_rs([q for q, _ in hs], [q for q, _ in ws], [s for _, s in hs], [s for _, s in ws])
        torch.cuda.synchronize()
        assert world.status()[0] == 0, world.status()
        total = sum(_fp8_ref(h[0], h[1], w[0], w[1]) for h, w in zip(hs, ws))
        rows = m // nranks
        for r in range(nranks):
            torch.testing.assert_close(outs[r].float(), total[r * rows : (r + 1) * rows], rtol=2e-2, atol=4e-2)


def test_fp8_layers_single_rank_api():
    from torchcomms_b200.ops.tp import AllGatherGemm, GemmReduceScatter, quantize_rows

    m, n, k = 512, 768, 1024   # m % 256 == 0: the CTA-pair kernels
    x, w = _rand((m, k), 5), _rand((n, k), 6, scale=0.05)
    qw, sw = quantize_rows(w)
    qx, sx = quantize_rows(x)
    up = AllGatherGemm(None, m, k, fp8=True)
    y = up(qw, x, scale_w=sw)                    # bf16 activations are quantised on the way in
    down = GemmReduceScatter(None, m, n, fp8=True)
    out = down(qx, qw, sx, sw)
    torch.cuda.synchronize()
    assert up.status()[0] == 0 and down.status()[0] == 0
    ref = _fp8_ref(qx, sx, qw, sw)
    torch.testing.assert_close(y.float(), ref, rtol=1e-2, atol=2e-2)
    torch.testing.assert_close(out.float(), ref, rtol=1e-2, atol=2e-2)


def _tp_worker(rank, world):
    import torchcomms_b200 as tc
    from torchcomms_b200.ops.tp import AllGatherGemm, GemmReduceScatter

    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    comm = tc.new_comm("b200", dev, name="tp", timeout=timedelta(seconds=60), abort_process_on_timeout_or_error=False)
    m_local, hidden, ffn_local = 256, 1024, 768
    m = m_local * world
    up = AllGatherGemm(comm, m_local, hidden)
    down = GemmReduceScatter(comm, m, hidden)
    for it in range(4):
        # every rank can rebuild every other rank's inputs from the seeds
        xs = [_rand((m_local, hidden), 1000 * it + r, dev) for r in range(world)]
        w_up = _rand((ffn_local, hidden), 5000 + 10 * it + rank, dev, 0.05)
        y = up(w_up, xs[rank])
        hs = [_rand((m, ffn_local), 7000 + 10 * it + r, dev) for r in range(world)]
        w_downs = [_rand((hidden, ffn_local), 9000 + 10 * it + r, dev, 0.05) for r in range(world)]
        out = down(hs[rank], w_downs[rank])
        torch.cuda.synchronize()
        ref_y = torch.cat(xs).float() @ w_up.float().t()
        torch.testing.assert_close(y.float(), ref_y, rtol=2e-2, atol=2e-2)
        # the wire carries bf16 partial sums, so compare against the same rounding
        ref_out = sum((hs[r].float() @ w_downs[r].float().t()).to(torch.bfloat16).float() for r in range(world))
        ref_out = ref_out[rank * m_local : (rank + 1) * m_local]
        torch.testing.assert_close(out.float(), ref_out, rtol=2e-2, atol=6e-2)
    comm.finalize()


def test_tp_layers_multi_gpu():
    world = min(torch.cuda.device_count(), int(os.environ.get("B200COMMS_TEST_WORLD", "2")))
    if world < 2:
        pytest.skip("needs 2 GPUs")
    run_ranks(_tp_worker, world, timeout=150)


def test_tensor_parallel_mlp_fused_bf16_and_fp8_single_rank():
    """``TensorParallelMLP.forward_fused`` on one rank: the bf16 path matches the differentiable path, the fp8 path
    stays within fp8's precision of it."""
    import torchcomms_b200 as tc
    from torchcomms_b200.parallel.tensor import TensorParallelMLP

    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    os.environ.setdefault("MASTER_PORT", "29643")
    os.environ["RANK"], os.environ["WORLD_SIZE"] = "0", "1"
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(0)
    comm = tc.new_comm("b200", dev, name="tpmlp", abort_process_on_timeout_or_error=False)
    mlp = TensorParallelMLP(1024, 1536, comm, device=dev, dtype=torch.bfloat16)
    x = _rand((256, 1024), 77)
    with torch.no_grad():
        ref = mlp(x).float()
    y = mlp.forward_fused(x).float()
    y8 = mlp.forward_fused(x, fp8=True).float()
    torch.cuda.synchronize()
    assert float((y - ref).norm() / ref.norm()) < 0.02
    assert float((y8 - ref).norm() / ref.norm()) < 0.08
    comm.finalize()
