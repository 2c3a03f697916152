"""Fused all-reduce + residual add + RMSNorm: virtual ranks emulated in one
cooperative launch on one GPU, and the single-rank layer, against an fp32
PyTorch reference of the same three steps."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _reference(xs, residual, weight, eps):
    total = torch.stack([x.float() for x in xs]).sum(0)
    if residual is not None:
        total = total + residual.float()
    stored = total.to(torch.bfloat16)
    t = stored.float()
    normed = t * torch.rsqrt(t.pow(2).mean(-1, keepdim=True) + eps) * weight.float()
    return stored, normed


@pytest.mark.parametrize("nranks,rows,hidden", [(2, 1, 1024), (2, 128, 4096), (4, 17, 4096), (8, 32, 8192), (8, 5, 2048)])
@pytest.mark.parametrize("with_residual", [True, False])
def test_emulated_ranks_match_reference(nranks, rows, hidden, with_residual):
    from torchcomms_b200 import _comms

    dev = torch.device("cuda", 0)
    torch.manual_seed(nranks * 1000 + rows)
    world = _comms._EmuWorld(nranks, 1 << 20, 2000.0)
    weight = (1.0 + 0.1 * torch.randn(hidden, device=dev)).to(torch.bfloat16)
    for call in range(3):                                    # three calls: both parity halves, then reuse
        xs = [torch.randn(rows, hidden, device=dev).to(torch.bfloat16) for _ in range(nranks)]
        res0 = torch.randn(rows, hidden, device=dev).to(torch.bfloat16) if with_residual else None
        residuals = [res0.clone() for _ in range(nranks)] if with_residual else []
        outs = [torch.zeros(rows, hidden, dtype=torch.bfloat16, device=dev) for _ in range(nranks)]
        world.all_reduce_rmsnorm(xs, residuals, weight, outs, 1e-5)
        torch.cuda.synchronize()
        assert world.status()[0] == 0, world.status()
        stored, normed = _reference(xs, res0, weight, 1e-5)
        for r in range(nranks):
            assert torch.equal(outs[r], outs[0])            # replicas are bit-identical
            torch.testing.assert_close(outs[r].float(), normed, atol=3e-2, rtol=2e-2)
            if with_residual:
                assert torch.equal(residuals[r], residuals[0])
                # fp32 sum rounded once to bf16: at most one bf16 ulp from the reference order of additions
                torch.testing.assert_close(residuals[r].float(), stored.float(), atol=2e-2, rtol=1e-2)


def test_single_rank_layer_and_unfused_fallback():
    from torchcomms_b200.ops.ar_norm import MAX_ROWS, AllReduceRMSNorm

    dev = torch.device("cuda", 0)
    torch.manual_seed(7)
    hidden = 4096
    fused = AllReduceRMSNorm(None, hidden, eps=1e-6)
    weight = (1.0 + 0.1 * torch.randn(hidden, device=dev)).to(torch.bfloat16)
    for rows in (1, 64, MAX_ROWS, MAX_ROWS + 40):            # the last one takes the two-kernel path
        x = torch.randn(rows, hidden, device=dev).to(torch.bfloat16)
        res = torch.randn(rows, hidden, device=dev).to(torch.bfloat16)
        res0 = res.clone()
        out = fused(x, weight, residual=res)
        torch.cuda.synchronize()
        stored, normed = _reference([x], res0, weight, 1e-6)
        torch.testing.assert_close(res.float(), stored.float(), atol=2e-2, rtol=1e-2)
        torch.testing.assert_close(out.float(), normed, atol=3e-2, rtol=2e-2)
        plain = fused(x, weight)
        _, normed_plain = _reference([x], None, weight, 1e-6)
        torch.testing.assert_close(plain.float(), normed_plain, atol=3e-2, rtol=2e-2)
    assert fused.status()[0] == 0


def _rand(shape, seed, dev, scale=1.0):
    g = torch.Generator(device="cpu").manual_seed(seed)
    return (torch.randn(shape, generator=g) * scale).to(torch.bfloat16).to(dev)


def _backend_worker(rank, world):
    import time
    from datetime import timedelta

    import torchcomms_b200 as tc
    from torchcomms_b200.ops.ar_norm import AllReduceRMSNorm

    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    comm = tc.new_comm("b200", dev, name="arnorm", timeout=timedelta(seconds=60), abort_process_on_timeout_or_error=False,
                       hints={"use_multicast": "0"})
    hidden = 4096
    fused = AllReduceRMSNorm(comm, hidden)
    weight = _rand((hidden,), 1, dev, 0.1) + 1
    for it, rows in enumerate((1, 16, 128, 16, 16)):
        xs = [_rand((rows, hidden), 100 * it + r, dev) for r in range(world)]     # every rank rebuilds all inputs
        res = _rand((rows, hidden), 100 * it + 50, dev)
        res0 = res.clone()
        out = fused(xs[rank], weight, residual=res)
        torch.cuda.synchronize()
        stored, normed = _reference(xs, res0, weight, 1e-5)
        torch.testing.assert_close(res.float(), stored.float(), atol=2e-2, rtol=1e-2)
        torch.testing.assert_close(out.float(), normed, atol=3e-2, rtol=2e-2)
    assert fused.status() == [] or fused.status()[0] == 0
    # timing of the decode shape against the two-step path (device events, max over a few calls)
    rows = 16
    x, res = _rand((rows, hidden), 7, dev), _rand((rows, hidden), 8, dev)

    def timed(fn, iters=50):
        for _ in range(5):
            fn()
        comm.barrier(False)
        torch.cuda.synchronize()
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record()
        for _ in range(iters):
            fn()
        e.record()
        e.synchronize()
        return s.elapsed_time(e) * 1000.0 / iters

    us_fused = timed(lambda: fused(x, weight, residual=res))
    us_plain = timed(lambda: fused._unfused(x, weight, res))
    if rank == 0:
        print(f"ar_norm {world} GPUs [{rows}, {hidden}]: fused {us_fused:.1f} us, all_reduce + add + rmsnorm {us_plain:.1f} us", flush=True)
    comm.finalize()


def test_backend_layer_multi_gpu():
    import os

    from tests.mp_util import run_ranks

    world = min(torch.cuda.device_count(), int(os.environ.get("B200COMMS_TEST_WORLD", "2")))
    if world < 2:
        pytest.skip("needs 2 GPUs")
    run_ranks(_backend_worker, world, timeout=150)
