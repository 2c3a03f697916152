"""Numerics of the fused model kernels against plain PyTorch fp32 references,
and the training engine on one GPU."""
import os

import pytest
import torch
import torch.nn.functional as F

pytestmark = pytest.mark.gpu


def _bf(*shape, seed=0, scale=1.0):
    g = torch.Generator(device="cuda").manual_seed(seed)
    return (torch.randn(*shape, generator=g, device="cuda") * scale).to(torch.bfloat16)


@pytest.mark.parametrize("rows,cols", [(5, 64), (300, 4096), (17, 8192), (4, 16384)])
def test_rmsnorm_forward_backward(rows, cols):
    from torchcomms_b200.ops import fused

    x = _bf(rows, cols, seed=1).requires_grad_(True)
    w = (_bf(cols, seed=2, scale=0.1) + 1).detach().requires_grad_(True)
    y = fused.rms_norm(x, w, 1e-5)
    xf, wf = x.detach().float().requires_grad_(True), w.detach().float().requires_grad_(True)
    ref = xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + 1e-5) * wf
    torch.testing.assert_close(y.float(), ref, rtol=2e-2, atol=2e-2)
    if cols <= 8192:
        dy = _bf(rows, cols, seed=3)
        y.backward(dy)
        ref.backward(dy.float())
        torch.testing.assert_close(x.grad.float(), xf.grad, rtol=3e-2, atol=3e-2)
        torch.testing.assert_close(w.grad.float(), wf.grad, rtol=3e-2, atol=3e-2 * max(1.0, rows ** 0.5))


def test_swiglu_forward_backward():
    from torchcomms_b200.ops import fused

    gu = _bf(33, 2 * 1024, seed=4).requires_grad_(True)
    h = fused.swiglu(gu)
    guf = gu.detach().float().requires_grad_(True)
    g, u = guf.chunk(2, dim=-1)
    ref = F.silu(g) * u
    torch.testing.assert_close(h.float(), ref, rtol=2e-2, atol=2e-2)
    dh = _bf(33, 1024, seed=5)
    h.backward(dh)
    ref.backward(dh.float())
    torch.testing.assert_close(gu.grad.float(), guf.grad, rtol=3e-2, atol=3e-2)


def test_rope_matches_complex_rotation_and_inverts():
    from torchcomms_b200.ops import fused

    tokens, heads, hd = 50, 4, 128
    cos_t, sin_t = fused.rope_tables(64, hd, 500000.0, "cuda")
    pos = torch.arange(tokens, dtype=torch.int32, device="cuda") % 64
    x = _bf(tokens, heads, hd, seed=6).requires_grad_(True)
    y = fused.apply_rope(x, pos, cos_t, sin_t)
    xc = torch.view_as_complex(x.detach().float().reshape(tokens, heads, hd // 2, 2))
    rot = torch.polar(torch.ones_like(cos_t), torch.atan2(sin_t, cos_t))[pos.long()].unsqueeze(1)
    ref = torch.view_as_real(xc * rot).reshape(tokens, heads, hd)
    torch.testing.assert_close(y.float(), ref, rtol=2e-2, atol=2e-2)
    # the backward is the inverse rotation: rotating the output gradient back
    y.backward(y.detach())
    torch.testing.assert_close(x.grad.float(), x.detach().float(), rtol=3e-2, atol=3e-2)


@pytest.mark.parametrize("rows,vocab", [(7, 1000), (64, 32003), (9, 128256)])
def test_cross_entropy_loss_and_gradient(rows, vocab):
    from torchcomms_b200 import _comms

    logits = _bf(rows, vocab, seed=7, scale=2.0)
    targets = torch.randint(0, vocab, (rows,), device="cuda")
    targets[0] = -1  # ignored row
    lf = logits.float().requires_grad_(True)
    ref = F.cross_entropy(lf, targets, reduction="none", ignore_index=-1)
    (ref.sum() * 0.25).backward()
    work = logits.clone()
    loss = _comms.ops.cross_entropy_fwd_bwd_(work, targets, 0.25)
    torch.testing.assert_close(loss, ref.detach(), rtol=2e-2, atol=2e-2)
    torch.testing.assert_close(work.float(), lf.grad, rtol=3e-2, atol=2e-3)


def test_linear_cross_entropy_matches_unfused():
    from torchcomms_b200.ops import fused

    rows, dim, vocab = 300, 256, 5000
    x = _bf(rows, dim, seed=8).requires_grad_(True)
    w = _bf(vocab, dim, seed=9, scale=0.05).requires_grad_(True)
    t = torch.randint(0, vocab, (rows,), device="cuda")
    loss = fused.linear_cross_entropy(x, w, t, chunk_rows=128)
    loss.backward()
    xf, wf = x.detach().float().requires_grad_(True), w.detach().float().requires_grad_(True)
    ref = F.cross_entropy(xf @ wf.t(), t)
    ref.backward()
    torch.testing.assert_close(loss, ref.detach(), rtol=2e-2, atol=2e-2)
    torch.testing.assert_close(x.grad.float(), xf.grad, rtol=5e-2, atol=2e-4)
    torch.testing.assert_close(w.grad.float(), wf.grad, rtol=5e-2, atol=2e-4)


def test_adamw_matches_torch():
    from torchcomms_b200.ops import fused

    n = 100_003
    p = torch.randn(n, device="cuda")
    g = torch.randn(n, device="cuda")
    ref_p = p.clone().requires_grad_(True)
    opt = torch.optim.AdamW([ref_p], lr=1e-2, betas=(0.9, 0.95), eps=1e-8, weight_decay=0.1)
    m, v = torch.zeros_like(p), torch.zeros_like(p)
    for step in range(1, 4):
        ref_p.grad = g.clone()
        opt.step()
        fused.adamw_step_(p, g, m, v, lr=1e-2, beta1=0.9, beta2=0.95, eps=1e-8, weight_decay=0.1, step=step)
    torch.testing.assert_close(p, ref_p.detach(), rtol=1e-4, atol=1e-5)


def test_engine_step_on_gpu_matches_reference_forward():
    os.environ.setdefault("RANK", "0")
    os.environ.setdefault("WORLD_SIZE", "1")
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    os.environ.setdefault("MASTER_PORT", "29541")
    import torchcomms_b200 as tc
    from torchcomms_b200.models.llama import LlamaConfig
    from torchcomms_b200.ops import fused
    from torchcomms_b200.parallel.engine import TrainEngine

    comm = tc.new_comm("b200", torch.device("cuda", 0), name="engine_gpu")
    cfg = LlamaConfig.tiny()
    engine = TrainEngine(cfg, comm, lr=3e-3, weight_decay=0.0, seed=1, recompute_blocks=1)
    before = fused.kernel_launch_count()
    tokens = torch.randint(0, cfg.vocab_size, (2, 129), device="cuda")
    losses = [float(engine.step(tokens[:, :-1].contiguous(), tokens[:, 1:].contiguous())) for _ in range(5)]
    torch.cuda.synchronize()
    assert abs(losses[0] - torch.log(torch.tensor(float(cfg.vocab_size))).item()) < 0.5, losses
    assert losses[-1] < losses[0] - 0.05, losses
    assert fused.kernel_launch_count() - before > 50  # norms, rope, swiglu, loss, adamw, gathers, reductions
    comm.finalize()
