"""Autograd wrappers around the fused sm_100a model kernels.

CUDA tensors always take the hand-written kernels (``_comms.ops``); there is no
silent eager fallback on a GPU.  CPU tensors take a plain PyTorch restatement
of the same math so that the training engine can be exercised with the gloo
backend on machines without a GPU.
"""
from __future__ import annotations

import torch
import torch.nn.functional as F

from .. import _comms

_k = _comms.ops

__all__ = [
    "rms_norm",
    "swiglu",
    "apply_rope",
    "rope_tables",
    "linear_cross_entropy",
    "adamw_step_",
    "kernel_launch_count",
]


def kernel_launch_count() -> int:
    """Kernels launched by this library since process start."""
    return int(_k.kernel_launch_count())


# ------------------------------------------------------------------ RMSNorm


class _RmsNorm(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, w, eps):
        y, rstd = _k.rmsnorm_fwd(x, w, eps)
        ctx.save_for_backward(x, w, rstd)
        return y

    @staticmethod
    def backward(ctx, dy):
        x, w, rstd = ctx.saved_tensors
        dx, dw = _k.rmsnorm_bwd(dy.contiguous(), x, w, rstd)
        return dx, dw, None


def rms_norm(x: torch.Tensor, w: torch.Tensor, eps: float = 1e-5) -> torch.Tensor:
    if x.is_cuda:
        return _RmsNorm.apply(x.contiguous(), w, eps)
    xf = x.float()
    y = xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps) * w.float()
    return y.to(x.dtype)


# ------------------------------------------------------------------- SwiGLU


class _SwiGlu(torch.autograd.Function):
    @staticmethod
    def forward(ctx, gate_up):
        ctx.save_for_backward(gate_up)
        return _k.swiglu_fwd(gate_up)

    @staticmethod
    def backward(ctx, dh):
        (gate_up,) = ctx.saved_tensors
        return _k.swiglu_bwd(dh.contiguous(), gate_up)


def swiglu(gate_up: torch.Tensor) -> torch.Tensor:
    """``silu(gate) * up`` for ``gate_up = [..., 2*ffn]`` (gate first)."""
    if gate_up.is_cuda:
        return _SwiGlu.apply(gate_up.contiguous())
    gate, up = gate_up.float().chunk(2, dim=-1)
    return (F.silu(gate) * up).to(gate_up.dtype)


# --------------------------------------------------------------------- RoPE


def rope_tables(max_pos: int, head_dim: int, theta: float, device) -> tuple[torch.Tensor, torch.Tensor]:
    inv = 1.0 / (theta ** (torch.arange(0, head_dim, 2, dtype=torch.float32) / head_dim))
    ang = torch.outer(torch.arange(max_pos, dtype=torch.float32), inv)
    return ang.cos().to(device).contiguous(), ang.sin().to(device).contiguous()


class _Rope(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, pos, cos_t, sin_t):
        ctx.save_for_backward(pos, cos_t, sin_t)
        return _k.rope_(x.clone(memory_format=torch.contiguous_format), pos, cos_t, sin_t, False)

    @staticmethod
    def backward(ctx, dy):
        pos, cos_t, sin_t = ctx.saved_tensors
        return _k.rope_(dy.clone(memory_format=torch.contiguous_format), pos, cos_t, sin_t, True), None, None, None


def apply_rope(x: torch.Tensor, pos: torch.Tensor, cos_t: torch.Tensor, sin_t: torch.Tensor) -> torch.Tensor:
    """Rotates interleaved pairs of ``x = [tokens, heads, head_dim]`` by the angle of ``pos[token]``."""
    if x.is_cuda:
        return _Rope.apply(x, pos, cos_t, sin_t)
    xf = x.float().reshape(*x.shape[:-1], -1, 2)
    c = cos_t[pos.long()].unsqueeze(-2)  # [tokens, 1, hd/2]
    s = sin_t[pos.long()].unsqueeze(-2)
    a, b = xf[..., 0], xf[..., 1]
    out = torch.stack((a * c - b * s, a * s + b * c), dim=-1)
    return out.reshape(x.shape).to(x.dtype)


# ------------------------------------------------- linear + cross entropy


class _LinearCrossEntropy(torch.autograd.Function):
    """``mean(cross_entropy(x @ W^T, targets))`` without keeping the logits.

    Rows are processed in chunks: one GEMM makes a chunk of logits, a kernel
    turns it in place into its own gradient while emitting the per-row loss,
    and two more GEMMs fold that gradient into ``dx`` and ``dW``.  The
    gradients are therefore ready when forward returns; backward only scales
    them by the incoming gradient of the loss.
    """

    @staticmethod
    def forward(ctx, x, weight, targets, chunk_rows):
        rows = x.shape[0]
        # Mean over all rows; rows with a negative target contribute zero.
        scale = 1.0 / max(rows, 1)
        dx = torch.empty_like(x)
        dw = torch.zeros_like(weight)
        loss_sum = torch.zeros((), dtype=torch.float32, device=x.device)
        for r0 in range(0, rows, chunk_rows):
            r1 = min(rows, r0 + chunk_rows)
            logits = x[r0:r1] @ weight.t()
            if x.is_cuda:
                loss = _k.cross_entropy_fwd_bwd_(logits, targets[r0:r1].contiguous(), scale)
                dlogits = logits
            else:
                lf = logits.float()
                loss = F.cross_entropy(lf, targets[r0:r1], reduction="none", ignore_index=-1)
                p = torch.softmax(lf, dim=-1)
                onehot = F.one_hot(targets[r0:r1].clamp_min(0), lf.shape[-1]).float()
                dlogits = ((p - onehot) * (targets[r0:r1] >= 0).unsqueeze(-1) * scale).to(x.dtype)
            loss_sum += loss.sum()
            dx[r0:r1] = dlogits @ weight
            dw.addmm_(dlogits.t(), x[r0:r1])
        ctx.save_for_backward(dx, dw)
        return loss_sum * scale

    @staticmethod
    def backward(ctx, dloss):
        dx, dw = ctx.saved_tensors
        return dx * dloss.to(dx.dtype), dw * dloss.to(dw.dtype), None, None


def linear_cross_entropy(x: torch.Tensor, weight: torch.Tensor, targets: torch.Tensor, chunk_rows: int = 4096) -> torch.Tensor:
    """Mean token cross-entropy of the logits ``x @ weight.T`` (``x``: [rows, dim])."""
    return _LinearCrossEntropy.apply(x.contiguous(), weight, targets, chunk_rows)


# -------------------------------------------------------------------- AdamW


def adamw_step_(p, g, m, v, *, lr, beta1=0.9, beta2=0.95, eps=1e-8, weight_decay=0.0, step=1, grad_scale=1.0) -> None:
    """In-place AdamW on flat fp32 tensors (bias-corrected, decoupled weight decay)."""
    if p.is_cuda:
        _k.adamw_step_(p, g, m, v, lr, beta1, beta2, eps, weight_decay, step, grad_scale)
        return
    gr = g * grad_scale
    m.mul_(beta1).add_(gr, alpha=1 - beta1)
    v.mul_(beta2).addcmul_(gr, gr, value=1 - beta2)
    mhat = m / (1 - beta1**step)
    vhat = v / (1 - beta2**step)
    p.mul_(1 - lr * weight_decay).addcdiv_(mhat, vhat.sqrt() + eps, value=-lr)
