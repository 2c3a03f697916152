// Memory-bound model kernels used by the flagship training step (Llama-style
// decoder): RMSNorm, rotary embedding, SwiGLU, softmax cross-entropy fused
// with its gradient, and AdamW on flat fp32 shards. bf16 activations, fp32
// statistics and accumulation. Raw-pointer launch interface.
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace b200c {

// y = x * rsqrt(mean(x^2) + eps) * w ; rstd saved for the backward pass.
// cols must be a multiple of 8.
cudaError_t launch_rmsnorm_fwd(const __nv_bfloat16* x, const __nv_bfloat16* w, __nv_bfloat16* y, float* rstd,
                               int rows, int cols, float eps, cudaStream_t s);
// dx, and per-block partial weight gradients `dw_partial` [nblocks, cols]
// (fp32), which `launch_colsum` folds into dw. Returns the number of blocks
// it will use through *nblocks when dw_partial is null (sizing query).
cudaError_t launch_rmsnorm_bwd(const __nv_bfloat16* dy, const __nv_bfloat16* x, const __nv_bfloat16* w,
                               const float* rstd, __nv_bfloat16* dx, float* dw_partial, int* nblocks, int rows,
                               int cols, cudaStream_t s);
// out[c] = sum_r in[r, c]  (fp32 in, bf16 or fp32 out)
cudaError_t launch_colsum_bf16(const float* in, __nv_bfloat16* out, int rows, int cols, cudaStream_t s);

// out[i] = convert(in[i] * scale) for n elements; `in_kind` / `out_kind`: 0 = fp32, 1 = bf16.
// What a collective degenerates to on a single rank (cast, scale, copy) in one pass.
cudaError_t launch_cast_scale(const void* in, int in_kind, void* out, int out_kind, size_t n, float scale, cudaStream_t s);

// Rotary embedding in place on [tokens, heads, head_dim] with interleaved
// pairs; pos[t] indexes the cos/sin tables [max_pos, head_dim/2]. `inverse`
// rotates by the negative angle (the backward pass).
cudaError_t launch_rope(__nv_bfloat16* x, const int* pos, const float* cos_t, const float* sin_t, int tokens,
                        int heads, int head_dim, bool inverse, cudaStream_t s);

// h = silu(gate) * up where gate_up = [rows, 2*ffn] (gate first).
cudaError_t launch_swiglu_fwd(const __nv_bfloat16* gate_up, __nv_bfloat16* h, int rows, int ffn, cudaStream_t s);
cudaError_t launch_swiglu_bwd(const __nv_bfloat16* dh, const __nv_bfloat16* gate_up, __nv_bfloat16* dgate_up,
                              int rows, int ffn, cudaStream_t s);

// Row-wise softmax cross-entropy: writes loss[r] and overwrites logits with
// d(loss_sum * grad_scale)/dlogits. Rows whose target is < 0 are ignored.
cudaError_t launch_cross_entropy_fwd_bwd(__nv_bfloat16* logits, const int64_t* targets, float* loss, int rows,
                                         int vocab, float grad_scale, cudaStream_t s);

// AdamW on flat fp32 tensors. `grad_scale` multiplies the gradient first
// (loss scaling / averaging); `step` starts at 1.
cudaError_t launch_adamw(float* p, const float* g, float* m, float* v, size_t n, float lr, float beta1, float beta2,
                         float eps, float weight_decay, int step, float grad_scale, cudaStream_t s);

// Count of launches made through this header since process start (the
// benchmark reports it).
unsigned long long fused_ops_launch_count();

} // namespace b200c
