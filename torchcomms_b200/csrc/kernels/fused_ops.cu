// Memory-bound model kernels (sm_100a): RMSNorm fwd/bwd, RoPE, SwiGLU
// fwd/bwd, fused softmax cross-entropy + gradient, AdamW.
//
// All of them stream their operands once with 16-byte accesses and keep
// statistics in fp32; grids are sized to the 148 SMs of a B200 (persistent
// row loops where a reduction over rows is needed).
#include "fused_ops.h"

#include <atomic>

#include "launch_count.h"

namespace b200c {

namespace {

std::atomic<unsigned long long> g_launches{0};

constexpr int kSms = 148;

__device__ __forceinline__ float2 bf2_to_f2(uint32_t v) {
  return make_float2(__uint_as_float(v << 16), __uint_as_float(v & 0xffff0000u));
}
__device__ __forceinline__ uint32_t f2_to_bf2(float a, float b) {
  __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
  return *reinterpret_cast<uint32_t*>(&h);
}
__device__ __forceinline__ void unpack8(uint4 v, float* f) {
  float2 a = bf2_to_f2(v.x), b = bf2_to_f2(v.y), c = bf2_to_f2(v.z), d = bf2_to_f2(v.w);
  f[0] = a.x; f[1] = a.y; f[2] = b.x; f[3] = b.y; f[4] = c.x; f[5] = c.y; f[6] = d.x; f[7] = d.y;
}
__device__ __forceinline__ uint4 pack8(const float* f) {
  return make_uint4(f2_to_bf2(f[0], f[1]), f2_to_bf2(f[2], f[3]), f2_to_bf2(f[4], f[5]), f2_to_bf2(f[6], f[7]));
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

// Block-wide sum; every thread gets the result. `scratch` holds 32 floats.
__device__ __forceinline__ float block_sum(float v, float* scratch) {
  const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
  v = warp_sum(v);
  __syncthreads();
  if (lane == 0) scratch[wid] = v;
  __syncthreads();
  const int nw = (blockDim.x + 31) >> 5;
  float t = lane < nw ? scratch[lane] : 0.0f;
  return warp_sum(t);
}
__device__ __forceinline__ float block_max(float v, float* scratch) {
  const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
  v = warp_max(v);
  __syncthreads();
  if (lane == 0) scratch[wid] = v;
  __syncthreads();
  const int nw = (blockDim.x + 31) >> 5;
  float t = lane < nw ? scratch[lane] : -INFINITY;
  return warp_max(t);
}

// ------------------------------------------------------------- RMSNorm ------

constexpr int kNormThreads = 256;
constexpr int kNormMaxVec = 4;  // cols <= 256 * 4 * 8 = 8192 stay in registers

__global__ void __launch_bounds__(kNormThreads) k_rmsnorm_fwd(const __nv_bfloat16* __restrict__ x,
                                                               const __nv_bfloat16* __restrict__ w,
                                                               __nv_bfloat16* __restrict__ y, float* __restrict__ rstd,
                                                               int rows, int cols, float eps) {
  __shared__ float scratch[32];
  const int nvec = cols / 8;
  for (int r = blockIdx.x; r < rows; r += gridDim.x) {
    const uint4* xr = reinterpret_cast<const uint4*>(x + static_cast<size_t>(r) * cols);
    uint4* yr = reinterpret_cast<uint4*>(y + static_cast<size_t>(r) * cols);
    // The first kNormMaxVec vectors of each thread stay in registers between
    // the two passes; wider rows re-read the remainder (L2 hit).
    uint4 keep[kNormMaxVec];
    float ss = 0.0f;
#pragma unroll
    for (int k = 0; k < kNormMaxVec; ++k) {
      const int v = threadIdx.x + k * kNormThreads;
      if (v < nvec) {
        keep[k] = xr[v];
        float f[8];
        unpack8(keep[k], f);
#pragma unroll
        for (int i = 0; i < 8; ++i) ss += f[i] * f[i];
      }
    }
    for (int v = threadIdx.x + kNormMaxVec * kNormThreads; v < nvec; v += kNormThreads) {
      float f[8];
      unpack8(xr[v], f);
#pragma unroll
      for (int i = 0; i < 8; ++i) ss += f[i] * f[i];
    }
    ss = block_sum(ss, scratch);
    const float rs = rsqrtf(ss / static_cast<float>(cols) + eps);
    if (threadIdx.x == 0) rstd[r] = rs;
#pragma unroll
    for (int k = 0; k < kNormMaxVec; ++k) {
      const int v = threadIdx.x + k * kNormThreads;
      if (v < nvec) {
        float f[8], g[8];
        unpack8(keep[k], f);
        unpack8(reinterpret_cast<const uint4*>(w)[v], g);
#pragma unroll
        for (int i = 0; i < 8; ++i) f[i] = f[i] * rs * g[i];
        yr[v] = pack8(f);
      }
    }
    for (int v = threadIdx.x + kNormMaxVec * kNormThreads; v < nvec; v += kNormThreads) {
      float f[8], g[8];
      unpack8(xr[v], f);
      unpack8(reinterpret_cast<const uint4*>(w)[v], g);
#pragma unroll
      for (int i = 0; i < 8; ++i) f[i] = f[i] * rs * g[i];
      yr[v] = pack8(f);
    }
  }
}

// Each block walks rows blockIdx.x, +gridDim.x, ... and keeps its share of the
// weight gradient in registers (thread t owns vectors t, t+256, ...).
__global__ void __launch_bounds__(kNormThreads) k_rmsnorm_bwd(const __nv_bfloat16* __restrict__ dy,
                                                               const __nv_bfloat16* __restrict__ x,
                                                               const __nv_bfloat16* __restrict__ w,
                                                               const float* __restrict__ rstd,
                                                               __nv_bfloat16* __restrict__ dx,
                                                               float* __restrict__ dw_partial, int rows, int cols) {
  __shared__ float scratch[32];
  const int nvec = cols / 8;
  float dw[kNormMaxVec][8];
#pragma unroll
  for (int k = 0; k < kNormMaxVec; ++k)
#pragma unroll
    for (int i = 0; i < 8; ++i) dw[k][i] = 0.0f;

  for (int r = blockIdx.x; r < rows; r += gridDim.x) {
    const uint4* xr = reinterpret_cast<const uint4*>(x + static_cast<size_t>(r) * cols);
    const uint4* dyr = reinterpret_cast<const uint4*>(dy + static_cast<size_t>(r) * cols);
    uint4* dxr = reinterpret_cast<uint4*>(dx + static_cast<size_t>(r) * cols);
    const float rs = rstd[r];
    // dot = sum(dy * w * xhat)
    float dot = 0.0f;
    for (int v = threadIdx.x; v < nvec; v += kNormThreads) {
      float fx[8], fd[8], fw[8];
      unpack8(xr[v], fx);
      unpack8(dyr[v], fd);
      unpack8(reinterpret_cast<const uint4*>(w)[v], fw);
#pragma unroll
      for (int i = 0; i < 8; ++i) dot += fd[i] * fw[i] * fx[i] * rs;
    }
    dot = block_sum(dot, scratch) / static_cast<float>(cols);
#pragma unroll
    for (int k = 0; k < kNormMaxVec; ++k) {
      const int v = threadIdx.x + k * kNormThreads;
      if (v < nvec) {
        float fx[8], fd[8], fw[8], o[8];
        unpack8(xr[v], fx);
        unpack8(dyr[v], fd);
        unpack8(reinterpret_cast<const uint4*>(w)[v], fw);
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          const float xhat = fx[i] * rs;
          o[i] = rs * (fd[i] * fw[i] - xhat * dot);
          dw[k][i] += fd[i] * xhat;
        }
        dxr[v] = pack8(o);
      }
    }
  }
  float* out = dw_partial + static_cast<size_t>(blockIdx.x) * cols;
#pragma unroll
  for (int k = 0; k < kNormMaxVec; ++k) {
    const int v = threadIdx.x + k * kNormThreads;
    if (v < nvec) {
#pragma unroll
      for (int i = 0; i < 8; ++i) out[v * 8 + i] = dw[k][i];
    }
  }
}

__global__ void k_colsum_bf16(const float* __restrict__ in, __nv_bfloat16* __restrict__ out, int rows, int cols) {
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= cols) return;
  float s = 0.0f;
  for (int r = 0; r < rows; ++r) s += in[static_cast<size_t>(r) * cols + c];
  out[c] = __float2bfloat16_rn(s);
}

// ---------------------------------------------------------------- RoPE ------

__global__ void k_rope(__nv_bfloat16* __restrict__ x, const int* __restrict__ pos, const float* __restrict__ cos_t,
                       const float* __restrict__ sin_t, int tokens, int heads, int head_dim, float sign) {
  // One thread rotates 4 pairs (8 bf16 = 16 bytes).
  const int vec_per_head = head_dim / 8;
  const size_t total = static_cast<size_t>(tokens) * heads * vec_per_head;
  for (size_t i = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<size_t>(gridDim.x) * blockDim.x) {
    const int v = static_cast<int>(i % vec_per_head);
    const size_t th = i / vec_per_head;
    const int t = static_cast<int>(th / heads);
    const int p = pos[t];
    uint4* ptr = reinterpret_cast<uint4*>(x) + i;
    float f[8];
    unpack8(*ptr, f);
    const float* c = cos_t + static_cast<size_t>(p) * (head_dim / 2) + v * 4;
    const float* s = sin_t + static_cast<size_t>(p) * (head_dim / 2) + v * 4;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float a = f[2 * j], b = f[2 * j + 1];
      const float cs = c[j], sn = s[j] * sign;
      f[2 * j] = a * cs - b * sn;
      f[2 * j + 1] = a * sn + b * cs;
    }
    *ptr = pack8(f);
  }
}

// -------------------------------------------------------------- SwiGLU ------

__global__ void k_swiglu_fwd(const __nv_bfloat16* __restrict__ gate_up, __nv_bfloat16* __restrict__ h, int rows, int ffn) {
  const int vec_per_row = ffn / 8;
  const size_t total = static_cast<size_t>(rows) * vec_per_row;
  for (size_t i = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<size_t>(gridDim.x) * blockDim.x) {
    const size_t r = i / vec_per_row;
    const int v = static_cast<int>(i % vec_per_row);
    const uint4* row = reinterpret_cast<const uint4*>(gate_up + r * 2 * static_cast<size_t>(ffn));
    float g[8], u[8], o[8];
    unpack8(row[v], g);
    unpack8(row[vec_per_row + v], u);
#pragma unroll
    for (int k = 0; k < 8; ++k) {
      const float sig = 1.0f / (1.0f + __expf(-g[k]));
      o[k] = g[k] * sig * u[k];
    }
    reinterpret_cast<uint4*>(h)[i] = pack8(o);
  }
}

__global__ void k_swiglu_bwd(const __nv_bfloat16* __restrict__ dh, const __nv_bfloat16* __restrict__ gate_up,
                             __nv_bfloat16* __restrict__ dgate_up, int rows, int ffn) {
  const int vec_per_row = ffn / 8;
  const size_t total = static_cast<size_t>(rows) * vec_per_row;
  for (size_t i = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<size_t>(gridDim.x) * blockDim.x) {
    const size_t r = i / vec_per_row;
    const int v = static_cast<int>(i % vec_per_row);
    const uint4* row = reinterpret_cast<const uint4*>(gate_up + r * 2 * static_cast<size_t>(ffn));
    uint4* drow = reinterpret_cast<uint4*>(dgate_up + r * 2 * static_cast<size_t>(ffn));
    float g[8], u[8], d[8], dg[8], du[8];
    unpack8(row[v], g);
    unpack8(row[vec_per_row + v], u);
    unpack8(reinterpret_cast<const uint4*>(dh)[i], d);
#pragma unroll
    for (int k = 0; k < 8; ++k) {
      const float sig = 1.0f / (1.0f + __expf(-g[k]));
      const float silu = g[k] * sig;
      dg[k] = d[k] * u[k] * (sig + silu * (1.0f - sig));
      du[k] = d[k] * silu;
    }
    drow[v] = pack8(dg);
    drow[vec_per_row + v] = pack8(du);
  }
}

// ------------------------------------------------------- cross-entropy ------

constexpr int kCeThreads = 512;

__global__ void __launch_bounds__(kCeThreads) k_cross_entropy(__nv_bfloat16* __restrict__ logits,
                                                              const int64_t* __restrict__ targets,
                                                              float* __restrict__ loss, int rows, int vocab,
                                                              float grad_scale) {
  __shared__ float scratch[32];
  for (int r = blockIdx.x; r < rows; r += gridDim.x) {
    __nv_bfloat16* row = logits + static_cast<size_t>(r) * vocab;
    const int64_t tgt = targets[r];
    const bool row_aligned = (reinterpret_cast<uintptr_t>(row) & 15u) == 0;
    const int nvec = row_aligned ? vocab / 8 : 0;
    // pass 1: online max / sum-exp per thread, merged across the block
    float mx = -INFINITY, sum = 0.0f;
    auto feed = [&](float z) {
      if (z > mx) {
        sum = sum * __expf(mx - z) + 1.0f;
        mx = z;
      } else {
        sum += __expf(z - mx);
      }
    };
    for (int v = threadIdx.x; v < nvec; v += kCeThreads) {
      float f[8];
      unpack8(reinterpret_cast<const uint4*>(row)[v], f);
#pragma unroll
      for (int i = 0; i < 8; ++i) feed(f[i]);
    }
    for (int c = nvec * 8 + threadIdx.x; c < vocab; c += kCeThreads) feed(__bfloat162float(row[c]));
    const float gmx = block_max(mx, scratch);
    const float gsum = block_sum(mx == -INFINITY ? 0.0f : sum * __expf(mx - gmx), scratch);
    const float lse = gmx + __logf(gsum);
    const bool ignore = tgt < 0 || tgt >= vocab;
    if (threadIdx.x == 0) {
      loss[r] = ignore ? 0.0f : lse - __bfloat162float(row[tgt]);
    }
    __syncthreads();  // the target logit was read before anybody overwrites it
    // pass 2: gradient in place
    const float gs = ignore ? 0.0f : grad_scale;
    for (int v = threadIdx.x; v < nvec; v += kCeThreads) {
      float f[8];
      unpack8(reinterpret_cast<const uint4*>(row)[v], f);
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const int c = v * 8 + i;
        f[i] = (__expf(f[i] - lse) - (c == tgt ? 1.0f : 0.0f)) * gs;
      }
      reinterpret_cast<uint4*>(row)[v] = pack8(f);
    }
    for (int c = nvec * 8 + threadIdx.x; c < vocab; c += kCeThreads) {
      const float z = __bfloat162float(row[c]);
      row[c] = __float2bfloat16_rn((__expf(z - lse) - (c == tgt ? 1.0f : 0.0f)) * gs);
    }
    __syncthreads();
  }
}

// ------------------------------------------------------------ cast copy -----

template <typename In, typename Out>
__global__ void __launch_bounds__(256) k_cast_scale(const In* __restrict__ in, Out* __restrict__ out, size_t n, float scale) {
  // 8 elements per thread and step, two steps in flight.
  const size_t nvec = n / 8;
  const size_t stride = static_cast<size_t>(gridDim.x) * blockDim.x;
  for (size_t v = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x; v < nvec; v += stride) {
    float f[8];
    if constexpr (sizeof(In) == 4) {
      const float4 a = __ldcs(reinterpret_cast<const float4*>(in) + 2 * v);
      const float4 b = __ldcs(reinterpret_cast<const float4*>(in) + 2 * v + 1);
      f[0] = a.x; f[1] = a.y; f[2] = a.z; f[3] = a.w;
      f[4] = b.x; f[5] = b.y; f[6] = b.z; f[7] = b.w;
    } else {
      unpack8(__ldcs(reinterpret_cast<const uint4*>(in) + v), f);
    }
#pragma unroll
    for (int i = 0; i < 8; ++i) f[i] *= scale;
    if constexpr (sizeof(Out) == 4) {
      reinterpret_cast<float4*>(out)[2 * v] = make_float4(f[0], f[1], f[2], f[3]);
      reinterpret_cast<float4*>(out)[2 * v + 1] = make_float4(f[4], f[5], f[6], f[7]);
    } else {
      reinterpret_cast<uint4*>(out)[v] = pack8(f);
    }
  }
  if (blockIdx.x == 0) {
    for (size_t i = nvec * 8 + threadIdx.x; i < n; i += blockDim.x) {
      float x;
      if constexpr (sizeof(In) == 4) x = reinterpret_cast<const float*>(in)[i];
      else x = __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(in)[i]);
      x *= scale;
      if constexpr (sizeof(Out) == 4) reinterpret_cast<float*>(out)[i] = x;
      else reinterpret_cast<__nv_bfloat16*>(out)[i] = __float2bfloat16_rn(x);
    }
  }
}

// --------------------------------------------------------------- AdamW ------

// sqrt and division as the hardware approximations (about 1 ulp): the IEEE
// sequences cost several times the arithmetic of the rest of the update and
// made this memory-bound kernel issue-bound.
__device__ __forceinline__ float fast_sqrt(float x) {
  float r;
  asm("sqrt.approx.f32 %0, %1;" : "=f"(r) : "f"(x));
  return r;
}

__device__ __forceinline__ float adamw_one(float p, float g, float& m, float& v, float lr, float beta1, float beta2,
                                           float eps, float decay, float inv_bias1, float inv_bias2, float grad_scale) {
  const float gr = g * grad_scale;
  m = beta1 * m + (1.0f - beta1) * gr;
  v = beta2 * v + (1.0f - beta2) * gr * gr;
  const float denom = fast_sqrt(v * inv_bias2) + eps;
  return p * decay - __fdividef(lr * (m * inv_bias1), denom);
}

__global__ void __launch_bounds__(256) k_adamw(float* __restrict__ p, const float* __restrict__ g, float* __restrict__ m,
                                               float* __restrict__ v, size_t n, float lr, float beta1, float beta2,
                                               float eps, float weight_decay, float bias1, float bias2, float grad_scale) {
  const size_t nvec = n / 4;
  const float inv_bias1 = 1.0f / bias1, inv_bias2 = 1.0f / bias2, decay = 1.0f - lr * weight_decay;
  const size_t stride = static_cast<size_t>(gridDim.x) * blockDim.x;
  size_t i = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x;
  // Two vectors per thread and step: eight 16-byte loads in flight.
  for (; i + stride < nvec; i += 2 * stride) {
    float4 pp[2], gg[2], mm[2], vv[2];
#pragma unroll
    for (int u = 0; u < 2; ++u) {
      const size_t j = i + u * stride;
      pp[u] = reinterpret_cast<float4*>(p)[j];
      gg[u] = __ldcs(reinterpret_cast<const float4*>(g) + j);  // the gradient is not read again
      mm[u] = reinterpret_cast<float4*>(m)[j];
      vv[u] = reinterpret_cast<float4*>(v)[j];
    }
#pragma unroll
    for (int u = 0; u < 2; ++u) {
      float* pa = &pp[u].x;
      const float* ga = &gg[u].x;
      float* ma = &mm[u].x;
      float* va = &vv[u].x;
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        pa[k] = adamw_one(pa[k], ga[k], ma[k], va[k], lr, beta1, beta2, eps, decay, inv_bias1, inv_bias2, grad_scale);
      }
      const size_t j = i + u * stride;
      reinterpret_cast<float4*>(p)[j] = pp[u];
      reinterpret_cast<float4*>(m)[j] = mm[u];
      reinterpret_cast<float4*>(v)[j] = vv[u];
    }
  }
  for (; i < nvec; i += stride) {
    float4 pp = reinterpret_cast<float4*>(p)[i];
    const float4 gg = reinterpret_cast<const float4*>(g)[i];
    float4 mm = reinterpret_cast<float4*>(m)[i];
    float4 vv = reinterpret_cast<float4*>(v)[i];
    float* pa = &pp.x;
    const float* ga = &gg.x;
    float* ma = &mm.x;
    float* va = &vv.x;
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      pa[k] = adamw_one(pa[k], ga[k], ma[k], va[k], lr, beta1, beta2, eps, decay, inv_bias1, inv_bias2, grad_scale);
    }
    reinterpret_cast<float4*>(p)[i] = pp;
    reinterpret_cast<float4*>(m)[i] = mm;
    reinterpret_cast<float4*>(v)[i] = vv;
  }
  // tail
  if (blockIdx.x == 0) {
    for (size_t t = nvec * 4 + threadIdx.x; t < n; t += blockDim.x) {
      p[t] = adamw_one(p[t], g[t], m[t], v[t], lr, beta1, beta2, eps, decay, inv_bias1, inv_bias2, grad_scale);
    }
  }
}

int grid_for(size_t work_items, int threads) {
  const size_t want = (work_items + threads - 1) / threads;
  const size_t cap = static_cast<size_t>(kSms) * 8;
  return static_cast<int>(want < 1 ? 1 : (want > cap ? cap : want));
}

} // namespace

void note_kernel_launch(int n) { g_launches.fetch_add(static_cast<unsigned long long>(n), std::memory_order_relaxed); }
unsigned long long kernel_launch_count() { return g_launches.load(std::memory_order_relaxed); }
unsigned long long fused_ops_launch_count() { return kernel_launch_count(); }

cudaError_t launch_rmsnorm_fwd(const __nv_bfloat16* x, const __nv_bfloat16* w, __nv_bfloat16* y, float* rstd, int rows,
                               int cols, float eps, cudaStream_t s) {
  if (cols % 8 != 0 || rows <= 0) return cudaErrorInvalidValue;
  const int blocks = rows < kSms * 8 ? rows : kSms * 8;
  k_rmsnorm_fwd<<<blocks, kNormThreads, 0, s>>>(x, w, y, rstd, rows, cols, eps);
  note_kernel_launch();
  return cudaGetLastError();
}

cudaError_t launch_rmsnorm_bwd(const __nv_bfloat16* dy, const __nv_bfloat16* x, const __nv_bfloat16* w,
                               const float* rstd, __nv_bfloat16* dx, float* dw_partial, int* nblocks, int rows,
                               int cols, cudaStream_t s) {
  if (cols % 8 != 0 || rows <= 0 || cols > kNormThreads * kNormMaxVec * 8) return cudaErrorInvalidValue;
  const int blocks = rows < kSms * 2 ? rows : kSms * 2;
  if (nblocks) *nblocks = blocks;
  if (dw_partial == nullptr) return cudaSuccess;
  k_rmsnorm_bwd<<<blocks, kNormThreads, 0, s>>>(dy, x, w, rstd, dx, dw_partial, rows, cols);
  note_kernel_launch();
  return cudaGetLastError();
}

cudaError_t launch_cast_scale(const void* in, int in_kind, void* out, int out_kind, size_t n, float scale, cudaStream_t s) {
  if (n == 0) return cudaSuccess;
  const size_t in_bytes = in_kind == 0 ? 4 : 2, out_bytes = out_kind == 0 ? 4 : 2;
  // Vector accesses of 8 elements: 32-byte (fp32) or 16-byte (bf16) alignment of the bases.
  if ((reinterpret_cast<uintptr_t>(in) % (8 * in_bytes)) != 0 || (reinterpret_cast<uintptr_t>(out) % (8 * out_bytes)) != 0) {
    return cudaErrorInvalidValue;
  }
  const int grid = grid_for(n / 8 + 1, 256);
  if (in_kind == 0 && out_kind == 0) k_cast_scale<float, float><<<grid, 256, 0, s>>>(static_cast<const float*>(in), static_cast<float*>(out), n, scale);
  else if (in_kind == 0 && out_kind == 1) k_cast_scale<float, __nv_bfloat16><<<grid, 256, 0, s>>>(static_cast<const float*>(in), static_cast<__nv_bfloat16*>(out), n, scale);
  else if (in_kind == 1 && out_kind == 0) k_cast_scale<__nv_bfloat16, float><<<grid, 256, 0, s>>>(static_cast<const __nv_bfloat16*>(in), static_cast<float*>(out), n, scale);
  else k_cast_scale<__nv_bfloat16, __nv_bfloat16><<<grid, 256, 0, s>>>(static_cast<const __nv_bfloat16*>(in), static_cast<__nv_bfloat16*>(out), n, scale);
  note_kernel_launch();
  return cudaGetLastError();
}

cudaError_t launch_colsum_bf16(const float* in, __nv_bfloat16* out, int rows, int cols, cudaStream_t s) {
  k_colsum_bf16<<<(cols + 255) / 256, 256, 0, s>>>(in, out, rows, cols);
  note_kernel_launch();
  return cudaGetLastError();
}

cudaError_t launch_rope(__nv_bfloat16* x, const int* pos, const float* cos_t, const float* sin_t, int tokens, int heads,
                        int head_dim, bool inverse, cudaStream_t s) {
  if (head_dim % 8 != 0) return cudaErrorInvalidValue;
  const size_t total = static_cast<size_t>(tokens) * heads * (head_dim / 8);
  k_rope<<<grid_for(total, 256), 256, 0, s>>>(x, pos, cos_t, sin_t, tokens, heads, head_dim, inverse ? -1.0f : 1.0f);
  note_kernel_launch();
  return cudaGetLastError();
}

cudaError_t launch_swiglu_fwd(const __nv_bfloat16* gate_up, __nv_bfloat16* h, int rows, int ffn, cudaStream_t s) {
  if (ffn % 8 != 0) return cudaErrorInvalidValue;
  k_swiglu_fwd<<<grid_for(static_cast<size_t>(rows) * (ffn / 8), 256), 256, 0, s>>>(gate_up, h, rows, ffn);
  note_kernel_launch();
  return cudaGetLastError();
}

cudaError_t launch_swiglu_bwd(const __nv_bfloat16* dh, const __nv_bfloat16* gate_up, __nv_bfloat16* dgate_up, int rows,
                              int ffn, cudaStream_t s) {
  if (ffn % 8 != 0) return cudaErrorInvalidValue;
  k_swiglu_bwd<<<grid_for(static_cast<size_t>(rows) * (ffn / 8), 256), 256, 0, s>>>(dh, gate_up, dgate_up, rows, ffn);
  note_kernel_launch();
  return cudaGetLastError();
}

cudaError_t launch_cross_entropy_fwd_bwd(__nv_bfloat16* logits, const int64_t* targets, float* loss, int rows, int vocab,
                                         float grad_scale, cudaStream_t s) {
  if (rows <= 0 || vocab <= 0) return cudaErrorInvalidValue;
  const int blocks = rows < kSms * 4 ? rows : kSms * 4;
  k_cross_entropy<<<blocks, kCeThreads, 0, s>>>(logits, targets, loss, rows, vocab, grad_scale);
  note_kernel_launch();
  return cudaGetLastError();
}

cudaError_t launch_adamw(float* p, const float* g, float* m, float* v, size_t n, float lr, float beta1, float beta2,
                         float eps, float weight_decay, int step, float grad_scale, cudaStream_t s) {
  if (n == 0) return cudaSuccess;
  const float bias1 = 1.0f - powf(beta1, static_cast<float>(step));
  const float bias2 = 1.0f - powf(beta2, static_cast<float>(step));
  k_adamw<<<grid_for(n / 4 + 1, 256), 256, 0, s>>>(p, g, m, v, n, lr, beta1, beta2, eps, weight_decay, bias1, bias2,
                                                    grad_scale);
  note_kernel_launch();
  return cudaGetLastError();
}

} // namespace b200c
