// Shared pieces of the peer-memory collective kernels: 16-byte packs of each
// element type, reductions, conversions, and the launch helper that runs an
// operation either for real (one rank per GPU) or as several virtual ranks in
// one cooperative launch on a single GPU (tests).
#pragma once

#include <algorithm>
#include <type_traits>
#include <vector>

#include "collectives.h"
#include "launch_count.h"

namespace b200c {
namespace coll {

// ------------------------------------------------------------ packs --------

template <typename T>
struct Pack;

template <>
struct Pack<float> {
  static constexpr int N = 4;
  static __device__ __forceinline__ void unpack(uint4 v, float* f) {
    f[0] = __uint_as_float(v.x);
    f[1] = __uint_as_float(v.y);
    f[2] = __uint_as_float(v.z);
    f[3] = __uint_as_float(v.w);
  }
  static __device__ __forceinline__ uint4 pack(const float* f) {
    return make_uint4(__float_as_uint(f[0]), __float_as_uint(f[1]), __float_as_uint(f[2]), __float_as_uint(f[3]));
  }
  static __device__ __forceinline__ float to_float(float x) { return x; }
  static __device__ __forceinline__ float from_float(float x) { return x; }
  static __device__ __forceinline__ uint4 mc_sum(const void* p) {
    float4 r = multimem_ld_reduce_add_f32x4(p);
    return make_uint4(__float_as_uint(r.x), __float_as_uint(r.y), __float_as_uint(r.z), __float_as_uint(r.w));
  }
};

template <>
struct Pack<__nv_bfloat16> {
  static constexpr int N = 8;
  static __device__ __forceinline__ void unpack(uint4 v, float* f) {
    float2 a = bf16x2_to_float2(v.x), b = bf16x2_to_float2(v.y), c = bf16x2_to_float2(v.z), d = bf16x2_to_float2(v.w);
    f[0] = a.x; f[1] = a.y; f[2] = b.x; f[3] = b.y; f[4] = c.x; f[5] = c.y; f[6] = d.x; f[7] = d.y;
  }
  static __device__ __forceinline__ uint4 pack(const float* f) {
    return make_uint4(float2_to_bf16x2(f[0], f[1]), float2_to_bf16x2(f[2], f[3]), float2_to_bf16x2(f[4], f[5]),
                      float2_to_bf16x2(f[6], f[7]));
  }
  static __device__ __forceinline__ float to_float(__nv_bfloat16 x) { return __bfloat162float(x); }
  static __device__ __forceinline__ __nv_bfloat16 from_float(float x) { return __float2bfloat16_rn(x); }
  static __device__ __forceinline__ uint4 mc_sum(const void* p) { return multimem_ld_reduce_add_bf16x8(p); }
};

template <>
struct Pack<__half> {
  static constexpr int N = 8;
  static __device__ __forceinline__ void unpack(uint4 v, float* f) {
    float2 a = f16x2_to_float2(v.x), b = f16x2_to_float2(v.y), c = f16x2_to_float2(v.z), d = f16x2_to_float2(v.w);
    f[0] = a.x; f[1] = a.y; f[2] = b.x; f[3] = b.y; f[4] = c.x; f[5] = c.y; f[6] = d.x; f[7] = d.y;
  }
  static __device__ __forceinline__ uint4 pack(const float* f) {
    return make_uint4(float2_to_f16x2(f[0], f[1]), float2_to_f16x2(f[2], f[3]), float2_to_f16x2(f[4], f[5]),
                      float2_to_f16x2(f[6], f[7]));
  }
  static __device__ __forceinline__ float to_float(__half x) { return __half2float(x); }
  static __device__ __forceinline__ __half from_float(float x) { return __float2half_rn(x); }
  static __device__ __forceinline__ uint4 mc_sum(const void* p) { return multimem_ld_reduce_add_f16x8(p); }
};

template <RedKind R>
__device__ __forceinline__ float red(float a, float b) {
  if constexpr (R == RedKind::SUM) return a + b;
  if constexpr (R == RedKind::PROD) return a * b;
  if constexpr (R == RedKind::MIN) return fminf(a, b);
  return fmaxf(a, b);
}

// Sums (or otherwise reduces) one 16-byte vector at byte offset `off` of the
// staging heaps of all ranks, accumulating in fp32. Loads are issued together
// so that up to kMaxRanks NVLink reads are in flight per thread.
template <typename T, RedKind R>
__device__ __forceinline__ void reduce_peers(const CommDev& c, size_t off, float* acc) {
  constexpr int N = Pack<T>::N;
  uint4 v[kMaxRanks];
#pragma unroll
  for (int i = 0; i < kMaxRanks; ++i) {
    if (i < c.nranks) {
      // Start at a different peer on every rank so that the ranks do not all
      // hit the same memory at once.
      int p = c.rank + i;
      if (p >= c.nranks) p -= c.nranks;
      v[i] = ld16(c.heap[p] + off);
    }
  }
  Pack<T>::unpack(v[0], acc);
#pragma unroll
  for (int i = 1; i < kMaxRanks; ++i) {
    if (i < c.nranks) {
      float f[N];
      Pack<T>::unpack(v[i], f);
#pragma unroll
      for (int k = 0; k < N; ++k) acc[k] = red<R>(acc[k], f[k]);
    }
  }
}

// Writes n_valid (<= N) converted values to dst; one 16-byte store per 16
// bytes of output when `aligned`, scalar stores otherwise.
template <typename OutT, int N>
__device__ __forceinline__ void store_values(OutT* dst, const float* f, int n_valid, bool aligned) {
  constexpr int kOutPerVec = 16 / sizeof(OutT);
  if (aligned && n_valid == N) {
    if constexpr (N == kOutPerVec) {
      st16(dst, Pack<OutT>::pack(f));
    } else {
      static_assert(N == 2 * kOutPerVec || N == kOutPerVec, "unsupported output width");
      st16(dst, Pack<OutT>::pack(f));
      st16(dst + kOutPerVec, Pack<OutT>::pack(f + kOutPerVec));
    }
  } else {
    for (int k = 0; k < n_valid; ++k) dst[k] = Pack<OutT>::from_float(f[k]);
  }
}

// Block-cooperative copy with conversion into a staging slot (16-byte aligned).
template <typename DstT, typename SrcT>
__device__ __forceinline__ void block_convert(DstT* __restrict__ dst, const SrcT* __restrict__ src, size_t n) {
  if constexpr (sizeof(DstT) == sizeof(SrcT)) {
    block_copy(dst, src, n * sizeof(SrcT));
  } else {
    // SrcT = float, DstT = 16-bit float: 8 elements per step.
    constexpr int N = Pack<DstT>::N;
    const bool aligned = (reinterpret_cast<uintptr_t>(src) & 15u) == 0;
    const size_t nvec = aligned ? n / N : 0;
    for (size_t v = threadIdx.x; v < nvec; v += blockDim.x) {
      const uint4 a = ld16(src + v * N);
      const uint4 b = ld16(src + v * N + 4);
      float f[8];
      Pack<float>::unpack(a, f);
      Pack<float>::unpack(b, f + 4);
      st16(dst + v * N, Pack<DstT>::pack(f));
    }
    for (size_t i = nvec * N + threadIdx.x; i < n; i += blockDim.x) {
      dst[i] = Pack<DstT>::from_float(static_cast<float>(src[i]));
    }
  }
}

// ------------------------------------------------- stochastic rounding -------
//
// fp32 -> bf16 with the discarded 16 mantissa bits compared against 16 random
// bits, so that the expected value of the rounded number equals the input
// (gradients summed in bf16 over many steps do not lose small updates).
// Random bits: Philox-4x32 with 7 rounds, counter = (vector index, stream),
// key = seed; one call yields the 128 bits that 8 elements need. The
// conversion itself is Blackwell's cvt.rs.bf16x2.f32.
// Parity: comms/utils/kernels/rng/philox_rng.cuh:27-60 and
// stochastic_rounding/stochastic_rounding.cuh:13-75.

__device__ __forceinline__ uint4 philox4x32_7(uint4 ctr, uint2 key) {
  constexpr uint32_t kM0 = 0xD2511F53u, kM1 = 0xCD9E8D57u, kW0 = 0x9E3779B9u, kW1 = 0xBB67AE85u;
#pragma unroll
  for (int r = 0; r < 7; ++r) {
    const uint32_t hi0 = __umulhi(kM0, ctr.x), lo0 = kM0 * ctr.x;
    const uint32_t hi1 = __umulhi(kM1, ctr.z), lo1 = kM1 * ctr.z;
    ctr = make_uint4(hi1 ^ ctr.y ^ key.x, lo1, hi0 ^ ctr.w ^ key.y, lo0);
    key.x += kW0;
    key.y += kW1;
  }
  return ctr;
}

// {hi, lo} -> packed bf16x2 (hi in the upper half), each rounded with its own 16 random bits of `rbits`.
__device__ __forceinline__ uint32_t cvt_rs_bf16x2(float hi, float lo, uint32_t rbits) {
  uint32_t r;
  asm("cvt.rs.bf16x2.f32 %0, %1, %2, %3;" : "=r"(r) : "f"(hi), "f"(lo), "r"(rbits));
  return r;
}

// Block-cooperative fp32 -> bf16 conversion with stochastic rounding into a
// 16-byte aligned staging slot. `stream_id` must differ between calls that
// share a seed and cover different data (rank, destination, chunk offset).
__device__ __forceinline__ void block_convert_sr(__nv_bfloat16* __restrict__ dst, const float* __restrict__ src, size_t n,
                                                 unsigned long long seed, unsigned long long stream_id) {
  const uint2 key = make_uint2(static_cast<uint32_t>(seed), static_cast<uint32_t>(seed >> 32));
  const size_t nvec = (n + 7) / 8;
  for (size_t v = threadIdx.x; v < nvec; v += blockDim.x) {
    float f[8];
#pragma unroll
    for (int k = 0; k < 8; ++k) f[k] = v * 8 + k < n ? src[v * 8 + k] : 0.0f;
    const uint4 rnd = philox4x32_7(make_uint4(static_cast<uint32_t>(v), static_cast<uint32_t>(v >> 32),
                                              static_cast<uint32_t>(stream_id), static_cast<uint32_t>(stream_id >> 32)),
                                   key);
    uint4 o;
    o.x = cvt_rs_bf16x2(f[1], f[0], rnd.x);
    o.y = cvt_rs_bf16x2(f[3], f[2], rnd.y);
    o.z = cvt_rs_bf16x2(f[5], f[4], rnd.z);
    o.w = cvt_rs_bf16x2(f[7], f[6], rnd.w);
    if (v * 8 + 8 <= n) {
      st16(dst + v * 8, o);
    } else {
      const __nv_bfloat16* ob = reinterpret_cast<const __nv_bfloat16*>(&o);
      for (size_t k = 0; v * 8 + k < n; ++k) dst[v * 8 + k] = ob[k];
    }
  }
}

// --------------------------------------------------------- launchers -------

template <typename Op>
__global__ void __launch_bounds__(256, 3) k_real(CommDev c, typename Op::Args a) {
  Op::run(c, a);
}
template <typename Op>
__global__ void __launch_bounds__(256, 3) k_emu(const CommDev* cs, const typename Op::Args* as) {
  Op::run(cs[blockIdx.y], as[blockIdx.y]);
}

template <typename Op>
cudaError_t launch_op(const CommDev* comms, int emu_ranks, const typename Op::Args* args, int blocks,
                      int threads, cudaStream_t stream, bool exact_grid = false) {
  using Args = typename Op::Args;
  if (blocks < 1) blocks = 1;
  if (exact_grid && blocks > kMaxBlocks) return cudaErrorInvalidConfiguration;
  if (blocks > kMaxBlocks) blocks = kMaxBlocks;
  if (threads > 256) threads = 256;
  {
    // Blocks wait on their peers' blocks, so all of them must be resident at
    // once: never launch more than the device can hold. Identical GPUs give
    // the same bound on every rank, which keeps the grids equal.
    static int resident_cap = 0;
    if (resident_cap == 0) {
      int dev = 0, sms = 0, per_sm = 0;
      cudaGetDevice(&dev);
      cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
      cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, k_real<Op>, 256, 0);
      resident_cap = sms * (per_sm > 0 ? per_sm : 1);
    }
    const int cap = emu_ranks > 0 ? resident_cap / emu_ranks : resident_cap;
    // One block per piece (latency kernels): a smaller grid would skip data.
    if (exact_grid && blocks > cap) return cudaErrorInvalidConfiguration;
    if (blocks > cap) blocks = cap > 0 ? cap : 1;
  }
  note_kernel_launch();
  if (emu_ranks <= 0) {
    k_real<Op><<<blocks, threads, 0, stream>>>(comms[0], args[0]);
    return cudaGetLastError();
  }
  // Emulation: all virtual ranks in one cooperative launch.
  CommDev* d_comms = nullptr;
  Args* d_args = nullptr;
  cudaError_t e = cudaMalloc(&d_comms, sizeof(CommDev) * emu_ranks);
  if (e != cudaSuccess) return e;
  e = cudaMalloc(&d_args, sizeof(Args) * emu_ranks);
  if (e != cudaSuccess) { cudaFree(d_comms); return e; }
  cudaMemcpyAsync(d_comms, comms, sizeof(CommDev) * emu_ranks, cudaMemcpyHostToDevice, stream);
  cudaMemcpyAsync(d_args, args, sizeof(Args) * emu_ranks, cudaMemcpyHostToDevice, stream);
  void* params[] = {&d_comms, &d_args};
  e = cudaLaunchCooperativeKernel(reinterpret_cast<void*>(&k_emu<Op>), dim3(blocks, emu_ranks), dim3(threads),
                                  params, 0, stream);
  cudaError_t e2 = cudaStreamSynchronize(stream);
  cudaFree(d_comms);
  cudaFree(d_args);
  return e != cudaSuccess ? e : e2;
}

__device__ __forceinline__ size_t min_sz(size_t a, size_t b) { return a < b ? a : b; }

} // namespace coll
} // namespace b200c
