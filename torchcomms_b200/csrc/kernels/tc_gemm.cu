// tcgen05 / TMEM GEMM kernels (sm_100a). See tc_gemm.h.
//
// Roles inside a CTA of 192 threads (+ optional copy warps in fused kernels):
//   warp 0, one lane : TMA producer - fills a ring of shared-memory stages
//   warp 1           : allocates tensor memory; one lane issues tcgen05.mma
//   warps 2..5       : epilogue - tcgen05.ld the fp32 accumulator, convert,
//                      store (each warp owns the 32 TMEM lanes of its
//                      warp-id % 4 quadrant)
#include "tc_gemm.h"

#include <algorithm>
#include <mutex>

#include "launch_count.h"
#include "tc_gemm.cuh"

namespace b200c {

namespace {

using namespace tc;

// ------------------------------------------------------- tensor maps ------

using EncodeTiledFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                   const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                   CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, []() {
    void* sym = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess) {
      fn = reinterpret_cast<EncodeTiledFn>(sym);
    }
  });
  return fn;
}

// Row-major bf16 matrix [rows, cols]; box = [box_rows, 64 columns], 128-byte swizzle.
bool make_map(CUtensorMap* map, const void* base, uint64_t rows, uint64_t cols, uint32_t box_rows) {
  EncodeTiledFn fn = encode_fn();
  if (fn == nullptr) return false;
  const cuuint64_t dims[2] = {cols, rows};
  const cuuint64_t strides[1] = {cols * 2};
  const cuuint32_t box[2] = {static_cast<cuuint32_t>(kBlockK), box_rows};
  const cuuint32_t elem[2] = {1, 1};
  return fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, elem,
            CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

// ------------------------------------------------------ shared layout ------

template <int BN>
struct TileCfg {
  static constexpr int kStages = BN == 256 ? 4 : 6;
  static constexpr int kABytes = kBlockM * kBlockK * 2;
  static constexpr int kBBytes = BN * kBlockK * 2;
  static constexpr int kStageBytes = kABytes + kBBytes;
  static constexpr int kSmemBytes = kStages * kStageBytes + 1024 /*alignment slack*/ + 256 /*barriers*/;
  static constexpr uint32_t kTmemCols = BN;  // power of two >= 32
};

struct Barriers {
  uint64_t full[8];
  uint64_t empty[8];
  uint64_t acc_full;
  uint32_t tmem_base;
  uint32_t failed;
};

__device__ __forceinline__ uint32_t pack_bf16(uint32_t a, uint32_t b) {
  __nv_bfloat162 h = __floats2bfloat162_rn(__uint_as_float(a), __uint_as_float(b));
  return *reinterpret_cast<uint32_t*>(&h);
}

// One output tile: mainloop over K with the producer / MMA roles, accumulator
// left in tensor memory. `k_iters` blocks of 64. Called by warps 0 and 1 only.
template <int BN>
__device__ __forceinline__ void tile_mainloop(const CUtensorMap* map_a, const CUtensorMap* map_b, char* stages,
                                              Barriers* bars, int m0, int n0, int k_iters, uint32_t& it,
                                              uint32_t tmem_acc, int warp, int lane) {
  using Cfg = TileCfg<BN>;
  constexpr uint32_t idesc = make_idesc_bf16(kBlockM, BN);
  if (warp == 0 && lane == 0) {
    for (int kb = 0; kb < k_iters; ++kb) {
      const uint32_t i = it + kb;
      const int s = i % Cfg::kStages;
      const uint32_t ph = (i / Cfg::kStages) & 1u;
      if (!mbar_wait(&bars->empty[s], ph ^ 1u)) {
        bars->failed = 1;
        break;
      }
      mbar_expect_tx(&bars->full[s], Cfg::kStageBytes);
      char* sa = stages + s * Cfg::kStageBytes;
      tma_load_2d(sa, map_a, &bars->full[s], kb * kBlockK, m0);
      tma_load_2d(sa + Cfg::kABytes, map_b, &bars->full[s], kb * kBlockK, n0);
    }
  } else if (warp == 1 && lane == 0) {
    for (int kb = 0; kb < k_iters; ++kb) {
      const uint32_t i = it + kb;
      const int s = i % Cfg::kStages;
      const uint32_t ph = (i / Cfg::kStages) & 1u;
      if (!mbar_wait(&bars->full[s], ph)) {
        bars->failed = 1;
        break;
      }
      tc_fence_after_sync();
      const uint32_t sa = smem_u32(stages + s * Cfg::kStageBytes);
      const uint64_t da = make_smem_desc(sa);
      const uint64_t db = make_smem_desc(sa + Cfg::kABytes);
#pragma unroll
      for (int kk = 0; kk < kBlockK / kUmmaK; ++kk) {
        // 16 bf16 = 32 bytes further along K inside the swizzled row
        umma_bf16(tmem_acc, da + static_cast<uint64_t>(kk * 2), db + static_cast<uint64_t>(kk * 2), idesc, (kb | kk) != 0);
      }
      umma_commit(&bars->empty[s]);  // stage reusable once these MMAs have read it
    }
    umma_commit(&bars->acc_full);    // accumulator complete
  }
  it += static_cast<uint32_t>(k_iters);
}

// ------------------------------------------------------------ plain GEMM ---

template <int BN>
__global__ void __launch_bounds__(192, 1) k_gemm_bf16_nt(const __grid_constant__ CUtensorMap map_a,
                                                          const __grid_constant__ CUtensorMap map_b,
                                                          __nv_bfloat16* __restrict__ c, int m, int n, int k,
                                                          uint32_t* status) {
  using Cfg = TileCfg<BN>;
  extern __shared__ char smem_raw[];
  char* stages = reinterpret_cast<char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
  Barriers* bars = reinterpret_cast<Barriers*>(stages + Cfg::kStages * Cfg::kStageBytes);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n0 = blockIdx.x * BN, m0 = blockIdx.y * kBlockM;

  if (threadIdx.x == 0) {
    for (int s = 0; s < Cfg::kStages; ++s) {
      mbar_init(&bars->full[s], 1);
      mbar_init(&bars->empty[s], 1);
    }
    mbar_init(&bars->acc_full, 1);
    bars->failed = 0;
    fence_barrier_init();
  }
  if (warp == 1) {
    tmem_alloc(&bars->tmem_base, Cfg::kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_acc = bars->tmem_base;

  uint32_t it = 0;
  if (warp < 2) {
    tile_mainloop<BN>(&map_a, &map_b, stages, bars, m0, n0, k / kBlockK, it, tmem_acc, warp, lane);
  } else {
    // Epilogue warps: quadrant q of the accumulator's 128 lanes.
    const int q = warp & 3;
    const bool ok = mbar_wait(&bars->acc_full, 0);
    tc_fence_after_sync();
    const int row = m0 + q * 32 + lane;
    if (ok) {
      for (int c0 = 0; c0 < BN; c0 += 32) {
        uint32_t r[32];
        tmem_ld_32x32(tmem_acc + (static_cast<uint32_t>(q * 32) << 16) + static_cast<uint32_t>(c0), r);
        tmem_ld_wait();
        if (row < m) {
          uint4* dst = reinterpret_cast<uint4*>(c + static_cast<size_t>(row) * n + n0 + c0);
#pragma unroll
          for (int v = 0; v < 4; ++v) {
            dst[v] = make_uint4(pack_bf16(r[8 * v], r[8 * v + 1]), pack_bf16(r[8 * v + 2], r[8 * v + 3]),
                                pack_bf16(r[8 * v + 4], r[8 * v + 5]), pack_bf16(r[8 * v + 6], r[8 * v + 7]));
          }
        }
      }
    } else {
      bars->failed = 1;
    }
  }
  tc_fence_before_sync();
  __syncthreads();
  if (warp == 1) {
    tmem_dealloc(tmem_acc, Cfg::kTmemCols);
  }
  if (threadIdx.x == 0 && bars->failed && status != nullptr) {
    status[0] = status[0] | kStatusTimeout;
  }
}

template <int BN>
cudaError_t launch_plain(const void* a, const void* b, void* c, int m, int n, int k, uint32_t* status, cudaStream_t s) {
  using Cfg = TileCfg<BN>;
  CUtensorMap map_a, map_b;
  if (!make_map(&map_a, a, m, k, kBlockM) || !make_map(&map_b, b, n, k, BN)) return cudaErrorInvalidValue;
  static bool attr_set = false;
  if (!attr_set) {
    cudaError_t e = cudaFuncSetAttribute(k_gemm_bf16_nt<BN>, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::kSmemBytes);
    if (e != cudaSuccess) return e;
    attr_set = true;
  }
  dim3 grid(n / BN, (m + kBlockM - 1) / kBlockM);
  k_gemm_bf16_nt<BN><<<grid, 192, Cfg::kSmemBytes, s>>>(map_a, map_b, static_cast<__nv_bfloat16*>(c), m, n, k, status);
  note_kernel_launch();
  return cudaGetLastError();
}

// TC_FUSED_PART

} // namespace

cudaError_t launch_gemm_bf16_nt(const void* a, const void* b, void* c, int m, int n, int k, uint32_t* status,
                                cudaStream_t stream) {
  if (k % kBlockK != 0 || n % 128 != 0 || m <= 0) return cudaErrorInvalidValue;
  if ((reinterpret_cast<uintptr_t>(a) | reinterpret_cast<uintptr_t>(b) | reinterpret_cast<uintptr_t>(c)) & 15u) {
    return cudaErrorInvalidValue;
  }
  if (n % 256 == 0) return launch_plain<256>(a, b, c, m, n, k, status, stream);
  return launch_plain<128>(a, b, c, m, n, k, status, stream);
}

} // namespace b200c
