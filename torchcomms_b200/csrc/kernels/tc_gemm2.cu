// bf16 GEMM on CTA pairs (tcgen05 cta_group::2). See tc_gemm.h.
//
// A cluster of two CTAs owns a 256 x 256 output tile. Each CTA loads its own
// 128 rows of A and HALF of the B tile (128 of the 256 rows of B) per k-step,
// so the pair reads every B element once instead of twice; the leader CTA
// issues one 256 x 256 x 16 MMA for both, accumulating into the tensor memory
// of both. The smaller per-CTA stage (32 KB) also buys a 6-deep TMA ring.
//
// Roles per CTA (192 threads): warp 0 lane 0 TMA producer (both CTAs), warp 1
// tensor-memory allocation (both CTAs) and MMA issue (leader only), warps 2-5
// epilogue (both CTAs: tcgen05.ld -> bf16 -> swizzled staging -> TMA store).
// Barriers: `full` lives in the leader and counts the bytes of all four loads
// of a stage; `empty` and `acc_full` exist in both CTAs and are released by
// the leader's commits (arrival delivered to both CTAs); `acc_empty` lives in
// the leader and collects the eight epilogue warps of the pair.
// No load uses cluster multicast.
#include "tc_gemm.h"

#include <algorithm>

#include "launch_count.h"
#include "tc_gemm.cuh"

namespace b200c {

namespace {

using namespace tc;

constexpr int kBN = 256;
constexpr int kStages = 6;
constexpr int kABytes = kBlockM * kBlockK * 2;        // 16 KB: this CTA's 128 rows of A
constexpr int kBHalfBytes = (kBN / 2) * kBlockK * 2;  // 16 KB: this CTA's half of the B tile
constexpr int kStageBytes = kABytes + kBHalfBytes;
constexpr int kOutChunkCols = 64;
constexpr int kOutChunkBytes = kBlockM * kOutChunkCols * 2;
constexpr int kSmemBytes = kStages * kStageBytes + 2 * kOutChunkBytes + 1024 + 256;
constexpr int kThreads = 192;

struct PairBarriers {
  uint64_t full[8];
  uint64_t empty[8];
  uint64_t acc_full[2];
  uint64_t acc_empty[2];
  uint32_t tmem_base;
  uint32_t failed;
};

struct PairMaps {
  CUtensorMap a;    // box 128 rows x 64 columns
  CUtensorMap b;    // box 128 rows x 64 columns (half of the 256-row B tile)
  CUtensorMap out;  // box 128 rows x 64 columns
};

// Pair-tile `t` of the schedule: groups of `gm` 256-row tiles, n-major inside a group.
__device__ __forceinline__ void pair_tile_at(int t, int tiles_m, int tiles_n, int gm, int* pm, int* pn) {
  const int per_group = gm * tiles_n;
  const int group = t / per_group;
  const int first = group * gm;
  const int gsz = min(gm, tiles_m - first);
  const int rem = t - group * per_group;
  *pm = first + rem % gsz;
  *pn = rem / gsz;
}

__global__ void __launch_bounds__(kThreads, 1)
    k_gemm_pair(const __grid_constant__ PairMaps maps, int m, int n, int k, int gm, uint32_t* status) {
  constexpr uint32_t idesc = make_idesc_bf16(2 * kBlockM, kBN);
  extern __shared__ char smem_raw[];
  // The carve-up must be identical in both CTAs (the MMA addresses both with one descriptor).
  char* stages = reinterpret_cast<char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
  char* obuf = stages + kStages * kStageBytes;
  PairBarriers* bars = reinterpret_cast<PairBarriers*>(obuf + 2 * kOutChunkBytes);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t cta = cluster_ctarank();  // 0 leads
  const bool leader = cta == 0;
  const int cluster_id = blockIdx.x >> 1, nclusters = gridDim.x >> 1;
  const int tiles_m = (m + 2 * kBlockM - 1) / (2 * kBlockM), tiles_n = (n + kBN - 1) / kBN;
  const int total_tiles = tiles_m * tiles_n;
  const int k_iters = (k + kBlockK - 1) / kBlockK;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) {
      mbar_init(&bars->full[s], 1);
      mbar_init(&bars->empty[s], 1);
    }
    for (int s = 0; s < 2; ++s) {
      mbar_init(&bars->acc_full[s], 1);
      mbar_init(&bars->acc_empty[s], 8);  // four epilogue warps in each CTA of the pair
    }
    bars->failed = 0;
    fence_barrier_init();
  }
  if (warp == 1) {
    tmem_alloc_pair(&bars->tmem_base, 2 * kBN);
    tmem_relinquish_pair();
  }
  tc_fence_before_sync();
  __syncthreads();
  cluster_sync_all();  // both CTAs' barriers exist before anybody signals across
  tc_fence_after_sync();
  const uint32_t tmem_base = bars->tmem_base;

  if (warp == 0) {
    // ---------------- TMA producer (each CTA loads its own A rows and its half of B)
    if (lane == 0) {
      uint32_t it = 0;
      for (int t = cluster_id; t < total_tiles && !bars->failed; t += nclusters) {
        int pm, pn;
        pair_tile_at(t, tiles_m, tiles_n, gm, &pm, &pn);
        const int a_row = (pm * 2 + static_cast<int>(cta)) * kBlockM;
        const int b_row = pn * kBN + static_cast<int>(cta) * (kBN / 2);
        for (int kb = 0; kb < k_iters; ++kb, ++it) {
          const int s = it % kStages;
          const uint32_t ph = (it / kStages) & 1u;
          if (!mbar_wait(&bars->empty[s], ph ^ 1u)) {
            bars->failed = 1;
            break;
          }
          // The leader's barrier counts all four loads of the stage.
          if (leader) mbar_expect_tx(&bars->full[s], 2 * kStageBytes);
          char* sa = stages + s * kStageBytes;
          tma_load_2d_pair(sa, &maps.a, &bars->full[s], kb * kBlockK, a_row);
          tma_load_2d_pair(sa + kABytes, &maps.b, &bars->full[s], kb * kBlockK, b_row);
        }
      }
    }
  } else if (warp == 1) {
    // ---------------- MMA issuer (leader CTA only)
    if (leader && lane == 0) {
      uint32_t it = 0, tile_iter = 0;
      for (int t = cluster_id; t < total_tiles && !bars->failed; t += nclusters, ++tile_iter) {
        const uint32_t as = tile_iter & 1u, aph = (tile_iter >> 1) & 1u;
        if (!mbar_wait(&bars->acc_empty[as], aph ^ 1u)) {
          bars->failed = 1;
          break;
        }
        tc_fence_after_sync();
        const uint32_t tmem_acc = tmem_base + as * kBN;
        for (int kb = 0; kb < k_iters; ++kb, ++it) {
          const int s = it % kStages;
          const uint32_t ph = (it / kStages) & 1u;
          if (!mbar_wait(&bars->full[s], ph)) {
            bars->failed = 1;
            break;
          }
          tc_fence_after_sync();
          const uint32_t sa = smem_u32(stages + s * kStageBytes);
          const uint64_t da = make_smem_desc(sa), db = make_smem_desc(sa + kABytes);
#pragma unroll
          for (int kk = 0; kk < kBlockK / kUmmaK; ++kk) {
            umma_bf16_pair(tmem_acc, da + static_cast<uint64_t>(kk * 2), db + static_cast<uint64_t>(kk * 2), idesc, (kb | kk) != 0);
          }
          umma_commit_pair(&bars->empty[s], 3);  // both CTAs may refill the stage
        }
        umma_commit_pair(&bars->acc_full[as], 3);  // both CTAs' epilogues may read
      }
    }
  } else {
    // ---------------- epilogue (both CTAs, own 128 rows)
    const int q = warp & 3;
    const int row_in_tile = q * 32 + lane;
    const bool issuer = warp == 2 && lane == 0;
    uint32_t tile_iter = 0, chunk_iter = 0;
    for (int t = cluster_id; t < total_tiles; t += nclusters, ++tile_iter) {
      const uint32_t as = tile_iter & 1u, aph = (tile_iter >> 1) & 1u;
      int pm, pn;
      pair_tile_at(t, tiles_m, tiles_n, gm, &pm, &pn);
      if (!mbar_wait(&bars->acc_full[as], aph)) {
        bars->failed = 1;
        break;
      }
      tc_fence_after_sync();
      const int out_row = (pm * 2 + static_cast<int>(cta)) * kBlockM;
      for (int j = 0; j < kBN / kOutChunkCols; ++j, ++chunk_iter) {
        char* buf = obuf + (chunk_iter & 1u) * kOutChunkBytes;
        if (issuer) tma_store_wait_read<1>();
        asm volatile("bar.sync 1, 128;" ::: "memory");
#pragma unroll
        for (int half = 0; half < 2; ++half) {
          uint32_t r[32];
          tmem_ld_32x32(tmem_base + as * kBN + (static_cast<uint32_t>(q * 32) << 16) +
                            static_cast<uint32_t>(j * kOutChunkCols + half * 32),
                        r);
          tmem_ld_wait();
#pragma unroll
          for (int v = 0; v < 4; ++v) {
            const int chunk16 = half * 4 + v;
            uint4* dst = reinterpret_cast<uint4*>(buf + row_in_tile * 128 + ((chunk16 ^ (row_in_tile & 7)) << 4));
            *dst = make_uint4(pack_bf16(r[8 * v], r[8 * v + 1]), pack_bf16(r[8 * v + 2], r[8 * v + 3]),
                              pack_bf16(r[8 * v + 4], r[8 * v + 5]), pack_bf16(r[8 * v + 6], r[8 * v + 7]));
          }
        }
        if (j == kBN / kOutChunkCols - 1) {
          tc_fence_before_sync();
          __syncwarp();
          if (lane == 0) mbar_arrive_leader(&bars->acc_empty[as]);
        }
        fence_proxy_async_smem();
        asm volatile("bar.sync 1, 128;" ::: "memory");
        if (issuer && out_row < m && pn * kBN + j * kOutChunkCols < n) {
          tma_store_2d(&maps.out, buf, pn * kBN + j * kOutChunkCols, out_row);
          tma_store_commit();
        }
      }
    }
    if (issuer) tma_store_wait_all<0>();
  }

  tc_fence_before_sync();
  __syncthreads();
  cluster_sync_all();  // the peer may still be reading this CTA's shared memory / signalling its barriers
  if (warp == 1) {
    tmem_dealloc_pair(tmem_base, 2 * kBN);
  }
  if (threadIdx.x == 0 && bars->failed && status != nullptr) status[0] = status[0] | kStatusTimeout;
}

} // namespace

cudaError_t launch_gemm_bf16_nt_pair(const void* a, const void* b, void* c, int m, int n, int k, uint32_t* status,
                                     cudaStream_t stream) {
  if (m <= 0 || n <= 0 || k <= 0 || k % 8 != 0 || n % 8 != 0) return cudaErrorInvalidValue;
  if ((reinterpret_cast<uintptr_t>(a) | reinterpret_cast<uintptr_t>(b) | reinterpret_cast<uintptr_t>(c)) & 15u) {
    return cudaErrorInvalidValue;
  }
  PairMaps maps;
  if (!make_map(&maps.a, a, m, k, kBlockM) || !make_map(&maps.b, b, n, k, kBlockM) || !make_map(&maps.out, c, m, n, kBlockM)) return cudaErrorInvalidValue;
  cudaError_t e = cudaFuncSetAttribute(k_gemm_pair, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes);
  if (e != cudaSuccess) return e;
  const int tiles_m = (m + 2 * kBlockM - 1) / (2 * kBlockM), tiles_n = (n + kBN - 1) / kBN;
  cudaLaunchConfig_t cfg = {};
  cfg.blockDim = dim3(kThreads);
  cfg.dynamicSmemBytes = kSmemBytes;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 2;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  // As many pairs as the device can hold at once (each CTA fills an SM).
  int max_clusters = 0;
  cfg.gridDim = dim3(2);
  e = cudaOccupancyMaxActiveClusters(&max_clusters, k_gemm_pair, &cfg);
  if (e != cudaSuccess) return e;
  if (max_clusters < 1) return cudaErrorInvalidConfiguration;
  const int clusters = std::min(max_clusters, tiles_m * tiles_n);
  cfg.gridDim = dim3(2 * clusters);
  // A rows of a group stay in L2 while the pairs sweep over n: at most 8 pair-tiles and ~40 MB.
  const size_t a_tile_bytes = static_cast<size_t>(2 * kBlockM) * k * 2;
  const int gm = std::max(1, std::min({8, tiles_m, static_cast<int>((40u << 20) / std::max<size_t>(a_tile_bytes, 1))}));
  e = cudaLaunchKernelEx(&cfg, k_gemm_pair, maps, m, n, k, gm, status);
  note_kernel_launch();
  return e != cudaSuccess ? e : cudaGetLastError();
}

} // namespace b200c
