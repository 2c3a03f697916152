// tcgen05 / TMEM GEMM kernels (sm_100a). See tc_gemm.h.
//
// One persistent kernel, three modes (plain, all-gather -> GEMM, GEMM ->
// reduce-scatter). Roles inside a CTA:
//   warp 0, one lane : TMA producer - fills a ring of shared-memory stages
//   warp 1           : allocates tensor memory; one lane issues tcgen05.mma
//   warps 2..5       : epilogue - tcgen05.ld the fp32 accumulator, convert to
//                      bf16 into a swizzled staging tile, TMA-store it (each
//                      warp owns the 32 TMEM lanes of its warp-id % 4 quadrant)
//   warps 6..9       : all-gather mode only - copy the peers' rows
#include "tc_gemm.h"

#include <algorithm>
#include <cstdlib>
#include <string>

#include "launch_count.h"
#include "tc_gemm.cuh"

namespace b200c {

namespace {

using namespace tc;

// ------------------------------------------------------ shared layout ------

template <int BN>
struct TileCfg {
  static constexpr int kStages = BN == 256 ? 4 : 6;
  static constexpr int kABytes = kBlockM * kBlockK * 2;
  static constexpr int kBBytes = BN * kBlockK * 2;
  static constexpr int kStageBytes = kABytes + kBBytes;
};

// ------------------------------------------------- persistent kernel -------
//
// One CTA per SM; tiles are handed out round-robin in an order that (a) keeps
// a group of `gm` m-tiles resident in L2 while the wave sweeps over n, and
// (b) follows the data's arrival (all-gather) or departure (reduce-scatter).
// Control words of the fused modes (local global memory, zeroed once):
//   ctrl[0] call epoch, ctrl[1] finished-CTA ticket, ctrl[2] start flag,
//   ctrl[4 + i] arrival counter of m-tile ordinal i (all-gather mode).

constexpr int kTpBN = 256;
constexpr int kCopyThreads = 128;
constexpr int kGemmThreads = 192;
constexpr int kCtrlTiles = 4;
constexpr int kOutChunkCols = 64;                                  // one 128-byte swizzle row of bf16
constexpr int kOutChunkBytes = kBlockM * kOutChunkCols * 2;        // 16 KB
constexpr int kTpSmemBytes = TileCfg<kTpBN>::kStages * TileCfg<kTpBN>::kStageBytes + 2 * kOutChunkBytes + 1024 + 256;

enum class TpMode : int { PLAIN = 0, AG_GEMM = 1, GEMM_RS = 2 };

template <TpMode MODE>
constexpr int tp_threads() {
  return MODE == TpMode::PLAIN ? kGemmThreads : kGemmThreads + kCopyThreads;  // fused modes: four more warps (copy / reduce)
}

struct TpBarriers {
  uint64_t full[8];
  uint64_t empty[8];
  uint64_t acc_full[2];
  uint64_t acc_empty[2];
  uint32_t tmem_base;
  uint32_t failed;
  uint32_t epoch;
  uint32_t is_last;
  int reduce_ok;
  uint32_t fwd_ready;   // reduce-scatter: tiles for other ranks that the epilogue has put into the send staging
};

struct TpMaps {
  CUtensorMap a_local;          // A rows that are in this rank's own buffer
  CUtensorMap a_full;           // A rows in the gathered buffer (all-gather mode)
  CUtensorMap b;
  CUtensorMap b_half;           // box of 128 rows of B: what one CTA of a pair loads
  CUtensorMap out[kMaxRanks];   // [0]: y; reduce-scatter: [rank] = this rank's own receive staging
  CUtensorMap out_send;         // reduce-scatter: local staging [m, n] of the partial tiles bound for other ranks
};

struct TpParams {
  // all-gather mode
  const char* x_shards[kMaxRanks];
  char* x_full;
  // reduce-scatter mode
  const char* partials_local;
  char* partials[kMaxRanks];     // every owner's receive staging [nranks, m_local, n] (peer pointers)
  const char* send_stage;        // local [m_total, n] bf16
  uint32_t* arrived[kMaxRanks];
  __nv_bfloat16* out;
  // common
  uint32_t* ctrl;
  uint32_t* status;   // plain mode: where a failed wait is recorded (may be null)
  int m_total, m_local, n, k, gm;   // k in 16-bit units: K for bf16, K / 2 for e4m3
  // e4m3 operands: C = (row_scale[m] * col_scale[n]) * (A_q x B_q^T)
  int fp8;
  const float* scale_a;                     // [m_total] (plain, reduce-scatter)
  const float* scale_a_shards[kMaxRanks];   // all-gather: rank r's [m_local], symmetric
  float* scale_a_full;                      // all-gather: local [m_total], filled by the copy warps
  const float* scale_b;                     // [n]
};

// Row scale of global row `grow` of m-tile ordinal `ord` (see mtile_of).
template <TpMode MODE>
__device__ __forceinline__ float row_scale_of(const TpParams& p, const CommDev& c, int ord, int tiles_per_src, int grow) {
  if (grow >= p.m_total) return 0.0f;
  if (MODE == TpMode::AG_GEMM) {
    return ord < tiles_per_src ? p.scale_a_shards[c.rank][grow - c.rank * p.m_local] : __ldcg(p.scale_a_full + grow);
  }
  return p.scale_a[grow];
}

__device__ __forceinline__ uint32_t ld_acquire_gpu(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

// Polls `done()` until it holds, the communicator's wait budget (wall time)
// runs out, or the communicator has failed. False = gave up. The status word
// lives in host memory, so it is looked at only every 200 us of waiting.
template <typename Pred>
__device__ __forceinline__ bool poll_until(const CommDev& c, Pred done) {
  unsigned long long start = 0, next_check = 0;
  for (uint32_t spins = 0;; ++spins) {
    if (done()) return true;
    if ((spins & 255u) == 255u) {
      const unsigned long long now = globaltimer_ns();
      if (start == 0) {
        start = now;
        next_check = now + 200000ull;
      } else if (now >= next_check) {
        next_check = now + 200000ull;
        if (comm_is_dead(c) || now - start > c.timeout_ns) return false;
      }
    }
  }
}

// Cross-GPU barrier executed by ONE warp (lanes < nranks signal and poll).
__device__ __forceinline__ bool warp_rank_barrier(const CommDev& c, int row, uint32_t phase) {
  const int lane = threadIdx.x & 31;
  uint32_t* ep = &c.epochs[kFlagSetTp * kMaxBlocks + row];
  uint32_t v = 0;
  if (lane == 0) v = *ep + 1;
  v = __shfl_sync(0xffffffffu, v, 0);
  bool ok = true;
  if (lane < c.nranks) {
    __threadfence_system();
    st_relaxed_sys(flag_slot(c, lane, kFlagSetTp, row, c.rank), v);
    ok = wait_flag_reached(c, flag_slot(c, c.rank, kFlagSetTp, row, lane), v, lane, phase);
  }
  ok = __all_sync(0xffffffffu, ok);
  if (lane == 0) *ep = v;
  __syncwarp();
  return ok;
}

struct TileCoord {
  int ord;  // m-tile ordinal in schedule order
  int ni;
};

// Tile `t` of the schedule: groups of `gm` m-tile ordinals, n-major inside a
// group, so that CTAs working side by side share B tiles through L2 and the
// group's A rows stay resident while the wave moves along n.
__device__ __forceinline__ TileCoord tile_at(int t, int tiles_m, int tiles_n, int gm) {
  const int per_group = gm * tiles_n;
  const int group = t / per_group;
  const int first = group * gm;
  const int gsz = min(gm, tiles_m - first);
  const int rem = t - group * per_group;
  return TileCoord{first + rem % gsz, rem / gsz};
}

// Traffic that is touched once (staged tiles on their way to the owner, the slots the owner sums): marked
// evict-first so that it does not push the GEMM's operand tiles out of L2.
__device__ __forceinline__ uint4 ld16_once(const void* p) {
  uint4 v;
  asm volatile("ld.global.cs.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
  return v;
}
__device__ __forceinline__ void st16_once(void* p, uint4 v) {
  asm volatile("st.global.cs.v4.u32 [%0], {%1,%2,%3,%4};" ::"l"(p), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
}

// Like wait_flag_reached, for warps that share an SM with the GEMM pipeline: sleeps between polls so that the
// polling does not take issue slots from the producer, MMA and epilogue warps.
__device__ __forceinline__ bool wait_flag_quietly(const CommDev& c, const uint32_t* addr, uint32_t want, int peer, uint32_t phase) {
  unsigned long long start = 0, next_status = 0;
  while (true) {
    const uint32_t v = ld_relaxed_sys(addr);
    if (static_cast<int32_t>(v - want) >= 0) {
      fence_acq_rel_sys();
      return true;
    }
    __nanosleep(200);
    const unsigned long long now = globaltimer_ns();
    if (start == 0) {
      start = now;
      next_status = now + 200000ull;
    } else if (now >= next_status) {
      next_status = now + 200000ull;
      if (comm_is_dead(c)) return false;
      if (now - start > c.timeout_ns) {
        report_timeout(c, peer, phase);
        return false;
      }
    }
  }
}

// Sum of the `nslots` partial copies of one 128 x BN tile (bf16, fp32 accumulation) into `out`.
// Every thread keeps U vectors of S slots in flight (U x S 16-byte loads): with four reduce warps per SM
// it takes that many to run at memory speed rather than at the latency of a load.
template <int BN, int U, int S>
__device__ __forceinline__ void reduce_tile(const __nv_bfloat16* __restrict__ base, __nv_bfloat16* __restrict__ out, int wm, int ni,
                                            int n, size_t slot_elems, int nslots, int tid, int nthreads) {
  constexpr int kVecs = kBlockM * BN / 8;  // vectors of 8 bf16 in the tile
  for (int v0 = tid; v0 < kVecs; v0 += nthreads * U) {
    size_t off[U];
    float acc[U][8];
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const int v = v0 + u * nthreads;
      const int r = v / (BN / 8), cv = v % (BN / 8);
      off[u] = (static_cast<size_t>(wm * kBlockM + r)) * n + ni * BN + cv * 8;
#pragma unroll
      for (int i = 0; i < 8; ++i) acc[u][i] = 0.0f;
    }
    for (int s0 = 0; s0 < nslots; s0 += S) {
      uint4 q[S][U];
#pragma unroll
      for (int j = 0; j < S; ++j) {
#pragma unroll
        for (int u = 0; u < U; ++u) {
          if (s0 + j < nslots && v0 + u * nthreads < kVecs) {
            q[j][u] = ld16_once(base + static_cast<size_t>(s0 + j) * slot_elems + off[u]);
          } else {
            q[j][u] = make_uint4(0u, 0u, 0u, 0u);
          }
        }
      }
#pragma unroll
      for (int j = 0; j < S; ++j) {
#pragma unroll
        for (int u = 0; u < U; ++u) {
          const uint32_t* pw = &q[j][u].x;
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            acc[u][2 * i] += __uint_as_float(pw[i] << 16);
            acc[u][2 * i + 1] += __uint_as_float(pw[i] & 0xffff0000u);
          }
        }
      }
    }
#pragma unroll
    for (int u = 0; u < U; ++u) {
      if (v0 + u * nthreads < kVecs) {
        uint4 o;
        uint32_t* po = &o.x;
#pragma unroll
        for (int i = 0; i < 4; ++i) po[i] = pack_bf16(__float_as_uint(acc[u][2 * i]), __float_as_uint(acc[u][2 * i + 1]));
        st16_once(out + off[u], o);
      }
    }
  }
}

// Forward warps of the reduce-scatter: copy one 128 x BN bf16 tile from the local send staging (rows `src_row0`..
// of a [*, n] matrix) to the owner's receive staging (rows `dst_row0`.. of its [*, n] matrix) with plain 16-byte
// stores over NVLink, 8 per thread in flight.
template <int BN>
__device__ __forceinline__ void forward_tile(const char* __restrict__ src, char* __restrict__ dst, int src_row0, int dst_row0,
                                             int col0, int n, int tid, int nthreads) {
  constexpr int kVecs = kBlockM * BN / 8;
  constexpr int U = 8;
  for (int v0 = tid; v0 < kVecs; v0 += nthreads * U) {
    uint4 q[U];
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const int v = v0 + u * nthreads;
      if (v < kVecs) {
        const int r = v / (BN / 8), cv = v % (BN / 8);
        q[u] = ld16_once(src + ((static_cast<size_t>(src_row0 + r)) * n + col0 + cv * 8) * 2);
      }
    }
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const int v = v0 + u * nthreads;
      if (v < kVecs) {
        const int r = v / (BN / 8), cv = v % (BN / 8);
        st16(dst + ((static_cast<size_t>(dst_row0 + r)) * n + col0 + cv * 8) * 2, q[u]);
      }
    }
  }
}

// Waits (bounded, sleeping between polls) until the epilogue has handed over `want` tiles. One thread calls it.
__device__ __forceinline__ bool wait_fwd_ready(const CommDev& c, TpBarriers* bars, uint32_t want) {
  volatile uint32_t* ready = &bars->fwd_ready;
  volatile uint32_t* failed = &bars->failed;
  unsigned long long start = 0;
  while (true) {
    if (*failed != 0) return false;
    if (*ready >= want) return true;
    __nanosleep(200);
    const unsigned long long now = globaltimer_ns();
    if (start == 0) {
      start = now;
    } else if (now - start > kLocalWaitNs) {
      return false;
    }
  }
}

// Phase stamps of the fused kernels (CommDev::trace, one row per CTA, nanoseconds of this GPU's timer):
// 0 start, 1 last tile's loads issued, 2 last MMA committed, 3 last tile stored (and flagged), 4 copy warps
// done (all-gather) or forward warps done (reduce-scatter), 5 first own tile complete on every rank (reduce-scatter), 6 reduce warps done, 7 CTA done,
// 8 closing cross-GPU barrier passed (last CTA only).
// Body of the single-CTA kernels. `maps` must live in kernel-parameter,
// constant or global memory (its address goes to TMA).
template <TpMode MODE, bool FP8>
__device__ __forceinline__ void tp_gemm_body(const TpMaps& maps, const CommDev& c, const TpParams& p) {
  using Cfg = TileCfg<kTpBN>;
  constexpr int BN = kTpBN;
  constexpr uint32_t idesc = FP8 ? make_idesc_e4m3(kBlockM, BN) : make_idesc_bf16(kBlockM, BN);
  constexpr bool kFused = MODE != TpMode::PLAIN;
  extern __shared__ char smem_raw[];
  char* stages = reinterpret_cast<char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
  char* obuf = stages + Cfg::kStages * Cfg::kStageBytes;
  TpBarriers* bars = reinterpret_cast<TpBarriers*>(obuf + 2 * kOutChunkBytes);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int G = gridDim.x;
  const int tiles_m = (p.m_total + kBlockM - 1) / kBlockM, tiles_n = (p.n + BN - 1) / BN;
  const int tiles_per_src = kFused ? p.m_local / kBlockM : tiles_m;
  const int total_tiles = tiles_m * tiles_n;
  const int k_iters = (p.k + kBlockK - 1) / kBlockK;

  if (threadIdx.x == 0) {
    for (int s = 0; s < Cfg::kStages; ++s) {
      mbar_init(&bars->full[s], 1);
      mbar_init(&bars->empty[s], 1);
    }
    for (int s = 0; s < 2; ++s) {
      mbar_init(&bars->acc_full[s], 1);
      mbar_init(&bars->acc_empty[s], 4);  // one arrival per epilogue warp
    }
    bars->failed = 0;
    bars->is_last = 0;
    bars->fwd_ready = 0;
    bars->epoch = kFused ? ld_acquire_gpu(&p.ctrl[0]) : 0u;
    fence_barrier_init();
  }
  if (warp == 1) {
    tmem_alloc(&bars->tmem_base, 2 * BN);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = bars->tmem_base;
  const uint32_t epoch = bars->epoch;  // calls completed before this one
  if (kFused && threadIdx.x == 0) trace_stamp_ns(c, 0);

  // m-tile ordinal -> real m-tile. All-gather: own rows first, then the
  // sources in ring order (the order in which the copy warps fetch them).
  // Reduce-scatter: the next rank's rows first, own rows last.
  auto mtile_of = [&](int ord) {
    if (!kFused) return ord;
    const int j = ord / tiles_per_src, w = ord % tiles_per_src;
    const int src = MODE == TpMode::AG_GEMM ? (c.rank + j) % c.nranks : (c.rank + 1 + j) % c.nranks;
    return src * tiles_per_src + w;
  };

  if (warp == 0) {
    // ---------------- TMA producer
    if (lane == 0) {
      uint32_t it = 0;
      for (int t = blockIdx.x; t < total_tiles && !bars->failed; t += G) {
        const TileCoord tc_ = tile_at(t, tiles_m, tiles_n, p.gm);
        const int ord = tc_.ord, ni = tc_.ni;
        const int mi = mtile_of(ord);
        const CUtensorMap* ma = &maps.a_local;
        int a_row = mi * kBlockM;
        if (MODE == TpMode::AG_GEMM) {
          if (ord < tiles_per_src) {
            a_row = (mi - c.rank * tiles_per_src) * kBlockM;
          } else {
            ma = &maps.a_full;
            // Rows of a peer: wait until every CTA's copy warps delivered their slice.
            const uint32_t want = (epoch + 1) * static_cast<uint32_t>(G);
            const bool ok = poll_until(c, [&]() {
              return static_cast<int32_t>(ld_acquire_gpu(&p.ctrl[kCtrlTiles + ord]) - want) >= 0;
            });
            if (!ok) {
              bars->failed = 1;
              break;
            }
            fence_proxy_async();  // written with ordinary stores, read by TMA through the async proxy
          }
        }
        for (int kb = 0; kb < k_iters; ++kb, ++it) {
          const int s = it % Cfg::kStages;
          const uint32_t ph = (it / Cfg::kStages) & 1u;
          if (!mbar_wait(&bars->empty[s], ph ^ 1u)) {
            bars->failed = 1;
            break;
          }
          mbar_expect_tx(&bars->full[s], Cfg::kStageBytes);
          char* sa = stages + s * Cfg::kStageBytes;
          tma_load_2d(sa, ma, &bars->full[s], kb * kBlockK, a_row);
          tma_load_2d(sa + Cfg::kABytes, &maps.b, &bars->full[s], kb * kBlockK, ni * BN);
        }
      }
      if (kFused) trace_stamp_ns(c, 1);
    }
  } else if (warp == 1) {
    // ---------------- MMA issuer
    if (lane == 0) {
      uint32_t it = 0, tile_iter = 0;
      for (int t = blockIdx.x; t < total_tiles && !bars->failed; t += G, ++tile_iter) {
        const uint32_t as = tile_iter & 1u, aph = (tile_iter >> 1) & 1u;
        if (!mbar_wait(&bars->acc_empty[as], aph ^ 1u)) {
          bars->failed = 1;
          break;
        }
        tc_fence_after_sync();
        const uint32_t tmem_acc = tmem_base + as * BN;
        for (int kb = 0; kb < k_iters; ++kb, ++it) {
          const int s = it % Cfg::kStages;
          const uint32_t ph = (it / Cfg::kStages) & 1u;
          if (!mbar_wait(&bars->full[s], ph)) {
            bars->failed = 1;
            break;
          }
          tc_fence_after_sync();
          const uint32_t sa = smem_u32(stages + s * Cfg::kStageBytes);
          const uint64_t da = make_smem_desc(sa), db = make_smem_desc(sa + Cfg::kABytes);
#pragma unroll
          for (int kk = 0; kk < kBlockK / kUmmaK; ++kk) {
            // 16 bf16 (or 32 e4m3) = 32 bytes further along K inside the swizzled row
            if (FP8) {
              umma_f8(tmem_acc, da + static_cast<uint64_t>(kk * 2), db + static_cast<uint64_t>(kk * 2), idesc, (kb | kk) != 0);
            } else {
              umma_bf16(tmem_acc, da + static_cast<uint64_t>(kk * 2), db + static_cast<uint64_t>(kk * 2), idesc, (kb | kk) != 0);
            }
          }
          umma_commit(&bars->empty[s]);  // stage reusable once these MMAs have read it
        }
        umma_commit(&bars->acc_full[as]);  // accumulator complete
      }
      if (kFused) trace_stamp_ns(c, 2);
    }
  } else if (warp < 6) {
    // ---------------- epilogue: TMEM -> bf16 -> swizzled staging -> TMA store
    const int q = warp & 3;
    const int row_in_tile = q * 32 + lane;
    const bool issuer = warp == 2 && lane == 0;
    uint32_t tile_iter = 0, chunk_iter = 0;
    for (int t = blockIdx.x; t < total_tiles; t += G, ++tile_iter) {
      const uint32_t as = tile_iter & 1u, aph = (tile_iter >> 1) & 1u;
      const TileCoord tc_ = tile_at(t, tiles_m, tiles_n, p.gm);
      const int ni = tc_.ni;
      const int mi = mtile_of(tc_.ord);
      if (!mbar_wait(&bars->acc_full[as], aph)) {
        bars->failed = 1;
        break;
      }
      tc_fence_after_sync();
      const float row_scale = FP8 ? row_scale_of<MODE>(p, c, tc_.ord, tiles_per_src, mi * kBlockM + row_in_tile) : 1.0f;
      const CUtensorMap* mo = &maps.out[0];
      int out_row = mi * kBlockM;
      int owner = 0;
      if (MODE == TpMode::GEMM_RS) {
        owner = mi / tiles_per_src;
        if (owner == c.rank) {
          // own rows: straight into slot `rank` of this rank's receive staging, viewed as [nranks * m_local, n]
          mo = &maps.out[c.rank];
          out_row = c.rank * p.m_local + (mi - owner * tiles_per_src) * kBlockM;
        } else {
          // another rank's rows: into the local send staging (a TMA store into peer memory drains far too
          // slowly to keep up with the tensor cores); the forward warps move the tile on with plain stores
          mo = &maps.out_send;
        }
      }
      for (int j = 0; j < BN / kOutChunkCols; ++j, ++chunk_iter) {
        char* buf = obuf + (chunk_iter & 1u) * kOutChunkBytes;
        // The store that read this buffer two chunks ago has drained it.
        if (issuer) tma_store_wait_read<1>();
        asm volatile("bar.sync 1, 128;" ::: "memory");
#pragma unroll
        for (int half = 0; half < 2; ++half) {
          uint32_t r[32];
          tmem_ld_32x32(tmem_base + as * BN + (static_cast<uint32_t>(q * 32) << 16) +
                            static_cast<uint32_t>(j * kOutChunkCols + half * 32),
                        r);
          tmem_ld_wait();
          if (FP8) scale_acc32(r, row_scale, p.scale_b, ni * BN + j * kOutChunkCols + half * 32, p.n);
#pragma unroll
          for (int v = 0; v < 4; ++v) {
            const int chunk16 = half * 4 + v;
            uint4* dst = reinterpret_cast<uint4*>(buf + row_in_tile * 128 + ((chunk16 ^ (row_in_tile & 7)) << 4));
            *dst = make_uint4(pack_bf16(r[8 * v], r[8 * v + 1]), pack_bf16(r[8 * v + 2], r[8 * v + 3]),
                              pack_bf16(r[8 * v + 4], r[8 * v + 5]), pack_bf16(r[8 * v + 6], r[8 * v + 7]));
          }
        }
        if (j == BN / kOutChunkCols - 1) {
          // Accumulator fully read: the MMA warp may reuse this TMEM stage.
          tc_fence_before_sync();
          __syncwarp();
          if (lane == 0) mbar_arrive(&bars->acc_empty[as]);
        }
        fence_proxy_async_smem();
        asm volatile("bar.sync 1, 128;" ::: "memory");
        if (issuer && ni * BN + j * kOutChunkCols < p.n) {  // chunks wholly past the last column are skipped
          tma_store_2d(mo, buf, ni * BN + j * kOutChunkCols, out_row);
          tma_store_commit();
        }
      }
      if (MODE == TpMode::GEMM_RS && issuer) {
        // The tile's four stores have landed (local memory either way).
        tma_store_wait_all<0>();
        if (owner == c.rank) {
          __threadfence_system();
          const int tile_local = (mi - owner * tiles_per_src) * tiles_n + ni;
          st_relaxed_sys(p.arrived[owner] + static_cast<size_t>(tile_local) * c.nranks + c.rank, epoch + 1);
        } else {
          __threadfence();
          atomicAdd(&bars->fwd_ready, 1u);   // hand the tile to the forward warps
        }
      }
    }
    if (issuer) {
      tma_store_wait_all<0>();
      trace_stamp_ns(c, 3);
    }
  } else {
    // ---------------- copy warps (all-gather mode): fetch the peers' shards
    if (MODE == TpMode::AG_GEMM) {
      const int ct = threadIdx.x - kGemmThreads;
      if (blockIdx.x == 0 && warp == 6) {
        // Everybody's shard is written before anybody reads it.
        const bool ok = warp_rank_barrier(c, 0, 0xa1);
        if (lane == 0) {
          __threadfence();
          atomicExch(&p.ctrl[2], ok ? epoch + 1 : 0xffffffffu);
        }
      }
      if (ct == 0) {
        bool started = false;
        poll_until(c, [&]() {
          const uint32_t v = ld_acquire_gpu(&p.ctrl[2]);
          if (v == epoch + 1) started = true;
          return started || v == 0xffffffffu;
        });
        if (!started) bars->failed = 1;
      }
      asm volatile("bar.sync 2, 128;" ::: "memory");
      const size_t tile_bytes = static_cast<size_t>(kBlockM) * p.k * 2;
      const size_t slice = ((tile_bytes + G - 1) / G + 15) / 16 * 16;
      const size_t b0 = static_cast<size_t>(blockIdx.x) * slice;
      for (int ord = tiles_per_src; ord < tiles_m; ++ord) {
        const int mi = mtile_of(ord);
        const int src = mi / tiles_per_src;
        const size_t src_off = static_cast<size_t>(mi - src * tiles_per_src) * tile_bytes;
        if (b0 < tile_bytes) {
          const size_t nbytes = tile_bytes - b0 < slice ? tile_bytes - b0 : slice;
          const uint4* from = reinterpret_cast<const uint4*>(p.x_shards[src] + src_off + b0);
          uint4* to = reinterpret_cast<uint4*>(p.x_full + static_cast<size_t>(mi) * tile_bytes + b0);
          const size_t nvec = nbytes / 16;
          size_t i = ct;
          for (; i + 3 * kCopyThreads < nvec; i += 4 * kCopyThreads) {
            const uint4 v0 = from[i], v1 = from[i + kCopyThreads], v2 = from[i + 2 * kCopyThreads], v3 = from[i + 3 * kCopyThreads];
            to[i] = v0;
            to[i + kCopyThreads] = v1;
            to[i + 2 * kCopyThreads] = v2;
            to[i + 3 * kCopyThreads] = v3;
          }
          for (; i < nvec; i += kCopyThreads) to[i] = from[i];
          fence_proxy_async();  // these rows are read next by TMA (async proxy)
        }
        if (FP8 && blockIdx.x == 0 && ct < kBlockM) {  // the tile's row scales travel with it
          p.scale_a_full[mi * kBlockM + ct] = p.scale_a_shards[src][(mi - src * tiles_per_src) * kBlockM + ct];
        }
        asm volatile("bar.sync 2, 128;" ::: "memory");
        if (ct == 0) {
          __threadfence();
          atomicAdd(&p.ctrl[kCtrlTiles + ord], 1u);
        }
      }
      if (ct == 0) trace_stamp_ns(c, 4);
    }
    // ---------------- reduce warps (reduce-scatter mode): sum the nranks partial tiles of this rank's
    // rows as they arrive, in the order in which this rank produces its own (last) contribution, while
    // the tensor cores are still busy with the remaining tiles.
    if (MODE == TpMode::GEMM_RS) {
      const int ct = threadIdx.x - kGemmThreads;
      const int my_tiles = tiles_per_src * tiles_n;
      const int first_own = (c.nranks - 1) * tiles_per_src;   // ordinal of this rank's first own m-tile
      // First the tiles this CTA computes for other ranks (they come first in the schedule): as soon as the
      // epilogue has put one into the send staging, move it into its owner's receive staging and flag it.
      uint32_t handed = 0;
      bool fwd_ok = true;
      for (int t = blockIdx.x; t < first_own * tiles_n && fwd_ok; t += G) {
        const TileCoord tc_ = tile_at(t, tiles_m, tiles_n, p.gm);
        const int mi = mtile_of(tc_.ord), ni = tc_.ni;
        const int owner = mi / tiles_per_src;
        ++handed;
        if (ct == 0) bars->reduce_ok = wait_fwd_ready(c, bars, handed) ? 1 : 0;
        asm volatile("bar.sync 2, 128;" ::: "memory");
        fwd_ok = bars->reduce_ok != 0;
        if (fwd_ok) {
          const int local_row = (mi - owner * tiles_per_src) * kBlockM;
          forward_tile<BN>(p.send_stage, p.partials[owner], mi * kBlockM, c.rank * p.m_local + local_row, ni * BN, p.n, ct,
                           kCopyThreads);
        }
        asm volatile("bar.sync 2, 128;" ::: "memory");
        if (fwd_ok && ct == 0) {
          __threadfence_system();
          const int tile_local = (mi - owner * tiles_per_src) * tiles_n + ni;
          st_relaxed_sys(p.arrived[owner] + static_cast<size_t>(tile_local) * c.nranks + c.rank, epoch + 1);
        }
      }
      if (ct == 0) {
        if (!fwd_ok) bars->failed = 1;
        trace_stamp_ns(c, 4);
      }
      for (int t_own = blockIdx.x; t_own < my_tiles; t_own += G) {
        const TileCoord tc_ = tile_at(first_own * tiles_n + t_own, tiles_m, tiles_n, p.gm);
        const int wm = tc_.ord - first_own, ni = tc_.ni;
        if (ct == 0) bars->reduce_ok = 1;
        asm volatile("bar.sync 2, 128;" ::: "memory");
        if (ct < c.nranks) {
          const uint32_t* flag = p.arrived[c.rank] + static_cast<size_t>(wm * tiles_n + ni) * c.nranks + ct;
          if (!wait_flag_quietly(c, flag, epoch + 1, ct, 0xa3)) bars->reduce_ok = 0;
        }
        asm volatile("bar.sync 2, 128;" ::: "memory");
        if (!bars->reduce_ok) {
          if (ct == 0) bars->failed = 1;
          break;
        }
        if (ct == 0 && t_own < G) trace_stamp_ns(c, 5);
        const __nv_bfloat16* base = reinterpret_cast<const __nv_bfloat16*>(p.partials_local);
        reduce_tile<BN, 4, 4>(base, p.out, wm, ni, p.n, static_cast<size_t>(p.m_local) * p.n, c.nranks, ct, kCopyThreads);
        asm volatile("bar.sync 2, 128;" ::: "memory");
      }
      if (ct == 0) trace_stamp_ns(c, 6);
    }
  }

  tc_fence_before_sync();
  __syncthreads();

  // ---------------- teardown. Fused modes: the last CTA to finish advances
  // the epoch and joins the closing cross-GPU barrier.
  __syncthreads();
  if (warp == 1) {
    tmem_dealloc(tmem_base, 2 * BN);
  }
  if (!kFused) {
    if (threadIdx.x == 0 && bars->failed && p.status != nullptr) p.status[0] = p.status[0] | kStatusTimeout;
    return;
  }
  if (threadIdx.x == 0) {
    trace_stamp_ns(c, 7);
    if (bars->failed) c.status[0] = c.status[0] | kStatusTimeout;
    __threadfence();
    const uint32_t ticket = atomicAdd(&p.ctrl[1], 1u);
    bars->is_last = ticket == static_cast<uint32_t>(G - 1) ? 1u : 0u;
  }
  __syncthreads();
  if (bars->is_last && warp == 0) {
    __threadfence();
    warp_rank_barrier(c, 1, 0xa2);
    if (lane == 0) {
      trace_stamp_ns(c, 8);
      p.ctrl[1] = 0;
      __threadfence();
      atomicExch(&p.ctrl[0], epoch + 1);
    }
  }
}

template <TpMode MODE, bool FP8>
__global__ void __launch_bounds__(tp_threads<MODE>(), 1) k_tp_gemm(const __grid_constant__ TpMaps maps, CommDev c, TpParams p) {
  tp_gemm_body<MODE, FP8>(maps, c, p);
}

// Several ranks in ONE launch on one GPU (tests): blockIdx.y is the rank, each
// rank gets gridDim.x CTAs, and the launch is cooperative so that all of them
// are resident while they wait on one another.
constexpr int kTpEmuRanks = 4;
struct TpEmu {
  TpMaps maps[kTpEmuRanks];
  CommDev c[kTpEmuRanks];
  TpParams p[kTpEmuRanks];
};

template <TpMode MODE, bool FP8>
__global__ void __launch_bounds__(tp_threads<MODE>(), 1) k_tp_gemm_emu(const __grid_constant__ TpEmu e) {
  tp_gemm_body<MODE, FP8>(e.maps[blockIdx.y], e.c[blockIdx.y], e.p[blockIdx.y]);
}

// ------------------------------------- fused kernels on CTA pairs ----------
//
// Same protocol as k_tp_gemm, with the mainloop of the pair GEMM (clusters of
// two CTAs, tcgen05 cta_group::2, 256 x 256 tile per pair, 6-stage ring of
// 32 KB per CTA). A pair takes two consecutive 128-row m-tiles of ONE source
// rank (the launcher requires m_local % 256 == 0), CTA r of the pair owns the
// r-th of them: its A rows, its epilogue, its flags. Everything that concerns
// peers - copy warps, arrival counters, partial-tile flags, the reduce phase,
// the epoch and the closing barrier - stays per CTA exactly as above.

constexpr int kPairStages = 6;
constexpr int kPairStageBytes = kBlockM * kBlockK * 2 + (kTpBN / 2) * kBlockK * 2;  // 16 KB of A + 16 KB of B
constexpr int kPairSmemBytes = kPairStages * kPairStageBytes + 2 * kOutChunkBytes + 1024 + 256;

template <TpMode MODE, bool FP8>
__global__ void __launch_bounds__(tp_threads<MODE>(), 1) k_tp_gemm_pair(const __grid_constant__ TpMaps maps, CommDev c, TpParams p) {
  constexpr int BN = kTpBN;
  constexpr int kAB = kBlockM * kBlockK * 2;
  constexpr uint32_t idesc = FP8 ? make_idesc_e4m3(2 * kBlockM, BN) : make_idesc_bf16(2 * kBlockM, BN);
  extern __shared__ char smem_raw[];
  char* stages = reinterpret_cast<char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
  char* obuf = stages + kPairStages * kPairStageBytes;
  TpBarriers* bars = reinterpret_cast<TpBarriers*>(obuf + 2 * kOutChunkBytes);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int cta = static_cast<int>(cluster_ctarank());  // 0 leads
  const bool leader = cta == 0;
  const int G = gridDim.x;
  const int cluster_id = blockIdx.x >> 1, nclusters = gridDim.x >> 1;
  const int tiles_m = p.m_total / kBlockM, tiles_n = p.n / BN, tiles_per_src = p.m_local / kBlockM;
  const int pair_tiles_m = tiles_m / 2;
  const int total_tiles = pair_tiles_m * tiles_n;
  const int k_iters = p.k / kBlockK;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kPairStages; ++s) {
      mbar_init(&bars->full[s], 1);
      mbar_init(&bars->empty[s], 1);
    }
    for (int s = 0; s < 2; ++s) {
      mbar_init(&bars->acc_full[s], 1);
      mbar_init(&bars->acc_empty[s], 8);  // four epilogue warps in each CTA of the pair
    }
    bars->failed = 0;
    bars->is_last = 0;
    bars->fwd_ready = 0;
    bars->epoch = ld_acquire_gpu(&p.ctrl[0]);
    fence_barrier_init();
  }
  if (warp == 1) {
    tmem_alloc_pair(&bars->tmem_base, 2 * BN);
    tmem_relinquish_pair();
  }
  tc_fence_before_sync();
  __syncthreads();
  cluster_sync_all();
  tc_fence_after_sync();
  const uint32_t tmem_base = bars->tmem_base;
  const uint32_t epoch = bars->epoch;
  if (threadIdx.x == 0) trace_stamp_ns(c, 0);

  // 128-row m-tile ordinal -> real m-tile (same order as k_tp_gemm).
  auto mtile_of = [&](int ord) {
    const int j = ord / tiles_per_src, w = ord % tiles_per_src;
    const int src = MODE == TpMode::AG_GEMM ? (c.rank + j) % c.nranks : (c.rank + 1 + j) % c.nranks;
    return src * tiles_per_src + w;
  };
  // Pair tile t -> this CTA's m-tile ordinal and the n-tile.
  auto my_tile = [&](int t, int* ord, int* ni) {
    const TileCoord tc_ = tile_at(t, pair_tiles_m, tiles_n, p.gm);
    *ord = tc_.ord * 2 + cta;
    *ni = tc_.ni;
  };

  if (warp == 0) {
    // ---------------- TMA producer: own A rows, own half of the B tile
    if (lane == 0) {
      uint32_t it = 0;
      for (int t = cluster_id; t < total_tiles && !bars->failed; t += nclusters) {
        int ord, ni;
        my_tile(t, &ord, &ni);
        const int mi = mtile_of(ord);
        const CUtensorMap* ma = &maps.a_local;
        int a_row = mi * kBlockM;
        if (MODE == TpMode::AG_GEMM) {
          if (ord < tiles_per_src) {
            a_row = (mi - c.rank * tiles_per_src) * kBlockM;
          } else {
            ma = &maps.a_full;
            const uint32_t want = (epoch + 1) * static_cast<uint32_t>(G);
            const bool ok = poll_until(c, [&]() {
              return static_cast<int32_t>(ld_acquire_gpu(&p.ctrl[kCtrlTiles + ord]) - want) >= 0;
            });
            if (!ok) {
              bars->failed = 1;
              break;
            }
            fence_proxy_async();
          }
        }
        const int b_row = ni * BN + cta * (BN / 2);
        for (int kb = 0; kb < k_iters; ++kb, ++it) {
          const int s = it % kPairStages;
          const uint32_t ph = (it / kPairStages) & 1u;
          if (!mbar_wait(&bars->empty[s], ph ^ 1u)) {
            bars->failed = 1;
            break;
          }
          if (leader) mbar_expect_tx(&bars->full[s], 2 * kPairStageBytes);  // all four loads of the stage
          char* sa = stages + s * kPairStageBytes;
          tma_load_2d_pair(sa, ma, &bars->full[s], kb * kBlockK, a_row);
          tma_load_2d_pair(sa + kAB, &maps.b_half, &bars->full[s], kb * kBlockK, b_row);
        }
      }
      trace_stamp_ns(c, 1);
    }
  } else if (warp == 1) {
    // ---------------- MMA issuer (leader only)
    if (leader && lane == 0) {
      uint32_t it = 0, tile_iter = 0;
      for (int t = cluster_id; t < total_tiles && !bars->failed; t += nclusters, ++tile_iter) {
        const uint32_t as = tile_iter & 1u, aph = (tile_iter >> 1) & 1u;
        if (!mbar_wait(&bars->acc_empty[as], aph ^ 1u)) {
          bars->failed = 1;
          break;
        }
        tc_fence_after_sync();
        const uint32_t tmem_acc = tmem_base + as * BN;
        for (int kb = 0; kb < k_iters; ++kb, ++it) {
          const int s = it % kPairStages;
          const uint32_t ph = (it / kPairStages) & 1u;
          if (!mbar_wait(&bars->full[s], ph)) {
            bars->failed = 1;
            break;
          }
          tc_fence_after_sync();
          const uint32_t sa = smem_u32(stages + s * kPairStageBytes);
          const uint64_t da = make_smem_desc(sa), db = make_smem_desc(sa + kAB);
#pragma unroll
          for (int kk = 0; kk < kBlockK / kUmmaK; ++kk) {
            if (FP8) {
              umma_f8_pair(tmem_acc, da + static_cast<uint64_t>(kk * 2), db + static_cast<uint64_t>(kk * 2), idesc, (kb | kk) != 0);
            } else {
              umma_bf16_pair(tmem_acc, da + static_cast<uint64_t>(kk * 2), db + static_cast<uint64_t>(kk * 2), idesc, (kb | kk) != 0);
            }
          }
          umma_commit_pair(&bars->empty[s], 3);
        }
        umma_commit_pair(&bars->acc_full[as], 3);
      }
      trace_stamp_ns(c, 2);
    }
  } else if (warp < 6) {
    // ---------------- epilogue (both CTAs, own 128 rows)
    const int q = warp & 3;
    const int row_in_tile = q * 32 + lane;
    const bool issuer = warp == 2 && lane == 0;
    uint32_t tile_iter = 0, chunk_iter = 0;
    for (int t = cluster_id; t < total_tiles; t += nclusters, ++tile_iter) {
      const uint32_t as = tile_iter & 1u, aph = (tile_iter >> 1) & 1u;
      int ord, ni;
      my_tile(t, &ord, &ni);
      const int mi = mtile_of(ord);
      if (!mbar_wait(&bars->acc_full[as], aph)) {
        bars->failed = 1;
        break;
      }
      tc_fence_after_sync();
      const float row_scale = FP8 ? row_scale_of<MODE>(p, c, ord, tiles_per_src, mi * kBlockM + row_in_tile) : 1.0f;
      const CUtensorMap* mo = &maps.out[0];
      int out_row = mi * kBlockM;
      int owner = 0;
      if (MODE == TpMode::GEMM_RS) {
        owner = mi / tiles_per_src;
        if (owner == c.rank) {
          mo = &maps.out[c.rank];
          out_row = c.rank * p.m_local + (mi - owner * tiles_per_src) * kBlockM;
        } else {
          mo = &maps.out_send;   // forwarded by the forward warps, see k_tp_gemm
        }
      }
      for (int j = 0; j < BN / kOutChunkCols; ++j, ++chunk_iter) {
        char* buf = obuf + (chunk_iter & 1u) * kOutChunkBytes;
        if (issuer) tma_store_wait_read<1>();
        asm volatile("bar.sync 1, 128;" ::: "memory");
#pragma unroll
        for (int half = 0; half < 2; ++half) {
          uint32_t r[32];
          tmem_ld_32x32(tmem_base + as * BN + (static_cast<uint32_t>(q * 32) << 16) +
                            static_cast<uint32_t>(j * kOutChunkCols + half * 32),
                        r);
          tmem_ld_wait();
          if (FP8) scale_acc32(r, row_scale, p.scale_b, ni * BN + j * kOutChunkCols + half * 32, p.n);
#pragma unroll
          for (int v = 0; v < 4; ++v) {
            const int chunk16 = half * 4 + v;
            uint4* dst = reinterpret_cast<uint4*>(buf + row_in_tile * 128 + ((chunk16 ^ (row_in_tile & 7)) << 4));
            *dst = make_uint4(pack_bf16(r[8 * v], r[8 * v + 1]), pack_bf16(r[8 * v + 2], r[8 * v + 3]),
                              pack_bf16(r[8 * v + 4], r[8 * v + 5]), pack_bf16(r[8 * v + 6], r[8 * v + 7]));
          }
        }
        if (j == BN / kOutChunkCols - 1) {
          tc_fence_before_sync();
          __syncwarp();
          if (lane == 0) mbar_arrive_leader(&bars->acc_empty[as]);
        }
        fence_proxy_async_smem();
        asm volatile("bar.sync 1, 128;" ::: "memory");
        if (issuer) {
          tma_store_2d(mo, buf, ni * BN + j * kOutChunkCols, out_row);
          tma_store_commit();
        }
      }
      if (MODE == TpMode::GEMM_RS && issuer) {
        tma_store_wait_all<0>();
        if (owner == c.rank) {
          __threadfence_system();
          const int tile_local = (mi - owner * tiles_per_src) * tiles_n + ni;
          st_relaxed_sys(p.arrived[owner] + static_cast<size_t>(tile_local) * c.nranks + c.rank, epoch + 1);
        } else {
          __threadfence();
          atomicAdd(&bars->fwd_ready, 1u);
        }
      }
    }
    if (issuer) {
      tma_store_wait_all<0>();
      trace_stamp_ns(c, 3);
    }
  } else {
    // ---------------- copy warps (all-gather mode), every CTA of the grid takes a slice of every remote m-tile
    if (MODE == TpMode::AG_GEMM) {
      const int ct = threadIdx.x - kGemmThreads;
      if (blockIdx.x == 0 && warp == 6) {
        const bool ok = warp_rank_barrier(c, 0, 0xa1);
        if (lane == 0) {
          __threadfence();
          atomicExch(&p.ctrl[2], ok ? epoch + 1 : 0xffffffffu);
        }
      }
      if (ct == 0) {
        bool started = false;
        poll_until(c, [&]() {
          const uint32_t v = ld_acquire_gpu(&p.ctrl[2]);
          if (v == epoch + 1) started = true;
          return started || v == 0xffffffffu;
        });
        if (!started) bars->failed = 1;
      }
      asm volatile("bar.sync 2, 128;" ::: "memory");
      const size_t tile_bytes = static_cast<size_t>(kBlockM) * p.k * 2;
      const size_t slice = ((tile_bytes + G - 1) / G + 15) / 16 * 16;
      const size_t b0 = static_cast<size_t>(blockIdx.x) * slice;
      for (int ord = tiles_per_src; ord < tiles_m; ++ord) {
        const int mi = mtile_of(ord);
        const int src = mi / tiles_per_src;
        const size_t src_off = static_cast<size_t>(mi - src * tiles_per_src) * tile_bytes;
        if (b0 < tile_bytes) {
          const size_t nbytes = tile_bytes - b0 < slice ? tile_bytes - b0 : slice;
          const uint4* from = reinterpret_cast<const uint4*>(p.x_shards[src] + src_off + b0);
          uint4* to = reinterpret_cast<uint4*>(p.x_full + static_cast<size_t>(mi) * tile_bytes + b0);
          const size_t nvec = nbytes / 16;
          size_t i = ct;
          for (; i + 3 * kCopyThreads < nvec; i += 4 * kCopyThreads) {
            const uint4 v0 = from[i], v1 = from[i + kCopyThreads], v2 = from[i + 2 * kCopyThreads], v3 = from[i + 3 * kCopyThreads];
            to[i] = v0;
            to[i + kCopyThreads] = v1;
            to[i + 2 * kCopyThreads] = v2;
            to[i + 3 * kCopyThreads] = v3;
          }
          for (; i < nvec; i += kCopyThreads) to[i] = from[i];
          fence_proxy_async();
        }
        if (FP8 && blockIdx.x == 0 && ct < kBlockM) {  // the tile's row scales travel with it
          p.scale_a_full[mi * kBlockM + ct] = p.scale_a_shards[src][(mi - src * tiles_per_src) * kBlockM + ct];
        }
        asm volatile("bar.sync 2, 128;" ::: "memory");
        if (ct == 0) {
          __threadfence();
          atomicAdd(&p.ctrl[kCtrlTiles + ord], 1u);
        }
      }
      if (ct == 0) trace_stamp_ns(c, 4);
    }
    // ---------------- reduce warps (reduce-scatter mode), as in k_tp_gemm: every CTA takes its half of
    // the pair tiles of this rank's own rows, in schedule order
    if (MODE == TpMode::GEMM_RS) {
      const int ct = threadIdx.x - kGemmThreads;
      const int first_own = (c.nranks - 1) * tiles_per_src;
      const int my_pair_tiles = (tiles_per_src / 2) * tiles_n;
      // forward this CTA's half of the pair tiles computed for other ranks (see k_tp_gemm)
      uint32_t handed = 0;
      bool fwd_ok = true;
      for (int t = cluster_id; t < (first_own / 2) * tiles_n && fwd_ok; t += nclusters) {
        int ord, ni;
        my_tile(t, &ord, &ni);
        const int mi = mtile_of(ord);
        const int owner = mi / tiles_per_src;
        ++handed;
        if (ct == 0) bars->reduce_ok = wait_fwd_ready(c, bars, handed) ? 1 : 0;
        asm volatile("bar.sync 2, 128;" ::: "memory");
        fwd_ok = bars->reduce_ok != 0;
        if (fwd_ok) {
          const int local_row = (mi - owner * tiles_per_src) * kBlockM;
          forward_tile<BN>(p.send_stage, p.partials[owner], mi * kBlockM, c.rank * p.m_local + local_row, ni * BN, p.n, ct,
                           kCopyThreads);
        }
        asm volatile("bar.sync 2, 128;" ::: "memory");
        if (fwd_ok && ct == 0) {
          __threadfence_system();
          const int tile_local = (mi - owner * tiles_per_src) * tiles_n + ni;
          st_relaxed_sys(p.arrived[owner] + static_cast<size_t>(tile_local) * c.nranks + c.rank, epoch + 1);
        }
      }
      if (ct == 0) {
        if (!fwd_ok) bars->failed = 1;
        trace_stamp_ns(c, 4);
      }
      for (int t_own = cluster_id; t_own < my_pair_tiles; t_own += nclusters) {
        int ord, ni;
        my_tile((first_own / 2) * tiles_n + t_own, &ord, &ni);
        const int wm = ord - first_own;
        if (ct == 0) bars->reduce_ok = 1;
        asm volatile("bar.sync 2, 128;" ::: "memory");
        if (ct < c.nranks) {
          const uint32_t* flag = p.arrived[c.rank] + static_cast<size_t>(wm * tiles_n + ni) * c.nranks + ct;
          if (!wait_flag_quietly(c, flag, epoch + 1, ct, 0xa3)) bars->reduce_ok = 0;
        }
        asm volatile("bar.sync 2, 128;" ::: "memory");
        if (!bars->reduce_ok) {
          if (ct == 0) bars->failed = 1;
          break;
        }
        if (ct == 0 && t_own < nclusters) trace_stamp_ns(c, 5);
        const __nv_bfloat16* base = reinterpret_cast<const __nv_bfloat16*>(p.partials_local);
        reduce_tile<BN, 4, 4>(base, p.out, wm, ni, p.n, static_cast<size_t>(p.m_local) * p.n, c.nranks, ct, kCopyThreads);
        asm volatile("bar.sync 2, 128;" ::: "memory");
      }
      if (ct == 0) trace_stamp_ns(c, 6);
    }
  }

  tc_fence_before_sync();
  __syncthreads();

  // ---------------- teardown
  __syncthreads();
  cluster_sync_all();  // the peer may still address this CTA's shared memory and barriers
  if (warp == 1) {
    tmem_dealloc_pair(tmem_base, 2 * BN);
  }
  if (threadIdx.x == 0) {
    trace_stamp_ns(c, 7);
    if (bars->failed) c.status[0] = c.status[0] | kStatusTimeout;
    __threadfence();
    const uint32_t ticket = atomicAdd(&p.ctrl[1], 1u);
    bars->is_last = ticket == static_cast<uint32_t>(G - 1) ? 1u : 0u;
  }
  __syncthreads();
  if (bars->is_last && warp == 0) {
    __threadfence();
    warp_rank_barrier(c, 1, 0xa2);
    if (lane == 0) {
      trace_stamp_ns(c, 8);
      p.ctrl[1] = 0;
      __threadfence();
      atomicExch(&p.ctrl[0], epoch + 1);
    }
  }
}

// ------------------------------------------------------------ launchers ----

int sm_count() {
  int dev = 0, sms = 0;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  return std::max(1, sms);
}

// Group height (in tiles of `tile_rows` rows): the A rows of a group are
// re-read by every wave that sweeps over n, so they should stay in L2 - at
// most ~40 MB of A per group and at most `cap` tiles - and a group should not
// mix rows that arrive at different times, so it divides the tiles of one
// source rank where it can.
int pick_group(int tiles_per_src, int tile_rows, int k, int cap) {
  const size_t tile_bytes = static_cast<size_t>(tile_rows) * k * 2;
  const int by_l2 = static_cast<int>(std::max<size_t>(1, (40u << 20) / std::max<size_t>(tile_bytes, 1)));
  const int limit = std::max(1, std::min({cap, by_l2, tiles_per_src}));
  for (int g = limit; g >= std::max(1, limit / 2); --g) {
    if (tiles_per_src % g == 0) return g;
  }
  return limit;  // awkward counts: groups straddle sources, still correct
}

template <TpMode MODE, bool FP8>
cudaError_t tp_launch_t(int grid, const TpMaps& maps, const CommDev& c, const TpParams& p, cudaStream_t stream) {
  // Per device, so not cached in a process-wide flag.
  cudaError_t e = cudaFuncSetAttribute(k_tp_gemm<MODE, FP8>, cudaFuncAttributeMaxDynamicSharedMemorySize, kTpSmemBytes);
  if (e != cudaSuccess) return e;
  k_tp_gemm<MODE, FP8><<<grid, tp_threads<MODE>(), kTpSmemBytes, stream>>>(maps, c, p);
  note_kernel_launch();
  return cudaGetLastError();
}

// The operand type (p.fp8) picks the instantiation: the bf16 kernels carry no trace of the fp8 path.
template <TpMode MODE>
cudaError_t tp_launch(int grid, const TpMaps& maps, const CommDev& c, const TpParams& p, cudaStream_t stream) {
  return p.fp8 ? tp_launch_t<MODE, true>(grid, maps, c, p, stream) : tp_launch_t<MODE, false>(grid, maps, c, p, stream);
}

// Pair kernels: on unless B200COMMS_TP_PAIRS=0; need two 128-row tiles per source rank.
bool use_pairs(int m_local) {
  static const bool enabled = [] {
    const char* v = std::getenv("B200COMMS_TP_PAIRS");
    return v == nullptr || std::string(v) != "0";
  }();
  return enabled && m_local % (2 * kBlockM) == 0;
}

// `want_pairs` <= 0: as many pairs as the device holds at once.
template <TpMode MODE, bool FP8>
cudaError_t tp_launch_pair_t(int want_pairs, const TpMaps& maps, const CommDev& c, const TpParams& p, cudaStream_t stream) {
  cudaError_t e = cudaFuncSetAttribute(k_tp_gemm_pair<MODE, FP8>, cudaFuncAttributeMaxDynamicSharedMemorySize, kPairSmemBytes);
  if (e != cudaSuccess) return e;
  cudaLaunchConfig_t cfg = {};
  cfg.blockDim = dim3(tp_threads<MODE>());
  cfg.dynamicSmemBytes = kPairSmemBytes;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 2;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  cfg.gridDim = dim3(2);
  int max_clusters = 0;
  e = cudaOccupancyMaxActiveClusters(&max_clusters, k_tp_gemm_pair<MODE, FP8>, &cfg);
  if (e != cudaSuccess) return e;
  if (max_clusters < 1) return cudaErrorInvalidConfiguration;
  const int clusters = want_pairs > 0 ? std::min(max_clusters, want_pairs) : max_clusters;
  cfg.gridDim = dim3(2 * clusters);
  e = cudaLaunchKernelEx(&cfg, k_tp_gemm_pair<MODE, FP8>, maps, c, p);
  note_kernel_launch();
  return e != cudaSuccess ? e : cudaGetLastError();
}

template <TpMode MODE>
cudaError_t tp_launch_pair(int want_pairs, const TpMaps& maps, const CommDev& c, const TpParams& p, cudaStream_t stream) {
  return p.fp8 ? tp_launch_pair_t<MODE, true>(want_pairs, maps, c, p, stream)
               : tp_launch_pair_t<MODE, false>(want_pairs, maps, c, p, stream);
}

} // namespace

cudaError_t launch_gemm_bf16_nt(const void* a, const void* b, void* c, int m, int n, int k, uint32_t* status,
                                cudaStream_t stream) {
  return launch_gemm_nt(a, b, c, m, n, k, nullptr, nullptr, status, stream);
}

cudaError_t launch_gemm_e4m3_nt(const void* a, const void* b, void* c, int m, int n, int k, const float* scale_a,
                                const float* scale_b, uint32_t* status, cudaStream_t stream) {
  if (scale_a == nullptr || scale_b == nullptr || k % 16 != 0) return cudaErrorInvalidValue;
  return launch_gemm_nt(a, b, c, m, n, k / 2, scale_a, scale_b, status, stream);
}

// k in 16-bit units; scales non-null = e4m3 operands.
cudaError_t launch_gemm_nt(const void* a, const void* b, void* c, int m, int n, int k, const float* scale_a,
                           const float* scale_b, uint32_t* status, cudaStream_t stream) {
  if (m <= 0 || n <= 0 || k <= 0 || k % 8 != 0 || n % 8 != 0) return cudaErrorInvalidValue;
  if ((reinterpret_cast<uintptr_t>(a) | reinterpret_cast<uintptr_t>(b) | reinterpret_cast<uintptr_t>(c)) & 15u) {
    return cudaErrorInvalidValue;
  }
  TpMaps maps;
  if (!make_map(&maps.a_local, a, m, k, kBlockM) || !make_map(&maps.b, b, n, k, kTpBN) ||
      !make_map(&maps.out[0], c, m, n, kBlockM)) {
    return cudaErrorInvalidValue;
  }
  maps.a_full = maps.a_local;
  maps.b_half = maps.b;
  for (int r = 1; r < kMaxRanks; ++r) maps.out[r] = maps.out[0];
  CommDev none{};
  none.nranks = 1;
  TpParams p{};
  p.status = status;
  p.m_total = m;
  p.m_local = m;
  p.n = n;
  p.k = k;
  p.fp8 = scale_a != nullptr ? 1 : 0;
  p.scale_a = scale_a;
  p.scale_b = scale_b;
  const int tiles_m = (m + kBlockM - 1) / kBlockM, tiles_n = (n + kTpBN - 1) / kTpBN;
  p.gm = pick_group(tiles_m, kBlockM, k, 16);
  return tp_launch<TpMode::PLAIN>(std::min(sm_count(), tiles_m * tiles_n), maps, none, p, stream);
}

size_t tp_ctrl_words(int m_total) {
  return static_cast<size_t>(kCtrlTiles) + static_cast<size_t>(m_total / kBlockM);
}

namespace {

// Tensor maps and parameters of one rank's all-gather GEMM. `pairs`: for the CTA-pair kernel.
cudaError_t build_ag(const CommDev& comm, const AgGemmArgs& a, bool pairs, TpMaps& maps, TpParams& p) {
  const int m_total = a.m_local * comm.nranks;
  const int k = a.fp8 ? a.k / 2 : a.k;   // in 16-bit units
  if (a.m_local <= 0 || a.m_local % kBlockM != 0 || a.n % kTpBN != 0 || a.k % (a.fp8 ? 2 * kBlockK : kBlockK) != 0) {
    return cudaErrorInvalidValue;
  }
  if (comm.nranks > kMaxRanks) return cudaErrorInvalidValue;
  if (a.fp8 && (a.scale_w == nullptr || a.scale_x_full == nullptr)) return cudaErrorInvalidValue;
  if (!make_map(&maps.a_local, a.x_shards[comm.rank], a.m_local, k, kBlockM) ||
      !make_map(&maps.a_full, a.x_full, m_total, k, kBlockM) || !make_map(&maps.b, a.w, a.n, k, kTpBN) ||
      !make_map(&maps.out[0], a.y, m_total, a.n, kBlockM)) {
    return cudaErrorInvalidValue;
  }
  for (int r = 1; r < kMaxRanks; ++r) maps.out[r] = maps.out[0];
  p = TpParams{};
  for (int r = 0; r < comm.nranks; ++r) p.x_shards[r] = static_cast<const char*>(a.x_shards[r]);
  p.x_full = static_cast<char*>(a.x_full);
  p.ctrl = a.ctrl;
  p.m_total = m_total;
  p.m_local = a.m_local;
  p.n = a.n;
  p.k = k;
  p.fp8 = a.fp8;
  if (a.fp8) {
    for (int r = 0; r < comm.nranks; ++r) {
      if (a.scale_x_shards[r] == nullptr) return cudaErrorInvalidValue;
      p.scale_a_shards[r] = a.scale_x_shards[r];
    }
    p.scale_a_full = a.scale_x_full;
    p.scale_b = a.scale_w;
  }
  if (pairs) {
    if (!make_map(&maps.b_half, a.w, a.n, k, kBlockM)) return cudaErrorInvalidValue;
    p.gm = pick_group(a.m_local / (2 * kBlockM), 2 * kBlockM, k, 8);
  } else {
    maps.b_half = maps.b;
    p.gm = pick_group(a.m_local / kBlockM, kBlockM, k, 16);
  }
  return cudaSuccess;
}

cudaError_t build_rs(const CommDev& comm, const GemmRsArgs& a, bool pairs, TpMaps& maps, TpParams& p) {
  const int k = a.fp8 ? a.k_local / 2 : a.k_local;   // in 16-bit units
  if (a.m <= 0 || a.m % (kBlockM * comm.nranks) != 0 || a.n % kTpBN != 0 || a.k_local % (a.fp8 ? 2 * kBlockK : kBlockK) != 0) {
    return cudaErrorInvalidValue;
  }
  if (comm.nranks > kMaxRanks) return cudaErrorInvalidValue;
  if (a.fp8 && (a.scale_h == nullptr || a.scale_w == nullptr)) return cudaErrorInvalidValue;
  if (!make_map(&maps.a_local, a.h, a.m, k, kBlockM) || !make_map(&maps.b, a.w, a.n, k, kTpBN)) {
    return cudaErrorInvalidValue;
  }
  maps.a_full = maps.a_local;
  // TMA stores stay on this GPU: own rows go into this rank's receive staging (viewed as [m, n]), the other
  // ranks' rows into the local send staging, from where the forward warps push them with plain stores.
  if (comm.nranks > 1 && a.send_stage == nullptr) return cudaErrorInvalidValue;
  if (!make_map(&maps.out[comm.rank], a.partials[comm.rank], a.m, a.n, kBlockM)) return cudaErrorInvalidValue;
  for (int r = 0; r < kMaxRanks; ++r) {
    if (r != comm.rank) maps.out[r] = maps.out[comm.rank];
  }
  if (!make_map(&maps.out_send, comm.nranks > 1 ? a.send_stage : a.partials[comm.rank], a.m, a.n, kBlockM)) {
    return cudaErrorInvalidValue;
  }
  p = TpParams{};
  p.partials_local = static_cast<const char*>(a.partials[comm.rank]);
  p.send_stage = static_cast<const char*>(a.send_stage);
  for (int r = 0; r < comm.nranks; ++r) {
    p.arrived[r] = a.arrived[r];
    p.partials[r] = static_cast<char*>(a.partials[r]);
  }
  p.out = static_cast<__nv_bfloat16*>(a.out);
  p.ctrl = a.ctrl;
  p.m_total = a.m;
  p.m_local = a.m / comm.nranks;
  p.n = a.n;
  p.k = k;
  p.fp8 = a.fp8;
  p.scale_a = a.scale_h;
  p.scale_b = a.scale_w;
  if (pairs) {
    if (!make_map(&maps.b_half, a.w, a.n, k, kBlockM)) return cudaErrorInvalidValue;
    p.gm = pick_group(p.m_local / (2 * kBlockM), 2 * kBlockM, k, 8);
  } else {
    maps.b_half = maps.b;
    p.gm = pick_group(p.m_local / kBlockM, kBlockM, k, 16);
  }
  return cudaSuccess;
}

template <TpMode MODE, bool FP8>
cudaError_t tp_launch_emu_t(const TpEmu& e, int nranks, cudaStream_t stream) {
  cudaError_t err = cudaFuncSetAttribute(k_tp_gemm_emu<MODE, FP8>, cudaFuncAttributeMaxDynamicSharedMemorySize, kTpSmemBytes);
  if (err != cudaSuccess) return err;
  const int per_rank = sm_count() / nranks;
  if (per_rank < 1) return cudaErrorInvalidConfiguration;
  void* params[] = {const_cast<TpEmu*>(&e)};
  note_kernel_launch();
  return cudaLaunchCooperativeKernel(reinterpret_cast<void*>(&k_tp_gemm_emu<MODE, FP8>), dim3(per_rank, nranks),
                                     dim3(tp_threads<MODE>()), params, kTpSmemBytes, stream);
}

template <TpMode MODE>
cudaError_t tp_launch_emu(const TpEmu& e, int nranks, cudaStream_t stream) {
  return e.p[0].fp8 ? tp_launch_emu_t<MODE, true>(e, nranks, stream) : tp_launch_emu_t<MODE, false>(e, nranks, stream);
}

} // namespace

cudaError_t launch_allgather_gemm(const CommDev& comm, const AgGemmArgs& a, cudaStream_t stream) {
  TpMaps maps;
  TpParams p;
  const bool pairs = a.m_local > 0 && use_pairs(a.m_local);
  cudaError_t e = build_ag(comm, a, pairs, maps, p);
  if (e != cudaSuccess) return e;
  if (pairs) return tp_launch_pair<TpMode::AG_GEMM>(0, maps, comm, p, stream);
  // All CTAs take part in the copy, so the grid is the whole GPU even when
  // there are fewer tiles than SMs.
  return tp_launch<TpMode::AG_GEMM>(sm_count(), maps, comm, p, stream);
}

cudaError_t launch_gemm_reduce_scatter(const CommDev& comm, const GemmRsArgs& a, cudaStream_t stream) {
  TpMaps maps;
  TpParams p;
  const bool pairs = a.m > 0 && comm.nranks > 0 && use_pairs(a.m / comm.nranks);
  cudaError_t e = build_rs(comm, a, pairs, maps, p);
  if (e != cudaSuccess) return e;
  const int tiles = (a.m / kBlockM) * (a.n / kTpBN);
  if (pairs) return tp_launch_pair<TpMode::GEMM_RS>(tiles / 2, maps, comm, p, stream);
  return tp_launch<TpMode::GEMM_RS>(std::min(sm_count(), tiles), maps, comm, p, stream);
}

cudaError_t launch_allgather_gemm_emu(const CommDev* comms, const AgGemmArgs* args, int nranks, cudaStream_t stream) {
  if (nranks < 1 || nranks > kTpEmuRanks) return cudaErrorInvalidValue;
  TpEmu e{};
  for (int r = 0; r < nranks; ++r) {
    e.c[r] = comms[r];
    cudaError_t err = build_ag(comms[r], args[r], false, e.maps[r], e.p[r]);
    if (err != cudaSuccess) return err;
  }
  return tp_launch_emu<TpMode::AG_GEMM>(e, nranks, stream);
}

cudaError_t launch_gemm_reduce_scatter_emu(const CommDev* comms, const GemmRsArgs* args, int nranks, cudaStream_t stream) {
  if (nranks < 1 || nranks > kTpEmuRanks) return cudaErrorInvalidValue;
  TpEmu e{};
  for (int r = 0; r < nranks; ++r) {
    e.c[r] = comms[r];
    cudaError_t err = build_rs(comms[r], args[r], false, e.maps[r], e.p[r]);
    if (err != cudaSuccess) return err;
  }
  return tp_launch_emu<TpMode::GEMM_RS>(e, nranks, stream);
}

} // namespace b200c
