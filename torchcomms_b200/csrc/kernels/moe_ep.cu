// MoE expert-parallel dispatch / combine kernels (sm_100a). See moe_ep.h.
#include "moe_ep.h"

#include <cooperative_groups.h>
#include <cuda_fp8.h>

#include <algorithm>
#include <vector>

#include "launch_count.h"

namespace cg = cooperative_groups;

namespace b200c {

namespace {

constexpr int kEpThreads = 256;
constexpr int kEpWarps = kEpThreads / 32;

__device__ __forceinline__ float2 bf2f(uint32_t v) {
  return make_float2(__uint_as_float(v << 16), __uint_as_float(v & 0xffff0000u));
}

// Destination-rank mask of one token, computed by the whole warp from the
// token's top-k expert ids (lane k holds id k).
__device__ __forceinline__ uint32_t dst_mask(const EpDev& e, int my_idx) {
  const int lane = threadIdx.x & 31;
  const bool valid = lane < e.topk && my_idx >= 0 && my_idx < e.num_experts;
  const int d = valid ? my_idx / e.experts_per_rank : -1;
  uint32_t mask = 0;
  for (int r = 0; r < e.nranks; ++r) {
    if (__any_sync(0xffffffffu, d == r)) mask |= 1u << r;
  }
  return mask;
}

// Cross-GPU barrier by block 0 of every rank, on flag row 0 of the EP set.
__device__ __forceinline__ bool ep_rank_barrier(const CommDev& c, uint32_t phase) {
  BlockEpoch ep;
  ep.load(c, kFlagSetEp);
  const bool ok = block_barrier(c, kFlagSetEp, ep, phase);
  ep.store(c, kFlagSetEp);
  return ok;
}

struct DispatchArgs {
  const void* x;          // [num_tokens, hidden] bf16
  const int* topk_idx;    // [num_tokens, topk]
  const float* topk_w;    // [num_tokens, topk]
  int num_tokens;
};

__device__ void ep_dispatch_body(const CommDev& c, const EpDev& e, const DispatchArgs& a) {
  cg::grid_group grid = cg::this_grid();
  __shared__ int s_cnt[kMaxRanks];
  __shared__ int s_slots[kEpWarps][kMaxRanks];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int gwarp = blockIdx.x * kEpWarps + warp, nwarps = gridDim.x * kEpWarps;

  trace_mark(c, 0);
  // A. reset the per-call counters
  if (blockIdx.x == 0 && threadIdx.x < e.nranks) {
    e.cnt[threadIdx.x] = 0;
    e.cursor[threadIdx.x] = 0;
  }
  if (threadIdx.x < kMaxRanks) s_cnt[threadIdx.x] = 0;
  grid.sync();

  // B. how many tokens go to each destination rank
  for (int t = gwarp; t < a.num_tokens; t += nwarps) {
    const int idx = lane < e.topk ? a.topk_idx[static_cast<size_t>(t) * e.topk + lane] : -1;
    const uint32_t mask = dst_mask(e, idx);
    if (lane < e.nranks && (mask >> lane) & 1u) atomicAdd(&s_cnt[lane], 1);
  }
  __syncthreads();
  if (threadIdx.x < e.nranks && s_cnt[threadIdx.x] > 0) atomicAdd(&e.cnt[threadIdx.x], s_cnt[threadIdx.x]);
  grid.sync();
  trace_mark(c, 1);

  // C. publish the counts to every rank, learn where this rank's rows start
  //    inside each destination's receive buffer (rows are packed by source).
  if (blockIdx.x == 0) {
    if (threadIdx.x < e.nranks) {
      const int d = threadIdx.x;
      const long long n = e.cnt[d];
      for (int p = 0; p < e.nranks; ++p) {
        e.count_matrix[p][e.rank * e.nranks + d] = n;
      }
    }
    ep_rank_barrier(c, 0x91);
    const long long* m = e.count_matrix[e.rank];
    if (threadIdx.x < e.nranks) {
      const int d = threadIdx.x;
      long long b = 0;
      for (int s = 0; s < e.rank; ++s) b += m[s * e.nranks + d];
      e.base[d] = b;
      e.recv_info[1 + d] = static_cast<int>(m[d * e.nranks + e.rank]);  // rows from source d
    }
    if (threadIdx.x == 0) {
      long long total = 0;
      for (int s = 0; s < e.nranks; ++s) total += m[s * e.nranks + e.rank];
      e.recv_info[0] = static_cast<int>(total);
    }
  }
  grid.sync();
  trace_mark(c, 2);

  // D. quantise and send
  const int groups = e.hidden / 128;
  const size_t row_bytes = e.fp8 ? static_cast<size_t>(e.hidden) : static_cast<size_t>(e.hidden) * 2;
  for (int t = gwarp; t < a.num_tokens; t += nwarps) {
    const int idx = lane < e.topk ? a.topk_idx[static_cast<size_t>(t) * e.topk + lane] : -1;
    const float w = lane < e.topk ? a.topk_w[static_cast<size_t>(t) * e.topk + lane] : 0.0f;
    const uint32_t mask = dst_mask(e, idx);
    if (lane < e.nranks) {
      int slot = -1;
      if ((mask >> lane) & 1u) {
        slot = static_cast<int>(e.base[lane]) + atomicAdd(&e.cursor[lane], 1);
        if (slot >= e.nranks * e.max_tokens) {  // cannot happen with consistent inputs; never write out of bounds
          c.status[0] = c.status[0] | kStatusBadArg;
          slot = -1;
        }
      }
      s_slots[warp][lane] = slot;
      e.send_slot[static_cast<size_t>(t) * e.nranks + lane] = slot;
    }
    __syncwarp();
    // metadata
    for (int d = 0; d < e.nranks; ++d) {
      const int slot = s_slots[warp][d];
      if (slot < 0) continue;
      if (lane < e.topk) {
        const bool here = idx >= 0 && idx / e.experts_per_rank == d;
        e.recv_topk_idx[d][static_cast<size_t>(slot) * e.topk + lane] = here ? idx - d * e.experts_per_rank : -1;
        e.recv_topk_w[d][static_cast<size_t>(slot) * e.topk + lane] = here ? w : 0.0f;
      }
      if (lane == 0) e.recv_src[d][slot] = e.rank * e.max_tokens + t;
    }
    // payload: 16 elements per lane and step, 8 lanes share one 128-element group
    const __nv_bfloat16* xr = static_cast<const __nv_bfloat16*>(a.x) + static_cast<size_t>(t) * e.hidden;
    for (int e0 = lane * 16; e0 < e.hidden; e0 += 512) {
      const uint4 v0 = ld16(xr + e0);
      const uint4 v1 = ld16(xr + e0 + 8);
      if (!e.fp8) {
        for (int d = 0; d < e.nranks; ++d) {
          const int slot = s_slots[warp][d];
          if (slot < 0) continue;
          char* dst = e.recv_x[d] + static_cast<size_t>(slot) * row_bytes + static_cast<size_t>(e0) * 2;
          st16(dst, v0);
          st16(dst + 16, v1);
        }
        continue;
      }
      float f[16];
      {
        const uint32_t* p0 = &v0.x;
        const uint32_t* p1 = &v1.x;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const float2 a0 = bf2f(p0[i]), a1 = bf2f(p1[i]);
          f[2 * i] = a0.x;
          f[2 * i + 1] = a0.y;
          f[8 + 2 * i] = a1.x;
          f[8 + 2 * i + 1] = a1.y;
        }
      }
      float amax = 0.0f;
#pragma unroll
      for (int i = 0; i < 16; ++i) amax = fmaxf(amax, fabsf(f[i]));
      amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 1));
      amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 2));
      amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 4));
      amax = fmaxf(amax, 1e-4f);
      const float scale = amax / 448.0f;
      const float inv = 448.0f / amax;
      uint32_t q[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const __nv_fp8x2_storage_t lo = __nv_cvt_float2_to_fp8x2(make_float2(f[4 * i] * inv, f[4 * i + 1] * inv), __NV_SATFINITE, __NV_E4M3);
        const __nv_fp8x2_storage_t hi = __nv_cvt_float2_to_fp8x2(make_float2(f[4 * i + 2] * inv, f[4 * i + 3] * inv), __NV_SATFINITE, __NV_E4M3);
        q[i] = static_cast<uint32_t>(lo) | (static_cast<uint32_t>(hi) << 16);
      }
      const uint4 packed = make_uint4(q[0], q[1], q[2], q[3]);
      const int group = e0 / 128;
      for (int d = 0; d < e.nranks; ++d) {
        const int slot = s_slots[warp][d];
        if (slot < 0) continue;
        st16(e.recv_x[d] + static_cast<size_t>(slot) * row_bytes + e0, packed);
        if ((lane & 7) == 0) e.recv_scales[d][static_cast<size_t>(slot) * groups + group] = scale;
      }
    }
    __syncwarp();
  }
  trace_mark(c, 3);
  grid.sync();
  // E. every rank's rows have landed before anybody returns
  if (blockIdx.x == 0) {
    ep_rank_barrier(c, 0x92);
    trace_mark(c, 4);
  }
}

__global__ void __launch_bounds__(kEpThreads) k_ep_dispatch(CommDev c, EpDev e, DispatchArgs a) {
  ep_dispatch_body(c, e, a);
}
__global__ void __launch_bounds__(kEpThreads) k_ep_dispatch_emu(const CommDev* cs, const EpDev* es, const DispatchArgs* as) {
  ep_dispatch_body(cs[blockIdx.y], es[blockIdx.y], as[blockIdx.y]);
}

struct CombineArgs {
  void* out;             // [num_tokens, hidden] bf16
  const float* weights;  // [num_tokens, nranks] or nullptr
  const void* bias;      // [num_tokens, hidden] bf16 or nullptr
  int num_tokens;
  const int* send_slot;  // [num_tokens, nranks] handle of the dispatch to undo; nullptr = the last one's
  float* topk_w_out;     // [num_tokens, topk] or nullptr
};

// Pull combine: the token's owner reads the expert output of every rank the
// token went to straight out of that rank's `combine_x` (the row is the slot
// the dispatch recorded in `send_slot`) and forms the weighted sum in
// registers. Each row crosses NVLink once and nothing is staged. Every block
// meets its peers' blocks before (all expert outputs are complete) and after
// (nobody still reads this rank's outputs), so the kernel needs no grid-wide
// synchronisation.
__device__ void ep_combine_body(const CommDev& c, const EpDev& e, const CombineArgs& a) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int gwarp = blockIdx.x * kEpWarps + warp, nwarps = gridDim.x * kEpWarps;
  const size_t row_bytes = static_cast<size_t>(e.hidden) * 2;
  const int cap_rows = e.nranks * e.max_tokens;
  const int* send_slot = a.send_slot != nullptr ? a.send_slot : e.send_slot;
  BlockEpoch ep;
  ep.load(c, kFlagSetEp);
  trace_mark(c, 0);
  bool ok = block_barrier(c, kFlagSetEp, ep, 0x93);
  trace_mark(c, 1);
  if (ok) {
    for (int t = gwarp; t < a.num_tokens; t += nwarps) {
      int slot = -1;
      float wt = 1.0f;
      if (lane < e.nranks) {
        slot = send_slot[static_cast<size_t>(t) * e.nranks + lane];
        if (slot >= cap_rows) {  // never read through a bad index
          c.status[0] = c.status[0] | kStatusBadArg;
          slot = -1;
        }
        if (a.weights != nullptr) wt = a.weights[static_cast<size_t>(t) * e.nranks + lane];
      }
      const uint32_t have = __ballot_sync(0xffffffffu, slot >= 0);
      if (a.topk_w_out != nullptr) {
        // Per-expert weights travel back with the rows: entry k is non-zero on the one rank that hosts expert k.
        float acc_w = 0.0f;
        for (int d = 0; d < e.nranks; ++d) {
          const int sd = __shfl_sync(0xffffffffu, slot, d);
          if (((have >> d) & 1u) && lane < e.topk) acc_w += e.comb_topk_w[d][static_cast<size_t>(sd) * e.topk + lane];
        }
        if (lane < e.topk) a.topk_w_out[static_cast<size_t>(t) * e.topk + lane] = acc_w;
      }
      // Two 16-byte columns per lane and step: up to 2 x nranks remote loads in flight per thread.
      for (int e0 = lane * 8; e0 < e.hidden; e0 += 512) {
        const bool second = e0 + 256 < e.hidden;
        uint4 rows[2][kMaxRanks];
#pragma unroll
        for (int i = 0; i < kMaxRanks; ++i) {
          if (i < e.nranks) {
            // Start at the next rank so that the ranks read different peers at any time.
            int d = e.rank + 1 + i;
            if (d >= e.nranks) d -= e.nranks;
            const int sd = __shfl_sync(0xffffffffu, slot, d);
            if ((have >> d) & 1u) {
              const char* src = e.combine_x[d] + static_cast<size_t>(sd) * row_bytes + static_cast<size_t>(e0) * 2;
              rows[0][i] = ld16_stream(src);
              if (second) rows[1][i] = ld16_stream(src + 512);
            }
          }
        }
#pragma unroll
        for (int h = 0; h < 2; ++h) {
          if (h == 1 && !second) break;
          const int col = e0 + h * 256;
          float acc[8];
#pragma unroll
          for (int i = 0; i < 8; ++i) acc[i] = 0.0f;
          if (a.bias != nullptr) {
            const uint4 b = ld16(static_cast<const __nv_bfloat16*>(a.bias) + static_cast<size_t>(t) * e.hidden + col);
            const uint32_t* p = &b.x;
#pragma unroll
            for (int i = 0; i < 4; ++i) {
              const float2 f = bf2f(p[i]);
              acc[2 * i] = f.x;
              acc[2 * i + 1] = f.y;
            }
          }
#pragma unroll
          for (int i = 0; i < kMaxRanks; ++i) {
            if (i < e.nranks) {
              int d = e.rank + 1 + i;
              if (d >= e.nranks) d -= e.nranks;
              const float wd = __shfl_sync(0xffffffffu, wt, d);
              if ((have >> d) & 1u) {
                const uint32_t* p = &rows[h][i].x;
#pragma unroll
                for (int k = 0; k < 4; ++k) {
                  const float2 f = bf2f(p[k]);
                  acc[2 * k] += wd * f.x;
                  acc[2 * k + 1] += wd * f.y;
                }
              }
            }
          }
          uint4 o;
          uint32_t* po = &o.x;
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            __nv_bfloat162 hh = __floats2bfloat162_rn(acc[2 * i], acc[2 * i + 1]);
            po[i] = *reinterpret_cast<uint32_t*>(&hh);
          }
          st16(static_cast<__nv_bfloat16*>(a.out) + static_cast<size_t>(t) * e.hidden + col, o);
        }
      }
    }
    trace_mark(c, 2);
    // Nobody overwrites its expert outputs while a peer still reads them.
    ok = block_barrier(c, kFlagSetEp, ep, 0x94);
    trace_mark(c, 3);
  }
  ep.store(c, kFlagSetEp);
}

__global__ void __launch_bounds__(kEpThreads) k_ep_combine(CommDev c, EpDev e, CombineArgs a) {
  ep_combine_body(c, e, a);
}
__global__ void __launch_bounds__(kEpThreads) k_ep_combine_emu(const CommDev* cs, const EpDev* es, const CombineArgs* as) {
  ep_combine_body(cs[blockIdx.y], es[blockIdx.y], as[blockIdx.y]);
}

struct PullArgs {
  void* out;             // [out_rows, hidden] bf16
  const int* recv_src;   // [rows] src_rank * max_tokens + token; nullptr = the last dispatch's
  const int* num_rows;   // device count; nullptr = the last dispatch's
  int out_rows;
};

// Cached dispatch: the receiver copies the rows it was sent by an earlier
// dispatch again, this time out of the sources' `stage_x` (bf16, as is). The
// same per-block meeting before and after as in the combine.
__device__ void ep_pull_body(const CommDev& c, const EpDev& e, const PullArgs& a) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int gwarp = blockIdx.x * kEpWarps + warp, nwarps = gridDim.x * kEpWarps;
  const size_t row_bytes = static_cast<size_t>(e.hidden) * 2;
  const int* recv_src = a.recv_src != nullptr ? a.recv_src : e.recv_src[e.rank];
  BlockEpoch ep;
  ep.load(c, kFlagSetEp);
  bool ok = block_barrier(c, kFlagSetEp, ep, 0x95);
  if (ok) {
    int rows = a.num_rows != nullptr ? a.num_rows[0] : e.recv_info[0];
    if (rows > a.out_rows) rows = a.out_rows;
    for (int r = gwarp; r < rows; r += nwarps) {
      const int src = recv_src[r];
      const int s = src / e.max_tokens, t = src - s * e.max_tokens;
      if (src < 0 || s >= e.nranks) {  // a handle that does not belong to this buffer: skip, never read through it
        if (lane == 0) c.status[0] = c.status[0] | kStatusBadArg;
        continue;
      }
      const char* from = e.stage_x[s] + static_cast<size_t>(t) * row_bytes;
      char* to = static_cast<char*>(a.out) + static_cast<size_t>(r) * row_bytes;
      for (size_t b = static_cast<size_t>(lane) * 16; b < row_bytes; b += 2048) {
        uint4 v[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          if (b + i * 512 < row_bytes) v[i] = ld16_stream(from + b + i * 512);
        }
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          if (b + i * 512 < row_bytes) st16(to + b + i * 512, v[i]);
        }
      }
    }
    // Nobody refills its staging rows while a peer still reads them.
    ok = block_barrier(c, kFlagSetEp, ep, 0x96);
  }
  ep.store(c, kFlagSetEp);
}

__global__ void __launch_bounds__(kEpThreads) k_ep_pull(CommDev c, EpDev e, PullArgs a) {
  ep_pull_body(c, e, a);
}
__global__ void __launch_bounds__(kEpThreads) k_ep_pull_emu(const CommDev* cs, const EpDev* es, const PullArgs* as) {
  ep_pull_body(cs[blockIdx.y], es[blockIdx.y], as[blockIdx.y]);
}

__global__ void k_ep_layout(const int* __restrict__ topk_idx, int num_tokens, int topk, int num_experts, int nranks,
                            int* __restrict__ per_rank, int* __restrict__ per_expert, int* __restrict__ in_rank) {
  const int epr = num_experts / nranks;
  for (int t = blockIdx.x * blockDim.x + threadIdx.x; t < num_tokens; t += gridDim.x * blockDim.x) {
    uint32_t mask = 0;
    for (int k = 0; k < topk; ++k) {
      const int idx = topk_idx[static_cast<size_t>(t) * topk + k];
      if (idx >= 0 && idx < num_experts) {
        atomicAdd(&per_expert[idx], 1);
        mask |= 1u << (idx / epr);
      }
    }
    for (int r = 0; r < nranks; ++r) {
      const int in = (mask >> r) & 1u;
      in_rank[static_cast<size_t>(t) * nranks + r] = in;
      if (in) atomicAdd(&per_rank[r], 1);
    }
  }
}

// One cooperative launch; the grid is sized so that every block is resident.
template <typename Args>
cudaError_t launch_coop(void* real_kernel, void* emu_kernel, const CommDev* comms, const EpDev* eps, int emu_ranks,
                        const std::vector<Args>& args, cudaStream_t stream) {
  int dev = 0, sms = 0, per_sm = 0;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, real_kernel, kEpThreads, 0);
  if (per_sm < 1) per_sm = 1;
  if (per_sm > 2) per_sm = 2;
  note_kernel_launch();
  if (emu_ranks <= 0) {
    CommDev c = comms[0];
    EpDev e = eps[0];
    Args a = args[0];
    void* params[] = {&c, &e, &a};
    return cudaLaunchCooperativeKernel(real_kernel, dim3(sms * per_sm), dim3(kEpThreads), params, 0, stream);
  }
  CommDev* dc = nullptr;
  EpDev* de = nullptr;
  Args* da = nullptr;
  cudaMalloc(&dc, sizeof(CommDev) * emu_ranks);
  cudaMalloc(&de, sizeof(EpDev) * emu_ranks);
  cudaMalloc(&da, sizeof(Args) * emu_ranks);
  cudaMemcpyAsync(dc, comms, sizeof(CommDev) * emu_ranks, cudaMemcpyHostToDevice, stream);
  cudaMemcpyAsync(de, eps, sizeof(EpDev) * emu_ranks, cudaMemcpyHostToDevice, stream);
  cudaMemcpyAsync(da, args.data(), sizeof(Args) * emu_ranks, cudaMemcpyHostToDevice, stream);
  void* params[] = {&dc, &de, &da};
  const int blocks = std::max(1, sms * per_sm / emu_ranks);
  cudaError_t err = cudaLaunchCooperativeKernel(emu_kernel, dim3(blocks, emu_ranks), dim3(kEpThreads), params, 0, stream);
  cudaError_t e2 = cudaStreamSynchronize(stream);
  cudaFree(dc);
  cudaFree(de);
  cudaFree(da);
  return err != cudaSuccess ? err : e2;
}

} // namespace

cudaError_t launch_ep_dispatch(const CommDev* comms, const EpDev* eps, int emu_ranks, const void* const* x,
                               const int* const* topk_idx, const float* const* topk_w, int num_tokens,
                               cudaStream_t stream) {
  const EpDev& e0 = eps[0];
  if (e0.hidden % 512 != 0 || e0.topk > 32 || e0.nranks > kMaxRanks || num_tokens > e0.max_tokens ||
      e0.num_experts % e0.nranks != 0) {
    return cudaErrorInvalidValue;
  }
  const int n = emu_ranks > 0 ? emu_ranks : 1;
  std::vector<DispatchArgs> args(n);
  for (int i = 0; i < n; ++i) args[i] = {x[i], topk_idx[i], topk_w[i], num_tokens};
  return launch_coop<DispatchArgs>(reinterpret_cast<void*>(&k_ep_dispatch), reinterpret_cast<void*>(&k_ep_dispatch_emu),
                                   comms, eps, emu_ranks, args, stream);
}

cudaError_t launch_ep_combine(const CommDev* comms, const EpDev* eps, int emu_ranks, void* const* out,
                              const float* const* weights, const void* const* bias, int num_tokens,
                              cudaStream_t stream, const int* const* send_slot, float* const* topk_w_out) {
  const EpDev& e0 = eps[0];
  if (e0.hidden % 256 != 0 || num_tokens > e0.max_tokens) return cudaErrorInvalidValue;
  const int n = emu_ranks > 0 ? emu_ranks : 1;
  std::vector<CombineArgs> args(n);
  for (int i = 0; i < n; ++i) {
    args[i] = {out[i], weights ? weights[i] : nullptr, bias ? bias[i] : nullptr, num_tokens,
               send_slot ? send_slot[i] : nullptr, topk_w_out ? topk_w_out[i] : nullptr};
  }
  return launch_coop<CombineArgs>(reinterpret_cast<void*>(&k_ep_combine), reinterpret_cast<void*>(&k_ep_combine_emu),
                                  comms, eps, emu_ranks, args, stream);
}

cudaError_t launch_ep_pull(const CommDev* comms, const EpDev* eps, int emu_ranks, void* const* out,
                           const int* const* recv_src, const int* const* num_rows, int out_rows, cudaStream_t stream) {
  const EpDev& e0 = eps[0];
  if (e0.hidden % 8 != 0 || out_rows < 0) return cudaErrorInvalidValue;
  const int n = emu_ranks > 0 ? emu_ranks : 1;
  std::vector<PullArgs> args(n);
  for (int i = 0; i < n; ++i) {
    args[i] = {out[i], recv_src ? recv_src[i] : nullptr, num_rows ? num_rows[i] : nullptr, out_rows};
  }
  return launch_coop<PullArgs>(reinterpret_cast<void*>(&k_ep_pull), reinterpret_cast<void*>(&k_ep_pull_emu), comms, eps,
                               emu_ranks, args, stream);
}

cudaError_t launch_ep_layout(const int* topk_idx, int num_tokens, int topk, int num_experts, int nranks,
                             int* tokens_per_rank, int* tokens_per_expert, int* is_token_in_rank, cudaStream_t stream) {
  if (num_experts % nranks != 0) return cudaErrorInvalidValue;
  cudaMemsetAsync(tokens_per_rank, 0, sizeof(int) * nranks, stream);
  cudaMemsetAsync(tokens_per_expert, 0, sizeof(int) * num_experts, stream);
  const int blocks = std::max(1, std::min(296, (num_tokens + 255) / 256));
  k_ep_layout<<<blocks, 256, 0, stream>>>(topk_idx, num_tokens, topk, num_experts, nranks, tokens_per_rank,
                                          tokens_per_expert, is_token_in_rank);
  note_kernel_launch();
  return cudaGetLastError();
}

} // namespace b200c
