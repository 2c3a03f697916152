// Low-latency MoE dispatch / combine kernels (sm_100a). See moe_ep_ll.h.
#include "moe_ep_ll.h"

#include <cooperative_groups.h>
#include <cuda_bf16.h>
#include <cuda_fp8.h>

#include <algorithm>
#include <vector>

#include "launch_count.h"

namespace cg = cooperative_groups;

namespace b200c {

namespace {

constexpr int kLlThreads = 256;
constexpr int kLlWarps = kLlThreads / 32;
constexpr int kLlChunkCols = 1024;  // columns of one work item of the send and combine loops (a multiple of 512)

__device__ __forceinline__ float2 bf2f(uint32_t v) {
  return make_float2(__uint_as_float(v << 16), __uint_as_float(v & 0xffff0000u));
}

// Waits until the count word carries this call's tag; returns the count, or -1
// when the wait ran out (the status word then says who was waited for).
__device__ __forceinline__ int wait_count(const CommDev& c, const unsigned long long* addr, unsigned int call, int peer) {
  unsigned long long start = 0, next_status = 0;
  uint32_t spins = 0;
  while (true) {
    const uint64_t v = ld_acquire_sys_u64(reinterpret_cast<const uint64_t*>(addr));
    if (static_cast<unsigned int>(v >> 32) == call) return static_cast<int>(v & 0xffffffffull);
    if (++spins >= 64u) {
      spins = 0;
      const unsigned long long now = globaltimer_ns();
      if (start == 0) {
        start = now;
        next_status = now + 200000ull;
      } else if (now >= next_status) {
        next_status = now + 200000ull;
        if (comm_is_dead(c)) return -1;
        if (now - start > c.timeout_ns) {
          report_timeout(c, peer, 0xa2);
          return -1;
        }
      }
    }
  }
}

struct LlDispatchArgs {
  const void* x;        // [num_tokens, hidden] bf16
  const int* topk_idx;  // [num_tokens, topk]
  EpLlRecv recv;
  int num_tokens;
};

__device__ void ll_dispatch_body(const CommDev& c, const EpLlDev& e, const LlDispatchArgs& a) {
  cg::grid_group grid = cg::this_grid();
  __shared__ int s_cnt[kMaxRanks];
  __shared__ int s_beg[kMaxRanks + 1];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int gwarp = blockIdx.x * kLlWarps + warp, nwarps = gridDim.x * kLlWarps;
  const int gtid = blockIdx.x * kLlThreads + threadIdx.x, gthreads = gridDim.x * kLlThreads;
  const int E = e.num_experts, N = e.nranks, M = e.max_tokens, Le = e.experts_per_rank;
  const unsigned int call = *e.call + 1;  // block 0 stores the new value after the first grid-wide meeting
  const int par = static_cast<int>(call & 1u);
  int* cnt = e.cnt + par * E;
  for (int i = gtid; i < E; i += gthreads) e.cnt[(par ^ 1) * E + i] = 0;  // the next call's counters

  const int groups = e.hidden / 128;
  const size_t row_bytes = e.fp8 ? static_cast<size_t>(e.hidden) : static_cast<size_t>(e.hidden) * 2;
  const size_t par_rows = static_cast<size_t>(par) * Le * N * M;

  trace_mark(c, 0);
  // A0. number the rows per expert (one warp per token)
  for (int t = gwarp; t < a.num_tokens; t += nwarps) {
    if (lane < e.topk) {
      const int idx = a.topk_idx[static_cast<size_t>(t) * e.topk + lane];
      int i = -1;
      if (idx >= 0 && idx < E) {
        i = atomicAdd(&cnt[idx], 1);
        if (i >= M) {  // more rows than a slot group holds: cannot happen while num_tokens <= max_tokens
          c.status[0] = c.status[0] | kStatusBadArg;
          i = -1;
        }
      }
      e.send_slot[static_cast<size_t>(t) * e.topk + lane] = i;
      if (i >= 0) {
        const int d = idx / Le;
        e.slot_src[d][par_rows + (static_cast<size_t>(idx - d * Le) * N + e.rank) * M + i] = t;
      }
    }
  }
  grid.sync();
  trace_mark(c, 1);
  if (blockIdx.x == 0 && threadIdx.x == 0) *e.call = call;

  // B. the row counts are final: tagged with the call, they go to every rank ahead of the rows
  for (int i = gtid; i < E * N; i += gthreads) {
    const int ex = i / N, p = i - ex * N;
    const unsigned long long v = (static_cast<unsigned long long>(call) << 32) | static_cast<unsigned int>(cnt[ex]);
    st_release_sys_u64(reinterpret_cast<uint64_t*>(e.counts[p] + (static_cast<size_t>(par) * E + ex) * N + e.rank), v);
  }
  trace_mark(c, 2);

  // A1. store the rows into their fixed slots; one work item = one token x kLlChunkCols columns
  const int nchunks = (e.hidden + kLlChunkCols - 1) / kLlChunkCols;
  for (int item = gwarp; item < a.num_tokens * nchunks; item += nwarps) {
    const int t = item / nchunks;
    const int col_lo = (item - t * nchunks) * kLlChunkCols;
    const int col_hi = min(e.hidden, col_lo + kLlChunkCols);
    int d = -1;
    long long row = -1;
    if (lane < e.topk) {
      const int idx = a.topk_idx[static_cast<size_t>(t) * e.topk + lane];
      const int i = e.send_slot[static_cast<size_t>(t) * e.topk + lane];
      if (i >= 0) {
        d = idx / Le;
        row = static_cast<long long>(par_rows) + (static_cast<long long>(idx - d * Le) * N + e.rank) * M + i;
      }
    }
    const __nv_bfloat16* xr = static_cast<const __nv_bfloat16*>(a.x) + static_cast<size_t>(t) * e.hidden;
    for (int e0 = col_lo + lane * 16; e0 < col_hi; e0 += 512) {
      const uint4 v0 = ld16(xr + e0);
      const uint4 v1 = ld16(xr + e0 + 8);
      if (!e.fp8) {
        for (int k = 0; k < e.topk; ++k) {
          const int dk = __shfl_sync(0xffffffffu, d, k);
          const long long rk = __shfl_sync(0xffffffffu, row, k);
          if (dk < 0) continue;
          char* dst = e.slot_x[dk] + static_cast<size_t>(rk) * row_bytes + static_cast<size_t>(e0) * 2;
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
        const __nv_fp8x2_storage_t lo =
            __nv_cvt_float2_to_fp8x2(make_float2(f[4 * i] * inv, f[4 * i + 1] * inv), __NV_SATFINITE, __NV_E4M3);
        const __nv_fp8x2_storage_t hi =
            __nv_cvt_float2_to_fp8x2(make_float2(f[4 * i + 2] * inv, f[4 * i + 3] * inv), __NV_SATFINITE, __NV_E4M3);
        q[i] = static_cast<uint32_t>(lo) | (static_cast<uint32_t>(hi) << 16);
      }
      const uint4 packed = make_uint4(q[0], q[1], q[2], q[3]);
      const int group = e0 / 128;
      for (int k = 0; k < e.topk; ++k) {
        const int dk = __shfl_sync(0xffffffffu, d, k);
        const long long rk = __shfl_sync(0xffffffffu, row, k);
        if (dk < 0) continue;
        st16(e.slot_x[dk] + static_cast<size_t>(rk) * row_bytes + e0, packed);
        if ((lane & 7) == 0) e.slot_scales[dk][static_cast<size_t>(rk) * groups + group] = scale;
      }
    }
    // This piece of every row is stored: tell the receivers (release-ordered, after the whole warp's stores).
    __syncwarp();
    if (d >= 0) red_add_release_sys_u32(e.slot_arrived[d] + row, 1u);
  }
  trace_mark(c, 3);

  // C1. where this rank's rows sit in each expert's packed tensor (the combine reads from there)
  const unsigned long long* mine = e.counts[e.rank] + static_cast<size_t>(par) * E * N;
  for (int ex = gtid; ex < E; ex += gthreads) {
    int b = 0;
    for (int s = 0; s < e.rank; ++s) {
      const int n = wait_count(c, mine + static_cast<size_t>(ex) * N + s, call, s);
      if (n < 0) break;
      b += n;
    }
    e.begin[ex] = b;
  }

  trace_mark(c, 4);
  // C2. pack the rows of each local expert, sources in rank order
  const int nsub = max(1, static_cast<int>(gridDim.x) / Le);
  for (int item = blockIdx.x; item < Le * nsub; item += gridDim.x) {
    const int le = item % Le, sub = item / Le;
    __syncthreads();
    if (threadIdx.x < N) {
      s_cnt[threadIdx.x] = wait_count(c, mine + static_cast<size_t>(e.rank * Le + le) * N + threadIdx.x, call, threadIdx.x);
    }
    __syncthreads();
    if (threadIdx.x == 0) {
      bool ok = true;
      for (int s = 0; s < N; ++s) ok = ok && s_cnt[s] >= 0 && s_cnt[s] <= M;
      int b = 0;
      for (int s = 0; s < N; ++s) {  // nothing is copied after a failed wait
        s_beg[s] = b;
        b += ok ? s_cnt[s] : 0;
      }
      s_beg[N] = b;
    }
    __syncthreads();
    const int total = s_beg[N];
    if (sub == 0) {
      if (threadIdx.x == 0) a.recv.packed_count[le] = total;
      if (threadIdx.x < N) {
        const int s = threadIdx.x;
        a.recv.layout_range[le * N + s] =
            (static_cast<long long>(s_beg[s]) << 32) | static_cast<unsigned int>(s_beg[s + 1] - s_beg[s]);
      }
    }
    for (int j = sub * kLlWarps + warp; j < total; j += nsub * kLlWarps) {
      int s = 0;
      while (s + 1 < N && j >= s_beg[s + 1]) ++s;
      const size_t from_row = par_rows + (static_cast<size_t>(le) * N + s) * M + (j - s_beg[s]);
      const size_t to_row = static_cast<size_t>(le) * N * M + j;
      // every piece of the row has landed?
      int landed = 1;
      if (lane == 0) {
        landed = wait_flag_reached(c, e.slot_arrived[e.rank] + from_row, static_cast<uint32_t>(nchunks), s, 0xa5) ? 1 : 0;
        e.slot_arrived[e.rank][from_row] = 0;   // this parity's slot is written again two calls from now
      }
      landed = __shfl_sync(0xffffffffu, landed, 0);
      if (!landed) continue;
      const char* from = e.slot_x[e.rank] + from_row * row_bytes;
      char* to = static_cast<char*>(a.recv.packed_x) + to_row * row_bytes;
      for (size_t b = static_cast<size_t>(lane) * 16; b < row_bytes; b += 512) st16(to + b, ld16_stream(from + b));
      if (e.fp8) {
        for (int g = lane; g < groups; g += 32) {
          a.recv.packed_scales[to_row * groups + g] = e.slot_scales[e.rank][from_row * groups + g];
        }
      }
      if (lane == 0) a.recv.packed_src[to_row] = e.slot_src[e.rank][from_row];
    }
  }
  trace_mark(c, 5);
}

__global__ void __launch_bounds__(kLlThreads) k_ep_ll_dispatch(CommDev c, EpLlDev e, LlDispatchArgs a) {
  ll_dispatch_body(c, e, a);
}
__global__ void __launch_bounds__(kLlThreads)
    k_ep_ll_dispatch_emu(const CommDev* cs, const EpLlDev* es, const LlDispatchArgs* as) {
  ll_dispatch_body(cs[blockIdx.y], es[blockIdx.y], as[blockIdx.y]);
}

struct LlCombineArgs {
  void* out;             // [num_tokens, hidden] bf16
  const int* topk_idx;   // [num_tokens, topk]
  const float* topk_w;   // [num_tokens, topk]
  const int* send_slot;  // handles of the dispatch to undo; nullptr = the last one's
  const int* begin;
  int num_tokens;
};

__device__ void ll_combine_body(const CommDev& c, const EpLlDev& e, const LlCombineArgs& a) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int gwarp = blockIdx.x * kLlWarps + warp, nwarps = gridDim.x * kLlWarps;
  const int N = e.nranks, M = e.max_tokens, Le = e.experts_per_rank;
  const size_t row_bytes = static_cast<size_t>(e.hidden) * 2;
  const int* send_slot = a.send_slot != nullptr ? a.send_slot : e.send_slot;
  const int* begin = a.begin != nullptr ? a.begin : e.begin;
  BlockEpoch ep;
  ep.load(c, kFlagSetEp);
  trace_mark(c, 0);
  bool ok = block_barrier(c, kFlagSetEp, ep, 0xa3);  // every rank's expert outputs are complete
  trace_mark(c, 1);
  if (ok) {
    // One work item = one token x kLlChunkCols columns, so that a decode batch still fills the GPU with loads.
    const int nchunks = (e.hidden + kLlChunkCols - 1) / kLlChunkCols;
    for (int item = gwarp; item < a.num_tokens * nchunks; item += nwarps) {
      const int t = item / nchunks;
      const int col_lo = (item - t * nchunks) * kLlChunkCols;
      const int col_hi = min(e.hidden, col_lo + kLlChunkCols);
      int d = -1;
      long long off = 0;
      float w = 0.0f;
      if (lane < e.topk) {
        const int idx = a.topk_idx[static_cast<size_t>(t) * e.topk + lane];
        const int i = send_slot[static_cast<size_t>(t) * e.topk + lane];
        if (idx >= 0 && idx < e.num_experts && i >= 0) {
          const int pos = begin[idx] + i;
          if (pos < N * M) {
            d = idx / Le;
            off = (static_cast<long long>(idx - d * Le) * N * M + pos) * static_cast<long long>(row_bytes);
            w = a.topk_w[static_cast<size_t>(t) * e.topk + lane];
          } else {  // a handle that does not belong to these counts: never read through it
            c.status[0] = c.status[0] | kStatusBadArg;
          }
        }
      }
      for (int e0 = col_lo + lane * 8; e0 < col_hi; e0 += 256) {
        float acc[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) acc[i] = 0.0f;
        for (int k0 = 0; k0 < e.topk; k0 += 8) {
          uint4 rows[8];
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            const int k = k0 + i;
            const int dk = __shfl_sync(0xffffffffu, d, k & 31);
            const long long ok_off = __shfl_sync(0xffffffffu, off, k & 31);
            if (k < e.topk && dk >= 0) rows[i] = ld16_stream(e.out_x[dk] + ok_off + static_cast<size_t>(e0) * 2);
          }
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            const int k = k0 + i;
            const int dk = __shfl_sync(0xffffffffu, d, k & 31);
            const float wk = __shfl_sync(0xffffffffu, w, k & 31);
            if (k < e.topk && dk >= 0) {
              const uint32_t* p = &rows[i].x;
#pragma unroll
              for (int j = 0; j < 4; ++j) {
                const float2 f = bf2f(p[j]);
                acc[2 * j] += wk * f.x;
                acc[2 * j + 1] += wk * f.y;
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
        st16(static_cast<__nv_bfloat16*>(a.out) + static_cast<size_t>(t) * e.hidden + e0, o);
      }
    }
    trace_mark(c, 2);
    ok = block_barrier(c, kFlagSetEp, ep, 0xa4);  // nobody overwrites its outputs while a peer still reads them
    trace_mark(c, 3);
  }
  ep.store(c, kFlagSetEp);
}

__global__ void __launch_bounds__(kLlThreads) k_ep_ll_combine(CommDev c, EpLlDev e, LlCombineArgs a) {
  ll_combine_body(c, e, a);
}
__global__ void __launch_bounds__(kLlThreads)
    k_ep_ll_combine_emu(const CommDev* cs, const EpLlDev* es, const LlCombineArgs* as) {
  ll_combine_body(cs[blockIdx.y], es[blockIdx.y], as[blockIdx.y]);
}

// One cooperative launch with every block resident (the dispatch meets grid-wide, both wait on peers).
template <typename Args>
cudaError_t launch_ll(void* real_kernel, void* emu_kernel, const CommDev* comms, const EpLlDev* eps, int emu_ranks,
                      const std::vector<Args>& args, cudaStream_t stream) {
  int dev = 0, sms = 0, per_sm = 0;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, real_kernel, kLlThreads, 0);
  if (per_sm < 1) return cudaErrorLaunchOutOfResources;
  note_kernel_launch();
  if (emu_ranks <= 0) {
    CommDev c = comms[0];
    EpLlDev e = eps[0];
    Args a = args[0];
    void* params[] = {&c, &e, &a};
    return cudaLaunchCooperativeKernel(real_kernel, dim3(sms), dim3(kLlThreads), params, 0, stream);
  }
  CommDev* dc = nullptr;
  EpLlDev* de = nullptr;
  Args* da = nullptr;
  cudaMalloc(&dc, sizeof(CommDev) * emu_ranks);
  cudaMalloc(&de, sizeof(EpLlDev) * emu_ranks);
  cudaMalloc(&da, sizeof(Args) * emu_ranks);
  cudaMemcpyAsync(dc, comms, sizeof(CommDev) * emu_ranks, cudaMemcpyHostToDevice, stream);
  cudaMemcpyAsync(de, eps, sizeof(EpLlDev) * emu_ranks, cudaMemcpyHostToDevice, stream);
  cudaMemcpyAsync(da, args.data(), sizeof(Args) * emu_ranks, cudaMemcpyHostToDevice, stream);
  void* params[] = {&dc, &de, &da};
  const int blocks = std::max(1, sms / emu_ranks);
  cudaError_t err = cudaLaunchCooperativeKernel(emu_kernel, dim3(blocks, emu_ranks), dim3(kLlThreads), params, 0, stream);
  cudaError_t e2 = cudaStreamSynchronize(stream);
  cudaFree(dc);
  cudaFree(de);
  cudaFree(da);
  return err != cudaSuccess ? err : e2;
}

} // namespace

cudaError_t launch_ep_ll_dispatch(const CommDev* comms, const EpLlDev* eps, int emu_ranks, const void* const* x,
                                  const int* const* topk_idx, const EpLlRecv* recv, int num_tokens, cudaStream_t stream) {
  const EpLlDev& e0 = eps[0];
  if (e0.hidden % 512 != 0 || e0.topk < 1 || e0.topk > 32 || e0.nranks > kMaxRanks || num_tokens > e0.max_tokens ||
      e0.num_experts % e0.nranks != 0) {
    return cudaErrorInvalidValue;
  }
  const int n = emu_ranks > 0 ? emu_ranks : 1;
  std::vector<LlDispatchArgs> args(n);
  for (int i = 0; i < n; ++i) args[i] = {x[i], topk_idx[i], recv[i], num_tokens};
  return launch_ll<LlDispatchArgs>(reinterpret_cast<void*>(&k_ep_ll_dispatch),
                                   reinterpret_cast<void*>(&k_ep_ll_dispatch_emu), comms, eps, emu_ranks, args, stream);
}

cudaError_t launch_ep_ll_combine(const CommDev* comms, const EpLlDev* eps, int emu_ranks, void* const* out,
                                 const int* const* topk_idx, const float* const* topk_w, int num_tokens,
                                 const int* const* send_slot, const int* const* begin, cudaStream_t stream) {
  const EpLlDev& e0 = eps[0];
  if (e0.hidden % 256 != 0 || e0.topk > 32 || num_tokens > e0.max_tokens) return cudaErrorInvalidValue;
  const int n = emu_ranks > 0 ? emu_ranks : 1;
  std::vector<LlCombineArgs> args(n);
  for (int i = 0; i < n; ++i) {
    args[i] = {out[i], topk_idx[i], topk_w[i], send_slot ? send_slot[i] : nullptr, begin ? begin[i] : nullptr, num_tokens};
  }
  return launch_ll<LlCombineArgs>(reinterpret_cast<void*>(&k_ep_ll_combine), reinterpret_cast<void*>(&k_ep_ll_combine_emu),
                                  comms, eps, emu_ranks, args, stream);
}

} // namespace b200c
