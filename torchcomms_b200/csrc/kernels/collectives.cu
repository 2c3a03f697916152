// Peer-memory collectives for one NVSwitch domain (sm_100a).
//
// Shape of every kernel: stage this rank's contribution in its own slice of
// the symmetric heap -> per-block cross-GPU barrier -> pull from the peers'
// slices (plain 16-byte loads over NVLink, or one multimem.ld_reduce that sums
// in the switch) straight into the user's output with the scale / cast fused
// in -> barrier so the slot can be reused. Block b of a rank only ever
// touches slot b, and only synchronises with block b of the other ranks, so
// blocks drift apart and copy phases of one overlap link phases of another.
//
// Replaces, in the reference: the one-shot / two-shot IPC all-reduce
// (comms/common/algorithms/all_reduce/all_reduce_dda.cuh:20-112), the ctran
// direct reduce-scatter and all-gather kernels
// (comms/ctran/algos/ReduceScatter/ReduceScatterDirect.cuh:70-160,
// comms/ctran/algos/AllGather/AllGatherDirect.cuh:50), the prims all-to-all-v
// (comms/prims/collectives/AllToAllv.cuh:113-263) incl. split sizes resident
// on the device (comms/ctran/algos/AllToAll/DeviceAllToAllvPipes.cu), and the
// barrier-as-all-reduce of comms/torchcomms/ncclx/TorchCommNCCLX.cpp:1907-1944.
#include "collectives.h"

#include "launch_count.h"

#include <algorithm>
#include <type_traits>
#include <vector>

namespace b200c {

namespace {

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

// --------------------------------------------------------- launchers -------

template <typename Op>
__global__ void __launch_bounds__(512) k_real(CommDev c, typename Op::Args a) {
  Op::run(c, a);
}
template <typename Op>
__global__ void __launch_bounds__(512) k_emu(const CommDev* cs, const typename Op::Args* as) {
  Op::run(cs[blockIdx.y], as[blockIdx.y]);
}

template <typename Op>
cudaError_t launch_op(const CommDev* comms, int emu_ranks, const typename Op::Args* args, int blocks,
                      int threads, cudaStream_t stream) {
  using Args = typename Op::Args;
  if (blocks < 1) blocks = 1;
  if (blocks > kMaxBlocks) blocks = kMaxBlocks;
  if (threads > 512) threads = 512;
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

// ------------------------------------------------------ all-reduce ---------

// Latency mode. Piece b (kSmallPiece bytes) of the message belongs to block b:
// stage -> ONE barrier -> every rank reduces the piece from all ranks. Two
// parity halves alternate per call, so the peers' reads of call k never
// collide with the staging of call k+1, and the barrier of call k+1 orders
// them before call k+2 reuses the half.
template <typename T, RedKind R>
struct ArOneShot {
  struct Args {
    const T* in;
    T* out;
    size_t count;
    float scale;
    int use_mc;
    size_t small_off;
  };
  static __device__ void run(const CommDev& c, const Args& a) {
    constexpr int N = Pack<T>::N;
    const size_t piece_elems = kSmallPiece / sizeof(T);
    const size_t e0 = static_cast<size_t>(blockIdx.x) * piece_elems;
    if (e0 >= a.count) return;  // same decision on every rank
    const size_t n = min_sz(piece_elems, a.count - e0);
    BlockEpoch ep;
    ep.load(c, kFlagSetSmall);
    const size_t parity = (ep.value + 1) & 1u;
    const size_t off = a.small_off + parity * (static_cast<size_t>(kSmallBlocks) * kSmallPiece) +
        static_cast<size_t>(blockIdx.x) * kSmallPiece;
    block_copy(c.heap[c.rank] + off, a.in + e0, n * sizeof(T));
    const bool ok = block_barrier(c, kFlagSetSmall, ep, 0x11);
    if (ok) {
      const size_t nvec = (n + N - 1) / N;
      const bool aligned = (reinterpret_cast<uintptr_t>(a.out + e0) & 15u) == 0;
      const bool mc = a.use_mc && c.mc_heap != nullptr && R == RedKind::SUM;
      for (size_t v = threadIdx.x; v < nvec; v += blockDim.x) {
        float acc[N];
        if (mc) {
          Pack<T>::unpack(Pack<T>::mc_sum(c.mc_heap + off + v * 16), acc);
        } else {
          reduce_peers<T, R>(c, off + v * 16, acc);
        }
#pragma unroll
        for (int k = 0; k < N; ++k) acc[k] *= a.scale;
        const size_t left = n - v * N;
        store_values<T, N>(a.out + e0 + v * N, acc, left < N ? static_cast<int>(left) : N, aligned);
      }
    }
    ep.store(c, kFlagSetSmall);
  }
};

// Bandwidth mode: reduce-scatter then all-gather inside the staging slot.
template <typename T, RedKind R>
struct ArTwoShot {
  struct Args {
    const T* in;
    T* out;
    size_t count;
    float scale;
    int use_mc;
    size_t bulk_off;
    size_t chunk_elems;  // multiple of Pack<T>::N
  };
  static __device__ void run(const CommDev& c, const Args& a) {
    constexpr int N = Pack<T>::N;
    BlockEpoch ep;
    ep.load(c, kFlagSetBulk);
    const size_t chunk_bytes = a.chunk_elems * sizeof(T);
    const size_t off = a.bulk_off + static_cast<size_t>(blockIdx.x) * chunk_bytes;
    T* slot = reinterpret_cast<T*>(c.heap[c.rank] + off);
    const size_t nchunks = (a.count + a.chunk_elems - 1) / a.chunk_elems;
    const bool mc = a.use_mc && c.mc_heap != nullptr && R == RedKind::SUM;
    bool ok = true;
    for (size_t ch = blockIdx.x; ch < nchunks; ch += gridDim.x) {
      const size_t e0 = ch * a.chunk_elems;
      const size_t n = min_sz(a.chunk_elems, a.count - e0);
      block_copy(slot, a.in + e0, n * sizeof(T));
      ok = block_barrier(c, kFlagSetBulk, ep, 0x21) && ok;
      // This rank reduces vectors [v0, v1) of the chunk and hands the result
      // to every rank, in place.
      const size_t nvec = (n + N - 1) / N;
      const size_t per = (nvec + c.nranks - 1) / c.nranks;
      const size_t v0 = min_sz(nvec, per * c.rank);
      const size_t v1 = min_sz(nvec, v0 + per);
      if (ok) {
        for (size_t v = v0 + threadIdx.x; v < v1; v += blockDim.x) {
          const size_t voff = off + v * 16;
          float acc[N];
          uint4 res;
          if (mc) {
            res = Pack<T>::mc_sum(c.mc_heap + voff);
            if (a.scale != 1.0f) {
              Pack<T>::unpack(res, acc);
#pragma unroll
              for (int k = 0; k < N; ++k) acc[k] *= a.scale;
              res = Pack<T>::pack(acc);
            }
            multimem_st16(c.mc_heap + voff, res);
          } else {
            reduce_peers<T, R>(c, voff, acc);
#pragma unroll
            for (int k = 0; k < N; ++k) acc[k] *= a.scale;
            res = Pack<T>::pack(acc);
#pragma unroll
            for (int p = 0; p < kMaxRanks; ++p) {
              if (p < c.nranks) st16(c.heap[p] + voff, res);
            }
          }
        }
      }
      ok = block_barrier(c, kFlagSetBulk, ep, 0x22) && ok;
      block_copy(a.out + e0, slot, n * sizeof(T));
      __syncthreads();  // the slot is rewritten by the next step's staging
    }
    ep.store(c, kFlagSetBulk);
  }
};

// --------------------------------------------------- reduce-scatter --------

template <typename InT, typename WireT, typename OutT, RedKind R>
struct RsOp {
  struct Args {
    const InT* in;   // nranks x count
    OutT* out;       // count
    size_t count;
    float scale;
    int use_mc;
    size_t bulk_off;
    size_t chunk_elems;  // multiple of Pack<WireT>::N
  };
  static __device__ void run(const CommDev& c, const Args& a) {
    constexpr int N = Pack<WireT>::N;
    BlockEpoch ep;
    ep.load(c, kFlagSetBulk);
    const size_t sub_bytes = a.chunk_elems * sizeof(WireT);       // one peer's share of a slot
    const size_t slot_bytes = sub_bytes * c.nranks;
    const size_t off = a.bulk_off + static_cast<size_t>(blockIdx.x) * slot_bytes;
    const size_t nchunks = (a.count + a.chunk_elems - 1) / a.chunk_elems;
    const bool mc = a.use_mc && c.mc_heap != nullptr && R == RedKind::SUM;
    bool ok = true;
    for (size_t ch = blockIdx.x; ch < nchunks; ch += gridDim.x) {
      const size_t e0 = ch * a.chunk_elems;
      const size_t n = min_sz(a.chunk_elems, a.count - e0);
      // Stage, per destination p, the part of my input that p will reduce.
      for (int p = 0; p < c.nranks; ++p) {
        if (p == c.rank && !mc) continue;  // own part is read from `in` directly
        block_convert<WireT, InT>(reinterpret_cast<WireT*>(c.heap[c.rank] + off + p * sub_bytes),
                                  a.in + static_cast<size_t>(p) * a.count + e0, n);
      }
      ok = block_barrier(c, kFlagSetBulk, ep, 0x31) && ok;
      if (ok) {
        const size_t nvec = (n + N - 1) / N;
        const size_t my_off = off + static_cast<size_t>(c.rank) * sub_bytes;
        const InT* own = a.in + static_cast<size_t>(c.rank) * a.count + e0;
        const bool out_aligned = (reinterpret_cast<uintptr_t>(a.out + e0) & 15u) == 0;
        for (size_t v = threadIdx.x; v < nvec; v += blockDim.x) {
          float acc[N];
          const size_t left = n - v * N;
          const int nv = left < N ? static_cast<int>(left) : N;
          if (mc) {
            Pack<WireT>::unpack(Pack<WireT>::mc_sum(c.mc_heap + my_off + v * 16), acc);
          } else {
            uint4 pv[kMaxRanks];
#pragma unroll
            for (int i = 1; i < kMaxRanks; ++i) {
              if (i < c.nranks) {
                int p = c.rank + i;
                if (p >= c.nranks) p -= c.nranks;
                pv[i] = ld16(c.heap[p] + my_off + v * 16);
              }
            }
#pragma unroll
            for (int k = 0; k < N; ++k) {
              acc[k] = k < nv ? Pack<InT>::to_float(own[v * N + k]) : 0.0f;
            }
#pragma unroll
            for (int i = 1; i < kMaxRanks; ++i) {
              if (i < c.nranks) {
                float f[N];
                Pack<WireT>::unpack(pv[i], f);
#pragma unroll
                for (int k = 0; k < N; ++k) acc[k] = red<R>(acc[k], f[k]);
              }
            }
          }
#pragma unroll
          for (int k = 0; k < N; ++k) acc[k] *= a.scale;
          store_values<OutT, N>(a.out + e0 + v * N, acc, nv, out_aligned);
        }
      }
      ok = block_barrier(c, kFlagSetBulk, ep, 0x32) && ok;
    }
    ep.store(c, kFlagSetBulk);
  }
};

// ------------------------------------------------------- all-gather --------

// `CastT` void: raw bytes. Otherwise the input is float and is narrowed to
// CastT while staging, so that only 16-bit values cross NVLink.
template <typename CastT>
struct AgOp {
  struct Args {
    const char* in;
    char* out;
    size_t wire_bytes;   // per-rank bytes after the optional cast
    int use_mc;
    size_t bulk_off;
    size_t chunk_bytes;  // multiple of 16
  };
  static __device__ void run(const CommDev& c, const Args& a) {
    BlockEpoch ep;
    ep.load(c, kFlagSetBulk);
    const size_t off = a.bulk_off + static_cast<size_t>(blockIdx.x) * a.chunk_bytes;
    char* slot = c.heap[c.rank] + off;
    const size_t nchunks = (a.wire_bytes + a.chunk_bytes - 1) / a.chunk_bytes;
    bool ok = true;
    for (size_t ch = blockIdx.x; ch < nchunks; ch += gridDim.x) {
      const size_t b0 = ch * a.chunk_bytes;
      const size_t n = min_sz(a.chunk_bytes, a.wire_bytes - b0);
      if constexpr (std::is_same<CastT, void>::value) {
        block_copy(slot, a.in + b0, n);
      } else {
        block_convert<CastT, float>(reinterpret_cast<CastT*>(slot),
                                    reinterpret_cast<const float*>(a.in) + b0 / sizeof(CastT), n / sizeof(CastT));
      }
      ok = block_barrier(c, kFlagSetBulk, ep, 0x41) && ok;
      if (ok) {
        for (int i = 0; i < c.nranks; ++i) {
          int q = c.rank + i;
          if (q >= c.nranks) q -= c.nranks;
          block_copy(a.out + static_cast<size_t>(q) * a.wire_bytes + b0, c.heap[q] + off, n);
        }
      }
      ok = block_barrier(c, kFlagSetBulk, ep, 0x42) && ok;
    }
    ep.store(c, kFlagSetBulk);
  }
};

// ------------------------------------------------------- all-to-all --------

struct A2aOp {
  struct Args {
    const char* in;
    char* out;
    // Per-peer byte ranges. With dev_send_len != nullptr the send lengths and
    // offsets are read from device memory (int64 element counts scaled by
    // elem_bytes) and the receive lengths are learnt from the senders.
    size_t send_off[kMaxRanks], send_len[kMaxRanks], recv_off[kMaxRanks], recv_len[kMaxRanks];
    const long long* dev_send_len;   // nranks element counts, or nullptr
    const long long* dev_recv_len;   // nranks element counts (only used to place outputs), or nullptr
    size_t elem_bytes;
    size_t bulk_off;
    size_t meta_off;      // kMaxBlocks x kMaxRanks x kMaxRanks uint64 per rank
    size_t chunk_bytes;   // per-peer bytes staged per step; multiple of 16
  };
  static __device__ void run(const CommDev& c, const Args& a) {
    __shared__ size_t s_send_off[kMaxRanks], s_send_len[kMaxRanks], s_recv_off[kMaxRanks], s_recv_len[kMaxRanks];
    __shared__ size_t s_max;
    BlockEpoch ep;
    ep.load(c, kFlagSetBulk);
    // 1. Tell every peer how much it will get from me, and learn the global
    //    maximum block length so that all ranks run the same number of steps.
    unsigned long long* meta_mine =
        reinterpret_cast<unsigned long long*>(c.heap[c.rank] + a.meta_off) +
        static_cast<size_t>(blockIdx.x) * kMaxRanks * kMaxRanks;
    if (threadIdx.x < c.nranks) {
      const int p = threadIdx.x;
      size_t len, soff;
      if (a.dev_send_len != nullptr) {
        size_t acc = 0;
        for (int i = 0; i < p; ++i) acc += static_cast<size_t>(a.dev_send_len[i]);
        soff = acc * a.elem_bytes;
        len = static_cast<size_t>(a.dev_send_len[p]) * a.elem_bytes;
      } else {
        soff = a.send_off[p];
        len = a.send_len[p];
      }
      s_send_off[p] = soff;
      s_send_len[p] = len;
      // Row `rank` of peer p's table: what rank sends to each destination.
      unsigned long long* meta_p = reinterpret_cast<unsigned long long*>(c.heap[p] + a.meta_off) +
          static_cast<size_t>(blockIdx.x) * kMaxRanks * kMaxRanks + static_cast<size_t>(c.rank) * kMaxRanks;
      // Every peer gets my whole send row (needed for the global maximum).
      for (int d = 0; d < c.nranks; ++d) {
        size_t l;
        if (a.dev_send_len != nullptr) l = static_cast<size_t>(a.dev_send_len[d]) * a.elem_bytes;
        else l = a.send_len[d];
        meta_p[d] = l;
      }
    }
    bool ok = block_barrier(c, kFlagSetBulk, ep, 0x51);
    if (threadIdx.x == 0) {
      size_t mx = 0, roff = 0;
      for (int q = 0; q < c.nranks; ++q) {
        for (int d = 0; d < c.nranks; ++d) {
          const size_t l = meta_mine[q * kMaxRanks + d];
          mx = l > mx ? l : mx;
        }
        const size_t rl = meta_mine[q * kMaxRanks + c.rank];
        s_recv_len[q] = rl;
        if (a.dev_send_len != nullptr) {
          s_recv_off[q] = roff;
          roff += rl;
        } else {
          s_recv_off[q] = a.recv_off[q];
        }
      }
      s_max = mx;
    }
    __syncthreads();
    const size_t nsteps = (s_max + a.chunk_bytes - 1) / a.chunk_bytes;
    if (blockIdx.x >= nsteps) {
      // No data step for this block: still close the round, so that a peer's
      // next call cannot rewrite the count table while it is being read here.
      block_barrier(c, kFlagSetBulk, ep, 0x54);
    }
    const size_t slot_bytes = a.chunk_bytes * c.nranks;
    const size_t off = a.bulk_off + static_cast<size_t>(blockIdx.x) * slot_bytes;
    for (size_t st = blockIdx.x; st < nsteps; st += gridDim.x) {
      const size_t b0 = st * a.chunk_bytes;
      for (int p = 0; p < c.nranks; ++p) {
        if (s_send_len[p] > b0) {
          block_copy(c.heap[c.rank] + off + p * a.chunk_bytes, a.in + s_send_off[p] + b0,
                     min_sz(a.chunk_bytes, s_send_len[p] - b0));
        }
      }
      ok = block_barrier(c, kFlagSetBulk, ep, 0x52) && ok;
      if (ok) {
        for (int i = 0; i < c.nranks; ++i) {
          int q = c.rank + i;
          if (q >= c.nranks) q -= c.nranks;
          if (s_recv_len[q] > b0) {
            block_copy(a.out + s_recv_off[q] + b0, c.heap[q] + off + static_cast<size_t>(c.rank) * a.chunk_bytes,
                       min_sz(a.chunk_bytes, s_recv_len[q] - b0));
          }
        }
      }
      ok = block_barrier(c, kFlagSetBulk, ep, 0x53) && ok;
    }
    ep.store(c, kFlagSetBulk);
  }
};

// -------------------------------------------------------- broadcast --------

struct BcastOp {
  struct Args {
    char* buf;
    size_t bytes;
    int root;
    int use_mc;
    size_t bulk_off;
    size_t chunk_bytes;
  };
  static __device__ void run(const CommDev& c, const Args& a) {
    BlockEpoch ep;
    ep.load(c, kFlagSetBulk);
    const size_t off = a.bulk_off + static_cast<size_t>(blockIdx.x) * a.chunk_bytes;
    const size_t nchunks = (a.bytes + a.chunk_bytes - 1) / a.chunk_bytes;
    bool ok = true;
    for (size_t ch = blockIdx.x; ch < nchunks; ch += gridDim.x) {
      const size_t b0 = ch * a.chunk_bytes;
      const size_t n = min_sz(a.chunk_bytes, a.bytes - b0);
      if (c.rank == a.root) {
        block_copy(c.heap[c.rank] + off, a.buf + b0, n);
      }
      ok = block_barrier(c, kFlagSetBulk, ep, 0x61) && ok;
      if (ok && c.rank != a.root) {
        block_copy(a.buf + b0, c.heap[a.root] + off, n);
      }
      ok = block_barrier(c, kFlagSetBulk, ep, 0x62) && ok;
    }
    ep.store(c, kFlagSetBulk);
  }
};

struct BarrierOp {
  struct Args {
    int unused;
  };
  static __device__ void run(const CommDev& c, const Args&) {
    BlockEpoch ep;
    ep.load(c, kFlagSetBarrier);
    block_barrier(c, kFlagSetBarrier, ep, 0x71);
    ep.store(c, kFlagSetBarrier);
  }
};

// Waits for a flag value nobody will ever write; exists to exercise the
// bounded-wait path (the wait gives up after c.timeout_ns and reports).
struct WaitUnsetOp {
  struct Args {
    int unused;
  };
  static __device__ void run(const CommDev& c, const Args&) {
    if (threadIdx.x == 0) {
      const uint32_t* slot = flag_slot(c, c.rank, kFlagSetBarrier, kMaxBlocks - 1, 0);
      const uint32_t want = ld_relaxed_sys(slot) + 0x40000000u;
      wait_flag_reached(c, slot, want, 0, 0x7f);
    }
  }
};

template <typename T, RedKind R>
cudaError_t ar_dispatch(const CommDev* comms, const HeapLayout& lay, int emu, const void* const* in,
                        void* const* out, size_t count, float scale, int algo, bool use_mc, LaunchShape s,
                        cudaStream_t stream) {
  const int n = emu > 0 ? emu : 1;
  if (algo == 0) {
    using Op = ArOneShot<T, R>;
    std::vector<typename Op::Args> args(n);
    for (int i = 0; i < n; ++i) {
      args[i] = {static_cast<const T*>(in[i]), static_cast<T*>(out[i]), count, scale, use_mc ? 1 : 0, lay.small_off};
    }
    const size_t bytes = count * sizeof(T);
    const int blocks = static_cast<int>((bytes + kSmallPiece - 1) / kSmallPiece);
    if (blocks > kSmallBlocks) return cudaErrorInvalidValue;
    return launch_op<Op>(comms, emu, args.data(), blocks, s.threads, stream);
  }
  using Op = ArTwoShot<T, R>;
  constexpr size_t kVec = Pack<T>::N;
  size_t chunk_elems = s.chunk_bytes / sizeof(T);
  chunk_elems = (chunk_elems / kVec) * kVec;
  if (chunk_elems == 0) return cudaErrorInvalidValue;
  if (static_cast<size_t>(s.blocks) * chunk_elems * sizeof(T) > lay.bulk_bytes) return cudaErrorInvalidValue;
  std::vector<typename Op::Args> args(n);
  for (int i = 0; i < n; ++i) {
    args[i] = {static_cast<const T*>(in[i]), static_cast<T*>(out[i]), count, scale, use_mc ? 1 : 0, lay.bulk_off, chunk_elems};
  }
  const size_t nchunks = (count + chunk_elems - 1) / chunk_elems;
  const int blocks = static_cast<int>(std::min<size_t>(s.blocks, std::max<size_t>(nchunks, 1)));
  return launch_op<Op>(comms, emu, args.data(), blocks, s.threads, stream);
}

template <typename T>
cudaError_t ar_dispatch_red(const CommDev* comms, const HeapLayout& lay, int emu, const void* const* in,
                            void* const* out, size_t count, RedKind red, float scale, int algo, bool use_mc,
                            LaunchShape s, cudaStream_t stream) {
  switch (red) {
    case RedKind::SUM: return ar_dispatch<T, RedKind::SUM>(comms, lay, emu, in, out, count, scale, algo, use_mc, s, stream);
    case RedKind::PROD: return ar_dispatch<T, RedKind::PROD>(comms, lay, emu, in, out, count, scale, algo, false, s, stream);
    case RedKind::MIN: return ar_dispatch<T, RedKind::MIN>(comms, lay, emu, in, out, count, scale, algo, false, s, stream);
    case RedKind::MAX: return ar_dispatch<T, RedKind::MAX>(comms, lay, emu, in, out, count, scale, algo, false, s, stream);
  }
  return cudaErrorInvalidValue;
}

template <typename InT, typename WireT, typename OutT, RedKind R>
cudaError_t rs_dispatch(const CommDev* comms, const HeapLayout& lay, int emu, const void* const* in,
                        void* const* out, size_t count, float scale, bool use_mc, LaunchShape s,
                        cudaStream_t stream) {
  using Op = RsOp<InT, WireT, OutT, R>;
  const int n = emu > 0 ? emu : 1;
  const int nranks = comms[0].nranks;
  constexpr size_t kVec = Pack<WireT>::N;
  size_t chunk_elems = s.chunk_bytes / sizeof(WireT);
  chunk_elems = (chunk_elems / kVec) * kVec;
  if (chunk_elems == 0) return cudaErrorInvalidValue;
  if (static_cast<size_t>(s.blocks) * chunk_elems * sizeof(WireT) * nranks > lay.bulk_bytes) return cudaErrorInvalidValue;
  std::vector<typename Op::Args> args(n);
  for (int i = 0; i < n; ++i) {
    args[i] = {static_cast<const InT*>(in[i]), static_cast<OutT*>(out[i]), count, scale, use_mc ? 1 : 0, lay.bulk_off, chunk_elems};
  }
  const size_t nchunks = (count + chunk_elems - 1) / chunk_elems;
  const int blocks = static_cast<int>(std::min<size_t>(s.blocks, std::max<size_t>(nchunks, 1)));
  return launch_op<Op>(comms, emu, args.data(), blocks, s.threads, stream);
}

template <typename T>
cudaError_t rs_same(const CommDev* comms, const HeapLayout& lay, int emu, const void* const* in, void* const* out,
                    size_t count, RedKind red, float scale, bool use_mc, LaunchShape s, cudaStream_t stream) {
  switch (red) {
    case RedKind::SUM: return rs_dispatch<T, T, T, RedKind::SUM>(comms, lay, emu, in, out, count, scale, use_mc, s, stream);
    case RedKind::PROD: return rs_dispatch<T, T, T, RedKind::PROD>(comms, lay, emu, in, out, count, scale, false, s, stream);
    case RedKind::MIN: return rs_dispatch<T, T, T, RedKind::MIN>(comms, lay, emu, in, out, count, scale, false, s, stream);
    case RedKind::MAX: return rs_dispatch<T, T, T, RedKind::MAX>(comms, lay, emu, in, out, count, scale, false, s, stream);
  }
  return cudaErrorInvalidValue;
}

} // namespace

cudaError_t launch_all_reduce(const CommDev* comms, const HeapLayout& lay, int emu_ranks, const void* const* in,
                              void* const* out, size_t count, DType dtype, RedKind red, float scale, int algo,
                              bool use_mc, LaunchShape shape, cudaStream_t stream) {
  switch (dtype) {
    case DType::F32: return ar_dispatch_red<float>(comms, lay, emu_ranks, in, out, count, red, scale, algo, use_mc, shape, stream);
    case DType::F16: return ar_dispatch_red<__half>(comms, lay, emu_ranks, in, out, count, red, scale, algo, use_mc, shape, stream);
    case DType::BF16: return ar_dispatch_red<__nv_bfloat16>(comms, lay, emu_ranks, in, out, count, red, scale, algo, use_mc, shape, stream);
  }
  return cudaErrorInvalidValue;
}

cudaError_t launch_reduce_scatter(const CommDev* comms, const HeapLayout& lay, int emu_ranks, const void* const* in,
                                  void* const* out, size_t count, DType in_dtype, DType wire_dtype, DType out_dtype,
                                  RedKind red, float scale, bool use_mc, LaunchShape shape, cudaStream_t stream) {
  using bf16 = __nv_bfloat16;
  if (in_dtype == wire_dtype && wire_dtype == out_dtype) {
    switch (in_dtype) {
      case DType::F32: return rs_same<float>(comms, lay, emu_ranks, in, out, count, red, scale, use_mc, shape, stream);
      case DType::F16: return rs_same<__half>(comms, lay, emu_ranks, in, out, count, red, scale, use_mc, shape, stream);
      case DType::BF16: return rs_same<bf16>(comms, lay, emu_ranks, in, out, count, red, scale, use_mc, shape, stream);
    }
  }
  if (wire_dtype != DType::BF16 || red != RedKind::SUM) return cudaErrorInvalidValue;
  if (in_dtype == DType::F32 && out_dtype == DType::F32)
    return rs_dispatch<float, bf16, float, RedKind::SUM>(comms, lay, emu_ranks, in, out, count, scale, use_mc, shape, stream);
  if (in_dtype == DType::F32 && out_dtype == DType::BF16)
    return rs_dispatch<float, bf16, bf16, RedKind::SUM>(comms, lay, emu_ranks, in, out, count, scale, use_mc, shape, stream);
  if (in_dtype == DType::BF16 && out_dtype == DType::F32)
    return rs_dispatch<bf16, bf16, float, RedKind::SUM>(comms, lay, emu_ranks, in, out, count, scale, use_mc, shape, stream);
  return cudaErrorInvalidValue;
}

cudaError_t launch_all_gather(const CommDev* comms, const HeapLayout& lay, int emu_ranks, const void* const* in,
                              void* const* out, size_t bytes, bool cast_f32_to_bf16, bool use_mc, LaunchShape shape,
                              cudaStream_t stream) {
  const int n = emu_ranks > 0 ? emu_ranks : 1;
  const size_t chunk = (shape.chunk_bytes / 16) * 16;
  if (chunk == 0 || static_cast<size_t>(shape.blocks) * chunk > lay.bulk_bytes) return cudaErrorInvalidValue;
  const size_t wire = cast_f32_to_bf16 ? bytes / 2 : bytes;
  const size_t nchunks = (wire + chunk - 1) / chunk;
  const int blocks = static_cast<int>(std::min<size_t>(shape.blocks, std::max<size_t>(nchunks, 1)));
  if (cast_f32_to_bf16) {
    using Op = AgOp<__nv_bfloat16>;
    std::vector<Op::Args> args(n);
    for (int i = 0; i < n; ++i)
      args[i] = {static_cast<const char*>(in[i]), static_cast<char*>(out[i]), wire, use_mc ? 1 : 0, lay.bulk_off, chunk};
    return launch_op<Op>(comms, emu_ranks, args.data(), blocks, shape.threads, stream);
  }
  using Op = AgOp<void>;
  std::vector<Op::Args> args(n);
  for (int i = 0; i < n; ++i)
    args[i] = {static_cast<const char*>(in[i]), static_cast<char*>(out[i]), wire, use_mc ? 1 : 0, lay.bulk_off, chunk};
  return launch_op<Op>(comms, emu_ranks, args.data(), blocks, shape.threads, stream);
}

cudaError_t launch_all_to_all(const CommDev* comms, const HeapLayout& lay, int emu_ranks, const void* const* in,
                              void* const* out, const size_t* send_off, const size_t* send_len,
                              const size_t* recv_off, const size_t* recv_len, size_t max_len, LaunchShape shape,
                              cudaStream_t stream) {
  const int n = emu_ranks > 0 ? emu_ranks : 1;
  const int nranks = comms[0].nranks;
  const size_t chunk = (shape.chunk_bytes / 16) * 16;
  if (chunk == 0 || static_cast<size_t>(shape.blocks) * chunk * nranks > lay.bulk_bytes) return cudaErrorInvalidValue;
  std::vector<A2aOp::Args> args(n);
  for (int i = 0; i < n; ++i) {
    A2aOp::Args& a = args[i];
    a = {};
    a.in = static_cast<const char*>(in[i]);
    a.out = static_cast<char*>(out[i]);
    for (int p = 0; p < nranks; ++p) {
      a.send_off[p] = send_off[i * nranks + p];
      a.send_len[p] = send_len[i * nranks + p];
      a.recv_off[p] = recv_off[i * nranks + p];
      a.recv_len[p] = recv_len[i * nranks + p];
    }
    a.dev_send_len = nullptr;
    a.dev_recv_len = nullptr;
    a.elem_bytes = 1;
    a.bulk_off = lay.bulk_off;
    a.meta_off = lay.small_off + 2 * static_cast<size_t>(kSmallBlocks) * kSmallPiece;
    a.chunk_bytes = chunk;
  }
  // The grid must be identical on every rank, and ranks see different split
  // sizes: the caller picks `shape.blocks` from rank-independent facts only.
  // The kernel learns the global maximum block length by itself.
  (void)max_len;
  return launch_op<A2aOp>(comms, emu_ranks, args.data(), shape.blocks, shape.threads, stream);
}

cudaError_t launch_all_to_all_device_splits(const CommDev* comms, const HeapLayout& lay, int emu_ranks,
                                            const void* const* in, void* const* out,
                                            const long long* const* dev_send_counts, size_t elem_bytes,
                                            LaunchShape shape, cudaStream_t stream) {
  const int n = emu_ranks > 0 ? emu_ranks : 1;
  const int nranks = comms[0].nranks;
  const size_t chunk = (shape.chunk_bytes / 16) * 16;
  if (chunk == 0 || static_cast<size_t>(shape.blocks) * chunk * nranks > lay.bulk_bytes) return cudaErrorInvalidValue;
  std::vector<A2aOp::Args> args(n);
  for (int i = 0; i < n; ++i) {
    A2aOp::Args& a = args[i];
    a = {};
    a.in = static_cast<const char*>(in[i]);
    a.out = static_cast<char*>(out[i]);
    a.dev_send_len = dev_send_counts[i];
    a.dev_recv_len = nullptr;
    a.elem_bytes = elem_bytes;
    a.bulk_off = lay.bulk_off;
    a.meta_off = lay.small_off + 2 * static_cast<size_t>(kSmallBlocks) * kSmallPiece;
    a.chunk_bytes = chunk;
  }
  return launch_op<A2aOp>(comms, emu_ranks, args.data(), shape.blocks, shape.threads, stream);
}

cudaError_t launch_broadcast(const CommDev* comms, const HeapLayout& lay, int emu_ranks, void* const* buf,
                             size_t bytes, int root, bool use_mc, LaunchShape shape, cudaStream_t stream) {
  const int n = emu_ranks > 0 ? emu_ranks : 1;
  const size_t chunk = (shape.chunk_bytes / 16) * 16;
  if (chunk == 0 || static_cast<size_t>(shape.blocks) * chunk > lay.bulk_bytes) return cudaErrorInvalidValue;
  std::vector<BcastOp::Args> args(n);
  for (int i = 0; i < n; ++i) args[i] = {static_cast<char*>(buf[i]), bytes, root, use_mc ? 1 : 0, lay.bulk_off, chunk};
  const size_t nchunks = (bytes + chunk - 1) / chunk;
  const int blocks = static_cast<int>(std::min<size_t>(shape.blocks, std::max<size_t>(nchunks, 1)));
  return launch_op<BcastOp>(comms, emu_ranks, args.data(), blocks, shape.threads, stream);
}

cudaError_t launch_barrier(const CommDev* comms, int emu_ranks, cudaStream_t stream) {
  const int n = emu_ranks > 0 ? emu_ranks : 1;
  std::vector<BarrierOp::Args> args(n);
  return launch_op<BarrierOp>(comms, emu_ranks, args.data(), 1, 32, stream);
}

cudaError_t launch_wait_unset_flag(const CommDev* comms, int emu_ranks, cudaStream_t stream) {
  const int n = emu_ranks > 0 ? emu_ranks : 1;
  std::vector<WaitUnsetOp::Args> args(n);
  return launch_op<WaitUnsetOp>(comms, emu_ranks, args.data(), 1, 32, stream);
}

} // namespace b200c
