// All-reduce over the symmetric heap (sm_100a): a one-shot latency kernel and
// a pipelined two-shot bandwidth kernel, each with an NVLS (multimem) and a
// plain peer load/store data path, scale and cast fused in.
//
// Replaces, in the reference: comms/common/algorithms/all_reduce/all_reduce_dda.cuh:20-112
// (flat one-shot and tree two-shot over IPC buffers) and the custom multimem
// all-reduce kernels under comms/ncclx/v2_31/contrib/custom_algos/allreduce.
#include "coll_common.cuh"

namespace b200c {
namespace coll {

// Latency mode. Piece b (kSmallPiece bytes, one 16-byte vector per thread) of
// the message belongs to block b: stage -> ONE barrier -> every rank reduces
// the piece from all ranks. Two parity halves alternate per call, so the
// peers' reads of call k never collide with the staging of call k+1, and the
// barrier of call k+1 orders them before call k+2 reuses the half.
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
    trace_mark(c, 0);
    block_copy(c.heap[c.rank] + off, a.in + e0, n * sizeof(T));
    trace_mark(c, 1);
    const bool ok = block_barrier(c, kFlagSetSmall, ep, 0x11);
    trace_mark(c, 2);
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
    trace_mark(c, 3);
    ep.store(c, kFlagSetSmall);
  }
};

// Bandwidth mode: a three-stage software pipeline per block over a ring of
// kPipeSlots staging slots.
//   A(k): copy chunk k of the input into slot k % S, post "ready k"
//   B(k): once every rank is ready with chunk k, reduce this rank's share of
//         it (switch reduction or peer loads) and write the result into every
//         rank's slot, post "done k"
//   C(k): once every rank is done with chunk k, copy the slot to the output
// Iteration i runs A(i), B(i-1), C(i-2) and posts both flags behind a single
// fence, so each wait is for a flag posted a whole stage earlier.
template <typename T, RedKind R>
struct ArPipe {
  struct Args {
    const T* in;
    T* out;
    size_t count;
    float scale;
    int use_mc;
    size_t bulk_off;
    size_t chunk_elems;  // multiple of Pack<T>::N
  };

  static __device__ __forceinline__ void reduce_share(const CommDev& c, const Args& a, size_t off, size_t n, bool mc) {
    constexpr int N = Pack<T>::N;
    const size_t nvec = (n + N - 1) / N;
    const size_t per = (nvec + c.nranks - 1) / c.nranks;
    const size_t v0 = min_sz(nvec, per * c.rank);
    const size_t v1 = min_sz(nvec, v0 + per);
    if (mc) {
      // Four independent switch reductions in flight per thread: a single
      // multimem.ld_reduce has microseconds of latency.
      constexpr int U = 4;
      for (size_t v = v0 + threadIdx.x; v < v1; v += static_cast<size_t>(U) * blockDim.x) {
        uint4 res[U];
#pragma unroll
        for (int u = 0; u < U; ++u) {
          const size_t vv = v + static_cast<size_t>(u) * blockDim.x;
          if (vv < v1) res[u] = Pack<T>::mc_sum(c.mc_heap + off + vv * 16);
        }
#pragma unroll
        for (int u = 0; u < U; ++u) {
          const size_t vv = v + static_cast<size_t>(u) * blockDim.x;
          if (vv < v1) {
            if (a.scale != 1.0f) {
              float acc[N];
              Pack<T>::unpack(res[u], acc);
#pragma unroll
              for (int k = 0; k < N; ++k) acc[k] *= a.scale;
              res[u] = Pack<T>::pack(acc);
            }
            multimem_st16(c.mc_heap + off + vv * 16, res[u]);
          }
        }
      }
    } else {
      for (size_t v = v0 + threadIdx.x; v < v1; v += blockDim.x) {
        const size_t voff = off + v * 16;
        float acc[N];
        reduce_peers<T, R>(c, voff, acc);
#pragma unroll
        for (int k = 0; k < N; ++k) acc[k] *= a.scale;
        const uint4 res = Pack<T>::pack(acc);
#pragma unroll
        for (int p = 0; p < kMaxRanks; ++p) {
          if (p < c.nranks) st16(c.heap[p] + voff, res);
        }
      }
    }
  }

  static __device__ void run(const CommDev& c, const Args& a) {
    constexpr int S = kPipeSlots;
    const size_t chunk_bytes = a.chunk_elems * sizeof(T);
    const size_t nchunks = (a.count + a.chunk_elems - 1) / a.chunk_elems;
    const long n = blockIdx.x < nchunks ? static_cast<long>((nchunks - blockIdx.x + gridDim.x - 1) / gridDim.x) : 0;
    const uint32_t base_r = c.epochs[kFlagSetReady * kMaxBlocks + blockIdx.x];
    const uint32_t base_d = c.epochs[kFlagSetDone * kMaxBlocks + blockIdx.x];
    const size_t slot0 = a.bulk_off + static_cast<size_t>(blockIdx.x) * S * chunk_bytes;
    const bool mc = a.use_mc && c.mc_heap != nullptr && R == RedKind::SUM;
    bool ok = true;
    trace_mark(c, 0);
    for (long k = 0; k < n + 2; ++k) {
      if (!ok) break;  // failed wait: stop staging, copying and posting
      if (k < n) {
        const size_t e0 = (blockIdx.x + static_cast<size_t>(k) * gridDim.x) * a.chunk_elems;
        const size_t cnt = min_sz(a.chunk_elems, a.count - e0);
        block_copy(c.heap[c.rank] + slot0 + (k % S) * chunk_bytes, a.in + e0, cnt * sizeof(T));
      }
      if (k == 0) trace_mark(c, 1);
      if (k >= 1 && k - 1 < n) {
        const long j = k - 1;
        ok = wait_all_peers(c, kFlagSetReady, base_r + static_cast<uint32_t>(j) + 1, 0x21) && ok;
        if (k == 1) trace_mark(c, 2);
        if (ok) {
          const size_t e0 = (blockIdx.x + static_cast<size_t>(j) * gridDim.x) * a.chunk_elems;
          reduce_share(c, a, slot0 + (j % S) * chunk_bytes, min_sz(a.chunk_elems, a.count - e0), mc);
        }
        if (k == 1) trace_mark(c, 3);
      }
      if (k >= 2 && k - 2 < n) {
        const long j = k - 2;
        ok = wait_all_peers(c, kFlagSetDone, base_d + static_cast<uint32_t>(j) + 1, 0x22) && ok;
        if (k == 2) trace_mark(c, 4);
        if (!ok) break;
        const size_t e0 = (blockIdx.x + static_cast<size_t>(j) * gridDim.x) * a.chunk_elems;
        const size_t cnt = min_sz(a.chunk_elems, a.count - e0);
        block_copy(a.out + e0, c.heap[c.rank] + slot0 + (j % S) * chunk_bytes, cnt * sizeof(T));
        if (k == 2) trace_mark(c, 5);
      }
      if (ok) post_flags(c, k < n, base_r + static_cast<uint32_t>(k) + 1, k >= 1 && k - 1 < n, base_d + static_cast<uint32_t>(k));
    }
    trace_mark(c, 6);
    __syncthreads();
    if (threadIdx.x == 0) {
      c.epochs[kFlagSetReady * kMaxBlocks + blockIdx.x] = base_r + static_cast<uint32_t>(n);
      c.epochs[kFlagSetDone * kMaxBlocks + blockIdx.x] = base_d + static_cast<uint32_t>(n);
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
    return launch_op<Op>(comms, emu, args.data(), blocks, 256, stream);
  }
  using Op = ArPipe<T, R>;
  constexpr size_t kVec = Pack<T>::N;
  size_t chunk_elems = s.chunk_bytes / sizeof(T);
  chunk_elems = (chunk_elems / kVec) * kVec;
  if (chunk_elems == 0) return cudaErrorInvalidValue;
  const size_t nchunks = (count + chunk_elems - 1) / chunk_elems;
  const int blocks = static_cast<int>(std::min<size_t>(s.blocks, std::max<size_t>(nchunks, 1)));
  if (static_cast<size_t>(blocks) * kPipeSlots * chunk_elems * sizeof(T) > lay.bulk_bytes) return cudaErrorInvalidValue;
  std::vector<typename Op::Args> args(n);
  for (int i = 0; i < n; ++i) {
    args[i] = {static_cast<const T*>(in[i]), static_cast<T*>(out[i]), count, scale, use_mc ? 1 : 0, lay.bulk_off, chunk_elems};
  }
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

} // namespace coll

cudaError_t launch_all_reduce(const CommDev* comms, const HeapLayout& lay, int emu_ranks, const void* const* in,
                              void* const* out, size_t count, DType dtype, RedKind red, float scale, int algo,
                              bool use_mc, LaunchShape shape, cudaStream_t stream) {
  using namespace coll;
  switch (dtype) {
    case DType::F32: return ar_dispatch_red<float>(comms, lay, emu_ranks, in, out, count, red, scale, algo, use_mc, shape, stream);
    case DType::F16: return ar_dispatch_red<__half>(comms, lay, emu_ranks, in, out, count, red, scale, algo, use_mc, shape, stream);
    case DType::BF16: return ar_dispatch_red<__nv_bfloat16>(comms, lay, emu_ranks, in, out, count, red, scale, algo, use_mc, shape, stream);
  }
  return cudaErrorInvalidValue;
}

} // namespace b200c
