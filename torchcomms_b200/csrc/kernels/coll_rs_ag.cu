// Reduce-scatter and all-gather over the symmetric heap (sm_100a), pipelined,
// with the precision change fused into the copies: reduce-scatter may narrow
// fp32 inputs to bf16 for the wire and widen the reduced result again; the
// all-gather may narrow an fp32 shard to bf16 while staging it.
//
// Replaces, in the reference: comms/ctran/algos/ReduceScatter/ReduceScatterDirect.cuh:70-160,
// comms/prims/collectives/ReduceScatterDirect.cu, comms/ctran/algos/AllGather/AllGatherDirect.cuh:50,
// comms/prims/collectives/AllGatherDirect.cu:17-72, and the quantised
// reduce-scatter of comms/ncclx/meta/collectives/quantCollectives.cc:15-60.
#include "coll_pipe2.cuh"

namespace b200c {
namespace coll {

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
    unsigned long long seed;  // non-zero: fp32 -> bf16 staging rounds stochastically
  };
  static __device__ size_t prologue(const CommDev&, const Args& a) {
    return (a.count + a.chunk_elems - 1) / a.chunk_elems;
  }
  static __device__ size_t slot_bytes(const CommDev& c, const Args& a) {
    return a.chunk_elems * sizeof(WireT) * c.nranks;  // one sub-slot per destination
  }
  static __device__ bool mc(const CommDev& c, const Args& a) {
    return a.use_mc && c.mc_heap != nullptr && R == RedKind::SUM;
  }
  static __device__ void stage(const CommDev& c, const Args& a, size_t chunk, size_t off) {
    const size_t e0 = chunk * a.chunk_elems;
    const size_t n = min_sz(a.chunk_elems, a.count - e0);
    const size_t sub = a.chunk_elems * sizeof(WireT);
    const bool use_mc = mc(c, a);
    // Per destination p, the part of my input that p will reduce.
    for (int p = 0; p < c.nranks; ++p) {
      if (p == c.rank && !use_mc) continue;  // own part is read from `in` directly
      if constexpr (std::is_same<InT, float>::value && std::is_same<WireT, __nv_bfloat16>::value) {
        if (a.seed != 0) {
          // One random stream per (source rank, destination, position): independent errors that average out in the sum.
          const unsigned long long stream_id =
              (static_cast<unsigned long long>(c.rank) * kMaxRanks + p) * ((a.count + 7) / 8 + 1) + e0 / 8 + 1;
          block_convert_sr(reinterpret_cast<__nv_bfloat16*>(c.heap[c.rank] + off + p * sub),
                           a.in + static_cast<size_t>(p) * a.count + e0, n, a.seed, stream_id);
          continue;
        }
      }
      block_convert<WireT, InT>(reinterpret_cast<WireT*>(c.heap[c.rank] + off + p * sub),
                                a.in + static_cast<size_t>(p) * a.count + e0, n);
    }
  }
  static __device__ void consume(const CommDev& c, const Args& a, size_t chunk, size_t off) {
    constexpr int N = Pack<WireT>::N;
    const size_t e0 = chunk * a.chunk_elems;
    const size_t n = min_sz(a.chunk_elems, a.count - e0);
    const size_t sub = a.chunk_elems * sizeof(WireT);
    const size_t nvec = (n + N - 1) / N;
    const size_t my_off = off + static_cast<size_t>(c.rank) * sub;
    const InT* own = a.in + static_cast<size_t>(c.rank) * a.count + e0;
    const bool out_aligned = (reinterpret_cast<uintptr_t>(a.out + e0) & 15u) == 0;
    if (mc(c, a)) {
      constexpr int U = 4;
      for (size_t v = threadIdx.x; v < nvec; v += static_cast<size_t>(U) * blockDim.x) {
        uint4 res[U];
#pragma unroll
        for (int u = 0; u < U; ++u) {
          const size_t vv = v + static_cast<size_t>(u) * blockDim.x;
          if (vv < nvec) res[u] = Pack<WireT>::mc_sum(c.mc_heap + my_off + vv * 16);
        }
#pragma unroll
        for (int u = 0; u < U; ++u) {
          const size_t vv = v + static_cast<size_t>(u) * blockDim.x;
          if (vv < nvec) {
            float acc[N];
            Pack<WireT>::unpack(res[u], acc);
#pragma unroll
            for (int k = 0; k < N; ++k) acc[k] *= a.scale;
            const size_t left = n - vv * N;
            store_values<OutT, N>(a.out + e0 + vv * N, acc, left < N ? static_cast<int>(left) : N, out_aligned);
          }
        }
      }
      return;
    }
    const bool own_aligned = (reinterpret_cast<uintptr_t>(own) & 15u) == 0;
    for (size_t v = threadIdx.x; v < nvec; v += blockDim.x) {
      float acc[N];
      const size_t left = n - v * N;
      const int nv = left < N ? static_cast<int>(left) : N;
      uint4 pv[kMaxRanks];
#pragma unroll
      for (int i = 1; i < kMaxRanks; ++i) {
        if (i < c.nranks) {
          int p = c.rank + i;
          if (p >= c.nranks) p -= c.nranks;
          pv[i] = ld16(c.heap[p] + my_off + v * 16);
        }
      }
      if (own_aligned && nv == N) {
        // N input elements: 16 bytes when sizeof(InT) == sizeof(WireT), 32 when the input is fp32 and the wire 16-bit.
        if constexpr (sizeof(InT) == sizeof(WireT)) {
          Pack<InT>::unpack(ld16(own + v * N), acc);
        } else {
          Pack<InT>::unpack(ld16(own + v * N), acc);
          Pack<InT>::unpack(ld16(own + v * N + Pack<InT>::N), acc + Pack<InT>::N);
        }
      } else {
#pragma unroll
        for (int k = 0; k < N; ++k) acc[k] = k < nv ? Pack<InT>::to_float(own[v * N + k]) : 0.0f;
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
#pragma unroll
      for (int k = 0; k < N; ++k) acc[k] *= a.scale;
      store_values<OutT, N>(a.out + e0 + v * N, acc, nv, out_aligned);
    }
  }
};

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
  static __device__ size_t prologue(const CommDev&, const Args& a) {
    return (a.wire_bytes + a.chunk_bytes - 1) / a.chunk_bytes;
  }
  // With the switch's multicast each rank PUSHES its chunk once and the switch
  // delivers it into sub-slot `rank` of every rank's slot (egress 1x instead
  // of nranks-1 pulls); the consumer then only copies out of its own memory.
  static __device__ bool mc(const CommDev& c, const Args& a) { return a.use_mc && c.mc_heap != nullptr; }
  static __device__ size_t slot_bytes(const CommDev& c, const Args& a) {
    return mc(c, a) ? a.chunk_bytes * c.nranks : a.chunk_bytes;
  }
  static __device__ void stage(const CommDev& c, const Args& a, size_t chunk, size_t off) {
    const size_t b0 = chunk * a.chunk_bytes;
    const size_t n = min_sz(a.chunk_bytes, a.wire_bytes - b0);
    if (mc(c, a)) {
      char* dst = c.mc_heap + off + static_cast<size_t>(c.rank) * a.chunk_bytes;
      const size_t nvec = (n + 15) / 16;  // the slot is padded to 16 bytes; the tail is never copied out
      if constexpr (std::is_same<CastT, void>::value) {
        const char* src = a.in + b0;
        if ((reinterpret_cast<uintptr_t>(src) & 15u) == 0 && n % 16 == 0) {
          const uint4* s4 = reinterpret_cast<const uint4*>(src);
          size_t i = threadIdx.x;
          for (; i + 3 * blockDim.x < nvec; i += 4 * blockDim.x) {
            const uint4 v0 = s4[i], v1 = s4[i + blockDim.x], v2 = s4[i + 2 * blockDim.x], v3 = s4[i + 3 * blockDim.x];
            multimem_st16(dst + i * 16, v0);
            multimem_st16(dst + (i + blockDim.x) * 16, v1);
            multimem_st16(dst + (i + 2 * blockDim.x) * 16, v2);
            multimem_st16(dst + (i + 3 * blockDim.x) * 16, v3);
          }
          for (; i < nvec; i += blockDim.x) multimem_st16(dst + i * 16, s4[i]);
        } else {
          for (size_t i = threadIdx.x; i < nvec; i += blockDim.x) {
            uint4 v = make_uint4(0, 0, 0, 0);
            char* vb = reinterpret_cast<char*>(&v);
            const size_t left = n - i * 16 < 16 ? n - i * 16 : 16;
            for (size_t k = 0; k < left; ++k) vb[k] = src[i * 16 + k];
            multimem_st16(dst + i * 16, v);
          }
        }
      } else {
        const float* src = reinterpret_cast<const float*>(a.in) + b0 / sizeof(CastT);
        const size_t ne = n / sizeof(CastT);
        for (size_t i = threadIdx.x; i < nvec; i += blockDim.x) {
          float f[8];
#pragma unroll
          for (int k = 0; k < 8; ++k) f[k] = i * 8 + k < ne ? src[i * 8 + k] : 0.0f;
          multimem_st16(dst + i * 16, Pack<CastT>::pack(f));
        }
      }
      return;
    }
    char* slot = c.heap[c.rank] + off;
    if constexpr (std::is_same<CastT, void>::value) {
      block_copy(slot, a.in + b0, n);
    } else {
      block_convert<CastT, float>(reinterpret_cast<CastT*>(slot),
                                  reinterpret_cast<const float*>(a.in) + b0 / sizeof(CastT), n / sizeof(CastT));
    }
  }
  static __device__ void consume(const CommDev& c, const Args& a, size_t chunk, size_t off) {
    const size_t b0 = chunk * a.chunk_bytes;
    const size_t n = min_sz(a.chunk_bytes, a.wire_bytes - b0);
    const bool push = mc(c, a);
    for (int i = 0; i < c.nranks; ++i) {
      int q = c.rank + i;
      if (q >= c.nranks) q -= c.nranks;
      const char* src = push ? c.heap[c.rank] + off + static_cast<size_t>(q) * a.chunk_bytes : c.heap[q] + off;
      block_copy(a.out + static_cast<size_t>(q) * a.wire_bytes + b0, src, n);
    }
  }
};

// Latency mode of the all-gather: block b owns the 4 KB piece b of every
// rank's input. One copy into the parity-buffered small region, one barrier,
// then every thread fetches its 16 bytes from all peers at once.
struct AgOneShot {
  struct Args {
    const char* in;
    char* out;
    size_t bytes;   // per rank
    size_t small_off;
  };
  static __device__ void run(const CommDev& c, const Args& a) {
    const size_t e0 = static_cast<size_t>(blockIdx.x) * kSmallPiece;
    if (e0 >= a.bytes) return;  // same decision on every rank
    const size_t n = min_sz(kSmallPiece, a.bytes - e0);
    BlockEpoch ep;
    ep.load(c, kFlagSetSmall);
    const size_t parity = (ep.value + 1) & 1u;
    const size_t off = a.small_off + parity * (static_cast<size_t>(kSmallBlocks) * kSmallPiece) +
        static_cast<size_t>(blockIdx.x) * kSmallPiece;
    block_copy(c.heap[c.rank] + off, a.in + e0, n);
    const bool ok = block_barrier(c, kFlagSetSmall, ep, 0x15);
    if (ok) {
      const bool aligned = ((reinterpret_cast<uintptr_t>(a.out + e0) | a.bytes | n) & 15u) == 0;
      if (aligned) {
        const size_t nvec = n / 16;
        for (size_t v = threadIdx.x; v < nvec; v += blockDim.x) {
          uint4 r[kMaxRanks];
#pragma unroll
          for (int q = 0; q < kMaxRanks; ++q) {
            if (q < c.nranks) r[q] = ld16(c.heap[q] + off + v * 16);
          }
#pragma unroll
          for (int q = 0; q < kMaxRanks; ++q) {
            if (q < c.nranks) *reinterpret_cast<uint4*>(a.out + static_cast<size_t>(q) * a.bytes + e0 + v * 16) = r[q];
          }
        }
      } else {
        for (int q = 0; q < c.nranks; ++q) block_copy(a.out + static_cast<size_t>(q) * a.bytes + e0, c.heap[q] + off, n);
      }
    }
    ep.store(c, kFlagSetSmall);
  }
};

// Latency mode of the reduce-scatter: a block's 4 KB piece holds one
// sub-piece per destination rank; after the barrier each rank sums its own
// sub-piece over all peers.
template <typename T, RedKind R>
struct RsOneShot {
  struct Args {
    const T* in;    // nranks x count
    T* out;         // count
    size_t count;
    float scale;
    size_t small_off;
  };
  static __device__ __host__ size_t sub_bytes(int nranks) { return (kSmallPiece / nranks) / 16 * 16; }
  static __device__ void run(const CommDev& c, const Args& a) {
    constexpr int N = Pack<T>::N;
    const size_t sub = sub_bytes(c.nranks);
    const size_t sub_elems = sub / sizeof(T);
    const size_t e0 = static_cast<size_t>(blockIdx.x) * sub_elems;
    if (e0 >= a.count) return;  // same decision on every rank
    const size_t n = min_sz(sub_elems, a.count - e0);
    BlockEpoch ep;
    ep.load(c, kFlagSetSmall);
    const size_t parity = (ep.value + 1) & 1u;
    const size_t off = a.small_off + parity * (static_cast<size_t>(kSmallBlocks) * kSmallPiece) +
        static_cast<size_t>(blockIdx.x) * kSmallPiece;
    for (int p = 0; p < c.nranks; ++p) {
      block_copy(c.heap[c.rank] + off + p * sub, a.in + static_cast<size_t>(p) * a.count + e0, n * sizeof(T));
    }
    const bool ok = block_barrier(c, kFlagSetSmall, ep, 0x16);
    if (ok) {
      const size_t nvec = (n + N - 1) / N;
      const bool aligned = (reinterpret_cast<uintptr_t>(a.out + e0) & 15u) == 0;
      const size_t mine = off + static_cast<size_t>(c.rank) * sub;
      for (size_t v = threadIdx.x; v < nvec; v += blockDim.x) {
        float acc[N];
        reduce_peers<T, R>(c, mine + v * 16, acc);
#pragma unroll
        for (int k = 0; k < N; ++k) acc[k] *= a.scale;
        const size_t left = n - v * N;
        store_values<T, N>(a.out + e0 + v * N, acc, left < N ? static_cast<int>(left) : N, aligned);
      }
    }
    ep.store(c, kFlagSetSmall);
  }
};

template <typename T>
cudaError_t rs_oneshot(const CommDev* comms, const HeapLayout& lay, int emu, const void* const* in, void* const* out,
                       size_t count, RedKind red, float scale, int threads, cudaStream_t stream) {
  const int n = emu > 0 ? emu : 1;
  const int nranks = comms[0].nranks;
  const size_t sub_elems = RsOneShot<T, RedKind::SUM>::sub_bytes(nranks) / sizeof(T);
  const size_t blocks = (count + sub_elems - 1) / sub_elems;
  if (blocks > static_cast<size_t>(kSmallBlocks)) return cudaErrorInvalidValue;
  auto go = [&](auto tag) {
    using Op = decltype(tag);
    std::vector<typename Op::Args> args(n);
    for (int i = 0; i < n; ++i) args[i] = {static_cast<const T*>(in[i]), static_cast<T*>(out[i]), count, scale, lay.small_off};
    return launch_op<Op>(comms, emu, args.data(), static_cast<int>(blocks), threads, stream, true);
  };
  switch (red) {
    case RedKind::SUM: return go(RsOneShot<T, RedKind::SUM>{});
    case RedKind::PROD: return go(RsOneShot<T, RedKind::PROD>{});
    case RedKind::MIN: return go(RsOneShot<T, RedKind::MIN>{});
    case RedKind::MAX: return go(RsOneShot<T, RedKind::MAX>{});
  }
  return cudaErrorInvalidValue;
}

template <typename InT, typename WireT, typename OutT, RedKind R>
cudaError_t rs_dispatch(const CommDev* comms, const HeapLayout& lay, int emu, const void* const* in,
                        void* const* out, size_t count, float scale, bool use_mc, LaunchShape s,
                        cudaStream_t stream, unsigned long long seed = 0) {
  using Op = RsOp<InT, WireT, OutT, R>;
  const int n = emu > 0 ? emu : 1;
  const int nranks = comms[0].nranks;
  constexpr size_t kVec = Pack<WireT>::N;
  size_t chunk_elems = s.chunk_bytes / sizeof(WireT);
  chunk_elems = (chunk_elems / kVec) * kVec;
  if (chunk_elems == 0) return cudaErrorInvalidValue;
  const size_t nchunks = (count + chunk_elems - 1) / chunk_elems;
  const int blocks = static_cast<int>(std::min<size_t>(s.blocks, std::max<size_t>(nchunks, 1)));
  if (static_cast<size_t>(blocks) * kPipeSlots * chunk_elems * sizeof(WireT) * nranks > lay.bulk_bytes) return cudaErrorInvalidValue;
  std::vector<typename Op::Args> args(n);
  for (int i = 0; i < n; ++i) {
    args[i] = {static_cast<const InT*>(in[i]), static_cast<OutT*>(out[i]), count, scale, use_mc ? 1 : 0, lay.bulk_off, chunk_elems, seed};
  }
  return launch_op<Pipe2<Op>>(comms, emu, args.data(), blocks, s.threads, stream);
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

} // namespace coll

cudaError_t launch_reduce_scatter(const CommDev* comms, const HeapLayout& lay, int emu_ranks, const void* const* in,
                                  void* const* out, size_t count, DType in_dtype, DType wire_dtype, DType out_dtype,
                                  RedKind red, float scale, bool use_mc, LaunchShape shape, cudaStream_t stream,
                                  unsigned long long sr_seed) {
  using namespace coll;
  using bf16 = __nv_bfloat16;
  if (shape.chunk_bytes == 0) {
    // Latency mode (same dtype on all three sides only).
    if (!(in_dtype == wire_dtype && wire_dtype == out_dtype)) return cudaErrorInvalidValue;
    switch (in_dtype) {
      case DType::F32: return rs_oneshot<float>(comms, lay, emu_ranks, in, out, count, red, scale, shape.threads, stream);
      case DType::F16: return rs_oneshot<__half>(comms, lay, emu_ranks, in, out, count, red, scale, shape.threads, stream);
      case DType::BF16: return rs_oneshot<bf16>(comms, lay, emu_ranks, in, out, count, red, scale, shape.threads, stream);
    }
  }
  if (in_dtype == wire_dtype && wire_dtype == out_dtype) {
    switch (in_dtype) {
      case DType::F32: return rs_same<float>(comms, lay, emu_ranks, in, out, count, red, scale, use_mc, shape, stream);
      case DType::F16: return rs_same<__half>(comms, lay, emu_ranks, in, out, count, red, scale, use_mc, shape, stream);
      case DType::BF16: return rs_same<bf16>(comms, lay, emu_ranks, in, out, count, red, scale, use_mc, shape, stream);
    }
  }
  if (wire_dtype != DType::BF16 || red != RedKind::SUM) return cudaErrorInvalidValue;
  if (in_dtype == DType::F32 && out_dtype == DType::F32)
    return rs_dispatch<float, bf16, float, RedKind::SUM>(comms, lay, emu_ranks, in, out, count, scale, use_mc, shape, stream, sr_seed);
  if (in_dtype == DType::F32 && out_dtype == DType::BF16)
    return rs_dispatch<float, bf16, bf16, RedKind::SUM>(comms, lay, emu_ranks, in, out, count, scale, use_mc, shape, stream, sr_seed);
  if (in_dtype == DType::BF16 && out_dtype == DType::F32)
    return rs_dispatch<bf16, bf16, float, RedKind::SUM>(comms, lay, emu_ranks, in, out, count, scale, use_mc, shape, stream);
  return cudaErrorInvalidValue;
}

cudaError_t launch_all_gather(const CommDev* comms, const HeapLayout& lay, int emu_ranks, const void* const* in,
                              void* const* out, size_t bytes, bool cast_f32_to_bf16, bool use_mc, LaunchShape shape,
                              cudaStream_t stream) {
  using namespace coll;
  const int n = emu_ranks > 0 ? emu_ranks : 1;
  if (shape.chunk_bytes == 0) {
    // Latency mode.
    if (cast_f32_to_bf16 || bytes > static_cast<size_t>(kSmallBlocks) * kSmallPiece) return cudaErrorInvalidValue;
    std::vector<AgOneShot::Args> args(n);
    for (int i = 0; i < n; ++i) args[i] = {static_cast<const char*>(in[i]), static_cast<char*>(out[i]), bytes, lay.small_off};
    const int blocks = static_cast<int>((bytes + kSmallPiece - 1) / kSmallPiece);
    return launch_op<AgOneShot>(comms, emu_ranks, args.data(), blocks, shape.threads, stream, true);
  }
  const size_t chunk = (shape.chunk_bytes / 16) * 16;
  if (chunk == 0) return cudaErrorInvalidValue;
  const size_t wire = cast_f32_to_bf16 ? bytes / 2 : bytes;
  const size_t nchunks = (wire + chunk - 1) / chunk;
  const int blocks = static_cast<int>(std::min<size_t>(shape.blocks, std::max<size_t>(nchunks, 1)));
  const size_t slot_mult = use_mc && comms[0].mc_heap != nullptr ? static_cast<size_t>(comms[0].nranks) : 1;
  if (static_cast<size_t>(blocks) * kPipeSlots * chunk * slot_mult > lay.bulk_bytes) return cudaErrorInvalidValue;
  if (cast_f32_to_bf16) {
    using Op = AgOp<__nv_bfloat16>;
    std::vector<Op::Args> args(n);
    for (int i = 0; i < n; ++i)
      args[i] = {static_cast<const char*>(in[i]), static_cast<char*>(out[i]), wire, use_mc ? 1 : 0, lay.bulk_off, chunk};
    return launch_op<Pipe2<Op>>(comms, emu_ranks, args.data(), blocks, shape.threads, stream);
  }
  using Op = AgOp<void>;
  std::vector<Op::Args> args(n);
  for (int i = 0; i < n; ++i)
    args[i] = {static_cast<const char*>(in[i]), static_cast<char*>(out[i]), wire, use_mc ? 1 : 0, lay.bulk_off, chunk};
  return launch_op<Pipe2<Op>>(comms, emu_ranks, args.data(), blocks, shape.threads, stream);
}

} // namespace b200c
