// One-pass collectives on symmetric buffers (sm_100a).
//
// A symmetric buffer is memory that every rank of the communicator has mapped
// at a known address (`SymmView::ptr[r]`), optionally with an NVLS multicast
// alias (`SymmView::mc`). When the tensor a collective works on lives in such
// a buffer nothing is staged: the data crosses NVLink exactly once, straight
// between the users' tensors, and only the two barriers go through the
// communicator's flag region.
//
//   all-gather      every rank stores its shard (cast to bf16 on the way if
//                   asked) into slot `rank` of every rank's output:
//                   one `multimem.st` per 16 bytes, or nranks peer stores
//   reduce-scatter  every rank reads slice `rank` of every rank's input:
//                   one `multimem.ld_reduce` per 16 bytes (the switch adds),
//                   or nranks peer loads summed in fp32; scale and the cast
//                   to the output type happen in registers
//   all-reduce      in place: each rank reduces 1/nranks of the buffer as
//                   above and stores the result back into every copy
//   all-to-all(v)   every rank stores its block for rank p straight into p's
//                   output; receive offsets travel with the opening barrier
//
// Each kernel opens with a per-block barrier across ranks (every rank's
// earlier work on the buffers is complete and its buffers may be written) and
// closes with one (all transfers have landed; the buffers may be reused).
// Waits are bounded: a wait that runs out sets the status word and the kernel
// returns.
//
// Replaces, in the reference: the symmetric-window kernels of
// comms/ncclx/v2_30/src/device/symmetric/{all_gather,reduce_scatter,all_reduce}.cuh
// (AllGather_ST / STMC, ReduceScatter_LD / LDMC, AllReduce_RSxLD_AGxST /
// RSxLDMC_AGxSTMC; ids in src/include/sym_kernels.h:33-55) and the push
// all-to-all of comms/prims/collectives/AllToAllv.cuh:113-263.
#include <cstring>

#include "coll_common.cuh"

namespace b200c {
namespace coll {

constexpr int kSymmThreads = 512;
constexpr int kSymmUnroll = 4;

template <typename Op>
__global__ void __launch_bounds__(kSymmThreads, 1) k_symm_real(CommDev c, typename Op::Args a) {
  Op::run(c, a);
}
template <typename Op>
__global__ void __launch_bounds__(kSymmThreads, 1) k_symm_emu(const CommDev* cs, const typename Op::Args* as) {
  Op::run(cs[blockIdx.y], as[blockIdx.y]);
}

// Same contract as launch_op(): `emu_ranks > 0` runs all virtual ranks in one
// cooperative launch. The grid is the caller's; it must be identical on every
// rank because block b of one rank meets block b of the others.
template <typename Op>
cudaError_t launch_symm(const CommDev* comms, int emu_ranks, const typename Op::Args* args, int blocks,
                        cudaStream_t stream) {
  using Args = typename Op::Args;
  if (blocks < 1) blocks = 1;
  if (blocks > kMaxBlocks) blocks = kMaxBlocks;
  note_kernel_launch();
  if (emu_ranks <= 0) {
    k_symm_real<Op><<<blocks, kSymmThreads, 0, stream>>>(comms[0], args[0]);
    return cudaGetLastError();
  }
  int dev = 0, sms = 0, per_sm = 0;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, k_symm_emu<Op>, kSymmThreads, 0);
  if (blocks * emu_ranks > sms * (per_sm > 0 ? per_sm : 1)) return cudaErrorInvalidConfiguration;
  CommDev* d_comms = nullptr;
  Args* d_args = nullptr;
  cudaError_t e = cudaMalloc(&d_comms, sizeof(CommDev) * emu_ranks);
  if (e != cudaSuccess) return e;
  e = cudaMalloc(&d_args, sizeof(Args) * emu_ranks);
  if (e != cudaSuccess) {
    cudaFree(d_comms);
    return e;
  }
  cudaMemcpyAsync(d_comms, comms, sizeof(CommDev) * emu_ranks, cudaMemcpyHostToDevice, stream);
  cudaMemcpyAsync(d_args, args, sizeof(Args) * emu_ranks, cudaMemcpyHostToDevice, stream);
  void* params[] = {&d_comms, &d_args};
  e = cudaLaunchCooperativeKernel(reinterpret_cast<void*>(&k_symm_emu<Op>), dim3(blocks, emu_ranks),
                                  dim3(kSymmThreads), params, 0, stream);
  const cudaError_t e2 = cudaStreamSynchronize(stream);
  cudaFree(d_comms);
  cudaFree(d_args);
  return e != cudaSuccess ? e : e2;
}

// Vectors [v0, v1) of `nvec` that block `b` of `nb` owns (contiguous, so a
// block streams through one region).
__device__ __forceinline__ void block_range(size_t nvec, int b, int nb, size_t* v0, size_t* v1) {
  const size_t per = (nvec + nb - 1) / nb;
  *v0 = min_sz(nvec, per * static_cast<size_t>(b));
  *v1 = min_sz(nvec, *v0 + per);
}

// ---------------------------------------------------------- all-gather -----

// One 16-byte wire vector `v` of this rank's shard. With Cast the shard is
// fp32 and 8 values are narrowed to bf16.
template <bool Cast>
__device__ __forceinline__ uint4 load_wire_vec(const char* in, size_t v, bool aligned) {
  if constexpr (Cast) {
    const float* src = reinterpret_cast<const float*>(in) + v * 8;
    float f[8];
    if (aligned) {
      Pack<float>::unpack(ld16_stream(src), f);
      Pack<float>::unpack(ld16_stream(src + 4), f + 4);
    } else {
#pragma unroll
      for (int k = 0; k < 8; ++k) f[k] = src[k];
    }
    return Pack<__nv_bfloat16>::pack(f);
  } else {
    if (aligned) return ld16_stream(in + v * 16);
    uint4 r;
    char* rb = reinterpret_cast<char*>(&r);
    for (int k = 0; k < 16; ++k) rb[k] = in[v * 16 + k];
    return r;
  }
}

template <bool Cast>
struct SymAg {
  struct Args {
    const char* in;      // this rank's shard (fp32 when Cast)
    SymmView out;        // nranks x wire_bytes, symmetric
    size_t wire_bytes;   // per rank, after the cast; multiple of 16
    int use_mc;
  };
  static __device__ void run(const CommDev& c, const Args& a) {
    BlockEpoch ep;
    ep.load(c, kFlagSetSymAg);
    trace_mark(c, 0);
    bool ok = block_barrier(c, kFlagSetSymAg, ep, 0x41);
    trace_mark(c, 1);
    if (ok) {
      size_t v0, v1;
      block_range(a.wire_bytes / 16, blockIdx.x, gridDim.x, &v0, &v1);
      const size_t base = static_cast<size_t>(c.rank) * a.wire_bytes;
      const bool aligned = (reinterpret_cast<uintptr_t>(a.in) & 15u) == 0;
      const bool mc = a.use_mc && a.out.mc != nullptr;
      constexpr int U = kSymmUnroll;
      for (size_t v = v0 + threadIdx.x; v < v1; v += static_cast<size_t>(U) * blockDim.x) {
        uint4 r[U];
#pragma unroll
        for (int u = 0; u < U; ++u) {
          const size_t vv = v + static_cast<size_t>(u) * blockDim.x;
          if (vv < v1) r[u] = load_wire_vec<Cast>(a.in, vv, aligned);
        }
#pragma unroll
        for (int u = 0; u < U; ++u) {
          const size_t vv = v + static_cast<size_t>(u) * blockDim.x;
          if (vv >= v1) continue;
          if (mc) {
            multimem_st16(a.out.mc + base + vv * 16, r[u]);
          } else {
#pragma unroll
            for (int i = 0; i < kMaxRanks; ++i) {
              if (i < c.nranks) {
                int p = c.rank + i;
                if (p >= c.nranks) p -= c.nranks;
                st16(a.out.ptr[p] + base + vv * 16, r[u]);
              }
            }
          }
        }
      }
      trace_mark(c, 2);
      ok = block_barrier(c, kFlagSetSymAg, ep, 0x42);
      trace_mark(c, 3);
    }
    ep.store(c, kFlagSetSymAg);
  }
};

// ------------------------------------------------------- reduce-scatter ----

// Sum over ranks of the 16-byte vector at byte offset `off` of a symmetric
// buffer, in fp32.
template <typename WireT>
__device__ __forceinline__ void symm_sum(const CommDev& c, const SymmView& s, size_t off, bool mc, float* acc) {
  constexpr int N = Pack<WireT>::N;
  if (mc) {
    Pack<WireT>::unpack(Pack<WireT>::mc_sum(s.mc + off), acc);
    return;
  }
  uint4 v[kMaxRanks];
#pragma unroll
  for (int i = 0; i < kMaxRanks; ++i) {
    if (i < c.nranks) {
      int p = c.rank + i;
      if (p >= c.nranks) p -= c.nranks;
      v[i] = ld16_stream(s.ptr[p] + off);
    }
  }
  Pack<WireT>::unpack(v[0], acc);
#pragma unroll
  for (int i = 1; i < kMaxRanks; ++i) {
    if (i < c.nranks) {
      float f[N];
      Pack<WireT>::unpack(v[i], f);
#pragma unroll
      for (int k = 0; k < N; ++k) acc[k] += f[k];
    }
  }
}

template <typename WireT, typename OutT>
struct SymRs {
  struct Args {
    SymmView in;     // nranks x count elements of WireT, symmetric
    OutT* out;       // count elements
    size_t count;    // multiple of Pack<WireT>::N
    float scale;
    int use_mc;
  };
  template <int U>
  static __device__ __forceinline__ void body(const CommDev& c, const Args& a, bool mc, size_t base, size_t v0, size_t v1,
                                              bool out_aligned) {
    constexpr int N = Pack<WireT>::N;
    for (size_t v = v0 + threadIdx.x; v < v1; v += static_cast<size_t>(U) * blockDim.x) {
      float acc[U][N];
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const size_t vv = v + static_cast<size_t>(u) * blockDim.x;
        if (vv < v1) symm_sum<WireT>(c, a.in, base + vv * 16, mc, acc[u]);
      }
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const size_t vv = v + static_cast<size_t>(u) * blockDim.x;
        if (vv >= v1) continue;
#pragma unroll
        for (int k = 0; k < N; ++k) acc[u][k] *= a.scale;
        store_values<OutT, N>(a.out + vv * N, acc[u], N, out_aligned);
      }
    }
  }
  static __device__ void run(const CommDev& c, const Args& a) {
    constexpr int N = Pack<WireT>::N;
    BlockEpoch ep;
    ep.load(c, kFlagSetSymRs);
    trace_mark(c, 0);
    bool ok = block_barrier(c, kFlagSetSymRs, ep, 0x43);
    trace_mark(c, 1);
    if (ok) {
      size_t v0, v1;
      block_range(a.count / N, blockIdx.x, gridDim.x, &v0, &v1);
      const size_t base = static_cast<size_t>(c.rank) * a.count * sizeof(WireT);
      const bool mc = a.use_mc && a.in.mc != nullptr;
      const bool out_aligned = (reinterpret_cast<uintptr_t>(a.out) & 15u) == 0;
      // Peer loads are latency-bound: keep about 16 of them in flight per
      // thread (vectors x ranks). With the switch adding there is one load per vector.
      if (mc) {
        body<kSymmUnroll>(c, a, true, base, v0, v1, out_aligned);
      } else if (c.nranks <= 2) {
        body<8>(c, a, false, base, v0, v1, out_aligned);
      } else if (c.nranks <= 4) {
        body<4>(c, a, false, base, v0, v1, out_aligned);
      } else {
        body<2>(c, a, false, base, v0, v1, out_aligned);
      }
      trace_mark(c, 2);
      ok = block_barrier(c, kFlagSetSymRs, ep, 0x44);
      trace_mark(c, 3);
    }
    ep.store(c, kFlagSetSymRs);
  }
};

// ----------------------------------------------------------- all-reduce ----

template <typename T>
struct SymAr {
  struct Args {
    SymmView buf;    // count elements, symmetric, reduced in place
    size_t count;    // multiple of Pack<T>::N
    float scale;
    int use_mc;
  };
  template <int U>
  static __device__ __forceinline__ void body(const CommDev& c, const Args& a, bool mc, size_t v0, size_t v1) {
    constexpr int N = Pack<T>::N;
    for (size_t v = v0 + threadIdx.x; v < v1; v += static_cast<size_t>(U) * blockDim.x) {
      float acc[U][N];
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const size_t vv = v + static_cast<size_t>(u) * blockDim.x;
        if (vv < v1) symm_sum<T>(c, a.buf, vv * 16, mc, acc[u]);
      }
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const size_t vv = v + static_cast<size_t>(u) * blockDim.x;
        if (vv >= v1) continue;
        if (a.scale != 1.0f) {
#pragma unroll
          for (int k = 0; k < N; ++k) acc[u][k] *= a.scale;
        }
        const uint4 res = Pack<T>::pack(acc[u]);
        if (mc) {
          multimem_st16(a.buf.mc + vv * 16, res);
        } else {
#pragma unroll
          for (int i = 0; i < kMaxRanks; ++i) {
            if (i < c.nranks) {
              int p = c.rank + i;
              if (p >= c.nranks) p -= c.nranks;
              st16(a.buf.ptr[p] + vv * 16, res);
            }
          }
        }
      }
    }
  }
  static __device__ void run(const CommDev& c, const Args& a) {
    constexpr int N = Pack<T>::N;
    BlockEpoch ep;
    ep.load(c, kFlagSetSymAr);
    trace_mark(c, 0);
    bool ok = block_barrier(c, kFlagSetSymAr, ep, 0x45);
    trace_mark(c, 1);
    if (ok) {
      // Rank r owns vectors [r * per, (r + 1) * per): nobody else reads or
      // writes them in any copy, which is what makes "in place" safe.
      const size_t nvec = a.count / N;
      const size_t per = (nvec + c.nranks - 1) / c.nranks;
      const size_t s0 = min_sz(nvec, per * c.rank);
      const size_t s1 = min_sz(nvec, s0 + per);
      size_t v0, v1;
      block_range(s1 - s0, blockIdx.x, gridDim.x, &v0, &v1);
      v0 += s0;
      v1 += s0;
      const bool mc = a.use_mc && a.buf.mc != nullptr;
      if (mc) {
        body<kSymmUnroll>(c, a, true, v0, v1);
      } else if (c.nranks <= 2) {
        body<8>(c, a, false, v0, v1);
      } else if (c.nranks <= 4) {
        body<4>(c, a, false, v0, v1);
      } else {
        body<2>(c, a, false, v0, v1);
      }
      trace_mark(c, 2);
      ok = block_barrier(c, kFlagSetSymAr, ep, 0x46);
      trace_mark(c, 3);
    }
    ep.store(c, kFlagSetSymAr);
  }
};

// ------------------------------------------------------------ all-to-all ---

// Copies `len` bytes, vectors [sub * per, ...) of the block group that serves
// one peer. 16-byte accesses when everything is aligned, bytes otherwise.
__device__ __forceinline__ void push_range(char* __restrict__ dst, const char* __restrict__ src, size_t len, int sub,
                                           int nsub) {
  const bool aligned =
      ((reinterpret_cast<uintptr_t>(dst) | reinterpret_cast<uintptr_t>(src)) & 15u) == 0;
  if (aligned) {
    const size_t nvec = len / 16;
    size_t v0, v1;
    block_range(nvec, sub, nsub, &v0, &v1);
    constexpr int U = kSymmUnroll;
    for (size_t v = v0 + threadIdx.x; v < v1; v += static_cast<size_t>(U) * blockDim.x) {
      uint4 r[U];
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const size_t vv = v + static_cast<size_t>(u) * blockDim.x;
        if (vv < v1) r[u] = ld16_stream(src + vv * 16);
      }
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const size_t vv = v + static_cast<size_t>(u) * blockDim.x;
        if (vv < v1) st16(dst + vv * 16, r[u]);
      }
    }
    if (sub == nsub - 1) {
      for (size_t i = nvec * 16 + threadIdx.x; i < len; i += blockDim.x) dst[i] = src[i];
    }
  } else {
    size_t b0, b1;
    block_range(len, sub, nsub, &b0, &b1);
    for (size_t i = b0 + threadIdx.x; i < b1; i += blockDim.x) dst[i] = src[i];
  }
}

struct SymA2a {
  struct Args {
    const char* in;
    SymmView out;                  // symmetric
    size_t in_bytes, out_bytes;    // capacities, for the bounds checks
    size_t send_off[kMaxRanks], send_len[kMaxRanks];
    size_t recv_off[kMaxRanks], recv_len[kMaxRanks];
    // Non-null: send lengths are int64 element counts in device memory
    // (blocks packed back to back); receive offsets are then derived from the
    // senders' counts.
    const long long* dev_send_counts;
    size_t elem_bytes;
    size_t meta_off;               // kMaxBlocks x kMaxRanks x 2 uint64 per rank, in the communicator's heap
    int exchange;                  // 0: every rank knows where its blocks go (equal splits)
  };
  static __device__ void run(const CommDev& c, const Args& a) {
    __shared__ unsigned long long s_soff[kMaxRanks], s_slen[kMaxRanks], s_doff[kMaxRanks];
    BlockEpoch ep;
    ep.load(c, kFlagSetSymA2a);
    trace_mark(c, 0);
    unsigned long long* meta_mine = reinterpret_cast<unsigned long long*>(c.heap[c.rank] + a.meta_off) +
        static_cast<size_t>(blockIdx.x) * kMaxRanks * 2;
    const bool dev = a.dev_send_counts != nullptr;
    if (threadIdx.x < c.nranks) {
      const int p = threadIdx.x;
      unsigned long long soff = a.send_off[p], slen = a.send_len[p];
      if (dev) {
        // A negative count (or one that overruns the input) is a caller bug:
        // report it and send nothing rather than read out of bounds.
        unsigned long long acc = 0;
        bool bad = false;
        for (int i = 0; i <= p; ++i) {
          const long long cnt = a.dev_send_counts[i];
          if (cnt < 0) bad = true;
          if (i < p) acc += static_cast<unsigned long long>(cnt < 0 ? 0 : cnt);
        }
        const long long mine = a.dev_send_counts[p];
        soff = acc * a.elem_bytes;
        slen = bad ? 0ull : static_cast<unsigned long long>(mine) * a.elem_bytes;
        if (bad) c.status[0] = c.status[0] | kStatusBadArg;
      }
      if (soff + slen > a.in_bytes) {
        c.status[0] = c.status[0] | kStatusBadArg;
        slen = soff < a.in_bytes ? a.in_bytes - soff : 0;
      }
      s_soff[p] = soff;
      s_slen[p] = slen;
      s_doff[p] = 0;
      if (a.exchange) {
        // The flag store of the barrier below publishes this together with everything else.
        unsigned long long* meta_p = reinterpret_cast<unsigned long long*>(c.heap[p] + a.meta_off) +
            (static_cast<size_t>(blockIdx.x) * kMaxRanks + c.rank) * 2;
        if (dev) {
          // Device counts: tell rank p how many bytes it gets from here; it answers with an offset.
          meta_p[0] = slen;
        } else {
          // Host splits: this rank already knows where p's block goes in its
          // output and how much room it has. Tell p; no second round is needed.
          unsigned long long roff = a.recv_off[p], cap = a.recv_len[p];
          if (roff + cap > a.out_bytes) {
            c.status[0] = c.status[0] | kStatusBadArg;
            cap = roff < a.out_bytes ? a.out_bytes - roff : 0;
          }
          meta_p[0] = roff;
          meta_p[1] = cap;
        }
      }
    }
    bool ok = block_barrier(c, kFlagSetSymA2a, ep, 0x47);
    if (ok && a.exchange && !dev) {
      if (threadIdx.x < c.nranks) {
        const int p = threadIdx.x;
        s_doff[p] = meta_mine[p * 2];
        const unsigned long long cap = meta_mine[p * 2 + 1];
        if (s_slen[p] > cap) {  // sender and receiver disagree about the split sizes
          c.status[0] = c.status[0] | kStatusBadArg;
          s_slen[p] = cap;
        }
      }
    } else if (ok && a.exchange) {
      // Second round: now that every sender's length is known, lay the
      // incoming blocks out (host-given offsets, or back to back for device
      // counts), clamp them to the output, and tell each sender where to put
      // its block.
      if (threadIdx.x < c.nranks) {
        const int q = threadIdx.x;
        unsigned long long roff = a.recv_off[q];
        if (dev) {
          roff = 0;
          for (int i = 0; i < q; ++i) roff += meta_mine[i * 2];
        }
        unsigned long long rlen = meta_mine[q * 2];
        const unsigned long long cap = dev ? (roff < a.out_bytes ? a.out_bytes - roff : 0) : a.recv_len[q];
        if (rlen > cap || roff + rlen > a.out_bytes) {
          c.status[0] = c.status[0] | kStatusBadArg;
          rlen = cap < rlen ? cap : rlen;
          if (roff + rlen > a.out_bytes) rlen = roff < a.out_bytes ? a.out_bytes - roff : 0;
        }
        unsigned long long* meta_q = reinterpret_cast<unsigned long long*>(c.heap[q] + a.meta_off) +
            (static_cast<size_t>(blockIdx.x) * kMaxRanks + c.rank) * 2;
        // Word 1 of the pair carries the offset; the granted length goes into
        // a second table behind the first.
        meta_q[1] = roff;
        unsigned long long* grant_q = reinterpret_cast<unsigned long long*>(c.heap[q] + a.meta_off) +
            static_cast<size_t>(kMaxBlocks) * kMaxRanks * 2 + (static_cast<size_t>(blockIdx.x) * kMaxRanks + c.rank);
        *grant_q = rlen;
      }
      ok = block_barrier(c, kFlagSetSymA2a, ep, 0x48);
      if (ok && threadIdx.x < c.nranks) {
        const int p = threadIdx.x;
        const unsigned long long* grant_mine = reinterpret_cast<unsigned long long*>(c.heap[c.rank] + a.meta_off) +
            static_cast<size_t>(kMaxBlocks) * kMaxRanks * 2 + static_cast<size_t>(blockIdx.x) * kMaxRanks;
        s_doff[p] = meta_mine[p * 2 + 1];
        const unsigned long long g = grant_mine[p];
        if (g < s_slen[p]) s_slen[p] = g;
      }
    } else if (ok) {
      if (threadIdx.x < c.nranks) {
        const int p = threadIdx.x;
        // Equal splits: block `rank` of p's output, as p's recv_off says on
        // every rank alike.
        s_doff[p] = a.recv_off[c.rank];
        if (s_doff[p] + s_slen[p] > a.out_bytes) {
          c.status[0] = c.status[0] | kStatusBadArg;
          s_slen[p] = 0;
        }
      }
    }
    __syncthreads();
    trace_mark(c, 1);
    if (ok) {
      // Block groups: blocks b, b + nranks, ... serve peer (rank + b) % nranks.
      const int nsub = gridDim.x / c.nranks > 0 ? gridDim.x / c.nranks : 1;
      if (gridDim.x >= static_cast<unsigned>(c.nranks)) {
        const int i = blockIdx.x % c.nranks;
        const int sub = blockIdx.x / c.nranks;
        if (sub < nsub) {
          int p = c.rank + i;
          if (p >= c.nranks) p -= c.nranks;
          push_range(a.out.ptr[p] + s_doff[p], a.in + s_soff[p], s_slen[p], sub, nsub);
        }
      } else {
        // Fewer blocks than peers: every block walks all peers and takes its share of each.
        for (int i = 0; i < c.nranks; ++i) {
          int p = c.rank + i;
          if (p >= c.nranks) p -= c.nranks;
          push_range(a.out.ptr[p] + s_doff[p], a.in + s_soff[p], s_slen[p], blockIdx.x, gridDim.x);
        }
      }
      trace_mark(c, 2);
      ok = block_barrier(c, kFlagSetSymA2a, ep, 0x49);
      trace_mark(c, 3);
    }
    ep.store(c, kFlagSetSymA2a);
  }
};

// ------------------------------------------- sequence <-> heads exchange ----
//
// The all-to-all of Ulysses-style sequence parallelism with its two layout
// changes folded in. With n ranks, h heads and s sequence positions per rank:
//   to_heads:  in [b, h, s, d] (all heads, local positions)  ->
//              out [b, h/n, n*s, d] (own heads, all positions, in rank order)
//   to_seq:    the inverse.
// A plain all-to-all needs a permuted copy of the input before it and one of
// the output after it; here every [s, d] slab (contiguous on both sides) goes
// from the caller's tensor straight to its place in the peer's tensor, so the
// data is read once and written once, over NVLink.
// Parity: the scatter-gather collective of comms/ncclx/v2_31/contrib/pace
// (csrc/collective/sg: all-to-all with the tensor layouts of sequence
// parallel attention fused in).
struct SymSeqHeads {
  struct Args {
    const char* in;
    SymmView out;            // symmetric
    int batch, heads;        // heads = h, all of them
    size_t slab_bytes;       // s * d * element size
    int to_heads;
  };
  // Slab `L` of this rank's traffic. Consecutive slabs go to consecutive peers (ring order from the next rank
  // on), so every block's share of the work is spread over all links and the local copy alike.
  static __device__ __forceinline__ void locate(const CommDev& c, const Args& a, size_t L, int* peer, size_t* src_slab,
                                                size_t* dst_slab) {
    const int n = c.nranks, hn = a.heads / n;
    const size_t rem = L / n;
    const int i = static_cast<int>(L - rem * n);
    const size_t bb = rem / hn, j = rem - bb * hn;
    int p = c.rank + 1 + i;
    if (p >= n) p -= n;
    *peer = p;
    const size_t grouped_mine = (bb * hn + j) * n;            // [b, h/n, n, ...] index of slab (bb, j, 0)
    if (a.to_heads) {
      *src_slab = bb * a.heads + static_cast<size_t>(p) * hn + j;
      *dst_slab = grouped_mine + c.rank;
    } else {
      *src_slab = grouped_mine + p;
      *dst_slab = bb * a.heads + static_cast<size_t>(c.rank) * hn + j;
    }
  }
  static __device__ void run(const CommDev& c, const Args& a) {
    BlockEpoch ep;
    ep.load(c, kFlagSetSymA2a);
    trace_mark(c, 0);
    bool ok = block_barrier(c, kFlagSetSymA2a, ep, 0x4a);
    trace_mark(c, 1);
    if (ok) {
      const size_t slabs = static_cast<size_t>(a.batch) * a.heads;
      bool aligned = (reinterpret_cast<uintptr_t>(a.in) & 15u) == 0 && a.slab_bytes % 16 == 0;
      for (int r = 0; r < c.nranks; ++r) aligned = aligned && (reinterpret_cast<uintptr_t>(a.out.ptr[r]) & 15u) == 0;
      if (aligned) {
        const size_t vps = a.slab_bytes / 16;
        size_t v0, v1;
        block_range(slabs * vps, blockIdx.x, gridDim.x, &v0, &v1);
        constexpr int U = kSymmUnroll;
        if (vps >= static_cast<size_t>(blockDim.x) && v1 > v0) {
          // Large slabs: the block walks its range slab by slab, so the index arithmetic is done once per slab.
          for (size_t L = v0 / vps; L * vps < v1; ++L) {
            int p;
            size_t ss, ds;
            locate(c, a, L, &p, &ss, &ds);
            const size_t w0 = (v0 > L * vps ? v0 - L * vps : 0), w1 = min_sz(vps, v1 - L * vps);
            const char* src = a.in + ss * a.slab_bytes;
            char* dst = a.out.ptr[p] + ds * a.slab_bytes;
            for (size_t w = w0 + threadIdx.x; w < w1; w += static_cast<size_t>(U) * blockDim.x) {
              uint4 r[U];
#pragma unroll
              for (int u = 0; u < U; ++u) {
                const size_t ww = w + static_cast<size_t>(u) * blockDim.x;
                if (ww < w1) r[u] = ld16_stream(src + ww * 16);
              }
#pragma unroll
              for (int u = 0; u < U; ++u) {
                const size_t ww = w + static_cast<size_t>(u) * blockDim.x;
                if (ww < w1) st16(dst + ww * 16, r[u]);
              }
            }
          }
        } else {
          for (size_t v = v0 + threadIdx.x; v < v1; v += static_cast<size_t>(U) * blockDim.x) {
            uint4 r[U];
            char* dst[U];
#pragma unroll
            for (int u = 0; u < U; ++u) {
              const size_t vv = v + static_cast<size_t>(u) * blockDim.x;
              if (vv < v1) {
                const size_t L = vv / vps, w = vv - L * vps;
                int p;
                size_t ss, ds;
                locate(c, a, L, &p, &ss, &ds);
                r[u] = ld16_stream(a.in + ss * a.slab_bytes + w * 16);
                dst[u] = a.out.ptr[p] + ds * a.slab_bytes + w * 16;
              }
            }
#pragma unroll
            for (int u = 0; u < U; ++u) {
              const size_t vv = v + static_cast<size_t>(u) * blockDim.x;
              if (vv < v1) st16(dst[u], r[u]);
            }
          }
        }
      } else {
        size_t b0, b1;
        block_range(slabs * a.slab_bytes, blockIdx.x, gridDim.x, &b0, &b1);
        for (size_t i = b0 + threadIdx.x; i < b1; i += blockDim.x) {
          const size_t L = i / a.slab_bytes, w = i - L * a.slab_bytes;
          int p;
          size_t ss, ds;
          locate(c, a, L, &p, &ss, &ds);
          a.out.ptr[p][ds * a.slab_bytes + w] = a.in[ss * a.slab_bytes + w];
        }
      }
      trace_mark(c, 2);
      ok = block_barrier(c, kFlagSetSymA2a, ep, 0x4b);
      trace_mark(c, 3);
    }
    ep.store(c, kFlagSetSymA2a);
  }
};

} // namespace coll

// ------------------------------------------------------------- launchers ----

cudaError_t launch_symm_all_gather(const CommDev* comms, int emu_ranks, const void* const* in, const SymmView* out,
                                   size_t in_bytes, bool cast_f32_to_bf16, bool use_mc, int blocks,
                                   cudaStream_t stream) {
  using namespace coll;
  const int n = emu_ranks > 0 ? emu_ranks : 1;
  const size_t wire = cast_f32_to_bf16 ? in_bytes / 2 : in_bytes;
  if (wire == 0 || wire % 16 != 0) return cudaErrorInvalidValue;
  if (cast_f32_to_bf16) {
    using Op = SymAg<true>;
    std::vector<Op::Args> args(n);
    for (int i = 0; i < n; ++i) args[i] = {static_cast<const char*>(in[i]), out[i], wire, use_mc ? 1 : 0};
    return launch_symm<Op>(comms, emu_ranks, args.data(), blocks, stream);
  }
  using Op = SymAg<false>;
  std::vector<Op::Args> args(n);
  for (int i = 0; i < n; ++i) args[i] = {static_cast<const char*>(in[i]), out[i], wire, use_mc ? 1 : 0};
  return launch_symm<Op>(comms, emu_ranks, args.data(), blocks, stream);
}

namespace {
template <typename WireT, typename OutT>
cudaError_t symm_rs_go(const CommDev* comms, int emu_ranks, const SymmView* in, void* const* out, size_t count,
                       float scale, bool use_mc, int blocks, cudaStream_t stream) {
  using Op = coll::SymRs<WireT, OutT>;
  const int n = emu_ranks > 0 ? emu_ranks : 1;
  if (count == 0 || count % coll::Pack<WireT>::N != 0) return cudaErrorInvalidValue;
  std::vector<typename Op::Args> args(n);
  for (int i = 0; i < n; ++i) args[i] = {in[i], static_cast<OutT*>(out[i]), count, scale, use_mc ? 1 : 0};
  return coll::launch_symm<Op>(comms, emu_ranks, args.data(), blocks, stream);
}
} // namespace

cudaError_t launch_symm_reduce_scatter(const CommDev* comms, int emu_ranks, const SymmView* in, void* const* out,
                                       size_t count, DType wire_dtype, DType out_dtype, float scale, bool use_mc,
                                       int blocks, cudaStream_t stream) {
  using bf16 = __nv_bfloat16;
  if (wire_dtype == DType::BF16 && out_dtype == DType::BF16)
    return symm_rs_go<bf16, bf16>(comms, emu_ranks, in, out, count, scale, use_mc, blocks, stream);
  if (wire_dtype == DType::BF16 && out_dtype == DType::F32)
    return symm_rs_go<bf16, float>(comms, emu_ranks, in, out, count, scale, use_mc, blocks, stream);
  if (wire_dtype == DType::F32 && out_dtype == DType::F32)
    return symm_rs_go<float, float>(comms, emu_ranks, in, out, count, scale, use_mc, blocks, stream);
  if (wire_dtype == DType::F16 && out_dtype == DType::F16)
    return symm_rs_go<__half, __half>(comms, emu_ranks, in, out, count, scale, use_mc, blocks, stream);
  return cudaErrorInvalidValue;
}

cudaError_t launch_symm_all_reduce(const CommDev* comms, int emu_ranks, const SymmView* buf, size_t count, DType dtype,
                                   float scale, bool use_mc, int blocks, cudaStream_t stream) {
  using namespace coll;
  const int n = emu_ranks > 0 ? emu_ranks : 1;
  auto go = [&](auto tag) {
    using T = decltype(tag);
    using Op = SymAr<T>;
    if (count == 0 || count % Pack<T>::N != 0) return cudaErrorInvalidValue;
    std::vector<typename Op::Args> args(n);
    for (int i = 0; i < n; ++i) args[i] = {buf[i], count, scale, use_mc ? 1 : 0};
    return launch_symm<Op>(comms, emu_ranks, args.data(), blocks, stream);
  };
  switch (dtype) {
    case DType::F32: return go(float{});
    case DType::F16: return go(__half{});
    case DType::BF16: return go(__nv_bfloat16{});
  }
  return cudaErrorInvalidValue;
}

cudaError_t launch_symm_all_to_all(const CommDev* comms, const HeapLayout& lay, int emu_ranks, const void* const* in,
                                   const SymmView* out, const size_t* in_bytes, const size_t* out_bytes, const size_t* send_off,
                                   const size_t* send_len, const size_t* recv_off, const size_t* recv_len,
                                   const long long* const* dev_send_counts, size_t elem_bytes, bool exchange,
                                   int blocks, cudaStream_t stream) {
  using namespace coll;
  using Op = SymA2a;
  const int n = emu_ranks > 0 ? emu_ranks : 1;
  const int nranks = comms[0].nranks;
  if (lay.symm_meta_bytes < static_cast<size_t>(kMaxBlocks) * kMaxRanks * 3 * sizeof(unsigned long long)) {
    return cudaErrorInvalidValue;
  }
  std::vector<Op::Args> args(n);
  for (int i = 0; i < n; ++i) {
    Op::Args& a = args[i];
    std::memset(&a, 0, sizeof(a));
    a.in = static_cast<const char*>(in[i]);
    a.out = out[i];
    a.in_bytes = in_bytes[i];
    a.out_bytes = out_bytes[i];
    for (int p = 0; p < nranks; ++p) {
      if (send_off != nullptr) {
        a.send_off[p] = send_off[i * nranks + p];
        a.send_len[p] = send_len[i * nranks + p];
        a.recv_off[p] = recv_off[i * nranks + p];
        a.recv_len[p] = recv_len[i * nranks + p];
      }
    }
    a.dev_send_counts = dev_send_counts != nullptr ? dev_send_counts[i] : nullptr;
    a.elem_bytes = elem_bytes;
    a.meta_off = lay.symm_meta_off;
    a.exchange = (exchange || dev_send_counts != nullptr) ? 1 : 0;
  }
  // Whole block groups per peer.
  if (blocks >= nranks) blocks = blocks / nranks * nranks;
  return launch_symm<Op>(comms, emu_ranks, args.data(), blocks, stream);
}

cudaError_t launch_symm_seq_heads(const CommDev* comms, int emu_ranks, const void* const* in, const SymmView* out,
                                  int batch, int heads, size_t slab_bytes, bool to_heads, int blocks,
                                  cudaStream_t stream) {
  const int n = emu_ranks > 0 ? emu_ranks : 1;
  const int nranks = comms[0].nranks;
  if (batch < 1 || heads < nranks || heads % nranks != 0 || slab_bytes == 0) return cudaErrorInvalidValue;
  std::vector<coll::SymSeqHeads::Args> args(n);
  for (int r = 0; r < n; ++r) {
    args[r].in = static_cast<const char*>(in[r]);
    args[r].out = out[r];
    args[r].batch = batch;
    args[r].heads = heads;
    args[r].slab_bytes = slab_bytes;
    args[r].to_heads = to_heads ? 1 : 0;
  }
  return coll::launch_symm<coll::SymSeqHeads>(comms, emu_ranks, args.data(), blocks, stream);
}

} // namespace b200c
