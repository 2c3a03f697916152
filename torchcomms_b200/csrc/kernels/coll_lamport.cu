// Flag-less small all-reduce (sm_100a): the data is its own arrival signal.
//
// Every rank stores its message into slot `rank` of a receive buffer on every
// rank (one `multimem.st` per 16 bytes through the switch, or nranks peer
// stores) and then polls its OWN copy of that buffer until no word holds the
// poison value any more; the nranks slots are summed in fp32 in registers.
// No flag is written, no barrier is crossed and nothing is staged first, so a
// call costs one one-way NVLink trip plus the launch.
//
// Three receive buffers rotate, one per call. A call on buffer k % 3 also
// re-poisons buffer (k + 2) % 3, the one the previous call read. That is safe:
// a peer can only be one call ahead of this rank (it needs this rank's data to
// finish a call), and what it writes then goes to buffer (k + 1) % 3.
// The poison word is -0.0f (0x80000000); payload words with that bit pattern
// are sent as +0.0, which changes no sum. Block b only ever touches piece b of
// the buffers, and keeps its own call counter in device memory, so calls of
// different sizes and CUDA-graph replays stay consistent.
//
// The poll is bounded by the communicator's wait budget: when it runs out the
// kernel sets the status word and returns without writing the output.
//
// Replaces, in the reference: the poison-value ("Lamport") kernels of
// comms/ncclx/v2_31/contrib/custom_algos/allreduce/oneshot_mc_allreduce_kernel.cuh:40
// and twoshot_mc_poison_allreduce_kernel.cuh:67.
#include "coll_common.cuh"

namespace b200c {
namespace coll {

constexpr int kLamportThreads = static_cast<int>(kLamportPiece / 16);

__device__ __forceinline__ uint4 ld16_volatile(const void* p) {
  uint4 v;
  asm volatile("ld.volatile.global.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p)
               : "memory");
  return v;
}

// 16 bytes from / to user memory that may not be 16-byte aligned (the choice of
// this kernel depends on sizes only, so that every rank makes the same one).
__device__ __forceinline__ uint4 ld16_any(const char* p, bool aligned) {
  if (aligned) return ld16(p);
  uint4 r;
  char* rb = reinterpret_cast<char*>(&r);
#pragma unroll
  for (int k = 0; k < 16; ++k) rb[k] = p[k];
  return r;
}
__device__ __forceinline__ void st16_any(char* p, uint4 v, bool aligned) {
  if (aligned) {
    st16(p, v);
    return;
  }
  const char* vb = reinterpret_cast<const char*>(&v);
#pragma unroll
  for (int k = 0; k < 16; ++k) p[k] = vb[k];
}

__device__ __forceinline__ uint32_t unpoison(uint32_t w) {
  return w == kLamportPoison ? 0u : w;
}

template <typename T>
struct ArLamport {
  struct Args {
    const T* in;
    T* out;
    size_t count;
    float scale;
    size_t region_off;  // start of the three receive buffers in the communicator's heap
    int use_mc;
  };
  static __device__ __forceinline__ size_t slot_off(const Args& a, uint32_t buf, int slot) {
    return a.region_off +
        ((static_cast<size_t>(buf) * kLamportBlocks + blockIdx.x) * kMaxRanks + slot) * kLamportPiece;
  }
  static __device__ void run(const CommDev& c, const Args& a) {
    constexpr int N = Pack<T>::N;
    const size_t piece_elems = kLamportPiece / sizeof(T);
    const size_t e0 = static_cast<size_t>(blockIdx.x) * piece_elems;
    if (e0 >= a.count) return;  // same decision on every rank
    const size_t n = min_sz(piece_elems, a.count - e0);
    const size_t nvec = (n + N - 1) / N;
    const uint32_t call = c.epochs[kFlagSetLamport * kMaxBlocks + blockIdx.x];
    const uint32_t cur = call % 3u, prev = (call + 2u) % 3u;
    const size_t v = threadIdx.x;
    const bool active = v < nvec;
    trace_mark(c, 0);
    if (active) {
      // 1. send
      const size_t left = n - v * N;
      const bool full = left >= static_cast<size_t>(N);
      uint4 w;
      if (full && (reinterpret_cast<uintptr_t>(a.in + e0) & 15u) == 0) {
        w = ld16(a.in + e0 + v * N);
      } else {
        float f[N];
#pragma unroll
        for (int k = 0; k < N; ++k) f[k] = static_cast<size_t>(k) < left ? Pack<T>::to_float(a.in[e0 + v * N + k]) : 0.0f;
        w = Pack<T>::pack(f);
      }
      w.x = unpoison(w.x);
      w.y = unpoison(w.y);
      w.z = unpoison(w.z);
      w.w = unpoison(w.w);
      const size_t dst = slot_off(a, cur, c.rank) + v * 16;
      if (a.use_mc && c.mc_heap != nullptr) {
        multimem_st16(c.mc_heap + dst, w);
      } else {
#pragma unroll
        for (int i = 0; i < kMaxRanks; ++i) {
          if (i < c.nranks) {
            int p = c.rank + i;
            if (p >= c.nranks) p -= c.nranks;
            st16(c.heap[p] + dst, w);
          }
        }
      }
    }
    // 2. re-poison what the previous call read (the whole piece: that call may
    //    have been longer than this one).
    {
      const uint4 poison = make_uint4(kLamportPoison, kLamportPoison, kLamportPoison, kLamportPoison);
#pragma unroll
      for (int s = 0; s < kMaxRanks; ++s) {
        if (s < c.nranks) st16(c.heap[c.rank] + slot_off(a, prev, s) + v * 16, poison);
      }
    }
    trace_mark(c, 1);
    // 3. gather: poll the local copy of every slot
    bool ok = true;
    float acc[N];
#pragma unroll
    for (int k = 0; k < N; ++k) acc[k] = 0.0f;
    if (active) {
      unsigned long long start = 0;
      uint32_t spins = 0;
      uint4 got[kMaxRanks];
      uint32_t pending = (1u << c.nranks) - 1u;
      while (pending != 0u && ok) {
#pragma unroll
        for (int s = 0; s < kMaxRanks; ++s) {
          if (s < c.nranks && (pending >> s & 1u)) {
            const uint4 x = ld16_volatile(c.heap[c.rank] + slot_off(a, cur, s) + v * 16);
            if (x.x != kLamportPoison && x.y != kLamportPoison && x.z != kLamportPoison && x.w != kLamportPoison) {
              got[s] = x;
              pending &= ~(1u << s);
            }
          }
        }
        if (pending != 0u && ++spins >= 64u) {
          spins = 0;
          const unsigned long long now = globaltimer_ns();
          if (start == 0) {
            start = now;
          } else if (now - start > 200000ull) {
            // Rarely: the status word lives in host memory.
            if (comm_is_dead(c)) {
              ok = false;
            } else if (now - start > c.timeout_ns) {
              int missing = 0;
              for (int s = 0; s < c.nranks; ++s) {
                if (pending >> s & 1u) missing = s;
              }
              report_timeout(c, missing, 0x61);
              ok = false;
            }
          }
        }
      }
      if (ok) {
#pragma unroll
        for (int s = 0; s < kMaxRanks; ++s) {
          if (s < c.nranks) {
            float f[N];
            Pack<T>::unpack(got[s], f);
#pragma unroll
            for (int k = 0; k < N; ++k) acc[k] += f[k];
          }
        }
#pragma unroll
        for (int k = 0; k < N; ++k) acc[k] *= a.scale;
        const size_t left = n - v * N;
        const bool aligned = (reinterpret_cast<uintptr_t>(a.out + e0) & 15u) == 0;
        store_values<T, N>(a.out + e0 + v * N, acc, left < static_cast<size_t>(N) ? static_cast<int>(left) : N, aligned);
      }
    }
    trace_mark(c, 2);
    __syncthreads();
    if (threadIdx.x == 0) c.epochs[kFlagSetLamport * kMaxBlocks + blockIdx.x] = call + 1u;
  }
};

// The same arrival protocol for the other small collectives. One block owns
// 4 KB of every rank's part; what differs is what is sent where and what the
// receiver does with its nranks slots:
//   GATHER   every rank's part goes to everybody (multicast when available);
//            the receiver copies slot s to part s of the output
//   SCATTER  part p of the input goes to rank p only; the receiver copies slot
//            s to part s of the output (all-to-all with equal parts)
//   REDUCE   part p of the input goes to rank p only; the receiver sums its
//            slots in fp32 (reduce-scatter)
// Parts are whole 16-byte vectors of a floating type (a payload word equal to
// the poison word is sent as +0.0, which would corrupt integer data).
enum class LamportMode : int { GATHER = 0, SCATTER = 1, REDUCE = 2 };

template <typename T, LamportMode M>
struct XchgLamport {
  struct Args {
    const char* in;
    char* out;
    size_t part_bytes;   // bytes per rank part; multiple of 16
    float scale;         // REDUCE only
    size_t region_off;
    int use_mc;
  };
  static __device__ __forceinline__ size_t slot_off(const Args& a, uint32_t buf, int slot) {
    return a.region_off +
        ((static_cast<size_t>(buf) * kLamportBlocks + blockIdx.x) * kMaxRanks + slot) * kLamportPiece;
  }
  static __device__ void run(const CommDev& c, const Args& a) {
    constexpr int N = Pack<T>::N;
    const size_t b0 = static_cast<size_t>(blockIdx.x) * kLamportPiece;
    if (b0 >= a.part_bytes) return;  // same decision on every rank
    const size_t nvec = min_sz(kLamportPiece, a.part_bytes - b0) / 16;
    const uint32_t call = c.epochs[kFlagSetLamport * kMaxBlocks + blockIdx.x];
    const uint32_t cur = call % 3u, prev = (call + 2u) % 3u;
    const size_t v = threadIdx.x;
    const bool active = v < nvec;
    const bool in_al = (reinterpret_cast<uintptr_t>(a.in) & 15u) == 0;
    const bool out_al = (reinterpret_cast<uintptr_t>(a.out) & 15u) == 0;
    if (active) {
      if (M == LamportMode::GATHER) {
        uint4 w = ld16_any(a.in + b0 + v * 16, in_al);
        w.x = unpoison(w.x);
        w.y = unpoison(w.y);
        w.z = unpoison(w.z);
        w.w = unpoison(w.w);
        const size_t dst = slot_off(a, cur, c.rank) + v * 16;
        if (a.use_mc && c.mc_heap != nullptr) {
          multimem_st16(c.mc_heap + dst, w);
        } else {
#pragma unroll
          for (int i = 0; i < kMaxRanks; ++i) {
            if (i < c.nranks) {
              int p = c.rank + i;
              if (p >= c.nranks) p -= c.nranks;
              st16(c.heap[p] + dst, w);
            }
          }
        }
      } else {
        uint4 w[kMaxRanks];
#pragma unroll
        for (int i = 0; i < kMaxRanks; ++i) {
          if (i < c.nranks) {
            int p = c.rank + i;
            if (p >= c.nranks) p -= c.nranks;
            w[i] = ld16_any(a.in + static_cast<size_t>(p) * a.part_bytes + b0 + v * 16, in_al);
          }
        }
        const size_t dst = slot_off(a, cur, c.rank) + v * 16;
#pragma unroll
        for (int i = 0; i < kMaxRanks; ++i) {
          if (i < c.nranks) {
            int p = c.rank + i;
            if (p >= c.nranks) p -= c.nranks;
            uint4 x = w[i];
            x.x = unpoison(x.x);
            x.y = unpoison(x.y);
            x.z = unpoison(x.z);
            x.w = unpoison(x.w);
            st16(c.heap[p] + dst, x);
          }
        }
      }
    }
    {
      const uint4 poison = make_uint4(kLamportPoison, kLamportPoison, kLamportPoison, kLamportPoison);
#pragma unroll
      for (int s = 0; s < kMaxRanks; ++s) {
        if (s < c.nranks) st16(c.heap[c.rank] + slot_off(a, prev, s) + v * 16, poison);
      }
    }
    if (active) {
      bool ok = true;
      unsigned long long start = 0;
      uint32_t spins = 0;
      uint4 got[kMaxRanks];
      uint32_t pending = (1u << c.nranks) - 1u;
      while (pending != 0u && ok) {
#pragma unroll
        for (int s = 0; s < kMaxRanks; ++s) {
          if (s < c.nranks && (pending >> s & 1u)) {
            const uint4 x = ld16_volatile(c.heap[c.rank] + slot_off(a, cur, s) + v * 16);
            if (x.x != kLamportPoison && x.y != kLamportPoison && x.z != kLamportPoison && x.w != kLamportPoison) {
              got[s] = x;
              pending &= ~(1u << s);
            }
          }
        }
        if (pending != 0u && ++spins >= 64u) {
          spins = 0;
          const unsigned long long now = globaltimer_ns();
          if (start == 0) {
            start = now;
          } else if (now - start > 200000ull) {
            if (comm_is_dead(c)) {
              ok = false;
            } else if (now - start > c.timeout_ns) {
              int missing = 0;
              for (int s = 0; s < c.nranks; ++s) {
                if (pending >> s & 1u) missing = s;
              }
              report_timeout(c, missing, 0x62);
              ok = false;
            }
          }
        }
      }
      if (ok) {
        if (M == LamportMode::REDUCE) {
          float acc[N];
#pragma unroll
          for (int k = 0; k < N; ++k) acc[k] = 0.0f;
#pragma unroll
          for (int s = 0; s < kMaxRanks; ++s) {
            if (s < c.nranks) {
              float f[N];
              Pack<T>::unpack(got[s], f);
#pragma unroll
              for (int k = 0; k < N; ++k) acc[k] += f[k];
            }
          }
#pragma unroll
          for (int k = 0; k < N; ++k) acc[k] *= a.scale;
          st16_any(a.out + b0 + v * 16, Pack<T>::pack(acc), out_al);
        } else {
#pragma unroll
          for (int s = 0; s < kMaxRanks; ++s) {
            if (s < c.nranks) st16_any(a.out + static_cast<size_t>(s) * a.part_bytes + b0 + v * 16, got[s], out_al);
          }
        }
      }
    }
    __syncthreads();
    if (threadIdx.x == 0) c.epochs[kFlagSetLamport * kMaxBlocks + blockIdx.x] = call + 1u;
  }
};

// All-to-all with unequal parts (floating types). Every rank knows from the call's arguments how many bytes it sends
// to and receives from each peer, so no lengths travel: the sender stores len(rank -> p) bytes into p's slot, the
// receiver polls exactly len(s -> rank) bytes of slot s. Which blocks take part must not depend on the rank: it is
// `cap_bytes`, a bound that every rank derives from the same quantity (the size of the symmetric receive buffer).
// Lengths need not be multiples of 16: the last vector of a part is sent padded with zeros and only its valid bytes
// are written to the output.
struct XchgvLamport {
  struct Args {
    const char* in;
    char* out;
    size_t send_off[kMaxRanks], send_len[kMaxRanks];
    size_t recv_off[kMaxRanks], recv_len[kMaxRanks];
    size_t cap_bytes;
    size_t region_off;
  };
  static __device__ __forceinline__ size_t slot_off(const Args& a, uint32_t buf, int slot) {
    return a.region_off +
        ((static_cast<size_t>(buf) * kLamportBlocks + blockIdx.x) * kMaxRanks + slot) * kLamportPiece;
  }
  // 16 bytes starting at p of which only `valid` (1..16) may be read; the rest reads as zero.
  static __device__ __forceinline__ uint4 load_tail(const char* p, size_t valid, bool aligned) {
    if (valid >= 16) return ld16_any(p, aligned);
    uint4 w = make_uint4(0u, 0u, 0u, 0u);
    unsigned char* b = reinterpret_cast<unsigned char*>(&w);
    for (size_t i = 0; i < valid; ++i) b[i] = static_cast<unsigned char>(p[i]);
    return w;
  }
  static __device__ __forceinline__ void store_tail(char* p, uint4 w, size_t valid, bool aligned) {
    if (valid >= 16) {
      st16_any(p, w, aligned);
      return;
    }
    const unsigned char* b = reinterpret_cast<const unsigned char*>(&w);
    for (size_t i = 0; i < valid; ++i) p[i] = static_cast<char>(b[i]);
  }
  static __device__ void run(const CommDev& c, const Args& a) {
    const size_t b0 = static_cast<size_t>(blockIdx.x) * kLamportPiece;
    if (b0 >= a.cap_bytes) return;  // same decision on every rank
    const uint32_t call = c.epochs[kFlagSetLamport * kMaxBlocks + blockIdx.x];
    const uint32_t cur = call % 3u, prev = (call + 2u) % 3u;
    const size_t pos = b0 + static_cast<size_t>(threadIdx.x) * 16;   // this thread's vector within every part
    const size_t v16 = static_cast<size_t>(threadIdx.x) * 16;
#pragma unroll
    for (int i = 0; i < kMaxRanks; ++i) {
      if (i < c.nranks) {
        int p = c.rank + i;
        if (p >= c.nranks) p -= c.nranks;
        if (pos < a.send_len[p]) {
          const char* src = a.in + a.send_off[p] + pos;
          uint4 w = load_tail(src, a.send_len[p] - pos, (reinterpret_cast<uintptr_t>(src) & 15u) == 0);
          w.x = unpoison(w.x);
          w.y = unpoison(w.y);
          w.z = unpoison(w.z);
          w.w = unpoison(w.w);
          st16(c.heap[p] + slot_off(a, cur, c.rank) + v16, w);
        }
      }
    }
    {
      const uint4 poison = make_uint4(kLamportPoison, kLamportPoison, kLamportPoison, kLamportPoison);
#pragma unroll
      for (int s = 0; s < kMaxRanks; ++s) {
        if (s < c.nranks) st16(c.heap[c.rank] + slot_off(a, prev, s) + v16, poison);
      }
    }
    uint32_t pending = 0;
#pragma unroll
    for (int s = 0; s < kMaxRanks; ++s) {
      if (s < c.nranks && pos < a.recv_len[s]) pending |= 1u << s;
    }
    bool ok = true;
    unsigned long long start = 0;
    uint32_t spins = 0;
    while (pending != 0u && ok) {
#pragma unroll
      for (int s = 0; s < kMaxRanks; ++s) {
        if (s < c.nranks && (pending >> s & 1u)) {
          const uint4 x = ld16_volatile(c.heap[c.rank] + slot_off(a, cur, s) + v16);
          if (x.x != kLamportPoison && x.y != kLamportPoison && x.z != kLamportPoison && x.w != kLamportPoison) {
            char* dst = a.out + a.recv_off[s] + pos;
            store_tail(dst, x, a.recv_len[s] - pos, (reinterpret_cast<uintptr_t>(dst) & 15u) == 0);
            pending &= ~(1u << s);
          }
        }
      }
      if (pending != 0u && ++spins >= 64u) {
        spins = 0;
        const unsigned long long now = globaltimer_ns();
        if (start == 0) {
          start = now;
        } else if (now - start > 200000ull) {
          if (comm_is_dead(c)) {
            ok = false;
          } else if (now - start > c.timeout_ns) {
            int missing = 0;
            for (int s = 0; s < c.nranks; ++s) {
              if (pending >> s & 1u) missing = s;
            }
            report_timeout(c, missing, 0x63);
            ok = false;
          }
        }
      }
    }
    __syncthreads();
    if (threadIdx.x == 0) c.epochs[kFlagSetLamport * kMaxBlocks + blockIdx.x] = call + 1u;
  }
};

__global__ void k_fill_u32(uint32_t* p, size_t words, uint32_t value) {
  for (size_t i = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x; i < words;
       i += static_cast<size_t>(gridDim.x) * blockDim.x) {
    p[i] = value;
  }
}

} // namespace coll

cudaError_t launch_lamport_init(char* region, cudaStream_t stream) {
  note_kernel_launch();
  coll::k_fill_u32<<<64, 256, 0, stream>>>(reinterpret_cast<uint32_t*>(region), kLamportBytes / 4, kLamportPoison);
  return cudaGetLastError();
}

cudaError_t launch_all_reduce_lamport(const CommDev* comms, const HeapLayout& lay, int emu_ranks, const void* const* in,
                                      void* const* out, size_t count, DType dtype, float scale, bool use_mc,
                                      cudaStream_t stream) {
  using namespace coll;
  const int n = emu_ranks > 0 ? emu_ranks : 1;
  if (lay.lamport_bytes < kLamportBytes) return cudaErrorInvalidValue;
  const size_t bytes = count * dtype_size(dtype);
  if (bytes == 0 || bytes > static_cast<size_t>(kLamportBlocks) * kLamportPiece) return cudaErrorInvalidValue;
  const int blocks = static_cast<int>((bytes + kLamportPiece - 1) / kLamportPiece);
  auto go = [&](auto tag) {
    using T = decltype(tag);
    using Op = ArLamport<T>;
    std::vector<typename Op::Args> args(n);
    for (int i = 0; i < n; ++i) {
      args[i] = {static_cast<const T*>(in[i]), static_cast<T*>(out[i]), count, scale, lay.lamport_off, use_mc ? 1 : 0};
    }
    return launch_op<Op>(comms, emu_ranks, args.data(), blocks, kLamportThreads, stream, true);
  };
  switch (dtype) {
    case DType::F32: return go(float{});
    case DType::F16: return go(__half{});
    case DType::BF16: return go(__nv_bfloat16{});
  }
  return cudaErrorInvalidValue;
}

cudaError_t launch_exchange_lamport(const CommDev* comms, const HeapLayout& lay, int emu_ranks, int mode,
                                    const void* const* in, void* const* out, size_t part_bytes, DType dtype, float scale,
                                    bool use_mc, cudaStream_t stream) {
  using namespace coll;
  const int n = emu_ranks > 0 ? emu_ranks : 1;
  if (lay.lamport_bytes < kLamportBytes) return cudaErrorInvalidValue;
  if (part_bytes == 0 || part_bytes % 16 != 0 || part_bytes > static_cast<size_t>(kLamportBlocks) * kLamportPiece) {
    return cudaErrorInvalidValue;
  }
  const int blocks = static_cast<int>((part_bytes + kLamportPiece - 1) / kLamportPiece);
  auto go = [&](auto tag, auto mode_tag) {
    using T = decltype(tag);
    using Op = XchgLamport<T, decltype(mode_tag)::value>;
    std::vector<typename Op::Args> args(n);
    for (int i = 0; i < n; ++i) {
      args[i] = {static_cast<const char*>(in[i]), static_cast<char*>(out[i]), part_bytes, scale, lay.lamport_off, use_mc ? 1 : 0};
    }
    return launch_op<Op>(comms, emu_ranks, args.data(), blocks, kLamportThreads, stream, true);
  };
  using G = std::integral_constant<LamportMode, LamportMode::GATHER>;
  using S = std::integral_constant<LamportMode, LamportMode::SCATTER>;
  using R = std::integral_constant<LamportMode, LamportMode::REDUCE>;
  if (mode == 0) return go(float{}, G{});
  if (mode == 1) return go(float{}, S{});
  if (mode != 2) return cudaErrorInvalidValue;
  switch (dtype) {
    case DType::F32: return go(float{}, R{});
    case DType::F16: return go(__half{}, R{});
    case DType::BF16: return go(__nv_bfloat16{}, R{});
  }
  return cudaErrorInvalidValue;
}

cudaError_t launch_exchangev_lamport(const CommDev* comms, const HeapLayout& lay, int emu_ranks, const void* const* in,
                                     void* const* out, const size_t* send_off, const size_t* send_len, const size_t* recv_off,
                                     const size_t* recv_len, size_t cap_bytes, cudaStream_t stream) {
  using namespace coll;
  const int n = emu_ranks > 0 ? emu_ranks : 1;
  const int nr = comms[0].nranks;
  if (lay.lamport_bytes < kLamportBytes) return cudaErrorInvalidValue;
  if (cap_bytes == 0 || cap_bytes > static_cast<size_t>(kLamportBlocks) * kLamportPiece) return cudaErrorInvalidValue;
  std::vector<XchgvLamport::Args> args(n);
  for (int i = 0; i < n; ++i) {
    XchgvLamport::Args& a = args[i];
    a = XchgvLamport::Args{};
    a.in = static_cast<const char*>(in[i]);
    a.out = static_cast<char*>(out[i]);
    for (int p = 0; p < nr; ++p) {
      a.send_off[p] = send_off[i * kMaxRanks + p];
      a.send_len[p] = send_len[i * kMaxRanks + p];
      a.recv_off[p] = recv_off[i * kMaxRanks + p];
      a.recv_len[p] = recv_len[i * kMaxRanks + p];
      if (a.send_len[p] > cap_bytes || a.recv_len[p] > cap_bytes) return cudaErrorInvalidValue;
    }
    a.cap_bytes = cap_bytes;
    a.region_off = lay.lamport_off;
  }
  const int blocks = static_cast<int>((cap_bytes + kLamportPiece - 1) / kLamportPiece);
  return launch_op<XchgvLamport>(comms, emu_ranks, args.data(), blocks, kLamportThreads, stream, true);
}

} // namespace b200c
