// Device-side building blocks shared by every peer-memory kernel: the
// communicator descriptor, system-scope flag loads/stores, bounded waits that
// report instead of trapping, the per-block cross-GPU barrier, 16-byte copies,
// and NVLS multimem wrappers.
//
// Parity (what these replace in the reference): comms/common/AtomicUtils.cuh
// (ld.acquire.sys / st.release.sys wrappers), comms/common/IpcGpuBarrier.cuh:11-197
// (per-block mailbox barrier keyed on blockIdx), comms/prims/core/CopyUtils.cuh:93-140
// (16-byte strided copies), comms/prims/transport/nvl/MultimemNvlReduce.cuh:48-120
// (multimem.ld_reduce / multimem.st), comms/common/fault_tolerance/AbortDevice.cuh
// (bounded device waits; here a wait that runs out sets a status word and the
// kernel falls through to its normal exit - it never traps).
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace b200c {

constexpr int kMaxRanks = 8;        // one NVSwitch domain
constexpr int kMaxBlocks = 640;     // flag rows per flag set (148 SMs x up to 4 resident blocks)
constexpr int kFlagSets = 16;       // independent users of the flag region
constexpr int kFlagSetReady = 0;    // pipelined collectives: "chunk k is staged"
constexpr int kFlagSetDone = 1;     // pipelined collectives: "chunk k is consumed"
constexpr int kFlagSetSmall = 2;    // latency mode: one barrier per call, parity buffers
constexpr int kFlagSetBarrier = 3;  // stand-alone barrier
constexpr int kFlagSetMeta = 4;     // all-to-all count exchange
constexpr int kFlagSetWindow = 5;   // one-sided window signals
constexpr int kFlagSetEp = 6;       // MoE dispatch / combine
constexpr int kFlagSetTp = 7;       // tensor-parallel fused GEMMs
// One set per kind of one-pass collective on symmetric buffers, so that an
// all-gather, a reduce-scatter and an all-reduce of one communicator may run
// at the same time on different streams.
constexpr int kFlagSetSymAg = 8;
constexpr int kFlagSetSymRs = 9;
constexpr int kFlagSetSymAr = 10;
constexpr int kFlagSetSymA2a = 11;
constexpr int kFlagSetLamport = 12; // flag-less small all-reduce: only the per-block call counter is used
constexpr int kPipeSlots = 3;       // staging slots per block in the pipelined collectives

// Bits of the status word a kernel may set (host-visible, mapped pinned memory).
constexpr uint32_t kStatusTimeout = 1u;   // a bounded wait ran out
constexpr uint32_t kStatusAbort = 2u;     // set by the HOST: kernels stop waiting
constexpr uint32_t kStatusBadArg = 4u;    // a bounds / alignment check failed

// Everything a kernel needs to talk to its peers. Passed by value.
struct CommDev {
  int rank;
  int nranks;
  // Symmetric staging region of every rank mapped into this process
  // (heap[rank] is the local one). Same layout on every rank.
  char* heap[kMaxRanks];
  // NVLS multicast mapping of the same region, or nullptr.
  char* mc_heap;
  // Flag region: kFlagSets x kMaxBlocks x kMaxRanks uint32 per rank.
  uint32_t* flags[kMaxRanks];
  uint32_t* mc_flags;
  // Local, private: one epoch counter per (flag set, block).
  uint32_t* epochs;
  // Status record in mapped pinned host memory: [0] status bits,
  // [1] rank, [2] block, [3] peer waited for, [4] phase tag.
  volatile uint32_t* status;
  unsigned long long timeout_ns;  // budget of one wait
  size_t heap_bytes;              // size of the staging region
  // Optional phase trace: kTraceSlots stamps of the device's nanosecond timer per
  // block (nullptr = off). For performance work, see trace_mark().
  long long* trace;
};

constexpr int kTraceSlots = 16;

// Everything below is device code; host translation units only need the
// descriptor above.
#ifdef __CUDACC__

// ---------------------------------------------------------------- PTX ------

__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ uint32_t ld_relaxed_sys(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.relaxed.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void st_release_sys(uint32_t* p, uint32_t v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ void st_relaxed_sys(uint32_t* p, uint32_t v) {
  asm volatile("st.relaxed.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint64_t ld_acquire_sys_u64(const uint64_t* p) {
  uint64_t v;
  asm volatile("ld.acquire.sys.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void st_release_sys_u64(uint64_t* p, uint64_t v) {
  asm volatile("st.release.sys.global.u64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
}
__device__ __forceinline__ uint64_t atom_add_release_sys_u64(uint64_t* p, uint64_t v) {
  uint64_t old;
  asm volatile("atom.add.release.sys.global.u64 %0, [%1], %2;" : "=l"(old) : "l"(p), "l"(v) : "memory");
  return old;
}
__device__ __forceinline__ void red_add_release_sys_u32(uint32_t* p, uint32_t v) {
  asm volatile("red.release.sys.global.add.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ void fence_acq_rel_sys() {
  asm volatile("fence.acq_rel.sys;" ::: "memory");
}
__device__ __forceinline__ unsigned long long globaltimer_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
  return t;
}

// 16-byte global accesses. Peer data is read after an acquire, so plain
// (weak) loads are sufficient; stores to peers are plain as well and are
// published by the release that follows them.
__device__ __forceinline__ uint4 ld16(const void* p) {
  return *reinterpret_cast<const uint4*>(p);
}
__device__ __forceinline__ void st16(void* p, uint4 v) {
  *reinterpret_cast<uint4*>(p) = v;
}
// Streaming variants for data touched once (keeps L2 for the staging slots).
__device__ __forceinline__ uint4 ld16_stream(const void* p) {
  uint4 v;
  asm volatile("ld.global.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p));
  return v;
}

// NVLS: one load that returns the sum over every rank's copy of the address.
__device__ __forceinline__ float4 multimem_ld_reduce_add_f32x4(const void* mc) {
  float4 v;
  asm volatile("multimem.ld_reduce.relaxed.sys.global.add.v4.f32 {%0,%1,%2,%3}, [%4];"
               : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w)
               : "l"(mc)
               : "memory");
  return v;
}
__device__ __forceinline__ uint4 multimem_ld_reduce_add_bf16x8(const void* mc) {
  uint4 v;
  asm volatile("multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v4.bf16x2 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(mc)
               : "memory");
  return v;
}
__device__ __forceinline__ uint4 multimem_ld_reduce_add_f16x8(const void* mc) {
  uint4 v;
  asm volatile("multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v4.f16x2 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(mc)
               : "memory");
  return v;
}
// NVLS: one store that lands in every rank's copy of the address.
__device__ __forceinline__ void multimem_st16(void* mc, uint4 v) {
  asm volatile("multimem.st.relaxed.sys.global.v4.f32 [%0], {%1,%2,%3,%4};" ::"l"(mc),
               "f"(__uint_as_float(v.x)), "f"(__uint_as_float(v.y)), "f"(__uint_as_float(v.z)),
               "f"(__uint_as_float(v.w))
               : "memory");
}
__device__ __forceinline__ void multimem_red_add_u32(uint32_t* mc, uint32_t v) {
  asm volatile("multimem.red.release.sys.global.add.u32 [%0], %1;" ::"l"(mc), "r"(v) : "memory");
}

// ------------------------------------------------------------ waiting ------

// Records why a wait gave up. First reporter wins the detail words; the
// status bit is what the host acts on.
__device__ __forceinline__ void report_timeout(const CommDev& c, int peer, uint32_t phase) {
  volatile uint32_t* s = c.status;
  if ((s[0] & kStatusTimeout) == 0) {
    s[1] = static_cast<uint32_t>(c.rank);
    s[2] = blockIdx.x;
    s[3] = static_cast<uint32_t>(peer);
    s[4] = phase;
  }
  s[0] = s[0] | kStatusTimeout;
  __threadfence_system();
}

__device__ __forceinline__ bool comm_is_dead(const CommDev& c) {
  return (c.status[0] & (kStatusTimeout | kStatusAbort)) != 0;
}

// Spins until *addr has reached `want` (wrap-safe comparison). Gives up after
// c.timeout_ns, or at once when the status word already carries a failure;
// returns false then, and the caller carries on to its normal exit.
__device__ __forceinline__ bool wait_flag_reached(const CommDev& c, const uint32_t* addr, uint32_t want,
                                                  int peer, uint32_t phase) {
  unsigned long long start = 0, next_status = 0;
  uint32_t spins = 0;
  while (true) {
    // Relaxed polling; one acquire fence once the value is there.
    const uint32_t v = ld_relaxed_sys(addr);
    if (static_cast<int32_t>(v - want) >= 0) {
      fence_acq_rel_sys();
      return true;
    }
    if (++spins >= 64u) {
      spins = 0;
      const unsigned long long now = globaltimer_ns();
      if (start == 0) {
        start = now;
        next_status = now + 200000ull;
      } else if (now >= next_status) {
        // The status word lives in host memory: reading it crosses PCIe, so
        // look at it rarely (every 200 us of waiting), never in the hot path.
        next_status = now + 200000ull;
        if (comm_is_dead(c)) {
          return false;
        }
        if (now - start > c.timeout_ns) {
          report_timeout(c, peer, phase);
          return false;
        }
      }
    }
  }
}

__device__ __forceinline__ bool wait_u64_reached(const CommDev& c, const uint64_t* addr, uint64_t want,
                                                 int peer, uint32_t phase) {
  unsigned long long start = 0, next_status = 0;
  uint32_t spins = 0;
  while (true) {
    const uint64_t v = ld_acquire_sys_u64(addr);
    if (static_cast<int64_t>(v - want) >= 0) {
      return true;
    }
    if (++spins >= 64u) {
      spins = 0;
      const unsigned long long now = globaltimer_ns();
      if (start == 0) {
        start = now;
        next_status = now + 200000ull;
      } else if (now >= next_status) {
        next_status = now + 200000ull;
        if (comm_is_dead(c)) {
          return false;
        }
        if (now - start > c.timeout_ns) {
          report_timeout(c, peer, phase);
          return false;
        }
      }
    }
  }
}

// ------------------------------------------------------------ barrier ------

__device__ __forceinline__ uint32_t* flag_slot(const CommDev& c, int owner, int set, int block, int sender) {
  return c.flags[owner] + (static_cast<size_t>(set) * kMaxBlocks + block) * kMaxRanks + sender;
}

// Per-block epoch bookkeeping: every barrier of a given (flag set, block) uses
// the next value of a counter kept in local memory, so kernels need no
// host-side sequence numbers and are safe to replay from a CUDA graph.
struct BlockEpoch {
  uint32_t value;
  __device__ __forceinline__ void load(const CommDev& c, int set) {
    value = c.epochs[set * kMaxBlocks + blockIdx.x];
  }
  __device__ __forceinline__ void store(const CommDev& c, int set) {
    __syncthreads();
    if (threadIdx.x == 0) {
      c.epochs[set * kMaxBlocks + blockIdx.x] = value;
    }
  }
};

// Cross-GPU barrier among the blocks with this blockIdx.x on every rank.
// Everything this block wrote before the call (locally or to peers) is
// visible to the peer blocks after their matching call returns.
// All threads of the block must call it. Returns false if a wait ran out.
__device__ __forceinline__ bool block_barrier(const CommDev& c, int set, BlockEpoch& ep, uint32_t phase) {
  __shared__ int s_ok;
  __syncthreads();
  ep.value += 1;
  if (threadIdx.x == 0) {
    s_ok = 1;
  }
  __syncthreads();
  if (threadIdx.x < c.nranks) {
    // Release: a system fence (one warp instruction for all signalling lanes)
    // makes the whole block's earlier writes visible system-wide before the
    // relaxed flag store that follows it; each lane then polls one peer.
    const int peer = threadIdx.x;
    __threadfence_system();
    st_relaxed_sys(flag_slot(c, peer, set, blockIdx.x, c.rank), ep.value);
    if (!wait_flag_reached(c, flag_slot(c, c.rank, set, blockIdx.x, peer), ep.value, peer, phase)) {
      s_ok = 0;
    }
  }
  __syncthreads();
  return s_ok != 0;
}

// Split-phase signalling for pipelined kernels: a block posts monotonically
// increasing step counts ("ready", "done") to its peers and carries on; the
// matching waits happen one pipeline stage later, when the flags have long
// arrived, so no step ends in a blocking two-sided barrier.

// Waits until every rank's flag of this block in `set` has reached `want`.
// All threads of the block must call it.
__device__ __forceinline__ bool wait_all_peers(const CommDev& c, int set, uint32_t want, uint32_t phase) {
  __shared__ int s_ok_wait;
  __syncthreads();
  if (threadIdx.x == 0) {
    s_ok_wait = 1;
  }
  __syncthreads();
  if (threadIdx.x < c.nranks) {
    const int peer = threadIdx.x;
    if (!wait_flag_reached(c, flag_slot(c, c.rank, set, blockIdx.x, peer), want, peer, phase)) {
      s_ok_wait = 0;
    }
  }
  __syncthreads();
  return s_ok_wait != 0;
}

// Publishes step counts to every rank once all of this block's earlier
// writes (local and remote) are visible system-wide. All threads call it.
__device__ __forceinline__ void post_flags(const CommDev& c, bool post_ready, uint32_t ready_val, bool post_done,
                                           uint32_t done_val) {
  __syncthreads();
  if (threadIdx.x < c.nranks && (post_ready || post_done)) {
    const int peer = threadIdx.x;
    __threadfence_system();
    if (post_ready) {
      st_relaxed_sys(flag_slot(c, peer, kFlagSetReady, blockIdx.x, c.rank), ready_val);
    }
    if (post_done) {
      st_relaxed_sys(flag_slot(c, peer, kFlagSetDone, blockIdx.x, c.rank), done_val);
    }
  }
}

// Stamps the device's nanosecond timer into slot `slot` of this block's trace row (thread 0 of the block).
__device__ __forceinline__ void trace_mark(const CommDev& c, int slot) {
  if (c.trace != nullptr && threadIdx.x == 0 && slot < kTraceSlots) {
    c.trace[static_cast<size_t>(blockIdx.x) * kTraceSlots + slot] = static_cast<long long>(globaltimer_ns());
  }
}

// Stamps the device's nanosecond timer into slot `slot` of this block's trace row. Call from ONE thread
// (any thread: the fused GEMM kernels stamp from the warp that owns the phase). Comparable across the SMs
// of one GPU, not across GPUs.
__device__ __forceinline__ void trace_stamp_ns(const CommDev& c, int slot) {
  if (c.trace != nullptr && slot < kTraceSlots) {
    c.trace[static_cast<size_t>(blockIdx.x) * kTraceSlots + slot] = static_cast<long long>(globaltimer_ns());
  }
}

// ------------------------------------------------------------- copies ------

// Block-cooperative copy of `bytes` bytes. Uses 16-byte accesses when both
// pointers allow it and finishes (or entirely runs) with byte accesses.
__device__ __forceinline__ void block_copy(void* __restrict__ dst, const void* __restrict__ src, size_t bytes) {
  const bool aligned = ((reinterpret_cast<uintptr_t>(dst) | reinterpret_cast<uintptr_t>(src)) & 15u) == 0;
  size_t done = 0;
  if (aligned) {
    const size_t nvec = bytes / 16;
    const uint4* s = reinterpret_cast<const uint4*>(src);
    uint4* d = reinterpret_cast<uint4*>(dst);
    size_t i = threadIdx.x;
    // 4 independent loads in flight per thread.
    for (; i + 3 * blockDim.x < nvec; i += 4 * blockDim.x) {
      const uint4 a = s[i];
      const uint4 b = s[i + blockDim.x];
      const uint4 e = s[i + 2 * blockDim.x];
      const uint4 f = s[i + 3 * blockDim.x];
      d[i] = a;
      d[i + blockDim.x] = b;
      d[i + 2 * blockDim.x] = e;
      d[i + 3 * blockDim.x] = f;
    }
    for (; i < nvec; i += blockDim.x) {
      d[i] = s[i];
    }
    done = nvec * 16;
  }
  const char* sb = static_cast<const char*>(src);
  char* db = static_cast<char*>(dst);
  for (size_t i = done + threadIdx.x; i < bytes; i += blockDim.x) {
    db[i] = sb[i];
  }
}

// ---------------------------------------------------------- conversions ----

__device__ __forceinline__ float2 bf16x2_to_float2(uint32_t v) {
  // bf16 is the upper half of an fp32.
  return make_float2(__uint_as_float(v << 16), __uint_as_float(v & 0xffff0000u));
}
__device__ __forceinline__ uint32_t float2_to_bf16x2(float a, float b) {
  __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
  return *reinterpret_cast<uint32_t*>(&h);
}
__device__ __forceinline__ float2 f16x2_to_float2(uint32_t v) {
  return __half22float2(*reinterpret_cast<const __half2*>(&v));
}
__device__ __forceinline__ uint32_t float2_to_f16x2(float a, float b) {
  __half2 h = __floats2half2_rn(a, b);
  return *reinterpret_cast<uint32_t*>(&h);
}

#endif // __CUDACC__

} // namespace b200c
