// Device-side point-to-point primitives over NVLink peer memory, for kernels
// that build their own collective schedules:
//
//   * ThreadGroup   - who cooperates on one primitive: a thread, a warp, a
//                     range of warps (named barrier) or the whole block.
//   * P2pDev        - send / recv / forward between ranks through per-pair
//                     slot FIFOs in symmetric memory: the sender copies a
//                     chunk into a free slot of the receiver and publishes a
//                     chunk counter; the receiver copies it out and returns
//                     the slot by writing its own counter into the sender's
//                     memory. `forward` receives from one peer and sends to
//                     another (and optionally keeps a local copy) without an
//                     intermediate buffer: the step of ring and pipeline
//                     algorithms.
//   * LL packets    - 8-byte {data, flag} words written with one store, so
//                     that the data carries its own arrival flag (one NVLink
//                     trip, no separate signal); for messages of a few KB.
//
// Every wait is bounded (CommDev::timeout_ns -> status word -> false).
// Counters persist in device memory, so calls may be replayed from a graph.
//
// Counterparts in the reference: comms/prims (ThreadGroup.cuh, the NVL
// transport's send / recv / forward device methods, the LL packet helpers).
#pragma once

#include "device_prims.cuh"

namespace b200c {

// What the host fills in for one rank; device code uses it through P2pDev below.
struct P2pDevData {
  CommDev comm;                 // rank, nranks, status word, wait budget
  char* slots[kMaxRanks];       // slots[p]: rank p's receive area, [sender][nslots][slot_bytes]
  uint64_t* ready[kMaxRanks];   // ready[p][sender]: chunks `sender` has published to p (lives on p)
  uint64_t* done[kMaxRanks];    // done[p][receiver]: chunks of p that `receiver` has consumed (lives on p)
  uint64_t* sent;               // local [peer]: chunks sent so far
  uint64_t* rcvd;               // local [peer]: chunks received so far
  int nslots;
  size_t slot_bytes;
};

#ifdef __CUDACC__

struct ThreadGroup {
  enum Kind : int { kThread = 0, kWarp = 1, kWarps = 2, kBlock = 3 };
  int kind;
  int rank;        // this thread's index within the group
  int size;        // threads in the group
  int barrier_id;  // kWarps: named barrier (1..15), distinct per concurrently active group

  static __device__ __forceinline__ ThreadGroup thread() { return {kThread, 0, 1, 0}; }
  static __device__ __forceinline__ ThreadGroup warp() { return {kWarp, static_cast<int>(threadIdx.x & 31), 32, 0}; }
  static __device__ __forceinline__ ThreadGroup block() {
    return {kBlock, static_cast<int>(threadIdx.x), static_cast<int>(blockDim.x), 0};
  }
  // Warps [first_warp, first_warp + nwarps) of the block; call from those warps only.
  static __device__ __forceinline__ ThreadGroup warps(int first_warp, int nwarps, int barrier_id) {
    return {kWarps, static_cast<int>(threadIdx.x) - first_warp * 32, nwarps * 32, barrier_id};
  }
  __device__ __forceinline__ bool leader() const { return rank == 0; }
  __device__ __forceinline__ void sync() const {
    if (kind == kWarp) {
      __syncwarp();
    } else if (kind == kWarps) {
      asm volatile("bar.sync %0, %1;" ::"r"(barrier_id), "r"(size) : "memory");
    } else if (kind == kBlock) {
      __syncthreads();
    }
  }
  // Group-cooperative copy; 16-byte accesses when both pointers and the size allow, bytes otherwise.
  __device__ __forceinline__ void copy(void* __restrict__ dst, const void* __restrict__ src, size_t bytes) const {
    const bool aligned = ((reinterpret_cast<uintptr_t>(dst) | reinterpret_cast<uintptr_t>(src) | bytes) & 15u) == 0;
    if (aligned) {
      const size_t n = bytes / 16;
      for (size_t i = rank; i < n; i += size) {
        st16(static_cast<char*>(dst) + i * 16, ld16(static_cast<const char*>(src) + i * 16));
      }
    } else {
      for (size_t i = rank; i < bytes; i += size) static_cast<char*>(dst)[i] = static_cast<const char*>(src)[i];
    }
  }
};

struct P2pDev : P2pDevData {
  __device__ __forceinline__ char* slot_of(int owner, int sender, uint64_t seq) const {
    return slots[owner] + (static_cast<size_t>(sender) * nslots + seq % nslots) * slot_bytes;
  }
  // All threads of `g` learn whether thread 0's wait succeeded.
  __device__ __forceinline__ bool group_wait(const ThreadGroup& g, const uint64_t* addr, uint64_t want, int peer, uint32_t phase) const {
    __shared__ int s_ok[16];
    bool ok = true;
    if (g.kind == ThreadGroup::kThread) return wait_u64_reached(comm, addr, want, peer, phase);
    if (g.kind == ThreadGroup::kWarp) {
      if (g.leader()) ok = wait_u64_reached(comm, addr, want, peer, phase);
      return __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
    }
    const int cell = g.kind == ThreadGroup::kBlock ? 0 : g.barrier_id;
    if (g.leader()) s_ok[cell] = wait_u64_reached(comm, addr, want, peer, phase) ? 1 : 0;
    g.sync();
    ok = s_ok[cell] != 0;
    g.sync();
    return ok;
  }

  // Sends `bytes` from `src` to `peer`. Blocks (bounded) while all of the pair's slots are still in use.
  __device__ __forceinline__ bool send(const ThreadGroup& g, int peer, const void* src, size_t bytes) const {
    uint64_t seq = sent[peer];
    g.sync();   // everybody has read the counter before the leader advances it
    bool ok = true;
    for (size_t off = 0; off < bytes && ok; off += slot_bytes, ++seq) {
      const size_t n = bytes - off < slot_bytes ? bytes - off : slot_bytes;
      if (seq >= static_cast<uint64_t>(nslots)) {
        ok = group_wait(g, done[comm.rank] + peer, seq - nslots + 1, peer, 0xb1);
        if (!ok) break;
      }
      g.copy(slot_of(peer, comm.rank, seq), static_cast<const char*>(src) + off, n);
      g.sync();
      if (g.leader()) {
        __threadfence_system();
        st_release_sys_u64(ready[peer] + comm.rank, seq + 1);
      }
    }
    g.sync();
    if (g.leader()) sent[peer] = seq;
    return ok;
  }

  // Receives `bytes` from `peer` into `dst`.
  __device__ __forceinline__ bool recv(const ThreadGroup& g, int peer, void* dst, size_t bytes) const {
    uint64_t seq = rcvd[peer];
    g.sync();
    bool ok = true;
    for (size_t off = 0; off < bytes && ok; off += slot_bytes, ++seq) {
      const size_t n = bytes - off < slot_bytes ? bytes - off : slot_bytes;
      ok = group_wait(g, ready[comm.rank] + peer, seq + 1, peer, 0xb2);
      if (!ok) break;
      g.copy(static_cast<char*>(dst) + off, slot_of(comm.rank, peer, seq), n);
      g.sync();
      if (g.leader()) st_release_sys_u64(done[peer] + comm.rank, seq + 1);
    }
    g.sync();
    if (g.leader()) rcvd[peer] = seq;
    return ok;
  }

  // Receives `bytes` from `from` and sends them on to `to`, chunk by chunk; `keep` (optional) gets a copy.
  __device__ __forceinline__ bool forward(const ThreadGroup& g, int from, int to, void* keep, size_t bytes) const {
    uint64_t rseq = rcvd[from], sseq = sent[to];
    g.sync();
    bool ok = true;
    for (size_t off = 0; off < bytes && ok; off += slot_bytes, ++rseq, ++sseq) {
      const size_t n = bytes - off < slot_bytes ? bytes - off : slot_bytes;
      ok = group_wait(g, ready[comm.rank] + from, rseq + 1, from, 0xb3);
      if (ok && sseq >= static_cast<uint64_t>(nslots)) ok = group_wait(g, done[comm.rank] + to, sseq - nslots + 1, to, 0xb4);
      if (!ok) break;
      const char* in = slot_of(comm.rank, from, rseq);
      g.copy(slot_of(to, comm.rank, sseq), in, n);
      if (keep != nullptr) g.copy(static_cast<char*>(keep) + off, in, n);
      g.sync();
      if (g.leader()) {
        __threadfence_system();
        st_release_sys_u64(ready[to] + comm.rank, sseq + 1);
        st_release_sys_u64(done[from] + comm.rank, rseq + 1);
      }
    }
    g.sync();
    if (g.leader()) {
      rcvd[from] = rseq;
      sent[to] = sseq;
    }
    return ok;
  }
};

// ------------------------------------------------------------- LL packets --
// One 8-byte word = 4 bytes of payload + a 4-byte flag, stored and loaded as a
// unit, so that a reader that sees the expected flag also sees the payload.

__device__ __forceinline__ void ll_store(uint64_t* dst, uint32_t data, uint32_t flag) {
  asm volatile("st.relaxed.sys.global.u64 [%0], %1;" ::"l"(dst), "l"((static_cast<uint64_t>(flag) << 32) | data) : "memory");
}

// Spins (bounded) until the word carries `flag`; false = gave up.
__device__ __forceinline__ bool ll_load(const CommDev& c, const uint64_t* src, uint32_t flag, uint32_t* data, int peer) {
  unsigned long long start = 0;
  for (uint32_t spins = 0;; ++spins) {
    uint64_t v;
    asm volatile("ld.relaxed.sys.global.u64 %0, [%1];" : "=l"(v) : "l"(src) : "memory");
    if (static_cast<uint32_t>(v >> 32) == flag) {
      *data = static_cast<uint32_t>(v);
      return true;
    }
    if ((spins & 63u) == 63u) {
      const unsigned long long now = globaltimer_ns();
      if (start == 0) {
        start = now;
      } else if (now - start > c.timeout_ns) {
        report_timeout(c, peer, 0xb5);
        return false;
      }
    }
  }
}

#endif // __CUDACC__

} // namespace b200c
