// Device-side view of a one-sided window, usable from user CUDA kernels.
//
// A `DeviceWindow` lives in device memory (its address is what
// TorchCommWindow.get_device_window() returns). Through it a kernel can store
// into any rank's registered buffer over NVLink (`put`), raise and wait on
// signals, count completed puts, and run a block-scope barrier across ranks,
// without any host involvement. All waits are bounded: when the budget runs
// out they return false and set the communicator's status word.
//
// Parity: comms/torchcomms/device/TorchCommDeviceWindow.hpp:42-260 (put, signal,
// wait_signal, wait_signal_from, read/reset_signal, wait/read/reset_counter,
// fence, flush, barrier, get_nvlink_address, get_multimem_address, CoopScope)
// and comms/torchcomms/RegisteredBuffer.hpp:30-52. Signals are per-(id, sender)
// 64-bit slots in the owner's memory, as in
// comms/torchcomms/device/ncclx/TorchCommDeviceNCCLX.cuh:149-215,301-329.
#pragma once

#include "device_prims.cuh"

namespace b200c {

enum class CoopScope : int { THREAD = 0, WARP = 1, BLOCK = 2 };
enum class SignalOp : int { SET = 0, ADD = 1 };
enum class CmpOp : int { EQ = 0, NE = 1, GE = 2, GT = 3, LE = 4, LT = 5 };

// A local source buffer a kernel may `put` from.
struct RegisteredBuffer {
  char* base;
  size_t size;
};

struct DeviceWindow {
  int rank;
  int nranks;
  size_t bytes;                      // size of every rank's registered buffer
  char* data[kMaxRanks];             // registered buffer of each rank, mapped here
  char* mc_data;                     // multicast mapping of the buffers, or nullptr
  int signal_count;
  int counter_count;
  int barrier_count;
  // signals[r]: rank r's signal table, signal_count x nranks uint64 (slot [id][sender])
  uint64_t* signals[kMaxRanks];
  uint64_t* counters;                // local, counter_count uint64
  uint64_t* barrier_flags[kMaxRanks];  // barrier_count x nranks uint64 per rank
  uint64_t* barrier_epochs;          // local, barrier_count uint64
  volatile uint32_t* status;         // communicator status word (mapped pinned host memory)
  unsigned long long timeout_ns;

#ifdef __CUDACC__  // device-side methods; host code only needs the layout above
  __device__ __forceinline__ CommDev as_comm() const {
    CommDev c{};
    c.rank = rank;
    c.nranks = nranks;
    c.status = status;
    c.timeout_ns = timeout_ns;
    return c;
  }

  __device__ __forceinline__ char* get_nvlink_address(int peer, size_t offset = 0) const { return data[peer] + offset; }
  __device__ __forceinline__ char* get_multimem_address(size_t offset = 0) const {
    return mc_data ? mc_data + offset : nullptr;
  }

  // Orders this thread's earlier stores before its later signal / flag writes
  // as seen by any GPU.
  __device__ __forceinline__ void fence() const { __threadfence_system(); }
  // Stores over NVLink are posted; a system fence is also what drains them.
  __device__ __forceinline__ void flush() const { __threadfence_system(); }

  __device__ __forceinline__ void signal(int peer, int signal_id, SignalOp op = SignalOp::ADD, uint64_t value = 1) const {
    uint64_t* slot = signals[peer] + static_cast<size_t>(signal_id) * nranks + rank;
    if (op == SignalOp::ADD) {
      atom_add_release_sys_u64(slot, value);
    } else {
      st_release_sys_u64(slot, value);
    }
  }

  __device__ __forceinline__ uint64_t read_signal(int signal_id) const {
    uint64_t sum = 0;
    for (int p = 0; p < nranks; ++p) {
      sum += ld_acquire_sys_u64(signals[rank] + static_cast<size_t>(signal_id) * nranks + p);
    }
    return sum;
  }
  __device__ __forceinline__ uint64_t read_signal_from(int signal_id, int peer) const {
    return ld_acquire_sys_u64(signals[rank] + static_cast<size_t>(signal_id) * nranks + peer);
  }
  __device__ __forceinline__ void reset_signal(int signal_id) const {
    for (int p = 0; p < nranks; ++p) {
      st_release_sys_u64(signals[rank] + static_cast<size_t>(signal_id) * nranks + p, 0);
    }
  }

  static __device__ __forceinline__ bool compare(uint64_t v, CmpOp cmp, uint64_t want) {
    switch (cmp) {
      case CmpOp::EQ: return v == want;
      case CmpOp::NE: return v != want;
      case CmpOp::GE: return v >= want;
      case CmpOp::GT: return v > want;
      case CmpOp::LE: return v <= want;
      default: return v < want;
    }
  }

  // Waits until the sum over senders of signal `signal_id` satisfies the
  // comparison. One thread polls; callers synchronise their group afterwards.
  __device__ __forceinline__ bool wait_signal(int signal_id, CmpOp cmp, uint64_t value) const {
    const CommDev c = as_comm();
    unsigned long long start = 0;
    uint32_t spins = 0;
    while (true) {
      if (compare(read_signal(signal_id), cmp, value)) return true;
      if (++spins >= 64u) {
        spins = 0;
        if (comm_is_dead(c)) return false;
        const unsigned long long now = globaltimer_ns();
        if (start == 0) start = now;
        else if (now - start > timeout_ns) { report_timeout(c, -1, 0x80u + signal_id); return false; }
        __nanosleep(64);
      }
    }
  }
  __device__ __forceinline__ bool wait_signal_from(int peer, int signal_id, CmpOp cmp, uint64_t value) const {
    const CommDev c = as_comm();
    unsigned long long start = 0;
    uint32_t spins = 0;
    while (true) {
      if (compare(read_signal_from(signal_id, peer), cmp, value)) return true;
      if (++spins >= 64u) {
        spins = 0;
        if (comm_is_dead(c)) return false;
        const unsigned long long now = globaltimer_ns();
        if (start == 0) start = now;
        else if (now - start > timeout_ns) { report_timeout(c, peer, 0x80u + signal_id); return false; }
        __nanosleep(64);
      }
    }
  }

  __device__ __forceinline__ uint64_t read_counter(int counter_id) const {
    return ld_acquire_sys_u64(counters + counter_id);
  }
  __device__ __forceinline__ void reset_counter(int counter_id) const { st_release_sys_u64(counters + counter_id, 0); }
  __device__ __forceinline__ bool wait_counter(int counter_id, CmpOp cmp, uint64_t value) const {
    const CommDev c = as_comm();
    unsigned long long start = 0;
    uint32_t spins = 0;
    while (true) {
      if (compare(read_counter(counter_id), cmp, value)) return true;
      if (++spins >= 64u) {
        spins = 0;
        if (comm_is_dead(c)) return false;
        const unsigned long long now = globaltimer_ns();
        if (start == 0) start = now;
        else if (now - start > timeout_ns) { report_timeout(c, -1, 0xc0u + counter_id); return false; }
        __nanosleep(64);
      }
    }
  }

  // Copies `bytes` from a registered local buffer into rank `dst_rank`'s
  // window at `dst_offset`, cooperatively over `scope`. If signal_id >= 0 the
  // destination's signal is raised (ADD 1) once the data is visible there; if
  // counter_id >= 0 the local counter is bumped when the stores were issued
  // and fenced. Every thread of the scope must call it with the same arguments.
  __device__ __forceinline__ void put(size_t dst_offset, const RegisteredBuffer& src, size_t src_offset, int dst_rank,
                                      size_t bytes, int signal_id = -1, int counter_id = -1,
                                      CoopScope scope = CoopScope::BLOCK) const {
    char* dst = data[dst_rank] + dst_offset;
    const char* from = src.base + src_offset;
    int lane = 0, width = 1;
    if (scope == CoopScope::WARP) {
      lane = threadIdx.x & 31;
      width = 32;
    } else if (scope == CoopScope::BLOCK) {
      lane = threadIdx.x;
      width = blockDim.x;
    }
    const bool aligned = ((reinterpret_cast<uintptr_t>(dst) | reinterpret_cast<uintptr_t>(from)) & 15u) == 0;
    size_t done = 0;
    if (aligned) {
      const size_t nvec = bytes / 16;
      for (size_t i = lane; i < nvec; i += width) {
        st16(dst + i * 16, ld16(from + i * 16));
      }
      done = nvec * 16;
    }
    for (size_t i = done + lane; i < bytes; i += width) {
      dst[i] = from[i];
    }
    __threadfence_system();
    if (scope == CoopScope::WARP) {
      __syncwarp();
    } else if (scope == CoopScope::BLOCK) {
      __syncthreads();
    }
    if (lane == 0) {
      if (signal_id >= 0) signal(dst_rank, signal_id, SignalOp::ADD, 1);
      if (counter_id >= 0) atom_add_release_sys_u64(counters + counter_id, 1);
    }
  }

  // Block-scope barrier across all ranks on barrier slot `barrier_id`. The
  // same block index must call it on every rank.
  __device__ __forceinline__ bool barrier(int barrier_id) const {
    __shared__ int s_ok;
    __syncthreads();
    if (threadIdx.x == 0) s_ok = 1;
    __syncthreads();
    const uint64_t epoch = barrier_epochs[barrier_id] + 1;
    const CommDev c = as_comm();
    if (threadIdx.x < nranks) {
      const int peer = threadIdx.x;
      __threadfence_system();
      st_release_sys_u64(barrier_flags[peer] + static_cast<size_t>(barrier_id) * nranks + rank, epoch);
      if (!wait_u64_reached(c, barrier_flags[rank] + static_cast<size_t>(barrier_id) * nranks + peer, epoch, peer, 0xe0)) {
        s_ok = 0;
      }
    }
    __syncthreads();
    if (threadIdx.x == 0) barrier_epochs[barrier_id] = epoch;
    __syncthreads();
    return s_ok != 0;
  }
#endif // __CUDACC__
};

} // namespace b200c
