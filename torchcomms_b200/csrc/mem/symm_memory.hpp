// Peer-memory registry: symmetric allocations that every rank of a
// communicator can load from and store to, optionally bound to an NVLS
// multicast object.
//
// One process per GPU. A segment is created with the CUDA virtual-memory API
// (cuMemCreate with a POSIX-fd shareable handle), its descriptor travels to
// the peers over unix-domain sockets (SCM_RIGHTS), and every rank maps all
// members back to back into one reserved address range, so that
// `peer_ptr(r) = base + r * bytes`. When the device supports multicast the same
// physical memory is bound into a multicast object whose mapping (`mc_ptr`)
// makes `multimem.*` instructions reach every rank's copy through the switch.
// Where shareable VMM handles are not permitted the segment falls back to
// cudaMalloc + CUDA IPC handles (no multicast then).
//
// Parity: comms/prims/memory (CuMemAllocation.cc:104, CuMemMapping.cc:32-45,
// GpuMemHandler.cc:123-134 mode selection, NvlMemExchange.cc:63-97 fd passing,
// MultimemHandler.cc:67-70,369,458 multicast create / add-device-before-bind)
// and comms/ctran/utils/CtranMulticast.h.
#pragma once

#include <c10/util/intrusive_ptr.h>
#include <torch/csrc/distributed/c10d/Store.hpp>

#include <map>
#include <memory>
#include <mutex>
#include <string>
#include <vector>

#include "../cuda/driver_api.hpp"

namespace b200c {

enum class SymmMode : int { LOCAL = 0, VMM_FD = 1, CUDA_IPC = 2 };

struct SymmSegment {
  size_t bytes = 0;                 // per-rank size
  int rank = 0, nranks = 1;
  SymmMode mode = SymmMode::LOCAL;
  std::vector<char*> peer_ptrs;     // [nranks]; peer_ptrs[rank] is local memory
  char* mc_ptr = nullptr;           // multicast mapping or null
  char* local() const { return peer_ptrs[rank]; }

  // teardown bookkeeping
  CUdeviceptr va_base = 0;
  size_t va_bytes = 0;
  std::vector<CUmemGenericAllocationHandle> handles;  // [nranks] (VMM)
  CUmemGenericAllocationHandle mc_handle = 0;
  CUdeviceptr mc_va = 0;
  CUdevice cu_device = 0;
  bool owns_local = true;           // false when the local memory belongs to the user (windows)
  std::vector<void*> ipc_opened;    // peers opened through CUDA IPC
};

// Passes file descriptors between the ranks of one communicator.
class FdChannel {
 public:
  FdChannel(const std::string& token, int rank, int nranks);
  ~FdChannel();
  void send_fd(int peer, int fd, uint64_t tag);
  // Blocks until the descriptor tagged (src, tag) arrived; throws after timeout_ms.
  int recv_fd(int src, uint64_t tag, int timeout_ms);

 private:
  std::string address_of(int rank) const;
  std::string token_;
  int rank_, nranks_;
  int sock_ = -1;
  std::map<std::pair<int, uint64_t>, int> stash_;
};

class SymmMemory {
 public:
  SymmMemory(c10::intrusive_ptr<c10d::Store> store, int rank, int nranks, int device_index,
             std::shared_ptr<DriverApi> driver, std::chrono::milliseconds timeout, bool allow_multicast,
             std::shared_ptr<CudaApi> cuda = nullptr);
  ~SymmMemory();

  // Collective over the communicator. Memory is zero-filled.
  std::shared_ptr<SymmSegment> allocate(size_t bytes, bool want_multicast);
  // Collective: makes `local` (size `bytes`, owned by the caller) reachable
  // from every rank. Uses the exportable-allocation registry when the pointer
  // came from the symmetric allocator, CUDA IPC otherwise.
  // With `want_multicast`, memory from the symmetric allocator that every rank
  // passes whole (same size, a multiple of the multicast granularity) is also
  // bound to a multicast object.
  std::shared_ptr<SymmSegment> attach_user_buffer(void* local, size_t bytes, bool want_multicast = false);
  // Local teardown; callers barrier first so that no peer still uses it.
  void release(const std::shared_ptr<SymmSegment>& seg);

  SymmMode mode() const { return mode_; }
  bool multicast_available() const { return mc_ok_; }

 private:
  void decide_mode();
  void barrier(const std::string& what);
  std::vector<std::string> all_gather_bytes(const std::string& key, const std::string& mine);
  void map_vmm(SymmSegment& seg, CUmemGenericAllocationHandle local_handle, uint64_t seq);
  void try_multicast(SymmSegment& seg, uint64_t seq);
  void exchange_ipc(SymmSegment& seg, void* local_base, size_t offset, uint64_t seq);

  c10::intrusive_ptr<c10d::Store> store_;
  int rank_, nranks_, device_;
  std::shared_ptr<DriverApi> drv_;
  std::shared_ptr<CudaApi> cuda_;
  std::chrono::milliseconds timeout_;
  bool allow_mc_;
  SymmMode mode_ = SymmMode::LOCAL;
  bool mc_ok_ = false;
  size_t gran_ = 2u << 20;
  uint64_t seq_ = 0;
  std::unique_ptr<FdChannel> fds_;
  CUdevice cu_dev_ = 0;
};

// Process-wide table of allocations made by the symmetric allocator
// (exported C functions b200c_symm_alloc / b200c_symm_free, plugged into
// PyTorch through CUDAPluggableAllocator). Lets a window find the VMM handle
// behind a tensor's storage.
struct ExportableAlloc {
  CUmemGenericAllocationHandle handle = 0;
  CUdeviceptr base = 0;
  size_t bytes = 0;
  int device = 0;
};

class ExportableRegistry {
 public:
  static ExportableRegistry& get();
  void add(const ExportableAlloc& a);
  bool remove(CUdeviceptr base, ExportableAlloc* out);
  // Finds the allocation containing [ptr, ptr+bytes).
  bool find(const void* ptr, size_t bytes, ExportableAlloc* out) const;
  size_t live() const;

 private:
  mutable std::mutex mu_;
  std::map<CUdeviceptr, ExportableAlloc> allocs_;
};

} // namespace b200c
