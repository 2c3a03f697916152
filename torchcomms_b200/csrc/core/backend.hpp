// Abstract communication backend and one-sided window.
//
// A backend owns the transport for one communicator. The facade (Comm) does
// argument validation, op-id allocation and hook dispatch, then forwards here.
// Backends shipped in-tree: "b200" (CUDA, peer-memory kernels + NCCL; also
// registered as "nccl" and "ncclx"), "gloo" (CPU) and "fake" (no transport).
//
// Parity: comms/torchcomms/TorchCommBackend.hpp:21,34-459 (ABI "1.3": init /
// finalize / p2p / 14 collectives / split / window / persistent all-gather /
// fault-tolerance entry points) and comms/torchcomms/TorchCommWindow.hpp:14-150.
#pragma once

#include <atomic>
#include <unordered_map>

#include <memory>

#include "hooks.hpp"
#include "options.hpp"

namespace b200c {

constexpr const char* kBackendAbiVersion = "b200c-2";   // 2: CommOptions gained `name`

class Backend;

class B200C_API Window : public std::enable_shared_from_this<Window> {
 public:
  virtual ~Window() = default;

  // Collective: every rank registers a buffer of the same size. `owning`
  // keeps the tensor alive for the lifetime of the registration.
  virtual void tensor_register(const at::Tensor& t, bool owning) = 0;
  virtual void tensor_deregister() = 0;
  virtual std::shared_ptr<Window> clone() = 0;

  virtual WorkPtr put(const at::Tensor& src, int dst_rank, int64_t target_offset_nelems,
                      bool async_op, const OpOptions& o) = 0;
  virtual WorkPtr signal(int dst_rank, bool async_op, const OpOptions& o) = 0;
  virtual WorkPtr wait_signal(int peer_rank, bool async_op, const OpOptions& o) = 0;
  virtual at::Tensor map_remote_tensor(int rank) = 0;
  virtual WindowAttr get_attr(int peer_rank) = 0;

  // Device-side handle: address of a DeviceWindow struct in device memory.
  virtual uintptr_t get_device_window(int signal_count, int counter_count, int barrier_count) = 0;
  virtual uintptr_t register_local_buffer(const at::Tensor& t) = 0;
  virtual void deregister_local_buffer(uintptr_t handle) = 0;

  std::optional<at::Tensor> get_tensor() const { return tensor_; }
  int64_t get_size() const { return tensor_ ? static_cast<int64_t>(tensor_->nbytes()) : 0; }
  // Cached metadata so tracing/compile layers need not touch the tensor.
  at::ScalarType dtype() const { return dtype_; }
  const std::vector<int64_t>& shape() const { return shape_; }
  at::Device device() const { return device_; }

 protected:
  void cache_meta(const at::Tensor& t) {
    dtype_ = t.scalar_type();
    shape_ = t.sizes().vec();
    device_ = t.device();
  }
  std::optional<at::Tensor> tensor_;
  at::ScalarType dtype_ = at::kFloat;
  std::vector<int64_t> shape_;
  at::Device device_{at::kCPU};
};

// Handle for a persistent all-gather (output registered once, executed often).
struct AllGatherPHandle {
  at::Tensor output;
  uint64_t id = 0;
  bool freed = false;
};

class B200C_API Backend : public std::enable_shared_from_this<Backend> {
 public:
  virtual ~Backend() = default;

  virtual void init(at::Device device, const std::string& name, const CommOptions& opts) = 0;
  virtual void finalize() = 0;
  virtual int rank() const = 0;
  virtual int size() const = 0;
  virtual std::string backend_name() const = 0;
  virtual std::string backend_version() const { return kBackendAbiVersion; }
  virtual std::string comm_name() const = 0;
  virtual at::Device device() const = 0;
  virtual const CommOptions& options() const = 0;

  // Internal state as a string map, for `comm_dump()` / `comm_dump_all()`
  // (comms/torchcomms/ncclx/TorchCommNCCLXPy.cpp:59-184). Backends add their own keys.
  virtual std::unordered_map<std::string, std::string> comm_dump() const {
    return {{"name", comm_name()}, {"backend", backend_name()}, {"rank", std::to_string(rank())}, {"size", std::to_string(size())}};
  }

  // Point to point.
  virtual WorkPtr send(const at::Tensor& t, int dst, bool async_op, const OpOptions& o) = 0;
  virtual WorkPtr recv(at::Tensor& t, int src, bool async_op, const OpOptions& o) = 0;
  virtual WorkPtr batch_op_issue(const std::vector<P2POp>& ops, bool async_op, const OpOptions& o) = 0;

  // Collectives.
  virtual WorkPtr broadcast(at::Tensor& t, int root, bool async_op, const OpOptions& o) = 0;
  virtual WorkPtr all_reduce(at::Tensor& t, const ReduceOp& op, bool async_op, const OpOptions& o) = 0;
  virtual WorkPtr reduce(const at::Tensor& t, int root, const ReduceOp& op, bool async_op, const OpOptions& o) = 0;
  virtual WorkPtr all_gather(const std::vector<at::Tensor>& outs, const at::Tensor& in, bool async_op, const OpOptions& o) = 0;
  virtual WorkPtr all_gather_v(const std::vector<at::Tensor>& outs, const at::Tensor& in, bool async_op, const OpOptions& o) = 0;
  virtual WorkPtr all_gather_single(at::Tensor& out, const at::Tensor& in, bool async_op, const OpOptions& o) = 0;
  virtual WorkPtr reduce_scatter(at::Tensor& out, const std::vector<at::Tensor>& ins, const ReduceOp& op, bool async_op, const OpOptions& o) = 0;
  virtual WorkPtr reduce_scatter_v(at::Tensor& out, const std::vector<at::Tensor>& ins, const ReduceOp& op, bool async_op, const OpOptions& o) = 0;
  virtual WorkPtr reduce_scatter_single(at::Tensor& out, const at::Tensor& in, const ReduceOp& op, bool async_op, const OpOptions& o) = 0;
  virtual WorkPtr all_to_all_single(at::Tensor& out, const at::Tensor& in, bool async_op, const OpOptions& o) = 0;
  virtual WorkPtr all_to_all_v_single(at::Tensor& out, const at::Tensor& in,
                                      const std::vector<int64_t>& out_splits,
                                      const std::vector<int64_t>& in_splits,
                                      bool async_op, const OpOptions& o) = 0;
  virtual WorkPtr all_to_all(const std::vector<at::Tensor>& outs, const std::vector<at::Tensor>& ins, bool async_op, const OpOptions& o) = 0;
  virtual WorkPtr barrier(bool async_op, const OpOptions& o) = 0;
  virtual WorkPtr scatter(at::Tensor& out, const std::vector<at::Tensor>& ins, int root, bool async_op, const OpOptions& o) = 0;
  virtual WorkPtr gather(const std::vector<at::Tensor>& outs, const at::Tensor& in, int root, bool async_op, const OpOptions& o) = 0;
  // Default: view `out` as size() chunks on the root and call gather().
  virtual WorkPtr gather_single(at::Tensor& out, const at::Tensor& in, int root, bool async_op, const OpOptions& o);

  // Sub-communicator over `ranks` (parent-local ranks). Non-members get null.
  virtual std::shared_ptr<Backend> split(const std::vector<int>& ranks, const std::string& name, const CommOptions& opts) = 0;

  // One-sided windows.
  virtual std::shared_ptr<Window> new_window(const std::optional<at::Tensor>& tensor);

  // Persistent all-gather.
  virtual std::shared_ptr<AllGatherPHandle> all_gather_p_init(at::Tensor& output, const OpOptions& o);
  virtual WorkPtr all_gather_p_exec(const std::shared_ptr<AllGatherPHandle>& h, const at::Tensor& in, bool async_op, const OpOptions& o);
  virtual void all_gather_p_free(const std::shared_ptr<AllGatherPHandle>& h);

  // Fault tolerance / elasticity.
  virtual bool supports_reconfigure() const { return false; }
  virtual InitHandle get_init_handle() const;
  virtual WorkPtr reconfigure(const ReconfigureOptions& o);
  virtual void abort() {}
  virtual bool is_aborted() const { return false; }
  virtual bool is_abort_supported() const { return false; }

  virtual void set_timeout(Millis t) = 0;
  virtual void set_hints(const Hints& h) { (void)h; }

  // Two-rank communicator with `peer` (a rank of this communicator), created
  // by those two ranks alone: bootstrapped through the store under a prefix
  // built from `name`, never through a collective on this communicator. The
  // lower rank is rank 0 of the pair. Used by the "-lazy" backends.
  virtual std::shared_ptr<Backend> create_pair_comm(int peer, const std::string& name);

  // Registers user memory for zero-copy collectives.
  virtual void tensor_register(const at::Tensor& t) { (void)t; }
  virtual void tensor_deregister(const at::Tensor& t) { (void)t; }

  // Called by the facade once somebody registers a pre- or post-hook: from
  // then on every operation's work must report its start and end (recorders
  // follow operations through work hooks), so backends may no longer hand out
  // works that skip the bookkeeping.
  void set_observed() { observed_.store(true, std::memory_order_relaxed); }
  bool observed() const { return observed_.load(std::memory_order_relaxed); }

  // Observer tables owned by the facade and shared with the backend so the
  // watchdog can fire them.
  virtual void attach_hook_tables(std::shared_ptr<HookTable<AbortHook>> abort_hooks,
                                  std::shared_ptr<HookTable<GraphReplayHook>> replay_hooks) {
    abort_hooks_ = std::move(abort_hooks);
    replay_hooks_ = std::move(replay_hooks);
  }

 protected:
  void run_abort_hooks() const;
  std::shared_ptr<HookTable<AbortHook>> abort_hooks_;
  std::shared_ptr<HookTable<GraphReplayHook>> replay_hooks_;
  std::atomic<bool> observed_{false};
};

// Exported by out-of-tree backends that are loaded with dlopen: the symbol
// `b200c_create_backend_<name>` returns a pointer to one of these.
struct DynamicBackendLoader {
  const char* (*abi_version)();
  Backend* (*create)();
  void (*destroy)(Backend*);
};

} // namespace b200c
