// The user-facing communicator object and the backend factory.
//
// Comm validates arguments, hands out process-wide monotonically increasing
// operation ids, runs pre/post hooks around the backend call and keeps the
// member list (global ranks) of the communicator. It is not thread safe: one
// thread issues operations on a given communicator at a time.
//
// Parity: comms/torchcomms/TorchComm.hpp:50-345, TorchComm.cpp:20-107,190-204,
// 548-568,627-675; comms/torchcomms/TorchCommFactory.cpp:25-244;
// comms/torchcomms/TorchCommBatch.hpp:27-61; comms/torchcomms/HealthCheck.hpp.
#pragma once

#include "backend.hpp"

namespace b200c {

class Comm;

// Accumulates point-to-point operations and issues them as one group.
class B200C_API BatchSendRecv {
 public:
  explicit BatchSendRecv(std::shared_ptr<Comm> parent) : parent_(std::move(parent)) {}
  void send(const at::Tensor& t, int dst);
  void recv(at::Tensor& t, int src);
  WorkPtr issue(bool async_op, const OpOptions& o = {});
  std::vector<P2POp> ops;

 private:
  std::shared_ptr<Comm> parent_;
};

// Training iteration the process is in, set by the trainer (`set_trainer_iteration`) and attached to
// flight-recorder entries and communicator dumps so that a trace can be lined up with the step that
// produced it. -1 until set. Parity: the trainer context of comms/utils (iteration tagging).
B200C_API void set_trainer_iteration(int64_t iteration);
B200C_API int64_t trainer_iteration();

// State of every communicator alive in this process, by communicator name
// (comms/torchcomms/ncclx/TorchCommNCCLXPy.cpp:137-184, `comm_dump_all`).
B200C_API std::unordered_map<std::string, std::unordered_map<std::string, std::string>> comm_dump_all();

class B200C_API Comm : public std::enable_shared_from_this<Comm> {
 public:
  Comm(std::shared_ptr<Backend> impl, std::vector<int> global_ranks = {});
  ~Comm();

  void finalize();
  int get_rank() const { return impl_->rank(); }
  int get_size() const { return impl_->size(); }
  std::string get_name() const { return impl_->comm_name(); }
  std::string get_backend() const { return impl_->backend_name(); }
  std::string get_backend_version() const { return impl_->backend_version(); }
  at::Device get_device() const { return impl_->device(); }
  const CommOptions& get_options() const { return impl_->options(); }
  std::shared_ptr<Backend> get_backend_impl() const { return impl_; }
  friend std::unordered_map<std::string, std::unordered_map<std::string, std::string>> comm_dump_all();
  const std::vector<int>& get_ranks() const { return ranks_; }

  WorkPtr send(const at::Tensor& t, int dst, bool async_op, const OpOptions& o = {});
  WorkPtr recv(at::Tensor& t, int src, bool async_op, const OpOptions& o = {});
  WorkPtr broadcast(at::Tensor& t, int root, bool async_op, const OpOptions& o = {});
  WorkPtr all_reduce(at::Tensor& t, const ReduceOp& op, bool async_op, const OpOptions& o = {});
  WorkPtr reduce(const at::Tensor& t, int root, const ReduceOp& op, bool async_op, const OpOptions& o = {});
  WorkPtr all_gather(const std::vector<at::Tensor>& outs, const at::Tensor& in, bool async_op, const OpOptions& o = {});
  WorkPtr all_gather_v(const std::vector<at::Tensor>& outs, const at::Tensor& in, bool async_op, const OpOptions& o = {});
  WorkPtr all_gather_single(at::Tensor& out, const at::Tensor& in, bool async_op, const OpOptions& o = {});
  WorkPtr reduce_scatter(at::Tensor& out, const std::vector<at::Tensor>& ins, const ReduceOp& op, bool async_op, const OpOptions& o = {});
  WorkPtr reduce_scatter_v(at::Tensor& out, const std::vector<at::Tensor>& ins, const ReduceOp& op, bool async_op, const OpOptions& o = {});
  WorkPtr reduce_scatter_single(at::Tensor& out, const at::Tensor& in, const ReduceOp& op, bool async_op, const OpOptions& o = {});
  WorkPtr all_to_all_single(at::Tensor& out, const at::Tensor& in, bool async_op, const OpOptions& o = {});
  WorkPtr all_to_all_v_single(at::Tensor& out, const at::Tensor& in,
                              const std::vector<int64_t>& out_splits,
                              const std::vector<int64_t>& in_splits,
                              bool async_op, const OpOptions& o = {});
  WorkPtr all_to_all(const std::vector<at::Tensor>& outs, const std::vector<at::Tensor>& ins, bool async_op, const OpOptions& o = {});
  WorkPtr barrier(bool async_op, const OpOptions& o = {});
  WorkPtr scatter(at::Tensor& out, const std::vector<at::Tensor>& ins, int root, bool async_op, const OpOptions& o = {});
  WorkPtr gather(const std::vector<at::Tensor>& outs, const at::Tensor& in, int root, bool async_op, const OpOptions& o = {});
  WorkPtr gather_single(at::Tensor& out, const at::Tensor& in, int root, bool async_op, const OpOptions& o = {});

  // Returns null for ranks that pass an empty list.
  std::shared_ptr<Comm> split(const std::vector<int>& ranks, const std::string& name, const CommOptions& opts = {});
  std::shared_ptr<BatchSendRecv> batch_op_create();
  WorkPtr batch_op_issue(const std::vector<P2POp>& ops, bool async_op, const OpOptions& o);
  std::shared_ptr<Window> new_window(const std::optional<at::Tensor>& tensor = std::nullopt);

  std::shared_ptr<AllGatherPHandle> all_gather_p_init(at::Tensor& output, const OpOptions& o = {});
  WorkPtr all_gather_p_exec(const std::shared_ptr<AllGatherPHandle>& h, const at::Tensor& in, bool async_op, const OpOptions& o = {});
  void all_gather_p_free(const std::shared_ptr<AllGatherPHandle>& h);

  InitHandle get_init_handle() const { return impl_->get_init_handle(); }
  WorkPtr reconfigure(const ReconfigureOptions& o);
  void abort() { impl_->abort(); }
  bool is_abort_supported() const { return impl_->is_abort_supported(); }
  bool is_aborted() const { return impl_->is_aborted(); }
  void set_timeout(Millis t) { impl_->set_timeout(t); }
  void set_hints(const Hints& h) { impl_->set_hints(h); }
  void tensor_register(const at::Tensor& t) { impl_->tensor_register(t); }
  void tensor_deregister(const at::Tensor& t) { impl_->tensor_deregister(t); }

  RemovableHandle register_pre_hook(PreHook h) {
    impl_->set_observed();
    return pre_hooks_->add(std::move(h));
  }
  RemovableHandle register_post_hook(PostHook h) {
    impl_->set_observed();
    return post_hooks_->add(std::move(h));
  }
  RemovableHandle register_abort_hook(AbortHook h) { return abort_hooks_->add(std::move(h)); }
  RemovableHandle register_graph_replay_hook(GraphReplayHook h) { return replay_hooks_->add(std::move(h)); }

  // Next process-wide operation id (exposed for tests).
  static size_t next_op_id();
  static constexpr size_t kFinalizeOpId = static_cast<size_t>(-1);

 private:
  void check_rank(int r, const char* what) const;
  template <typename F>
  WorkPtr run_op(OpRecord rec, F&& call);

  std::shared_ptr<Backend> impl_;
  std::vector<int> ranks_;
  std::shared_ptr<HookTable<PreHook>> pre_hooks_ = std::make_shared<HookTable<PreHook>>();
  std::shared_ptr<HookTable<PostHook>> post_hooks_ = std::make_shared<HookTable<PostHook>>();
  std::shared_ptr<HookTable<AbortHook>> abort_hooks_ = std::make_shared<HookTable<AbortHook>>();
  std::shared_ptr<HookTable<GraphReplayHook>> replay_hooks_ = std::make_shared<HookTable<GraphReplayHook>>();
  bool finalized_ = false;
};

// Process-wide registry of backend constructors.
class B200C_API Factory {
 public:
  using Maker = std::function<std::shared_ptr<Backend>()>;
  static Factory& get();

  void register_backend(const std::string& name, Maker maker);
  bool is_registered(const std::string& name) const;
  std::vector<std::string> registered() const;
  // Looks `name` up in the registry; failing that, dlopens the library named
  // by TORCHCOMMS_BACKEND_LIB_PATH_<NAME> (or B200COMMS_BACKEND_LIB_PATH_<NAME>)
  // and checks its ABI string. Calls init() on the result.
  std::shared_ptr<Backend> create(const std::string& name, at::Device device,
                                  const std::string& comm_name, const CommOptions& opts);

 private:
  std::shared_ptr<Backend> load_dynamic(const std::string& name);
  mutable std::mutex mu_;
  std::unordered_map<std::string, Maker> makers_;
};

B200C_API std::shared_ptr<Comm> new_comm(const std::string& backend, at::Device device,
                               const std::string& name, const CommOptions& opts = {});

// Process-wide health flag: flips to unhealthy once any watchdog saw a
// timeout or an asynchronous error.
class B200C_API HealthCheck {
 public:
  static void mark_unhealthy(const std::string& why);
  static bool healthy();
  static std::string reason();
  static void reset(); // tests only
};

} // namespace b200c
