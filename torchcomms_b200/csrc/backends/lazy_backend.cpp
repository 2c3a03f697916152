// "<backend>-lazy": collectives on the primary communicator, send / recv on
// two-rank communicators created on first use for each peer.
//
// A pair communicator has its own stream (CUDA) or its own connection pair
// (gloo), so point-to-point traffic to different peers overlaps with itself
// and with collectives on the primary - what a pipeline schedule wants.
// Creation involves only the two ranks of the pair: it bootstraps through a
// store prefix derived from the pair, not through a collective split.
// batch_op_issue stays on the primary because one batch may touch several
// peers.
//
// Parity: comms/torchcomms/lazy/LazyBackend.hpp:27-617 and
// nccl/TorchCommNCCLLazy.cpp:34-129 ("nccl-lazy").
#include <mutex>
#include <unordered_map>

#include "../core/comm.hpp"
#include "../core/logging.hpp"

namespace b200c {

namespace {

class LazyBackend final : public Backend {
 public:
  LazyBackend(std::string primary_name, std::string registered_as)
      : primary_name_(std::move(primary_name)), registered_as_(std::move(registered_as)) {}

  void init(at::Device device, const std::string& name, const CommOptions& opts) override {
    primary_ = Factory::get().create(primary_name_, device, name, opts);
  }
  void attach_hook_tables(std::shared_ptr<HookTable<AbortHook>> abort_hooks,
                          std::shared_ptr<HookTable<GraphReplayHook>> replay_hooks) override {
    Backend::attach_hook_tables(abort_hooks, replay_hooks);
    primary_->attach_hook_tables(abort_hooks, replay_hooks);
    for (auto& b : snapshot()) b->attach_hook_tables(abort_hooks, replay_hooks);
  }
  void finalize() override {
    std::unordered_map<int, std::shared_ptr<Backend>> pairs;
    {
      std::lock_guard<std::mutex> g(mu_);
      pairs.swap(pairs_);
    }
    for (auto& kv : pairs) kv.second->finalize();  // pairs first, then the primary
    primary_->finalize();
  }
  int rank() const override { return primary_->rank(); }
  int size() const override { return primary_->size(); }
  std::string backend_name() const override { return registered_as_; }
  std::string backend_version() const override { return primary_->backend_version(); }
  std::string comm_name() const override { return primary_->comm_name(); }
  at::Device device() const override { return primary_->device(); }
  const CommOptions& options() const override { return primary_->options(); }

  WorkPtr send(const at::Tensor& t, int dst, bool async_op, const OpOptions& o) override {
    if (dst == rank()) return primary_->send(t, dst, async_op, o);
    return channel_for(dst)->send(t, local_rank_of_peer(dst), async_op, o);
  }
  WorkPtr recv(at::Tensor& t, int src, bool async_op, const OpOptions& o) override {
    if (src == rank()) return primary_->recv(t, src, async_op, o);
    return channel_for(src)->recv(t, local_rank_of_peer(src), async_op, o);
  }
  WorkPtr batch_op_issue(const std::vector<P2POp>& ops, bool async_op, const OpOptions& o) override {
    return primary_->batch_op_issue(ops, async_op, o);
  }

  WorkPtr broadcast(at::Tensor& t, int root, bool a, const OpOptions& o) override { return primary_->broadcast(t, root, a, o); }
  WorkPtr all_reduce(at::Tensor& t, const ReduceOp& op, bool a, const OpOptions& o) override { return primary_->all_reduce(t, op, a, o); }
  WorkPtr reduce(const at::Tensor& t, int root, const ReduceOp& op, bool a, const OpOptions& o) override {
    return primary_->reduce(t, root, op, a, o);
  }
  WorkPtr all_gather(const std::vector<at::Tensor>& outs, const at::Tensor& in, bool a, const OpOptions& o) override {
    return primary_->all_gather(outs, in, a, o);
  }
  WorkPtr all_gather_v(const std::vector<at::Tensor>& outs, const at::Tensor& in, bool a, const OpOptions& o) override {
    return primary_->all_gather_v(outs, in, a, o);
  }
  WorkPtr all_gather_single(at::Tensor& out, const at::Tensor& in, bool a, const OpOptions& o) override {
    return primary_->all_gather_single(out, in, a, o);
  }
  WorkPtr reduce_scatter(at::Tensor& out, const std::vector<at::Tensor>& ins, const ReduceOp& op, bool a, const OpOptions& o) override {
    return primary_->reduce_scatter(out, ins, op, a, o);
  }
  WorkPtr reduce_scatter_v(at::Tensor& out, const std::vector<at::Tensor>& ins, const ReduceOp& op, bool a, const OpOptions& o) override {
    return primary_->reduce_scatter_v(out, ins, op, a, o);
  }
  WorkPtr reduce_scatter_single(at::Tensor& out, const at::Tensor& in, const ReduceOp& op, bool a, const OpOptions& o) override {
    return primary_->reduce_scatter_single(out, in, op, a, o);
  }
  WorkPtr all_to_all_single(at::Tensor& out, const at::Tensor& in, bool a, const OpOptions& o) override {
    return primary_->all_to_all_single(out, in, a, o);
  }
  WorkPtr all_to_all_v_single(at::Tensor& out, const at::Tensor& in, const std::vector<int64_t>& os,
                              const std::vector<int64_t>& is, bool a, const OpOptions& o) override {
    return primary_->all_to_all_v_single(out, in, os, is, a, o);
  }
  WorkPtr all_to_all(const std::vector<at::Tensor>& outs, const std::vector<at::Tensor>& ins, bool a, const OpOptions& o) override {
    return primary_->all_to_all(outs, ins, a, o);
  }
  WorkPtr barrier(bool a, const OpOptions& o) override { return primary_->barrier(a, o); }
  WorkPtr scatter(at::Tensor& out, const std::vector<at::Tensor>& ins, int root, bool a, const OpOptions& o) override {
    return primary_->scatter(out, ins, root, a, o);
  }
  WorkPtr gather(const std::vector<at::Tensor>& outs, const at::Tensor& in, int root, bool a, const OpOptions& o) override {
    return primary_->gather(outs, in, root, a, o);
  }
  WorkPtr gather_single(at::Tensor& out, const at::Tensor& in, int root, bool a, const OpOptions& o) override {
    return primary_->gather_single(out, in, root, a, o);
  }

  std::shared_ptr<Backend> split(const std::vector<int>& ranks, const std::string& name, const CommOptions& opts) override {
    auto sub = primary_->split(ranks, name, opts);
    if (!sub) return nullptr;
    auto lazy = std::make_shared<LazyBackend>(primary_name_, registered_as_);
    lazy->primary_ = std::move(sub);
    return lazy;
  }
  std::shared_ptr<Window> new_window(const std::optional<at::Tensor>& t) override { return primary_->new_window(t); }
  std::shared_ptr<AllGatherPHandle> all_gather_p_init(at::Tensor& out, const OpOptions& o) override {
    return primary_->all_gather_p_init(out, o);
  }
  WorkPtr all_gather_p_exec(const std::shared_ptr<AllGatherPHandle>& h, const at::Tensor& in, bool a, const OpOptions& o) override {
    return primary_->all_gather_p_exec(h, in, a, o);
  }
  void all_gather_p_free(const std::shared_ptr<AllGatherPHandle>& h) override { primary_->all_gather_p_free(h); }

  bool supports_reconfigure() const override { return false; }  // a pair's membership cannot follow a new world
  void abort() override {
    for (auto& b : snapshot()) b->abort();
    primary_->abort();
  }
  bool is_aborted() const override { return primary_->is_aborted(); }
  bool is_abort_supported() const override { return primary_->is_abort_supported(); }
  void set_timeout(Millis t) override {
    primary_->set_timeout(t);
    for (auto& b : snapshot()) b->set_timeout(t);
  }
  void set_hints(const Hints& h) override {
    primary_->set_hints(h);
    for (auto& b : snapshot()) b->set_hints(h);
  }
  void tensor_register(const at::Tensor& t) override { primary_->tensor_register(t); }
  void tensor_deregister(const at::Tensor& t) override { primary_->tensor_deregister(t); }

  int pair_count() const {
    std::lock_guard<std::mutex> g(mu_);
    return static_cast<int>(pairs_.size());
  }
  std::shared_ptr<Backend> primary() const { return primary_; }

 private:
  // Inside a pair the lower global rank is 0 and the higher is 1.
  int local_rank_of_peer(int peer) const { return rank() < peer ? 1 : 0; }

  std::vector<std::shared_ptr<Backend>> snapshot() const {
    std::lock_guard<std::mutex> g(mu_);
    std::vector<std::shared_ptr<Backend>> v;
    for (auto& kv : pairs_) v.push_back(kv.second);
    return v;
  }

  std::shared_ptr<Backend> channel_for(int peer) {
    TORCH_CHECK(peer >= 0 && peer < size(), "peer rank ", peer, " is outside [0, ", size(), ")");
    {
      std::lock_guard<std::mutex> g(mu_);
      auto it = pairs_.find(peer);
      if (it != pairs_.end()) return it->second;
    }
    // Bootstrap outside the lock: abort() from a watchdog must not wait for it.
    const int lo = std::min(rank(), peer), hi = std::max(rank(), peer);
    auto made = primary_->create_pair_comm(peer, "pair_" + std::to_string(lo) + "_" + std::to_string(hi));
    made->attach_hook_tables(abort_hooks_, replay_hooks_);
    std::lock_guard<std::mutex> g(mu_);
    auto [it, inserted] = pairs_.emplace(peer, made);
    (void)inserted;
    return it->second;
  }

  std::string primary_name_, registered_as_;
  std::shared_ptr<Backend> primary_;
  mutable std::mutex mu_;
  std::unordered_map<int, std::shared_ptr<Backend>> pairs_;
};

} // namespace

void register_lazy_backends() {
  for (const char* base : {"b200", "nccl", "ncclx", "gloo", "fake"}) {
    const std::string b = base, n = b + "-lazy";
    Factory::get().register_backend(n, [b, n] { return std::make_shared<LazyBackend>(b, n); });
  }
}

int lazy_pair_count(const std::shared_ptr<Backend>& b) {
  auto l = std::dynamic_pointer_cast<LazyBackend>(b);
  return l ? l->pair_count() : -1;
}

std::shared_ptr<Backend> lazy_primary(const std::shared_ptr<Backend>& b) {
  auto l = std::dynamic_pointer_cast<LazyBackend>(b);
  return l ? l->primary() : nullptr;
}

} // namespace b200c
