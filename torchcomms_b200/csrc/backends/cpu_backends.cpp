// "fake" and "gloo" backends.
#include "cpu_backends.hpp"

#include <cstdio>
#include <mutex>
#include <thread>
#include <unistd.h>

#include <random>

#include "../core/logging.hpp"

namespace b200c {

// ----------------------------------------------------------------- fake ----

void FakeBackend::init(at::Device device, const std::string& name, const CommOptions& opts) {
  device_ = device;
  name_ = name;
  opts_ = opts;
  rank_ = hint_or<int>(opts.hints, "fake_rank", 0);
  size_ = hint_or<int>(opts.hints, "fake_size", 1);
  TORCH_CHECK(size_ >= 1 && rank_ >= 0 && rank_ < size_, "fake backend: bad rank/size hints");
  initialized_ = true;
  calls.push_back("init");
}

void FakeBackend::finalize() {
  TORCH_CHECK(initialized_, "fake backend: finalize before init or twice");
  initialized_ = false;
  calls.push_back("finalize");
}

namespace {

// One-sided window of the fake backend: the registered tensor is host memory of the only rank, `put`
// to oneself is a copy, signals are counters. It follows the rules of the real windows (one
// registration at a time, contiguous tensors, `put` inside the registered range, matching dtype).
class FakeWindow final : public Window {
 public:
  FakeWindow(int rank, int size) : rank_(rank), size_(size), pending_(static_cast<size_t>(size), 0) {}

  void tensor_register(const at::Tensor& t, bool /*owning*/) override {
    TORCH_CHECK(!tensor_, "window already has a registered tensor");
    TORCH_CHECK(t.defined() && t.is_contiguous(), "window tensors must be contiguous");
    tensor_ = t;
    cache_meta(t);
  }
  void tensor_deregister() override {
    TORCH_CHECK(tensor_.has_value(), "no tensor is registered with this window");
    tensor_.reset();
  }
  std::shared_ptr<Window> clone() override {
    auto w = std::make_shared<FakeWindow>(rank_, size_);
    if (tensor_) {
      w->tensor_register(tensor_->clone(), true);
    }
    return w;
  }
  WorkPtr put(const at::Tensor& src, int dst_rank, int64_t target_offset_nelems, bool, const OpOptions&) override {
    TORCH_CHECK(tensor_.has_value(), "put: no tensor is registered with this window");
    check_rank(dst_rank, "put");
    TORCH_CHECK(src.is_contiguous(), "put: the source must be contiguous");
    TORCH_CHECK(src.scalar_type() == tensor_->scalar_type(), "put: dtype differs from the window's");
    TORCH_CHECK(target_offset_nelems >= 0 &&
                    (src.numel() + target_offset_nelems) * static_cast<int64_t>(src.element_size()) <=
                        static_cast<int64_t>(tensor_->nbytes()),
                "put: the range lies outside the window");
    tensor_->view({-1}).narrow(0, target_offset_nelems, src.numel()).copy_(src.reshape({-1}));
    return c10::make_intrusive<CompletedWork>();
  }
  WorkPtr signal(int dst_rank, bool, const OpOptions&) override {
    check_rank(dst_rank, "signal");
    ++pending_[static_cast<size_t>(dst_rank)];
    return c10::make_intrusive<CompletedWork>();
  }
  WorkPtr wait_signal(int peer_rank, bool, const OpOptions&) override {
    check_rank(peer_rank, "wait_signal");
    TORCH_CHECK(pending_[static_cast<size_t>(peer_rank)] > 0, "wait_signal: no signal from rank ", peer_rank,
                " is pending (this would wait forever)");
    --pending_[static_cast<size_t>(peer_rank)];
    return c10::make_intrusive<CompletedWork>();
  }
  at::Tensor map_remote_tensor(int rank) override {
    check_rank(rank, "map_remote_tensor");
    TORCH_CHECK(tensor_.has_value(), "map_remote_tensor: no tensor is registered with this window");
    return *tensor_;
  }
  WindowAttr get_attr(int peer_rank) override {
    check_rank(peer_rank, "get_attr");
    return WindowAttr{};
  }
  uintptr_t get_device_window(int, int, int) override { TORCH_CHECK(false, "device windows need the CUDA backend"); }
  uintptr_t register_local_buffer(const at::Tensor&) override { TORCH_CHECK(false, "device windows need the CUDA backend"); }
  void deregister_local_buffer(uintptr_t) override { TORCH_CHECK(false, "device windows need the CUDA backend"); }

 private:
  void check_rank(int r, const char* what) const {
    TORCH_CHECK(r >= 0 && r < size_, what, ": rank ", r, " is outside [0, ", size_, ")");
  }
  int rank_, size_;
  std::vector<int> pending_;
};

}  // namespace

std::shared_ptr<Window> FakeBackend::new_window(const std::optional<at::Tensor>& tensor) {
  calls.push_back("new_window");
  auto w = std::make_shared<FakeWindow>(rank_, size_);
  if (tensor) {
    w->tensor_register(*tensor, true);
  }
  return w;
}

WorkPtr FakeBackend::done(const char* what) {
  TORCH_CHECK(initialized_, "fake backend: used after finalize");
  calls.emplace_back(what);
  return c10::make_intrusive<CompletedWork>();
}

WorkPtr FakeBackend::all_gather(const std::vector<at::Tensor>& outs, const at::Tensor& in, bool, const OpOptions&) {
  for (auto& o : outs) {
    if (o.numel() == in.numel()) {
      o.view_as(in).copy_(in);
    }
  }
  return done("all_gather");
}

WorkPtr FakeBackend::all_gather_single(at::Tensor& out, const at::Tensor& in, bool, const OpOptions&) {
  TORCH_CHECK(out.numel() == in.numel() * size_, "all_gather_single: output numel must be input numel * size");
  auto flat = out.view({size_, -1});
  for (int r = 0; r < size_; ++r) {
    flat[r].copy_(in.reshape({-1}));
  }
  return done("all_gather_single");
}

WorkPtr FakeBackend::reduce_scatter(at::Tensor& out, const std::vector<at::Tensor>& ins, const ReduceOp&, bool, const OpOptions&) {
  TORCH_CHECK(static_cast<int>(ins.size()) == size_, "reduce_scatter: need size() inputs");
  out.copy_(ins[rank_].view_as(out));
  return done("reduce_scatter");
}

WorkPtr FakeBackend::reduce_scatter_single(at::Tensor& out, const at::Tensor& in, const ReduceOp&, bool, const OpOptions&) {
  TORCH_CHECK(in.numel() == out.numel() * size_, "reduce_scatter_single: input numel must be output numel * size");
  out.copy_(in.view({size_, -1})[rank_].view_as(out));
  return done("reduce_scatter_single");
}

WorkPtr FakeBackend::all_to_all_single(at::Tensor& out, const at::Tensor& in, bool, const OpOptions&) {
  TORCH_CHECK(out.numel() == in.numel(), "all_to_all_single: numel mismatch");
  out.copy_(in.view_as(out));
  return done("all_to_all_single");
}

WorkPtr FakeBackend::all_to_all_v_single(at::Tensor& out, const at::Tensor& in, const std::vector<int64_t>&, const std::vector<int64_t>&, bool, const OpOptions&) {
  if (out.numel() == in.numel()) {
    out.copy_(in.view_as(out));
  }
  return done("all_to_all_v_single");
}

WorkPtr FakeBackend::all_to_all(const std::vector<at::Tensor>& outs, const std::vector<at::Tensor>& ins, bool, const OpOptions&) {
  for (size_t i = 0; i < outs.size() && i < ins.size(); ++i) {
    if (outs[i].numel() == ins[i].numel()) {
      outs[i].copy_(ins[i].view_as(outs[i]));
    }
  }
  return done("all_to_all");
}

WorkPtr FakeBackend::scatter(at::Tensor& out, const std::vector<at::Tensor>& ins, int root, bool, const OpOptions&) {
  if (rank_ == root && static_cast<int>(ins.size()) == size_) {
    out.copy_(ins[rank_].view_as(out));
  }
  return done("scatter");
}

WorkPtr FakeBackend::gather(const std::vector<at::Tensor>& outs, const at::Tensor& in, int root, bool, const OpOptions&) {
  if (rank_ == root) {
    for (auto& o : outs) {
      if (o.numel() == in.numel()) {
        o.copy_(in.view_as(o));
      }
    }
  }
  return done("gather");
}

std::shared_ptr<Backend> FakeBackend::split(const std::vector<int>& ranks, const std::string& name, const CommOptions& opts) {
  calls.push_back("split");
  if (ranks.empty()) {
    return nullptr;
  }
  auto child = std::make_shared<FakeBackend>();
  CommOptions o = opts;
  int idx = 0;
  for (size_t i = 0; i < ranks.size(); ++i) {
    if (ranks[i] == rank_) {
      idx = static_cast<int>(i);
    }
  }
  o.hints["fake_rank"] = std::to_string(idx);
  o.hints["fake_size"] = std::to_string(ranks.size());
  child->init(device_, name, o);
  return child;
}

WorkPtr FakeBackend::reconfigure(const ReconfigureOptions& o) {
  calls.push_back("reconfigure");
  size_ = std::max<int>(1, static_cast<int>(o.handles.size()));
  rank_ = 0;
  for (size_t i = 0; i < o.handles.size(); ++i) {
    if (o.handles[i] == get_init_handle()) {
      rank_ = static_cast<int>(i);
    }
  }
  aborted_ = false;
  initialized_ = true;
  return c10::make_intrusive<CompletedWork>();
}

// ----------------------------------------------------------------- gloo ----

namespace {

GlooPgMaker& pg_maker() {
  static GlooPgMaker m;
  return m;
}

c10d::ReduceOp to_c10d(const ReduceOp& op, at::ScalarType dtype) {
  switch (op.type()) {
    case RedOpType::SUM:
    case RedOpType::AVG:
    case RedOpType::PREMUL_SUM:
      return c10d::ReduceOp::SUM;
    case RedOpType::PRODUCT: return c10d::ReduceOp::PRODUCT;
    case RedOpType::MIN: return c10d::ReduceOp::MIN;
    case RedOpType::MAX: return c10d::ReduceOp::MAX;
    case RedOpType::BAND:
    case RedOpType::BOR:
    case RedOpType::BXOR:
      TORCH_CHECK(c10::isIntegralType(dtype, /*includeBool=*/true),
                  "bitwise reductions need an integral tensor, got ", dtype);
      return op.type() == RedOpType::BAND ? c10d::ReduceOp::BAND
          : op.type() == RedOpType::BOR  ? c10d::ReduceOp::BOR
                                         : c10d::ReduceOp::BXOR;
  }
  return c10d::ReduceOp::SUM;
}

void check_contig(const at::Tensor& t, const char* what) {
  TORCH_CHECK(t.defined(), what, ": undefined tensor");
  TORCH_CHECK(t.is_contiguous(), "Tensor must be contiguous for ", what);
}

// Host image of a tensor: the tensor itself on CPU, a copy for device tensors.
at::Tensor host_of(const at::Tensor& t) {
  return t.device().is_cpu() ? t : t.to(at::kCPU);
}

void premultiply(at::Tensor& host, const ReduceOp& op) {
  if (op.type() == RedOpType::PREMUL_SUM) {
    host.mul_(op.factor_as_double());
  }
}

void postdivide(at::Tensor& host, const ReduceOp& op, int n) {
  if (op.type() == RedOpType::AVG) {
    if (c10::isFloatingType(host.scalar_type())) {
      host.div_(n);
    } else {
      host.div_(n, "trunc");
    }
  }
}

} // namespace

void set_gloo_pg_maker(GlooPgMaker maker) {
  pg_maker() = std::move(maker);
}

class GlooWork final : public Work {
 public:
  GlooWork(std::vector<c10::intrusive_ptr<c10d::Work>> inner, std::function<void()> post,
           Millis timeout, std::weak_ptr<Backend> owner)
      : inner_(std::move(inner)), post_(std::move(post)), owner_(std::move(owner)) {
    set_timeout(timeout);
    set_status(WorkStatus::INPROGRESS);
  }

  // A caller may drop the work of an asynchronous operation without waiting. Collectives run to
  // completion on the process group's own threads, but a point-to-point transfer is cancelled when
  // its handle goes away, which would leave the peer waiting forever: hand unfinished transfers (and
  // the copy-back that follows them) to a helper thread that sees them through.
  ~GlooWork() override {
    std::vector<c10::intrusive_ptr<c10d::Work>> inner;
    std::function<void()> post;
    {
      std::lock_guard<std::mutex> g(wait_mu_);
      if (done_) {
        return;
      }
      done_ = true;
      inner.swap(inner_);
      post.swap(post_);
    }
    if (inner.empty()) {
      return;
    }
    std::thread([inner = std::move(inner), post = std::move(post)]() mutable {
      try {
        for (auto& w : inner) {
          if (w) w->wait();
        }
        at::NoGradGuard no_grad;   // the copy-back writes into the caller's tensors: never part of an autograd graph
        if (post) post();
      } catch (...) {
        // nobody is left to report to; the peer sees its own timeout
      }
    }).detach();
  }

 protected:
  void do_wait() override {
    // Several threads may wait on one work (the caller, and the thread that completes the
    // c10d future of the same operation): the first one waits, the others wait for it.
    std::lock_guard<std::mutex> g(wait_mu_);
    if (done_) {
      return;
    }
    done_ = true;
    try {
      for (auto& w : inner_) {
        if (w) {
          const Millis t = timeout();
          w->wait(t == kNoTimeout ? ::kNoTimeout : t);
        }
      }
      if (post_) {
        // The copy-back / scaling writes into the caller's output in place. wait() may be called where gradient
        // recording is on and the output already belongs to a graph (result of a traceable operator): the write
        // is the operation's own completion, not a step of the user's computation.
        at::NoGradGuard no_grad;
        post_();
      }
      set_status(WorkStatus::COMPLETED);
    } catch (const std::exception& e) {
      const std::string msg = e.what();
      const bool timed_out = msg.find("imed out") != std::string::npos ||
          msg.find("imeout") != std::string::npos;
      set_error(msg);
      set_status(timed_out ? WorkStatus::TIMEDOUT : WorkStatus::ERROR);
      if (auto owner = owner_.lock()) {
        static_cast<GlooBackend*>(owner.get())->on_failure(msg, timed_out);
      }
    }
    inner_.clear();
    post_ = nullptr;
  }

 private:
  std::vector<c10::intrusive_ptr<c10d::Work>> inner_;
  std::function<void()> post_;
  std::weak_ptr<Backend> owner_;
  std::mutex wait_mu_;
  bool done_ = false;
};

// A gloo process group whose collective is stuck on a dead or absent peer
// cannot be cancelled, and its destructor waits for that collective. After a
// failure or an abort the group is therefore parked here and never destroyed:
// its threads and sockets live until the process ends, and nothing waits for
// them.
static void retire_process_group(c10::intrusive_ptr<c10d::Backend>& pg) {
  static auto* parked = new std::vector<c10::intrusive_ptr<c10d::Backend>>();
  static std::mutex mu;
  if (pg) {
    std::lock_guard<std::mutex> g(mu);
    parked->push_back(std::move(pg));
  }
  pg.reset();
}

GlooBackend::~GlooBackend() {
  if (pg_ && !finalized_) {
    B200C_LOG(WARN, name_, "gloo communicator destroyed without finalize()");
  }
}

void GlooBackend::connect(const c10::intrusive_ptr<c10d::Store>& store, int rank, int size) {
  TORCH_CHECK(pg_maker(), "gloo backend: process-group maker was not installed (import torchcomms_b200 first)");
  rank_ = rank;
  size_ = size;
  pg_ = pg_maker()(store, rank, size, opts_.timeout);
  TORCH_CHECK(pg_, "gloo backend: could not create the process group");
  // The mesh is connected once every rank is through a first barrier.
  c10d::BarrierOptions bo;
  bo.timeout = opts_.timeout;
  pg_->barrier(bo)->wait(opts_.timeout);
}

void GlooBackend::init(at::Device device, const std::string& name, const CommOptions& opts) {
  device_ = device;
  name_ = name;
  opts_ = opts;
  std::random_device rd;
  char host[256] = {0};
  gethostname(host, sizeof(host) - 1);
  // "<launcher rank>:<unique id>:<host>:<pid>" behind the backend name, the layout of the reference's
  // handles (comms/torchcomms/ncclx/TorchCommNCCLXReconfigure.cpp:176-205: "ncclx:<rank>:<uuid>:<host:port>").
  int launcher_rank = -1;
  try {
    launcher_rank = query_ranksize().first;
  } catch (const std::exception&) {
  }
  char uid[32];
  std::snprintf(uid, sizeof(uid), "%08x%08x", static_cast<unsigned>(rd()), static_cast<unsigned>(rd()));
  handle_token_ = std::to_string(launcher_rank) + ":" + uid + "." + name + ":" + std::string(host) + ":" + std::to_string(getpid());
  if (opts.enable_reconfigure) {
    TORCH_CHECK(opts.store, "enable_reconfigure needs a store shared by all candidate ranks");
    store_ = opts.store;
    return; // membership arrives with reconfigure()
  }
  auto [rank, size] = query_ranksize();
  store_ = opts.store ? scoped_store(opts.store, "b200c/gloo/" + name)
                      : create_prefix_store("b200c/gloo/" + name, rank, size, opts.timeout);
  connect(store_, rank, size);
}

void GlooBackend::ensure_ready() const {
  TORCH_CHECK(!finalized_, "gloo communicator '", name_, "' was finalized");
  TORCH_CHECK(!aborted_, "gloo communicator '", name_, "' was aborted");
  TORCH_CHECK(pg_, "gloo communicator '", name_, "' is not initialised (reconfigure() pending?)");
}

void GlooBackend::finalize() {
  TORCH_CHECK(!finalized_, "gloo communicator '", name_, "' was already finalized");
  finalized_ = true;
  pg_.reset();
  store_.reset();
}

void GlooBackend::on_failure(const std::string& what, bool timed_out) {
  HealthCheck::mark_unhealthy(name_ + ": " + what);
  B200C_LOG(ERROR, name_, (timed_out ? "operation timed out: " : "operation failed: ") << what);
  if (opts_.abort_process_on_timeout_or_error) {
    run_abort_hooks();
    B200C_LOG(ERROR, name_, "aborting the process (abort_process_on_timeout_or_error is set)");
    std::abort();
  }
  aborted_ = true;
  retire_process_group(pg_);
}

void GlooBackend::abort() {
  aborted_ = true;
  if (pg_) {
    pg_->abort();
  }
  retire_process_group(pg_);
  run_abort_hooks();
}

WorkPtr GlooBackend::finish(c10::intrusive_ptr<c10d::Work> inner, std::function<void()> post,
                            bool async_op, const OpOptions& o) {
  std::vector<c10::intrusive_ptr<c10d::Work>> v;
  v.push_back(std::move(inner));
  auto w = c10::make_intrusive<GlooWork>(std::move(v), std::move(post), effective_timeout(o), weak_from_this());
  if (!async_op) {
    w->wait();
  }
  return w;
}

WorkPtr GlooBackend::send(const at::Tensor& t, int dst, bool async_op, const OpOptions& o) {
  ensure_ready();
  check_contig(t, "send");
  std::vector<at::Tensor> v{host_of(t)};
  auto inner = pg_->send(v, dst, 0);
  return finish(inner, nullptr, async_op, o);
}

WorkPtr GlooBackend::recv(at::Tensor& t, int src, bool async_op, const OpOptions& o) {
  ensure_ready();
  check_contig(t, "recv");
  at::Tensor host = t.device().is_cpu() ? t : at::empty_like(t, t.options().device(at::kCPU));
  std::vector<at::Tensor> v{host};
  auto inner = pg_->recv(v, src, 0);
  at::Tensor dst = t;
  return finish(inner, [host, dst]() mutable {
    if (!dst.device().is_cpu()) {
      dst.copy_(host);
    }
  }, async_op, o);
}

WorkPtr GlooBackend::batch_op_issue(const std::vector<P2POp>& ops, bool async_op, const OpOptions& o) {
  ensure_ready();
  std::vector<c10::intrusive_ptr<c10d::Work>> inner;
  std::vector<std::pair<at::Tensor, at::Tensor>> copies; // (host, device) to copy back
  for (auto& op : ops) {
    check_contig(op.tensor, "batch_op_issue");
    if (op.kind == P2PKind::SEND) {
      std::vector<at::Tensor> v{host_of(op.tensor)};
      inner.push_back(pg_->send(v, op.peer, 0));
    } else {
      at::Tensor host = op.tensor.device().is_cpu()
          ? op.tensor
          : at::empty_like(op.tensor, op.tensor.options().device(at::kCPU));
      std::vector<at::Tensor> v{host};
      inner.push_back(pg_->recv(v, op.peer, 0));
      if (!op.tensor.device().is_cpu()) {
        copies.emplace_back(host, op.tensor);
      }
    }
  }
  auto w = c10::make_intrusive<GlooWork>(std::move(inner), [copies]() mutable {
    for (auto& c : copies) {
      c.second.copy_(c.first);
    }
  }, effective_timeout(o), weak_from_this());
  if (!async_op) {
    w->wait();
  }
  return w;
}

WorkPtr GlooBackend::broadcast(at::Tensor& t, int root, bool async_op, const OpOptions& o) {
  ensure_ready();
  check_contig(t, "broadcast");
  at::Tensor host = host_of(t);
  std::vector<at::Tensor> v{host};
  c10d::BroadcastOptions bo;
  bo.rootRank = root;
  bo.timeout = effective_timeout(o);
  auto inner = pg_->broadcast(v, bo);
  at::Tensor dst = t;
  return finish(inner, [host, dst]() mutable {
    if (!dst.device().is_cpu()) {
      dst.copy_(host);
    }
  }, async_op, o);
}

WorkPtr GlooBackend::all_reduce(at::Tensor& t, const ReduceOp& op, bool async_op, const OpOptions& o) {
  ensure_ready();
  check_contig(t, "all_reduce");
  at::Tensor host = host_of(t);
  premultiply(host, op);
  std::vector<at::Tensor> v{host};
  c10d::AllreduceOptions ao;
  ao.reduceOp = to_c10d(op, t.scalar_type());
  ao.timeout = effective_timeout(o);
  auto inner = pg_->allreduce(v, ao);
  at::Tensor dst = t;
  const int n = size_;
  return finish(inner, [host, dst, op, n]() mutable {
    postdivide(host, op, n);
    if (!dst.device().is_cpu()) {
      dst.copy_(host);
    }
  }, async_op, o);
}

WorkPtr GlooBackend::reduce(const at::Tensor& t, int root, const ReduceOp& op, bool async_op, const OpOptions& o) {
  ensure_ready();
  check_contig(t, "reduce");
  at::Tensor host = host_of(t);
  premultiply(host, op);
  std::vector<at::Tensor> v{host};
  c10d::ReduceOptions ro;
  ro.reduceOp = to_c10d(op, t.scalar_type());
  ro.rootRank = root;
  ro.timeout = effective_timeout(o);
  auto inner = pg_->reduce(v, ro);
  at::Tensor dst = t;
  const int n = size_;
  const bool is_root = rank_ == root;
  return finish(inner, [host, dst, op, n, is_root]() mutable {
    if (is_root) {
      postdivide(host, op, n);
      if (!dst.device().is_cpu()) {
        dst.copy_(host);
      }
    }
  }, async_op, o);
}

WorkPtr GlooBackend::all_gather(const std::vector<at::Tensor>& outs, const at::Tensor& in, bool async_op, const OpOptions& o) {
  ensure_ready();
  TORCH_CHECK(static_cast<int>(outs.size()) == size_, "all_gather: need size() output tensors");
  check_contig(in, "all_gather");
  std::vector<at::Tensor> host_outs;
  for (auto& t : outs) {
    check_contig(t, "all_gather");
    TORCH_CHECK(t.numel() == in.numel(), "all_gather: every output must match the input's numel");
    host_outs.push_back(t.device().is_cpu() ? t : at::empty_like(t, t.options().device(at::kCPU)));
  }
  std::vector<std::vector<at::Tensor>> ov{host_outs};
  std::vector<at::Tensor> iv{host_of(in)};
  c10d::AllgatherOptions ao;
  ao.timeout = effective_timeout(o);
  auto inner = pg_->allgather(ov, iv, ao);
  auto dsts = outs;
  return finish(inner, [host_outs, dsts]() mutable {
    for (size_t i = 0; i < dsts.size(); ++i) {
      if (!dsts[i].device().is_cpu()) {
        dsts[i].copy_(host_outs[i]);
      }
    }
  }, async_op, o);
}

WorkPtr GlooBackend::all_gather_v(const std::vector<at::Tensor>& outs, const at::Tensor& in, bool async_op, const OpOptions& o) {
  ensure_ready();
  TORCH_CHECK(static_cast<int>(outs.size()) == size_, "all_gather_v: need size() output tensors");
  check_contig(in, "all_gather_v");
  TORCH_CHECK(outs[rank_].numel() == in.numel(), "all_gather_v: own output slot must match the input");
  // One broadcast per member, each rooted at the owner of that slot.
  std::vector<c10::intrusive_ptr<c10d::Work>> inner;
  std::vector<at::Tensor> hosts;
  for (int r = 0; r < size_; ++r) {
    check_contig(outs[r], "all_gather_v");
    at::Tensor host = outs[r].device().is_cpu() ? outs[r] : at::empty_like(outs[r], outs[r].options().device(at::kCPU));
    if (r == rank_) {
      host.view({-1}).copy_(in.reshape({-1}));
    }
    hosts.push_back(host);
    std::vector<at::Tensor> v{host};
    c10d::BroadcastOptions bo;
    bo.rootRank = r;
    bo.timeout = effective_timeout(o);
    inner.push_back(pg_->broadcast(v, bo));
  }
  auto dsts = outs;
  auto w = c10::make_intrusive<GlooWork>(std::move(inner), [hosts, dsts]() mutable {
    for (size_t i = 0; i < dsts.size(); ++i) {
      if (!dsts[i].device().is_cpu()) {
        dsts[i].copy_(hosts[i]);
      }
    }
  }, effective_timeout(o), weak_from_this());
  if (!async_op) {
    w->wait();
  }
  return w;
}

WorkPtr GlooBackend::all_gather_single(at::Tensor& out, const at::Tensor& in, bool async_op, const OpOptions& o) {
  ensure_ready();
  check_contig(out, "all_gather_single");
  check_contig(in, "all_gather_single");
  TORCH_CHECK(out.numel() == in.numel() * size_, "all_gather_single: output numel must be input numel * size");
  at::Tensor host_out = out.device().is_cpu() ? out : at::empty_like(out, out.options().device(at::kCPU));
  at::Tensor host_in = host_of(in);
  c10d::AllgatherOptions ao;
  ao.timeout = effective_timeout(o);
  auto inner = pg_->_allgather_base(host_out, host_in, ao);
  at::Tensor dst = out;
  return finish(inner, [host_out, host_in, dst]() mutable {
    if (!dst.device().is_cpu()) {
      dst.copy_(host_out);
    }
  }, async_op, o);
}

WorkPtr GlooBackend::reduce_scatter_single(at::Tensor& out, const at::Tensor& in, const ReduceOp& op, bool async_op, const OpOptions& o) {
  ensure_ready();
  check_contig(out, "reduce_scatter_single");
  check_contig(in, "reduce_scatter_single");
  TORCH_CHECK(in.numel() == out.numel() * size_, "reduce_scatter_single: input numel must be output numel * size");
  // All-reduce a private copy, then keep this rank's slice.
  at::Tensor host = in.to(at::kCPU).clone();
  premultiply(host, op);
  std::vector<at::Tensor> v{host};
  c10d::AllreduceOptions ao;
  ao.reduceOp = to_c10d(op, in.scalar_type());
  ao.timeout = effective_timeout(o);
  auto inner = pg_->allreduce(v, ao);
  at::Tensor dst = out;
  const int n = size_, r = rank_;
  return finish(inner, [host, dst, op, n, r]() mutable {
    at::Tensor mine = host.view({n, -1})[r];
    postdivide(mine, op, n);
    dst.view({-1}).copy_(mine);
  }, async_op, o);
}

WorkPtr GlooBackend::reduce_scatter(at::Tensor& out, const std::vector<at::Tensor>& ins, const ReduceOp& op, bool async_op, const OpOptions& o) {
  TORCH_CHECK(static_cast<int>(ins.size()) == size_, "reduce_scatter: need size() input tensors");
  for (auto& t : ins) {
    TORCH_CHECK(t.numel() == out.numel(), "reduce_scatter: every input must match the output's numel");
  }
  return reduce_scatter_v(out, ins, op, async_op, o);
}

WorkPtr GlooBackend::reduce_scatter_v(at::Tensor& out, const std::vector<at::Tensor>& ins, const ReduceOp& op, bool async_op, const OpOptions& o) {
  ensure_ready();
  TORCH_CHECK(static_cast<int>(ins.size()) == size_, "reduce_scatter_v: need size() input tensors");
  check_contig(out, "reduce_scatter_v");
  TORCH_CHECK(ins[rank_].numel() == out.numel(), "reduce_scatter_v: own input slot must match the output");
  std::vector<at::Tensor> flat;
  int64_t offset = 0, my_off = 0;
  for (int r = 0; r < size_; ++r) {
    check_contig(ins[r], "reduce_scatter_v");
    if (r == rank_) {
      my_off = offset;
    }
    offset += ins[r].numel();
    flat.push_back(ins[r].to(at::kCPU).reshape({-1}));
  }
  at::Tensor host = at::cat(flat);
  premultiply(host, op);
  std::vector<at::Tensor> v{host};
  c10d::AllreduceOptions ao;
  ao.reduceOp = to_c10d(op, out.scalar_type());
  ao.timeout = effective_timeout(o);
  auto inner = pg_->allreduce(v, ao);
  at::Tensor dst = out;
  const int n = size_;
  const int64_t len = out.numel();
  return finish(inner, [host, dst, op, n, my_off, len]() mutable {
    at::Tensor mine = host.narrow(0, my_off, len);
    postdivide(mine, op, n);
    dst.view({-1}).copy_(mine);
  }, async_op, o);
}

WorkPtr GlooBackend::all_to_all_single(at::Tensor& out, const at::Tensor& in, bool async_op, const OpOptions& o) {
  TORCH_CHECK(out.numel() == in.numel(), "all_to_all_single: input and output numel differ");
  TORCH_CHECK(in.numel() % std::max(size_, 1) == 0, "all_to_all_single: numel must divide by size()");
  return all_to_all_v_single(out, in, {}, {}, async_op, o);
}

WorkPtr GlooBackend::all_to_all_v_single(at::Tensor& out, const at::Tensor& in,
                                         const std::vector<int64_t>& out_splits,
                                         const std::vector<int64_t>& in_splits,
                                         bool async_op, const OpOptions& o) {
  ensure_ready();
  check_contig(out, "all_to_all_v_single");
  check_contig(in, "all_to_all_v_single");
  at::Tensor host_out = out.device().is_cpu() ? out : at::empty_like(out, out.options().device(at::kCPU));
  at::Tensor host_in = host_of(in);
  std::vector<int64_t> os = out_splits, is = in_splits;
  c10d::AllToAllOptions ao;
  ao.timeout = effective_timeout(o);
  // Equal-split calls on multi-dimensional tensors exchange dim-0 slices; a
  // flat view keeps the element counts right when dim 0 is not divisible.
  if (os.empty() && is.empty()) {
    host_out = host_out.view({-1});
    host_in = host_in.view({-1});
  }
  auto inner = pg_->alltoall_base(host_out, host_in, os, is, ao);
  at::Tensor dst = out;
  return finish(inner, [host_out, host_in, dst]() mutable {
    if (!dst.device().is_cpu()) {
      dst.view({-1}).copy_(host_out.view({-1}));
    }
  }, async_op, o);
}

WorkPtr GlooBackend::all_to_all(const std::vector<at::Tensor>& outs, const std::vector<at::Tensor>& ins, bool async_op, const OpOptions& o) {
  ensure_ready();
  TORCH_CHECK(static_cast<int>(outs.size()) == size_ && static_cast<int>(ins.size()) == size_,
              "all_to_all: need size() input and output tensors");
  // gloo has no list all-to-all: flatten into one split exchange.
  std::vector<int64_t> in_splits, out_splits;
  std::vector<at::Tensor> flat_ins;
  int64_t out_total = 0;
  for (int r = 0; r < size_; ++r) {
    check_contig(outs[r], "all_to_all");
    check_contig(ins[r], "all_to_all");
    TORCH_CHECK(outs[r].scalar_type() == ins[r].scalar_type(), "all_to_all: dtype mismatch");
    in_splits.push_back(ins[r].numel());
    out_splits.push_back(outs[r].numel());
    out_total += outs[r].numel();
    flat_ins.push_back(ins[r].to(at::kCPU).reshape({-1}));
  }
  at::Tensor host_in = at::cat(flat_ins);
  at::Tensor host_out = at::empty({out_total}, host_in.options());
  c10d::AllToAllOptions ao;
  ao.timeout = effective_timeout(o);
  // The process group may move from the count vectors: hand it copies.
  std::vector<int64_t> out_counts = out_splits, in_counts = in_splits;
  auto inner = pg_->alltoall_base(host_out, host_in, out_counts, in_counts, ao);
  auto dsts = outs;
  return finish(inner, [host_out, host_in, out_splits, dsts]() mutable {
    int64_t off = 0;
    for (size_t i = 0; i < dsts.size(); ++i) {
      dsts[i].view({-1}).copy_(host_out.narrow(0, off, out_splits[i]));
      off += out_splits[i];
    }
  }, async_op, o);
}

WorkPtr GlooBackend::barrier(bool async_op, const OpOptions& o) {
  ensure_ready();
  c10d::BarrierOptions bo;
  bo.timeout = effective_timeout(o);
  return finish(pg_->barrier(bo), nullptr, async_op, o);
}

WorkPtr GlooBackend::scatter(at::Tensor& out, const std::vector<at::Tensor>& ins, int root, bool async_op, const OpOptions& o) {
  ensure_ready();
  check_contig(out, "scatter");
  at::Tensor host_out = out.device().is_cpu() ? out : at::empty_like(out, out.options().device(at::kCPU));
  std::vector<at::Tensor> ov{host_out};
  std::vector<std::vector<at::Tensor>> iv;
  if (rank_ == root) {
    TORCH_CHECK(static_cast<int>(ins.size()) == size_, "scatter: the root needs size() input tensors");
    std::vector<at::Tensor> hosts;
    for (auto& t : ins) {
      check_contig(t, "scatter");
      TORCH_CHECK(t.numel() == out.numel(), "scatter: every input must match the output's numel");
      hosts.push_back(host_of(t));
    }
    iv.push_back(std::move(hosts));
  }
  c10d::ScatterOptions so;
  so.rootRank = root;
  so.timeout = effective_timeout(o);
  auto inner = pg_->scatter(ov, iv, so);
  at::Tensor dst = out;
  return finish(inner, [host_out, iv, dst]() mutable {
    if (!dst.device().is_cpu()) {
      dst.copy_(host_out);
    }
  }, async_op, o);
}

WorkPtr GlooBackend::gather(const std::vector<at::Tensor>& outs, const at::Tensor& in, int root, bool async_op, const OpOptions& o) {
  ensure_ready();
  check_contig(in, "gather");
  std::vector<std::vector<at::Tensor>> ov;
  std::vector<at::Tensor> hosts;
  if (rank_ == root) {
    TORCH_CHECK(static_cast<int>(outs.size()) == size_, "gather: the root needs size() output tensors");
    for (auto& t : outs) {
      check_contig(t, "gather");
      TORCH_CHECK(t.numel() == in.numel(), "gather: every output must match the input's numel");
      hosts.push_back(t.device().is_cpu() ? t : at::empty_like(t, t.options().device(at::kCPU)));
    }
    ov.push_back(hosts);
  }
  std::vector<at::Tensor> iv{host_of(in)};
  c10d::GatherOptions go;
  go.rootRank = root;
  go.timeout = effective_timeout(o);
  auto inner = pg_->gather(ov, iv, go);
  auto dsts = outs;
  return finish(inner, [hosts, iv, dsts]() mutable {
    for (size_t i = 0; i < hosts.size(); ++i) {
      if (!dsts[i].device().is_cpu()) {
        dsts[i].copy_(hosts[i]);
      }
    }
  }, async_op, o);
}

std::shared_ptr<Backend> GlooBackend::split(const std::vector<int>& ranks, const std::string& name, const CommOptions& opts) {
  ensure_ready();
  const uint64_t gen = split_counter_++;
  if (ranks.empty()) {
    return nullptr;
  }
  int color = ranks[0], idx = -1;
  for (size_t i = 0; i < ranks.size(); ++i) {
    color = std::min(color, ranks[i]);
    if (ranks[i] == rank_) {
      idx = static_cast<int>(i);
    }
  }
  TORCH_CHECK(idx >= 0, "split: calling rank is not a member of the new group");
  auto child = std::make_shared<GlooBackend>();
  child->device_ = device_;
  child->name_ = (name.empty() ? name_ : name) + "_" + std::to_string(color);
  child->opts_ = opts;
  if (!opts.store) {
    child->opts_.store = opts_.store;
  }
  child->handle_token_ = handle_token_ + "/" + child->name_;
  child->store_ = scoped_store(store_, "split/" + std::to_string(gen) + "/" + std::to_string(color));
  child->connect(child->store_, idx, static_cast<int>(ranks.size()));
  return child;
}

std::shared_ptr<Backend> GlooBackend::create_pair_comm(int peer, const std::string& name) {
  ensure_ready();
  TORCH_CHECK(peer >= 0 && peer < size_ && peer != rank_, "create_pair_comm: bad peer ", peer);
  auto child = std::make_shared<GlooBackend>();
  child->device_ = device_;
  child->name_ = name_ + "::" + name;
  child->opts_ = opts_;
  child->handle_token_ = handle_token_ + "/" + child->name_;
  child->store_ = scoped_store(store_, "pair/" + name);
  child->connect(child->store_, rank_ < peer ? 0 : 1, 2);
  return child;
}

InitHandle GlooBackend::get_init_handle() const {
  return "gloo:" + handle_token_;
}

WorkPtr GlooBackend::reconfigure(const ReconfigureOptions& o) {
  TORCH_CHECK(!finalized_, "gloo communicator '", name_, "' was finalized");
  TORCH_CHECK(opts_.enable_reconfigure, "reconfigure() needs a communicator created with enable_reconfigure=True");
  std::vector<InitHandle> members = o.handles;
  if (!o.handles_ordered) {
    std::sort(members.begin(), members.end());
  }
  const InitHandle me = get_init_handle();
  int idx = -1;
  for (size_t i = 0; i < members.size(); ++i) {
    if (members[i] == me) {
      idx = static_cast<int>(i);
    }
  }
  TORCH_CHECK(idx >= 0, "reconfigure: this rank's init handle is not in the member list");
  if (o.timeout) {
    opts_.timeout = *o.timeout;
  }
  pg_.reset();
  aborted_ = false;
  auto scoped = scoped_store(store_, "b200c/gloo/reconf/" + std::to_string(o.uuid));
  connect(scoped, idx, static_cast<int>(members.size()));
  return c10::make_intrusive<CompletedWork>();
}

} // namespace b200c
