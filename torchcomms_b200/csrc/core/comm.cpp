// Facade, backend defaults, factory and health flag.
#include "comm.hpp"

#include <dlfcn.h>

#include <ATen/record_function.h>
#include <torch/csrc/distributed/c10d/control_plane/Handlers.hpp>

#include <algorithm>
#include <atomic>
#include <cctype>
#include <set>

#include "logging.hpp"

namespace b200c {

// ------------------------------------------------------ Backend defaults ----

WorkPtr Backend::gather_single(at::Tensor& out, const at::Tensor& in, int root, bool async_op, const OpOptions& o) {
  std::vector<at::Tensor> outs;
  if (rank() == root) {
    TORCH_CHECK(out.numel() == in.numel() * size(),
                "gather_single: output must hold size() copies of the input");
    auto flat = out.view({size(), -1});
    for (int r = 0; r < size(); ++r) {
      outs.push_back(flat[r].view(in.sizes()));
    }
  }
  return gather(outs, in, root, async_op, o);
}

std::shared_ptr<Window> Backend::new_window(const std::optional<at::Tensor>&) {
  throw std::runtime_error("backend '" + backend_name() + "' has no one-sided window support");
}

std::shared_ptr<AllGatherPHandle> Backend::all_gather_p_init(at::Tensor& output, const OpOptions&) {
  static std::atomic<uint64_t> ids{1};
  auto h = std::make_shared<AllGatherPHandle>();
  h->output = output;
  h->id = ids++;
  return h;
}

WorkPtr Backend::all_gather_p_exec(const std::shared_ptr<AllGatherPHandle>& h, const at::Tensor& in,
                                   bool async_op, const OpOptions& o) {
  TORCH_CHECK(h && !h->freed, "all_gather_p_exec: handle was freed");
  return all_gather_single(h->output, in, async_op, o);
}

void Backend::all_gather_p_free(const std::shared_ptr<AllGatherPHandle>& h) {
  if (h) {
    h->freed = true;
    h->output = at::Tensor();
  }
}

InitHandle Backend::get_init_handle() const {
  throw std::runtime_error("backend '" + backend_name() + "' does not support reconfigure");
}

WorkPtr Backend::reconfigure(const ReconfigureOptions&) {
  throw std::runtime_error("backend '" + backend_name() + "' does not support reconfigure");
}

void Backend::run_abort_hooks() const {
  if (!abort_hooks_) {
    return;
  }
  for (auto& h : abort_hooks_->snapshot()) {
    try {
      h();
    } catch (const std::exception& e) {
      B200C_LOG(ERROR, "abort", "abort hook raised: " << e.what());
    }
  }
}

// ----------------------------------------------------------------- Comm ----

namespace {
std::atomic<size_t> g_next_op_id{0};
}

size_t Comm::next_op_id() {
  return g_next_op_id.fetch_add(1, std::memory_order_relaxed);
}

namespace {
// Communicators alive in this process, for comm_dump_all(). Never destroyed:
// communicators may be released during static teardown.
std::mutex& live_comms_mu() {
  static std::mutex* m = new std::mutex();
  return *m;
}
std::set<Comm*>& live_comms() {
  static std::set<Comm*>* s = new std::set<Comm*>();
  return *s;
}
}  // namespace

Comm::Comm(std::shared_ptr<Backend> impl, std::vector<int> global_ranks)
    : impl_(std::move(impl)), ranks_(std::move(global_ranks)) {
  // A communicator created for reconfigure() has no membership yet (size < 1).
  if (ranks_.empty() && impl_->size() > 0) {
    ranks_.resize(impl_->size());
    for (int i = 0; i < impl_->size(); ++i) {
      ranks_[i] = i;
    }
  }
  impl_->attach_hook_tables(abort_hooks_, replay_hooks_);
  std::lock_guard<std::mutex> g(live_comms_mu());
  live_comms().insert(this);
}

namespace {
std::atomic<int64_t> g_trainer_iteration{-1};
}
void set_trainer_iteration(int64_t iteration) { g_trainer_iteration.store(iteration, std::memory_order_relaxed); }
int64_t trainer_iteration() { return g_trainer_iteration.load(std::memory_order_relaxed); }

std::unordered_map<std::string, std::unordered_map<std::string, std::string>> comm_dump_all() {
  std::unordered_map<std::string, std::unordered_map<std::string, std::string>> out;
  std::lock_guard<std::mutex> g(live_comms_mu());
  for (Comm* c : live_comms()) {
    try {
      auto d = c->get_backend_impl()->comm_dump();
      d["finalized"] = c->finalized_ ? "1" : "0";
      d["iteration"] = std::to_string(trainer_iteration());
      out[c->get_name()] = std::move(d);
    } catch (const std::exception& e) {
      out[c->get_name()] = {{"error", e.what()}};
    }
  }
  return out;
}

Comm::~Comm() {
  {
    std::lock_guard<std::mutex> g(live_comms_mu());
    live_comms().erase(this);
  }
  if (!finalized_) {
    B200C_LOG(WARN, "comm", "communicator destroyed without finalize()");
  }
}

std::shared_ptr<Backend> Backend::create_pair_comm(int, const std::string&) {
  TORCH_CHECK(false, "backend '", backend_name(), "' cannot create per-peer communicators");
}

void Comm::check_rank(int r, const char* what) const {
  TORCH_CHECK(r >= 0 && r < impl_->size(), what, " rank ", r, " is outside [0, ", impl_->size(), ")");
}

template <typename F>
WorkPtr Comm::run_op(OpRecord rec, F&& call) {
  TORCH_CHECK(!finalized_, "communicator '", impl_->comm_name(), "' was finalized");
  const size_t id = next_op_id();
  // Profiler span around the enqueue of every operation (shows up in Kineto
  // traces next to the kernels it launched). Built only when somebody listens.
  at::RecordFunction span(at::RecordScope::USER_SCOPE);
  if (span.isActive()) {
    std::string label = "torchcomms_b200::";
    label += op_name(rec.op);
    if (span.needsInputs()) {
      std::vector<c10::IValue> ins;
      for (const auto& t : rec.inputs) ins.emplace_back(t);
      ins.emplace_back(static_cast<int64_t>(id));
      ins.emplace_back(impl_->comm_name());
      span.before(label, c10::ArrayRef<const c10::IValue>(ins.data(), ins.size()));
    } else {
      span.before(label);
    }
  }
  if (!pre_hooks_->empty()) {
    for (auto& h : pre_hooks_->snapshot()) {
      h(rec.op, id, rec);
    }
  }
  WorkPtr w = call();
  if (!post_hooks_->empty()) {
    rec.work = c10::weak_intrusive_ptr<Work>(w);
    for (auto& h : post_hooks_->snapshot()) {
      h(id, rec);
    }
  }
  return w;
}

void Comm::finalize() {
  TORCH_CHECK(!finalized_, "communicator '", impl_->comm_name(), "' was already finalized");
  OpRecord rec;
  rec.op = OpName::finalize;
  for (auto& h : pre_hooks_->snapshot()) {
    h(rec.op, kFinalizeOpId, rec);
  }
  finalized_ = true;
  impl_->finalize();
  for (auto& h : post_hooks_->snapshot()) {
    h(kFinalizeOpId, rec);
  }
}

WorkPtr Comm::send(const at::Tensor& t, int dst, bool async_op, const OpOptions& o) {
  check_rank(dst, "destination");
  OpRecord r;
  r.op = OpName::send;
  r.inputs = {t};
  r.root = dst;
  r.async_op = async_op;
  return run_op(std::move(r), [&] { return impl_->send(t, dst, async_op, o); });
}

WorkPtr Comm::recv(at::Tensor& t, int src, bool async_op, const OpOptions& o) {
  check_rank(src, "source");
  OpRecord r;
  r.op = OpName::recv;
  r.outputs = {t};
  r.root = src;
  r.async_op = async_op;
  return run_op(std::move(r), [&] { return impl_->recv(t, src, async_op, o); });
}

WorkPtr Comm::broadcast(at::Tensor& t, int root, bool async_op, const OpOptions& o) {
  check_rank(root, "root");
  OpRecord r;
  r.op = OpName::broadcast;
  r.inputs = {t};
  r.outputs = {t};
  r.in_place = true;
  r.root = root;
  r.async_op = async_op;
  return run_op(std::move(r), [&] { return impl_->broadcast(t, root, async_op, o); });
}

WorkPtr Comm::all_reduce(at::Tensor& t, const ReduceOp& op, bool async_op, const OpOptions& o) {
  OpRecord r;
  r.op = OpName::all_reduce;
  r.inputs = {t};
  r.outputs = {t};
  r.in_place = true;
  r.red_op = op.type();
  r.async_op = async_op;
  return run_op(std::move(r), [&] { return impl_->all_reduce(t, op, async_op, o); });
}

WorkPtr Comm::reduce(const at::Tensor& t, int root, const ReduceOp& op, bool async_op, const OpOptions& o) {
  check_rank(root, "root");
  OpRecord r;
  r.op = OpName::reduce;
  r.inputs = {t};
  r.outputs = {t};
  r.in_place = true;
  r.root = root;
  r.red_op = op.type();
  r.async_op = async_op;
  return run_op(std::move(r), [&] { return impl_->reduce(t, root, op, async_op, o); });
}

WorkPtr Comm::all_gather(const std::vector<at::Tensor>& outs, const at::Tensor& in, bool async_op, const OpOptions& o) {
  OpRecord r;
  r.op = OpName::all_gather;
  r.inputs = {in};
  r.outputs = outs;
  r.async_op = async_op;
  return run_op(std::move(r), [&] { return impl_->all_gather(outs, in, async_op, o); });
}

WorkPtr Comm::all_gather_v(const std::vector<at::Tensor>& outs, const at::Tensor& in, bool async_op, const OpOptions& o) {
  OpRecord r;
  r.op = OpName::all_gather_v;
  r.inputs = {in};
  r.outputs = outs;
  r.async_op = async_op;
  return run_op(std::move(r), [&] { return impl_->all_gather_v(outs, in, async_op, o); });
}

WorkPtr Comm::all_gather_single(at::Tensor& out, const at::Tensor& in, bool async_op, const OpOptions& o) {
  OpRecord r;
  r.op = OpName::all_gather_single;
  r.inputs = {in};
  r.outputs = {out};
  r.async_op = async_op;
  return run_op(std::move(r), [&] { return impl_->all_gather_single(out, in, async_op, o); });
}

WorkPtr Comm::reduce_scatter(at::Tensor& out, const std::vector<at::Tensor>& ins, const ReduceOp& op, bool async_op, const OpOptions& o) {
  OpRecord r;
  r.op = OpName::reduce_scatter;
  r.inputs = ins;
  r.outputs = {out};
  r.red_op = op.type();
  r.async_op = async_op;
  return run_op(std::move(r), [&] { return impl_->reduce_scatter(out, ins, op, async_op, o); });
}

WorkPtr Comm::reduce_scatter_v(at::Tensor& out, const std::vector<at::Tensor>& ins, const ReduceOp& op, bool async_op, const OpOptions& o) {
  OpRecord r;
  r.op = OpName::reduce_scatter_v;
  r.inputs = ins;
  r.outputs = {out};
  r.red_op = op.type();
  r.async_op = async_op;
  return run_op(std::move(r), [&] { return impl_->reduce_scatter_v(out, ins, op, async_op, o); });
}

WorkPtr Comm::reduce_scatter_single(at::Tensor& out, const at::Tensor& in, const ReduceOp& op, bool async_op, const OpOptions& o) {
  OpRecord r;
  r.op = OpName::reduce_scatter_single;
  r.inputs = {in};
  r.outputs = {out};
  r.red_op = op.type();
  r.async_op = async_op;
  return run_op(std::move(r), [&] { return impl_->reduce_scatter_single(out, in, op, async_op, o); });
}

WorkPtr Comm::all_to_all_single(at::Tensor& out, const at::Tensor& in, bool async_op, const OpOptions& o) {
  OpRecord r;
  r.op = OpName::all_to_all_single;
  r.inputs = {in};
  r.outputs = {out};
  r.async_op = async_op;
  return run_op(std::move(r), [&] { return impl_->all_to_all_single(out, in, async_op, o); });
}

WorkPtr Comm::all_to_all_v_single(at::Tensor& out, const at::Tensor& in,
                                  const std::vector<int64_t>& out_splits,
                                  const std::vector<int64_t>& in_splits,
                                  bool async_op, const OpOptions& o) {
  OpRecord r;
  r.op = OpName::all_to_all_v_single;
  r.inputs = {in};
  r.outputs = {out};
  r.in_splits = in_splits;
  r.out_splits = out_splits;
  r.async_op = async_op;
  return run_op(std::move(r), [&] {
    return impl_->all_to_all_v_single(out, in, out_splits, in_splits, async_op, o);
  });
}

WorkPtr Comm::all_to_all(const std::vector<at::Tensor>& outs, const std::vector<at::Tensor>& ins, bool async_op, const OpOptions& o) {
  OpRecord r;
  r.op = OpName::all_to_all;
  r.inputs = ins;
  r.outputs = outs;
  r.async_op = async_op;
  return run_op(std::move(r), [&] { return impl_->all_to_all(outs, ins, async_op, o); });
}

WorkPtr Comm::barrier(bool async_op, const OpOptions& o) {
  OpRecord r;
  r.op = OpName::barrier;
  r.async_op = async_op;
  return run_op(std::move(r), [&] { return impl_->barrier(async_op, o); });
}

WorkPtr Comm::scatter(at::Tensor& out, const std::vector<at::Tensor>& ins, int root, bool async_op, const OpOptions& o) {
  check_rank(root, "root");
  OpRecord r;
  r.op = OpName::scatter;
  r.inputs = ins;
  r.outputs = {out};
  r.root = root;
  r.async_op = async_op;
  return run_op(std::move(r), [&] { return impl_->scatter(out, ins, root, async_op, o); });
}

WorkPtr Comm::gather(const std::vector<at::Tensor>& outs, const at::Tensor& in, int root, bool async_op, const OpOptions& o) {
  check_rank(root, "root");
  OpRecord r;
  r.op = OpName::gather;
  r.inputs = {in};
  r.outputs = outs;
  r.root = root;
  r.async_op = async_op;
  return run_op(std::move(r), [&] { return impl_->gather(outs, in, root, async_op, o); });
}

WorkPtr Comm::gather_single(at::Tensor& out, const at::Tensor& in, int root, bool async_op, const OpOptions& o) {
  check_rank(root, "root");
  OpRecord r;
  r.op = OpName::gather_single;
  r.inputs = {in};
  r.outputs = {out};
  r.root = root;
  r.async_op = async_op;
  return run_op(std::move(r), [&] { return impl_->gather_single(out, in, root, async_op, o); });
}

std::shared_ptr<Comm> Comm::split(const std::vector<int>& ranks, const std::string& name, const CommOptions& opts) {
  TORCH_CHECK(!finalized_, "communicator '", impl_->comm_name(), "' was finalized");
  std::set<int> seen;
  for (int r : ranks) {
    check_rank(r, "split");
    TORCH_CHECK(seen.insert(r).second, "split: rank ", r, " appears twice");
  }
  if (!ranks.empty()) {
    TORCH_CHECK(seen.count(impl_->rank()) == 1,
                "split: the calling rank ", impl_->rank(), " is not in the non-empty rank list");
  }
  OpRecord rec;
  rec.op = OpName::split;
  rec.ranks = ranks;
  rec.name = name;
  const size_t id = next_op_id();
  for (auto& h : pre_hooks_->snapshot()) {
    h(rec.op, id, rec);
  }
  CommOptions child_opts = opts;
  child_opts.name = name;
  std::shared_ptr<Backend> child = impl_->split(ranks, name, child_opts);
  for (auto& h : post_hooks_->snapshot()) {
    h(id, rec);
  }
  if (!child) {
    return nullptr;
  }
  std::vector<int> globals;
  globals.reserve(ranks.size());
  for (int r : ranks) {
    globals.push_back(ranks_[r]);
  }
  return std::make_shared<Comm>(std::move(child), std::move(globals));
}

std::shared_ptr<BatchSendRecv> Comm::batch_op_create() {
  return std::make_shared<BatchSendRecv>(shared_from_this());
}

WorkPtr Comm::batch_op_issue(const std::vector<P2POp>& ops, bool async_op, const OpOptions& o) {
  for (auto& op : ops) {
    check_rank(op.peer, "peer");
  }
  OpRecord r;
  r.op = OpName::batch_op_issue;
  r.p2p_ops = ops;
  r.async_op = async_op;
  return run_op(std::move(r), [&] { return impl_->batch_op_issue(ops, async_op, o); });
}

std::shared_ptr<Window> Comm::new_window(const std::optional<at::Tensor>& tensor) {
  TORCH_CHECK(!finalized_, "communicator '", impl_->comm_name(), "' was finalized");
  OpRecord rec;
  rec.op = OpName::new_window;
  if (tensor) {
    rec.inputs = {*tensor};
  }
  const size_t id = next_op_id();
  for (auto& h : pre_hooks_->snapshot()) {
    h(rec.op, id, rec);
  }
  auto w = impl_->new_window(tensor);
  for (auto& h : post_hooks_->snapshot()) {
    h(id, rec);
  }
  return w;
}

std::shared_ptr<AllGatherPHandle> Comm::all_gather_p_init(at::Tensor& output, const OpOptions& o) {
  return impl_->all_gather_p_init(output, o);
}

WorkPtr Comm::all_gather_p_exec(const std::shared_ptr<AllGatherPHandle>& h, const at::Tensor& in, bool async_op, const OpOptions& o) {
  TORCH_CHECK(h, "all_gather_p_exec: null handle");
  OpRecord r;
  r.op = OpName::all_gather_single;
  r.inputs = {in};
  r.outputs = {h->output};
  r.async_op = async_op;
  return run_op(std::move(r), [&] { return impl_->all_gather_p_exec(h, in, async_op, o); });
}

void Comm::all_gather_p_free(const std::shared_ptr<AllGatherPHandle>& h) {
  impl_->all_gather_p_free(h);
}

WorkPtr Comm::reconfigure(const ReconfigureOptions& o) {
  WorkPtr w = impl_->reconfigure(o);
  // Membership may have changed: the communicator becomes its own world.
  w->wait_blocking();
  ranks_.resize(impl_->size());
  for (int i = 0; i < impl_->size(); ++i) {
    ranks_[i] = i;
  }
  return w;
}

void BatchSendRecv::send(const at::Tensor& t, int dst) {
  ops.push_back(P2POp{P2PKind::SEND, t, dst});
}

void BatchSendRecv::recv(at::Tensor& t, int src) {
  ops.push_back(P2POp{P2PKind::RECV, t, src});
}

WorkPtr BatchSendRecv::issue(bool async_op, const OpOptions& o) {
  return parent_->batch_op_issue(ops, async_op, o);
}

// -------------------------------------------------------------- Factory ----

Factory& Factory::get() {
  static Factory* inst = new Factory();
  return *inst;
}

void Factory::register_backend(const std::string& name, Maker maker) {
  std::lock_guard<std::mutex> g(mu_);
  makers_[name] = std::move(maker);
}

bool Factory::is_registered(const std::string& name) const {
  std::lock_guard<std::mutex> g(mu_);
  return makers_.count(name) != 0;
}

std::vector<std::string> Factory::registered() const {
  std::lock_guard<std::mutex> g(mu_);
  std::vector<std::string> out;
  for (auto& kv : makers_) {
    out.push_back(kv.first);
  }
  std::sort(out.begin(), out.end());
  return out;
}

std::shared_ptr<Backend> Factory::load_dynamic(const std::string& name) {
  std::string upper = name;
  std::transform(upper.begin(), upper.end(), upper.begin(), [](unsigned char c) {
    return c == '-' ? '_' : std::toupper(c);
  });
  std::string path = env_to_value<std::string>(("TORCHCOMMS_BACKEND_LIB_PATH_" + upper).c_str(), "");
  if (path.empty()) {
    path = env_to_value<std::string>(("B200COMMS_BACKEND_LIB_PATH_" + upper).c_str(), "");
  }
  if (path.empty()) {
    return nullptr;
  }
  void* lib = dlopen(path.c_str(), RTLD_NOW | RTLD_LOCAL);
  TORCH_CHECK(lib != nullptr, "cannot load backend library '", path, "': ", dlerror());
  std::string sym_name = "b200c_create_backend_" + name;
  std::replace(sym_name.begin(), sym_name.end(), '-', '_');
  using LoaderFn = DynamicBackendLoader* (*)();
  auto fn = reinterpret_cast<LoaderFn>(dlsym(lib, sym_name.c_str()));
  TORCH_CHECK(fn != nullptr, "library '", path, "' does not export ", sym_name);
  DynamicBackendLoader* loader = fn();
  TORCH_CHECK(loader && loader->abi_version && loader->create && loader->destroy,
              "library '", path, "' returned an incomplete loader table");
  const std::string abi = loader->abi_version();
  TORCH_CHECK(abi == kBackendAbiVersion, "backend library '", path, "' was built for ABI '", abi,
              "', this core speaks '", kBackendAbiVersion, "'");
  auto destroy = loader->destroy;
  return std::shared_ptr<Backend>(loader->create(), [destroy](Backend* b) { destroy(b); });
}

std::shared_ptr<Backend> Factory::create(const std::string& name, at::Device device,
                                         const std::string& comm_name, const CommOptions& opts) {
  Maker maker;
  {
    std::lock_guard<std::mutex> g(mu_);
    auto it = makers_.find(name);
    if (it != makers_.end()) {
      maker = it->second;
    }
  }
  std::shared_ptr<Backend> b = maker ? maker() : load_dynamic(name);
  TORCH_CHECK(b != nullptr, "unknown communication backend '", name,
              "' (not registered and no TORCHCOMMS_BACKEND_LIB_PATH_* library set)");
  TORCH_CHECK(!opts.enable_reconfigure || b->supports_reconfigure(),
              "backend '", name, "' does not support enable_reconfigure");
  CommOptions with_name = opts;
  with_name.name = comm_name;
  b->init(device, comm_name, with_name);
  return b;
}

std::shared_ptr<Comm> new_comm(const std::string& backend, at::Device device,
                               const std::string& name, const CommOptions& opts) {
  auto impl = Factory::get().create(backend, device, name, opts);
  return std::make_shared<Comm>(std::move(impl));
}

// ---------------------------------------------------------- HealthCheck ----

namespace {
std::mutex g_health_mu;
bool g_healthy = true;
std::string g_health_reason;
} // namespace

void HealthCheck::mark_unhealthy(const std::string& why) {
  std::lock_guard<std::mutex> g(g_health_mu);
  if (g_healthy) {
    g_healthy = false;
    g_health_reason = why;
  }
}

namespace {
// Served by c10d's control plane (the worker server of torch.distributed):
// GET /handler/torchcomms_health_check -> {"healthy": true|false}.
// Registered once per process even if two copies of this library get loaded.
const bool g_health_handler_registered = [] {
  const auto names = c10d::control_plane::getHandlerNames();
  if (std::find(names.begin(), names.end(), "torchcomms_health_check") != names.end()) return false;
  c10d::control_plane::registerHandler(
    "torchcomms_health_check", [](const c10d::control_plane::Request&, c10d::control_plane::Response& res) {
      const bool ok = HealthCheck::healthy();
      std::string body = std::string("{\"healthy\": ") + (ok ? "true" : "false");
      if (!ok) {
        std::string why = HealthCheck::reason();
        for (auto& ch : why) {
          if (ch == '"' || ch == '\\' || static_cast<unsigned char>(ch) < 0x20) ch = ' ';
        }
        body += ", \"reason\": \"" + why + "\"";
      }
      body += "}";
      res.setContent(std::move(body), "application/json");
      res.setStatus(200);
    });
  return true;
}();
} // namespace

bool HealthCheck::healthy() {
  std::lock_guard<std::mutex> g(g_health_mu);
  return g_healthy;
}

std::string HealthCheck::reason() {
  std::lock_guard<std::mutex> g(g_health_mu);
  return g_health_reason;
}

void HealthCheck::reset() {
  std::lock_guard<std::mutex> g(g_health_mu);
  g_healthy = true;
  g_health_reason.clear();
}

} // namespace b200c
