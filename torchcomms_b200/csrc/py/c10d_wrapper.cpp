// Adapter that presents a communicator as a c10d::Backend, so DeviceMesh,
// FSDP, DTensor and plain torch.distributed calls run on it unchanged.
//
// Semantics worth knowing:
//  * every c10d entry point takes exactly one tensor per list;
//  * `opts.asyncOp` is forwarded as `async_op`;
//  * the returned Work's wait() is a stream dependency on CUDA; a synchronous
//    barrier additionally blocks the host;
//  * wait(timeout != 0) is not supported and raises;
//  * send/recv between startCoalescing() and endCoalescing() are collected into
//    one batched point-to-point group.
//
// Parity: comms/torchcomms/BackendWrapper.hpp:20-219, BackendWrapper.cpp:18-58
// (reduce-op mapping), :200-236 (future / wait), :298 (allreduce), :714
// (monitoredBarrier over p2p), :942-949 (coalescing), :1046 (split).
#include <thread>
#include <torch/csrc/distributed/c10d/Backend.hpp>
#include <torch/csrc/distributed/c10d/Work.hpp>

#include "py_common.hpp"

namespace b200c {

namespace {

ReduceOp from_c10d(const c10d::ReduceOp& op) {
  switch (op.op_) {
    case c10d::ReduceOp::SUM: return RedOpType::SUM;
    case c10d::ReduceOp::AVG: return RedOpType::AVG;
    case c10d::ReduceOp::PRODUCT: return RedOpType::PRODUCT;
    case c10d::ReduceOp::MIN: return RedOpType::MIN;
    case c10d::ReduceOp::MAX: return RedOpType::MAX;
    case c10d::ReduceOp::BAND: return RedOpType::BAND;
    case c10d::ReduceOp::BOR: return RedOpType::BOR;
    case c10d::ReduceOp::BXOR: return RedOpType::BXOR;
    case c10d::ReduceOp::PREMUL_SUM: {
      auto* sup = dynamic_cast<c10d::NCCLPreMulSumSupplement*>(op.supplement_.get());
      TORCH_CHECK(sup != nullptr, "PREMUL_SUM without a factor");
      if (sup->tensor_factor.defined()) {
        return ReduceOp::premul_sum(sup->tensor_factor);
      }
      return ReduceOp::premul_sum(sup->double_factor);
    }
    default:
      TORCH_CHECK(false, "unsupported c10d reduce op");
  }
}

OpOptions with_timeout(Millis t, Millis fallback) {
  OpOptions o;
  const Millis eff = (t == c10d::kUnsetTimeout) ? fallback : t;
  o.timeout = eff;
  o.timeout_set = true;
  return o;
}

class WorkWrapper final : public c10d::Work {
 public:
  WorkWrapper(WorkPtr inner, std::vector<at::Tensor> outputs, bool host_block, int rank, c10d::OpType type)
      : c10d::Work(rank, type), inner_(std::move(inner)), outputs_(std::move(outputs)), host_block_(host_block) {}

  bool isCompleted() override { return inner_->is_completed(); }
  bool isSuccess() const override {
    const auto s = inner_->status();
    return s != WorkStatus::ERROR && s != WorkStatus::TIMEDOUT;
  }
  bool wait(std::chrono::milliseconds timeout = ::kNoTimeout) override {
    TORCH_CHECK(timeout == ::kNoTimeout, "wait(timeout) is not supported; set the timeout on the operation");
    if (host_block_) {
      inner_->wait_blocking();
    } else {
      inner_->wait();
    }
    return true;
  }
  void synchronize() override { inner_->wait(); }
  std::vector<at::Tensor> result() override { return outputs_; }

  c10::intrusive_ptr<c10::ivalue::Future> getFuture() override {
    if (future_) {
      return future_;
    }
    std::vector<c10::Device> devices;
    for (auto& t : outputs_) {
      if (t.defined() && !t.device().is_cpu() &&
          std::find(devices.begin(), devices.end(), t.device()) == devices.end()) {
        devices.push_back(t.device());
      }
    }
    future_ = c10::make_intrusive<c10::ivalue::Future>(c10::ListType::create(c10::TensorType::get()), devices);
    if (!devices.empty()) {
      // Device work: make the current stream depend on the collective, then
      // complete the future there; consumers synchronise through its events.
      inner_->wait();
      future_->markCompleted(c10::IValue(outputs_));
    } else {
      // Host work. Callers such as DistributedDataParallel keep only the future and drop the
      // work, and a work of the gloo backend completes when somebody waits on it, so a helper
      // thread waits and then completes the future (or gives it the error).
      auto fut = future_;
      auto outs = outputs_;
      auto inner = inner_;
      if (inner->is_completed()) {
        fut->markCompleted(c10::IValue(outs));
      } else {
        std::thread([fut, outs, inner]() {
          try {
            inner->wait();
            if (!fut->completed()) {
              fut->markCompleted(c10::IValue(outs));
            }
          } catch (...) {
            if (!fut->completed()) {
              fut->setError(std::current_exception());
            }
          }
        }).detach();
      }
    }
    return future_;
  }

 private:
  WorkPtr inner_;
  std::vector<at::Tensor> outputs_;
  bool host_block_;
  c10::intrusive_ptr<c10::ivalue::Future> future_;
};

class BackendWrapper final : public c10d::Backend {
 public:
  explicit BackendWrapper(std::shared_ptr<Comm> comm)
      : c10d::Backend(comm->get_rank(), comm->get_size()), comm_(std::move(comm)) {
    options_ = c10::make_intrusive<c10d::Backend::Options>("torchcomms_b200", comm_->get_options().timeout);
  }

  std::shared_ptr<Comm> get_comm() const { return comm_; }
  const std::string getBackendName() const override { return "torchcomms_b200"; }
  c10::intrusive_ptr<Options> getBackendOptions() override { return options_; }
  bool supportsSplitting() const override { return true; }
  bool supportsCoalescing() const override { return true; }
  void setTimeout(std::chrono::milliseconds t) override {
    options_->timeout = t;
    comm_->set_timeout(t);
  }

  c10::intrusive_ptr<c10d::Work> wrap(WorkPtr w, std::vector<at::Tensor> outs, c10d::OpType type, bool host_block = false) {
    return c10::make_intrusive<WorkWrapper>(std::move(w), std::move(outs), host_block, getRank(), type);
  }
  static at::Tensor& one(std::vector<at::Tensor>& v, const char* what) {
    TORCH_CHECK(v.size() == 1, what, ": exactly one tensor per call is supported, got ", v.size());
    return v[0];
  }
  OpOptions opt(Millis t) const { return with_timeout(t, options_->timeout); }

  c10::intrusive_ptr<c10d::Work> broadcast(std::vector<at::Tensor>& tensors, const c10d::BroadcastOptions& o) override {
    auto& t = one(tensors, "broadcast");
    return wrap(comm_->broadcast(t, static_cast<int>(o.rootRank), o.asyncOp, opt(o.timeout)), {t}, c10d::OpType::BROADCAST);
  }
  c10::intrusive_ptr<c10d::Work> allreduce(std::vector<at::Tensor>& tensors, const c10d::AllreduceOptions& o) override {
    auto& t = one(tensors, "allreduce");
    return wrap(comm_->all_reduce(t, from_c10d(o.reduceOp), o.asyncOp, opt(o.timeout)), {t}, c10d::OpType::ALLREDUCE);
  }
  c10::intrusive_ptr<c10d::Work> allreduce_coalesced(std::vector<at::Tensor>& tensors, const c10d::AllreduceCoalescedOptions& o) override {
    WorkPtr last;
    for (auto& t : tensors) {
      last = comm_->all_reduce(t, from_c10d(o.reduceOp), o.asyncOp, opt(o.timeout));
    }
    if (!last) {
      last = c10::make_intrusive<CompletedWork>();
    }
    return wrap(last, tensors, c10d::OpType::ALLREDUCE_COALESCED);
  }
  c10::intrusive_ptr<c10d::Work> reduce(std::vector<at::Tensor>& tensors, const c10d::ReduceOptions& o) override {
    auto& t = one(tensors, "reduce");
    return wrap(comm_->reduce(t, static_cast<int>(o.rootRank), from_c10d(o.reduceOp), o.asyncOp, opt(o.timeout)), {t}, c10d::OpType::REDUCE);
  }
  c10::intrusive_ptr<c10d::Work> allgather(std::vector<std::vector<at::Tensor>>& outs, std::vector<at::Tensor>& ins, const c10d::AllgatherOptions& o) override {
    TORCH_CHECK(outs.size() == 1, "allgather: exactly one output list is supported");
    auto& in = one(ins, "allgather");
    bool same = true;
    for (auto& t : outs[0]) {
      same = same && t.numel() == in.numel();
    }
    WorkPtr w = same ? comm_->all_gather(outs[0], in, o.asyncOp, opt(o.timeout))
                     : comm_->all_gather_v(outs[0], in, o.asyncOp, opt(o.timeout));
    return wrap(w, outs[0], c10d::OpType::ALLGATHER);
  }
  c10::intrusive_ptr<c10d::Work> _allgather_base(at::Tensor& out, at::Tensor& in, const c10d::AllgatherOptions& o) override {
    return wrap(comm_->all_gather_single(out, in, o.asyncOp, opt(o.timeout)), {out}, c10d::OpType::_ALLGATHER_BASE);
  }
  c10::intrusive_ptr<c10d::Work> allgather_into_tensor_coalesced(std::vector<at::Tensor>& outs, std::vector<at::Tensor>& ins, const c10d::AllgatherOptions& o) override {
    TORCH_CHECK(outs.size() == ins.size(), "allgather_into_tensor_coalesced: list lengths differ");
    WorkPtr last = c10::make_intrusive<CompletedWork>();
    for (size_t i = 0; i < ins.size(); ++i) {
      last = comm_->all_gather_single(outs[i], ins[i], o.asyncOp, opt(o.timeout));
    }
    return wrap(last, outs, c10d::OpType::COALESCED);
  }
  c10::intrusive_ptr<c10d::Work> gather(std::vector<std::vector<at::Tensor>>& outs, std::vector<at::Tensor>& ins, const c10d::GatherOptions& o) override {
    auto& in = one(ins, "gather");
    std::vector<at::Tensor> out_list = outs.empty() ? std::vector<at::Tensor>{} : outs[0];
    return wrap(comm_->gather(out_list, in, static_cast<int>(o.rootRank), o.asyncOp, opt(o.timeout)), out_list, c10d::OpType::GATHER);
  }
  c10::intrusive_ptr<c10d::Work> scatter(std::vector<at::Tensor>& outs, std::vector<std::vector<at::Tensor>>& ins, const c10d::ScatterOptions& o) override {
    auto& out = one(outs, "scatter");
    std::vector<at::Tensor> in_list = ins.empty() ? std::vector<at::Tensor>{} : ins[0];
    return wrap(comm_->scatter(out, in_list, static_cast<int>(o.rootRank), o.asyncOp, opt(o.timeout)), {out}, c10d::OpType::SCATTER);
  }
  c10::intrusive_ptr<c10d::Work> reduce_scatter(std::vector<at::Tensor>& outs, std::vector<std::vector<at::Tensor>>& ins, const c10d::ReduceScatterOptions& o) override {
    auto& out = one(outs, "reduce_scatter");
    TORCH_CHECK(ins.size() == 1, "reduce_scatter: exactly one input list is supported");
    bool same = true;
    for (auto& t : ins[0]) {
      same = same && t.numel() == out.numel();
    }
    WorkPtr w = same ? comm_->reduce_scatter(out, ins[0], from_c10d(o.reduceOp), o.asyncOp, opt(o.timeout))
                     : comm_->reduce_scatter_v(out, ins[0], from_c10d(o.reduceOp), o.asyncOp, opt(o.timeout));
    return wrap(w, {out}, c10d::OpType::REDUCE_SCATTER);
  }
  c10::intrusive_ptr<c10d::Work> _reduce_scatter_base(at::Tensor& out, at::Tensor& in, const c10d::ReduceScatterOptions& o) override {
    return wrap(comm_->reduce_scatter_single(out, in, from_c10d(o.reduceOp), o.asyncOp, opt(o.timeout)), {out}, c10d::OpType::_REDUCE_SCATTER_BASE);
  }
  c10::intrusive_ptr<c10d::Work> reduce_scatter_tensor_coalesced(std::vector<at::Tensor>& outs, std::vector<at::Tensor>& ins, const c10d::ReduceScatterOptions& o) override {
    TORCH_CHECK(outs.size() == ins.size(), "reduce_scatter_tensor_coalesced: list lengths differ");
    WorkPtr last = c10::make_intrusive<CompletedWork>();
    for (size_t i = 0; i < ins.size(); ++i) {
      last = comm_->reduce_scatter_single(outs[i], ins[i], from_c10d(o.reduceOp), o.asyncOp, opt(o.timeout));
    }
    return wrap(last, outs, c10d::OpType::COALESCED);
  }
  c10::intrusive_ptr<c10d::Work> alltoall_base(at::Tensor& out, at::Tensor& in, std::vector<int64_t>& os, std::vector<int64_t>& is, const c10d::AllToAllOptions& o) override {
    WorkPtr w = (os.empty() && is.empty())
        ? comm_->all_to_all_single(out, in, o.asyncOp, opt(o.timeout))
        : comm_->all_to_all_v_single(out, in, os, is, o.asyncOp, opt(o.timeout));
    return wrap(w, {out}, c10d::OpType::ALLTOALL_BASE);
  }
  c10::intrusive_ptr<c10d::Work> alltoall(std::vector<at::Tensor>& outs, std::vector<at::Tensor>& ins, const c10d::AllToAllOptions& o) override {
    return wrap(comm_->all_to_all(outs, ins, o.asyncOp, opt(o.timeout)), outs, c10d::OpType::ALLTOALL);
  }
  c10::intrusive_ptr<c10d::Work> barrier(const c10d::BarrierOptions& o) override {
    // A synchronous barrier also blocks the host, as torch.distributed users expect.
    return wrap(comm_->barrier(o.asyncOp, opt(o.timeout)), {}, c10d::OpType::BARRIER, /*host_block=*/!o.asyncOp);
  }

  c10::intrusive_ptr<c10d::Work> send(std::vector<at::Tensor>& tensors, int dst, int /*tag*/) override {
    auto& t = one(tensors, "send");
    if (coalescing_) {
      batch_->send(t, dst);
      return wrap(c10::make_intrusive<CompletedWork>(), {}, c10d::OpType::SEND);
    }
    return wrap(comm_->send(t, dst, true, opt(c10d::kUnsetTimeout)), {}, c10d::OpType::SEND);
  }
  c10::intrusive_ptr<c10d::Work> recv(std::vector<at::Tensor>& tensors, int src, int /*tag*/) override {
    auto& t = one(tensors, "recv");
    if (coalescing_) {
      batch_->recv(t, src);
      return wrap(c10::make_intrusive<CompletedWork>(), {t}, c10d::OpType::RECV);
    }
    return wrap(comm_->recv(t, src, true, opt(c10d::kUnsetTimeout)), {t}, c10d::OpType::RECV);
  }
  void startCoalescing() override {
    TORCH_CHECK(!coalescing_, "startCoalescing called twice");
    coalescing_ = true;
    batch_ = comm_->batch_op_create();
  }
  c10::intrusive_ptr<c10d::Work> endCoalescing() override {
    TORCH_CHECK(coalescing_, "endCoalescing without startCoalescing");
    coalescing_ = false;
    auto batch = std::move(batch_);
    std::vector<at::Tensor> outs;
    for (auto& op : batch->ops) {
      if (op.kind == P2PKind::RECV) {
        outs.push_back(op.tensor);
      }
    }
    WorkPtr w = batch->ops.empty() ? WorkPtr(c10::make_intrusive<CompletedWork>())
                                   : batch->issue(true, opt(c10d::kUnsetTimeout));
    return wrap(w, outs, c10d::OpType::COALESCED);
  }

  // Every rank reports to rank 0 with a one-element message; rank 0 names the
  // ranks that did not arrive in time, then releases everybody.
  void monitoredBarrier(const c10d::BarrierOptions& o, bool waitAllRanks) override {
    (void)waitAllRanks;
    const Millis t = (o.timeout == c10d::kUnsetTimeout) ? options_->timeout : o.timeout;
    at::Tensor token = at::zeros({1}, at::TensorOptions().dtype(at::kInt).device(comm_->get_device()));
    OpOptions oo;
    oo.timeout = t;
    oo.timeout_set = true;
    if (getRank() == 0) {
      std::vector<int> missing;
      for (int r = 1; r < getSize(); ++r) {
        try {
          comm_->recv(token, r, true, oo)->wait_blocking();
        } catch (const std::exception&) {
          missing.push_back(r);
        }
      }
      if (!missing.empty()) {
        std::ostringstream os;
        os << "monitoredBarrier: ranks";
        for (int r : missing) os << " " << r;
        os << " failed to arrive within " << t.count() << " ms";
        TORCH_CHECK(false, os.str());
      }
      for (int r = 1; r < getSize(); ++r) {
        comm_->send(token, r, true, oo)->wait_blocking();
      }
    } else {
      comm_->send(token, 0, true, oo)->wait_blocking();
      comm_->recv(token, 0, true, oo)->wait_blocking();
    }
  }

  void shutdown() override {
    if (!shut_) {
      shut_ = true;
      comm_->finalize();
    }
  }
  void abort() override { comm_->abort(); }

 private:
  std::shared_ptr<Comm> comm_;
  c10::intrusive_ptr<Options> options_;
  bool coalescing_ = false;
  std::shared_ptr<BatchSendRecv> batch_;
  bool shut_ = false;
};

} // namespace

void bind_c10d_wrapper(py::module_& m) {
  py::class_<BackendWrapper, c10::intrusive_ptr<BackendWrapper>, c10d::Backend>(m, "_BackendWrapper")
      .def(py::init([](std::shared_ptr<Comm> comm) { return c10::make_intrusive<BackendWrapper>(std::move(comm)); }),
           py::arg("comm"))
      .def("get_comm", &BackendWrapper::get_comm);
}

} // namespace b200c
