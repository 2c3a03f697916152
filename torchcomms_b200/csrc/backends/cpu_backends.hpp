// CPU-side backends: "fake" (no transport, for unit tests) and "gloo"
// (TCP full mesh through the c10d gloo process group).
//
// Parity: comms/torchcomms/fake/TorchCommFake.hpp:13 and
// comms/torchcomms/gloo/TorchCommGloo.hpp:22-224, TorchCommGloo.cpp:85-190,
// 346-441 (PREMUL_SUM = pre-multiply, AVG = sum then divide, bitwise ops for
// integral types, CUDA tensors staged through the host),
// gloo/TorchCommGlooReconfigure.cpp (elastic membership).
#pragma once

#include <torch/csrc/distributed/c10d/Backend.hpp>

#include "../core/comm.hpp"

namespace b200c {

// A backend that moves no data. Rank and size default to 0 of 1 and can be
// overridden with hints {"fake_rank", "fake_size"}. Every call is appended to
// `calls` so tests can assert on what the facade forwarded.
class B200C_API FakeBackend : public Backend {
 public:
  void init(at::Device device, const std::string& name, const CommOptions& opts) override;
  void finalize() override;
  int rank() const override { return rank_; }
  int size() const override { return size_; }
  std::string backend_name() const override { return "fake"; }
  std::string comm_name() const override { return name_; }
  at::Device device() const override { return device_; }
  const CommOptions& options() const override { return opts_; }

  WorkPtr send(const at::Tensor&, int, bool, const OpOptions&) override { return done("send"); }
  WorkPtr recv(at::Tensor&, int, bool, const OpOptions&) override { return done("recv"); }
  WorkPtr batch_op_issue(const std::vector<P2POp>&, bool, const OpOptions&) override { return done("batch_op_issue"); }
  WorkPtr broadcast(at::Tensor&, int, bool, const OpOptions&) override { return done("broadcast"); }
  WorkPtr all_reduce(at::Tensor&, const ReduceOp&, bool, const OpOptions&) override { return done("all_reduce"); }
  WorkPtr reduce(const at::Tensor&, int, const ReduceOp&, bool, const OpOptions&) override { return done("reduce"); }
  WorkPtr all_gather(const std::vector<at::Tensor>& outs, const at::Tensor& in, bool, const OpOptions&) override;
  WorkPtr all_gather_v(const std::vector<at::Tensor>& outs, const at::Tensor& in, bool a, const OpOptions& o) override { return all_gather(outs, in, a, o); }
  WorkPtr all_gather_single(at::Tensor& out, const at::Tensor& in, bool, const OpOptions&) override;
  WorkPtr reduce_scatter(at::Tensor& out, const std::vector<at::Tensor>& ins, const ReduceOp&, bool, const OpOptions&) override;
  WorkPtr reduce_scatter_v(at::Tensor& out, const std::vector<at::Tensor>& ins, const ReduceOp& op, bool a, const OpOptions& o) override { return reduce_scatter(out, ins, op, a, o); }
  WorkPtr reduce_scatter_single(at::Tensor& out, const at::Tensor& in, const ReduceOp&, bool, const OpOptions&) override;
  WorkPtr all_to_all_single(at::Tensor& out, const at::Tensor& in, bool, const OpOptions&) override;
  WorkPtr all_to_all_v_single(at::Tensor& out, const at::Tensor& in, const std::vector<int64_t>&, const std::vector<int64_t>&, bool, const OpOptions&) override;
  WorkPtr all_to_all(const std::vector<at::Tensor>& outs, const std::vector<at::Tensor>& ins, bool, const OpOptions&) override;
  WorkPtr barrier(bool, const OpOptions&) override { return done("barrier"); }
  WorkPtr scatter(at::Tensor& out, const std::vector<at::Tensor>& ins, int root, bool, const OpOptions&) override;
  WorkPtr gather(const std::vector<at::Tensor>& outs, const at::Tensor& in, int root, bool, const OpOptions&) override;
  std::shared_ptr<Backend> split(const std::vector<int>& ranks, const std::string& name, const CommOptions& opts) override;
  void set_timeout(Millis t) override { opts_.timeout = t; }
  bool supports_reconfigure() const override { return true; }
  InitHandle get_init_handle() const override { return "fake:" + std::to_string(rank_); }
  WorkPtr reconfigure(const ReconfigureOptions& o) override;
  void abort() override { aborted_ = true; run_abort_hooks(); }
  bool is_aborted() const override { return aborted_; }
  bool is_abort_supported() const override { return true; }
  // A host-memory window for the single rank: enough to exercise the window API's rules without a GPU.
  std::shared_ptr<Window> new_window(const std::optional<at::Tensor>& tensor) override;

  std::vector<std::string> calls;

 private:
  WorkPtr done(const char* what);
  int rank_ = 0, size_ = 1;
  std::string name_;
  at::Device device_{at::kCPU};
  CommOptions opts_;
  bool aborted_ = false;
  bool initialized_ = false;
};

// Builds the c10d gloo process group. Installed by the Python module at
// import time (the gloo headers are not shipped with PyTorch wheels, so the
// object is created through torch.distributed and handed over as a
// c10d::Backend).
using GlooPgMaker = std::function<c10::intrusive_ptr<c10d::Backend>(
    const c10::intrusive_ptr<c10d::Store>& store, int rank, int size, Millis timeout)>;
void set_gloo_pg_maker(GlooPgMaker maker);

class GlooBackend : public Backend {
 public:
  ~GlooBackend() override;
  void init(at::Device device, const std::string& name, const CommOptions& opts) override;
  void finalize() override;
  int rank() const override { return rank_; }
  int size() const override { return size_; }
  std::string backend_name() const override { return "gloo"; }
  std::string comm_name() const override { return name_; }
  at::Device device() const override { return device_; }
  const CommOptions& options() const override { return opts_; }

  WorkPtr send(const at::Tensor& t, int dst, bool async_op, const OpOptions& o) override;
  WorkPtr recv(at::Tensor& t, int src, bool async_op, const OpOptions& o) override;
  WorkPtr batch_op_issue(const std::vector<P2POp>& ops, bool async_op, const OpOptions& o) override;
  WorkPtr broadcast(at::Tensor& t, int root, bool async_op, const OpOptions& o) override;
  WorkPtr all_reduce(at::Tensor& t, const ReduceOp& op, bool async_op, const OpOptions& o) override;
  WorkPtr reduce(const at::Tensor& t, int root, const ReduceOp& op, bool async_op, const OpOptions& o) override;
  WorkPtr all_gather(const std::vector<at::Tensor>& outs, const at::Tensor& in, bool async_op, const OpOptions& o) override;
  WorkPtr all_gather_v(const std::vector<at::Tensor>& outs, const at::Tensor& in, bool async_op, const OpOptions& o) override;
  WorkPtr all_gather_single(at::Tensor& out, const at::Tensor& in, bool async_op, const OpOptions& o) override;
  WorkPtr reduce_scatter(at::Tensor& out, const std::vector<at::Tensor>& ins, const ReduceOp& op, bool async_op, const OpOptions& o) override;
  WorkPtr reduce_scatter_v(at::Tensor& out, const std::vector<at::Tensor>& ins, const ReduceOp& op, bool async_op, const OpOptions& o) override;
  WorkPtr reduce_scatter_single(at::Tensor& out, const at::Tensor& in, const ReduceOp& op, bool async_op, const OpOptions& o) override;
  WorkPtr all_to_all_single(at::Tensor& out, const at::Tensor& in, bool async_op, const OpOptions& o) override;
  WorkPtr all_to_all_v_single(at::Tensor& out, const at::Tensor& in, const std::vector<int64_t>& out_splits, const std::vector<int64_t>& in_splits, bool async_op, const OpOptions& o) override;
  WorkPtr all_to_all(const std::vector<at::Tensor>& outs, const std::vector<at::Tensor>& ins, bool async_op, const OpOptions& o) override;
  WorkPtr barrier(bool async_op, const OpOptions& o) override;
  WorkPtr scatter(at::Tensor& out, const std::vector<at::Tensor>& ins, int root, bool async_op, const OpOptions& o) override;
  WorkPtr gather(const std::vector<at::Tensor>& outs, const at::Tensor& in, int root, bool async_op, const OpOptions& o) override;
  std::shared_ptr<Backend> split(const std::vector<int>& ranks, const std::string& name, const CommOptions& opts) override;
  std::shared_ptr<Backend> create_pair_comm(int peer, const std::string& name) override;
  void set_timeout(Millis t) override { opts_.timeout = t; }

  bool supports_reconfigure() const override { return true; }
  InitHandle get_init_handle() const override;
  WorkPtr reconfigure(const ReconfigureOptions& o) override;
  void abort() override;
  bool is_aborted() const override { return aborted_; }
  bool is_abort_supported() const override { return true; }

 private:
  friend class GlooWork;
  void connect(const c10::intrusive_ptr<c10d::Store>& store, int rank, int size);
  void ensure_ready() const;
  Millis effective_timeout(const OpOptions& o) const { return o.timeout_set ? o.timeout : opts_.timeout; }
  // Wraps a c10d work plus host-side post-processing into a Work.
  WorkPtr finish(c10::intrusive_ptr<c10d::Work> inner, std::function<void()> post, bool async_op, const OpOptions& o);
  void on_failure(const std::string& what, bool timed_out);

  int rank_ = -1, size_ = -1;
  std::string name_;
  at::Device device_{at::kCPU};
  CommOptions opts_;
  c10::intrusive_ptr<c10d::Store> store_;
  c10::intrusive_ptr<c10d::Backend> pg_;
  uint64_t split_counter_ = 0;
  uint64_t p2p_tag_ = 0;
  std::string handle_token_;
  bool aborted_ = false;
  bool finalized_ = false;
};

} // namespace b200c
