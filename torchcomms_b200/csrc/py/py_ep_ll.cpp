// Host side of the low-latency MoE dispatch / combine (`_comms.EpLlBuffer`):
// layout of the slot groups, count tables and expert-output tensor over one
// symmetric segment, tensor views, launches.
//
// Parity: comms/prims/collectives/link_ep/cpp/low_latency/LowLatencyRuntime.{h,cc}
// (buffer ownership, low_latency_dispatch / low_latency_combine entry points).
#include "py_common.hpp"

#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>

#include "../backends/cuda_backend.hpp"
#include "../kernels/moe_ep_ll.h"

namespace b200c {

namespace {

size_t align256(size_t v) { return (v + 255) / 256 * 256; }

class EpLlBuffer {
 public:
  EpLlBuffer(std::shared_ptr<CudaBackend> backend, int max_tokens, int hidden, int num_experts, int topk, bool fp8)
      : backend_(std::move(backend)), n_local_(1) {
    setup_dims(backend_->size(), max_tokens, hidden, num_experts, topk, fp8);
    c10::cuda::CUDAGuard g(backend_->device());
    // Zero-filled on every rank before anybody returns: the count tables read "no call yet".
    seg_ = backend_->symm().allocate(total_, false);
    std::vector<char*> bases(nranks_);
    for (int p = 0; p < nranks_; ++p) bases[p] = seg_->peer_ptrs[p];
    comms_ = {backend_->comm_dev()};
    eps_.resize(1);
    fill(eps_[0], backend_->rank(), bases);
  }
  // Emulation: `nranks` virtual ranks on the current device (kernel tests).
  EpLlBuffer(int nranks, int max_tokens, int hidden, int num_experts, int topk, bool fp8, double wait_ms)
      : n_local_(nranks) {
    setup_dims(nranks, max_tokens, hidden, num_experts, topk, fp8);
    const size_t flag_bytes = static_cast<size_t>(kFlagSets) * kMaxBlocks * kMaxRanks * sizeof(uint32_t);
    std::vector<char*> bases(nranks);
    auto zeroed = [this](size_t bytes) {
      void* p = nullptr;
      B200C_CUDA_CHECK(cudaMalloc(&p, bytes));
      B200C_CUDA_CHECK(cudaMemset(p, 0, bytes));
      emu_allocs_.push_back(p);
      return p;
    };
    std::vector<uint32_t*> flags(nranks), epochs(nranks);
    for (int r = 0; r < nranks; ++r) {
      bases[r] = static_cast<char*>(zeroed(total_));
      flags[r] = static_cast<uint32_t*>(zeroed(flag_bytes));
      epochs[r] = static_cast<uint32_t*>(zeroed(kFlagSets * kMaxBlocks * sizeof(uint32_t)));
    }
    B200C_CUDA_CHECK(cudaHostAlloc(reinterpret_cast<void**>(&status_host_), 64, cudaHostAllocMapped));
    std::memset(status_host_, 0, 64);
    uint32_t* sdev = nullptr;
    B200C_CUDA_CHECK(cudaHostGetDevicePointer(reinterpret_cast<void**>(&sdev), status_host_, 0));
    comms_.resize(nranks);
    eps_.resize(nranks);
    for (int r = 0; r < nranks; ++r) {
      CommDev& c = comms_[r];
      std::memset(&c, 0, sizeof(c));
      c.rank = r;
      c.nranks = nranks;
      for (int p = 0; p < nranks; ++p) c.flags[p] = flags[p];
      c.epochs = epochs[r];
      c.status = sdev;
      c.timeout_ns = static_cast<unsigned long long>(wait_ms * 1e6);
      fill(eps_[r], r, bases);
    }
  }
  ~EpLlBuffer() {
    for (void* p : local_allocs_) cudaFree(p);
    for (void* p : emu_allocs_) cudaFree(p);
    if (status_host_) cudaFreeHost(status_host_);
    if (seg_ && backend_ && backend_->symm_alive()) {
      try {
        backend_->symm().release(seg_);
      } catch (...) {
      }
    }
  }

  int local_experts() const { return num_experts_ / nranks_; }
  int rows_per_expert() const { return nranks_ * max_tokens_; }

  // Outputs per local rank: packed_x, packed_scales (fp8 only, else undefined), packed_src, packed_count, layout_range.
  std::vector<std::vector<at::Tensor>> dispatch(std::vector<at::Tensor> x, std::vector<at::Tensor> topk_idx) {
    TORCH_CHECK(static_cast<int>(x.size()) == n_local_ && static_cast<int>(topk_idx.size()) == n_local_,
                "one tensor per local rank expected");
    const int T = static_cast<int>(x[0].size(0));
    TORCH_CHECK(T <= max_tokens_, "dispatch: ", T, " tokens exceed the buffer capacity ", max_tokens_);
    const int64_t Le = local_experts(), R = rows_per_expert();
    std::vector<const void*> xp(n_local_);
    std::vector<const int*> ip(n_local_);
    std::vector<EpLlRecv> recv(n_local_);
    std::vector<std::vector<at::Tensor>> outs(n_local_);
    std::vector<at::Tensor> keep;
    for (int i = 0; i < n_local_; ++i) {
      TORCH_CHECK(x[i].is_cuda() && x[i].scalar_type() == at::kBFloat16 && x[i].is_contiguous() && x[i].dim() == 2 &&
                      x[i].size(0) == T && x[i].size(1) == hidden_,
                  "x: contiguous bf16 [tokens, hidden]");
      TORCH_CHECK(topk_idx[i].is_cuda() && topk_idx[i].scalar_type() == at::kInt && topk_idx[i].is_contiguous() &&
                      topk_idx[i].numel() == static_cast<int64_t>(T) * topk_,
                  "topk_idx: contiguous int32 [tokens, topk]");
      xp[i] = x[i].data_ptr();
      ip[i] = topk_idx[i].data_ptr<int>();
      auto opts = x[i].options();
      at::Tensor px = at::empty({Le, R, hidden_}, opts.dtype(fp8_ ? at::kFloat8_e4m3fn : at::kBFloat16));
      at::Tensor ps = fp8_ ? at::empty({Le, R, hidden_ / 128}, opts.dtype(at::kFloat)) : at::Tensor();
      at::Tensor src = at::empty({Le, R}, opts.dtype(at::kInt));
      at::Tensor count = at::empty({Le}, opts.dtype(at::kInt));
      at::Tensor range = at::empty({Le, nranks_}, opts.dtype(at::kLong));
      recv[i] = {px.data_ptr(), fp8_ ? ps.data_ptr<float>() : nullptr, src.data_ptr<int>(), count.data_ptr<int>(),
                 reinterpret_cast<long long*>(range.data_ptr<int64_t>())};
      outs[i] = {px, ps, src, count, range};
      keep.insert(keep.end(), {x[i], topk_idx[i], px, src, count, range});
      if (fp8_) keep.push_back(ps);
    }
    if (backend_) {
      backend_->run("ep_ll_dispatch/kernel", false, {}, keep, [&](cudaStream_t s) {
        comms_[0] = backend_->comm_dev();
        B200C_CUDA_CHECK(launch_ep_ll_dispatch(comms_.data(), eps_.data(), 0, xp.data(), ip.data(), recv.data(), T, s));
      });
    } else {
      B200C_CUDA_CHECK(launch_ep_ll_dispatch(comms_.data(), eps_.data(), n_local_, xp.data(), ip.data(), recv.data(), T,
                                             at::cuda::getCurrentCUDAStream().stream()));
    }
    return outs;
  }

  // out[t] = sum_k w[t, k] * (expert output row of (t, k)), the expert outputs being `view("out_x")` of every rank.
  void combine(std::vector<at::Tensor> out, std::vector<at::Tensor> topk_idx, std::vector<at::Tensor> topk_w,
               std::vector<at::Tensor> send_slot, std::vector<at::Tensor> begin) {
    TORCH_CHECK(static_cast<int>(out.size()) == n_local_ && static_cast<int>(topk_idx.size()) == n_local_ &&
                    static_cast<int>(topk_w.size()) == n_local_,
                "one tensor per local rank expected");
    TORCH_CHECK(send_slot.size() == begin.size() && (send_slot.empty() || static_cast<int>(send_slot.size()) == n_local_),
                "send_slot and begin go together, one per local rank");
    const int T = static_cast<int>(out[0].size(0));
    TORCH_CHECK(T <= max_tokens_, "combine: ", T, " tokens exceed the buffer capacity ", max_tokens_);
    std::vector<void*> op(n_local_);
    std::vector<const int*> ip(n_local_), sp(n_local_, nullptr), bp(n_local_, nullptr);
    std::vector<const float*> wp(n_local_);
    std::vector<at::Tensor> keep;
    for (int i = 0; i < n_local_; ++i) {
      TORCH_CHECK(out[i].is_cuda() && out[i].scalar_type() == at::kBFloat16 && out[i].is_contiguous() && out[i].dim() == 2 &&
                      out[i].size(0) == T && out[i].size(1) == hidden_,
                  "out: contiguous bf16 [tokens, hidden]");
      TORCH_CHECK(topk_idx[i].is_cuda() && topk_idx[i].scalar_type() == at::kInt && topk_idx[i].is_contiguous() &&
                      topk_idx[i].numel() == static_cast<int64_t>(T) * topk_,
                  "topk_idx: contiguous int32 [tokens, topk]");
      TORCH_CHECK(topk_w[i].is_cuda() && topk_w[i].scalar_type() == at::kFloat && topk_w[i].is_contiguous() &&
                      topk_w[i].numel() == static_cast<int64_t>(T) * topk_,
                  "topk_weights: contiguous float32 [tokens, topk]");
      op[i] = out[i].data_ptr();
      ip[i] = topk_idx[i].data_ptr<int>();
      wp[i] = topk_w[i].data_ptr<float>();
      keep.insert(keep.end(), {out[i], topk_idx[i], topk_w[i]});
      if (!send_slot.empty()) {
        TORCH_CHECK(send_slot[i].is_cuda() && send_slot[i].scalar_type() == at::kInt && send_slot[i].is_contiguous() &&
                        send_slot[i].numel() >= static_cast<int64_t>(T) * topk_,
                    "send_slot: contiguous int32 [tokens, topk]");
        TORCH_CHECK(begin[i].is_cuda() && begin[i].scalar_type() == at::kInt && begin[i].is_contiguous() &&
                        begin[i].numel() == num_experts_,
                    "begin: contiguous int32 [num_experts]");
        sp[i] = send_slot[i].data_ptr<int>();
        bp[i] = begin[i].data_ptr<int>();
        keep.insert(keep.end(), {send_slot[i], begin[i]});
      }
    }
    const int* const* spp = send_slot.empty() ? nullptr : sp.data();
    const int* const* bpp = send_slot.empty() ? nullptr : bp.data();
    if (backend_) {
      backend_->run("ep_ll_combine/kernel", false, {}, keep, [&](cudaStream_t s) {
        comms_[0] = backend_->comm_dev();
        B200C_CUDA_CHECK(launch_ep_ll_combine(comms_.data(), eps_.data(), 0, op.data(), ip.data(), wp.data(), T, spp, bpp, s));
      });
    } else {
      B200C_CUDA_CHECK(launch_ep_ll_combine(comms_.data(), eps_.data(), n_local_, op.data(), ip.data(), wp.data(), T, spp,
                                            bpp, at::cuda::getCurrentCUDAStream().stream()));
    }
  }

  at::Tensor view(int i, const std::string& what) {
    TORCH_CHECK(i >= 0 && i < n_local_, "bad local rank");
    const EpLlDev& e = eps_[i];
    auto opts = at::TensorOptions().device(at::kCUDA, at::cuda::current_device());
    if (what == "out_x") {
      return at::from_blob(e.out_x[e.rank], {local_experts(), rows_per_expert(), hidden_}, opts.dtype(at::kBFloat16));
    }
    if (what == "send_slot") return at::from_blob(e.send_slot, {max_tokens_, topk_}, opts.dtype(at::kInt));
    if (what == "begin") return at::from_blob(e.begin, {num_experts_}, opts.dtype(at::kInt));
    TORCH_CHECK(false, "unknown view '", what, "'");
  }
  std::vector<uint32_t> status() const {
    return status_host_ ? std::vector<uint32_t>(status_host_, status_host_ + 5) : std::vector<uint32_t>{};
  }
  size_t symmetric_bytes() const { return total_; }

 private:
  void setup_dims(int nranks, int max_tokens, int hidden, int num_experts, int topk, bool fp8) {
    TORCH_CHECK(hidden % 512 == 0, "hidden must be a multiple of 512");
    TORCH_CHECK(num_experts % nranks == 0, "num_experts must divide by the number of ranks");
    TORCH_CHECK(topk >= 1 && topk <= 32, "topk must be in 1..32");
    TORCH_CHECK(max_tokens >= 1, "max_tokens must be positive");
    nranks_ = nranks;
    max_tokens_ = max_tokens;
    hidden_ = hidden;
    num_experts_ = num_experts;
    topk_ = topk;
    fp8_ = fp8;
    const size_t slots = static_cast<size_t>(2) * (num_experts / nranks) * nranks * max_tokens;  // both parities
    size_t off = 0;
    auto take = [&off](size_t bytes) {
      const size_t at = off;
      off += align256(bytes);
      return at;
    };
    off_x_ = take(slots * hidden * (fp8 ? 1 : 2));
    off_scales_ = take(slots * (hidden / 128) * 4);
    off_src_ = take(slots * 4);
    off_arrived_ = take(slots * 4);
    counts_bytes_ = static_cast<size_t>(2) * num_experts * nranks * 8;
    off_counts_ = take(counts_bytes_);
    off_out_ = take(slots / 2 * hidden * 2);
    total_ = off;
  }
  void fill(EpLlDev& e, int rank, const std::vector<char*>& bases) {
    std::memset(&e, 0, sizeof(e));
    e.rank = rank;
    e.nranks = nranks_;
    e.num_experts = num_experts_;
    e.experts_per_rank = num_experts_ / nranks_;
    e.topk = topk_;
    e.hidden = hidden_;
    e.max_tokens = max_tokens_;
    e.fp8 = fp8_ ? 1 : 0;
    for (int p = 0; p < nranks_; ++p) {
      e.slot_x[p] = bases[p] + off_x_;
      e.slot_scales[p] = reinterpret_cast<float*>(bases[p] + off_scales_);
      e.slot_src[p] = reinterpret_cast<int*>(bases[p] + off_src_);
      e.slot_arrived[p] = reinterpret_cast<unsigned int*>(bases[p] + off_arrived_);
      e.counts[p] = reinterpret_cast<unsigned long long*>(bases[p] + off_counts_);
      e.out_x[p] = bases[p] + off_out_;
    }
    auto local = [this](size_t bytes) {
      void* p = nullptr;
      B200C_CUDA_CHECK(cudaMalloc(&p, bytes));
      B200C_CUDA_CHECK(cudaMemset(p, 0, bytes));
      local_allocs_.push_back(p);
      return p;
    };
    e.cnt = static_cast<int*>(local(sizeof(int) * 2 * num_experts_));
    e.call = static_cast<unsigned int*>(local(sizeof(unsigned int)));
    e.send_slot = static_cast<int*>(local(sizeof(int) * static_cast<size_t>(max_tokens_) * topk_));
    e.begin = static_cast<int*>(local(sizeof(int) * num_experts_));
  }

  std::shared_ptr<CudaBackend> backend_;
  std::shared_ptr<SymmSegment> seg_;
  int n_local_;
  int nranks_ = 1, max_tokens_ = 0, hidden_ = 0, num_experts_ = 0, topk_ = 0;
  bool fp8_ = true;
  size_t off_x_ = 0, off_scales_ = 0, off_src_ = 0, off_arrived_ = 0, off_counts_ = 0, off_out_ = 0, counts_bytes_ = 0, total_ = 0;
  std::vector<CommDev> comms_;
  std::vector<EpLlDev> eps_;
  std::vector<void*> local_allocs_, emu_allocs_;
  uint32_t* status_host_ = nullptr;
};

} // namespace

void bind_ep_ll(py::module_& m) {
  py::class_<EpLlBuffer>(m, "EpLlBuffer")
      .def(py::init([](std::shared_ptr<Backend> b, int max_tokens, int hidden, int num_experts, int topk, bool fp8) {
             auto cb = std::dynamic_pointer_cast<CudaBackend>(b);
             TORCH_CHECK(cb != nullptr, "EpLlBuffer needs a communicator on the CUDA backend");
             return std::make_unique<EpLlBuffer>(cb, max_tokens, hidden, num_experts, topk, fp8);
           }),
           py::arg("backend"), py::arg("max_tokens"), py::arg("hidden"), py::arg("num_experts"), py::arg("topk"),
           py::arg("fp8") = true)
      .def_static("emulated", [](int nranks, int max_tokens, int hidden, int num_experts, int topk, bool fp8, double wait_ms) {
        return std::make_unique<EpLlBuffer>(nranks, max_tokens, hidden, num_experts, topk, fp8, wait_ms);
      }, py::arg("nranks"), py::arg("max_tokens"), py::arg("hidden"), py::arg("num_experts"), py::arg("topk"),
         py::arg("fp8") = true, py::arg("wait_ms") = 2000.0)
      .def("dispatch", &EpLlBuffer::dispatch)
      .def("combine", &EpLlBuffer::combine, py::arg("out"), py::arg("topk_idx"), py::arg("topk_weights"),
           py::arg("send_slot") = std::vector<at::Tensor>{}, py::arg("begin") = std::vector<at::Tensor>{})
      .def("view", &EpLlBuffer::view, py::arg("local_rank"), py::arg("what"))
      .def("local_experts", &EpLlBuffer::local_experts)
      .def("rows_per_expert", &EpLlBuffer::rows_per_expert)
      .def("symmetric_bytes", &EpLlBuffer::symmetric_bytes)
      .def("status", &EpLlBuffer::status);
}

} // namespace b200c
