// Host side of MoE expert-parallel dispatch / combine: buffer layout over one
// symmetric segment, tensor views, launches (`_comms.EpBuffer`).
//
// Parity: comms/prims/collectives/link_ep/cpp/Buffer.{h,cc} (buffer ownership,
// intranode_dispatch / intranode_combine entry points).
#include "py_common.hpp"

#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>

#include "../backends/cuda_backend.hpp"
#include "../kernels/moe_ep.h"

namespace b200c {

namespace {

size_t align256(size_t v) { return (v + 255) / 256 * 256; }

class EpBuffer {
 public:
  // Real: one rank per process, memory from the communicator's symmetric allocator.
  EpBuffer(std::shared_ptr<CudaBackend> backend, int max_tokens, int hidden, int num_experts, int topk, bool fp8)
      : backend_(std::move(backend)), n_local_(1) {
    setup_dims(backend_->size(), max_tokens, hidden, num_experts, topk, fp8);
    c10::cuda::CUDAGuard g(backend_->device());
    seg_ = backend_->symm().allocate(total_, false);
    std::vector<char*> bases(nranks_);
    for (int p = 0; p < nranks_; ++p) bases[p] = seg_->peer_ptrs[p];
    comms_ = {backend_->comm_dev()};
    eps_.resize(1);
    fill(eps_[0], backend_->rank(), bases);
  }
  // Emulation: `nranks` virtual ranks on the current device (kernel tests).
  EpBuffer(int nranks, int max_tokens, int hidden, int num_experts, int topk, bool fp8, double wait_ms)
      : n_local_(nranks) {
    setup_dims(nranks, max_tokens, hidden, num_experts, topk, fp8);
    const size_t flag_bytes = static_cast<size_t>(kFlagSets) * kMaxBlocks * kMaxRanks * sizeof(uint32_t);
    std::vector<char*> bases(nranks);
    for (int r = 0; r < nranks; ++r) {
      void* p = nullptr;
      B200C_CUDA_CHECK(cudaMalloc(&p, total_));
      B200C_CUDA_CHECK(cudaMemset(p, 0, total_));
      emu_allocs_.push_back(p);
      bases[r] = static_cast<char*>(p);
      void* f = nullptr;
      B200C_CUDA_CHECK(cudaMalloc(&f, flag_bytes));
      B200C_CUDA_CHECK(cudaMemset(f, 0, flag_bytes));
      emu_allocs_.push_back(f);
      emu_flags_.push_back(static_cast<uint32_t*>(f));
      void* ep = nullptr;
      B200C_CUDA_CHECK(cudaMalloc(&ep, kFlagSets * kMaxBlocks * sizeof(uint32_t)));
      B200C_CUDA_CHECK(cudaMemset(ep, 0, kFlagSets * kMaxBlocks * sizeof(uint32_t)));
      emu_allocs_.push_back(ep);
      emu_epochs_.push_back(static_cast<uint32_t*>(ep));
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
      for (int p = 0; p < nranks; ++p) c.flags[p] = emu_flags_[p];
      c.epochs = emu_epochs_[r];
      c.status = sdev;
      c.timeout_ns = static_cast<unsigned long long>(wait_ms * 1e6);
      fill(eps_[r], r, bases);
    }
  }
  ~EpBuffer() {
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

  int rows() const { return nranks_ * max_tokens_; }

  void dispatch(std::vector<at::Tensor> x, std::vector<at::Tensor> topk_idx, std::vector<at::Tensor> topk_w) {
    check_lists(x, topk_idx, topk_w);
    const int T = static_cast<int>(x[0].size(0));
    std::vector<const void*> xp(n_local_);
    std::vector<const int*> ip(n_local_);
    std::vector<const float*> wp(n_local_);
    for (int i = 0; i < n_local_; ++i) {
      TORCH_CHECK(x[i].scalar_type() == at::kBFloat16 && x[i].is_contiguous() && x[i].size(0) == T && x[i].size(1) == hidden_,
                  "x: contiguous bf16 [tokens, hidden]");
      TORCH_CHECK(topk_idx[i].scalar_type() == at::kInt && topk_idx[i].is_contiguous() && topk_idx[i].numel() == T * topk_,
                  "topk_idx: contiguous int32 [tokens, topk]");
      TORCH_CHECK(topk_w[i].scalar_type() == at::kFloat && topk_w[i].is_contiguous() && topk_w[i].numel() == T * topk_,
                  "topk_weights: contiguous float32 [tokens, topk]");
      xp[i] = x[i].data_ptr();
      ip[i] = topk_idx[i].data_ptr<int>();
      wp[i] = topk_w[i].data_ptr<float>();
    }
    TORCH_CHECK(T <= max_tokens_, "dispatch: ", T, " tokens exceed the buffer capacity ", max_tokens_);
    if (backend_) {
      auto keep = std::vector<at::Tensor>{x[0], topk_idx[0], topk_w[0]};
      backend_->run("ep_dispatch/kernel", false, {}, keep, [&](cudaStream_t s) {
        comms_[0] = backend_->comm_dev();
        B200C_CUDA_CHECK(launch_ep_dispatch(comms_.data(), eps_.data(), 0, xp.data(), ip.data(), wp.data(), T, s));
      });
    } else {
      B200C_CUDA_CHECK(launch_ep_dispatch(comms_.data(), eps_.data(), n_local_, xp.data(), ip.data(), wp.data(), T,
                                          at::cuda::getCurrentCUDAStream().stream()));
    }
    last_tokens_ = T;
  }

  // `send_slot` (optional): handles of an earlier dispatch, int32 [tokens, nranks] as `view("send_slot")` gave them.
  // `topk_w_out` (optional): float32 [tokens, topk] outputs for the per-expert weights that travel back.
  void combine(std::vector<at::Tensor> out, std::vector<at::Tensor> weights, std::vector<at::Tensor> bias,
               std::vector<at::Tensor> send_slot, std::vector<at::Tensor> topk_w_out) {
    TORCH_CHECK(static_cast<int>(out.size()) == n_local_, "one output per local rank");
    const int T = static_cast<int>(out[0].size(0));
    std::vector<void*> op(n_local_);
    std::vector<const float*> wp(n_local_, nullptr);
    std::vector<const void*> bp(n_local_, nullptr);
    std::vector<const int*> sp(n_local_, nullptr);
    std::vector<float*> tp(n_local_, nullptr);
    TORCH_CHECK(send_slot.empty() || static_cast<int>(send_slot.size()) == n_local_, "one handle per local rank");
    TORCH_CHECK(topk_w_out.empty() || static_cast<int>(topk_w_out.size()) == n_local_, "one weight output per local rank");
    for (int i = 0; i < n_local_; ++i) {
      if (!send_slot.empty()) {
        TORCH_CHECK(send_slot[i].is_cuda() && send_slot[i].scalar_type() == at::kInt && send_slot[i].is_contiguous() &&
                        send_slot[i].numel() >= static_cast<int64_t>(T) * nranks_,
                    "send_slot: contiguous int32 [tokens, nranks]");
        sp[i] = send_slot[i].data_ptr<int>();
      }
      if (!topk_w_out.empty()) {
        TORCH_CHECK(topk_w_out[i].is_cuda() && topk_w_out[i].scalar_type() == at::kFloat && topk_w_out[i].is_contiguous() &&
                        topk_w_out[i].numel() == static_cast<int64_t>(T) * topk_,
                    "topk_w_out: contiguous float32 [tokens, topk]");
        tp[i] = topk_w_out[i].data_ptr<float>();
      }
      TORCH_CHECK(out[i].scalar_type() == at::kBFloat16 && out[i].is_contiguous() && out[i].size(1) == hidden_,
                  "out: contiguous bf16 [tokens, hidden]");
      op[i] = out[i].data_ptr();
      if (!weights.empty()) {
        TORCH_CHECK(weights[i].scalar_type() == at::kFloat && weights[i].is_contiguous() && weights[i].numel() == T * nranks_,
                    "weights: contiguous float32 [tokens, nranks]");
        wp[i] = weights[i].data_ptr<float>();
      }
      if (!bias.empty()) {
        TORCH_CHECK(bias[i].scalar_type() == at::kBFloat16 && bias[i].is_contiguous() && bias[i].numel() == out[i].numel(),
                    "bias: contiguous bf16 [tokens, hidden]");
        bp[i] = bias[i].data_ptr();
      }
    }
    const float* const* wpp = weights.empty() ? nullptr : wp.data();
    const void* const* bpp = bias.empty() ? nullptr : bp.data();
    const int* const* spp = send_slot.empty() ? nullptr : sp.data();
    float* const* tpp = topk_w_out.empty() ? nullptr : tp.data();
    if (backend_) {
      std::vector<at::Tensor> keep = out;
      keep.insert(keep.end(), send_slot.begin(), send_slot.end());
      keep.insert(keep.end(), topk_w_out.begin(), topk_w_out.end());
      backend_->run("ep_combine/kernel", false, {}, keep, [&](cudaStream_t s) {
        comms_[0] = backend_->comm_dev();
        B200C_CUDA_CHECK(launch_ep_combine(comms_.data(), eps_.data(), 0, op.data(), wpp, bpp, T, s, spp, tpp));
      });
    } else {
      B200C_CUDA_CHECK(launch_ep_combine(comms_.data(), eps_.data(), n_local_, op.data(), wpp, bpp, T,
                                         at::cuda::getCurrentCUDAStream().stream(), spp, tpp));
    }
  }

  // Cached dispatch: fills out[i] (bf16 [rows_i, hidden]) with the rows of the sources' `stage_x` named by
  // `recv_src` (handles of an earlier dispatch; empty = the last one's) and `num_rows` (0-d int32 device tensors).
  void pull(std::vector<at::Tensor> out, std::vector<at::Tensor> recv_src, std::vector<at::Tensor> num_rows) {
    TORCH_CHECK(static_cast<int>(out.size()) == n_local_, "one output per local rank");
    TORCH_CHECK(recv_src.empty() || static_cast<int>(recv_src.size()) == n_local_, "one handle per local rank");
    TORCH_CHECK(num_rows.size() == recv_src.size(), "recv_src and num_rows go together");
    std::vector<void*> op(n_local_);
    std::vector<const int*> sp(n_local_, nullptr), np(n_local_, nullptr);
    int out_rows = rows();
    for (int i = 0; i < n_local_; ++i) {
      TORCH_CHECK(out[i].is_cuda() && out[i].scalar_type() == at::kBFloat16 && out[i].is_contiguous() && out[i].dim() == 2 &&
                      out[i].size(1) == hidden_,
                  "out: contiguous bf16 [rows, hidden]");
      out_rows = std::min<int>(out_rows, static_cast<int>(out[i].size(0)));
      op[i] = out[i].data_ptr();
      if (!recv_src.empty()) {
        TORCH_CHECK(recv_src[i].is_cuda() && recv_src[i].scalar_type() == at::kInt && recv_src[i].is_contiguous() &&
                        recv_src[i].numel() >= out[i].size(0),
                    "recv_src: contiguous int32 with one entry per output row");
        TORCH_CHECK(num_rows[i].is_cuda() && num_rows[i].scalar_type() == at::kInt && num_rows[i].numel() == 1,
                    "num_rows: one int32 on the device");
        sp[i] = recv_src[i].data_ptr<int>();
        np[i] = num_rows[i].data_ptr<int>();
      }
    }
    const int* const* spp = recv_src.empty() ? nullptr : sp.data();
    const int* const* npp = recv_src.empty() ? nullptr : np.data();
    if (backend_) {
      std::vector<at::Tensor> keep = out;
      keep.insert(keep.end(), recv_src.begin(), recv_src.end());
      keep.insert(keep.end(), num_rows.begin(), num_rows.end());
      backend_->run("ep_pull/kernel", false, {}, keep, [&](cudaStream_t s) {
        comms_[0] = backend_->comm_dev();
        B200C_CUDA_CHECK(launch_ep_pull(comms_.data(), eps_.data(), 0, op.data(), spp, npp, out_rows, s));
      });
    } else {
      B200C_CUDA_CHECK(launch_ep_pull(comms_.data(), eps_.data(), n_local_, op.data(), spp, npp, out_rows,
                                      at::cuda::getCurrentCUDAStream().stream()));
    }
  }

  // Views of local rank `i`'s buffers (i = 0 outside emulation).
  at::Tensor view(int i, const std::string& what) {
    TORCH_CHECK(i >= 0 && i < n_local_, "bad local rank");
    const EpDev& e = eps_[i];
    const int r = e.rank;
    auto opts = at::TensorOptions().device(at::kCUDA, at::cuda::current_device());
    const int64_t R = rows();
    if (what == "recv_x") {
      return fp8_ ? at::from_blob(e.recv_x[r], {R, hidden_}, opts.dtype(at::kFloat8_e4m3fn))
                  : at::from_blob(e.recv_x[r], {R, hidden_}, opts.dtype(at::kBFloat16));
    }
    if (what == "recv_scales") return at::from_blob(e.recv_scales[r], {R, hidden_ / 128}, opts.dtype(at::kFloat));
    if (what == "recv_src") return at::from_blob(e.recv_src[r], {R}, opts.dtype(at::kInt));
    if (what == "recv_topk_idx") return at::from_blob(e.recv_topk_idx[r], {R, topk_}, opts.dtype(at::kInt));
    if (what == "recv_topk_weights") return at::from_blob(e.recv_topk_w[r], {R, topk_}, opts.dtype(at::kFloat));
    if (what == "combine_x") return at::from_blob(e.combine_x[r], {R, hidden_}, opts.dtype(at::kBFloat16));
    if (what == "stage_x") return at::from_blob(e.stage_x[r], {max_tokens_, hidden_}, opts.dtype(at::kBFloat16));
    if (what == "combine_topk_weights") return at::from_blob(e.comb_topk_w[r], {R, topk_}, opts.dtype(at::kFloat));
    if (what == "recv_info") return at::from_blob(e.recv_info, {1 + nranks_}, opts.dtype(at::kInt));
    if (what == "send_slot") return at::from_blob(e.send_slot, {max_tokens_, nranks_}, opts.dtype(at::kInt));
    TORCH_CHECK(false, "unknown view '", what, "'");
  }
  std::vector<uint32_t> status() const {
    return status_host_ ? std::vector<uint32_t>(status_host_, status_host_ + 5) : std::vector<uint32_t>{};
  }

 private:
  void setup_dims(int nranks, int max_tokens, int hidden, int num_experts, int topk, bool fp8) {
    TORCH_CHECK(hidden % 512 == 0, "hidden must be a multiple of 512");
    TORCH_CHECK(num_experts % nranks == 0, "num_experts must divide by the number of ranks");
    TORCH_CHECK(topk >= 1 && topk <= 32, "topk must be in 1..32");
    nranks_ = nranks;
    max_tokens_ = max_tokens;
    hidden_ = hidden;
    num_experts_ = num_experts;
    topk_ = topk;
    fp8_ = fp8;
    const size_t R = static_cast<size_t>(nranks) * max_tokens;
    size_t off = 0;
    auto take = [&off](size_t bytes) {
      const size_t at = off;
      off += align256(bytes);
      return at;
    };
    off_x_ = take(R * hidden * (fp8 ? 1 : 2));
    off_scales_ = take(R * (hidden / 128) * 4);
    off_src_ = take(R * 4);
    off_idx_ = take(R * topk * 4);
    off_w_ = take(R * topk * 4);
    off_count_ = take(static_cast<size_t>(nranks) * nranks * 8);
    off_combine_ = take(R * hidden * 2);
    off_stage_ = take(static_cast<size_t>(max_tokens) * hidden * 2);
    off_comb_w_ = take(R * topk * 4);
    total_ = off;
  }
  void fill(EpDev& e, int rank, const std::vector<char*>& bases) {
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
      e.recv_x[p] = bases[p] + off_x_;
      e.recv_scales[p] = reinterpret_cast<float*>(bases[p] + off_scales_);
      e.recv_src[p] = reinterpret_cast<int*>(bases[p] + off_src_);
      e.recv_topk_idx[p] = reinterpret_cast<int*>(bases[p] + off_idx_);
      e.recv_topk_w[p] = reinterpret_cast<float*>(bases[p] + off_w_);
      e.count_matrix[p] = reinterpret_cast<long long*>(bases[p] + off_count_);
      e.combine_x[p] = bases[p] + off_combine_;
      e.stage_x[p] = bases[p] + off_stage_;
      e.comb_topk_w[p] = reinterpret_cast<float*>(bases[p] + off_comb_w_);
    }
    auto local = [this](size_t bytes) {
      void* p = nullptr;
      B200C_CUDA_CHECK(cudaMalloc(&p, bytes));
      B200C_CUDA_CHECK(cudaMemset(p, 0, bytes));
      local_allocs_.push_back(p);
      return p;
    };
    e.cnt = static_cast<int*>(local(sizeof(int) * kMaxRanks));
    e.cursor = static_cast<int*>(local(sizeof(int) * kMaxRanks));
    e.base = static_cast<long long*>(local(sizeof(long long) * kMaxRanks));
    e.recv_info = static_cast<int*>(local(sizeof(int) * (1 + kMaxRanks)));
    e.send_slot = static_cast<int*>(local(sizeof(int) * static_cast<size_t>(max_tokens_) * nranks_));
  }
  void check_lists(const std::vector<at::Tensor>& a, const std::vector<at::Tensor>& b, const std::vector<at::Tensor>& c) const {
    TORCH_CHECK(static_cast<int>(a.size()) == n_local_ && static_cast<int>(b.size()) == n_local_ &&
                    static_cast<int>(c.size()) == n_local_,
                "one tensor per local rank expected");
  }

  std::shared_ptr<CudaBackend> backend_;
  std::shared_ptr<SymmSegment> seg_;
  int n_local_;
  int nranks_ = 1, max_tokens_ = 0, hidden_ = 0, num_experts_ = 0, topk_ = 0;
  bool fp8_ = true;
  size_t off_x_ = 0, off_scales_ = 0, off_src_ = 0, off_idx_ = 0, off_w_ = 0, off_count_ = 0, off_combine_ = 0, off_stage_ = 0, off_comb_w_ = 0, total_ = 0;
  std::vector<CommDev> comms_;
  std::vector<EpDev> eps_;
  std::vector<void*> local_allocs_, emu_allocs_;
  std::vector<uint32_t*> emu_flags_, emu_epochs_;
  uint32_t* status_host_ = nullptr;
  int last_tokens_ = 0;
};

} // namespace

void bind_ep(py::module_& m) {
  py::class_<EpBuffer>(m, "EpBuffer")
      .def(py::init([](std::shared_ptr<Backend> b, int max_tokens, int hidden, int num_experts, int topk, bool fp8) {
             auto cb = std::dynamic_pointer_cast<CudaBackend>(b);
             TORCH_CHECK(cb != nullptr, "EpBuffer needs a communicator on the CUDA backend");
             return std::make_unique<EpBuffer>(cb, max_tokens, hidden, num_experts, topk, fp8);
           }),
           py::arg("backend"), py::arg("max_tokens"), py::arg("hidden"), py::arg("num_experts"), py::arg("topk"),
           py::arg("fp8") = true)
      .def_static("emulated", [](int nranks, int max_tokens, int hidden, int num_experts, int topk, bool fp8, double wait_ms) {
        return std::make_unique<EpBuffer>(nranks, max_tokens, hidden, num_experts, topk, fp8, wait_ms);
      }, py::arg("nranks"), py::arg("max_tokens"), py::arg("hidden"), py::arg("num_experts"), py::arg("topk"),
         py::arg("fp8") = true, py::arg("wait_ms") = 2000.0)
      .def("dispatch", &EpBuffer::dispatch)
      .def("combine", &EpBuffer::combine, py::arg("out"), py::arg("weights") = std::vector<at::Tensor>{},
           py::arg("bias") = std::vector<at::Tensor>{}, py::arg("send_slot") = std::vector<at::Tensor>{},
           py::arg("topk_w_out") = std::vector<at::Tensor>{})
      .def("pull", &EpBuffer::pull, py::arg("out"), py::arg("recv_src") = std::vector<at::Tensor>{},
           py::arg("num_rows") = std::vector<at::Tensor>{})
      .def("view", &EpBuffer::view, py::arg("local_rank"), py::arg("what"))
      .def("rows", &EpBuffer::rows)
      .def("status", &EpBuffer::status);

  m.def("ep_layout", [](const at::Tensor& topk_idx, int num_experts, int nranks) {
    TORCH_CHECK(topk_idx.is_cuda() && topk_idx.scalar_type() == at::kInt && topk_idx.is_contiguous() && topk_idx.dim() == 2,
                "topk_idx: contiguous int32 CUDA tensor [tokens, topk]");
    c10::cuda::CUDAGuard g(topk_idx.device());
    const int T = static_cast<int>(topk_idx.size(0)), K = static_cast<int>(topk_idx.size(1));
    auto opts = topk_idx.options();
    at::Tensor per_rank = at::empty({nranks}, opts), per_expert = at::empty({num_experts}, opts);
    at::Tensor in_rank = at::empty({T, nranks}, opts);
    B200C_CUDA_CHECK(launch_ep_layout(topk_idx.data_ptr<int>(), T, K, num_experts, nranks, per_rank.data_ptr<int>(),
                                      per_expert.data_ptr<int>(), in_rank.data_ptr<int>(),
                                      at::cuda::getCurrentCUDAStream(topk_idx.device().index()).stream()));
    return std::make_tuple(per_rank, per_expert, in_rank);
  });
}

} // namespace b200c
