// Bindings of the tensor-parallel fused layers: all-gather -> GEMM and
// GEMM -> reduce-scatter as single tcgen05 kernels over peer memory.
#include "py_common.hpp"

#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>

#include <cstring>

#include "../backends/cuda_backend.hpp"
#include "../cuda/driver_api.hpp"
#include "../kernels/tc_gemm.h"

namespace b200c {

namespace {

size_t align256(size_t v) {
  return (v + 255) / 256 * 256;
}

// Owns the buffers of one layer shape. With a backend the activations /
// partial sums live in the communicator's symmetric memory; without one
// (single rank on the current device) in ordinary device memory, which is
// what the numerics tests and single-GPU profiles use.
class TpLayer {
 public:
  // kind: "ag_gemm" (rows = m_local per rank, cols = k) or "gemm_rs"
  // (rows = m over all ranks, cols = n).
  // fp8: operands are e4m3 with one fp32 scale per row (token) and per output channel; the all-gather layer
  // then carries [m_local] row scales behind its activation shard.
  TpLayer(std::shared_ptr<CudaBackend> backend, const std::string& kind, int rows, int cols, double wait_ms, bool fp8)
      : backend_(std::move(backend)), ag_(kind == "ag_gemm"), rows_(rows), cols_(cols), fp8_(fp8) {
    TORCH_CHECK(kind == "ag_gemm" || kind == "gemm_rs", "kind must be 'ag_gemm' or 'gemm_rs'");
    nranks_ = backend_ ? backend_->size() : 1;
    rank_ = backend_ ? backend_->rank() : 0;
    if (ag_) {
      TORCH_CHECK(rows % 128 == 0 && cols % (fp8 ? 128 : 64) == 0,
                  "ag_gemm: m_local % 128 == 0 and k % 64 == 0 (fp8: k % 128 == 0) required");
      data_bytes_ = align256(static_cast<size_t>(rows) * cols * (fp8 ? 1 : 2));
      flag_bytes_ = fp8 ? align256(static_cast<size_t>(rows) * 4) : 0;   // fp8: the row scales sit here
    } else {
      TORCH_CHECK(rows % (128 * nranks_) == 0 && cols % 256 == 0, "gemm_rs: m % (128*nranks) == 0 and n % 256 == 0 required");
      data_bytes_ = align256(static_cast<size_t>(rows) * cols * 2);  // [nranks, m/nranks, n]
      flag_bytes_ = align256(static_cast<size_t>(rows / nranks_ / 128) * (cols / 256) * nranks_ * 4);
    }
    const size_t total = data_bytes_ + flag_bytes_;
    if (backend_) {
      c10::cuda::CUDAGuard g(backend_->device());
      seg_ = backend_->symm().allocate(total, false);
      for (int p = 0; p < nranks_; ++p) bases_.push_back(seg_->peer_ptrs[p]);
    } else {
      void* p = nullptr;
      B200C_CUDA_CHECK(cudaMalloc(&p, total));
      B200C_CUDA_CHECK(cudaMemset(p, 0, total));
      local_.push_back(p);
      bases_.push_back(static_cast<char*>(p));
      const size_t fb = static_cast<size_t>(kFlagSets) * kMaxBlocks * kMaxRanks * sizeof(uint32_t);
      void* f = nullptr;
      B200C_CUDA_CHECK(cudaMalloc(&f, fb));
      B200C_CUDA_CHECK(cudaMemset(f, 0, fb));
      local_.push_back(f);
      void* ep = nullptr;
      B200C_CUDA_CHECK(cudaMalloc(&ep, kFlagSets * kMaxBlocks * sizeof(uint32_t)));
      B200C_CUDA_CHECK(cudaMemset(ep, 0, kFlagSets * kMaxBlocks * sizeof(uint32_t)));
      local_.push_back(ep);
      B200C_CUDA_CHECK(cudaHostAlloc(reinterpret_cast<void**>(&status_host_), 64, cudaHostAllocMapped));
      std::memset(status_host_, 0, 64);
      uint32_t* sdev = nullptr;
      B200C_CUDA_CHECK(cudaHostGetDevicePointer(reinterpret_cast<void**>(&sdev), status_host_, 0));
      std::memset(&solo_, 0, sizeof(solo_));
      solo_.rank = 0;
      solo_.nranks = 1;
      solo_.flags[0] = static_cast<uint32_t*>(f);
      solo_.epochs = static_cast<uint32_t*>(ep);
      solo_.status = sdev;
      solo_.timeout_ns = static_cast<unsigned long long>(wait_ms * 1e6);
    }
    const size_t ctrl_bytes = tp_ctrl_words(ag_ ? rows * nranks_ : 0) * sizeof(uint32_t);
    void* ctrl = nullptr;
    B200C_CUDA_CHECK(cudaMalloc(&ctrl, ctrl_bytes));
    B200C_CUDA_CHECK(cudaMemset(ctrl, 0, ctrl_bytes));
    local_.push_back(ctrl);
    ctrl_ = static_cast<uint32_t*>(ctrl);
    if (ag_ && nranks_ > 1) {
      void* full = nullptr;
      B200C_CUDA_CHECK(cudaMalloc(&full, static_cast<size_t>(rows) * nranks_ * cols * (fp8 ? 1 : 2)));
      local_.push_back(full);
      x_full_ = full;
    }
    if (!ag_ && nranks_ > 1) {
      // partial tiles bound for other ranks are staged here before the forward warps push them
      void* st = nullptr;
      B200C_CUDA_CHECK(cudaMalloc(&st, static_cast<size_t>(rows) * cols * 2));
      local_.push_back(st);
      send_stage_ = st;
    }
    if (ag_ && fp8) {
      void* sf = nullptr;
      B200C_CUDA_CHECK(cudaMalloc(&sf, static_cast<size_t>(rows) * nranks_ * 4));
      B200C_CUDA_CHECK(cudaMemset(sf, 0, static_cast<size_t>(rows) * nranks_ * 4));
      local_.push_back(sf);
      scale_full_ = static_cast<float*>(sf);
    }
    B200C_CUDA_CHECK(cudaDeviceSynchronize());
  }

  ~TpLayer() {
    for (void* p : local_) cudaFree(p);
    if (status_host_) cudaFreeHost(status_host_);
    if (seg_ && backend_ && backend_->symm_alive()) {
      try {
        backend_->symm().release(seg_);
      } catch (...) {
      }
    }
  }

  // ag_gemm: this rank's activation shard [m_local, k] in symmetric memory;
  // the producer of the activations writes here.
  at::Tensor input() {
    TORCH_CHECK(ag_, "input(): ag_gemm layers only");
    auto opts = at::TensorOptions().device(at::kCUDA, at::cuda::current_device()).dtype(fp8_ ? at::kFloat8_e4m3fn : at::kBFloat16);
    return at::from_blob(bases_[rank_], {rows_, cols_}, opts);
  }
  // fp8 ag_gemm: this rank's [m_local] fp32 row scales, in symmetric memory behind the shard.
  at::Tensor input_scales() {
    TORCH_CHECK(ag_ && fp8_, "input_scales(): fp8 ag_gemm layers only");
    auto opts = at::TensorOptions().device(at::kCUDA, at::cuda::current_device()).dtype(at::kFloat);
    return at::from_blob(bases_[rank_] + data_bytes_, {rows_}, opts);
  }

  // ag_gemm: y[nranks*m_local, n] = all_gather(input()) @ w[n, k]^T
  at::Tensor ag_gemm(const at::Tensor& w, const c10::optional<at::Tensor>& scale_w) {
    TORCH_CHECK(ag_, "not an ag_gemm layer");
    TORCH_CHECK(w.is_cuda() && w.is_contiguous() && w.scalar_type() == (fp8_ ? at::kFloat8_e4m3fn : at::kBFloat16) &&
                    w.dim() == 2 && w.size(1) == cols_,
                "w: contiguous [n, k] of the layer's operand type");
    TORCH_CHECK(w.size(0) % 256 == 0, "n must be a multiple of 256");
    TORCH_CHECK(!fp8_ || (scale_w.has_value() && scale_w->is_cuda() && scale_w->scalar_type() == at::kFloat &&
                          scale_w->is_contiguous() && scale_w->numel() == w.size(0)),
                "fp8: scale_w must be contiguous fp32 [n]");
    c10::cuda::CUDAGuard g(w.device());
    at::Tensor y = at::empty({static_cast<int64_t>(rows_) * nranks_, w.size(0)}, w.options().dtype(at::kBFloat16));
    AgGemmArgs a{};
    if (fp8_) {
      a.fp8 = 1;
      for (int p = 0; p < nranks_; ++p) a.scale_x_shards[p] = reinterpret_cast<const float*>(bases_[p] + data_bytes_);
      a.scale_x_full = scale_full_;
      a.scale_w = scale_w->data_ptr<float>();
    }
    for (int p = 0; p < nranks_; ++p) a.x_shards[p] = bases_[p];
    a.x_full = x_full_ ? x_full_ : bases_[rank_];  // single rank: never read
    a.w = w.data_ptr();
    a.y = y.data_ptr();
    a.m_local = rows_;
    a.n = static_cast<int>(w.size(0));
    a.k = cols_;
    a.ctrl = ctrl_;
    std::vector<at::Tensor> keep{w, y};
    if (fp8_) keep.push_back(*scale_w);
    launch([&](const CommDev& c, cudaStream_t s) { B200C_CUDA_CHECK(launch_allgather_gemm(c, a, s)); },
           fp8_ ? "ag_gemm_fp8/kernel" : "ag_gemm/kernel", keep);
    return y;
  }

  // gemm_rs: out[m/nranks, n] = reduce_scatter(h[m, k_local] @ w[n, k_local]^T)
  at::Tensor gemm_rs(const at::Tensor& h, const at::Tensor& w, const c10::optional<at::Tensor>& scale_h,
                     const c10::optional<at::Tensor>& scale_w) {
    TORCH_CHECK(!ag_, "not a gemm_rs layer");
    const auto dt = fp8_ ? at::kFloat8_e4m3fn : at::kBFloat16;
    TORCH_CHECK(h.is_cuda() && h.is_contiguous() && h.scalar_type() == dt && h.dim() == 2 && h.size(0) == rows_,
                "h: contiguous [m, k_local] of the layer's operand type");
    TORCH_CHECK(w.is_cuda() && w.is_contiguous() && w.scalar_type() == dt && w.dim() == 2 && w.size(0) == cols_ &&
                    w.size(1) == h.size(1),
                "w: contiguous [n, k_local] of the layer's operand type");
    TORCH_CHECK(h.size(1) % (fp8_ ? 128 : 64) == 0, "k_local must be a multiple of 64 (fp8: 128)");
    auto scale_ok = [](const c10::optional<at::Tensor>& s, int64_t n) {
      return s.has_value() && s->is_cuda() && s->scalar_type() == at::kFloat && s->is_contiguous() && s->numel() == n;
    };
    TORCH_CHECK(!fp8_ || (scale_ok(scale_h, rows_) && scale_ok(scale_w, cols_)), "fp8: scale_h fp32 [m] and scale_w fp32 [n]");
    c10::cuda::CUDAGuard g(h.device());
    at::Tensor out = at::empty({rows_ / nranks_, cols_}, h.options().dtype(at::kBFloat16));
    GemmRsArgs a{};
    if (fp8_) {
      a.fp8 = 1;
      a.scale_h = scale_h->data_ptr<float>();
      a.scale_w = scale_w->data_ptr<float>();
    }
    a.h = h.data_ptr();
    a.w = w.data_ptr();
    for (int p = 0; p < nranks_; ++p) {
      a.partials[p] = bases_[p];
      a.arrived[p] = reinterpret_cast<uint32_t*>(bases_[p] + data_bytes_);
    }
    a.send_stage = send_stage_;
    a.out = out.data_ptr();
    a.m = rows_;
    a.n = cols_;
    a.k_local = static_cast<int>(h.size(1));
    a.ctrl = ctrl_;
    std::vector<at::Tensor> keep{h, w, out};
    if (fp8_) keep.insert(keep.end(), {*scale_h, *scale_w});
    launch([&](const CommDev& c, cudaStream_t s) { B200C_CUDA_CHECK(launch_gemm_reduce_scatter(c, a, s)); },
           fp8_ ? "gemm_rs_fp8/kernel" : "gemm_rs/kernel", keep);
    return out;
  }

  std::vector<uint32_t> status() const {
    return status_host_ ? std::vector<uint32_t>(status_host_, status_host_ + 5) : std::vector<uint32_t>{};
  }

 private:
  template <class F>
  void launch(F&& fn, const char* what, std::vector<at::Tensor> keep) {
    if (backend_) {
      backend_->run(what, false, {}, keep, [&](cudaStream_t s) { fn(backend_->comm_dev(), s); });
    } else {
      fn(solo_, at::cuda::getCurrentCUDAStream().stream());
    }
  }

  std::shared_ptr<CudaBackend> backend_;
  bool ag_;
  int rows_, cols_;
  bool fp8_ = false;
  float* scale_full_ = nullptr;
  void* send_stage_ = nullptr;
  int nranks_ = 1, rank_ = 0;
  size_t data_bytes_ = 0, flag_bytes_ = 0;
  std::shared_ptr<SymmSegment> seg_;
  std::vector<char*> bases_;
  std::vector<void*> local_;
  uint32_t* ctrl_ = nullptr;
  void* x_full_ = nullptr;
  uint32_t* status_host_ = nullptr;
  CommDev solo_;
};

// Up to four ranks of one layer shape on ONE device (kernel tests): every
// rank's buffers are ordinary device memory of this GPU, the kernels of all
// ranks run as one cooperative launch and talk through the same flags and
// staging areas as separate GPUs would.
class TpEmuWorld {
 public:
  TpEmuWorld(int nranks, const std::string& kind, int rows, int cols, double wait_ms, bool fp8)
      : ag_(kind == "ag_gemm"), fp8_(fp8), nranks_(nranks), rows_(rows), cols_(cols) {
    TORCH_CHECK(kind == "ag_gemm" || kind == "gemm_rs", "kind must be 'ag_gemm' or 'gemm_rs'");
    TORCH_CHECK(nranks >= 1 && nranks <= 4, "1 to 4 emulated ranks");
    if (ag_) {
      TORCH_CHECK(rows % 128 == 0 && cols % (fp8 ? 128 : 64) == 0,
                  "ag_gemm: m_local % 128 == 0 and k % 64 == 0 (fp8: k % 128 == 0) required");
      data_bytes_ = align256(static_cast<size_t>(rows) * cols * (fp8 ? 1 : 2));
      flag_bytes_ = fp8 ? align256(static_cast<size_t>(rows) * 4) : 0;
    } else {
      TORCH_CHECK(rows % (128 * nranks) == 0 && cols % 256 == 0, "gemm_rs: m % (128*nranks) == 0 and n % 256 == 0 required");
      data_bytes_ = align256(static_cast<size_t>(rows) * cols * 2);
      flag_bytes_ = align256(static_cast<size_t>(rows / nranks / 128) * (cols / 256) * nranks * 4);
    }
    auto zeroed = [this](size_t bytes) {
      void* p = nullptr;
      B200C_CUDA_CHECK(cudaMalloc(&p, bytes));
      B200C_CUDA_CHECK(cudaMemset(p, 0, bytes));
      allocs_.push_back(p);
      return p;
    };
    B200C_CUDA_CHECK(cudaHostAlloc(reinterpret_cast<void**>(&status_host_), 64, cudaHostAllocMapped));
    std::memset(status_host_, 0, 64);
    uint32_t* sdev = nullptr;
    B200C_CUDA_CHECK(cudaHostGetDevicePointer(reinterpret_cast<void**>(&sdev), status_host_, 0));
    const size_t fb = static_cast<size_t>(kFlagSets) * kMaxBlocks * kMaxRanks * sizeof(uint32_t);
    std::vector<uint32_t*> flags(nranks);
    for (int r = 0; r < nranks; ++r) {
      bases_.push_back(static_cast<char*>(zeroed(data_bytes_ + flag_bytes_)));
      flags[r] = static_cast<uint32_t*>(zeroed(fb));
      ctrl_.push_back(static_cast<uint32_t*>(zeroed(tp_ctrl_words(ag_ ? rows * nranks : 0) * sizeof(uint32_t))));
      x_full_.push_back(ag_ ? zeroed(static_cast<size_t>(rows) * nranks * cols * 2) : nullptr);
      scale_full_.push_back(ag_ && fp8 ? static_cast<float*>(zeroed(static_cast<size_t>(rows) * nranks * 4)) : nullptr);
      send_stage_.push_back(!ag_ && nranks > 1 ? zeroed(static_cast<size_t>(rows) * cols * 2) : nullptr);
    }
    comms_.resize(nranks);
    for (int r = 0; r < nranks; ++r) {
      CommDev& c = comms_[r];
      std::memset(&c, 0, sizeof(c));
      c.rank = r;
      c.nranks = nranks;
      for (int p = 0; p < nranks; ++p) c.flags[p] = flags[p];
      c.epochs = static_cast<uint32_t*>(zeroed(kFlagSets * kMaxBlocks * sizeof(uint32_t)));
      c.status = sdev;
      c.timeout_ns = static_cast<unsigned long long>(wait_ms * 1e6);
    }
    B200C_CUDA_CHECK(cudaDeviceSynchronize());
  }
  ~TpEmuWorld() {
    for (void* p : allocs_) cudaFree(p);
    if (status_host_) cudaFreeHost(status_host_);
  }

  at::Tensor input(int r) {
    TORCH_CHECK(ag_ && r >= 0 && r < nranks_, "input(rank): ag_gemm worlds only");
    auto opts = at::TensorOptions().device(at::kCUDA, at::cuda::current_device()).dtype(fp8_ ? at::kFloat8_e4m3fn : at::kBFloat16);
    return at::from_blob(bases_[r], {rows_, cols_}, opts);
  }
  at::Tensor input_scales(int r) {
    TORCH_CHECK(ag_ && fp8_ && r >= 0 && r < nranks_, "input_scales(rank): fp8 ag_gemm worlds only");
    auto opts = at::TensorOptions().device(at::kCUDA, at::cuda::current_device()).dtype(at::kFloat);
    return at::from_blob(bases_[r] + data_bytes_, {rows_}, opts);
  }

  // ys[r] = all_gather(inputs) @ ws[r]^T
  std::vector<at::Tensor> ag_gemm(const std::vector<at::Tensor>& ws, const std::vector<at::Tensor>& scale_ws) {
    TORCH_CHECK(ag_ && static_cast<int>(ws.size()) == nranks_, "one weight shard per rank");
    TORCH_CHECK(fp8_ ? static_cast<int>(scale_ws.size()) == nranks_ : scale_ws.empty(), "fp8: one [n] scale vector per rank");
    const auto dt = fp8_ ? at::kFloat8_e4m3fn : at::kBFloat16;
    std::vector<AgGemmArgs> args(nranks_);
    std::vector<at::Tensor> ys;
    for (int r = 0; r < nranks_; ++r) {
      const at::Tensor& w = ws[r];
      TORCH_CHECK(w.is_cuda() && w.is_contiguous() && w.scalar_type() == dt && w.dim() == 2 &&
                      w.size(1) == cols_ && w.size(0) % 256 == 0 && w.size(0) == ws[0].size(0),
                  "w: contiguous [n, k], n % 256 == 0, the same n on every rank");
      ys.push_back(at::empty({static_cast<int64_t>(rows_) * nranks_, w.size(0)}, w.options().dtype(at::kBFloat16)));
      AgGemmArgs& a = args[r];
      a = AgGemmArgs{};
      if (fp8_) {
        TORCH_CHECK(scale_ws[r].is_cuda() && scale_ws[r].scalar_type() == at::kFloat && scale_ws[r].is_contiguous() &&
                        scale_ws[r].numel() == w.size(0),
                    "scale_w: contiguous fp32 [n]");
        a.fp8 = 1;
        for (int p = 0; p < nranks_; ++p) a.scale_x_shards[p] = reinterpret_cast<const float*>(bases_[p] + data_bytes_);
        a.scale_x_full = scale_full_[r];
        a.scale_w = scale_ws[r].data_ptr<float>();
      }
      for (int p = 0; p < nranks_; ++p) a.x_shards[p] = bases_[p];
      a.x_full = x_full_[r];
      a.w = w.data_ptr();
      a.y = ys[r].data_ptr();
      a.m_local = rows_;
      a.n = static_cast<int>(w.size(0));
      a.k = cols_;
      a.ctrl = ctrl_[r];
    }
    cudaStream_t s = at::cuda::getCurrentCUDAStream().stream();
    B200C_CUDA_CHECK(launch_allgather_gemm_emu(comms_.data(), args.data(), nranks_, s));
    return ys;
  }

  // outs[r] = rows of rank r of sum over ranks of hs[q] @ ws[q]^T
  std::vector<at::Tensor> gemm_rs(const std::vector<at::Tensor>& hs, const std::vector<at::Tensor>& ws,
                                  const std::vector<at::Tensor>& scale_hs, const std::vector<at::Tensor>& scale_ws) {
    TORCH_CHECK(!ag_ && static_cast<int>(hs.size()) == nranks_ && static_cast<int>(ws.size()) == nranks_,
                "one activation and one weight shard per rank");
    TORCH_CHECK(fp8_ ? static_cast<int>(scale_hs.size()) == nranks_ && static_cast<int>(scale_ws.size()) == nranks_
                     : scale_hs.empty() && scale_ws.empty(),
                "fp8: one [m] and one [n] scale vector per rank");
    const auto dt = fp8_ ? at::kFloat8_e4m3fn : at::kBFloat16;
    std::vector<GemmRsArgs> args(nranks_);
    std::vector<at::Tensor> outs;
    for (int r = 0; r < nranks_; ++r) {
      const at::Tensor &h = hs[r], &w = ws[r];
      TORCH_CHECK(h.is_cuda() && h.is_contiguous() && h.scalar_type() == dt && h.dim() == 2 && h.size(0) == rows_ &&
                      h.size(1) % (fp8_ ? 128 : 64) == 0 && h.size(1) == hs[0].size(1),
                  "h: contiguous [m, k_local], k_local % 64 == 0 (fp8: 128)");
      TORCH_CHECK(w.is_cuda() && w.is_contiguous() && w.scalar_type() == dt && w.dim() == 2 && w.size(0) == cols_ &&
                      w.size(1) == h.size(1),
                  "w: contiguous [n, k_local]");
      outs.push_back(at::empty({rows_ / nranks_, cols_}, h.options().dtype(at::kBFloat16)));
      GemmRsArgs& a = args[r];
      a = GemmRsArgs{};
      if (fp8_) {
        TORCH_CHECK(scale_hs[r].is_cuda() && scale_hs[r].scalar_type() == at::kFloat && scale_hs[r].is_contiguous() &&
                        scale_hs[r].numel() == rows_ && scale_ws[r].is_cuda() && scale_ws[r].scalar_type() == at::kFloat &&
                        scale_ws[r].is_contiguous() && scale_ws[r].numel() == cols_,
                    "scale_h: fp32 [m], scale_w: fp32 [n]");
        a.fp8 = 1;
        a.scale_h = scale_hs[r].data_ptr<float>();
        a.scale_w = scale_ws[r].data_ptr<float>();
      }
      a.h = h.data_ptr();
      a.w = w.data_ptr();
      for (int p = 0; p < nranks_; ++p) {
        a.partials[p] = bases_[p];
        a.arrived[p] = reinterpret_cast<uint32_t*>(bases_[p] + data_bytes_);
      }
      a.send_stage = send_stage_[r];
      a.out = outs[r].data_ptr();
      a.m = rows_;
      a.n = cols_;
      a.k_local = static_cast<int>(h.size(1));
      a.ctrl = ctrl_[r];
    }
    cudaStream_t s = at::cuda::getCurrentCUDAStream().stream();
    B200C_CUDA_CHECK(launch_gemm_reduce_scatter_emu(comms_.data(), args.data(), nranks_, s));
    return outs;
  }

  std::vector<uint32_t> status() const { return std::vector<uint32_t>(status_host_, status_host_ + 5); }

 private:
  bool ag_, fp8_;
  int nranks_, rows_, cols_;
  size_t data_bytes_ = 0, flag_bytes_ = 0;
  std::vector<char*> bases_;
  std::vector<uint32_t*> ctrl_;
  std::vector<void*> x_full_;
  std::vector<float*> scale_full_;
  std::vector<void*> send_stage_;
  std::vector<void*> allocs_;
  std::vector<CommDev> comms_;
  uint32_t* status_host_ = nullptr;
};

} // namespace

void bind_tp(py::module_& m) {
  py::class_<TpEmuWorld>(m, "TpEmuWorld")
      .def(py::init<int, const std::string&, int, int, double, bool>(), py::arg("nranks"), py::arg("kind"), py::arg("rows"),
           py::arg("cols"), py::arg("wait_ms") = 2000.0, py::arg("fp8") = false)
      .def("input", &TpEmuWorld::input)
      .def("input_scales", &TpEmuWorld::input_scales)
      .def("ag_gemm", &TpEmuWorld::ag_gemm, py::arg("ws"), py::arg("scale_ws") = std::vector<at::Tensor>{})
      .def("gemm_rs", &TpEmuWorld::gemm_rs, py::arg("hs"), py::arg("ws"), py::arg("scale_hs") = std::vector<at::Tensor>{},
           py::arg("scale_ws") = std::vector<at::Tensor>{})
      .def("status", &TpEmuWorld::status);
  py::class_<TpLayer, std::shared_ptr<TpLayer>>(m, "TpLayer")
      .def(py::init([](py::object backend, const std::string& kind, int rows, int cols, double wait_ms, bool fp8) {
             std::shared_ptr<CudaBackend> b;
             if (!backend.is_none()) b = backend.cast<std::shared_ptr<CudaBackend>>();
             return std::make_shared<TpLayer>(b, kind, rows, cols, wait_ms, fp8);
           }),
           py::arg("backend"), py::arg("kind"), py::arg("rows"), py::arg("cols"), py::arg("wait_ms") = 2000.0,
           py::arg("fp8") = false)
      .def("input", &TpLayer::input)
      .def("input_scales", &TpLayer::input_scales)
      .def("ag_gemm", &TpLayer::ag_gemm, py::arg("w"), py::arg("scale_w") = py::none(), py::call_guard<py::gil_scoped_release>())
      .def("gemm_rs", &TpLayer::gemm_rs, py::arg("h"), py::arg("w"), py::arg("scale_h") = py::none(),
           py::arg("scale_w") = py::none(), py::call_guard<py::gil_scoped_release>())
      .def("status", &TpLayer::status);
}

} // namespace b200c
