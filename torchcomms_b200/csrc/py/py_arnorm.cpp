// Binding of the fused all-reduce + residual add + RMSNorm layer.
#include "py_common.hpp"

#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>

#include <cstring>

#include "../backends/cuda_backend.hpp"
#include "../cuda/driver_api.hpp"
#include "../kernels/collectives.h"

namespace b200c {

namespace {

// Owns the staging of one hidden size. With a backend the staging lives in the
// communicator's symmetric memory; without one (single rank on the current
// device) in ordinary device memory.
class ArNormLayer {
 public:
  ArNormLayer(std::shared_ptr<CudaBackend> backend, int hidden, double wait_ms) : backend_(std::move(backend)), hidden_(hidden) {
    TORCH_CHECK(hidden >= 8 && hidden <= kArNormMaxHidden && hidden % 8 == 0, "hidden: a multiple of 8 up to ", kArNormMaxHidden);
    nranks_ = backend_ ? backend_->size() : 1;
    rank_ = backend_ ? backend_->rank() : 0;
    const size_t total = ar_norm_stage_bytes(hidden);
    if (backend_) {
      c10::cuda::CUDAGuard g(backend_->device());
      seg_ = backend_->symm().allocate(total, false);
      for (int p = 0; p < nranks_; ++p) bases_.push_back(seg_->peer_ptrs[p]);
    } else {
      void* p = nullptr;
      B200C_CUDA_CHECK(cudaMalloc(&p, total));
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
      B200C_CUDA_CHECK(cudaDeviceSynchronize());
    }
  }

  ~ArNormLayer() {
    for (void* p : local_) cudaFree(p);
    if (status_host_) cudaFreeHost(status_host_);
    if (seg_ && backend_ && backend_->symm_alive()) {
      try {
        backend_->symm().release(seg_);
      } catch (...) {
      }
    }
  }

  // out = rmsnorm(all_reduce(x) + residual) * weight; `residual` (optional) becomes all_reduce(x) + residual.
  at::Tensor forward(const at::Tensor& x, const std::optional<at::Tensor>& residual, const at::Tensor& weight, double eps) {
    auto ok = [&](const at::Tensor& t) { return t.is_cuda() && t.is_contiguous() && t.scalar_type() == at::kBFloat16; };
    TORCH_CHECK(ok(x) && x.dim() == 2 && x.size(1) == hidden_, "x: contiguous bf16 [rows, hidden]");
    TORCH_CHECK(x.size(0) >= 1 && x.size(0) <= kArNormMaxRows, "rows must be in 1..", kArNormMaxRows);
    TORCH_CHECK(ok(weight) && weight.numel() == hidden_, "weight: contiguous bf16 [hidden]");
    if (residual) {
      TORCH_CHECK(ok(*residual) && residual->sizes() == x.sizes(), "residual: contiguous bf16 with the shape of x");
    }
    c10::cuda::CUDAGuard g(x.device());
    at::Tensor out = at::empty_like(x);
    ArNormArgs a{};
    a.in = static_cast<const __nv_bfloat16*>(x.data_ptr());
    a.residual = residual ? static_cast<__nv_bfloat16*>(residual->data_ptr()) : nullptr;
    a.weight = static_cast<const __nv_bfloat16*>(weight.data_ptr());
    a.out = static_cast<__nv_bfloat16*>(out.data_ptr());
    for (int p = 0; p < nranks_; ++p) a.stage[p] = bases_[p];
    a.rows = static_cast<int>(x.size(0));
    a.hidden = hidden_;
    a.eps = static_cast<float>(eps);
    std::vector<at::Tensor> keep{x, weight, out};
    if (residual) keep.push_back(*residual);
    if (backend_) {
      backend_->run("all_reduce_rmsnorm/kernel", false, {}, keep,
                    [&](cudaStream_t s) { B200C_CUDA_CHECK(launch_all_reduce_rmsnorm(&backend_->comm_dev(), 0, &a, s)); });
    } else {
      B200C_CUDA_CHECK(launch_all_reduce_rmsnorm(&solo_, 0, &a, at::cuda::getCurrentCUDAStream().stream()));
    }
    return out;
  }

  std::vector<uint32_t> status() const {
    return status_host_ ? std::vector<uint32_t>(status_host_, status_host_ + 5) : std::vector<uint32_t>{};
  }

 private:
  std::shared_ptr<CudaBackend> backend_;
  int hidden_;
  int nranks_ = 1, rank_ = 0;
  std::shared_ptr<SymmSegment> seg_;
  std::vector<char*> bases_;
  std::vector<void*> local_;
  uint32_t* status_host_ = nullptr;
  CommDev solo_;
};

}  // namespace

void bind_arnorm(py::module_& m) {
  py::class_<ArNormLayer, std::shared_ptr<ArNormLayer>>(m, "ArNormLayer")
      .def(py::init([](py::object backend, int hidden, double wait_ms) {
             std::shared_ptr<CudaBackend> b;
             if (!backend.is_none()) b = backend.cast<std::shared_ptr<CudaBackend>>();
             return std::make_shared<ArNormLayer>(b, hidden, wait_ms);
           }),
           py::arg("backend"), py::arg("hidden"), py::arg("wait_ms") = 2000.0)
      .def("forward", &ArNormLayer::forward, py::arg("x"), py::arg("residual"), py::arg("weight"), py::arg("eps") = 1e-5,
           py::call_guard<py::gil_scoped_release>())
      .def("status", &ArNormLayer::status);
  m.attr("AR_NORM_MAX_ROWS") = kArNormMaxRows;
  m.attr("AR_NORM_MAX_HIDDEN") = kArNormMaxHidden;
}

}  // namespace b200c
