// Tensor-level bindings of the fused model kernels (`_comms.ops`).
#include "py_common.hpp"

#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>

#include "../cuda/driver_api.hpp"
#include "../kernels/fused_ops.h"
#include "../kernels/launch_count.h"
#include "../kernels/tc_gemm.h"

namespace b200c {

namespace {

const __nv_bfloat16* bf(const at::Tensor& t) {
  return reinterpret_cast<const __nv_bfloat16*>(t.data_ptr());
}
__nv_bfloat16* bf_mut(at::Tensor& t) {
  return reinterpret_cast<__nv_bfloat16*>(t.data_ptr());
}

void want(const at::Tensor& t, at::ScalarType dt, const char* name) {
  TORCH_CHECK(t.is_cuda() && t.is_contiguous(), name, ": contiguous CUDA tensor expected");
  TORCH_CHECK(t.scalar_type() == dt, name, ": expected dtype ", dt, ", got ", t.scalar_type());
}

cudaStream_t cur(const at::Tensor& t) {
  return at::cuda::getCurrentCUDAStream(t.device().index()).stream();
}

} // namespace

void bind_ops(py::module_& m) {
  auto ops = m.def_submodule("ops", "fused sm_100a model kernels");

  // Points the storage behind `t` (and so every view of it, including tensors
  // autograd saved) at the memory of `src`, or at nothing. The storage keeps
  // `src` alive. This is how a stage's flat parameter buffer moves between
  // rotating communication buffers without its parameter views being rebuilt.
  ops.def("rebind_storage_", [](at::Tensor t, std::optional<at::Tensor> src) {
    c10::StorageImpl* impl = t.storage().unsafeGetStorageImpl();
    if (!src.has_value()) {
      impl->set_data_ptr_noswap(at::DataPtr(nullptr, t.device()));
      impl->set_nbytes(0);
      return;
    }
    TORCH_CHECK(src->is_contiguous() && src->device() == t.device(), "rebind_storage_: contiguous source on the same device");
    auto* keep = new at::Tensor(*src);
    impl->set_data_ptr_noswap(
        at::DataPtr(src->data_ptr(), keep, [](void* ctx) { delete static_cast<at::Tensor*>(ctx); }, t.device()));
    impl->set_nbytes(src->nbytes());
  }, py::arg("tensor"), py::arg("source") = py::none());

  ops.def("rmsnorm_fwd", [](const at::Tensor& x, const at::Tensor& w, double eps) {
    want(x, at::kBFloat16, "x");
    want(w, at::kBFloat16, "w");
    const int cols = static_cast<int>(x.size(-1));
    const int rows = static_cast<int>(x.numel() / cols);
    TORCH_CHECK(w.numel() == cols, "weight must have ", cols, " elements");
    c10::cuda::CUDAGuard g(x.device());
    at::Tensor y = at::empty_like(x);
    at::Tensor rstd = at::empty({rows}, x.options().dtype(at::kFloat));
    B200C_CUDA_CHECK(launch_rmsnorm_fwd(bf(x), bf(w), bf_mut(y), rstd.data_ptr<float>(), rows, cols,
                                        static_cast<float>(eps), cur(x)));
    return std::make_pair(y, rstd);
  });

  ops.def("rmsnorm_bwd", [](const at::Tensor& dy, const at::Tensor& x, const at::Tensor& w, const at::Tensor& rstd) {
    want(dy, at::kBFloat16, "dy");
    want(x, at::kBFloat16, "x");
    want(w, at::kBFloat16, "w");
    want(rstd, at::kFloat, "rstd");
    const int cols = static_cast<int>(x.size(-1));
    const int rows = static_cast<int>(x.numel() / cols);
    c10::cuda::CUDAGuard g(x.device());
    int nblocks = 0;
    B200C_CUDA_CHECK(launch_rmsnorm_bwd(nullptr, nullptr, nullptr, nullptr, nullptr, nullptr, &nblocks, rows, cols, cur(x)));
    at::Tensor dx = at::empty_like(x);
    at::Tensor partial = at::empty({nblocks, cols}, x.options().dtype(at::kFloat));
    at::Tensor dw = at::empty_like(w);
    B200C_CUDA_CHECK(launch_rmsnorm_bwd(bf(dy), bf(x), bf(w), rstd.data_ptr<float>(), bf_mut(dx),
                                        partial.data_ptr<float>(), &nblocks, rows, cols, cur(x)));
    B200C_CUDA_CHECK(launch_colsum_bf16(partial.data_ptr<float>(), bf_mut(dw), nblocks, cols, cur(x)));
    return std::make_pair(dx, dw);
  });

  ops.def("rope_", [](at::Tensor x, const at::Tensor& pos, const at::Tensor& cos_t, const at::Tensor& sin_t, bool inverse) {
    want(x, at::kBFloat16, "x");
    want(pos, at::kInt, "pos");
    want(cos_t, at::kFloat, "cos");
    want(sin_t, at::kFloat, "sin");
    TORCH_CHECK(x.dim() >= 3, "x must be [..., tokens, heads, head_dim]");
    const int head_dim = static_cast<int>(x.size(-1));
    const int heads = static_cast<int>(x.size(-2));
    const int tokens = static_cast<int>(x.numel() / (static_cast<int64_t>(head_dim) * heads));
    TORCH_CHECK(pos.numel() == tokens, "pos must have one entry per token");
    TORCH_CHECK(cos_t.size(-1) == head_dim / 2 && sin_t.size(-1) == head_dim / 2, "cos/sin tables: [max_pos, head_dim/2]");
    c10::cuda::CUDAGuard g(x.device());
    B200C_CUDA_CHECK(launch_rope(bf_mut(x), pos.data_ptr<int>(), cos_t.data_ptr<float>(), sin_t.data_ptr<float>(), tokens,
                                 heads, head_dim, inverse, cur(x)));
    return x;
  });

  ops.def("swiglu_fwd", [](const at::Tensor& gate_up) {
    want(gate_up, at::kBFloat16, "gate_up");
    const int ffn = static_cast<int>(gate_up.size(-1) / 2);
    const int rows = static_cast<int>(gate_up.numel() / (2 * static_cast<int64_t>(ffn)));
    c10::cuda::CUDAGuard g(gate_up.device());
    auto sizes = gate_up.sizes().vec();
    sizes.back() = ffn;
    at::Tensor h = at::empty(sizes, gate_up.options());
    B200C_CUDA_CHECK(launch_swiglu_fwd(bf(gate_up), bf_mut(h), rows, ffn, cur(gate_up)));
    return h;
  });

  ops.def("swiglu_bwd", [](const at::Tensor& dh, const at::Tensor& gate_up) {
    want(dh, at::kBFloat16, "dh");
    want(gate_up, at::kBFloat16, "gate_up");
    const int ffn = static_cast<int>(gate_up.size(-1) / 2);
    const int rows = static_cast<int>(gate_up.numel() / (2 * static_cast<int64_t>(ffn)));
    c10::cuda::CUDAGuard g(gate_up.device());
    at::Tensor d = at::empty_like(gate_up);
    B200C_CUDA_CHECK(launch_swiglu_bwd(bf(dh), bf(gate_up), bf_mut(d), rows, ffn, cur(gate_up)));
    return d;
  });

  ops.def("cross_entropy_fwd_bwd_", [](at::Tensor logits, const at::Tensor& targets, double grad_scale) {
    want(logits, at::kBFloat16, "logits");
    want(targets, at::kLong, "targets");
    const int vocab = static_cast<int>(logits.size(-1));
    const int rows = static_cast<int>(logits.numel() / vocab);
    TORCH_CHECK(targets.numel() == rows, "one target per row");
    c10::cuda::CUDAGuard g(logits.device());
    at::Tensor loss = at::empty({rows}, logits.options().dtype(at::kFloat));
    B200C_CUDA_CHECK(launch_cross_entropy_fwd_bwd(bf_mut(logits), targets.data_ptr<int64_t>(), loss.data_ptr<float>(), rows,
                                                  vocab, static_cast<float>(grad_scale), cur(logits)));
    return loss;
  });

  ops.def("adamw_step_", [](at::Tensor p, const at::Tensor& grad, at::Tensor mom, at::Tensor var, double lr, double beta1,
                            double beta2, double eps, double weight_decay, int step, double grad_scale) {
    want(p, at::kFloat, "p");
    want(grad, at::kFloat, "grad");
    want(mom, at::kFloat, "m");
    want(var, at::kFloat, "v");
    TORCH_CHECK(grad.numel() == p.numel() && mom.numel() == p.numel() && var.numel() == p.numel(), "size mismatch");
    c10::cuda::CUDAGuard g(p.device());
    B200C_CUDA_CHECK(launch_adamw(p.data_ptr<float>(), grad.data_ptr<float>(), mom.data_ptr<float>(), var.data_ptr<float>(),
                                  static_cast<size_t>(p.numel()), static_cast<float>(lr), static_cast<float>(beta1),
                                  static_cast<float>(beta2), static_cast<float>(eps), static_cast<float>(weight_decay), step,
                                  static_cast<float>(grad_scale), cur(p)));
  });

  ops.def("gemm_bf16_nt", [](const at::Tensor& a, const at::Tensor& b) {
    want(a, at::kBFloat16, "a");
    want(b, at::kBFloat16, "b");
    TORCH_CHECK(a.dim() == 2 && b.dim() == 2 && a.size(1) == b.size(1), "a: [m, k], b: [n, k]");
    c10::cuda::CUDAGuard g(a.device());
    at::Tensor c = at::empty({a.size(0), b.size(0)}, a.options());
    at::Tensor status = at::zeros({2}, a.options().dtype(at::kInt));
    B200C_CUDA_CHECK(launch_gemm_bf16_nt(a.data_ptr(), b.data_ptr(), c.data_ptr(), static_cast<int>(a.size(0)),
                                         static_cast<int>(b.size(0)), static_cast<int>(a.size(1)),
                                         reinterpret_cast<uint32_t*>(status.data_ptr<int>()), cur(a)));
    return std::make_pair(c, status);
  });

  // c[m, n] (bf16) = scale_a[m] * scale_b[n] * (a[m, k] (e4m3) @ b[n, k]^T (e4m3)), fp32 accumulation in tensor memory.
  ops.def("gemm_e4m3_nt", [](const at::Tensor& a, const at::Tensor& b, const at::Tensor& scale_a, const at::Tensor& scale_b) {
    want(a, at::kFloat8_e4m3fn, "a");
    want(b, at::kFloat8_e4m3fn, "b");
    want(scale_a, at::kFloat, "scale_a");
    want(scale_b, at::kFloat, "scale_b");
    TORCH_CHECK(a.dim() == 2 && b.dim() == 2 && a.size(1) == b.size(1), "a: [m, k], b: [n, k]");
    TORCH_CHECK(scale_a.numel() == a.size(0) && scale_b.numel() == b.size(0), "one scale per row of a and per row of b");
    c10::cuda::CUDAGuard g(a.device());
    at::Tensor c = at::empty({a.size(0), b.size(0)}, a.options().dtype(at::kBFloat16));
    at::Tensor status = at::zeros({2}, a.options().dtype(at::kInt));
    B200C_CUDA_CHECK(launch_gemm_e4m3_nt(a.data_ptr(), b.data_ptr(), c.data_ptr(), static_cast<int>(a.size(0)),
                                         static_cast<int>(b.size(0)), static_cast<int>(a.size(1)), scale_a.data_ptr<float>(),
                                         scale_b.data_ptr<float>(), reinterpret_cast<uint32_t*>(status.data_ptr<int>()), cur(a)));
    return std::make_pair(c, status);
  });

  ops.def("gemm_bf16_nt_pair", [](const at::Tensor& a, const at::Tensor& b) {
    want(a, at::kBFloat16, "a");
    want(b, at::kBFloat16, "b");
    TORCH_CHECK(a.dim() == 2 && b.dim() == 2 && a.size(1) == b.size(1), "a: [m, k], b: [n, k]");
    c10::cuda::CUDAGuard g(a.device());
    at::Tensor c = at::empty({a.size(0), b.size(0)}, a.options());
    at::Tensor status = at::zeros({2}, a.options().dtype(at::kInt));
    B200C_CUDA_CHECK(launch_gemm_bf16_nt_pair(a.data_ptr(), b.data_ptr(), c.data_ptr(), static_cast<int>(a.size(0)),
                                              static_cast<int>(b.size(0)), static_cast<int>(a.size(1)),
                                              reinterpret_cast<uint32_t*>(status.data_ptr<int>()), cur(a)));
    return std::make_pair(c, status);
  });

  ops.def("kernel_launch_count", []() { return kernel_launch_count(); });
}

} // namespace b200c
