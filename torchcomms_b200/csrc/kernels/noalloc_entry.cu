// See noalloc_entry.h. The kernels are the ones behind ops.rmsnorm_bwd; only
// the home of the partial-gradient scratch differs.
#include "noalloc_entry.h"

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <mutex>

#include "fused_ops.h"

namespace {

// [block, col] fp32 partial sums of dw. Written in full by the first kernel
// (one row per block), read by the second; no initial value is assumed.
static __device__ __align__(256) float g_rms_partials[B200C_NOALLOC_MAX_BLOCKS * B200C_NOALLOC_MAX_COLS];

constexpr int kMaxDevices = 64;
std::mutex g_mu;
float* g_scratch[kMaxDevices] = {};

// Address of the array on the current device; looked up once per device.
cudaError_t scratch_for_current_device(float** out) {
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return e;
  if (dev < 0 || dev >= kMaxDevices) return cudaErrorInvalidDevice;
  std::lock_guard<std::mutex> lk(g_mu);
  if (g_scratch[dev] == nullptr) {
    float* ptr = nullptr;
    e = cudaGetSymbolAddress(reinterpret_cast<void**>(&ptr), g_rms_partials);
    if (e != cudaSuccess) return e;
    g_scratch[dev] = ptr;
  }
  *out = g_scratch[dev];
  return cudaSuccess;
}

bool aligned_to(const void* p, uintptr_t bytes) {
  return (reinterpret_cast<uintptr_t>(p) & (bytes - 1)) == 0;
}

bool aligned16(const void* p) {
  return aligned_to(p, 16);
}

// The scratch must hold one row per block of the widest launch (two blocks on
// each of the 148 SMs) and one row is as wide as the norm kernels reach
// (256 threads x 4 vectors x 8 bf16).
static_assert(B200C_NOALLOC_MAX_BLOCKS >= 2 * 148, "scratch rows: one per block of the first kernel");
static_assert(B200C_NOALLOC_MAX_COLS == 256 * 4 * 8, "scratch width: the widest row the norm kernels take");

} // namespace

extern "C" __attribute__((visibility("default"))) int b200c_rmsnorm_bwd_noalloc(const void* dy, const void* x,
                                                                                  const void* w, const float* rstd,
                                                                                  void* dx, void* dw, int rows, int cols,
                                                                                  void* stream) {
  if (dy == nullptr || x == nullptr || w == nullptr || rstd == nullptr || dx == nullptr || dw == nullptr) {
    return B200C_NOALLOC_BAD_ARG;
  }
  if (rows < 1 || cols < 8 || cols % 8 != 0) return B200C_NOALLOC_BAD_ARG;
  if (cols > B200C_NOALLOC_MAX_COLS) return B200C_NOALLOC_TOO_LARGE;
  if (!aligned16(dy) || !aligned16(x) || !aligned16(w) || !aligned16(dx)) return B200C_NOALLOC_BAD_ARG;
  if (!aligned_to(rstd, sizeof(float)) || !aligned_to(dw, sizeof(__nv_bfloat16))) return B200C_NOALLOC_BAD_ARG;
  float* partials = nullptr;
  cudaError_t e = scratch_for_current_device(&partials);
  if (e != cudaSuccess) return static_cast<int>(e);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  int blocks = 0;
  // Sizing query first: the block count decides how many scratch rows are used.
  e = b200c::launch_rmsnorm_bwd(nullptr, nullptr, nullptr, nullptr, nullptr, nullptr, &blocks, rows, cols, s);
  if (e != cudaSuccess) return static_cast<int>(e);
  if (blocks > B200C_NOALLOC_MAX_BLOCKS) return B200C_NOALLOC_TOO_LARGE;
  e = b200c::launch_rmsnorm_bwd(static_cast<const __nv_bfloat16*>(dy), static_cast<const __nv_bfloat16*>(x),
                                static_cast<const __nv_bfloat16*>(w), rstd, static_cast<__nv_bfloat16*>(dx), partials,
                                &blocks, rows, cols, s);
  if (e != cudaSuccess) return static_cast<int>(e);
  e = b200c::launch_colsum_bf16(partials, static_cast<__nv_bfloat16*>(dw), blocks, cols, s);
  return static_cast<int>(e);
}

extern "C" __attribute__((visibility("default"))) const char* b200c_noalloc_strerror(int code) {
  switch (code) {
    case B200C_NOALLOC_OK:
      return "ok";
    case B200C_NOALLOC_TOO_LARGE:
      return "shape exceeds the fixed scratch: cols must be <= 8192 (B200C_NOALLOC_MAX_COLS)";
    case B200C_NOALLOC_BAD_ARG:
      return "bad argument: pointers must be non-null, dy/x/w/dx 16-byte aligned, rstd and dw aligned to their "
             "element, rows >= 1, cols a positive multiple of 8";
    default:
      return code > 0 ? cudaGetErrorString(static_cast<cudaError_t>(code)) : "unknown code";
  }
}
