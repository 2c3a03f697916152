// Host-side launch interface of the peer-memory collective kernels.
//
// No PyTorch types here: callers pass raw pointers, a CommDev describing the
// symmetric heap, and a stream. Every launcher returns a cudaError_t.
//
// `emu_ranks > 0` selects the single-GPU emulation used by tests: `comms` and
// the per-rank argument arrays then hold `emu_ranks` entries, and one
// cooperative launch runs all virtual ranks side by side (blockIdx.y = rank),
// so kernels that wait on one another are guaranteed to be co-resident.
#pragma once

#include "device_prims.cuh"

namespace b200c {

enum class DType : int { F32 = 0, F16 = 1, BF16 = 2 };
enum class RedKind : int { SUM = 0, PROD = 1, MIN = 2, MAX = 3 };

inline size_t dtype_size(DType t) { return t == DType::F32 ? 4 : 2; }

// Heap layout (byte offsets into each rank's symmetric region).
struct HeapLayout {
  size_t bulk_off = 0;     // bulk staging: blocks x chunk slots
  size_t bulk_bytes = 0;
  size_t small_off = 0;    // latency staging: 2 parity halves x kSmallBlocks x kSmallPiece x nranks-wide
  size_t small_bytes = 0;
  size_t user_off = 0;     // windows / EP / TP scratch handed out by the backend
  size_t user_bytes = 0;
};

constexpr size_t kSmallPiece = 4 * 1024;   // bytes of payload one block stages in latency mode (one 16-byte vector per thread)
constexpr int kSmallBlocks = 128;          // at most this many pieces per latency-mode call

struct LaunchShape {
  int blocks = 1;
  int threads = 512;
  size_t chunk_bytes = 0;  // bulk mode: bytes staged per block per step; 0 selects the latency (one-shot) kernels
  size_t known_max = 0;    // all-to-all: largest block when every rank knows all lengths (skips the count exchange)
};

// In-place or out-of-place all-reduce of `count` elements.
//   algo 0: one-shot (latency mode; count*size <= kSmallBlocks*kSmallPiece)
//   algo 1: two-shot through the bulk staging region
// `scale` multiplies the reduced value (1/nranks for AVG, the factor for
// PREMUL_SUM). `use_mc` allows the NVLS multimem path (SUM only).
cudaError_t launch_all_reduce(const CommDev* comms, const HeapLayout& lay, int emu_ranks,
                              const void* const* in, void* const* out, size_t count, DType dtype,
                              RedKind red, float scale, int algo, bool use_mc, LaunchShape shape,
                              cudaStream_t stream);

// All-reduce + residual add + RMSNorm of a bf16 [rows, hidden] partial (one block per row).
constexpr int kArNormFlagRow0 = 512;     // first row of the latency flag set this kernel signals on
constexpr int kArNormMaxRows = 128;
constexpr int kArNormMaxHidden = 8192;
struct ArNormArgs {
  const __nv_bfloat16* in;       // this rank's partial sums
  __nv_bfloat16* residual;       // nullptr, or [rows, hidden] updated in place with sum + residual
  const __nv_bfloat16* weight;   // [hidden]
  __nv_bfloat16* out;            // [rows, hidden] normalised
  char* stage[kMaxRanks];        // every rank's staging: 2 x kArNormMaxRows x hidden bf16
  int rows;
  int hidden;                    // multiple of 8, <= kArNormMaxHidden
  float eps;
};
inline size_t ar_norm_stage_bytes(int hidden) { return 2ull * kArNormMaxRows * static_cast<size_t>(hidden) * 2; }
// `args` has one entry per emulated rank (one entry when emu_ranks == 0).
cudaError_t launch_all_reduce_rmsnorm(const CommDev* comms, int emu_ranks, const ArNormArgs* args, cudaStream_t stream);

// Reduce-scatter: `in` holds nranks x count elements of `in_dtype`; rank r
// receives the reduction of block r as `out_dtype`. Data crosses NVLink as
// `wire_dtype`. Supported type triples: all equal, or in in {F32,BF16},
// wire BF16, out in {F32,BF16}.
cudaError_t launch_reduce_scatter(const CommDev* comms, const HeapLayout& lay, int emu_ranks,
                                  const void* const* in, void* const* out, size_t count,
                                  DType in_dtype, DType wire_dtype, DType out_dtype, RedKind red,
                                  float scale, bool use_mc, LaunchShape shape, cudaStream_t stream,
                                  unsigned long long sr_seed = 0);
// `sr_seed` != 0 (fp32 input with a bf16 wire only): the narrowing to bf16
// rounds stochastically (Philox-4x32-7 bits, cvt.rs.bf16x2.f32) instead of to
// nearest, which keeps the reduced sum unbiased.

// All-gather of `bytes` bytes per rank (dtype-agnostic), or with a fused
// F32 -> BF16 cast when `cast_f32_to_bf16` (then `bytes` counts input bytes
// and the output holds nranks x bytes/2).
cudaError_t launch_all_gather(const CommDev* comms, const HeapLayout& lay, int emu_ranks,
                              const void* const* in, void* const* out, size_t bytes,
                              bool cast_f32_to_bf16, bool use_mc, LaunchShape shape, cudaStream_t stream);

// All-to-all with per-peer byte counts. send_off/send_len/recv_off/recv_len
// are arrays of nranks entries per rank (emu: emu_ranks x nranks, row-major).
// recv_len[q] on rank r must equal send_len[r] on rank q. `max_len` is the
// largest single block over all ranks (sizes the staging steps).
cudaError_t launch_all_to_all(const CommDev* comms, const HeapLayout& lay, int emu_ranks,
                              const void* const* in, void* const* out, const size_t* send_off,
                              const size_t* send_len, const size_t* recv_off, const size_t* recv_len,
                              size_t max_len, LaunchShape shape, cudaStream_t stream);

// All-to-all whose split sizes live on the device: `dev_send_counts` holds
// nranks int64 counts of `elem_bytes`-sized elements per rank; blocks are
// packed back to back in both input and output, and every rank learns what it
// receives from the senders inside the kernel (no host synchronisation).
cudaError_t launch_all_to_all_device_splits(const CommDev* comms, const HeapLayout& lay, int emu_ranks,
                                            const void* const* in, void* const* out,
                                            const long long* const* dev_send_counts, size_t elem_bytes,
                                            LaunchShape shape, cudaStream_t stream);

// Broadcast `bytes` bytes from `root`.
cudaError_t launch_broadcast(const CommDev* comms, const HeapLayout& lay, int emu_ranks,
                             void* const* buf, size_t bytes, int root, bool use_mc, LaunchShape shape,
                             cudaStream_t stream);

// Barrier across ranks (one block).
cudaError_t launch_barrier(const CommDev* comms, int emu_ranks, cudaStream_t stream);

// Test hook: a kernel that waits on a flag nobody sets, with the given wait
// budget, to exercise the bounded-wait error path. Sets kStatusTimeout.
cudaError_t launch_wait_unset_flag(const CommDev* comms, int emu_ranks, cudaStream_t stream);

} // namespace b200c
