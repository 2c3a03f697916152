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
  size_t symm_meta_off = 0;   // all-to-all on symmetric buffers: lengths, offsets and grants per (block, sender)
  size_t symm_meta_bytes = 0;
  size_t lamport_off = 0;     // flag-less small all-reduce: 3 rotating receive buffers
  size_t lamport_bytes = 0;
};

constexpr size_t kSymmMetaBytes = static_cast<size_t>(kMaxBlocks) * kMaxRanks * 3 * sizeof(unsigned long long);

// A buffer that every rank of the communicator has mapped: `ptr[r]` is rank
// r's copy as seen from this process (ptr[own rank] is local memory), `mc` the
// NVLS multicast alias of all copies or nullptr.
struct SymmView {
  char* ptr[kMaxRanks];
  char* mc;
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

// ---- one-pass collectives on symmetric buffers (coll_symm.cu) ----------------
// Nothing is staged: data moves once, between the users' tensors. `blocks` must
// be the same on every rank. `in` / `out` / views hold one entry per emulated
// rank (one entry when emu_ranks == 0).

// out (symmetric) = concatenation over ranks of `in` (in_bytes per rank; with
// the cast, fp32 in and bf16 out). The wire size per rank must be a multiple of 16.
cudaError_t launch_symm_all_gather(const CommDev* comms, int emu_ranks, const void* const* in, const SymmView* out,
                                   size_t in_bytes, bool cast_f32_to_bf16, bool use_mc, int blocks,
                                   cudaStream_t stream);
// out[count] = scale * sum over ranks of slice `rank` of the symmetric input
// (nranks x count elements of wire_dtype). count % (16 / wire size) == 0.
cudaError_t launch_symm_reduce_scatter(const CommDev* comms, int emu_ranks, const SymmView* in, void* const* out,
                                       size_t count, DType wire_dtype, DType out_dtype, float scale, bool use_mc,
                                       int blocks, cudaStream_t stream);
// In-place sum (times scale) of a symmetric buffer. count % (16 / element size) == 0.
cudaError_t launch_symm_all_reduce(const CommDev* comms, int emu_ranks, const SymmView* buf, size_t count, DType dtype,
                                   float scale, bool use_mc, int blocks, cudaStream_t stream);
// All-to-all(v) into a symmetric output. Offsets / lengths in bytes, nranks
// entries per (emulated) rank; `in_bytes` / `out_bytes` are the buffers'
// capacities, one entry per (emulated) rank. `exchange` = false: equal splits, every rank
// already knows where its blocks land. With `dev_send_counts` the lengths are
// int64 counts of `elem_bytes` in device memory and blocks are packed back to
// back on both sides. Lengths that do not fit the buffers are clamped and
// reported through the status word (kStatusBadArg).
cudaError_t launch_symm_all_to_all(const CommDev* comms, const HeapLayout& lay, int emu_ranks, const void* const* in,
                                   const SymmView* out, const size_t* in_bytes, const size_t* out_bytes, const size_t* send_off,
                                   const size_t* send_len, const size_t* recv_off, const size_t* recv_len,
                                   const long long* const* dev_send_counts, size_t elem_bytes, bool exchange,
                                   int blocks, cudaStream_t stream);

// Sequence <-> heads exchange of sequence-parallel attention, layout changes included. `out` symmetric.
// to_heads: in [batch, heads, s, d] -> out [batch, heads / nranks, nranks * s, d]; otherwise the inverse.
// `slab_bytes` = s * d * element size (one [s, d] slab, contiguous on both sides).
cudaError_t launch_symm_seq_heads(const CommDev* comms, int emu_ranks, const void* const* in, const SymmView* out,
                                  int batch, int heads, size_t slab_bytes, bool to_heads, int blocks,
                                  cudaStream_t stream);

// ---- flag-less small all-reduce (coll_lamport.cu) -----------------------------
constexpr int kLamportBlocks = 256;         // pieces per call
constexpr size_t kLamportPiece = 4 * 1024;  // payload bytes per piece and rank (one 16-byte vector per thread)
constexpr size_t kLamportBytes = 3ull * kLamportBlocks * kMaxRanks * kLamportPiece;
constexpr unsigned kLamportPoison = 0x80000000u;  // -0.0f: "nothing arrived yet"
// Fills the three receive buffers with the poison word (once, at set-up).
cudaError_t launch_lamport_init(char* region, cudaStream_t stream);
// out = scale * sum over ranks of in; count * element size <= kLamportBlocks * kLamportPiece.
cudaError_t launch_all_reduce_lamport(const CommDev* comms, const HeapLayout& lay, int emu_ranks,
                                      const void* const* in, void* const* out, size_t count, DType dtype,
                                      float scale, bool use_mc, cudaStream_t stream);

// The same flag-less protocol for small all-gather (mode 0: out = nranks parts, one from each
// rank), all-to-all with equal parts (mode 1) and reduce-scatter (mode 2: out = scale * sum of
// the parts addressed to this rank). `part_bytes` per rank: a multiple of 16, at most
// kLamportBlocks * kLamportPiece; pointers 16-byte aligned; floating-point payloads only.
cudaError_t launch_exchange_lamport(const CommDev* comms, const HeapLayout& lay, int emu_ranks, int mode,
                                    const void* const* in, void* const* out, size_t part_bytes, DType dtype, float scale,
                                    bool use_mc, cudaStream_t stream);
// The same arrival protocol for an all-to-all with unequal parts (floating types; any byte lengths). Per rank i and
// peer p: send_off / send_len / recv_off / recv_len [i * kMaxRanks + p] in bytes. `cap_bytes` bounds every part
// and must be derived from a quantity that is the same on every rank (it decides how many blocks take part).
cudaError_t launch_exchangev_lamport(const CommDev* comms, const HeapLayout& lay, int emu_ranks, const void* const* in,
                                     void* const* out, const size_t* send_off, const size_t* send_len, const size_t* recv_off,
                                     const size_t* recv_len, size_t cap_bytes, cudaStream_t stream);

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
                                            LaunchShape shape, cudaStream_t stream,
                                            const size_t* in_bytes = nullptr, const size_t* out_bytes = nullptr);
// `in_bytes` / `out_bytes`: capacities of the buffers, one entry per (emulated) rank. Counts that are negative
// or do not fit are clamped (nothing is read or written out of bounds) and
// reported through the status word (kStatusBadArg).

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
