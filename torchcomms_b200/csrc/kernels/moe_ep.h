// MoE expert-parallel dispatch / combine inside one NVSwitch domain.
//
// dispatch: every token goes once to each rank that hosts at least one of its
// top-k experts. ONE kernel counts, exchanges the counts with the peers
// (no host synchronisation), quantises each row to fp8 e4m3 with one fp32
// scale per 128 elements while it is in registers, and stores the row, its
// scales, source index and re-based top-k ids / weights straight into the
// destination rank's receive buffer over NVLink, packed by source rank.
// combine: the token's source rank reads the expert output of every rank the
// token went to straight out of that rank's output buffer (the row index was
// recorded by the dispatch) and sums them (optionally weighted, optionally
// plus a bias) in fp32 in registers: one pass over NVLink, nothing staged.
//
// Replaces, in the reference: comms/prims/collectives/link_ep (layout kernel
// cpp/intranode/kernels/Layout.cu:39-218, notify Notify.cu:97-440, dispatch
// Dispatch.cu:40-538, combine Combine.cu:24-466), which moves pre-quantised
// rows through ring FIFOs and learns the receive count through a CPU spin.
#pragma once

#include "device_prims.cuh"

namespace b200c {

struct EpDev {
  int rank, nranks;
  int num_experts, experts_per_rank, topk, hidden;
  int max_tokens;       // capacity: tokens per rank per call
  int fp8;              // 1: e4m3 rows + 1x128 fp32 scales; 0: bf16 rows
  // Receive side of every rank (symmetric, peer-mapped). Capacity nranks*max_tokens rows.
  char* recv_x[kMaxRanks];
  float* recv_scales[kMaxRanks];       // [rows, hidden/128]
  int* recv_src[kMaxRanks];            // [rows] src_rank * max_tokens + token
  int* recv_topk_idx[kMaxRanks];       // [rows, topk] local expert id or -1
  float* recv_topk_w[kMaxRanks];       // [rows, topk]
  long long* count_matrix[kMaxRanks];  // [nranks, nranks]: [s][d] tokens s sends to d
  char* combine_x[kMaxRanks];          // [rows, hidden] bf16: expert outputs, row-aligned with the received rows
  char* stage_x[kMaxRanks];            // [max_tokens, hidden] bf16: source-side rows that the receivers pull (cached dispatch)
  float* comb_topk_w[kMaxRanks];       // [rows, topk] fp32: expert-side per-expert weights (or their gradients) that combine returns
  // Local scratch.
  int* cnt;          // [nranks]
  int* cursor;       // [nranks]
  long long* base;   // [nranks] first slot of this rank's rows in each destination
  int* recv_info;    // [1 + nranks]: total rows received, then rows per source
  int* send_slot;    // [max_tokens, nranks] slot in the destination, -1 = not sent (the combine handle)
};

// All tensors are device pointers of the calling rank. `emu_ranks > 0`: arrays
// of per-virtual-rank descriptors / pointers, one cooperative launch.
cudaError_t launch_ep_dispatch(const CommDev* comms, const EpDev* eps, int emu_ranks, const void* const* x,
                               const int* const* topk_idx, const float* const* topk_w, int num_tokens,
                               cudaStream_t stream);
// out[t] = bias[t] + sum over destinations d of w[t, d] * combine_x_d[slot(t, d)]   (w, bias optional)
// `send_slot` (optional, per rank): the handle of an earlier dispatch instead of the last one's.
// `topk_w_out` (optional, per rank): [num_tokens, topk] fp32, the sum over destinations of comb_topk_w_d[slot(t, d)].
cudaError_t launch_ep_combine(const CommDev* comms, const EpDev* eps, int emu_ranks, void* const* out,
                              const float* const* weights, const void* const* bias, int num_tokens,
                              cudaStream_t stream, const int* const* send_slot = nullptr,
                              float* const* topk_w_out = nullptr);
// Cached dispatch (no quantisation, no new layout): row r of `out` (bf16 [out_rows, hidden]) is row `token` of
// `stage_x` on rank `src_rank`, where recv_src[r] = src_rank * max_tokens + token comes from an earlier dispatch
// (`recv_src` per rank, nullptr = the last one's). `num_rows` (device, per rank; nullptr = the last dispatch's
// count) rows are filled, never more than `out_rows`.
cudaError_t launch_ep_pull(const CommDev* comms, const EpDev* eps, int emu_ranks, void* const* out,
                           const int* const* recv_src, const int* const* num_rows, int out_rows, cudaStream_t stream);
// Layout only: tokens per rank, tokens per expert, token-in-rank mask (int32 outputs).
cudaError_t launch_ep_layout(const int* topk_idx, int num_tokens, int topk, int num_experts, int nranks,
                             int* tokens_per_rank, int* tokens_per_expert, int* is_token_in_rank, cudaStream_t stream);

} // namespace b200c
