// Low-latency MoE dispatch / combine for decode-sized batches.
//
// dispatch: every (token, expert) pair is one row. The sender numbers its rows
// per expert with a local counter and stores each row (quantised to fp8 e4m3
// with 1x128 scales, or bf16) into a slot of the destination that is fixed by
// (local expert, source rank, row number), so nothing has to be agreed before
// the data moves. As soon as the rows are numbered, the sender writes its row
// count of every expert to every rank, tagged with the call number; the rows
// follow, each piece raising the row's arrival counter at the receiver with a
// release-ordered add once it has been stored. The receiver waits for the
// counts of its own experts (bounded), and packs the rows of each expert,
// sources in rank order, as they arrive, into a dense [local experts,
// nranks * max_tokens, hidden] tensor that a grouped GEMM can consume, with
// the count per expert beside it. No system-wide fence, one grid-wide meeting.
// combine: the token's owner reads the expert outputs straight out of the
// expert ranks' (symmetric) output tensors. It knows the packed position of
// each of its rows from its own row numbers and the counts everybody
// published, and forms the weighted top-k sum in registers.
//
// Receive slots and count tables are double-buffered by call parity, so the
// dispatch ends without a cross-GPU barrier.
//
// Replaces, in the reference: comms/prims/collectives/link_ep/cpp/low_latency/
// kernels/Dispatch.cu and Combine.cu (send / receive phases over IBGDA with
// per-expert receive buffers and a push combine into an [experts, tokens]
// buffer at the source), link_ep/buffer.py:550-625.
#pragma once

#include "device_prims.cuh"

namespace b200c {

struct EpLlDev {
  int rank, nranks;
  int num_experts, experts_per_rank, topk, hidden;
  int max_tokens;  // tokens per rank and call, also rows per (expert, source) slot group
  int fp8;
  // Symmetric, peer-mapped. The first three hold two parities back to back.
  char* slot_x[kMaxRanks];                 // [2][local experts][nranks][max_tokens] rows
  float* slot_scales[kMaxRanks];           // [2][local experts][nranks][max_tokens][hidden/128]
  int* slot_src[kMaxRanks];                // [2][local experts][nranks][max_tokens] source token
  unsigned int* slot_arrived[kMaxRanks];   // same shape: pieces of the row that have landed (reset by the receiver)
  unsigned long long* counts[kMaxRanks];   // [2][num_experts][nranks]: (call << 32) | rows that source sent to that expert
  char* out_x[kMaxRanks];                  // [local experts][nranks * max_tokens][hidden] bf16 expert outputs
  // Local.
  int* cnt;                   // [2][num_experts] send counters, the idle parity is zeroed for the next call
  unsigned int* call;         // [1] calls so far
  int* send_slot;             // [max_tokens][topk] row number within (expert, this source), -1 = not sent
  int* begin;                 // [num_experts] packed position of this rank's first row at each expert
};

struct EpLlRecv {
  void* packed_x;           // [local experts][nranks * max_tokens][hidden] fp8 or bf16
  float* packed_scales;     // [local experts][nranks * max_tokens][hidden/128] (fp8)
  int* packed_src;          // [local experts][nranks * max_tokens] source token index
  int* packed_count;        // [local experts]
  long long* layout_range;  // [local experts][nranks]: (first packed row << 32) | rows
};

cudaError_t launch_ep_ll_dispatch(const CommDev* comms, const EpLlDev* eps, int emu_ranks, const void* const* x,
                                  const int* const* topk_idx, const EpLlRecv* recv, int num_tokens, cudaStream_t stream);
// out[t] = sum_k w[t, k] * out_x_{rank of expert k}[local expert][begin + row number]
// `send_slot`, `begin` (optional, per rank): handles of an earlier dispatch.
cudaError_t launch_ep_ll_combine(const CommDev* comms, const EpLlDev* eps, int emu_ranks, void* const* out,
                                 const int* const* topk_idx, const float* const* topk_w, int num_tokens,
                                 const int* const* send_slot, const int* const* begin, cudaStream_t stream);

} // namespace b200c
