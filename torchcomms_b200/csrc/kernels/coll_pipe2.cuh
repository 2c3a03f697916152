// Two-stage pipeline shared by the pull-style collectives (reduce-scatter,
// all-gather, all-to-all, broadcast).
//
// A block owns chunks blockIdx.x, +gridDim.x, ... and a ring of kPipeSlots
// staging slots in its rank's heap.
//   stage(k):   write this rank's contribution to chunk k into slot k % S
//               (after every rank has finished consuming chunk k - S), then
//               post "ready k"
//   consume(k): once every rank is ready with chunk k, pull what this rank
//               needs from the peers' slots straight into the user's output,
//               then post "done k"
// Iteration i runs stage(i) and consume(i-1) and posts both flags behind one
// fence. Before returning the block waits until every rank is done with its
// last chunk, so the next kernel may lay the staging region out differently.
#pragma once

#include "coll_common.cuh"

namespace b200c {
namespace coll {

// Op provides:
//   struct Args;
//   static __device__ size_t prologue(const CommDev&, const Args&);   // total number of chunks (same on every rank)
//   static __device__ size_t slot_bytes(const CommDev&, const Args&);
//   static __device__ void stage(const CommDev&, const Args&, size_t chunk, size_t slot_off);
//   static __device__ void consume(const CommDev&, const Args&, size_t chunk, size_t slot_off);
template <typename Op>
struct Pipe2 {
  using Args = typename Op::Args;
  static __device__ void run(const CommDev& c, const Args& a) {
    constexpr int S = kPipeSlots;
    const size_t nchunks = Op::prologue(c, a);
    const size_t slot_bytes = Op::slot_bytes(c, a);
    const long n = blockIdx.x < nchunks ? static_cast<long>((nchunks - blockIdx.x + gridDim.x - 1) / gridDim.x) : 0;
    const uint32_t base_r = c.epochs[kFlagSetReady * kMaxBlocks + blockIdx.x];
    const uint32_t base_d = c.epochs[kFlagSetDone * kMaxBlocks + blockIdx.x];
    const size_t slot0 = a.bulk_off + static_cast<size_t>(blockIdx.x) * S * slot_bytes;
    bool ok = true;
    trace_mark(c, 0);
    for (long k = 0; k < n + 1; ++k) {
      // A failed wait (timeout, abort) ends the pipeline: nothing more is
      // staged, copied or posted, so the kernel returns within one wait.
      if (!ok) break;
      if (k < n) {
        if (k >= S) {
          ok = wait_all_peers(c, kFlagSetDone, base_d + static_cast<uint32_t>(k - S) + 1, 0x31) && ok;
        }
        if (ok) Op::stage(c, a, blockIdx.x + static_cast<size_t>(k) * gridDim.x, slot0 + (k % S) * slot_bytes);
      }
      if (k == 0) trace_mark(c, 1);
      if (k >= 1) {
        const long j = k - 1;
        ok = wait_all_peers(c, kFlagSetReady, base_r + static_cast<uint32_t>(j) + 1, 0x32) && ok;
        if (k == 1) trace_mark(c, 2);
        if (ok) {
          Op::consume(c, a, blockIdx.x + static_cast<size_t>(j) * gridDim.x, slot0 + (j % S) * slot_bytes);
        }
        if (k == 1) trace_mark(c, 3);
      }
      if (ok) post_flags(c, k < n, base_r + static_cast<uint32_t>(k) + 1, k >= 1, base_d + static_cast<uint32_t>(k));
    }
    if (n > 0 && ok) {
      // Drain: nobody reads this block's slots any more once this returns.
      wait_all_peers(c, kFlagSetDone, base_d + static_cast<uint32_t>(n), 0x33);
    }
    trace_mark(c, 4);
    __syncthreads();
    if (threadIdx.x == 0) {
      c.epochs[kFlagSetReady * kMaxBlocks + blockIdx.x] = base_r + static_cast<uint32_t>(n);
      c.epochs[kFlagSetDone * kMaxBlocks + blockIdx.x] = base_d + static_cast<uint32_t>(n);
    }
  }
};

} // namespace coll
} // namespace b200c
