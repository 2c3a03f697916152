// All-reduce + residual add + RMSNorm in one kernel, for the small token
// batches of tensor-parallel decode: the row-parallel projection leaves a
// partial [rows, hidden] on every rank; each rank needs
//   x   = sum_r partial_r (+ residual)        (residual updated in place)
//   out = x * rsqrt(mean(x^2) + eps) * weight
// One block per row. The block stages its row in this rank's peer-visible
// staging, meets the same block of every peer at one barrier, then reads the
// row from all peers (fp32 accumulation), adds the residual, reduces the sum
// of squares inside the block and writes both outputs; the all-reduce result
// never goes to memory on its own.
//
// Staging is private to this operation (two parity halves, so a fast rank's
// next call cannot overwrite a row a slow rank still reads) and its flags are
// rows 512.. of the latency flag set, which the other latency kernels (at most
// 128 blocks) never touch.
//
// Parity: the reference's vendored NVIDIA contrib tree has this fusion as
// `nccl_ubx` (comms/ncclx/v2_31/contrib/nccl_ubx: all-reduce + residual +
// RMSNorm); its own collectives stop at the plain one-shot all-reduce
// (comms/common/algorithms/all_reduce/all_reduce_dda.cuh:20-112).
#include "coll_common.cuh"
#include "collectives.h"

namespace b200c {

namespace coll {

struct ArNorm {
  using Args = ArNormArgs;

  static __device__ __forceinline__ bool row_barrier(const CommDev& c, int frow, uint32_t value, uint32_t phase) {
    __shared__ int s_ok;
    __syncthreads();
    if (threadIdx.x == 0) s_ok = 1;
    __syncthreads();
    if (threadIdx.x < c.nranks) {
      const int peer = threadIdx.x;
      __threadfence_system();  // the block's staged row is visible before the flag
      st_relaxed_sys(flag_slot(c, peer, kFlagSetSmall, frow, c.rank), value);
      if (!wait_flag_reached(c, flag_slot(c, c.rank, kFlagSetSmall, frow, peer), value, peer, phase)) s_ok = 0;
    }
    __syncthreads();
    return s_ok != 0;
  }

  static __device__ void run(const CommDev& c, const Args& a) {
    using P = Pack<__nv_bfloat16>;
    constexpr int N = P::N;            // 8 values per 16-byte vector
    constexpr int kVecPerThread = kArNormMaxHidden / N / 256;  // 4
    __shared__ float s_part[8];
    const int row = blockIdx.x;
    if (row >= a.rows) return;  // same decision on every rank
    const int frow = kArNormFlagRow0 + row;
    const uint32_t epoch = c.epochs[kFlagSetSmall * kMaxBlocks + frow] + 1;
    const size_t row_bytes = static_cast<size_t>(a.hidden) * sizeof(__nv_bfloat16);
    const size_t off = (static_cast<size_t>(epoch & 1u) * kArNormMaxRows + row) * row_bytes;
    const size_t row_elems = static_cast<size_t>(row) * a.hidden;
    block_copy(a.stage[c.rank] + off, a.in + row_elems, row_bytes);
    const bool ok = row_barrier(c, frow, epoch, 0x17);
    if (ok) {
      const int nvec = a.hidden / N;
      float x[kVecPerThread][N];
      float ss = 0.f;
#pragma unroll
      for (int j = 0; j < kVecPerThread; ++j) {
        const int v = static_cast<int>(threadIdx.x) + j * 256;
        if (v < nvec) {
          // All loads are issued before the first use; they are summed in rank order, so every
          // rank rounds the same way and the replicas stay bit-identical.
          uint4 p[kMaxRanks];
#pragma unroll
          for (int r = 0; r < kMaxRanks; ++r) {
            if (r < c.nranks) p[r] = ld16(a.stage[r] + off + static_cast<size_t>(v) * 16);
          }
          float acc[N];
          P::unpack(p[0], acc);
#pragma unroll
          for (int r = 1; r < kMaxRanks; ++r) {
            if (r < c.nranks) {
              float f[N];
              P::unpack(p[r], f);
#pragma unroll
              for (int k = 0; k < N; ++k) acc[k] += f[k];
            }
          }
          if (a.residual != nullptr) {
            float f[N];
            P::unpack(ld16(a.residual + row_elems + static_cast<size_t>(v) * N), f);
#pragma unroll
            for (int k = 0; k < N; ++k) acc[k] += f[k];
          }
          // The normalisation sees the value as it is stored (bf16), like an unfused norm reading it back.
          const uint4 packed = P::pack(acc);
          if (a.residual != nullptr) st16(a.residual + row_elems + static_cast<size_t>(v) * N, packed);
          P::unpack(packed, x[j]);
#pragma unroll
          for (int k = 0; k < N; ++k) ss += x[j][k] * x[j][k];
        }
      }
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
      if ((threadIdx.x & 31) == 0) s_part[threadIdx.x >> 5] = ss;
      __syncthreads();
      float total = 0.f;
#pragma unroll
      for (int w = 0; w < 8; ++w) total += s_part[w];
      const float rstd = rsqrtf(total / static_cast<float>(a.hidden) + a.eps);
#pragma unroll
      for (int j = 0; j < kVecPerThread; ++j) {
        const int v = static_cast<int>(threadIdx.x) + j * 256;
        if (v < nvec) {
          float w[N], y[N];
          P::unpack(ld16(a.weight + static_cast<size_t>(v) * N), w);
#pragma unroll
          for (int k = 0; k < N; ++k) y[k] = x[j][k] * rstd * w[k];
          st16(a.out + row_elems + static_cast<size_t>(v) * N, P::pack(y));
        }
      }
    }
    __syncthreads();
    if (threadIdx.x == 0) c.epochs[kFlagSetSmall * kMaxBlocks + frow] = epoch;
  }
};

}  // namespace coll

cudaError_t launch_all_reduce_rmsnorm(const CommDev* comms, int emu_ranks, const ArNormArgs* args, cudaStream_t stream) {
  const int n = emu_ranks > 0 ? emu_ranks : 1;
  for (int i = 0; i < n; ++i) {
    const ArNormArgs& a = args[i];
    if (a.rows < 1 || a.rows > kArNormMaxRows || a.hidden < 8 || a.hidden > kArNormMaxHidden || a.hidden % 8 != 0) {
      return cudaErrorInvalidValue;
    }
    if (a.rows != args[0].rows || a.hidden != args[0].hidden) return cudaErrorInvalidValue;
    const uintptr_t bits = reinterpret_cast<uintptr_t>(a.in) | reinterpret_cast<uintptr_t>(a.out) |
        reinterpret_cast<uintptr_t>(a.weight) | reinterpret_cast<uintptr_t>(a.residual) |
        reinterpret_cast<uintptr_t>(a.stage[comms[i].rank]);
    if (bits & 15u) return cudaErrorMisalignedAddress;
  }
  return coll::launch_op<coll::ArNorm>(comms, emu_ranks, args, args[0].rows, 256, stream, true);
}

}  // namespace b200c
