// tcgen05 / TMEM GEMMs (sm_100a) and their fusion with tensor-parallel
// collectives. Raw-pointer launch interface.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

#include "device_prims.cuh"

namespace b200c {

// C[M, N] (bf16) = A[M, K] (bf16, row-major) x B[N, K]^T (bf16, row-major),
// fp32 accumulation in tensor memory. K % 64 == 0, N % 128 == 0.
// `status` (device or mapped host memory, may be null) receives a non-zero
// word if a bounded wait inside the kernel ran out.
cudaError_t launch_gemm_bf16_nt(const void* a, const void* b, void* c, int m, int n, int k, uint32_t* status,
                                cudaStream_t stream);

// The same with fp8 operands: C[M, N] (bf16) = scale_a[m] * scale_b[n] * (A[M, K] (e4m3) x B[N, K]^T (e4m3)),
// one fp32 scale per row of A (per token) and per row of B (per output channel), applied to the fp32
// accumulator in the epilogue. K % 16 == 0. An e4m3 row has the bytes of a bf16 row of half the length, so
// tiles, tensor maps and pipeline are those of the bf16 kernel; only the tcgen05.mma kind differs.
cudaError_t launch_gemm_e4m3_nt(const void* a, const void* b, void* c, int m, int n, int k, const float* scale_a,
                                const float* scale_b, uint32_t* status, cudaStream_t stream);
// Common entry of the two above (k in 16-bit units, scales null = bf16).
cudaError_t launch_gemm_nt(const void* a, const void* b, void* c, int m, int n, int k, const float* scale_a,
                           const float* scale_b, uint32_t* status, cudaStream_t stream);

// The same product on CTA pairs (clusters of two CTAs, tcgen05 cta_group::2):
// each pair owns a 256 x 256 tile and reads every B element once. Same
// argument rules; any m, n % 8 == 0, k % 8 == 0.
cudaError_t launch_gemm_bf16_nt_pair(const void* a, const void* b, void* c, int m, int n, int k, uint32_t* status,
                                     cudaStream_t stream);

// Column-parallel layer fused with the all-gather of its input.
// x_shards[r] is rank r's [m_local, k] bf16 activation shard in symmetric
// memory (x_shards[rank] local); `x_full` is local scratch [nranks*m_local, k]
// that the kernel's copy warps fill from the peers while the tensor cores
// already work on the rows that have arrived (own rows first, then the
// sources in ring order); w is this rank's [n, k] weight shard;
// y [nranks*m_local, n]. m_local % 128 == 0, n % 256 == 0, k % 64 == 0.
// `ctrl`: local device memory of tp_ctrl_words(nranks*m_local) uint32, zeroed
// once when allocated; the kernel keeps its call epoch and arrival counters
// there, so the same launch may be replayed from a CUDA graph.
// The kernel opens and closes with a cross-rank barrier: a peer's shard is
// complete before it is read, and no rank returns while its shard is in use.
struct AgGemmArgs {
  const void* x_shards[kMaxRanks];
  void* x_full;
  const void* w;
  void* y;
  int m_local, n, k;
  uint32_t* ctrl;
  // fp8 = 1: x shards and w are e4m3 (k counts e4m3 elements, k % 128 == 0). scale_x_shards[r]: rank r's
  // [m_local] fp32 row scales (symmetric, next to its shard); scale_x_full: local scratch [nranks*m_local]
  // that the copy warps fill with the peers' scales; scale_w: [n] fp32.
  int fp8;
  const float* scale_x_shards[kMaxRanks];
  float* scale_x_full;
  const float* scale_w;
};
cudaError_t launch_allgather_gemm(const CommDev& comm, const AgGemmArgs& args, cudaStream_t stream);

// Row-parallel layer fused with the reduce-scatter of its output.
// h [m, k_local] bf16 local, w [n, k_local] local; every rank computes the
// partial product for all m rows; rows [r*m/nranks, (r+1)*m/nranks) belong to
// rank r. The epilogue TMA-stores each partial tile into local memory: a
// tile of this rank's own rows straight into its `partials` staging, a tile
// of another rank's rows into `send_stage` (local, [m, n] bf16), from where
// four forward warps per CTA push it into the owner's `partials` staging with
// plain 16-byte stores over NVLink (symmetric; partials[r] = owner r's buffer
// of [nranks, m/nranks, n] bf16, slot index = source rank) and raise the
// tile's flag there. The same warps then sum the nranks slots of this rank's
// rows in fp32 into `out` [m/nranks, n] bf16 as the flags arrive, while the
// tensor cores finish the remaining tiles. Tiles for the next rank are
// computed first, the rank's own last. m % (128*nranks) == 0, n % 256 == 0,
// k_local % 64 == 0.
// `arrived` (symmetric, arrived[r] on owner r, zeroed once): one uint32 per
// (tile of the owner's rows, source). `ctrl`: as above (tp_ctrl_words(0)).
struct GemmRsArgs {
  const void* h;
  const void* w;
  void* partials[kMaxRanks];
  void* send_stage;   // local [m, n] bf16 (may be null on a single rank)
  uint32_t* arrived[kMaxRanks];
  void* out;
  int m, n, k_local;
  uint32_t* ctrl;
  // fp8 = 1: h and w are e4m3 (k_local % 128 == 0) with scale_h [m] and scale_w [n]; the partial tiles that
  // travel are bf16 as before (already scaled).
  int fp8;
  const float* scale_h;
  const float* scale_w;
};
cudaError_t launch_gemm_reduce_scatter(const CommDev& comm, const GemmRsArgs& args, cudaStream_t stream);

size_t tp_ctrl_words(int m_total);

// Tests: up to 4 ranks in ONE cooperative launch on the current device (the single-CTA kernels, each rank on
// its share of the SMs). comms[r] / args[r] describe rank r; all pointers are device memory of this GPU.
cudaError_t launch_allgather_gemm_emu(const CommDev* comms, const AgGemmArgs* args, int nranks, cudaStream_t stream);
cudaError_t launch_gemm_reduce_scatter_emu(const CommDev* comms, const GemmRsArgs* args, int nranks, cudaStream_t stream);

} // namespace b200c
