// Thin, mockable seam over the NCCL C API, bound at run time with dlopen
// (PyTorch already has libnccl.so.2 in the process). Only the stable public
// entry points are used; the declarations below restate that public ABI.
//
// NCCL serves point-to-point traffic (pipeline send/recv), dtypes and
// reductions the peer-memory kernels do not cover, and acts as the baseline
// path selectable with hints {"algo": "nccl"}.
//
// Parity: comms/torchcomms/nccl/NcclApi.hpp / comms/torchcomms/ncclx/NcclxApi.hpp:86
// (virtual wrapper that unit tests replace with a mock).
#pragma once

#include <cuda_runtime.h>

#include <memory>
#include <string>

namespace b200c {

// Public NCCL ABI (nccl.h): opaque comm, 128-byte unique id, enums.
struct NcclComm;
struct NcclUniqueId {
  char internal[128];
};
enum NcclResult : int { kNcclSuccess = 0, kNcclInProgress = 7 };
enum NcclDataType : int {
  kNcclInt8 = 0, kNcclUint8 = 1, kNcclInt32 = 2, kNcclUint32 = 3, kNcclInt64 = 4, kNcclUint64 = 5,
  kNcclFloat16 = 6, kNcclFloat32 = 7, kNcclFloat64 = 8, kNcclBfloat16 = 9, kNcclFloat8e4m3 = 10, kNcclFloat8e5m2 = 11,
};
enum NcclRedOp : int { kNcclSum = 0, kNcclProd = 1, kNcclMax = 2, kNcclMin = 3, kNcclAvg = 4 };

class NcclApi {
 public:
  virtual ~NcclApi() = default;
  virtual bool available() = 0;
  virtual std::string version() = 0;
  virtual NcclResult getUniqueId(NcclUniqueId* id) = 0;
  virtual NcclResult commInitRank(NcclComm** comm, int nranks, NcclUniqueId id, int rank) = 0;
  virtual NcclResult commDestroy(NcclComm* comm) = 0;
  virtual NcclResult commAbort(NcclComm* comm) = 0;
  virtual NcclResult commGetAsyncError(NcclComm* comm, NcclResult* async_error) = 0;
  virtual NcclResult groupStart() = 0;
  virtual NcclResult groupEnd() = 0;
  virtual NcclResult send(const void* buf, size_t count, NcclDataType t, int peer, NcclComm* comm, cudaStream_t s) = 0;
  virtual NcclResult recv(void* buf, size_t count, NcclDataType t, int peer, NcclComm* comm, cudaStream_t s) = 0;
  virtual NcclResult broadcast(const void* send, void* recv, size_t count, NcclDataType t, int root, NcclComm* comm, cudaStream_t s) = 0;
  virtual NcclResult allReduce(const void* send, void* recv, size_t count, NcclDataType t, NcclRedOp op, NcclComm* comm, cudaStream_t s) = 0;
  virtual NcclResult reduce(const void* send, void* recv, size_t count, NcclDataType t, NcclRedOp op, int root, NcclComm* comm, cudaStream_t s) = 0;
  virtual NcclResult allGather(const void* send, void* recv, size_t sendcount, NcclDataType t, NcclComm* comm, cudaStream_t s) = 0;
  virtual NcclResult reduceScatter(const void* send, void* recv, size_t recvcount, NcclDataType t, NcclRedOp op, NcclComm* comm, cudaStream_t s) = 0;
  // scalar lives on the host (residence = host immediate)
  virtual NcclResult redOpCreatePreMulSum(NcclRedOp* op, void* scalar, NcclDataType t, NcclComm* comm) = 0;
  virtual NcclResult redOpDestroy(NcclRedOp op, NcclComm* comm) = 0;
  virtual std::string errorString(NcclResult r) = 0;

  static std::shared_ptr<NcclApi> real();
};

} // namespace b200c
