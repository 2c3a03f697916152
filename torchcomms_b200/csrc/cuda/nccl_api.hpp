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

// The settable fields of ncclConfig_t (public NCCL ABI, layout of 2.28; 2.27
// has the same fields up to nvlsCTAs). kUnset / empty = leave NCCL's default.
struct NcclConfig {
  static constexpr int kUnset = -2147483647 - 1;  // NCCL_CONFIG_UNDEF_INT
  int blocking = kUnset;
  int cgaClusterSize = kUnset;
  int minCTAs = kUnset;
  int maxCTAs = kUnset;
  std::string netName;
  int splitShare = kUnset;
  int trafficClass = kUnset;
  std::string commName;
  int collnetEnable = kUnset;
  int CTAPolicy = kUnset;
  int shrinkShare = kUnset;
  int nvlsCTAs = kUnset;
  int nChannelsPerNetPeer = kUnset;
  int nvlinkCentricSched = kUnset;
  bool any() const {
    return blocking != kUnset || cgaClusterSize != kUnset || minCTAs != kUnset || maxCTAs != kUnset || !netName.empty() ||
        splitShare != kUnset || trafficClass != kUnset || !commName.empty() || collnetEnable != kUnset ||
        CTAPolicy != kUnset || shrinkShare != kUnset || nvlsCTAs != kUnset || nChannelsPerNetPeer != kUnset ||
        nvlinkCentricSched != kUnset;
  }
};

class NcclApi {
 public:
  virtual ~NcclApi() = default;
  virtual bool available() = 0;
  virtual std::string version() = 0;
  virtual NcclResult getUniqueId(NcclUniqueId* id) = 0;
  virtual NcclResult commInitRank(NcclComm** comm, int nranks, NcclUniqueId id, int rank) = 0;
  // ncclCommInitRankConfig with the given fields set. The default forwards to
  // commInitRank (for implementations that have no configuration to honour).
  virtual NcclResult commInitRankConfig(NcclComm** comm, int nranks, NcclUniqueId id, int rank, const NcclConfig& cfg) {
    (void)cfg;
    return commInitRank(comm, nranks, id, rank);
  }
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
  // What new communicators use: the real library unless a test installed a fake.
  static std::shared_ptr<NcclApi> current();
  static void install(std::shared_ptr<NcclApi> fake);   // nullptr restores the real one
};

} // namespace b200c
