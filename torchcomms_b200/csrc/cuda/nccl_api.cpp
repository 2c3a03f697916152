// dlopen-bound NCCL.
#include "nccl_api.hpp"

#include <dlfcn.h>

#include <cstddef>
#include <mutex>
#include <stdexcept>

namespace b200c {

namespace {

// ncclConfig_t as published in nccl.h of NCCL 2.28 (2.27 ends after nvlsCTAs).
struct RawNcclConfig {
  size_t size;
  unsigned int magic;
  unsigned int version;
  int blocking;
  int cgaClusterSize;
  int minCTAs;
  int maxCTAs;
  const char* netName;
  int splitShare;
  int trafficClass;
  const char* commName;
  int collnetEnable;
  int CTAPolicy;
  int shrinkShare;
  int nvlsCTAs;
  int nChannelsPerNetPeer;
  int nvlinkCentricSched;
};

class RealNccl final : public NcclApi {
 public:
  bool available() override {
    load();
    return lib_ != nullptr && fn_init_ != nullptr;
  }
  std::string version() override {
    load();
    int v = 0;
    if (fn_version_ && fn_version_(&v) == kNcclSuccess) {
      return std::to_string(v / 10000) + "." + std::to_string((v / 100) % 100) + "." + std::to_string(v % 100);
    }
    return "unknown";
  }
  NcclResult getUniqueId(NcclUniqueId* id) override { return need(fn_uid_)(id); }
  NcclResult commInitRank(NcclComm** comm, int nranks, NcclUniqueId id, int rank) override {
    return need(fn_init_)(comm, nranks, id, rank);
  }
  NcclResult commInitRankConfig(NcclComm** comm, int nranks, NcclUniqueId id, int rank, const NcclConfig& cfg) override {
    load();
    int code = 0;
    if (fn_init_config_ == nullptr || fn_version_ == nullptr || fn_version_(&code) != kNcclSuccess || code < 22700 || !cfg.any()) {
      return commInitRank(comm, nranks, id, rank);
    }
    RawNcclConfig raw{};
    raw.size = code >= 22800 ? sizeof(RawNcclConfig) : offsetof(RawNcclConfig, nChannelsPerNetPeer);
    raw.magic = 0xcafebeef;
    raw.version = static_cast<unsigned int>(code);
    raw.blocking = cfg.blocking;
    raw.cgaClusterSize = cfg.cgaClusterSize;
    raw.minCTAs = cfg.minCTAs;
    raw.maxCTAs = cfg.maxCTAs;
    raw.netName = cfg.netName.empty() ? nullptr : cfg.netName.c_str();
    raw.splitShare = cfg.splitShare;
    raw.trafficClass = cfg.trafficClass;
    raw.commName = cfg.commName.empty() ? nullptr : cfg.commName.c_str();
    raw.collnetEnable = cfg.collnetEnable;
    raw.CTAPolicy = cfg.CTAPolicy;
    raw.shrinkShare = cfg.shrinkShare;
    raw.nvlsCTAs = cfg.nvlsCTAs;
    raw.nChannelsPerNetPeer = cfg.nChannelsPerNetPeer;
    raw.nvlinkCentricSched = cfg.nvlinkCentricSched;
    return fn_init_config_(comm, nranks, id, rank, &raw);
  }
  NcclResult commDestroy(NcclComm* comm) override { return need(fn_destroy_)(comm); }
  NcclResult commAbort(NcclComm* comm) override { return need(fn_abort_)(comm); }
  NcclResult commGetAsyncError(NcclComm* comm, NcclResult* e) override { return need(fn_async_)(comm, e); }
  NcclResult groupStart() override { return need(fn_gstart_)(); }
  NcclResult groupEnd() override { return need(fn_gend_)(); }
  NcclResult send(const void* b, size_t n, NcclDataType t, int peer, NcclComm* c, cudaStream_t s) override {
    return need(fn_send_)(b, n, t, peer, c, s);
  }
  NcclResult recv(void* b, size_t n, NcclDataType t, int peer, NcclComm* c, cudaStream_t s) override {
    return need(fn_recv_)(b, n, t, peer, c, s);
  }
  NcclResult broadcast(const void* sb, void* rb, size_t n, NcclDataType t, int root, NcclComm* c, cudaStream_t s) override {
    return need(fn_bcast_)(sb, rb, n, t, root, c, s);
  }
  NcclResult allReduce(const void* sb, void* rb, size_t n, NcclDataType t, NcclRedOp op, NcclComm* c, cudaStream_t s) override {
    return need(fn_ar_)(sb, rb, n, t, op, c, s);
  }
  NcclResult reduce(const void* sb, void* rb, size_t n, NcclDataType t, NcclRedOp op, int root, NcclComm* c, cudaStream_t s) override {
    return need(fn_reduce_)(sb, rb, n, t, op, root, c, s);
  }
  NcclResult allGather(const void* sb, void* rb, size_t n, NcclDataType t, NcclComm* c, cudaStream_t s) override {
    return need(fn_ag_)(sb, rb, n, t, c, s);
  }
  NcclResult reduceScatter(const void* sb, void* rb, size_t n, NcclDataType t, NcclRedOp op, NcclComm* c, cudaStream_t s) override {
    return need(fn_rs_)(sb, rb, n, t, op, c, s);
  }
  NcclResult redOpCreatePreMulSum(NcclRedOp* op, void* scalar, NcclDataType t, NcclComm* c) override {
    return need(fn_premul_)(op, scalar, t, /*ncclScalarHostImmediate=*/1, c);
  }
  NcclResult redOpDestroy(NcclRedOp op, NcclComm* c) override { return need(fn_opdestroy_)(op, c); }
  std::string errorString(NcclResult r) override {
    load();
    if (fn_errstr_) {
      return std::string(fn_errstr_(r)) + " (ncclResult " + std::to_string(static_cast<int>(r)) + ")";
    }
    return "ncclResult " + std::to_string(static_cast<int>(r));
  }

 private:
  template <typename F>
  F need(F f) {
    load();
    if (f == nullptr) {
      throw std::runtime_error("NCCL is not available in this process (libnccl.so.2 could not be loaded)");
    }
    return f;
  }
  template <typename F>
  void bind(F& f, const char* name) {
    f = lib_ ? reinterpret_cast<F>(dlsym(lib_, name)) : nullptr;
  }
  void load() {
    std::call_once(once_, [this]() {
      lib_ = dlopen("libnccl.so.2", RTLD_NOW | RTLD_GLOBAL);
      if (!lib_) {
        lib_ = dlopen("libnccl.so", RTLD_NOW | RTLD_GLOBAL);
      }
      bind(fn_version_, "ncclGetVersion");
      bind(fn_uid_, "ncclGetUniqueId");
      bind(fn_init_, "ncclCommInitRank");
      bind(fn_init_config_, "ncclCommInitRankConfig");
      bind(fn_destroy_, "ncclCommDestroy");
      bind(fn_abort_, "ncclCommAbort");
      bind(fn_async_, "ncclCommGetAsyncError");
      bind(fn_gstart_, "ncclGroupStart");
      bind(fn_gend_, "ncclGroupEnd");
      bind(fn_send_, "ncclSend");
      bind(fn_recv_, "ncclRecv");
      bind(fn_bcast_, "ncclBroadcast");
      bind(fn_ar_, "ncclAllReduce");
      bind(fn_reduce_, "ncclReduce");
      bind(fn_ag_, "ncclAllGather");
      bind(fn_rs_, "ncclReduceScatter");
      bind(fn_premul_, "ncclRedOpCreatePreMulSum");
      bind(fn_opdestroy_, "ncclRedOpDestroy");
      bind(fn_errstr_, "ncclGetErrorString");
    });
  }

  std::once_flag once_;
  void* lib_ = nullptr;
  NcclResult (*fn_version_)(int*) = nullptr;
  NcclResult (*fn_uid_)(NcclUniqueId*) = nullptr;
  NcclResult (*fn_init_)(NcclComm**, int, NcclUniqueId, int) = nullptr;
  NcclResult (*fn_init_config_)(NcclComm**, int, NcclUniqueId, int, RawNcclConfig*) = nullptr;
  NcclResult (*fn_destroy_)(NcclComm*) = nullptr;
  NcclResult (*fn_abort_)(NcclComm*) = nullptr;
  NcclResult (*fn_async_)(NcclComm*, NcclResult*) = nullptr;
  NcclResult (*fn_gstart_)() = nullptr;
  NcclResult (*fn_gend_)() = nullptr;
  NcclResult (*fn_send_)(const void*, size_t, NcclDataType, int, NcclComm*, cudaStream_t) = nullptr;
  NcclResult (*fn_recv_)(void*, size_t, NcclDataType, int, NcclComm*, cudaStream_t) = nullptr;
  NcclResult (*fn_bcast_)(const void*, void*, size_t, NcclDataType, int, NcclComm*, cudaStream_t) = nullptr;
  NcclResult (*fn_ar_)(const void*, void*, size_t, NcclDataType, NcclRedOp, NcclComm*, cudaStream_t) = nullptr;
  NcclResult (*fn_reduce_)(const void*, void*, size_t, NcclDataType, NcclRedOp, int, NcclComm*, cudaStream_t) = nullptr;
  NcclResult (*fn_ag_)(const void*, void*, size_t, NcclDataType, NcclComm*, cudaStream_t) = nullptr;
  NcclResult (*fn_rs_)(const void*, void*, size_t, NcclDataType, NcclRedOp, NcclComm*, cudaStream_t) = nullptr;
  NcclResult (*fn_premul_)(NcclRedOp*, void*, NcclDataType, int, NcclComm*) = nullptr;
  NcclResult (*fn_opdestroy_)(NcclRedOp, NcclComm*) = nullptr;
  const char* (*fn_errstr_)(NcclResult) = nullptr;
};

} // namespace

namespace {
std::mutex& nccl_override_mu() {
  static std::mutex m;
  return m;
}
std::shared_ptr<NcclApi>& nccl_override() {
  static std::shared_ptr<NcclApi> p;
  return p;
}
} // namespace

std::shared_ptr<NcclApi> NcclApi::current() {
  std::lock_guard<std::mutex> g(nccl_override_mu());
  return nccl_override() ? nccl_override() : real();
}
void NcclApi::install(std::shared_ptr<NcclApi> fake) {
  std::lock_guard<std::mutex> g(nccl_override_mu());
  nccl_override() = std::move(fake);
}

std::shared_ptr<NcclApi> NcclApi::real() {
  static std::shared_ptr<NcclApi> inst = std::make_shared<RealNccl>();
  return inst;
}

} // namespace b200c
