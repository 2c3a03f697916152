// Test fakes of the CUDA runtime, the CUDA driver and NCCL, installable from
// Python, so that the CUDA backend's host logic - bootstrap, stream / event
// protocol, routing, graph bookkeeping, watchdog, hint parsing - runs on a
// machine without a GPU. Nothing is launched: the fake runtime is told what
// would have been launched and keeps a log of every call.
//
// Parity: the gMock seams of the reference's backend unit tests,
// comms/torchcomms/ncclx/tests/unit/cpp/mocks/NcclxMock.hpp:26 and CudaMock.hpp,
// driving TorchCommNCCLXTest / TorchWorkNCCLXQueueTest / GraphEventTrackerTest /
// HintParsingTest.
#include "py_common.hpp"

#include <sys/mman.h>
#include <unistd.h>

#include <cstdlib>
#include <cstring>
#include <map>
#include <mutex>
#include <set>
#include <sstream>

#include "../cuda/driver_api.hpp"
#include "../cuda/nccl_api.hpp"

namespace b200c {

namespace {

std::string handle_name(const char* prefix, const void* p) {
  std::ostringstream o;
  o << prefix << reinterpret_cast<uintptr_t>(p);
  return o.str();
}

class FakeRuntime final : public CudaApi {
 public:
  // ---- what tests script
  void set_capturing(bool on, unsigned long long graph_id) {
    std::lock_guard<std::mutex> g(mu_);
    capturing_ = on;
    graph_id_ = graph_id;
  }
  void set_stuck(bool on) {
    std::lock_guard<std::mutex> g(mu_);
    stuck_ = on;
  }
  // Runs the callbacks a destroyed graph would have run.
  int destroy_graph(unsigned long long graph_id) {
    std::vector<std::pair<cudaHostFn_t, void*>> todo;
    {
      std::lock_guard<std::mutex> g(mu_);
      auto range = retained_.equal_range(graph_id);
      for (auto it = range.first; it != range.second; ++it) todo.push_back(it->second);
      retained_.erase(graph_id);
    }
    for (auto& cb : todo) cb.first(cb.second);
    return static_cast<int>(todo.size());
  }
  std::vector<std::string> log() {
    std::lock_guard<std::mutex> g(mu_);
    return log_;
  }
  void clear_log() {
    std::lock_guard<std::mutex> g(mu_);
    log_.clear();
  }
  int live_events() {
    std::lock_guard<std::mutex> g(mu_);
    return static_cast<int>(events_.size());
  }
  int events_created() {
    std::lock_guard<std::mutex> g(mu_);
    return static_cast<int>(next_event_ - 1);
  }
  void set_current_stream(uintptr_t s) {
    std::lock_guard<std::mutex> g(mu_);
    current_ = reinterpret_cast<cudaStream_t>(s);
  }

  // ---- CudaApi
  bool is_real() override { return false; }
  void noteLaunch(const char* what, cudaStream_t s) override {
    std::lock_guard<std::mutex> g(mu_);
    launched_since_record_[s] = true;
    log_.push_back("launch " + std::string(what) + " " + handle_name("s", s));
  }
  cudaStream_t currentStream(int) override {
    std::lock_guard<std::mutex> g(mu_);
    return current_;
  }
  cudaError_t eventCreate(cudaEvent_t* e, unsigned) override {
    std::lock_guard<std::mutex> g(mu_);
    *e = reinterpret_cast<cudaEvent_t>(next_event_++);
    events_.insert(*e);
    return cudaSuccess;
  }
  cudaError_t eventDestroy(cudaEvent_t e) override {
    std::lock_guard<std::mutex> g(mu_);
    events_.erase(e);
    end_like_.erase(e);
    return cudaSuccess;
  }
  cudaError_t eventRecord(cudaEvent_t e, cudaStream_t s) override {
    std::lock_guard<std::mutex> g(mu_);
    // An event recorded right behind a launch marks the end of an operation;
    // while "stuck" such events never complete.
    end_like_[e] = launched_since_record_[s] && stuck_;
    launched_since_record_[s] = false;
    log_.push_back("record " + handle_name("e", e) + " " + handle_name("s", s));
    return cudaSuccess;
  }
  cudaError_t eventQuery(cudaEvent_t e) override {
    std::lock_guard<std::mutex> g(mu_);
    auto it = end_like_.find(e);
    return it != end_like_.end() && it->second ? cudaErrorNotReady : cudaSuccess;
  }
  cudaError_t eventSynchronize(cudaEvent_t) override { return cudaSuccess; }
  cudaError_t streamWaitEvent(cudaStream_t s, cudaEvent_t e) override {
    std::lock_guard<std::mutex> g(mu_);
    log_.push_back("wait " + handle_name("s", s) + " " + handle_name("e", e));
    return cudaSuccess;
  }
  cudaError_t streamIsCapturing(cudaStream_t, bool* capturing, unsigned long long* graph_id) override {
    std::lock_guard<std::mutex> g(mu_);
    *capturing = capturing_;
    *graph_id = capturing_ ? graph_id_ : 0;
    return cudaSuccess;
  }
  const char* errorString(cudaError_t e) override { return e == cudaSuccess ? "ok" : "fake runtime error"; }
  cudaError_t getDeviceCount(int* n) override {
    *n = 8;
    return cudaSuccess;
  }
  cudaError_t setDevice(int) override { return cudaSuccess; }
  cudaError_t deviceSynchronize() override {
    std::lock_guard<std::mutex> g(mu_);
    launched_since_record_.clear();  // everything launched so far has finished
    return cudaSuccess;
  }
  cudaError_t streamPriorityRange(int* least, int* greatest) override {
    *least = 0;
    *greatest = -5;
    return cudaSuccess;
  }
  cudaError_t streamCreateWithPriority(cudaStream_t* s, unsigned, int priority) override {
    std::lock_guard<std::mutex> g(mu_);
    *s = reinterpret_cast<cudaStream_t>(next_stream_++);
    log_.push_back("stream_create " + handle_name("s", *s) + " priority " + std::to_string(priority));
    return cudaSuccess;
  }
  cudaError_t streamDestroy(cudaStream_t) override { return cudaSuccess; }
  cudaError_t streamSynchronize(cudaStream_t s) override {
    std::lock_guard<std::mutex> g(mu_);
    log_.push_back("sync " + handle_name("s", s));
    return cudaSuccess;
  }
  cudaError_t mallocDevice(void** p, size_t bytes) override {
    *p = std::calloc(1, bytes);
    return *p != nullptr ? cudaSuccess : cudaErrorMemoryAllocation;
  }
  cudaError_t freeDevice(void* p) override {
    std::free(p);
    return cudaSuccess;
  }
  cudaError_t memsetDevice(void* p, int v, size_t bytes) override {
    std::memset(p, v, bytes);
    return cudaSuccess;
  }
  cudaError_t hostAllocMapped(void** host, void** dev, size_t bytes) override {
    *host = std::calloc(1, bytes);
    *dev = *host;
    return *host != nullptr ? cudaSuccess : cudaErrorMemoryAllocation;
  }
  cudaError_t freeHost(void* p) override {
    std::free(p);
    return cudaSuccess;
  }
  cudaError_t exchangeCaptureMode(cudaStreamCaptureMode*) override { return cudaSuccess; }
  cudaError_t streamCaptureGraph(cudaStream_t, cudaGraph_t* graph) override {
    std::lock_guard<std::mutex> g(mu_);
    *graph = capturing_ ? reinterpret_cast<cudaGraph_t>(static_cast<uintptr_t>(graph_id_)) : nullptr;
    return cudaSuccess;
  }
  cudaError_t graphRetainCallback(cudaGraph_t graph, cudaHostFn_t destroy, void* arg) override {
    std::lock_guard<std::mutex> g(mu_);
    retained_.emplace(static_cast<unsigned long long>(reinterpret_cast<uintptr_t>(graph)), std::make_pair(destroy, arg));
    log_.push_back("graph_retain " + handle_name("g", graph));
    return cudaSuccess;
  }

 private:
  std::mutex mu_;
  std::vector<std::string> log_;
  std::set<cudaEvent_t> events_;
  std::map<cudaEvent_t, bool> end_like_;
  std::map<cudaStream_t, bool> launched_since_record_;
  std::multimap<unsigned long long, std::pair<cudaHostFn_t, void*>> retained_;
  uintptr_t next_event_ = 1, next_stream_ = 0x100;
  cudaStream_t current_ = reinterpret_cast<cudaStream_t>(0x10);
  bool capturing_ = false, stuck_ = false;
  unsigned long long graph_id_ = 0;
};

class FakeNccl final : public NcclApi {
 public:
  explicit FakeNccl(std::shared_ptr<FakeRuntime> rt) : rt_(std::move(rt)) {}
  std::vector<std::string> log() {
    std::lock_guard<std::mutex> g(mu_);
    return log_;
  }
  std::map<std::string, std::string> last_config() {
    std::lock_guard<std::mutex> g(mu_);
    return last_config_;
  }
  void set_async_error(int code) { async_error_.store(code); }

  bool available() override { return true; }
  std::string version() override { return "2.28.9-fake"; }
  NcclResult getUniqueId(NcclUniqueId* id) override {
    std::memset(id->internal, 0x5a, sizeof(id->internal));
    return kNcclSuccess;
  }
  NcclResult commInitRank(NcclComm** comm, int nranks, NcclUniqueId, int rank) override {
    note("ncclCommInitRank nranks=" + std::to_string(nranks) + " rank=" + std::to_string(rank));
    *comm = reinterpret_cast<NcclComm*>(static_cast<uintptr_t>(0x7000 + next_comm_++));
    return kNcclSuccess;
  }
  NcclResult commInitRankConfig(NcclComm** comm, int nranks, NcclUniqueId, int rank, const NcclConfig& c) override {
    {
      std::lock_guard<std::mutex> g(mu_);
      last_config_.clear();
      auto put = [this](const char* k, int v) {
        if (v != NcclConfig::kUnset) last_config_[k] = std::to_string(v);
      };
      put("blocking", c.blocking);
      put("cgaClusterSize", c.cgaClusterSize);
      put("minCTAs", c.minCTAs);
      put("maxCTAs", c.maxCTAs);
      put("splitShare", c.splitShare);
      put("trafficClass", c.trafficClass);
      put("collnetEnable", c.collnetEnable);
      put("CTAPolicy", c.CTAPolicy);
      put("shrinkShare", c.shrinkShare);
      put("nvlsCTAs", c.nvlsCTAs);
      put("nChannelsPerNetPeer", c.nChannelsPerNetPeer);
      put("nvlinkCentricSched", c.nvlinkCentricSched);
      if (!c.netName.empty()) last_config_["netName"] = c.netName;
      if (!c.commName.empty()) last_config_["commName"] = c.commName;
    }
    note("ncclCommInitRankConfig nranks=" + std::to_string(nranks) + " rank=" + std::to_string(rank));
    *comm = reinterpret_cast<NcclComm*>(static_cast<uintptr_t>(0x7000 + next_comm_++));
    return kNcclSuccess;
  }
  NcclResult commDestroy(NcclComm*) override { return note("ncclCommDestroy"); }
  NcclResult commAbort(NcclComm*) override { return note("ncclCommAbort"); }
  NcclResult commGetAsyncError(NcclComm*, NcclResult* e) override {
    *e = static_cast<NcclResult>(async_error_.load());
    return kNcclSuccess;
  }
  NcclResult groupStart() override { return note("ncclGroupStart"); }
  NcclResult groupEnd() override { return note("ncclGroupEnd"); }
  NcclResult send(const void*, size_t n, NcclDataType, int peer, NcclComm*, cudaStream_t s) override {
    return op("ncclSend count=" + std::to_string(n) + " peer=" + std::to_string(peer), s);
  }
  NcclResult recv(void*, size_t n, NcclDataType, int peer, NcclComm*, cudaStream_t s) override {
    return op("ncclRecv count=" + std::to_string(n) + " peer=" + std::to_string(peer), s);
  }
  NcclResult broadcast(const void*, void*, size_t n, NcclDataType, int root, NcclComm*, cudaStream_t s) override {
    return op("ncclBroadcast count=" + std::to_string(n) + " root=" + std::to_string(root), s);
  }
  NcclResult allReduce(const void*, void*, size_t n, NcclDataType, NcclRedOp o, NcclComm*, cudaStream_t s) override {
    return op("ncclAllReduce count=" + std::to_string(n) + " op=" + std::to_string(static_cast<int>(o)), s);
  }
  NcclResult reduce(const void*, void*, size_t n, NcclDataType, NcclRedOp, int root, NcclComm*, cudaStream_t s) override {
    return op("ncclReduce count=" + std::to_string(n) + " root=" + std::to_string(root), s);
  }
  NcclResult allGather(const void*, void*, size_t n, NcclDataType, NcclComm*, cudaStream_t s) override {
    return op("ncclAllGather sendcount=" + std::to_string(n), s);
  }
  NcclResult reduceScatter(const void*, void*, size_t n, NcclDataType, NcclRedOp, NcclComm*, cudaStream_t s) override {
    return op("ncclReduceScatter recvcount=" + std::to_string(n), s);
  }
  NcclResult redOpCreatePreMulSum(NcclRedOp* o, void*, NcclDataType, NcclComm*) override {
    *o = static_cast<NcclRedOp>(100);
    return note("ncclRedOpCreatePreMulSum");
  }
  NcclResult redOpDestroy(NcclRedOp, NcclComm*) override { return note("ncclRedOpDestroy"); }
  std::string errorString(NcclResult r) override { return "fake ncclResult " + std::to_string(static_cast<int>(r)); }

 private:
  NcclResult note(const std::string& what) {
    std::lock_guard<std::mutex> g(mu_);
    log_.push_back(what);
    return kNcclSuccess;
  }
  NcclResult op(const std::string& what, cudaStream_t s) {
    rt_->noteLaunch(what.substr(0, what.find(' ')).c_str(), s);
    return note(what);
  }
  std::shared_ptr<FakeRuntime> rt_;
  std::mutex mu_;
  std::vector<std::string> log_;
  std::map<std::string, std::string> last_config_;
  std::atomic<int> async_error_{0};
  int next_comm_ = 0;
};

// Virtual-memory and multicast calls succeed; address ranges are backed by
// ordinary host memory of this process, so code that clears or lays out a
// segment works, and exported handles are real file descriptors, so they can
// travel between rank processes over SCM_RIGHTS like the real ones.
class FakeDriver final : public DriverApi {
 public:
  explicit FakeDriver(bool multicast) : multicast_(multicast) {}
  bool available() override { return true; }
  CUresult memCreate(CUmemGenericAllocationHandle* h, size_t, const CUmemAllocationProp*) override {
    *h = next_handle_++;
    return CUDA_SUCCESS;
  }
  CUresult memRelease(CUmemGenericAllocationHandle) override { return CUDA_SUCCESS; }
  CUresult memAddressReserve(CUdeviceptr* ptr, size_t size, size_t) override {
    void* p = ::mmap(nullptr, size, PROT_READ | PROT_WRITE, MAP_PRIVATE | MAP_ANONYMOUS, -1, 0);
    if (p == MAP_FAILED) return CUDA_ERROR_OUT_OF_MEMORY;
    *ptr = reinterpret_cast<CUdeviceptr>(p);
    return CUDA_SUCCESS;
  }
  CUresult memAddressFree(CUdeviceptr ptr, size_t size) override {
    ::munmap(reinterpret_cast<void*>(ptr), size);
    return CUDA_SUCCESS;
  }
  CUresult memMap(CUdeviceptr, size_t, size_t, CUmemGenericAllocationHandle) override { return CUDA_SUCCESS; }
  CUresult memUnmap(CUdeviceptr, size_t) override { return CUDA_SUCCESS; }
  CUresult memSetAccess(CUdeviceptr, size_t, const CUmemAccessDesc*, size_t) override { return CUDA_SUCCESS; }
  CUresult memExportToShareableHandle(void* out, CUmemGenericAllocationHandle, CUmemAllocationHandleType) override {
    const int fd = ::memfd_create("b200c-fake-handle", 0);
    if (fd < 0) return CUDA_ERROR_OPERATING_SYSTEM;
    *static_cast<int*>(out) = fd;
    return CUDA_SUCCESS;
  }
  CUresult memImportFromShareableHandle(CUmemGenericAllocationHandle* h, void*, CUmemAllocationHandleType) override {
    *h = next_handle_++;
    return CUDA_SUCCESS;
  }
  CUresult memGetAllocationGranularity(size_t* g, const CUmemAllocationProp*, CUmemAllocationGranularity_flags) override {
    *g = 2u << 20;
    return CUDA_SUCCESS;
  }
  CUresult multicastCreate(CUmemGenericAllocationHandle* h, const CUmulticastObjectProp*) override {
    *h = next_handle_++;
    return CUDA_SUCCESS;
  }
  CUresult multicastAddDevice(CUmemGenericAllocationHandle, CUdevice) override { return CUDA_SUCCESS; }
  CUresult multicastBindMem(CUmemGenericAllocationHandle, size_t, CUmemGenericAllocationHandle, size_t, size_t) override {
    return CUDA_SUCCESS;
  }
  CUresult multicastUnbind(CUmemGenericAllocationHandle, CUdevice, size_t, size_t) override { return CUDA_SUCCESS; }
  CUresult multicastGetGranularity(size_t* g, const CUmulticastObjectProp*, CUmulticastGranularity_flags) override {
    *g = 2u << 20;
    return CUDA_SUCCESS;
  }
  CUresult deviceGet(CUdevice* dev, int ordinal) override {
    *dev = ordinal;
    return CUDA_SUCCESS;
  }
  CUresult deviceGetAttribute(int* v, CUdevice_attribute attr, CUdevice) override {
    *v = attr == CU_DEVICE_ATTRIBUTE_MULTICAST_SUPPORTED ? (multicast_ ? 1 : 0) : 1;
    return CUDA_SUCCESS;
  }
  std::string errorString(CUresult r) override { return "fake CUresult " + std::to_string(static_cast<int>(r)); }

 private:
  bool multicast_;
  std::atomic<CUmemGenericAllocationHandle> next_handle_{1};
};

struct FakeGpu {
  std::shared_ptr<FakeRuntime> runtime;
  std::shared_ptr<FakeNccl> nccl;
  std::shared_ptr<FakeDriver> driver;
};

} // namespace

void bind_fakes(py::module_& m) {
  py::class_<FakeGpu, std::shared_ptr<FakeGpu>>(m, "_FakeGpu")
      .def("log", [](FakeGpu& f) { return f.runtime->log(); })
      .def("clear_log", [](FakeGpu& f) { f.runtime->clear_log(); })
      .def("nccl_log", [](FakeGpu& f) { return f.nccl->log(); })
      .def("nccl_config", [](FakeGpu& f) { return f.nccl->last_config(); })
      .def("set_capturing", [](FakeGpu& f, bool on, unsigned long long id) { f.runtime->set_capturing(on, id); },
           py::arg("on"), py::arg("graph_id") = 1)
      .def("set_stuck", [](FakeGpu& f, bool on) { f.runtime->set_stuck(on); })
      .def("set_current_stream", [](FakeGpu& f, uintptr_t s) { f.runtime->set_current_stream(s); })
      .def("destroy_graph", [](FakeGpu& f, unsigned long long id) { return f.runtime->destroy_graph(id); },
           py::call_guard<py::gil_scoped_release>())
      .def("set_nccl_async_error", [](FakeGpu& f, int code) { f.nccl->set_async_error(code); })
      .def("live_events", [](FakeGpu& f) { return f.runtime->live_events(); })
      .def("events_created", [](FakeGpu& f) { return f.runtime->events_created(); });

  // Communicators created from now on run against the fakes ("b200" needs no GPU then).
  m.def("_install_fake_gpu", [](bool multicast) {
    auto f = std::make_shared<FakeGpu>();
    f->runtime = std::make_shared<FakeRuntime>();
    f->nccl = std::make_shared<FakeNccl>(f->runtime);
    f->driver = std::make_shared<FakeDriver>(multicast);
    CudaApi::install(f->runtime);
    NcclApi::install(f->nccl);
    DriverApi::install(f->driver);
    return f;
  }, py::arg("multicast") = true);
  m.def("_uninstall_fake_gpu", []() {
    CudaApi::install(nullptr);
    NcclApi::install(nullptr);
    DriverApi::install(nullptr);
  });
}

} // namespace b200c
