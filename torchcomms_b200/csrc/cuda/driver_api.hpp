// Seams over the CUDA driver (virtual-memory management, multicast) and the
// small part of the CUDA runtime the work tracker and watchdog use. Both are
// virtual so that unit tests run the host logic on a machine without a GPU by
// installing fakes; the real implementations resolve the driver entry points
// at first use (the extension has no link-time dependency on libcuda).
//
// Parity: comms/torchcomms/device/cuda/CudaApi.hpp (mockable runtime wrapper)
// and the lazy driver-symbol loader under comms/prims/platform.
#pragma once

#include <cuda.h>
#include <cuda_runtime.h>

#include <memory>
#include <string>

namespace b200c {

class DriverApi {
 public:
  virtual ~DriverApi() = default;
  virtual bool available() = 0;  // libcuda could be loaded and initialised
  virtual CUresult memCreate(CUmemGenericAllocationHandle* h, size_t size, const CUmemAllocationProp* prop) = 0;
  virtual CUresult memRelease(CUmemGenericAllocationHandle h) = 0;
  virtual CUresult memAddressReserve(CUdeviceptr* ptr, size_t size, size_t align) = 0;
  virtual CUresult memAddressFree(CUdeviceptr ptr, size_t size) = 0;
  virtual CUresult memMap(CUdeviceptr ptr, size_t size, size_t offset, CUmemGenericAllocationHandle h) = 0;
  virtual CUresult memUnmap(CUdeviceptr ptr, size_t size) = 0;
  virtual CUresult memSetAccess(CUdeviceptr ptr, size_t size, const CUmemAccessDesc* desc, size_t count) = 0;
  virtual CUresult memExportToShareableHandle(void* out, CUmemGenericAllocationHandle h, CUmemAllocationHandleType t) = 0;
  virtual CUresult memImportFromShareableHandle(CUmemGenericAllocationHandle* h, void* os_handle, CUmemAllocationHandleType t) = 0;
  virtual CUresult memGetAllocationGranularity(size_t* g, const CUmemAllocationProp* prop, CUmemAllocationGranularity_flags f) = 0;
  virtual CUresult multicastCreate(CUmemGenericAllocationHandle* h, const CUmulticastObjectProp* prop) = 0;
  virtual CUresult multicastAddDevice(CUmemGenericAllocationHandle h, CUdevice dev) = 0;
  virtual CUresult multicastBindMem(CUmemGenericAllocationHandle mc, size_t mc_off, CUmemGenericAllocationHandle mem, size_t mem_off, size_t size) = 0;
  virtual CUresult multicastUnbind(CUmemGenericAllocationHandle mc, CUdevice dev, size_t mc_off, size_t size) = 0;
  virtual CUresult multicastGetGranularity(size_t* g, const CUmulticastObjectProp* prop, CUmulticastGranularity_flags f) = 0;
  virtual CUresult deviceGet(CUdevice* dev, int ordinal) = 0;
  virtual CUresult deviceGetAttribute(int* v, CUdevice_attribute attr, CUdevice dev) = 0;
  virtual std::string errorString(CUresult r) = 0;

  static std::shared_ptr<DriverApi> real();
  // What new communicators use: the real driver unless a test installed a fake.
  static std::shared_ptr<DriverApi> current();
  static void install(std::shared_ptr<DriverApi> fake);   // nullptr restores the real one
};

// Runtime calls used by work objects and the watchdog.
class CudaApi {
 public:
  virtual ~CudaApi() = default;
  virtual cudaError_t eventCreate(cudaEvent_t* e, unsigned flags) = 0;
  virtual cudaError_t eventDestroy(cudaEvent_t e) = 0;
  virtual cudaError_t eventRecord(cudaEvent_t e, cudaStream_t s) = 0;
  virtual cudaError_t eventQuery(cudaEvent_t e) = 0;
  virtual cudaError_t eventSynchronize(cudaEvent_t e) = 0;
  virtual cudaError_t streamWaitEvent(cudaStream_t s, cudaEvent_t e) = 0;
  virtual cudaError_t streamIsCapturing(cudaStream_t s, bool* capturing, unsigned long long* graph_id) = 0;
  virtual const char* errorString(cudaError_t e) = 0;

  // False for test fakes: no CUDA context exists, so device guards are
  // skipped and kernels are not launched (the fake is told what would have
  // been launched instead).
  virtual bool is_real() { return true; }
  virtual void noteLaunch(const char* what, cudaStream_t s) {
    (void)what;
    (void)s;
  }
  // The calling thread's current stream on `device` (PyTorch's notion).
  virtual cudaStream_t currentStream(int device);

  // Resources of the CUDA backend. These have working defaults (the runtime
  // call itself), so a test fake overrides only what it wants to script.
  virtual cudaError_t getDeviceCount(int* n) { return cudaGetDeviceCount(n); }
  virtual cudaError_t setDevice(int d) { return cudaSetDevice(d); }
  virtual cudaError_t deviceSynchronize() { return cudaDeviceSynchronize(); }
  virtual cudaError_t streamPriorityRange(int* least, int* greatest) {
    return cudaDeviceGetStreamPriorityRange(least, greatest);
  }
  virtual cudaError_t streamCreateWithPriority(cudaStream_t* s, unsigned flags, int priority) {
    return cudaStreamCreateWithPriority(s, flags, priority);
  }
  virtual cudaError_t streamDestroy(cudaStream_t s) { return cudaStreamDestroy(s); }
  virtual cudaError_t streamSynchronize(cudaStream_t s) { return cudaStreamSynchronize(s); }
  virtual cudaError_t mallocDevice(void** p, size_t bytes) { return cudaMalloc(p, bytes); }
  virtual cudaError_t freeDevice(void* p) { return cudaFree(p); }
  virtual cudaError_t memsetDevice(void* p, int v, size_t bytes) { return cudaMemset(p, v, bytes); }
  // Pinned host memory that the device can address (status word, replay counters).
  virtual cudaError_t hostAllocMapped(void** host, void** dev, size_t bytes) {
    cudaError_t e = cudaHostAlloc(host, bytes, cudaHostAllocMapped);
    if (e != cudaSuccess) return e;
    return cudaHostGetDevicePointer(dev, *host, 0);
  }
  virtual cudaError_t freeHost(void* p) { return cudaFreeHost(p); }
  virtual cudaError_t exchangeCaptureMode(cudaStreamCaptureMode* mode) {
    return cudaThreadExchangeStreamCaptureMode(mode);
  }
  // The graph a capturing stream is building (null when not capturing).
  virtual cudaError_t streamCaptureGraph(cudaStream_t s, cudaGraph_t* graph) {
    cudaStreamCaptureStatus st = cudaStreamCaptureStatusNone;
    unsigned long long id = 0;
    *graph = nullptr;
    return cudaStreamGetCaptureInfo(s, &st, &id, graph, nullptr, nullptr);
  }
  // Ties `destroy(arg)` to the lifetime of `graph`: it runs (on a driver
  // thread) once the graph and every executable made from it are gone.
  virtual cudaError_t graphRetainCallback(cudaGraph_t graph, cudaHostFn_t destroy, void* arg) {
    cudaUserObject_t obj = nullptr;
    cudaError_t e = cudaUserObjectCreate(&obj, arg, destroy, 1, cudaUserObjectNoDestructorSync);
    if (e != cudaSuccess) return e;
    return cudaGraphRetainUserObject(graph, obj, 1, cudaGraphUserObjectMove);
  }

  static std::shared_ptr<CudaApi> real();
  static std::shared_ptr<CudaApi> current();
  static void install(std::shared_ptr<CudaApi> fake);
};

#define B200C_CU_CHECK(drv, expr)                                                          \
  do {                                                                                     \
    CUresult _r = (expr);                                                                  \
    if (_r != CUDA_SUCCESS) {                                                              \
      throw std::runtime_error(std::string(#expr) + " failed: " + (drv)->errorString(_r)); \
    }                                                                                      \
  } while (0)

#define B200C_CUDA_CHECK(expr)                                                                  \
  do {                                                                                          \
    cudaError_t _e = (expr);                                                                    \
    if (_e != cudaSuccess) {                                                                    \
      throw std::runtime_error(std::string(#expr) + " failed: " + cudaGetErrorString(_e));      \
    }                                                                                           \
  } while (0)

} // namespace b200c
