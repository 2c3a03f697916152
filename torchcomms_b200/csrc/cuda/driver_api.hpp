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

  static std::shared_ptr<CudaApi> real();
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
