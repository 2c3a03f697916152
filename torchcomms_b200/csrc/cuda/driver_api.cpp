// Real implementations of the driver / runtime seams.
#include "driver_api.hpp"

#include <dlfcn.h>

#include <ATen/cuda/CUDAContext.h>

#include <mutex>
#include <stdexcept>

namespace b200c {

namespace {

// Entry points are fetched through the runtime (cudaGetDriverEntryPoint), so
// the right ABI version of each symbol is picked and libcuda is never linked.
class RealDriver final : public DriverApi {
 public:
  bool available() override {
    load();
    return ok_;
  }

#define B200C_DRV(name) reinterpret_cast<decltype(&::name)>(sym(#name))

  CUresult memCreate(CUmemGenericAllocationHandle* h, size_t size, const CUmemAllocationProp* prop) override {
    return B200C_DRV(cuMemCreate)(h, size, prop, 0);
  }
  CUresult memRelease(CUmemGenericAllocationHandle h) override { return B200C_DRV(cuMemRelease)(h); }
  CUresult memAddressReserve(CUdeviceptr* ptr, size_t size, size_t align) override {
    return B200C_DRV(cuMemAddressReserve)(ptr, size, align, 0, 0);
  }
  CUresult memAddressFree(CUdeviceptr ptr, size_t size) override { return B200C_DRV(cuMemAddressFree)(ptr, size); }
  CUresult memMap(CUdeviceptr ptr, size_t size, size_t offset, CUmemGenericAllocationHandle h) override {
    return B200C_DRV(cuMemMap)(ptr, size, offset, h, 0);
  }
  CUresult memUnmap(CUdeviceptr ptr, size_t size) override { return B200C_DRV(cuMemUnmap)(ptr, size); }
  CUresult memSetAccess(CUdeviceptr ptr, size_t size, const CUmemAccessDesc* desc, size_t count) override {
    return B200C_DRV(cuMemSetAccess)(ptr, size, desc, count);
  }
  CUresult memExportToShareableHandle(void* out, CUmemGenericAllocationHandle h, CUmemAllocationHandleType t) override {
    return B200C_DRV(cuMemExportToShareableHandle)(out, h, t, 0);
  }
  CUresult memImportFromShareableHandle(CUmemGenericAllocationHandle* h, void* os_handle, CUmemAllocationHandleType t) override {
    return B200C_DRV(cuMemImportFromShareableHandle)(h, os_handle, t);
  }
  CUresult memGetAllocationGranularity(size_t* g, const CUmemAllocationProp* prop, CUmemAllocationGranularity_flags f) override {
    return B200C_DRV(cuMemGetAllocationGranularity)(g, prop, f);
  }
  CUresult multicastCreate(CUmemGenericAllocationHandle* h, const CUmulticastObjectProp* prop) override {
    return B200C_DRV(cuMulticastCreate)(h, prop);
  }
  CUresult multicastAddDevice(CUmemGenericAllocationHandle h, CUdevice dev) override {
    return B200C_DRV(cuMulticastAddDevice)(h, dev);
  }
  CUresult multicastBindMem(CUmemGenericAllocationHandle mc, size_t mc_off, CUmemGenericAllocationHandle mem, size_t mem_off, size_t size) override {
    return B200C_DRV(cuMulticastBindMem)(mc, mc_off, mem, mem_off, size, 0);
  }
  CUresult multicastUnbind(CUmemGenericAllocationHandle mc, CUdevice dev, size_t mc_off, size_t size) override {
    return B200C_DRV(cuMulticastUnbind)(mc, dev, mc_off, size);
  }
  CUresult multicastGetGranularity(size_t* g, const CUmulticastObjectProp* prop, CUmulticastGranularity_flags f) override {
    return B200C_DRV(cuMulticastGetGranularity)(g, prop, f);
  }
  CUresult deviceGet(CUdevice* dev, int ordinal) override { return B200C_DRV(cuDeviceGet)(dev, ordinal); }
  CUresult deviceGetAttribute(int* v, CUdevice_attribute attr, CUdevice dev) override {
    return B200C_DRV(cuDeviceGetAttribute)(v, attr, dev);
  }
  std::string errorString(CUresult r) override {
    const char* s = nullptr;
    auto fn = reinterpret_cast<decltype(&::cuGetErrorString)>(sym("cuGetErrorString", /*required=*/false));
    if (fn && fn(r, &s) == CUDA_SUCCESS && s) {
      return std::string(s) + " (CUresult " + std::to_string(static_cast<int>(r)) + ")";
    }
    return "CUresult " + std::to_string(static_cast<int>(r));
  }

 private:
  void load() {
    std::call_once(once_, [this]() {
      // The runtime must have a context before entry points are queried.
      ok_ = cudaFree(nullptr) == cudaSuccess;
    });
  }
  void* sym(const char* name, bool required = true) {
    load();
    void* fn = nullptr;
    if (ok_) {
      cudaDriverEntryPointQueryResult q;
      if (cudaGetDriverEntryPoint(name, &fn, cudaEnableDefault, &q) != cudaSuccess ||
          q != cudaDriverEntryPointSuccess) {
        fn = nullptr;
      }
    }
    if (fn == nullptr && required) {
      throw std::runtime_error(std::string("CUDA driver entry point not available: ") + name);
    }
    return fn;
  }
  std::once_flag once_;
  bool ok_ = false;
};

class RealCuda final : public CudaApi {
 public:
  cudaError_t eventCreate(cudaEvent_t* e, unsigned flags) override { return cudaEventCreateWithFlags(e, flags); }
  cudaError_t eventDestroy(cudaEvent_t e) override { return cudaEventDestroy(e); }
  cudaError_t eventRecord(cudaEvent_t e, cudaStream_t s) override { return cudaEventRecord(e, s); }
  cudaError_t eventQuery(cudaEvent_t e) override { return cudaEventQuery(e); }
  cudaError_t eventSynchronize(cudaEvent_t e) override { return cudaEventSynchronize(e); }
  cudaError_t streamWaitEvent(cudaStream_t s, cudaEvent_t e) override { return cudaStreamWaitEvent(s, e, 0); }
  cudaError_t streamIsCapturing(cudaStream_t s, bool* capturing, unsigned long long* graph_id) override {
    cudaStreamCaptureStatus st = cudaStreamCaptureStatusNone;
    unsigned long long id = 0;
    cudaError_t e = cudaStreamGetCaptureInfo(s, &st, &id);
    *capturing = st == cudaStreamCaptureStatusActive;
    *graph_id = id;
    return e;
  }
  const char* errorString(cudaError_t e) override { return cudaGetErrorString(e); }
};

} // namespace

cudaStream_t CudaApi::currentStream(int device) {
  return at::cuda::getCurrentCUDAStream(static_cast<c10::DeviceIndex>(device)).stream();
}

namespace {
std::mutex& override_mu() {
  static std::mutex m;
  return m;
}
std::shared_ptr<DriverApi>& driver_override() {
  static std::shared_ptr<DriverApi> p;
  return p;
}
std::shared_ptr<CudaApi>& cuda_override() {
  static std::shared_ptr<CudaApi> p;
  return p;
}
} // namespace

std::shared_ptr<DriverApi> DriverApi::current() {
  std::lock_guard<std::mutex> g(override_mu());
  return driver_override() ? driver_override() : real();
}
void DriverApi::install(std::shared_ptr<DriverApi> fake) {
  std::lock_guard<std::mutex> g(override_mu());
  driver_override() = std::move(fake);
}
std::shared_ptr<CudaApi> CudaApi::current() {
  std::lock_guard<std::mutex> g(override_mu());
  return cuda_override() ? cuda_override() : real();
}
void CudaApi::install(std::shared_ptr<CudaApi> fake) {
  std::lock_guard<std::mutex> g(override_mu());
  cuda_override() = std::move(fake);
}

std::shared_ptr<DriverApi> DriverApi::real() {
  static std::shared_ptr<DriverApi> inst = std::make_shared<RealDriver>();
  return inst;
}

std::shared_ptr<CudaApi> CudaApi::real() {
  static std::shared_ptr<CudaApi> inst = std::make_shared<RealCuda>();
  return inst;
}

} // namespace b200c
