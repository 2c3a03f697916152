// `_comms.P2pEmu`: virtual ranks on one GPU for the device-side point-to-point primitives
// (slot FIFOs, counters and LL tables in ordinary device memory; one cooperative launch per call).
#include "py_common.hpp"

#include <ATen/cuda/CUDAContext.h>

#include <cstring>

#include "../cuda/driver_api.hpp"
#include "../kernels/device_p2p.cuh"
#include "../kernels/p2p_selftest.h"

namespace b200c {

namespace {

class P2pEmu {
 public:
  P2pEmu(int nranks, int nslots, size_t slot_bytes, double wait_ms) : n_(nranks) {
    TORCH_CHECK(nranks >= 1 && nranks <= kMaxRanks && nslots >= 1 && slot_bytes >= 16 && slot_bytes % 16 == 0,
                "1..8 ranks, at least one slot, slot size a multiple of 16 bytes");
    B200C_CUDA_CHECK(cudaHostAlloc(reinterpret_cast<void**>(&status_host_), 64, cudaHostAllocMapped));
    std::memset(status_host_, 0, 64);
    uint32_t* sdev = nullptr;
    B200C_CUDA_CHECK(cudaHostGetDevicePointer(reinterpret_cast<void**>(&sdev), status_host_, 0));
    std::vector<char*> slots(n_);
    std::vector<uint64_t*> ready(n_), done(n_);
    for (int r = 0; r < n_; ++r) {
      slots[r] = static_cast<char*>(zeroed(static_cast<size_t>(n_) * nslots * slot_bytes));
      ready[r] = static_cast<uint64_t*>(zeroed(sizeof(uint64_t) * kMaxRanks));
      done[r] = static_cast<uint64_t*>(zeroed(sizeof(uint64_t) * kMaxRanks));
    }
    std::vector<P2pDevData> devs(n_);
    for (int r = 0; r < n_; ++r) {
      P2pDevData& d = devs[r];
      std::memset(&d, 0, sizeof(d));
      d.comm.rank = r;
      d.comm.nranks = n_;
      d.comm.status = sdev;
      d.comm.timeout_ns = static_cast<unsigned long long>(wait_ms * 1e6);
      for (int p = 0; p < n_; ++p) {
        d.slots[p] = slots[p];
        d.ready[p] = ready[p];
        d.done[p] = done[p];
      }
      d.sent = static_cast<uint64_t*>(zeroed(sizeof(uint64_t) * kMaxRanks));
      d.rcvd = static_cast<uint64_t*>(zeroed(sizeof(uint64_t) * kMaxRanks));
      d.nslots = nslots;
      d.slot_bytes = slot_bytes;
    }
    devs_dev_ = static_cast<P2pDevData*>(zeroed(sizeof(P2pDevData) * n_));
    B200C_CUDA_CHECK(cudaMemcpy(devs_dev_, devs.data(), sizeof(P2pDevData) * n_, cudaMemcpyHostToDevice));
    ptrs_dev_ = static_cast<void**>(zeroed(sizeof(void*) * 2 * kMaxRanks));
  }
  ~P2pEmu() {
    for (void* p : allocs_) cudaFree(p);
    if (status_host_) cudaFreeHost(status_host_);
  }

  // bufs[r]: uint8 buffer of rank r (the root's is the source); all of the same size.
  void ring_broadcast(std::vector<at::Tensor> bufs, int root) {
    TORCH_CHECK(static_cast<int>(bufs.size()) == n_ && root >= 0 && root < n_, "one buffer per rank");
    std::vector<void*> host(2 * kMaxRanks, nullptr);
    for (int r = 0; r < n_; ++r) {
      TORCH_CHECK(bufs[r].is_cuda() && bufs[r].is_contiguous() && bufs[r].nbytes() == bufs[0].nbytes(), "equal contiguous CUDA buffers");
      host[r] = bufs[r].data_ptr();
    }
    cudaStream_t s = at::cuda::getCurrentCUDAStream().stream();
    B200C_CUDA_CHECK(cudaMemcpyAsync(ptrs_dev_, host.data(), sizeof(void*) * 2 * kMaxRanks, cudaMemcpyHostToDevice, s));
    B200C_CUDA_CHECK(launch_p2p_ring_broadcast(devs_dev_, reinterpret_cast<char* const*>(ptrs_dev_), n_, bufs[0].nbytes(), root, s));
    B200C_CUDA_CHECK(cudaStreamSynchronize(s));
  }

  // tables[r]: int64 [words] LL table of rank r; outs[r]: int32 [words].
  void ll_exchange(std::vector<at::Tensor> tables, std::vector<at::Tensor> outs, int64_t epoch) {
    TORCH_CHECK(static_cast<int>(tables.size()) == n_ && static_cast<int>(outs.size()) == n_, "one table and one output per rank");
    const int words = static_cast<int>(outs[0].numel());
    std::vector<void*> host(2 * kMaxRanks, nullptr);
    for (int r = 0; r < n_; ++r) {
      TORCH_CHECK(tables[r].is_cuda() && tables[r].scalar_type() == at::kLong && tables[r].is_contiguous() && tables[r].numel() >= words &&
                      outs[r].is_cuda() && outs[r].scalar_type() == at::kInt && outs[r].is_contiguous() && outs[r].numel() == words,
                  "tables: int64 [words], outs: int32 [words]");
      host[r] = tables[r].data_ptr();
      host[kMaxRanks + r] = outs[r].data_ptr();
    }
    cudaStream_t s = at::cuda::getCurrentCUDAStream().stream();
    B200C_CUDA_CHECK(cudaMemcpyAsync(ptrs_dev_, host.data(), sizeof(void*) * 2 * kMaxRanks, cudaMemcpyHostToDevice, s));
    B200C_CUDA_CHECK(launch_ll_exchange(devs_dev_, reinterpret_cast<uint64_t* const*>(ptrs_dev_),
                                        reinterpret_cast<uint32_t* const*>(ptrs_dev_ + kMaxRanks), n_, words,
                                        static_cast<uint32_t>(epoch), s));
    B200C_CUDA_CHECK(cudaStreamSynchronize(s));
  }

  std::vector<uint32_t> status() const { return std::vector<uint32_t>(status_host_, status_host_ + 5); }

 private:
  void* zeroed(size_t bytes) {
    void* p = nullptr;
    B200C_CUDA_CHECK(cudaMalloc(&p, bytes));
    B200C_CUDA_CHECK(cudaMemset(p, 0, bytes));
    allocs_.push_back(p);
    return p;
  }
  int n_;
  P2pDevData* devs_dev_ = nullptr;
  void** ptrs_dev_ = nullptr;
  std::vector<void*> allocs_;
  uint32_t* status_host_ = nullptr;
};

} // namespace

void bind_p2p(py::module_& m) {
  py::class_<P2pEmu>(m, "P2pEmu")
      .def(py::init<int, int, size_t, double>(), py::arg("nranks"), py::arg("nslots") = 2, py::arg("slot_bytes") = 16384,
           py::arg("wait_ms") = 2000.0)
      .def("ring_broadcast", &P2pEmu::ring_broadcast, py::arg("bufs"), py::arg("root") = 0)
      .def("ll_exchange", &P2pEmu::ll_exchange, py::arg("tables"), py::arg("outs"), py::arg("epoch"))
      .def("status", &P2pEmu::status);
}

} // namespace b200c
