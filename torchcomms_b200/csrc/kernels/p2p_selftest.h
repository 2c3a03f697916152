// Launchers of the test kernels for device_p2p.cuh. All pointer arrays and descriptors are in device memory.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

namespace b200c {

struct P2pDevData;

cudaError_t launch_p2p_ring_broadcast(const P2pDevData* devs_dev, char* const* bufs_dev, int nranks, size_t bytes, int root,
                                      cudaStream_t stream);
cudaError_t launch_ll_exchange(const P2pDevData* devs_dev, uint64_t* const* tables_dev, uint32_t* const* outs_dev, int nranks,
                               int words, uint32_t epoch, cudaStream_t stream);

} // namespace b200c
