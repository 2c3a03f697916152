// Test kernels for the device-side point-to-point primitives (device_p2p.cuh):
// a pipelined broadcast along the ring built from send / forward / recv, and
// an exchange of LL packets with the next rank. Virtual ranks run as the
// blocks (blockIdx.y) of ONE cooperative launch on one GPU; on real ranks the
// same device code runs with one launch per GPU.
#include "p2p_selftest.h"

#include "device_p2p.cuh"

namespace b200c {

namespace {

// Rank `root` sends `bytes` from bufs[root] around the ring; every other rank ends with a copy in its buf.
// Warps 0-3 of a block send / forward, warps 4-7 receive at the end of the chain: both directions of a
// rank's traffic have their own thread group, as a collective kernel would arrange it.
__global__ void k_p2p_ring_broadcast(const P2pDev* devs, char* const* bufs, size_t bytes, int root) {
  const P2pDev& d = devs[blockIdx.y];
  const int n = d.comm.nranks, me = d.comm.rank;
  if (n < 2) return;
  const int next = (me + 1) % n, prev = (me + n - 1) % n;
  const int pos = (me - root + n) % n;  // position along the chain
  const int warp = threadIdx.x >> 5;
  if (warp < 4) {
    const ThreadGroup g = ThreadGroup::warps(0, 4, 1);
    if (pos == 0) {
      d.send(g, next, bufs[me], bytes);
    } else if (pos < n - 1) {
      d.forward(g, prev, next, bufs[me], bytes);
    }
  } else if (warp < 8) {
    const ThreadGroup g = ThreadGroup::warps(4, 4, 2);
    if (pos == n - 1) d.recv(g, prev, bufs[me], bytes);
  }
}

// Every rank writes `words` LL packets (payload = base + i, flag = epoch) into the next rank's table and
// reads what the previous rank wrote; out[i] receives the payloads.
__global__ void k_ll_exchange(const P2pDev* devs, uint64_t* const* tables, uint32_t* const* outs, int words, uint32_t epoch) {
  const P2pDev& d = devs[blockIdx.y];
  const int n = d.comm.nranks, me = d.comm.rank;
  const int next = (me + 1) % n, prev = (me + n - 1) % n;
  for (int i = threadIdx.x; i < words; i += blockDim.x) {
    ll_store(tables[next] + i, static_cast<uint32_t>(me * 100000 + i) + epoch, epoch);
  }
  for (int i = threadIdx.x; i < words; i += blockDim.x) {
    uint32_t v = 0;
    if (ll_load(d.comm, tables[me] + i, epoch, &v, prev)) outs[me][i] = v;
  }
}

} // namespace

cudaError_t launch_p2p_ring_broadcast(const P2pDevData* devs, char* const* bufs_dev, int nranks, size_t bytes, int root,
                                      cudaStream_t stream) {
  const P2pDev* devs_dev = static_cast<const P2pDev*>(devs);
  void* params[] = {&devs_dev, &bufs_dev, &bytes, &root};
  return cudaLaunchCooperativeKernel(reinterpret_cast<void*>(&k_p2p_ring_broadcast), dim3(1, nranks), dim3(256), params, 0, stream);
}

cudaError_t launch_ll_exchange(const P2pDevData* devs, uint64_t* const* tables_dev, uint32_t* const* outs_dev, int nranks,
                               int words, uint32_t epoch, cudaStream_t stream) {
  const P2pDev* devs_dev = static_cast<const P2pDev*>(devs);
  void* params[] = {&devs_dev, &tables_dev, &outs_dev, &words, &epoch};
  return cudaLaunchCooperativeKernel(reinterpret_cast<void*>(&k_ll_exchange), dim3(1, nranks), dim3(256), params, 0, stream);
}

} // namespace b200c
