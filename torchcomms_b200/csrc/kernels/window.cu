// Host-launched kernels behind the one-sided window API: put (device-issued
// stores into the peer's buffer), signal and wait_signal, plus the graph
// replay counter node.
//
// Replaces, in the reference: comms/ctran/algos/RMA/PutSignal.cu:16-174
// (put / signal / wait-signal kernels with 64-bit system-scope flags) and
// comms/torchcomms/device/cuda/AtomicAddKernel.cu:9-17 (replay counter).
#include "window.h"

namespace b200c {

namespace {

__global__ void __launch_bounds__(512) k_window_put(const DeviceWindow* w, const char* src, size_t bytes, int dst_rank,
                                                    size_t dst_off) {
  // Each block moves one contiguous slice.
  const size_t per = ((bytes + gridDim.x - 1) / gridDim.x + 15) / 16 * 16;
  const size_t b0 = static_cast<size_t>(blockIdx.x) * per;
  if (b0 >= bytes) return;
  const size_t n = bytes - b0 < per ? bytes - b0 : per;
  if (dst_off + bytes > w->bytes) {
    if (threadIdx.x == 0) w->status[0] = w->status[0] | kStatusBadArg;
    return;
  }
  block_copy(w->data[dst_rank] + dst_off + b0, src + b0, n);
}

__global__ void k_window_signal(const DeviceWindow* w, int dst_rank, int signal_id) {
  // Runs after the puts on the same stream: fence, then raise the signal.
  __threadfence_system();
  w->signal(dst_rank, signal_id, SignalOp::ADD, 1);
}

__global__ void k_window_wait(const DeviceWindow* w, int peer, int signal_id, uint64_t* expected) {
  const uint64_t want = expected[peer] + 1;
  if (w->wait_signal_from(peer, signal_id, CmpOp::GE, want)) {
    expected[peer] = want;
  }
}

__global__ void k_counter_inc(unsigned long long* counter) {
  // Mapped pinned host memory: the watchdog reads it without touching the GPU.
  atomicAdd_system(counter, 1ull);
}

__global__ void k_stamp_ns(unsigned long long* slot) {
  // The device's nanosecond timer into mapped pinned host memory: when the stream reached this point.
  unsigned long long t;
  asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
  *reinterpret_cast<volatile unsigned long long*>(slot) = t;
  __threadfence_system();
}

// Ping-pong through the device API; exists for tests of DeviceWindow.
__global__ void k_window_selftest(const DeviceWindow* wins, int nranks, RegisteredBuffer* srcs, size_t bytes) {
  const DeviceWindow& w = wins[blockIdx.y];
  const int next = (w.rank + 1) % nranks;
  w.put(0, srcs[blockIdx.y], 0, next, bytes, /*signal_id=*/1, /*counter_id=*/0, CoopScope::BLOCK);
  __shared__ int ok;
  if (threadIdx.x == 0) {
    ok = w.wait_signal(1, CmpOp::GE, 1) ? 1 : 0;
  }
  __syncthreads();
  w.barrier(0);
}

} // namespace

cudaError_t launch_window_put(const DeviceWindow* dev_window, const void* src, size_t bytes, int dst_rank,
                              size_t dst_off, cudaStream_t stream) {
  if (bytes == 0) return cudaSuccess;
  int blocks = static_cast<int>((bytes + (256 * 1024) - 1) / (256 * 1024));
  if (blocks < 1) blocks = 1;
  if (blocks > 128) blocks = 128;
  k_window_put<<<blocks, 512, 0, stream>>>(dev_window, static_cast<const char*>(src), bytes, dst_rank, dst_off);
  return cudaGetLastError();
}

cudaError_t launch_window_signal(const DeviceWindow* dev_window, int dst_rank, int signal_id, cudaStream_t stream) {
  k_window_signal<<<1, 1, 0, stream>>>(dev_window, dst_rank, signal_id);
  return cudaGetLastError();
}

cudaError_t launch_window_wait_signal(const DeviceWindow* dev_window, int peer, int signal_id, uint64_t* expected,
                                      cudaStream_t stream) {
  k_window_wait<<<1, 1, 0, stream>>>(dev_window, peer, signal_id, expected);
  return cudaGetLastError();
}

cudaError_t launch_timestamp(unsigned long long* mapped_slot, cudaStream_t stream) {
  k_stamp_ns<<<1, 1, 0, stream>>>(mapped_slot);
  return cudaGetLastError();
}

cudaError_t launch_counter_increment(unsigned long long* mapped_counter, cudaStream_t stream) {
  k_counter_inc<<<1, 1, 0, stream>>>(mapped_counter);
  return cudaGetLastError();
}

cudaError_t launch_window_selftest(const DeviceWindow* dev_windows, int nranks, RegisteredBuffer* dev_srcs, size_t bytes,
                                   cudaStream_t stream) {
  void* params[] = {&dev_windows, &nranks, &dev_srcs, &bytes};
  return cudaLaunchCooperativeKernel(reinterpret_cast<void*>(&k_window_selftest), dim3(1, nranks), dim3(128), params, 0,
                                     stream);
}

} // namespace b200c
