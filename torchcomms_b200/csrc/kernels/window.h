// Launchers of the window kernels (host API path) and of the replay counter.
#pragma once

#include "device_window.cuh"

namespace b200c {

// All `dev_window` arguments are DEVICE pointers to a DeviceWindow.
cudaError_t launch_window_put(const DeviceWindow* dev_window, const void* src, size_t bytes, int dst_rank,
                              size_t dst_off, cudaStream_t stream);
cudaError_t launch_window_signal(const DeviceWindow* dev_window, int dst_rank, int signal_id, cudaStream_t stream);
// `expected` is a device array of nranks counters private to this rank: the
// number of signals from each peer that earlier waits already consumed.
cudaError_t launch_window_wait_signal(const DeviceWindow* dev_window, int peer, int signal_id, uint64_t* expected,
                                      cudaStream_t stream);
// One-thread kernel that increments a counter in mapped pinned host memory;
// captured into CUDA graphs so the watchdog can count replays.
cudaError_t launch_counter_increment(unsigned long long* mapped_counter, cudaStream_t stream);
// One thread writes the device's nanosecond timer (%globaltimer) into `mapped_slot` (mapped pinned host memory).
cudaError_t launch_timestamp(unsigned long long* mapped_slot, cudaStream_t stream);
// Test helper: every virtual rank puts to its right neighbour through the
// device API, waits for its own signal and joins a barrier (one cooperative
// launch over `nranks` windows on one GPU).
cudaError_t launch_window_selftest(const DeviceWindow* dev_windows, int nranks, RegisteredBuffer* dev_srcs, size_t bytes,
                                   cudaStream_t stream);

} // namespace b200c
