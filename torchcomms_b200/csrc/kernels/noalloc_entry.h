// C entry point that allocates nothing: RMSNorm backward (dx and dw) with its
// scratch in a fixed device array inside this library.
//
// This has no counterpart in the reference; it exists for callers that must
// not allocate while they run. Two kinds of caller are meant: host code with
// no tensor library in the process (a C or C++ runtime that loads this shared
// object and owns raw device pointers), and code that runs while kernels that
// wait on other GPUs are in flight, where cudaMalloc / cudaFree would
// serialise the whole device behind those kernels.
//
// The ordinary entry point (ops.rmsnorm_bwd in the Python module) asks the
// tensor allocator for a [blocks, cols] fp32 buffer of partial weight
// gradients on every call. Here that buffer is a file-scope
// `static __device__` array, so:
//   * limits: cols <= B200C_NOALLOC_MAX_COLS (8192), cols % 8 == 0,
//     rows >= 1; the array holds 296 x 8192 floats (9.25 MiB of device memory
//     per device, reserved when the module is loaded). Larger shapes are
//     rejected with B200C_NOALLOC_TOO_LARGE; nothing is launched.
//   * the first call on each device looks the array's address up
//     (cudaGetSymbolAddress) with that device current. Make that first call
//     before any stream capture begins; later calls only launch kernels.
//   * nothing in the array needs to start at zero: every block overwrites its
//     whole row of partials before the second kernel reads it.
//   * calls that overlap on one device (two streams, two threads) share the
//     array and race; keep calls on one stream or order them with events.
#pragma once

#ifdef __cplusplus
extern "C" {
#endif

#define B200C_NOALLOC_MAX_COLS 8192
#define B200C_NOALLOC_MAX_BLOCKS 296

#define B200C_NOALLOC_OK 0
#define B200C_NOALLOC_TOO_LARGE (-1)   // cols beyond B200C_NOALLOC_MAX_COLS
#define B200C_NOALLOC_BAD_ARG (-2)     // null pointer, rows < 1, cols % 8 != 0, misaligned pointer
// Any positive value is a cudaError_t from the set-up or a launch.

// dy, x, dx: bf16 [rows, cols]; w, dw: bf16 [cols]; rstd: fp32 [rows] (from
// the forward pass). All device pointers. dy, x, w and dx are read and written
// 16 bytes at a time and must be 16-byte aligned; rstd (4 bytes) and dw
// (2 bytes) need only the alignment of their element type. Each of these is
// checked before anything is launched. `stream` is a cudaStream_t (null = the
// default stream). Uses the current device.
int b200c_rmsnorm_bwd_noalloc(const void* dy, const void* x, const void* w, const float* rstd, void* dx, void* dw,
                              int rows, int cols, void* stream);

// Human-readable text for a return value of the function above.
const char* b200c_noalloc_strerror(int code);

#ifdef __cplusplus
}
#endif
