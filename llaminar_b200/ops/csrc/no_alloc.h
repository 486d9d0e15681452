// C entry point of the quantised GEMV that performs no device or host allocation.
//
// This function has no counterpart in the reference implementation; it exists for callers of this
// library that are not allowed to allocate: a host application that has handed every byte of device
// memory to its own arena (so cudaMalloc would fail or break its accounting), or a plug-in ABI whose
// contract forbids allocator calls on the serving path.  Such callers pass their own input and output
// buffers; the split-K partial sums and arrival counters that the kernel needs live in a fixed array
// inside the library image instead of in memory obtained at run time.
#pragma once
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

// Largest problem the built-in scratch covers: rows of activations and (128-padded) output features.
#define LLAMINAR_NOALLOC_MAX_ROWS 4
#define LLAMINAR_NOALLOC_MAX_N 65536

// out[m, n] (bf16, row stride n) = x[m, k] (bf16, row stride k) * dequant(W)[n, k]^T
//   w       weight chunks in this library's tile-major layout (see ops/layout.py), device pointer
//   fmt     format id (0 Q4_K, 1 Q5_K, 2 Q6_K, 3 Q8_0, 4 Q4_0, 5 IQ3_S)
//   stream  a cudaStream_t (nullptr: the legacy default stream)
// Returns 0 on success, a non-zero code otherwise (llaminar_gemv_noalloc_error() gives the text).
//
// * The scratch is ~1 MiB of device memory (LLAMINAR_NOALLOC_MAX_ROWS x LLAMINAR_NOALLOC_MAX_N floats plus
//   512 counters) that every GPU loading this library holds until the process exits.
// * Call with the device that owns w, x, out and `stream` current (cudaSetDevice): the scratch used and the launch
//   belong to the current device, and the first call checks that `out` lives there.
// * The first call on each device looks up the device address of that array; make that first call
//   before any stream capture begins on the device.
// * All calls share the one array.  Each call clears the part it uses on `stream` before the kernel runs,
//   so leftovers of an earlier call do no harm, but two calls that overlap on the GPU (different streams,
//   or different host threads without ordering) race on it: serialise them.
// * Problems with n (rounded up to 128) > LLAMINAR_NOALLOC_MAX_N or m > LLAMINAR_NOALLOC_MAX_ROWS are rejected.
int llaminar_gemv_noalloc(const void* w, int fmt, int n, int k, const void* x, int m, void* out, void* stream);
const char* llaminar_gemv_noalloc_error(void);

#ifdef __cplusplus
}
#endif
