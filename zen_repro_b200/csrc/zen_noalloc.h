// Allocation-free entry point of the native library.  It has no counterpart in the reference.
//
// Who needs it: code that must not allocate device memory when it calls in.  Examples are a host
// thread that runs inside someone else's memory plan (an inference server or an embedding host that
// has handed all device memory to its own pool), a process whose allocator may not be re-entered at
// the call site (a completion callback), and C callers that have no PyTorch allocator at all.  The
// regular entry points leave scratch to the caller, who normally gets it from torch's caching
// allocator; this one brings its own.
#pragma once
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

// Largest scratch the library keeps for this entry point, in floats (4 MiB).  A call needs
// ceil(rows / 32) * cols floats.
#define ZEN_COLSUM_NOALLOC_MAX_FLOATS (1u << 20)

// Column sums of a row-major [rows, cols] matrix: out[c] = sum_r a[r][c] (accumulate = 0) or
// out[c] += sum_r a[r][c] (accumulate != 0).  dtype: 0 fp32, 1 bf16, 2 fp16 (for `a` and `out`).
// `a` and `out` are device pointers supplied by the caller; cols must be a multiple of 8 and `a`
// 16-byte aligned.  Same arithmetic, launch shapes and summation order as zen_colsum.
//
// The partial sums live in a fixed array inside the library (one copy per GPU that loads the
// library, held until the process exits).  Consequences:
//   * nothing is allocated or freed here, by the CUDA runtime or by any library;
//   * sizes whose scratch would exceed ZEN_COLSUM_NOALLOC_MAX_FLOATS are refused with
//     ZEN_NOALLOC_TOO_LARGE and nothing is launched;
//   * all calls on one GPU share the array and it keeps the previous call's contents.  Every
//     element that a call reads is first written by that same call, so nothing has to be cleared;
//     but two calls that overlap on the GPU (different streams) would race on it: serialise them;
//   * the first call on each device looks up the array's device address (cudaGetSymbolAddress);
//     make that first call outside of any stream capture.
// Returns 0, a cudaError_t value, or one of the negative codes below.
#define ZEN_NOALLOC_TOO_LARGE (-20)
#define ZEN_NOALLOC_BAD_ARG (-21)
int zen_colsum_noalloc(const void* a, void* out, int rows, int cols, int accumulate, int dtype, void* stream);

// Text for the last non-zero code returned by zen_colsum_noalloc on this thread.
const char* zen_noalloc_last_error(void);

#ifdef __cplusplus
}
#endif
