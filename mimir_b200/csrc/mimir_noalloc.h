// Column sums for callers that must not allocate device memory.
//
// This entry point has no counterpart in the reference framework.  It exists
// for hosts that embed the library where cudaMalloc is off limits: code running
// under a fixed memory plan drawn up at start-up (an inference server that hands
// every byte of the device to its own arena, a real-time loop that forbids
// calls which may synchronise the device or fail late), or a plug-in loaded by
// a process whose allocator the plug-in may not touch.  mimir_colsum() needs a
// scratch buffer from its caller; those callers have nowhere to get one.
#pragma once
#include <cuda_runtime.h>

#ifdef __cplusplus
extern "C" {
#endif

// Largest column count the built-in scratch array serves (64 partial rows of
// this many floats: 4 MiB that every GPU loading the library holds until exit).
#define MIMIR_COLSUM_NOALLOC_MAX_N 16384

// out[N] (bf16) = column sums of x[rows, N] (bf16, row pitch ld elements), or
// out += sums when accumulate != 0.  Same arithmetic as mimir_colsum(), but the
// partial sums live in a fixed array inside the library, so the call allocates
// nothing: no cudaMalloc, no cudaFree, no allocating library routine.
//
//  * N must be a multiple of 8 and at most MIMIR_COLSUM_NOALLOC_MAX_N, ld a
//    multiple of 8 and at least N; otherwise the call returns -1 and
//    mimir_last_error() says why.
//  * The first call on each device looks up the array's device address (once,
//    with that device current).  Make that first call outside any stream capture.
//  * All calls on a device share the one array and it keeps the last call's
//    contents.  Nothing in it has to start at zero (each call overwrites every
//    word it later reads), but two calls whose kernels overlap on the GPU, on
//    different streams, race on it: order them yourself.
// Returns 0 on success.
int mimir_colsum_noalloc(const void* x, int rows, int N, int ld, void* out, int accumulate,
                         cudaStream_t stream);

#ifdef __cplusplus
}
#endif
