// Host-side runtime shared by every launcher in the library: per-device error
// word in host-mapped memory, launch counter, TMA descriptor encoder, SM count.
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

#define MIMIR_API extern "C" __attribute__((visibility("default")))

namespace mimir {

// Device pointer of the calling thread's current device's error word (host-mapped).
unsigned* error_word_dev();
// Counts one kernel launch (graph capture counts once; replays are added by the host).
void count_launch(int n = 1);
int sm_count();
// Records a host-side argument refusal: sets kErrShape in the error word and
// keeps a message readable through mimir_last_error().
int refuse(const char* fmt, ...);

// Encodes a tiled tensor map for a row-major bf16/f16/f32/u8 tensor of `rank` dims.
// dims/strides are given innermost first; strides in BYTES for dims 1..rank-1.
// swizzle: 0 none, 1 32B, 2 64B, 3 128B.  Returns 0 on success.
int encode_tmap(CUtensorMap* out, const void* base, int elem_bytes, int rank, const uint64_t* dims,
                const uint64_t* strides_bytes, const uint32_t* box, int swizzle);

inline int ceil_div(int a, int b) { return (a + b - 1) / b; }

}  // namespace mimir
