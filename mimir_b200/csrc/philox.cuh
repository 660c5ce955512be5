// Philox4x32-10 block function shared by the random-number kernels: counter = block index,
// key = the 64-bit seed; the four output words are elements 4*ctr .. 4*ctr+3 of the stream
// (reference: backend/internal/gen/gen.go:577-610).
#pragma once
#include <stdint.h>

namespace mimir {

__device__ __forceinline__ uint4 philox4x32_10(uint64_t ctr, uint64_t seed) {
  uint32_t c0 = static_cast<uint32_t>(ctr), c1 = static_cast<uint32_t>(ctr >> 32), c2 = 0, c3 = 0;
  uint32_t k0 = static_cast<uint32_t>(seed), k1 = static_cast<uint32_t>(seed >> 32);
#pragma unroll
  for (int r = 0; r < 10; ++r) {
    const uint32_t hi0 = __umulhi(0xD2511F53u, c0), lo0 = 0xD2511F53u * c0;
    const uint32_t hi1 = __umulhi(0xCD9E8D57u, c2), lo1 = 0xCD9E8D57u * c2;
    c0 = hi1 ^ c1 ^ k0; c1 = lo1; c2 = hi0 ^ c3 ^ k1; c3 = lo0;
    k0 += 0x9E3779B9u; k1 += 0xBB67AE85u;
  }
  return make_uint4(c0, c1, c2, c3);
}

// Uniform in [0, 1) from one output word: the top 24 bits / 2^24, as the host generator computes it.
__device__ __forceinline__ float philox_unit(uint32_t word) {
  return static_cast<float>(word >> 8) * (1.0f / 16777216.0f);
}

}  // namespace mimir
