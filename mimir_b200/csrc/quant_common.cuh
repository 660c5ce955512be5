// Pieces shared by the quantized-inference kernels: warp reductions, the argument block
// of the one-shot all-reduce, system-scope flag accesses and the bounded wait on a peer's flag.
#pragma once
#include "common.cuh"
#include "runtime.h"

namespace mimir {

constexpr int kQMaxRanks = 8;
constexpr int kQMaxBatch = 32;

__device__ __forceinline__ float warp_sum_f(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float warp_max_f(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

struct QArArgs {
  float* partial[kQMaxRanks];  // every rank's partial buffer [B][N] for this call (symmetric memory)
  unsigned* sig[kQMaxRanks];   // every rank's signal pad
  unsigned* epoch;             // device counter, advanced by this kernel
  unsigned* block_counter;     // device word, zero between launches
  const __nv_bfloat16* residual;  // [B][N] or nullptr
  __nv_bfloat16* out;             // [B][N] bf16
  int rank, world, slot;
  unsigned long long wait_ns;
};

__device__ __forceinline__ void st_release_sys_u32(unsigned* p, unsigned v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ unsigned ld_acquire_sys_u32(const unsigned* p) {
  unsigned v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ float4 ld_sys_f4(const float* p) {
  float4 v;
  asm volatile("ld.relaxed.sys.global.v4.f32 {%0, %1, %2, %3}, [%4];"
               : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w)
               : "l"(p)
               : "memory");
  return v;
}
__device__ __forceinline__ bool wait_flag_ge(const unsigned* flag, unsigned want, unsigned long long limit_ns,
                                             unsigned* err) {
  if (static_cast<int>(ld_acquire_sys_u32(flag) - want) >= 0) return true;
  const uint64_t t0 = global_timer_ns();
  for (;;) {
    for (int i = 0; i < 32; ++i) {
      if (static_cast<int>(ld_acquire_sys_u32(flag) - want) >= 0) return true;
      __nanosleep(100);
    }
    if (global_timer_ns() - t0 > limit_ns) { raise_error(err, kErrPeerTimeout); return false; }
  }
}


// Limit (nanoseconds) of every wait on another GPU's flag in these kernels; settable from the host.
unsigned long long q_peer_wait_ns();

}  // namespace mimir
