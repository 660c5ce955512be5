// Peer-memory runtime and the fused data-parallel bucket kernel.
//
// One process per GPU.  Each rank allocates its flat parameter buffer, flat
// gradient buffer and a signal pad with cudaMalloc, exports them as CUDA IPC
// handles, and maps every peer's buffers.  Kernels then read and write peer
// memory directly over NVLink (plain ld/st with system scope, no TMA, no
// library collectives).
//
// dp_bucket_kernel replaces, for one bucket of parameters, the reference's
// ReduceGrads / AllReduceGrads -> optimizer Step -> BroadcastParams sequence
// (tensor/group.go:301-478, train/parallel.go:226-286, :366-393) with ONE
// kernel: handshake ("my gradients of this bucket are final") -> reduce-scatter
// by peer loads (each rank sums its 1/world slice over all ranks, in fp32) ->
// cast/scale + AdamW on the slice (optimizer state is sharded: a rank keeps
// master/m/v only for the slices it owns) -> all-gather by peer stores of the
// new bf16 parameters -> "done" signal.  It runs on a side stream as soon as
// backward has produced the bucket, so the transfer overlaps the rest of
// backward.  Every replica ends a step with bit-identical parameters, because
// each element is computed by exactly one rank (train/parallel.go:31-36 asks
// for bit-identical replicas).
//
// Waits on peers are bounded: when the limit passes the kernel ORs
// kErrPeerTimeout into the error word and returns; nothing traps or spins
// forever.  The host reads the word and aborts the step.
#include "common.cuh"
#include "runtime.h"
#include <cstring>

namespace mimir {

constexpr int kMaxRanks = 8;
static unsigned long long g_peer_wait_ns = 10000000000ull;  // default limit for peer waits: 10 s

__device__ __forceinline__ void st_release_sys(unsigned* p, unsigned v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ unsigned ld_acquire_sys(const unsigned* p) {
  unsigned v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ uint4 ld_sys_v4(const void* p) {
  uint4 v;
  asm volatile("ld.relaxed.sys.global.v4.u32 {%0, %1, %2, %3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p)
               : "memory");
  return v;
}
__device__ __forceinline__ void st_sys_v4(void* p, uint4 v) {
  asm volatile("st.relaxed.sys.global.v4.u32 [%0], {%1, %2, %3, %4};" ::"l"(p), "r"(v.x), "r"(v.y),
               "r"(v.z), "r"(v.w)
               : "memory");
}

// Waits until *flag >= want (wrap-safe), at most limit_ns.  Returns false on timeout.
__device__ __forceinline__ bool wait_flag(const unsigned* flag, unsigned want, unsigned long long limit_ns,
                                          unsigned* err) {
  if (static_cast<int>(ld_acquire_sys(flag) - want) >= 0) return true;
  const uint64_t t0 = global_timer_ns();
  for (;;) {
    for (int i = 0; i < 64; ++i) {
      if (static_cast<int>(ld_acquire_sys(flag) - want) >= 0) return true;
      __nanosleep(200);
    }
    if (global_timer_ns() - t0 > limit_ns) {
      raise_error(err, kErrPeerTimeout);
      return false;
    }
  }
}

struct DpBucketArgs {
  const __nv_bfloat16* grads[kMaxRanks];  // every rank's flat gradient buffer
  __nv_bfloat16* params[kMaxRanks];       // every rank's flat parameter buffer
  unsigned* sig[kMaxRanks];               // every rank's signal pad
  float* master;                          // local shards (elements of this rank's slices, packed)
  float* exp_avg;
  float* exp_avg_sq;
  const float* hyper;       // device: {lr, 1-beta1^t, sqrt(1-beta2^t), grad scale}
  const unsigned* epoch;    // device: current step number (flag value of this step)
  unsigned* block_counter;  // device: one word per bucket, zero between launches
  unsigned long long start;      // bucket start (elements) in the flat buffers
  unsigned long long count;      // bucket length, divisible by 8 * world
  unsigned long long decay_n;    // the first decay_n elements of the bucket get weight decay
  unsigned long long shard_off;  // start of this bucket's slice inside the local shard arrays
  float beta1, beta2, eps, wd;
  int rank, world;
  int slot_ready, slot_done;  // signal slots of this bucket: words [slot * kMaxRanks + sender]
  unsigned long long wait_ns;
};

__global__ void __launch_bounds__(256)
dp_bucket_kernel(DpBucketArgs a, unsigned* err) {
  __shared__ int s_ok;
  const unsigned epoch = *a.epoch;
  // ---- handshake: tell every rank that my gradients of this bucket are final
  if (blockIdx.x == 0 && threadIdx.x < a.world) {
    __threadfence_system();
    st_release_sys(a.sig[threadIdx.x] + a.slot_ready * kMaxRanks + a.rank, epoch);
  }
  if (threadIdx.x == 0) s_ok = 1;
  __syncthreads();
  if (threadIdx.x < a.world) {
    if (!wait_flag(a.sig[a.rank] + a.slot_ready * kMaxRanks + threadIdx.x, epoch, a.wait_ns, err))
      s_ok = 0;
  }
  __syncthreads();
  if (s_ok) {
    // ---- reduce-scatter + AdamW + all-gather on my slice
    const float lr = a.hyper[0], bc1 = a.hyper[1], bc2s = a.hyper[2], gscale = a.hyper[3];
    const unsigned long long slice = a.count / a.world;
    const unsigned long long s0 = a.start + slice * a.rank;  // flat index of my slice
    const unsigned long long n8 = slice / 8;
    const float step = lr / bc1;
    for (unsigned long long i = static_cast<unsigned long long>(blockIdx.x) * blockDim.x + threadIdx.x;
         i < n8; i += static_cast<unsigned long long>(gridDim.x) * blockDim.x) {
      const unsigned long long e = s0 + i * 8;  // flat element index
      uint4 gv[kMaxRanks];
#pragma unroll
      for (int r = 0; r < kMaxRanks; ++r)
        if (r < a.world) gv[r] = ld_sys_v4(a.grads[r] + e);
      float g[8] = {0, 0, 0, 0, 0, 0, 0, 0};
#pragma unroll
      for (int r = 0; r < kMaxRanks; ++r) {
        if (r < a.world) {
          float2 x0 = unpack_bf16x2(gv[r].x), x1 = unpack_bf16x2(gv[r].y), x2 = unpack_bf16x2(gv[r].z),
                 x3 = unpack_bf16x2(gv[r].w);
          g[0] += x0.x; g[1] += x0.y; g[2] += x1.x; g[3] += x1.y;
          g[4] += x2.x; g[5] += x2.y; g[6] += x3.x; g[7] += x3.y;
        }
      }
      const unsigned long long li = a.shard_off + i * 8;  // index into the local shards
      float4 p0 = *reinterpret_cast<float4*>(a.master + li), p1 = *reinterpret_cast<float4*>(a.master + li + 4);
      float4 m0 = *reinterpret_cast<float4*>(a.exp_avg + li), m1 = *reinterpret_cast<float4*>(a.exp_avg + li + 4);
      float4 v0 = *reinterpret_cast<float4*>(a.exp_avg_sq + li), v1 = *reinterpret_cast<float4*>(a.exp_avg_sq + li + 4);
      float p[8] = {p0.x, p0.y, p0.z, p0.w, p1.x, p1.y, p1.z, p1.w};
      float mm[8] = {m0.x, m0.y, m0.z, m0.w, m1.x, m1.y, m1.z, m1.w};
      float vv[8] = {v0.x, v0.y, v0.z, v0.w, v1.x, v1.y, v1.z, v1.w};
      const float wd = (e - a.start) < a.decay_n ? a.wd : 0.f;
      const float decay = 1.f - lr * wd;
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const float gj = g[j] * gscale;
        p[j] *= decay;
        mm[j] = a.beta1 * mm[j] + (1.f - a.beta1) * gj;
        vv[j] = a.beta2 * vv[j] + (1.f - a.beta2) * gj * gj;
        p[j] -= step * mm[j] / (sqrtf(vv[j]) / bc2s + a.eps);
      }
      *reinterpret_cast<float4*>(a.master + li) = make_float4(p[0], p[1], p[2], p[3]);
      *reinterpret_cast<float4*>(a.master + li + 4) = make_float4(p[4], p[5], p[6], p[7]);
      *reinterpret_cast<float4*>(a.exp_avg + li) = make_float4(mm[0], mm[1], mm[2], mm[3]);
      *reinterpret_cast<float4*>(a.exp_avg + li + 4) = make_float4(mm[4], mm[5], mm[6], mm[7]);
      *reinterpret_cast<float4*>(a.exp_avg_sq + li) = make_float4(vv[0], vv[1], vv[2], vv[3]);
      *reinterpret_cast<float4*>(a.exp_avg_sq + li + 4) = make_float4(vv[4], vv[5], vv[6], vv[7]);
      uint4 o;
      o.x = pack_bf16x2(p[0], p[1]); o.y = pack_bf16x2(p[2], p[3]);
      o.z = pack_bf16x2(p[4], p[5]); o.w = pack_bf16x2(p[6], p[7]);
#pragma unroll
      for (int r = 0; r < kMaxRanks; ++r)
        if (r < a.world) st_sys_v4(a.params[r] + e, o);
    }
  }
  // ---- the last block to finish tells every rank that my slice is written
  __threadfence_system();
  __syncthreads();
  __shared__ unsigned s_last;
  if (threadIdx.x == 0) s_last = atomicAdd(a.block_counter, 1u) == gridDim.x - 1 ? 1u : 0u;
  __syncthreads();
  if (s_last) {
    if (threadIdx.x == 0) *a.block_counter = 0;  // ready for the next launch
    if (threadIdx.x < a.world) {
      __threadfence_system();
      st_release_sys(a.sig[threadIdx.x] + a.slot_done * kMaxRanks + a.rank, epoch);
    }
  }
}

// Runs at the start of a step on the main stream: waits until every rank has
// finished writing its slices of every bucket in the previous step (so the local
// parameters are complete and nobody still reads the local gradients), then
// advances the epoch.
__global__ void dp_step_begin_kernel(unsigned* epoch, const unsigned* my_sig, int nslots_done,
                                     const int* done_slots, int world, unsigned long long wait_ns,
                                     unsigned* err) {
  const unsigned cur = *epoch;
  bool ok = true;
  if (cur != 0) {
    for (int i = threadIdx.x; i < nslots_done * world; i += blockDim.x) {
      const int slot = done_slots[i / world], r = i % world;
      if (!wait_flag(my_sig + slot * kMaxRanks + r, cur, wait_ns, err)) ok = false;
    }
  }
  __syncthreads();
  (void)ok;
  if (threadIdx.x == 0) *epoch = cur + 1;
}

// Test hook for the bounded wait: waits on a flag that nothing sets and reports
// through the error word.  Returns immediately after `limit_ns`.
__global__ void peer_wait_probe_kernel(const unsigned* flag, unsigned want, unsigned long long limit_ns,
                                       unsigned* status, unsigned* err) {
  status[0] = wait_flag(flag, want, limit_ns, err) ? 1u : 2u;
}

}  // namespace mimir

using namespace mimir;

// ---------------------------------------------------------------------------
// C ABI: peer memory
// ---------------------------------------------------------------------------
MIMIR_API int mimir_peer_alloc(long long bytes, void** out) {
  void* p = nullptr;
  if (cudaMalloc(&p, static_cast<size_t>(bytes)) != cudaSuccess) return refuse("peer alloc of %lld bytes failed", bytes);
  cudaMemset(p, 0, static_cast<size_t>(bytes));
  *out = p;
  return 0;
}
MIMIR_API int mimir_peer_free(void* p) { return cudaFree(p) == cudaSuccess ? 0 : -1; }

// handle: 64 bytes out
MIMIR_API int mimir_ipc_export(void* p, void* handle) {
  cudaIpcMemHandle_t h;
  if (cudaIpcGetMemHandle(&h, p) != cudaSuccess) return refuse("cudaIpcGetMemHandle failed");
  memcpy(handle, &h, sizeof(h));
  return 0;
}
MIMIR_API int mimir_ipc_open(const void* handle, void** out) {
  cudaIpcMemHandle_t h;
  memcpy(&h, handle, sizeof(h));
  void* p = nullptr;
  cudaError_t e = cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess);
  if (e != cudaSuccess) return refuse("cudaIpcOpenMemHandle failed: %s", cudaGetErrorString(e));
  *out = p;
  return 0;
}
MIMIR_API int mimir_ipc_close(void* p) { return cudaIpcCloseMemHandle(p) == cudaSuccess ? 0 : -1; }

MIMIR_API void mimir_set_peer_wait_ms(long long ms) {
  g_peer_wait_ns = static_cast<unsigned long long>(ms) * 1000000ull;
}

// ---------------------------------------------------------------------------
// C ABI: fused data-parallel bucket step
// ---------------------------------------------------------------------------
// ptrs: grads[world], params[world], sig[world] (device pointers valid in this process).
MIMIR_API int mimir_dp_bucket(void* const* grads, void* const* params, void* const* sig, float* master,
                              float* exp_avg, float* exp_avg_sq, const float* hyper, const void* epoch,
                              void* block_counter, long long start, long long count, long long decay_n,
                              long long shard_off, float beta1, float beta2, float eps, float wd, int rank,
                              int world, int slot_ready, int slot_done, int nblocks, cudaStream_t st) {
  if (world < 1 || world > kMaxRanks) return refuse("dp: world %d not in 1..%d", world, kMaxRanks);
  if (count % (8 * world) || start % 8 || decay_n % 8 || shard_off % 8)
    return refuse("dp: bucket range must be divisible by 8 * world");
  DpBucketArgs a;
  for (int r = 0; r < kMaxRanks; ++r) {
    a.grads[r] = r < world ? static_cast<const __nv_bfloat16*>(grads[r]) : nullptr;
    a.params[r] = r < world ? static_cast<__nv_bfloat16*>(params[r]) : nullptr;
    a.sig[r] = r < world ? static_cast<unsigned*>(sig[r]) : nullptr;
  }
  a.master = master; a.exp_avg = exp_avg; a.exp_avg_sq = exp_avg_sq;
  a.hyper = hyper;
  a.epoch = static_cast<const unsigned*>(epoch);
  a.block_counter = static_cast<unsigned*>(block_counter);
  a.start = start; a.count = count; a.decay_n = decay_n; a.shard_off = shard_off;
  a.beta1 = beta1; a.beta2 = beta2; a.eps = eps; a.wd = wd;
  a.rank = rank; a.world = world; a.slot_ready = slot_ready; a.slot_done = slot_done;
  a.wait_ns = g_peer_wait_ns;
  if (nblocks <= 0) nblocks = 32;
  dp_bucket_kernel<<<nblocks, 256, 0, st>>>(a, error_word_dev());
  count_launch();
  return cudaGetLastError() == cudaSuccess ? 0 : refuse("dp bucket launch failed");
}

MIMIR_API int mimir_dp_step_begin(void* epoch, const void* my_sig, int nslots_done, const int* done_slots_dev,
                                  int world, cudaStream_t st) {
  dp_step_begin_kernel<<<1, 128, 0, st>>>(static_cast<unsigned*>(epoch), static_cast<const unsigned*>(my_sig),
                                          nslots_done, done_slots_dev, world, g_peer_wait_ns, error_word_dev());
  count_launch();
  return 0;
}

// Bounded-wait self test: status[0] becomes 1 if the flag reached `want`, 2 if the wait ran out.
MIMIR_API int mimir_peer_wait_probe(const void* flag, unsigned want, long long limit_ms, void* status,
                                    cudaStream_t st) {
  peer_wait_probe_kernel<<<1, 1, 0, st>>>(static_cast<const unsigned*>(flag), want,
                                          static_cast<unsigned long long>(limit_ms) * 1000000ull,
                                          static_cast<unsigned*>(status), error_word_dev());
  count_launch();
  return 0;
}
