// GEMMs fused with their collective over NVLink peer memory (CTA-pair tcgen05
// kernel, see gemm2_sm100.cu for the pair protocol).
//
// COMM = 1  all-gather -> GEMM   (column-parallel / fully sharded weights).
//   C[M,N] = A[M,K] * W[N,K]^T with W sharded by rows over `world` ranks.  Every
//   rank keeps a full-size symmetric buffer and owns the rows of its shard in it.
//   A gather warp in every CTA copies its slice of each remote shard from the
//   owner's buffer into the local one with plain peer loads and bumps a per-shard
//   counter; the TMA producer waits for the counters of the shards a tile needs,
//   so tiles of the local shard start at once and the copy of shard s+1 overlaps
//   the math on shard s.  Each remote byte crosses NVLink once per GPU.
//   (Reference: matmulRule + allGather, tensor/layout.go:629-714, reshard.go:307-336.)
//
// COMM = 2  GEMM -> reduce-scatter  (row-parallel products, sharded weight grads).
//   Each rank computes a full-size partial C; rank o owns rows [o*M/world, ...).
//   The epilogue TMA-stores every finished bf16 sub-tile straight into the owner's
//   staging slab [source rank][rows][N] (peer memory), overlapping the transfer
//   with the remaining tiles; after a flag exchange every CTA sums the `world`
//   slabs of its rows in fp32 and writes the bf16 result.
//   (Reference: reduceScatter of partial sums, tensor/reshard.go:242-302.)
//
//   Slab reuse: a rank that has summed its slabs of call k publishes "read k" to every
//   peer (second half of the signal pad); the epilogue of call k+1 waits (bounded) for the
//   owner's "read k" before its first store into that owner's slab, so back-to-back calls
//   on the same object need no host barrier and no other collective in between.
//
// No TMA *load* touches peer memory with any cluster-wide qualifier: remote data is
// read with ld.relaxed.sys and written by TMA stores or st; all waits are bounded.
#include "gemm_pair.cuh"

namespace mimir {

constexpr int kCommRanks = 8;
constexpr int kCommThreads = 352;  // TMA warp, MMA warp, 8 epilogue warps, gather warp
constexpr int kCommEpiWarps = 8;
constexpr int kGatherInFlight = 16;   // 16-byte peer loads a gather lane keeps in flight
constexpr int kCommReadFlags = 512;  // word offset of the "owner has read call k" flags in a signal pad

struct CommArgs {
  // all-gather: every rank's full-size W buffer (rank r's shard is valid in buffer r)
  const __nv_bfloat16* w_full[kCommRanks];
  unsigned* shard_count;  // [world] arrivals per shard, monotonic
  // reduce-scatter: staging slabs and flags
  __nv_bfloat16* stage_local;  // [world][rows_per_rank][N] on this rank
  unsigned* sig[kCommRanks];   // every rank's signal pad
  __nv_bfloat16* out;          // [rows_per_rank][N] reduced result on this rank
  unsigned* epoch;             // device word: number of finished calls
  unsigned* done_count;        // device word, zero between calls
  int rank, world, rows_per_rank, slot;
  unsigned long long wait_ns;
};

struct TmArr {
  CUtensorMap m[kCommRanks];
};

__device__ __forceinline__ uint4 ld_peer_v4(const void* p) {
  uint4 v;
  asm volatile("ld.relaxed.sys.global.v4.u32 {%0, %1, %2, %3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p)
               : "memory");
  return v;
}
__device__ __forceinline__ unsigned ld_acquire_gpu(const unsigned* p) {
  unsigned v;
  asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ unsigned ld_acquire_sys_c(const unsigned* p) {
  unsigned v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void st_release_sys_c(unsigned* p, unsigned v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
// Bounded wait until *p >= want (wrap-safe); gpu scope for local counters.
template <bool SYS>
__device__ __forceinline__ bool wait_count(const unsigned* p, unsigned want, unsigned long long limit_ns,
                                           unsigned* err) {
  auto rd = [&]() { return SYS ? ld_acquire_sys_c(p) : ld_acquire_gpu(p); };
  if (static_cast<int>(rd() - want) >= 0) return true;
  const uint64_t t0 = global_timer_ns();
  for (;;) {
    for (int i = 0; i < 32; ++i) {
      if (static_cast<int>(rd() - want) >= 0) return true;
      __nanosleep(100);
    }
    if (global_timer_ns() - t0 > limit_ns) {
      raise_error(err, kErrPeerTimeout);
      return false;
    }
  }
}

template <int BN, bool A_MN, bool B_MN, int STAGES, int COMM>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kCommThreads, 1)
gemm_comm_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                 const __grid_constant__ CUtensorMap tmC, const __grid_constant__ TmArr tmStage, GemmEpi ep,
                 CommArgs cm, int M, int N, int K, unsigned* err) {
  constexpr int BNH = BN / 2;
  constexpr int A_BYTES = kBM * kBK * 2;
  constexpr int B_BYTES = BNH * kBK * 2;
  constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
  constexpr uint32_t TMEM_COLS = 2 * BN;
  constexpr uint32_t IDESC = make_idesc_bf16(2 * kBM, BN, A_MN, B_MN);

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  uint8_t* out_ring = smem + STAGES * STAGE_BYTES;
  uint64_t* full = reinterpret_cast<uint64_t*>(out_ring + kCommEpiWarps * 2 * 4096);
  uint64_t* empty = full + STAGES;
  uint64_t* tfull = empty + STAGES;
  uint64_t* tempty = tfull + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tempty + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  __shared__ unsigned s_flag;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t cta = cluster_ctarank();
  const int pair = static_cast<int>(cluster_id_x()), npairs = static_cast<int>(nclusters_x());
  const int m_tiles = (M + 2 * kBM - 1) / (2 * kBM), n_tiles = (N + BN - 1) / BN;
  const int kb_total = (K + kBK - 1) / kBK;
  const int units = m_tiles * n_tiles;
  const unsigned epoch = *cm.epoch;  // calls finished before this one
  const int rpr = cm.rows_per_rank;

  // COMM 1 walks the N-tiles starting at the local shard, all M-tiles of one N-tile in a row
  auto decode = [&](int u, int& m_idx, int& n_idx) {
    if (COMM == 1) {
      const int first = (cm.rank * rpr) / BN;
      m_idx = u % m_tiles;
      n_idx = (u / m_tiles + first) % n_tiles;
    } else {
      n_idx = u % n_tiles;
      m_idx = u / n_tiles;
    }
  };

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(&tfull[a], 1);
      mbar_init(&tempty[a], 2 * kCommEpiWarps);
    }
    *abort_flag = 0;
    fence_mbar_init();
  }
  if (warp == 1) {
    tmem_alloc_pair(tmem_slot, TMEM_COLS);
    tmem_relinquish_pair();
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    if (lane == 0) {
      tma_prefetch_desc(&tmA);
      tma_prefetch_desc(&tmB);
      uint32_t it = 0;
      bool ok = true;
      for (int u = pair; u < units && ok; u += npairs) {
        int m_idx, n_idx;
        decode(u, m_idx, n_idx);
        const int m0 = m_idx * 2 * kBM + static_cast<int>(cta) * kBM;
        const int n0 = n_idx * BN + static_cast<int>(cta) * BNH;
        if (COMM == 1) {
          // the B rows of this CTA must have arrived in the local buffer
          const int lo = n0 / rpr, hi = min(N - 1, n0 + BNH - 1) / rpr;
          for (int s = lo; s <= hi && ok; ++s)
            if (s != cm.rank)
              ok = wait_count<false>(cm.shard_count + s, gridDim.x, cm.wait_ns, err);
          if (!ok) { *abort_flag = 1; break; }
          asm volatile("fence.proxy.async;" ::: "memory");  // copied rows -> visible to the TMA loads
        }
        for (int kb = 0; kb < kb_total; ++kb, ++it) {
          const int s = it % STAGES;
          const uint32_t ph = (it / STAGES) & 1;
          if (!mbar_wait(&empty[s], ph ^ 1, abort_flag, err)) { ok = false; break; }
          uint8_t* sA = smem + s * STAGE_BYTES;
          uint8_t* sB = sA + A_BYTES;
          const uint32_t bar = map_to_cta(smem_u32(&full[s]), 0);
          if (cta == 0) mbar_arrive_expect_tx(&full[s], 2 * STAGE_BYTES);
          if (A_MN) {
#pragma unroll
            for (int c = 0; c < kBM / 64; ++c)
              tma_load_2d_pair(sA + c * (kBK * 128), &tmA, bar, m0 + c * 64, kb * kBK);
          } else {
            tma_load_2d_pair(sA, &tmA, bar, kb * kBK, m0);
          }
          if (B_MN) {
#pragma unroll
            for (int c = 0; c < BNH / 64; ++c)
              tma_load_2d_pair(sB + c * (kBK * 128), &tmB, bar, n0 + c * 64, kb * kBK);
          } else {
            tma_load_2d_pair(sB, &tmB, bar, kb * kBK, n0);
          }
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0 && cta == 0) {
      uint32_t it = 0, ti = 0;
      bool ok = true;
      for (int u = pair; u < units && ok; u += npairs, ++ti) {
        const uint32_t acc = ti & 1, acc_ph = (ti >> 1) & 1;
        if (!mbar_wait(&tempty[acc], acc_ph ^ 1, abort_flag, err)) break;
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * BN;
        for (int kb = 0; kb < kb_total; ++kb, ++it) {
          const int s = it % STAGES;
          const uint32_t ph = (it / STAGES) & 1;
          if (!mbar_wait(&full[s], ph, abort_flag, err)) { ok = false; break; }
          tc_fence_after();
          const uint32_t sA = smem_u32(smem + s * STAGE_BYTES);
          const uint32_t sB = sA + A_BYTES;
          const uint64_t adesc = A_MN ? make_smem_desc_sw128(sA, kBK * 128, 1024) : make_smem_desc_sw128(sA, 16, 1024);
          const uint64_t bdesc = B_MN ? make_smem_desc_sw128(sB, kBK * 128, 1024) : make_smem_desc_sw128(sB, 16, 1024);
#pragma unroll
          for (int k = 0; k < kBK / 16; ++k)
            umma_ss_pair(d_tmem, adesc + (A_MN ? k * 128 : k * 2), bdesc + (B_MN ? k * 128 : k * 2), IDESC,
                         (kb > 0 || k > 0) ? 1u : 0u);
          umma_commit_pair(&empty[s], 3);
        }
        if (ok) umma_commit_pair(&tfull[acc], 3);
      }
    }
  } else if (warp < 2 + kCommEpiWarps) {
    const int q = warp & 3, half = (warp - 2) >> 2;
    const uint32_t tempty_leader0 = map_to_cta(smem_u32(&tempty[0]), 0);
    const uint32_t tempty_leader1 = map_to_cta(smem_u32(&tempty[1]), 0);
    uint32_t ti = 0, ring = 0;
    uint32_t owner_ready = 0;  // owners whose "read" flag of the previous call this warp has seen
    uint8_t* wbuf = out_ring + (warp - 2) * 2 * 4096;
    for (int u = pair; u < units; u += npairs, ++ti) {
      int m_idx, n_idx;
      decode(u, m_idx, n_idx);
      const uint32_t acc = ti & 1, acc_ph = (ti >> 1) & 1;
      if (!mbar_wait(&tfull[acc], acc_ph, abort_flag, err)) break;
      tc_fence_after();
      const int row0 = m_idx * 2 * kBM + static_cast<int>(cta) * kBM + q * 32;
      const uint32_t taddr = tmem_base + acc * BN + half * (BN / 2) + (static_cast<uint32_t>(q * 32) << 16);
      const int col_base = n_idx * BN + half * (BN / 2);
      if (COMM == 2) {
        // bf16 partial sub-tiles go to the staging slab of the rank that owns these rows
        const int owner = min(row0 / rpr, cm.world - 1);
        const CUtensorMap* tmo = &tmStage.m[owner];
        if (!((owner_ready >> owner) & 1u)) {
          // the owner must have finished summing the previous call's slabs before they are overwritten
          if (lane == 0)
            wait_count<true>(cm.sig[cm.rank] + kCommReadFlags + cm.slot * kCommRanks + owner, epoch, cm.wait_ns, err);
          __syncwarp();
          owner_ready |= 1u << owner;
        }
#pragma unroll 1
        for (int c = 0; c < BN / 128; ++c) {
          uint32_t r0[32], r1[32], pk[32];
          tmem_ld32(taddr + c * 64, r0);
          tmem_ld32(taddr + c * 64 + 32, r1);
          tmem_ld_wait();
          const int col0 = col_base + c * 64;
          if (col0 >= N || row0 >= M) continue;
#pragma unroll
          for (int g = 0; g < 16; ++g) {
            pk[g] = pack_bf16x2(__uint_as_float(r0[2 * g]), __uint_as_float(r0[2 * g + 1]));
            pk[16 + g] = pack_bf16x2(__uint_as_float(r1[2 * g]), __uint_as_float(r1[2 * g + 1]));
          }
          uint8_t* buf = wbuf + (ring & 1) * 4096;
          if (lane == 0) bulk_wait_group_read<1>();
          __syncwarp();
          const uint32_t base = smem_u32(buf) + lane * 128;
#pragma unroll
          for (int uu = 0; uu < 8; ++uu)
            st_shared_v4(base + ((uu ^ (lane & 7)) << 4), pk[4 * uu], pk[4 * uu + 1], pk[4 * uu + 2], pk[4 * uu + 3]);
          fence_proxy_async_smem();
          __syncwarp();
          if (lane == 0) {
            tma_store_3d(tmo, buf, col0, row0 - owner * rpr, cm.rank);
            bulk_commit_group();
          }
          ++ring;
        }
      } else {
        drain_accumulator_tma<BN / 128>(ep, &tmC, &tmC, taddr, row0, col_base, M, N, wbuf, ring, lane);
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster(acc ? tempty_leader1 : tempty_leader0);
    }
    // complete (not just read) every store before the flags go out
    if (lane == 0) asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");
  } else if (COMM == 1) {
    // gather warp: copy this CTA's slice of every remote shard into the local buffer
    const size_t shard_units = static_cast<size_t>(rpr) * K * 2 / 16;  // 16-byte units per shard
    const size_t per = (shard_units + gridDim.x - 1) / gridDim.x;
    const size_t u0 = per * blockIdx.x, u1 = min(shard_units, u0 + per);
    uint4* local = reinterpret_cast<uint4*>(const_cast<__nv_bfloat16*>(cm.w_full[cm.rank]));
    for (int k = 1; k < cm.world; ++k) {
      const int s = (cm.rank + k) % cm.world;
      const uint4* src = reinterpret_cast<const uint4*>(cm.w_full[s]) + static_cast<size_t>(s) * shard_units;
      uint4* dst = local + static_cast<size_t>(s) * shard_units;
      // NVLink round trips take microseconds: the link only fills when enough loads are in flight
      // (148 gather warps x 32 lanes x kGatherInFlight x 16 bytes, about 1.2 MB at 16)
      for (size_t i = u0 + lane; i < u1; i += 32 * kGatherInFlight) {
        uint4 v[kGatherInFlight];
#pragma unroll
        for (int j = 0; j < kGatherInFlight; ++j)
          if (i + j * 32 < u1) v[j] = ld_peer_v4(src + i + j * 32);
#pragma unroll
        for (int j = 0; j < kGatherInFlight; ++j)
          if (i + j * 32 < u1) dst[i + j * 32] = v[j];
      }
      __threadfence();
      __syncwarp();
      if (lane == 0) atomicAdd(cm.shard_count + s, 1u);
    }
  }

  tc_fence_before();
  __syncthreads();

  if (COMM == 2) {
    // ---- flag exchange, then sum the slabs every rank sent for my rows
    if (threadIdx.x == 0) {
      __threadfence_system();
      s_flag = atomicAdd(cm.done_count, 1u) == gridDim.x - 1 ? 1u : 0u;
    }
    __syncthreads();
    if (s_flag && threadIdx.x < cm.world) {
      __threadfence_system();
      st_release_sys_c(cm.sig[threadIdx.x] + cm.slot * kCommRanks + cm.rank, epoch + 1);
    }
    __syncthreads();
    if (threadIdx.x == 0) s_flag = 1;
    __syncthreads();
    if (threadIdx.x < cm.world) {
      if (!wait_count<true>(cm.sig[cm.rank] + cm.slot * kCommRanks + threadIdx.x, epoch + 1, cm.wait_ns, err))
        s_flag = 0;
    }
    __syncthreads();
    if (s_flag) {
      const size_t units = static_cast<size_t>(rpr) * N / 8;  // 8 bf16 per 16-byte unit
      const uint4* slabs = reinterpret_cast<const uint4*>(cm.stage_local);
      uint4* out = reinterpret_cast<uint4*>(cm.out);
      for (size_t i = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < units;
           i += static_cast<size_t>(gridDim.x) * blockDim.x) {
        float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
#pragma unroll
        for (int r = 0; r < kCommRanks; ++r) {
          if (r < cm.world) {
            const uint4 v = ld_peer_v4(slabs + static_cast<size_t>(r) * units + i);
            const float2 a = unpack_bf16x2(v.x), b = unpack_bf16x2(v.y), c = unpack_bf16x2(v.z), d = unpack_bf16x2(v.w);
            acc[0] += a.x; acc[1] += a.y; acc[2] += b.x; acc[3] += b.y;
            acc[4] += c.x; acc[5] += c.y; acc[6] += d.x; acc[7] += d.y;
          }
        }
        uint4 o;
        o.x = pack_bf16x2(acc[0], acc[1]); o.y = pack_bf16x2(acc[2], acc[3]);
        o.z = pack_bf16x2(acc[4], acc[5]); o.w = pack_bf16x2(acc[6], acc[7]);
        out[i] = o;
      }
    }
    __syncthreads();
  }
  // ---- the last CTA to get here re-arms the counters and closes the call
  if (threadIdx.x == 0) {
    __threadfence();
    const unsigned target = COMM == 2 ? 2 * gridDim.x - 1 : gridDim.x - 1;
    if (atomicAdd(cm.done_count, 1u) == target) {
      *cm.done_count = 0;
      if (COMM == 1)
        for (int s = 0; s < cm.world; ++s) cm.shard_count[s] = 0;
      if (COMM == 2) {
        // every CTA of this rank has summed its part: the slabs may be overwritten by call epoch + 1
        __threadfence_system();
        for (int p = 0; p < cm.world; ++p)
          st_release_sys_c(cm.sig[p] + kCommReadFlags + cm.slot * kCommRanks + cm.rank, epoch + 1);
      }
      __threadfence();
      *cm.epoch = epoch + 1;
    }
  }
  cluster_sync_all();
  if (warp == 1) {
    __syncwarp();
    tc_fence_after();
    tmem_dealloc_pair(tmem_base, TMEM_COLS);
  }
}

template <int BN, bool A_MN, bool B_MN, int STAGES, int COMM>
static int launch_comm(const CUtensorMap& tmA, const CUtensorMap& tmB, const CUtensorMap& tmC, const TmArr& tmS,
                       const GemmEpi& ep, const CommArgs& cm, int M, int N, int K, cudaStream_t stream) {
  constexpr int SMEM = STAGES * (kBM * kBK * 2 + (BN / 2) * kBK * 2) + kCommEpiWarps * 2 * 4096 + 1024 + 256;
  auto kern = gemm_comm_kernel<BN, A_MN, B_MN, STAGES, COMM>;
  static int max_pairs = 0;
  if (max_pairs == 0) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM) != cudaSuccess)
      return refuse("cannot reserve %d bytes of shared memory", SMEM);
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(2 * (sm_count() / 2));
    cfg.blockDim = dim3(kCommThreads);
    cfg.dynamicSmemBytes = SMEM;
    int n = 0;
    if (cudaOccupancyMaxActiveClusters(&n, kern, &cfg) != cudaSuccess || n <= 0) {
      cudaGetLastError();
      n = sm_count() / 2;
    }
    max_pairs = n < sm_count() / 2 ? n : sm_count() / 2;
  }
  // every CTA takes part in the gather / flag phases, so the grid must be fully resident
  const int units = ceil_div(M, 2 * kBM) * ceil_div(N, BN);
  int pairs = units < max_pairs ? units : max_pairs;
  if (pairs < 1) pairs = 1;
  kern<<<2 * pairs, kCommThreads, SMEM, stream>>>(tmA, tmB, tmC, tmS, ep, cm, M, N, K, error_word_dev());
  count_launch();
  return cudaGetLastError() == cudaSuccess ? 0 : refuse("fused gemm launch failed");
}

static unsigned long long g_comm_wait_ns = 10000000000ull;

}  // namespace mimir

using namespace mimir;

MIMIR_API void mimir_comm_set_peer_wait_ms(long long ms) {
  g_comm_wait_ns = static_cast<unsigned long long>(ms) * 1000000ull;
}

static int encode2d(CUtensorMap* tm, const void* base, int rows, int cols, int ld, bool mn_major, int box_rows) {
  uint64_t dims[2], strides[1] = {static_cast<uint64_t>(ld) * 2};
  uint32_t box[2];
  if (mn_major) { dims[0] = rows; dims[1] = cols; box[0] = 64; box[1] = kBK; }   // stored [K][rows]
  else { dims[0] = cols; dims[1] = rows; box[0] = kBK; box[1] = static_cast<uint32_t>(box_rows); }
  return encode_tmap(tm, base, 2, 2, dims, strides, box, 3);
}

// C[M,N] = epilogue(A[M,K] * W[N,K]^T) with W row-sharded: w_full[r] is rank r's full-size
// buffer (its own shard valid); rows_per_rank = N / world.  shard_count: `world` zeroed
// words, epoch / done_count: zeroed words (device memory owned by the caller, one set
// per concurrent call site).  Flags follow mimir_gemm_bf16.
MIMIR_API int mimir_gemm_allgather_b(const void* A, void* const* w_full, void* C, int M, int N, int K, int lda,
                                     int ldc, const void* bias, const void* aux, int ldaux, void* aux_out,
                                     int flags, void* shard_count, void* epoch, void* done_count, int rank,
                                     int world, cudaStream_t stream) {
  if (N % world || (N / world) % 8 || K % 8 || N % 8 || ldc % 8 || lda % 8)
    return refuse("gemm_allgather: N must divide by world, sizes by 8");
  if (flags & (kOutF32 | kAccumulate)) return refuse("gemm_allgather: bf16 output without accumulation only");
  CUtensorMap tmA, tmB, tmC;
  TmArr tmS = {};
  if (encode2d(&tmA, A, M, K, lda, false, kBM)) return -1;
  if (encode2d(&tmB, w_full[rank], N, K, K, false, 128)) return -1;
  {
    uint64_t dims[2] = {static_cast<uint64_t>(N), static_cast<uint64_t>(M)}, strides[1] = {static_cast<uint64_t>(ldc) * 2};
    uint32_t box[2] = {64, 32};
    if (encode_tmap(&tmC, C, 2, 2, dims, strides, box, 3)) return -1;
  }
  GemmEpi ep = {};
  ep.C = C; ep.bias = static_cast<const __nv_bfloat16*>(bias); ep.aux = static_cast<const __nv_bfloat16*>(aux);
  ep.aux_out = static_cast<__nv_bfloat16*>(aux_out); ep.ldc = ldc; ep.ldaux = ldaux;
  ep.flags = flags & ~kWritePre;  // the side output is not wired into this variant
  ep.alpha = 1.f;
  CommArgs cm = {};
  for (int r = 0; r < world; ++r) cm.w_full[r] = static_cast<const __nv_bfloat16*>(w_full[r]);
  cm.shard_count = static_cast<unsigned*>(shard_count);
  cm.epoch = static_cast<unsigned*>(epoch);
  cm.done_count = static_cast<unsigned*>(done_count);
  cm.rank = rank; cm.world = world; cm.rows_per_rank = N / world; cm.wait_ns = g_comm_wait_ns;
  return launch_comm<256, false, false, 5, 1>(tmA, tmB, tmC, tmS, ep, cm, M, N, K, stream);
}

// Reduce-scatter of C = A * B^T over ranks along the rows of C: rank o receives rows
// [o * M / world, ...) summed over all ranks in out[M / world][N] (bf16).
//   a_mn / b_mn as in mimir_gemm_bf16.  stage[r]: rank r's staging buffer
//   [world][M / world][N] bf16 (symmetric memory), sig[r]: rank r's signal pad.
MIMIR_API int mimir_gemm_reduce_scatter(const void* A, const void* B, int M, int N, int K, int lda, int ldb,
                                        int a_mn, int b_mn, void* const* stage, void* const* sig, void* out,
                                        void* epoch, void* done_count, int rank, int world, int slot,
                                        cudaStream_t stream) {
  if (M % world || (M / world) % 32 || N % 8 || lda % 8 || ldb % 8)
    return refuse("gemm_reduce_scatter: M / world must be a multiple of 32, sizes multiples of 8");
  if (a_mn && !b_mn) return refuse("gemm_reduce_scatter: NT, NN and TN products only");
  CUtensorMap tmA, tmB, tmC;
  TmArr tmS = {};
  if (encode2d(&tmA, A, M, K, lda, a_mn, kBM)) return -1;
  if (encode2d(&tmB, B, N, K, ldb, b_mn, 128)) return -1;
  tmC = tmA;
  const int rpr = M / world;
  for (int r = 0; r < world; ++r) {
    uint64_t d3[3] = {static_cast<uint64_t>(N), static_cast<uint64_t>(rpr), static_cast<uint64_t>(world)};
    uint64_t s3[2] = {static_cast<uint64_t>(N) * 2, static_cast<uint64_t>(rpr) * N * 2};
    uint32_t b3[3] = {64, 32, 1};
    if (encode_tmap(&tmS.m[r], stage[r], 2, 3, d3, s3, b3, 3)) return -1;
  }
  GemmEpi ep = {};
  ep.alpha = 1.f;
  CommArgs cm = {};
  cm.stage_local = static_cast<__nv_bfloat16*>(stage[rank]);
  for (int r = 0; r < world; ++r) cm.sig[r] = static_cast<unsigned*>(sig[r]);
  cm.out = static_cast<__nv_bfloat16*>(out);
  cm.epoch = static_cast<unsigned*>(epoch);
  cm.done_count = static_cast<unsigned*>(done_count);
  cm.rank = rank; cm.world = world; cm.rows_per_rank = rpr; cm.slot = slot; cm.wait_ns = g_comm_wait_ns;
  if (!a_mn && !b_mn) return launch_comm<256, false, false, 5, 2>(tmA, tmB, tmC, tmS, ep, cm, M, N, K, stream);
  if (!a_mn) return launch_comm<256, false, true, 5, 2>(tmA, tmB, tmC, tmS, ep, cm, M, N, K, stream);
  return launch_comm<256, true, true, 5, 2>(tmA, tmB, tmC, tmS, ep, cm, M, N, K, stream);
}
