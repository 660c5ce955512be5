// bf16 GEMM with CTA pairs: tcgen05.mma.cta_group::2 computes a 256 x BN tile on
// two SMs.  Each CTA of the pair stages its own 128 rows of A and its own half
// (BN/2 columns) of B with plain TMA loads, so every byte of B is fetched once
// per pair instead of once per SM; the accumulator (128 lanes x BN columns per
// CTA) stays double buffered in TMEM.  The leader CTA (cluster rank 0) issues
// the MMAs for both; its commits arrive on the barriers of both CTAs.
//
// Protocol (barriers live at the same shared-memory offset in both CTAs):
//   full[s]    used in the leader only.  The leader's producer posts the byte
//              count of BOTH CTAs' loads; each CTA's loads complete on it
//              (the peer addresses it through its cluster-mapped address).
//   empty[s]   in each CTA; the leader's tcgen05.commit arrives on both.
//   tfull[a]   in each CTA; the leader's commit arrives on both, each CTA's
//              epilogue warps then drain their own 128 accumulator rows.
//   tempty[a]  in the leader; the 4 epilogue warps of each CTA arrive on it.
// All waits are bounded; both CTAs meet at a cluster barrier before TMEM is freed.
//
// Same C ABI and epilogues as the 1-CTA kernel (gemm_sm100.cu), which remains
// the path for small problems.
#include "gemm_pair.cuh"

namespace mimir {

// warp 0 TMA, warp 1 MMA, warps 2..9 epilogue: two warps per TMEM lane quadrant, each
// draining half of the tile's columns, so that every scheduler holds two epilogue warps.
constexpr int kGemm2Threads = 320;
constexpr int kEpiWarps = 8;

template <int BN, bool A_MN, bool B_MN, int STAGES>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kGemm2Threads, 1)
gemm2_bf16_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                  const __grid_constant__ CUtensorMap tmC, const __grid_constant__ CUtensorMap tmPre, GemmEpi ep,
                  int M, int N, int K, int splits, int tma_out, unsigned* err) {
  constexpr int BNH = BN / 2;  // columns of B staged by each CTA
  constexpr int A_BYTES = kBM * kBK * 2;
  constexpr int B_BYTES = BNH * kBK * 2;
  constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
  constexpr uint32_t TMEM_COLS = 2 * BN;
  constexpr uint32_t IDESC = make_idesc_bf16(2 * kBM, BN, A_MN, B_MN);

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  uint8_t* out_ring = smem + STAGES * STAGE_BYTES;  // 8 warps x 2 x 4 KiB, for TMA stores
  uint64_t* full = reinterpret_cast<uint64_t*>(out_ring + kEpiWarps * 2 * 4096);
  uint64_t* empty = full + STAGES;
  uint64_t* tfull = empty + STAGES;
  uint64_t* tempty = tfull + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tempty + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t cta = cluster_ctarank();  // 0 = leader
  const int pair = static_cast<int>(cluster_id_x()), npairs = static_cast<int>(nclusters_x());
  const int m_tiles = (M + 2 * kBM - 1) / (2 * kBM), n_tiles = (N + BN - 1) / BN;
  const int kb_total = (K + kBK - 1) / kBK;
  const int kb_per = (kb_total + splits - 1) / splits;
  const int units = m_tiles * n_tiles * splits;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(&tfull[a], 1);
      mbar_init(&tempty[a], 2 * kEpiWarps);  // the epilogue warps of both CTAs
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
  cluster_sync_all();  // both CTAs' barriers and TMEM exist before anyone signals across
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    if (lane == 0) {
      tma_prefetch_desc(&tmA);
      tma_prefetch_desc(&tmB);
      uint32_t it = 0;
      bool ok = true;
      for (int u = pair; u < units && ok; u += npairs) {
        const int split = u % splits, tile = u / splits;
        const int n_idx = tile % n_tiles, m_idx = tile / n_tiles;
        const int kb0 = split * kb_per, kb1 = min(kb_total, kb0 + kb_per);
        const int m0 = m_idx * 2 * kBM + static_cast<int>(cta) * kBM;  // this CTA's A rows
        const int n0 = n_idx * BN + static_cast<int>(cta) * BNH;       // this CTA's B columns
        for (int kb = kb0; kb < kb1; ++kb, ++it) {
          const int s = it % STAGES;
          const uint32_t ph = (it / STAGES) & 1;
          if (!mbar_wait(&empty[s], ph ^ 1, abort_flag, err)) { ok = false; break; }
          uint8_t* sA = smem + s * STAGE_BYTES;
          uint8_t* sB = sA + A_BYTES;
          const uint32_t bar = map_to_cta(smem_u32(&full[s]), 0);  // the leader's barrier
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
        const int split = u % splits;
        const int kb0 = split * kb_per, kb1 = min(kb_total, kb0 + kb_per);
        const uint32_t acc = ti & 1, acc_ph = (ti >> 1) & 1;
        if (!mbar_wait(&tempty[acc], acc_ph ^ 1, abort_flag, err)) break;
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * BN;
        for (int kb = kb0; kb < kb1; ++kb, ++it) {
          const int s = it % STAGES;
          const uint32_t ph = (it / STAGES) & 1;
          if (!mbar_wait(&full[s], ph, abort_flag, err)) { ok = false; break; }
          tc_fence_after();
          const uint32_t sA = smem_u32(smem + s * STAGE_BYTES);
          const uint32_t sB = sA + A_BYTES;
          const uint64_t adesc = A_MN ? make_smem_desc_sw128(sA, kBK * 128, 1024)
                                      : make_smem_desc_sw128(sA, 16, 1024);
          const uint64_t bdesc = B_MN ? make_smem_desc_sw128(sB, kBK * 128, 1024)
                                      : make_smem_desc_sw128(sB, 16, 1024);
#pragma unroll
          for (int k = 0; k < kBK / 16; ++k) {
            const uint64_t ad = adesc + (A_MN ? k * 128 : k * 2);
            const uint64_t bd = bdesc + (B_MN ? k * 128 : k * 2);
            umma_ss_pair(d_tmem, ad, bd, IDESC, (kb > kb0 || k > 0) ? 1u : 0u);
          }
          umma_commit_pair(&empty[s], 3);  // frees the stage in both CTAs
        }
        if (ok) umma_commit_pair(&tfull[acc], 3);
      }
    }
  } else {
    const int q = warp & 3;           // TMEM lane quadrant
    const int half = (warp - 2) >> 2;  // which half of the tile's columns
    const uint32_t tempty_leader0 = map_to_cta(smem_u32(&tempty[0]), 0);
    const uint32_t tempty_leader1 = map_to_cta(smem_u32(&tempty[1]), 0);
    uint32_t ti = 0, ring = 0;
    uint8_t* wbuf = out_ring + (warp - 2) * 2 * 4096;
    for (int u = pair; u < units; u += npairs, ++ti) {
      const int split = u % splits, tile = u / splits;
      const int n_idx = tile % n_tiles, m_idx = tile / n_tiles;
      const uint32_t acc = ti & 1, acc_ph = (ti >> 1) & 1;
      if (!mbar_wait(&tfull[acc], acc_ph, abort_flag, err)) break;
      tc_fence_after();
      const int row0 = m_idx * 2 * kBM + static_cast<int>(cta) * kBM + q * 32;
      const uint32_t taddr = tmem_base + acc * BN + half * (BN / 2) + (static_cast<uint32_t>(q * 32) << 16);
      const int col_base = n_idx * BN + half * (BN / 2);
      if (tma_out == 1)
        drain_accumulator_tma<BN / 128>(ep, &tmC, &tmPre, taddr, row0, col_base, M, N, wbuf, ring, lane);
      else if (tma_out == 2)
        drain_partial_tma<BN / 64>(&tmC, taddr, row0, col_base, M, N, split, wbuf, ring, lane);
      else
        drain_accumulator<BN / 2>(ep, taddr, row0 + lane, col_base, M, N, split);
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster(acc ? tempty_leader1 : tempty_leader0);
    }
    if (lane == 0) bulk_wait_group_read<0>();  // the ring must outlive its last store's reads
  }

  tc_fence_before();
  __syncthreads();
  cluster_sync_all();  // nobody frees TMEM or exits while the peer may still signal it
  if (warp == 1) {
    __syncwarp();
    tc_fence_after();
    tmem_dealloc_pair(tmem_base, TMEM_COLS);
  }
}


template <int BN, bool A_MN, bool B_MN, int STAGES>
static int launch_gemm2(const CUtensorMap& tmA, const CUtensorMap& tmB, const CUtensorMap& tmC,
                        const CUtensorMap& tmPre, int tma_out, const GemmEpi& ep, int M, int N, int K,
                        int splits, cudaStream_t stream) {
  constexpr int SMEM = STAGES * (kBM * kBK * 2 + (BN / 2) * kBK * 2) + kEpiWarps * 2 * 4096 + 1024 + 256;
  auto kern = gemm2_bf16_kernel<BN, A_MN, B_MN, STAGES>;
  static int max_pairs = 0;
  if (max_pairs == 0) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM) != cudaSuccess)
      return refuse("cannot reserve %d bytes of shared memory", SMEM);
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(2 * (sm_count() / 2));
    cfg.blockDim = dim3(kGemm2Threads);
    cfg.dynamicSmemBytes = SMEM;
    int n = 0;
    if (cudaOccupancyMaxActiveClusters(&n, kern, &cfg) != cudaSuccess || n <= 0) {
      cudaGetLastError();
      n = sm_count() / 2;
    }
    max_pairs = n < sm_count() / 2 ? n : sm_count() / 2;
  }
  const int units = ceil_div(M, 2 * kBM) * ceil_div(N, BN) * splits;
  const int pairs = units < max_pairs ? units : max_pairs;
  kern<<<2 * pairs, kGemm2Threads, SMEM, stream>>>(tmA, tmB, tmC, tmPre, ep, M, N, K, splits, tma_out, error_word_dev());
  count_launch();
  return cudaGetLastError() == cudaSuccess ? 0 : refuse("gemm2 launch failed");
}

// Launches the CTA-pair kernel; called by mimir_gemm_bf16 when the problem is large enough.
int launch_gemm_pair(const void* A, const void* B, int M, int N, int K, int lda, int ldb, int a_mn, int b_mn,
                     const GemmEpi& ep, int bn, int splits, cudaStream_t stream) {
  CUtensorMap tmA, tmB;
  uint64_t dims[2], strides[1];
  uint32_t box[2];
  if (a_mn) { dims[0] = M; dims[1] = K; box[0] = 64; box[1] = kBK; }
  else      { dims[0] = K; dims[1] = M; box[0] = kBK; box[1] = kBM; }
  strides[0] = static_cast<uint64_t>(lda) * 2;
  if (encode_tmap(&tmA, A, 2, 2, dims, strides, box, 3)) return -1;
  if (b_mn) { dims[0] = N; dims[1] = K; box[0] = 64; box[1] = kBK; }
  else      { dims[0] = K; dims[1] = N; box[0] = kBK; box[1] = static_cast<uint32_t>(bn / 2); }
  strides[0] = static_cast<uint64_t>(ldb) * 2;
  if (encode_tmap(&tmB, B, 2, 2, dims, strides, box, 3)) return -1;
  // bf16 outputs without accumulation leave through TMA stores of 32 x 64 sub-tiles
  CUtensorMap tmC = tmA, tmPre = tmA;
  int tma_out = !(ep.flags & (kOutF32 | kAccumulate)) && !ep.partial;
  if (ep.partial) {
    // fp32 partial sums [splits][M][N]: 32-column (128-byte) boxes, clipped per split
    uint64_t d3[3] = {static_cast<uint64_t>(N), static_cast<uint64_t>(M), static_cast<uint64_t>(splits)};
    uint64_t s3[2] = {static_cast<uint64_t>(N) * 4, static_cast<uint64_t>(M) * N * 4};
    uint32_t b3[3] = {32, 32, 1};
    if (N % 4 == 0 && encode_tmap(&tmC, ep.partial, 4, 3, d3, s3, b3, 3) == 0) tma_out = 2;
  } else if (tma_out) {
    dims[0] = N; dims[1] = M; box[0] = 64; box[1] = 32;
    strides[0] = static_cast<uint64_t>(ep.ldc) * 2;
    if (encode_tmap(&tmC, ep.C, 2, 2, dims, strides, box, 3)) return -1;
    if ((ep.flags & kGelu) && (ep.flags & kWritePre)) {
      strides[0] = static_cast<uint64_t>(ep.ldaux) * 2;
      if (encode_tmap(&tmPre, ep.aux_out, 2, 2, dims, strides, box, 3)) return -1;
    }
  }
#define MIMIR_GEMM2_CASE(BN_, ST_)                                                                       \
  if (!a_mn && !b_mn) return launch_gemm2<BN_, false, false, ST_>(tmA, tmB, tmC, tmPre, tma_out, ep, M, N, K, splits, stream); \
  if (!a_mn && b_mn) return launch_gemm2<BN_, false, true, ST_>(tmA, tmB, tmC, tmPre, tma_out, ep, M, N, K, splits, stream);   \
  if (a_mn && b_mn) return launch_gemm2<BN_, true, true, ST_>(tmA, tmB, tmC, tmPre, tma_out, ep, M, N, K, splits, stream);     \
  return launch_gemm2<BN_, true, false, ST_>(tmA, tmB, tmC, tmPre, tma_out, ep, M, N, K, splits, stream);
  if (bn == 256) { MIMIR_GEMM2_CASE(256, 5) }
  MIMIR_GEMM2_CASE(128, 6)
#undef MIMIR_GEMM2_CASE
}

}  // namespace mimir

