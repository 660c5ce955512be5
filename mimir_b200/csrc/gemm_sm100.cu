// bf16 x bf16 -> fp32 GEMM on the 5th-generation tensor cores (tcgen05 + TMEM),
// operands staged by TMA, persistent over 148 SMs, warp-specialised:
//
//   warp 0      TMA producer    (one lane issues cp.async.bulk.tensor loads)
//   warp 1      MMA issuer      (one lane issues tcgen05.mma; owns the TMEM allocation)
//   warps 2..5  epilogue        (tcgen05.ld -> registers -> fused epilogue -> global)
//
// The accumulator is double-buffered in TMEM (2 x BN columns) so that the
// epilogue of tile i overlaps the main loop of tile i+1.  Operands may be
// K-major (rows of K contiguous: activations [M,K], weights [N,K]) or MN-major
// (the transposed storage), which covers forward (NT), input-gradient (NN) and
// weight-gradient (TN) products without a transpose pass.
//
// Replaces the reference's generated SIMT matmul / cuBLAS SGEMM + separate
// epilogue kernel (backend/internal/gen/gen.go:973-1037, gemm.go:55-128,
// internal/sched/fuse.go:312-325: bias / activation / residual epilogues, and
// :293-302: transposed and batch-summed products).
#include "gemm_common.cuh"

namespace mimir {

template <int BN, bool A_MN, bool B_MN, int STAGES>
__global__ void __launch_bounds__(kGemmThreads, 1)
gemm_bf16_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                 GemmEpi ep, int M, int N, int K, int splits, unsigned* err) {
  constexpr int A_BYTES = kBM * kBK * 2;
  constexpr int B_BYTES = BN * kBK * 2;
  constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
  constexpr uint32_t TMEM_COLS = 2 * BN;
  constexpr uint32_t IDESC = make_idesc_bf16(kBM, BN, A_MN, B_MN);

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  uint64_t* full = reinterpret_cast<uint64_t*>(smem + STAGES * STAGE_BYTES);
  uint64_t* empty = full + STAGES;
  uint64_t* tfull = empty + STAGES;
  uint64_t* tempty = tfull + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tempty + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int m_tiles = (M + kBM - 1) / kBM, n_tiles = (N + BN - 1) / BN;
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
      mbar_init(&tempty[a], 4);
    }
    *abort_flag = 0;
    fence_mbar_init();
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    if (lane == 0) {
      tma_prefetch_desc(&tmA);
      tma_prefetch_desc(&tmB);
      uint32_t it = 0;
      bool ok = true;
      for (int u = blockIdx.x; u < units && ok; u += gridDim.x) {
        const int split = u % splits, tile = u / splits;
        const int n_idx = tile % n_tiles, m_idx = tile / n_tiles;
        const int kb0 = split * kb_per, kb1 = min(kb_total, kb0 + kb_per);
        for (int kb = kb0; kb < kb1; ++kb, ++it) {
          const int s = it % STAGES;
          const uint32_t ph = (it / STAGES) & 1;
          if (!mbar_wait(&empty[s], ph ^ 1, abort_flag, err)) { ok = false; break; }
          uint8_t* sA = smem + s * STAGE_BYTES;
          uint8_t* sB = sA + A_BYTES;
          mbar_arrive_expect_tx(&full[s], STAGE_BYTES);
          if (A_MN) {
#pragma unroll
            for (int c = 0; c < kBM / 64; ++c)
              tma_load_2d(sA + c * (kBK * 128), &tmA, &full[s], m_idx * kBM + c * 64, kb * kBK);
          } else {
            tma_load_2d(sA, &tmA, &full[s], kb * kBK, m_idx * kBM);
          }
          if (B_MN) {
#pragma unroll
            for (int c = 0; c < BN / 64; ++c)
              tma_load_2d(sB + c * (kBK * 128), &tmB, &full[s], n_idx * BN + c * 64, kb * kBK);
          } else {
            tma_load_2d(sB, &tmB, &full[s], kb * kBK, n_idx * BN);
          }
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      uint32_t it = 0, ti = 0;
      bool ok = true;
      for (int u = blockIdx.x; u < units && ok; u += gridDim.x, ++ti) {
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
            // one UMMA consumes K=16: 32 bytes along a K-major row, or 16 rows
            // (2048 bytes) of an MN-major tile
            const uint64_t ad = adesc + (A_MN ? k * 128 : k * 2);
            const uint64_t bd = bdesc + (B_MN ? k * 128 : k * 2);
            umma_ss(d_tmem, ad, bd, IDESC, (kb > kb0 || k > 0) ? 1u : 0u);
          }
          umma_commit(&empty[s]);  // frees the stage once these MMAs have read it
        }
        if (ok) umma_commit(&tfull[acc]);
      }
    }
  } else {
    const int q = warp & 3;  // TMEM lane quadrant this warp may read
    uint32_t ti = 0;
    for (int u = blockIdx.x; u < units; u += gridDim.x, ++ti) {
      const int split = u % splits, tile = u / splits;
      const int n_idx = tile % n_tiles, m_idx = tile / n_tiles;
      const uint32_t acc = ti & 1, acc_ph = (ti >> 1) & 1;
      if (!mbar_wait(&tfull[acc], acc_ph, abort_flag, err)) break;
      tc_fence_after();
      const int row = m_idx * kBM + q * 32 + lane;
      const uint32_t taddr = tmem_base + acc * BN + (static_cast<uint32_t>(q * 32) << 16);
      drain_accumulator<BN>(ep, taddr, row, n_idx * BN, M, N, split);
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&tempty[acc]);
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    __syncwarp();
    tc_fence_after();
    tmem_dealloc(tmem_base, TMEM_COLS);
  }
}

// Sums the split-K partials and applies the epilogue.  One thread per 8 columns.
__global__ void gemm_splitk_reduce_kernel(GemmEpi ep, int M, int N, int splits) {
  const size_t idx = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  const int n8 = N / 8;
  if (idx >= static_cast<size_t>(M) * n8) return;
  const int row = static_cast<int>(idx / n8), col = static_cast<int>(idx % n8) * 8;
  float v[8] = {0, 0, 0, 0, 0, 0, 0, 0};
  for (int s = 0; s < splits; ++s) {
    const float* p = ep.partial + (static_cast<size_t>(s) * M + row) * N + col;
    float4 a = *reinterpret_cast<const float4*>(p), b = *reinterpret_cast<const float4*>(p + 4);
    v[0] += a.x; v[1] += a.y; v[2] += a.z; v[3] += a.w;
    v[4] += b.x; v[5] += b.y; v[6] += b.z; v[7] += b.w;
  }
  epilogue_store8(ep, v, row, col);
}

template <int BN, bool A_MN, bool B_MN, int STAGES>
static int launch_gemm(const CUtensorMap& tmA, const CUtensorMap& tmB, const GemmEpi& ep, int M,
                       int N, int K, int splits, cudaStream_t stream) {
  constexpr int SMEM = STAGES * (kBM * kBK * 2 + BN * kBK * 2) + 1024 + 256;
  auto kern = gemm_bf16_kernel<BN, A_MN, B_MN, STAGES>;
  static bool configured = false;
  if (!configured) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM) != cudaSuccess)
      return refuse("cannot reserve %d bytes of shared memory", SMEM);
    configured = true;
  }
  const int units = ceil_div(M, kBM) * ceil_div(N, BN) * splits;
  const int grid = units < sm_count() ? units : sm_count();
  kern<<<grid, kGemmThreads, SMEM, stream>>>(tmA, tmB, ep, M, N, K, splits, error_word_dev());
  count_launch();
  return cudaGetLastError() == cudaSuccess ? 0 : refuse("gemm launch failed");
}

int launch_gemm_pair(const void* A, const void* B, int M, int N, int K, int lda, int ldb, int a_mn, int b_mn,
                     const GemmEpi& ep, int bn, int splits, cudaStream_t stream);

}  // namespace mimir

using namespace mimir;

// Workspace bytes a call may need for split-K (upper bound over the heuristics).
MIMIR_API long long mimir_gemm_workspace_bytes(int M, int N) {
  return static_cast<long long>(16) * M * N * 4;
}

// C[M,N] = epilogue(alpha * A[M,K] * B[N,K]^T).
//   a_mn == 0: A stored row-major [M,K], lda elements per row.  a_mn == 1: stored [K,M].
//   b_mn == 0: B stored row-major [N,K], ldb elements per row.  b_mn == 1: stored [K,N].
// K-major operands need K % 8 == 0 (row pitch multiple of 16 bytes), MN-major
// ones the same of their row pitch; N % 8 == 0 and ldc % 8 == 0 for vector stores.
// bn_hint: 0 = pick, or 64/128/256.  splits_hint: 0 = pick, else split-K factor
// (needs workspace).  Returns 0, or -1 with mimir_last_error() set.
MIMIR_API int mimir_gemm_bf16(const void* A, const void* B, void* C, int M, int N, int K, int lda,
                              int ldb, int ldc, int a_mn, int b_mn, const void* bias,
                              const void* aux, int ldaux, void* aux_out, int flags, float alpha,
                              void* workspace, long long workspace_bytes, int splits_hint,
                              int bn_hint, cudaStream_t stream) {
  if (M <= 0 || N <= 0 || K <= 0) return refuse("gemm: empty problem %dx%dx%d", M, N, K);
  if (N % 8 || ldc % 8 || lda % 8 || ldb % 8) return refuse("gemm: N, lda, ldb, ldc must be multiples of 8");
  if ((flags & (kResidual | kMulDGelu | kWritePre)) && (ldaux % 8))
    return refuse("gemm: ldaux must be a multiple of 8");
  if ((reinterpret_cast<uintptr_t>(C) & 15) || (bias && (reinterpret_cast<uintptr_t>(bias) & 15)) ||
      (aux && (reinterpret_cast<uintptr_t>(aux) & 15)))
    return refuse("gemm: C, bias and aux must be 16-byte aligned");
  if ((flags & (kResidual | kMulDGelu)) && !aux) return refuse("gemm: aux operand missing");
  if ((flags & kWritePre) && !aux_out) return refuse("gemm: aux_out missing");

  const int nsm = sm_count();
  // bn_hint + 1000 forces the CTA-pair kernel, + 2000 forces the single-CTA kernel
  int pair_mode = bn_hint >= 2000 ? 2 : bn_hint >= 1000 ? 1 : 0;
  bn_hint %= 1000;
  int bn = bn_hint;
  const int kb_total = ceil_div(K, kBK);
  int splits = splits_hint;
  // Plan for the CTA-pair kernel.
  bool plan_pair = pair_mode != 2 && M >= 2 * kBM && N >= 128;
  if (plan_pair && (bn != 128 && bn != 256 || splits <= 0)) {
    // Measured on B200 (sweep over tile width x split-K for the GPT-2 shapes): the
    // 256-wide tile wins whenever N allows it; split-K only pays when the tiles
    // would leave more than half of the CTA pairs idle.
    const int npairs = nsm / 2;
    if (bn != 128 && bn != 256) bn = N >= 256 ? 256 : 128;
    if (splits <= 0) {
      const long long tiles2 = static_cast<long long>(ceil_div(M, 2 * kBM)) * ceil_div(N, bn);
      splits = 1;
      if (workspace && tiles2 * 2 <= npairs && kb_total >= 32) {
        splits = static_cast<int>(npairs / tiles2);
        if (splits > 8) splits = 8;
        if (splits > kb_total / 16) splits = kb_total / 16;
        while (splits > 1 && workspace_bytes < static_cast<long long>(splits) * M * N * 4) --splits;
        if (splits < 1) splits = 1;
      }
    }
    // tiny problems run better on the single-CTA kernel (no cluster launch, finer tiles)
    if (pair_mode == 0 && static_cast<long long>(ceil_div(M, 2 * kBM)) * ceil_div(N, bn) * splits < nsm / 8)
      plan_pair = false;
  }
  if (!plan_pair || pair_mode == 2) {
    plan_pair = pair_mode == 1;
    if (bn != 64 && bn != 128 && bn != 256) {
      // Prefer the wide tile unless its wave quantisation is clearly worse.
      auto eff = [&](int b) {
        long long t = static_cast<long long>(ceil_div(M, kBM)) * ceil_div(N, b);
        long long w = (t + nsm - 1) / nsm;
        return static_cast<double>(t) / static_cast<double>(w * nsm);
      };
      bn = (N >= 256 && eff(256) >= eff(128) - 0.08) ? 256 : 128;
      if (N <= 64) bn = 64;
    }
    const int tiles = ceil_div(M, kBM) * ceil_div(N, bn);
    if (splits <= 0) {
      splits = 1;
      if (workspace && tiles * 2 <= nsm && kb_total >= 8) {
        splits = nsm / tiles;
        if (splits > 16) splits = 16;
        if (splits > kb_total / 4) splits = kb_total / 4;
        if (splits < 1) splits = 1;
      }
    }
  }
  if (splits > kb_total) splits = kb_total;
  // every split must own at least one k-block
  while (splits > 1 && ceil_div(kb_total, splits) * (splits - 1) >= kb_total) --splits;
  if (splits > 1 && (!workspace ||
                     workspace_bytes < static_cast<long long>(splits) * M * N * 4))
    splits = 1;

  GemmEpi ep;
  ep.C = C;
  ep.bias = static_cast<const __nv_bfloat16*>(bias);
  ep.aux = static_cast<const __nv_bfloat16*>(aux);
  ep.aux_out = static_cast<__nv_bfloat16*>(aux_out);
  ep.partial = splits > 1 ? static_cast<float*>(workspace) : nullptr;
  ep.ldc = ldc;
  ep.ldaux = ldaux;
  ep.flags = flags;
  ep.alpha = alpha;

  const bool use_pair = plan_pair;
  if (use_pair && bn >= 128) {
    if (launch_gemm_pair(A, B, M, N, K, lda, ldb, a_mn, b_mn, ep, bn, splits, stream)) return -1;
    if (splits > 1) {
      const size_t n = static_cast<size_t>(M) * (N / 8);
      gemm_splitk_reduce_kernel<<<static_cast<unsigned>((n + 255) / 256), 256, 0, stream>>>(ep, M, N, splits);
      count_launch();
    }
    return 0;
  }

  CUtensorMap tmA, tmB;
  {
    uint64_t dims[2], strides[1];
    uint32_t box[2];
    if (a_mn) { dims[0] = M; dims[1] = K; box[0] = 64; box[1] = kBK; }
    else      { dims[0] = K; dims[1] = M; box[0] = kBK; box[1] = kBM; }
    strides[0] = static_cast<uint64_t>(lda) * 2;
    if (encode_tmap(&tmA, A, 2, 2, dims, strides, box, 3)) return -1;
    if (b_mn) { dims[0] = N; dims[1] = K; box[0] = 64; box[1] = kBK; }
    else      { dims[0] = K; dims[1] = N; box[0] = kBK; box[1] = static_cast<uint32_t>(bn); }
    strides[0] = static_cast<uint64_t>(ldb) * 2;
    if (encode_tmap(&tmB, B, 2, 2, dims, strides, box, 3)) return -1;
  }
  int rc;
#define MIMIR_GEMM_CASE(BN_, ST_)                                                             \
  if (!a_mn && !b_mn) rc = launch_gemm<BN_, false, false, ST_>(tmA, tmB, ep, M, N, K, splits, stream); \
  else if (!a_mn && b_mn) rc = launch_gemm<BN_, false, true, ST_>(tmA, tmB, ep, M, N, K, splits, stream); \
  else if (a_mn && b_mn) rc = launch_gemm<BN_, true, true, ST_>(tmA, tmB, ep, M, N, K, splits, stream); \
  else rc = launch_gemm<BN_, true, false, ST_>(tmA, tmB, ep, M, N, K, splits, stream);
  if (bn == 256) { MIMIR_GEMM_CASE(256, 4) }
  else if (bn == 128) { MIMIR_GEMM_CASE(128, 6) }
  else { MIMIR_GEMM_CASE(64, 8) }
#undef MIMIR_GEMM_CASE
  if (rc) return rc;
  if (splits > 1) {
    GemmEpi rep = ep;
    const size_t n = static_cast<size_t>(M) * (N / 8);
    gemm_splitk_reduce_kernel<<<static_cast<unsigned>((n + 255) / 256), 256, 0, stream>>>(rep, M, N,
                                                                                          splits);
    count_launch();
  }
  return 0;
}
