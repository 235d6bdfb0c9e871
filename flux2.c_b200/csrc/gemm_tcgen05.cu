// K1: persistent, warp-specialised bf16 GEMM for sm_100a.
//
//   Y[M,N] = X[M,K] * W[N,K]^T       X, W bf16 with K contiguous; f32 accumulation in TMEM.
//
// One CTA per SM walks a static tile list (128 x BN output tiles, m fastest so that CTAs running
// at the same time share W tiles through L2). Roles inside a CTA of 192 threads:
//   warp 0      TMA producer: cp.async.bulk.tensor loads of the X and W k-slices (64 wide, 128-byte
//               swizzle) into a ring of shared-memory stages, signalled through mbarriers;
//   warp 1      MMA issuer: one thread issues tcgen05.mma (M=128, N=BN, K=16) four times per stage and
//               commits the stage back to the producer; owns the TMEM allocation;
//   warps 2-5   epilogue: tcgen05.ld the finished accumulator (one TMEM lane = one output row per
//               thread) and apply the fused epilogue while the MMA warp already fills the second
//               accumulator (TMEM holds two BN-column accumulators).
//
// The epilogue modes replace, besides flux_linear_nobias (flux_kernels.c:210-320), the reference's
// separate passes gated_add (flux_transformer.c:90-97), silu*up (flux_transformer.c:1737-1763), the
// [Q|K|V|gate|up] split of the single-stream block (flux_transformer.c:3051-3058) and the final
// NLC -> NCHW transpose (flux_transformer.c:3547-3552).
#include "gemm.cuh"
#include "gemm_epilogue.cuh"
#include "launch.cuh"
#include "ptx.cuh"

#include <cudaTypedefs.h>
#include <stdio.h>

namespace fx {

static constexpr int BM = 128;
static constexpr int BK = 64;
static constexpr int GEMM_THREADS = 192;

template <int BN>
struct GemmCfg {
  static constexpr int STAGES = (BN == 256) ? 4 : 6;
  static constexpr int A_BYTES = BM * BK * 2;
  static constexpr int B_BYTES = BN * BK * 2;
  static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
  static constexpr int BAR_BYTES = 256;
  static constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + BAR_BYTES + 1024;  // +1024: manual alignment slack
  static constexpr int TMEM_COLS = 2 * BN;
};

template <int BN>
__global__ void __launch_bounds__(GEMM_THREADS, 1) gemm_bf16_tn_kernel(const __grid_constant__ GemmParams P) {
  using Cfg = GemmCfg<BN>;
  constexpr int STAGES = Cfg::STAGES;
  extern __shared__ uint8_t smem_raw[];
  uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t *bars = reinterpret_cast<uint64_t *>(smem + STAGES * Cfg::STAGE_BYTES);
  uint64_t *full = bars;
  uint64_t *empty = bars + STAGES;
  uint64_t *tfull = bars + 2 * STAGES;
  uint64_t *tempty = tfull + 2;
  uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(tempty + 2);
  volatile int *abort_flag = reinterpret_cast<volatile int *>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

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
    mbar_fence_init();
  }
  if (warp == 1) tmem_alloc(tmem_slot, Cfg::TMEM_COLS);
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;
  pdl_launch_dependents();
  pdl_wait();  // everything above touched only shared memory and TMEM

  auto fail = [&](int code) {
    *abort_flag = 1;
    atomicCAS(P.err, 0, code);
  };
  auto decode = [&](int tile, int &prob, int &m0, int &n0) {
    prob = 0;
    while (prob + 1 < P.nprob && tile >= P.tile_end[prob]) ++prob;
    const int local = tile - (prob ? P.tile_end[prob - 1] : 0);
    const int tm = P.p[prob].tiles_m;
    m0 = (local % tm) * BM;
    n0 = (local / tm) * BN;
  };

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer
    if (lane == 0) {
      for (int i = 0; i < P.nprob; ++i) {
        tma_prefetch_desc(&P.p[i].tmA);
        tma_prefetch_desc(&P.p[i].tmB);
      }
      uint32_t kiter = 0;
      bool ok = true;
      for (int tile = blockIdx.x; ok && tile < P.total_tiles; tile += gridDim.x) {
        int prob, m0, n0;
        decode(tile, prob, m0, n0);
        const GemmProblem &pb = P.p[prob];
        const int KB = pb.K / BK;
        for (int kb = 0; kb < KB; ++kb, ++kiter) {
          const int s = kiter % STAGES;
          const uint32_t ph = (kiter / STAGES) & 1;
          if (!mbar_wait(&empty[s], ph ^ 1, abort_flag)) {
            fail(KERR_WAIT_EMPTY);
            ok = false;
            break;
          }
          uint8_t *sa = smem + s * Cfg::STAGE_BYTES;
          uint8_t *sb = sa + Cfg::A_BYTES;
          mbar_arrive_expect_tx(&full[s], Cfg::STAGE_BYTES);
          tma_load_2d(sa, &pb.tmA, &full[s], kb * BK, m0);
          tma_load_2d(sb, &pb.tmB, &full[s], kb * BK, n0);
        }
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    // the whole warp runs the loop, one elected lane issues (see gemm2_tcgen05.cu): descriptors stay warp-uniform
    {
      const bool leader = elect_one();
      const uint32_t smem_base = smem_u32(smem);
      constexpr uint32_t idesc_bf16 = make_idesc_16(BM, BN, FMT_BF16, FMT_BF16, 0, 0);
      constexpr uint32_t idesc_f16 = make_idesc_16(BM, BN, FMT_F16, FMT_F16, 0, 0);
      uint32_t kiter = 0, it = 0;
      bool ok = true;
      for (int tile = blockIdx.x; ok && tile < P.total_tiles; tile += gridDim.x, ++it) {
        int prob, m0, n0;
        decode(tile, prob, m0, n0);
        const int KB = P.p[prob].K / BK;
        const uint32_t idesc = P.p[prob].x_f16 ? idesc_f16 : idesc_bf16;
        const int acc = it & 1;
        if (!mbar_wait_warp(&tempty[acc], ((it >> 1) & 1) ^ 1, abort_flag)) {
          if (lane == 0) fail(KERR_WAIT_TMEM_EMPTY);
          break;
        }
        tc_fence_after_sync();
        const uint32_t d = tmem_base + acc * BN;
        for (int kb = 0; kb < KB; ++kb, ++kiter) {
          const int s = kiter % STAGES;
          const uint32_t ph = (kiter / STAGES) & 1;
          if (!mbar_wait_warp(&full[s], ph, abort_flag)) {
            if (lane == 0) fail(KERR_WAIT_FULL);
            ok = false;
            break;
          }
          tc_fence_after_sync();
          const uint32_t sa = smem_base + s * Cfg::STAGE_BYTES;
          const uint64_t ad = make_smem_desc_sw128(sa, 16, 1024);
          const uint64_t bd = make_smem_desc_sw128(sa + Cfg::A_BYTES, 16, 1024);
          if (leader) {
#pragma unroll
            for (int k = 0; k < BK / 16; ++k)  // +32 bytes per K=16 slice inside the 128-byte swizzle row
              tc_mma_ss(d, ad + 2 * k, bd + 2 * k, idesc, (kb | k) ? 1u : 0u);
            tc_commit(&empty[s]);
          }
        }
        if (ok && leader) tc_commit(&tfull[acc]);
      }
    }
    __syncwarp();
  } else {
    // ------------------------------------------------------------------ epilogue (warps 2..5)
    const int q = warp & 3;  // the TMEM lane quarter this warp is allowed to read
    uint32_t it = 0;
    for (int tile = blockIdx.x; tile < P.total_tiles; tile += gridDim.x, ++it) {
      int prob, m0, n0;
      decode(tile, prob, m0, n0);
      const int acc = it & 1;
      const bool ok = mbar_wait_warp(&tfull[acc], (it >> 1) & 1, abort_flag);
      if (!ok) {
        if (lane == 0) fail(KERR_WAIT_TMEM_FULL);
        break;
      }
      tc_fence_after_sync();
      const uint32_t taddr = tmem_base + acc * BN + (static_cast<uint32_t>(q * 32) << 16);
      epilogue_tile<BN>(P.p[prob], m0, n0, taddr, q * 32 + lane, P.err + 1);
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(&tempty[acc]);
    }
  }

  // ------------------------------------------------------------------ teardown
  if (*abort_flag) {
    // Give loads and MMAs that may still be in flight time to land before shared memory and TMEM
    // are released (bounded: ~1 ms).
    const long long t0 = clock64();
    while (clock64() - t0 < 2000000LL) __nanosleep(1000);
  }
  tc_fence_before_sync();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, Cfg::TMEM_COLS);
  }
}

// ---------------------------------------------------------------------------------------------- host
static PFN_cuTensorMapEncodeTiled_v12000 g_encode = nullptr;

int gemm_init() {
  if (!g_encode) {
    void *fn = nullptr;
    cudaDriverEntryPointQueryResult qres;
    cudaError_t e = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &qres);
    if (e != cudaSuccess || qres != cudaDriverEntryPointSuccess || !fn) return -1;
    g_encode = reinterpret_cast<PFN_cuTensorMapEncodeTiled_v12000>(fn);
  }
  cudaError_t e1 = cudaFuncSetAttribute(gemm_bf16_tn_kernel<256>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                        GemmCfg<256>::SMEM_BYTES);
  cudaError_t e2 = cudaFuncSetAttribute(gemm_bf16_tn_kernel<128>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                        GemmCfg<128>::SMEM_BYTES);
  return (e1 == cudaSuccess && e2 == cudaSuccess) ? 0 : -2;
}

int make_tmap_2d_bf16(CUtensorMap *m, const void *base, uint64_t rows, uint64_t cols, uint64_t ld, uint32_t box_rows,
                      uint32_t box_cols) {
  if (!g_encode && gemm_init() != 0) return -1;
  if ((reinterpret_cast<uintptr_t>(base) & 15) || ((ld * 2) & 15) || ((box_cols * 2) & 15)) return -3;
  cuuint64_t dims[2] = {cols, rows};
  cuuint64_t strides[1] = {ld * 2};
  cuuint32_t box[2] = {box_cols, box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = g_encode(m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void *>(base), dims, strides, box, estr,
                        CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                        CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : -4;
}

int make_tmap_2d_f32(CUtensorMap *m, const void *base, uint64_t rows, uint64_t cols, uint64_t ld, uint32_t box_rows,
                     uint32_t box_cols) {
  if (!g_encode && gemm_init() != 0) return -1;
  if ((reinterpret_cast<uintptr_t>(base) & 15) || ((ld * 4) & 15) || box_cols * 4 != 128) return -3;
  cuuint64_t dims[2] = {cols, rows};
  cuuint64_t strides[1] = {ld * 4};
  cuuint32_t box[2] = {box_cols, box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = g_encode(m, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, const_cast<void *>(base), dims, strides, box, estr,
                        CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                        CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : -4;
}

int gemm_make_problem(GemmProblem *p, const void *X, long long ldx, const void *W, int M, int N, int K, int bn,
                      long long ldw) {
  if (ldw == 0) ldw = K;
  if (M <= 0 || N <= 0 || K <= 0 || (K % BK) || (N % bn) || (bn != 128 && bn != 256) || ldx < K || ldw < K) return -5;
  int rc = make_tmap_2d_bf16(&p->tmA, X, M, K, ldx, BM, BK);
  if (rc) return rc;
  rc = make_tmap_2d_bf16(&p->tmB, W, N, K, ldw, bn, BK);
  if (rc) return rc;
  p->M = M;
  p->N = N;
  p->K = K;
  p->x_f16 = 0;
  p->n_split = N;
  p->tiles_m = (M + BM - 1) / BM;
  p->tiles_n = N / bn;
  return 0;
}

int gemm_launch(GemmParams *P, int bn, int num_sms, cudaStream_t stream) {
  if (P->nprob < 1 || P->nprob > GEMM_MAX_PROBLEMS) return -5;
  int acc = 0;
  for (int i = 0; i < P->nprob; ++i) {
    acc += P->p[i].tiles_m * P->p[i].tiles_n;
    P->tile_end[i] = acc;
  }
  P->total_tiles = acc;
  for (int i = 0; i < P->nprob; ++i) {
    const GemmProblem &pb = P->p[i];
    if (pb.n_split % bn) return -6;
    for (int s = 0; s < 2; ++s)
      if (pb.seg[s].mode == EPI_SWIGLU_BF16 && bn != 256) return -7;
  }
  const int grid = P->total_tiles < num_sms ? P->total_tiles : num_sms;
  cudaError_t e =
      bn == 256 ? launch_kernel(gemm_bf16_tn_kernel<256>, dim3(grid), dim3(GEMM_THREADS), GemmCfg<256>::SMEM_BYTES,
                                stream, 1, *P)
                : launch_kernel(gemm_bf16_tn_kernel<128>, dim3(grid), dim3(GEMM_THREADS), GemmCfg<128>::SMEM_BYTES,
                                stream, 1, *P);
  return e == cudaSuccess ? 0 : -8;
}

}  // namespace fx
