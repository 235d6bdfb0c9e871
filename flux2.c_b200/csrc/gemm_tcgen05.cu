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

__device__ __forceinline__ float silu_f(float x) { return x / (1.0f + __expf(-x)); }

template <int BN>
__device__ __forceinline__ void epilogue_tile(const GemmProblem &pb, int m0, int n0, uint32_t taddr, int lane_row) {
  const bool second = n0 >= pb.n_split;
  const EpiSeg &sg = second ? pb.seg[1] : pb.seg[0];
  const int nrel = n0 - (second ? pb.n_split : 0);  // segment-relative first column of this tile
  const int row = m0 + lane_row;
  const bool row_ok = row < pb.M;
  uint32_t r[32];

  switch (sg.mode) {
    case EPI_STORE_BF16: {
      __nv_bfloat16 *dst = reinterpret_cast<__nv_bfloat16 *>(sg.out) + static_cast<size_t>(row) * sg.ld + sg.col0 + nrel;
#pragma unroll 1
      for (int c = 0; c < BN / 32; ++c) {
        tc_ld_32x32(taddr + c * 32, r);
        tc_wait_ld();
        if (row_ok) {
          uint4 *d4 = reinterpret_cast<uint4 *>(dst + c * 32);
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            uint4 v;
            v.x = pack_bf16x2(__uint_as_float(r[8 * j + 0]), __uint_as_float(r[8 * j + 1]));
            v.y = pack_bf16x2(__uint_as_float(r[8 * j + 2]), __uint_as_float(r[8 * j + 3]));
            v.z = pack_bf16x2(__uint_as_float(r[8 * j + 4]), __uint_as_float(r[8 * j + 5]));
            v.w = pack_bf16x2(__uint_as_float(r[8 * j + 6]), __uint_as_float(r[8 * j + 7]));
            d4[j] = v;
          }
        }
      }
    } break;
    case EPI_STORE_F32: {
      float *dst = reinterpret_cast<float *>(sg.out) + static_cast<size_t>(row) * sg.ld + sg.col0 + nrel;
#pragma unroll 1
      for (int c = 0; c < BN / 32; ++c) {
        tc_ld_32x32(taddr + c * 32, r);
        tc_wait_ld();
        if (row_ok) {
          uint4 *d4 = reinterpret_cast<uint4 *>(dst + c * 32);
#pragma unroll
          for (int j = 0; j < 8; ++j) d4[j] = make_uint4(r[4 * j], r[4 * j + 1], r[4 * j + 2], r[4 * j + 3]);
        }
      }
    } break;
    case EPI_GATED_RES_F32: {
      float *dst = reinterpret_cast<float *>(sg.out) + static_cast<size_t>(row) * sg.ld + sg.col0 + nrel;
      const float *gate = sg.gate + nrel;
#pragma unroll 1
      for (int c = 0; c < BN / 32; ++c) {
        tc_ld_32x32(taddr + c * 32, r);
        tc_wait_ld();
        if (row_ok) {
          float4 *d4 = reinterpret_cast<float4 *>(dst + c * 32);
          const float4 *g4 = reinterpret_cast<const float4 *>(gate + c * 32);
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            float4 h = d4[j];
            const float4 g = __ldg(g4 + j);
            h.x = fmaf(g.x, __uint_as_float(r[4 * j + 0]), h.x);
            h.y = fmaf(g.y, __uint_as_float(r[4 * j + 1]), h.y);
            h.z = fmaf(g.z, __uint_as_float(r[4 * j + 2]), h.z);
            h.w = fmaf(g.w, __uint_as_float(r[4 * j + 3]), h.w);
            d4[j] = h;
          }
        }
      }
    } break;
    case EPI_SWIGLU_BF16: {
      if constexpr (BN == 256) {
        __nv_bfloat16 *dst =
            reinterpret_cast<__nv_bfloat16 *>(sg.out) + static_cast<size_t>(row) * sg.ld + sg.col0 + nrel / 2;
        uint32_t u[32];
#pragma unroll 1
        for (int c = 0; c < 4; ++c) {
          tc_ld_32x32(taddr + c * 32, r);
          tc_ld_32x32(taddr + 128 + c * 32, u);
          tc_wait_ld();
          if (row_ok) {
            uint4 *d4 = reinterpret_cast<uint4 *>(dst + c * 32);
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              float o[8];
#pragma unroll
              for (int e = 0; e < 8; ++e)
                o[e] = silu_f(__uint_as_float(r[8 * j + e])) * __uint_as_float(u[8 * j + e]);
              uint4 v;
              v.x = pack_bf16x2(o[0], o[1]);
              v.y = pack_bf16x2(o[2], o[3]);
              v.z = pack_bf16x2(o[4], o[5]);
              v.w = pack_bf16x2(o[6], o[7]);
              d4[j] = v;
            }
          }
        }
      }
    } break;
    case EPI_STORE_F32_T: {
      float *dst = reinterpret_cast<float *>(sg.out) + static_cast<size_t>(sg.col0 + nrel) * sg.ld + row;
#pragma unroll 1
      for (int c = 0; c < BN / 32; ++c) {
        tc_ld_32x32(taddr + c * 32, r);
        tc_wait_ld();
        if (row_ok) {
#pragma unroll
          for (int j = 0; j < 32; ++j) dst[static_cast<size_t>(c * 32 + j) * sg.ld] = __uint_as_float(r[j]);
        }
      }
    } break;
    case EPI_QKV_NORM_ROPE: {
      const QkvNormRope &qk = sg.qk;
      const int pos = (qk.pos0 + row) % qk.seq;
      __nv_bfloat16 *dst = reinterpret_cast<__nv_bfloat16 *>(sg.out) + static_cast<size_t>(row) * sg.ld + sg.col0 + nrel;
#pragma unroll 1
      for (int hd = 0; hd < BN / 128; ++hd) {
        const int col = nrel + hd * 128;  // first column of this head inside the [Q|K|V] segment
        const uint32_t th = taddr + hd * 128;
        float rinv = 1.f;
        const bool rotate = col < 2 * qk.hidden;
        const float *w = nullptr;
        if (rotate) {
          float ss = 0.f;
#pragma unroll 1
          for (int c = 0; c < 4; ++c) {
            tc_ld_32x32(th + c * 32, r);
            tc_wait_ld();
#pragma unroll
            for (int j = 0; j < 32; ++j) ss = fmaf(__uint_as_float(r[j]), __uint_as_float(r[j]), ss);
          }
          rinv = rsqrtf(ss * (1.0f / 128.0f) + 1e-6f);
          const bool is_k = col >= qk.hidden;
          w = (pos < qk.n_txt) ? (is_k ? qk.wk_txt : qk.wq_txt) : (is_k ? qk.wk_img : qk.wq_img);
        }
#pragma unroll 1
        for (int c = 0; c < 4; ++c) {
          tc_ld_32x32(th + c * 32, r);
          tc_wait_ld();
          if (row_ok) {
            uint4 *d4 = reinterpret_cast<uint4 *>(dst + hd * 128 + c * 32);
            if (rotate) {
              const float4 *w4 = reinterpret_cast<const float4 *>(w + c * 32);
              const float4 *c4 = reinterpret_cast<const float4 *>(qk.cos_t + static_cast<size_t>(pos) * 128 + c * 32);
              const float4 *s4 = reinterpret_cast<const float4 *>(qk.sin_t + static_cast<size_t>(pos) * 128 + c * 32);
#pragma unroll
              for (int j = 0; j < 4; ++j) {
                uint32_t o[4];
#pragma unroll
                for (int e = 0; e < 2; ++e) {
                  const float4 ww = __ldg(w4 + 2 * j + e);
                  const float4 cc = __ldg(c4 + 2 * j + e);
                  const float4 sn = __ldg(s4 + 2 * j + e);
                  const float x0 = __uint_as_float(r[8 * j + 4 * e + 0]) * rinv * ww.x;
                  const float x1 = __uint_as_float(r[8 * j + 4 * e + 1]) * rinv * ww.y;
                  const float x2 = __uint_as_float(r[8 * j + 4 * e + 2]) * rinv * ww.z;
                  const float x3 = __uint_as_float(r[8 * j + 4 * e + 3]) * rinv * ww.w;
                  o[2 * e + 0] = pack_bf16x2(x0 * cc.x - x1 * sn.x, x1 * cc.x + x0 * sn.x);
                  o[2 * e + 1] = pack_bf16x2(x2 * cc.z - x3 * sn.z, x3 * cc.z + x2 * sn.z);
                }
                d4[j] = make_uint4(o[0], o[1], o[2], o[3]);
              }
            } else {
#pragma unroll
              for (int j = 0; j < 4; ++j) {
                uint4 v;
                v.x = pack_bf16x2(__uint_as_float(r[8 * j + 0]), __uint_as_float(r[8 * j + 1]));
                v.y = pack_bf16x2(__uint_as_float(r[8 * j + 2]), __uint_as_float(r[8 * j + 3]));
                v.z = pack_bf16x2(__uint_as_float(r[8 * j + 4]), __uint_as_float(r[8 * j + 5]));
                v.w = pack_bf16x2(__uint_as_float(r[8 * j + 6]), __uint_as_float(r[8 * j + 7]));
                d4[j] = v;
              }
            }
          }
        }
      }
    } break;
    default:
      break;
  }
}

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
    if (lane == 0) {
      constexpr uint32_t idesc = make_idesc_bf16(BM, BN, 0, 0);
      uint32_t kiter = 0, it = 0;
      bool ok = true;
      for (int tile = blockIdx.x; ok && tile < P.total_tiles; tile += gridDim.x, ++it) {
        int prob, m0, n0;
        decode(tile, prob, m0, n0);
        const int KB = P.p[prob].K / BK;
        const int acc = it & 1;
        if (!mbar_wait(&tempty[acc], ((it >> 1) & 1) ^ 1, abort_flag)) {
          fail(KERR_WAIT_TMEM_EMPTY);
          break;
        }
        tc_fence_after_sync();
        const uint32_t d = tmem_base + acc * BN;
        for (int kb = 0; kb < KB; ++kb, ++kiter) {
          const int s = kiter % STAGES;
          const uint32_t ph = (kiter / STAGES) & 1;
          if (!mbar_wait(&full[s], ph, abort_flag)) {
            fail(KERR_WAIT_FULL);
            ok = false;
            break;
          }
          tc_fence_after_sync();
          const uint32_t sa = smem_u32(smem + s * Cfg::STAGE_BYTES);
          const uint64_t ad = make_smem_desc_sw128(sa, 16, 1024);
          const uint64_t bd = make_smem_desc_sw128(sa + Cfg::A_BYTES, 16, 1024);
#pragma unroll
          for (int k = 0; k < BK / 16; ++k)  // +32 bytes per K=16 slice inside the 128-byte swizzle row
            tc_mma_ss(d, ad + 2 * k, bd + 2 * k, idesc, (kb | k) ? 1u : 0u);
          tc_commit(&empty[s]);
        }
        if (ok) tc_commit(&tfull[acc]);
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
      bool ok = mbar_wait(&tfull[acc], (it >> 1) & 1, abort_flag);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) {
        if (lane == 0) fail(KERR_WAIT_TMEM_FULL);
        break;
      }
      tc_fence_after_sync();
      const uint32_t taddr = tmem_base + acc * BN + (static_cast<uint32_t>(q * 32) << 16);
      epilogue_tile<BN>(P.p[prob], m0, n0, taddr, q * 32 + lane);
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

int gemm_make_problem(GemmProblem *p, const void *X, long long ldx, const void *W, int M, int N, int K, int bn) {
  if (M <= 0 || N <= 0 || K <= 0 || (K % BK) || (N % bn) || (bn != 128 && bn != 256) || ldx < K) return -5;
  int rc = make_tmap_2d_bf16(&p->tmA, X, M, K, ldx, BM, BK);
  if (rc) return rc;
  rc = make_tmap_2d_bf16(&p->tmB, W, N, K, K, bn, BK);
  if (rc) return rc;
  p->M = M;
  p->N = N;
  p->K = K;
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
  if (bn == 256)
    gemm_bf16_tn_kernel<256><<<grid, GEMM_THREADS, GemmCfg<256>::SMEM_BYTES, stream>>>(*P);
  else
    gemm_bf16_tn_kernel<128><<<grid, GEMM_THREADS, GemmCfg<128>::SMEM_BYTES, stream>>>(*P);
  return cudaGetLastError() == cudaSuccess ? 0 : -8;
}

}  // namespace fx
