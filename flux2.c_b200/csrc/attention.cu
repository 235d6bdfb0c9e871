// K2: joint text+image attention, flash style, on tcgen05.
//
//   O[q, head] = softmax(Q[q, head] . K[:, head]^T / sqrt(128)) . V[:, head]      no mask, all N keys
//
// replaces the reference's mha_forward / joint_attention (flux_transformer.c:1249-1330, 1335-1460;
// flash variant flux_kernels.c:700-969). Text and image tokens live in ONE [txt ; img ; refs] sequence
// in this engine, so the double-stream blocks' joint attention (both streams' queries against the
// concatenated keys) and the single-stream blocks' attention are the same launch.
//
// One CTA = 128 queries of one head (of one batch element). Q, K, V are read by TMA straight out of
// the fused projection output [B, N, ld] (bf16, 128-byte swizzle, 64-column boxes). Roles:
//   warp 0     TMA producer: Q once, then a two-stage ring of K/V tiles (128 keys each);
//   warp 1     MMA issuer:  S = Q K^T  (M128 N128 K128, both operands K-major) into one of two TMEM
//              score buffers, and  T = P V  (A = P from shared memory, B = V as an MN-major operand)
//              into one of two TMEM output-tile buffers; S(j+1) is issued before P V(j) so that the
//              tensor pipe works while the softmax warps handle tile j;
//   warps 2-9  softmax: two threads per query row (its TMEM lane), each owning 64 of the 128 score and
//              output columns, so that every SM sub-partition runs two softmax warps. Online softmax in
//              base 2 with f32 statistics (each thread scans the whole row for the maximum but
//              exponentiates only its half; the partial row sums are combined once at the end); P is rounded to bf16 and written to one of two shared-memory buffers in the
//              swizzled K-major layout the MMA expects; the running output lives in registers and is
//              rescaled and updated from the TMEM tile of the previous step (O = O*alpha + T).
#include "attention.cuh"
#include "gemm.cuh"
#include "launch.cuh"
#include "ptx.cuh"

#include <cudaTypedefs.h>

namespace fx {

static constexpr int ATT_THREADS = 576;    // warp 0 TMA, warp 1 MMA, warps 2..17 softmax
static constexpr int TILE = 128;           // queries per CTA, keys per step, head dim
static constexpr int CHUNK_BYTES = 16384;  // 128 rows x 64 bf16
static constexpr int OFF_Q = 0;
static constexpr int OFF_KV = 32768;  // stage s: K at OFF_KV + s*65536, V 32768 after it
static constexpr int OFF_P = OFF_KV + 2 * 65536;  // two P buffers of 32 KB
static constexpr int OFF_BAR = OFF_P + 2 * 32768;
static constexpr int ATT_SMEM = OFF_BAR + 2560;  // no alignment slack: the kernel checks the base instead

struct AttnBars {
  uint64_t q_full;
  uint64_t k_full[2], v_full[2], kv_empty[2];
  uint64_t s_full[2], s_empty[2];
  uint64_t p_full[2], p_empty[2];
  uint64_t o_full[2], o_empty[2];
  uint32_t tmem_slot;
  int abort_flag;
  uint64_t mx_full[2][4];  // [tile parity][lane quarter]: the four warps of a quarter published their maxima
  __nv_bfloat16 xchg[2][4][128];  // [tile parity][column quarter][row]: partial row maxima, rounded UP to bf16
                                  // (any common upper bound stabilises the softmax; shared memory is full)
};

__device__ __forceinline__ float ex2f(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

__global__ void __launch_bounds__(ATT_THREADS, 1) attn_fwd_kernel(const __grid_constant__ AttnParams P) {
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  uint8_t *smem = smem_raw;
  if (smem_u32(smem) & 1023u) {  // the 128-byte swizzle needs 1024-byte aligned tiles; never observed, but checked
    if (threadIdx.x == 0) atomicCAS(P.err, 0, KERR_BAD_SHAPE);
    return;
  }
  AttnBars *B = reinterpret_cast<AttnBars *>(smem + OFF_BAR);
  static_assert(sizeof(AttnBars) <= 2560, "barrier block does not fit");
  volatile int *abort_flag = &B->abort_flag;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int q0 = blockIdx.x * TILE;
  const int head = blockIdx.y;
  const int batch = blockIdx.z;
  const int T = (P.seq + TILE - 1) / TILE;  // key tiles

  if (threadIdx.x == 0) {
    mbar_init(&B->q_full, 1);
    for (int i = 0; i < 2; ++i) {
      mbar_init(&B->k_full[i], 1);
      mbar_init(&B->v_full[i], 1);
      mbar_init(&B->kv_empty[i], 1);
      mbar_init(&B->s_full[i], 1);
      mbar_init(&B->s_empty[i], 16);
      mbar_init(&B->p_full[i], 16);
      mbar_init(&B->p_empty[i], 1);
      mbar_init(&B->o_full[i], 1);
      mbar_init(&B->o_empty[i], 16);
      for (int qq = 0; qq < 4; ++qq) mbar_init(&B->mx_full[i][qq], 4);
    }
    B->abort_flag = 0;
    mbar_fence_init();
  }
  if (warp == 1) tmem_alloc(&B->tmem_slot, 512);
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem = B->tmem_slot;
  pdl_launch_dependents();
  pdl_wait();  // everything above touched only shared memory and TMEM

  auto fail = [&]() {
    *abort_flag = 1;
    atomicCAS(P.err, 0, KERR_WAIT_ATTN);
  };

  if (warp == 0) {
    // ---------------------------------------------------------------- TMA producer
    if (lane == 0) {
      tma_prefetch_desc(&P.tm);
      mbar_arrive_expect_tx(&B->q_full, 2 * CHUNK_BYTES);
      tma_load_3d(smem + OFF_Q, &P.tm, &B->q_full, P.q_col + head * 128, q0, batch);
      tma_load_3d(smem + OFF_Q + CHUNK_BYTES, &P.tm, &B->q_full, P.q_col + head * 128 + 64, q0, batch);
      for (int j = 0; j < T; ++j) {
        const int s = j & 1;
        if (!mbar_wait(&B->kv_empty[s], ((j >> 1) & 1) ^ 1, abort_flag)) {
          fail();
          break;
        }
        uint8_t *sk = smem + OFF_KV + s * 65536;
        uint8_t *sv = sk + 32768;
        mbar_arrive_expect_tx(&B->k_full[s], 2 * CHUNK_BYTES);
        tma_load_3d(sk, &P.tm, &B->k_full[s], P.k_col + head * 128, j * TILE, batch);
        tma_load_3d(sk + CHUNK_BYTES, &P.tm, &B->k_full[s], P.k_col + head * 128 + 64, j * TILE, batch);
        mbar_arrive_expect_tx(&B->v_full[s], 2 * CHUNK_BYTES);
        tma_load_3d(sv, &P.tm, &B->v_full[s], P.v_col + head * 128, j * TILE, batch);
        tma_load_3d(sv + CHUNK_BYTES, &P.tm, &B->v_full[s], P.v_col + head * 128 + 64, j * TILE, batch);
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    // ---------------------------------------------------------------- MMA issuer
    if (lane == 0) {
      const uint32_t fmt = P.f16 ? FMT_F16 : FMT_BF16;
      const uint32_t idesc_s = make_idesc_16(128, 128, fmt, fmt, 0, 0);  // Q (K-major) x K (K-major)
      const uint32_t idesc_o = make_idesc_16(128, 128, fmt, fmt, 0, 1);  // P (K-major) x V (MN-major)
      const uint32_t sq = smem_u32(smem + OFF_Q);
      auto issue_s = [&](int j) {
        const uint32_t sk = smem_u32(smem + OFF_KV + (j & 1) * 65536);
        const uint32_t d = tmem + (j & 1) * 128;
#pragma unroll
        for (int kc = 0; kc < 2; ++kc) {
          const uint64_t ad = make_smem_desc_sw128(sq + kc * CHUNK_BYTES, 16, 1024);
          const uint64_t bd = make_smem_desc_sw128(sk + kc * CHUNK_BYTES, 16, 1024);
#pragma unroll
          for (int k = 0; k < 4; ++k) tc_mma_ss(d, ad + 2 * k, bd + 2 * k, idesc_s, (kc | k) ? 1u : 0u);
        }
        tc_commit(&B->s_full[j & 1]);
      };
      bool ok = mbar_wait(&B->q_full, 0, abort_flag) && mbar_wait(&B->k_full[0], 0, abort_flag);
      if (ok) {
        tc_fence_after_sync();
        issue_s(0);
      }
      for (int j = 0; ok && j < T; ++j) {
        if (j + 1 < T) {
          const int s1 = (j + 1) & 1;
          const uint32_t ph = ((j + 1) >> 1) & 1;
          ok = mbar_wait(&B->k_full[s1], ph, abort_flag) && mbar_wait(&B->s_empty[s1], ph ^ 1, abort_flag);
          if (!ok) break;
          tc_fence_after_sync();
          issue_s(j + 1);
        }
        const int s = j & 1;
        const uint32_t ph = (j >> 1) & 1;
        ok = mbar_wait(&B->v_full[s], ph, abort_flag) && mbar_wait(&B->p_full[s], ph, abort_flag) &&
             mbar_wait(&B->o_empty[s], ph ^ 1, abort_flag);
        if (!ok) break;
        tc_fence_after_sync();
        const uint32_t sv = smem_u32(smem + OFF_KV + s * 65536 + 32768);
        const uint32_t sp = smem_u32(smem + OFF_P + s * 32768);
        const uint32_t d = tmem + 256 + s * 128;
#pragma unroll
        for (int kc = 0; kc < 2; ++kc) {
          const uint64_t ad = make_smem_desc_sw128(sp + kc * CHUNK_BYTES, 16, 1024);
#pragma unroll
          for (int k = 0; k < 4; ++k) {
            // V tile: rows = keys (128 B each, one 64-wide half of d per chunk); 16 keys per MMA.
            const uint64_t bd = make_smem_desc_sw128(sv + (kc * 64 + k * 16) * 128, CHUNK_BYTES, 1024);
            tc_mma_ss(d, ad + 2 * k, bd, idesc_o, (kc | k) ? 1u : 0u);
          }
        }
        tc_commit(&B->o_full[s]);
        tc_commit(&B->kv_empty[s]);
        tc_commit(&B->p_empty[s]);
      }
      if (!ok) fail();
    }
    __syncwarp();
  } else {
    // ---------------------------------------------------------------- softmax + output (warps 2..17)
    // Four threads share a query row: thread (q, cq) owns score columns and output columns [32 cq, 32 cq + 32).
    const int q = warp & 3;          // TMEM lane quarter this warp may read
    const int cq = (warp - 2) >> 2;  // column quarter
    const int row = q * 32 + lane;   // row inside the tile = TMEM lane
    const uint32_t lane_base = static_cast<uint32_t>(q * 32) << 16;
    const int sw = row & 7;
    const float scale = P.scale_log2;
    const bool f16 = P.f16 != 0;

    float o[32];
#pragma unroll
    for (int i = 0; i < 32; ++i) o[i] = 0.f;
    float m = -1e30f, l = 0.f, alpha_prev = 1.f;
    uint32_t s0[32], t0[32];
    bool ok = true;

    auto accumulate = [&](int jj, float a) -> bool {
      const int ob = jj & 1;
      bool w = mbar_wait_warp(&B->o_full[ob], (jj >> 1) & 1, abort_flag);
      if (!w) return false;
      tc_fence_after_sync();
      tc_ld_32x32(tmem + lane_base + 256 + ob * 128 + cq * 32, t0);
      tc_wait_ld();
#pragma unroll
      for (int i = 0; i < 32; ++i) o[i] = fmaf(o[i], a, __uint_as_float(t0[i]));
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(&B->o_empty[ob]);
      return true;
    };

    int j = 0;
    for (; j < T; ++j) {
      const int sb = j & 1;
      const uint32_t ph = (j >> 1) & 1;
      bool w = mbar_wait_warp(&B->s_full[sb], ph, abort_flag);
      if (!w) {
        ok = false;
        break;
      }
      tc_fence_after_sync();
      tc_ld_32x32(tmem + lane_base + sb * 128 + cq * 32, s0);
      tc_wait_ld();
      // the scores are in registers now: hand the TMEM buffer back to the MMA warp
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(&B->s_empty[sb]);

      const int valid = P.seq - j * TILE - cq * 32;  // columns of my quarter that are real keys
      if (valid < 32) {
#pragma unroll
        for (int i = 0; i < 32; ++i)
          if (i >= valid) s0[i] = __float_as_uint(-1e30f);
      }
      float mloc = -1e30f;
#pragma unroll
      for (int i = 0; i < 32; ++i) mloc = fmaxf(mloc, __uint_as_float(s0[i]));
      // publish my partial maximum, wait (bounded) for the three other quarters of this row
      B->xchg[sb][cq][row] = __float2bfloat16_ru(mloc);
      __syncwarp();
      if (lane == 0) mbar_arrive(&B->mx_full[sb][q]);
      w = mbar_wait_warp(&B->mx_full[sb][q], ph, abort_flag);
      if (!w) {
        ok = false;
        break;
      }
      mloc = fmaxf(fmaxf(__bfloat162float(B->xchg[sb][0][row]), __bfloat162float(B->xchg[sb][1][row])),
                   fmaxf(__bfloat162float(B->xchg[sb][2][row]), __bfloat162float(B->xchg[sb][3][row])));
      const float mx = fmaxf(m, mloc * scale);
      const float alpha = ex2f(m - mx);

      // the P buffer of this parity is free once P V(j-2) has completed
      w = mbar_wait_warp(&B->p_empty[sb], ph ^ 1, abort_flag);
      if (!w) {
        ok = false;
        break;
      }
      // p = 2^(s*scale - max); bf16 P into shared memory: my 32 keys are half of a swizzled 128-byte row
      float rowsum = 0.f;
      uint8_t *dst = smem + OFF_P + sb * 32768 + (cq >> 1) * CHUNK_BYTES + row * 128;
#pragma unroll
      for (int t = 0; t < 4; ++t) {
        float pv[8];
#pragma unroll
        for (int e = 0; e < 8; ++e) {
          pv[e] = ex2f(fmaf(__uint_as_float(s0[8 * t + e]), scale, -mx));
          rowsum += pv[e];
        }
        uint4 v;
        v.x = pack_16x2(pv[0], pv[1], f16);
        v.y = pack_16x2(pv[2], pv[3], f16);
        v.z = pack_16x2(pv[4], pv[5], f16);
        v.w = pack_16x2(pv[6], pv[7], f16);
        const int u = (cq & 1) * 4 + t;  // 16-byte unit inside the 128-byte row
        *reinterpret_cast<uint4 *>(dst + ((u ^ sw) << 4)) = v;
      }
      fence_proxy_async_smem();
      __syncwarp();
      if (lane == 0) mbar_arrive(&B->p_full[sb]);
      l = fmaf(l, alpha, rowsum);
      if (j > 0) {
        if (!accumulate(j - 1, alpha_prev)) {
          ok = false;
          break;
        }
      }
      alpha_prev = alpha;
      m = mx;
    }
    if (ok) ok = accumulate(T - 1, alpha_prev);
    if (!ok) {
      if (lane == 0) fail();
    } else {
      // total row sum = the four quarters' partial sums (all used the same running maximum). They are exchanged
      // in f32 through the first P buffer, which the last P V has finished reading, behind the same bounded
      // barrier as the maxima (next phase of the parity the loop did not use last).
      const int sb = T & 1;
      const uint32_t ph = (T >> 1) & 1;
      float *lsum = reinterpret_cast<float *>(smem + OFF_P);  // [4][128]
      lsum[cq * 128 + row] = l;
      __syncwarp();
      if (lane == 0) mbar_arrive(&B->mx_full[sb][q]);
      bool w = mbar_wait_warp(&B->mx_full[sb][q], ph, abort_flag);
      if (!w) {
        if (lane == 0) fail();
      } else if (q0 + row < P.seq) {
        l = (lsum[row] + lsum[128 + row]) + (lsum[256 + row] + lsum[384 + row]);
        const float inv = 1.0f / l;
        __nv_bfloat16 *dstg = reinterpret_cast<__nv_bfloat16 *>(P.out) +
                              (static_cast<size_t>(batch) * P.seq + q0 + row) * P.out_ld + P.out_col + head * 128 +
                              cq * 32;
        uint4 *d4 = reinterpret_cast<uint4 *>(dstg);
#pragma unroll
        for (int t = 0; t < 4; ++t) {
          uint4 v;
          v.x = pack_16x2(o[8 * t + 0] * inv, o[8 * t + 1] * inv, f16);
          v.y = pack_16x2(o[8 * t + 2] * inv, o[8 * t + 3] * inv, f16);
          v.z = pack_16x2(o[8 * t + 4] * inv, o[8 * t + 5] * inv, f16);
          v.w = pack_16x2(o[8 * t + 6] * inv, o[8 * t + 7] * inv, f16);
          d4[t] = v;
        }
      }
    }
  }

  if (*abort_flag) {
    const long long t0 = clock64();
    while (clock64() - t0 < 2000000LL) __nanosleep(1000);
  }
  tc_fence_before_sync();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc(tmem, 512);
  }
}

// ---------------------------------------------------------------------------------------------- host
static PFN_cuTensorMapEncodeTiled_v12000 g_encode3 = nullptr;

int attn_init() {
  if (!g_encode3) {
    void *fn = nullptr;
    cudaDriverEntryPointQueryResult qres;
    cudaError_t e = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &qres);
    if (e != cudaSuccess || qres != cudaDriverEntryPointSuccess || !fn) return -1;
    g_encode3 = reinterpret_cast<PFN_cuTensorMapEncodeTiled_v12000>(fn);
  }
  return cudaFuncSetAttribute(attn_fwd_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, ATT_SMEM) == cudaSuccess
             ? 0
             : -2;
}

int attn_make_params(AttnParams *p, const void *qkv, int batch, int seq, long long ld, int q_col, int k_col, int v_col,
                     void *out, long long out_ld, int out_col, int heads, int f16, int *err) {
  if (!g_encode3 && attn_init() != 0) return -1;
  if (seq <= 0 || batch <= 0 || heads <= 0 || (ld % 8) || (q_col % 64) || (k_col % 64) || (v_col % 64) ||
      (out_ld % 8) || (out_col % 8) || (reinterpret_cast<uintptr_t>(qkv) & 15) ||
      (reinterpret_cast<uintptr_t>(out) & 15))
    return -3;
  cuuint64_t dims[3] = {static_cast<cuuint64_t>(ld), static_cast<cuuint64_t>(seq), static_cast<cuuint64_t>(batch)};
  cuuint64_t strides[2] = {static_cast<cuuint64_t>(ld) * 2, static_cast<cuuint64_t>(ld) * 2 * seq};
  cuuint32_t box[3] = {64, 128, 1};
  cuuint32_t estr[3] = {1, 1, 1};
  CUresult r = g_encode3(&p->tm, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void *>(qkv), dims, strides, box,
                         estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                         CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return -4;
  p->seq = seq;
  p->batch = batch;
  p->heads = heads;
  p->q_col = q_col;
  p->k_col = k_col;
  p->v_col = v_col;
  p->out = out;
  p->out_ld = out_ld;
  p->out_col = out_col;
  p->scale_log2 = 1.4426950408889634f / sqrtf(128.0f);
  p->f16 = f16 != 0;
  p->kv_group = 1;
  p->causal = 0;
  p->key_mask = nullptr;
  p->err = err;
  return 0;
}

int attn_launch(const AttnParams *p, cudaStream_t stream) {
  dim3 grid((p->seq + TILE - 1) / TILE, p->heads, p->batch);
  return launch_kernel(attn_fwd_kernel, grid, dim3(ATT_THREADS), ATT_SMEM, stream, 1, *p) == cudaSuccess ? 0 : -8;
}

}  // namespace fx
