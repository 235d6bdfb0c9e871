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
#include "ptx.cuh"

#include <cudaTypedefs.h>

namespace fx {

static constexpr int ATT_THREADS = 320;    // warp 0 TMA, warp 1 MMA, warps 2..9 softmax
static constexpr int TILE = 128;           // queries per CTA, keys per step, head dim
static constexpr int CHUNK_BYTES = 16384;  // 128 rows x 64 bf16
static constexpr int OFF_Q = 0;
static constexpr int OFF_KV = 32768;  // stage s: K at OFF_KV + s*65536, V 32768 after it
static constexpr int OFF_P = OFF_KV + 2 * 65536;  // two P buffers of 32 KB
static constexpr int OFF_BAR = OFF_P + 2 * 32768;
static constexpr int ATT_SMEM = OFF_BAR + 2048 + 1024;

struct AttnBars {
  uint64_t q_full;
  uint64_t k_full[2], v_full[2], kv_empty[2];
  uint64_t s_full[2], s_empty[2];
  uint64_t p_full[2], p_empty[2];
  uint64_t o_full[2], o_empty[2];
  uint32_t tmem_slot;
  int abort_flag;
  float xchg[2][128];  // [column half][row]: partial row sums exchanged once, at the end, between the two
                       // threads that share a query row
};

__device__ __forceinline__ float ex2f(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ void pair_sync(int id) { asm volatile("bar.sync %0, 64;" ::"r"(id) : "memory"); }

__global__ void __launch_bounds__(ATT_THREADS, 1) attn_fwd_kernel(const __grid_constant__ AttnParams P) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  AttnBars *B = reinterpret_cast<AttnBars *>(smem + OFF_BAR);
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
      mbar_init(&B->s_empty[i], 8);
      mbar_init(&B->p_full[i], 8);
      mbar_init(&B->p_empty[i], 1);
      mbar_init(&B->o_full[i], 1);
      mbar_init(&B->o_empty[i], 8);
    }
    B->abort_flag = 0;
    mbar_fence_init();
  }
  if (warp == 1) tmem_alloc(&B->tmem_slot, 512);
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem = B->tmem_slot;

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
      constexpr uint32_t idesc_s = make_idesc_bf16(128, 128, 0, 0);  // Q (K-major) x K (K-major)
      constexpr uint32_t idesc_o = make_idesc_bf16(128, 128, 0, 1);  // P (K-major) x V (MN-major)
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
    // ---------------------------------------------------------------- softmax + output (warps 2..9)
    // Two threads share a query row: thread (q, hf) owns score columns and output columns [64 hf, 64 hf + 64).
    const int q = warp & 3;          // TMEM lane quarter this warp may read
    const int hf = (warp - 2) >> 2;  // column half
    const int row = q * 32 + lane;   // row inside the tile = TMEM lane
    const uint32_t lane_base = static_cast<uint32_t>(q * 32) << 16;
    const int sw = row & 7;
    const float scale = P.scale_log2;

    float o[64];
#pragma unroll
    for (int i = 0; i < 64; ++i) o[i] = 0.f;
    float m = -1e30f, l = 0.f, alpha_prev = 1.f;
    uint32_t s0[32], s1[32];
    bool ok = true;

    auto accumulate = [&](int jj, float a) -> bool {
      const int ob = jj & 1;
      bool w = mbar_wait(&B->o_full[ob], (jj >> 1) & 1, abort_flag);
      w = __all_sync(0xffffffffu, w);
      if (!w) return false;
      tc_fence_after_sync();
      const uint32_t to = tmem + lane_base + 256 + ob * 128 + hf * 64;
      tc_ld_32x32(to, s0);
      tc_ld_32x32(to + 32, s1);
      tc_wait_ld();
#pragma unroll
      for (int i = 0; i < 32; ++i) {
        o[i] = fmaf(o[i], a, __uint_as_float(s0[i]));
        o[32 + i] = fmaf(o[32 + i], a, __uint_as_float(s1[i]));
      }
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(&B->o_empty[ob]);
      return true;
    };

    for (int j = 0; j < T; ++j) {
      const int sb = j & 1;
      const uint32_t ph = (j >> 1) & 1;
      bool w = mbar_wait(&B->s_full[sb], ph, abort_flag);
      w = __all_sync(0xffffffffu, w);
      if (!w) {
        ok = false;
        break;
      }
      tc_fence_after_sync();
      // Row maximum over all 128 columns: the partner's half is read only for its maximum (TMEM reads are
      // cheap and this keeps the two warps of a row free of any per-tile synchronisation).
      const uint32_t tb = tmem + lane_base + sb * 128;
      const int valid_all = P.seq - j * TILE;          // real keys in this tile
      const int valid = valid_all - hf * 64;           // ... of them in my half
      const int valid_o = valid_all - (hf ^ 1) * 64;   // ... in the partner's half
      float mloc = -1e30f;
#pragma unroll 1
      for (int c = 0; c < 2; ++c) {
        tc_ld_32x32(tb + (hf ^ 1) * 64 + c * 32, s0);
        tc_wait_ld();
        if (valid_o >= 64) {
#pragma unroll
          for (int i = 0; i < 32; ++i) mloc = fmaxf(mloc, __uint_as_float(s0[i]));
        } else {
#pragma unroll
          for (int i = 0; i < 32; ++i)
            if (c * 32 + i < valid_o) mloc = fmaxf(mloc, __uint_as_float(s0[i]));
        }
      }
      tc_ld_32x32(tb + hf * 64, s0);
      tc_ld_32x32(tb + hf * 64 + 32, s1);
      tc_wait_ld();
      // the score buffer is in registers now: hand it back to the MMA warp
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(&B->s_empty[sb]);
      if (valid < 64) {
#pragma unroll
        for (int i = 0; i < 32; ++i) {
          if (i >= valid) s0[i] = __float_as_uint(-1e30f);
          if (32 + i >= valid) s1[i] = __float_as_uint(-1e30f);
        }
      }
#pragma unroll
      for (int i = 0; i < 32; ++i) mloc = fmaxf(mloc, fmaxf(__uint_as_float(s0[i]), __uint_as_float(s1[i])));
      const float mx = fmaxf(m, mloc * scale);
      const float alpha = ex2f(m - mx);

      // the P buffer of this parity is free once P V(j-2) has completed
      w = mbar_wait(&B->p_empty[sb], ph ^ 1, abort_flag);
      w = __all_sync(0xffffffffu, w);
      if (!w) {
        ok = false;
        break;
      }
      // p = 2^(s*scale - max); bf16 P into shared memory: my 64 keys are one swizzled 128-byte row of chunk hf
      float rowsum = 0.f;
      uint8_t *dst = smem + OFF_P + sb * 32768 + hf * CHUNK_BYTES + row * 128;
#pragma unroll
      for (int t = 0; t < 8; ++t) {
        float pv[8];
#pragma unroll
        for (int e = 0; e < 8; ++e) {
          const int i = 8 * t + e;
          const float sv = __uint_as_float(i < 32 ? s0[i] : s1[i - 32]);
          pv[e] = ex2f(fmaf(sv, scale, -mx));
          rowsum += pv[e];
        }
        uint4 v;
        v.x = pack_bf16x2(pv[0], pv[1]);
        v.y = pack_bf16x2(pv[2], pv[3]);
        v.z = pack_bf16x2(pv[4], pv[5]);
        v.w = pack_bf16x2(pv[6], pv[7]);
        *reinterpret_cast<uint4 *>(dst + ((t ^ sw) << 4)) = v;
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
    }
    // total row sum = my half + the partner's half (both halves used the same running maximum)
    // Every softmax warp passes here exactly once, whatever happened above, so the pair barrier cannot hang.
    B->xchg[hf][row] = l;
    pair_sync(1 + q);
    l += B->xchg[hf ^ 1][row];
    if (ok && q0 + row < P.seq) {
      const float inv = 1.0f / l;
      __nv_bfloat16 *dstg = reinterpret_cast<__nv_bfloat16 *>(P.out) +
                            (static_cast<size_t>(batch) * P.seq + q0 + row) * P.out_ld + P.out_col + head * 128 +
                            hf * 64;
      uint4 *d4 = reinterpret_cast<uint4 *>(dstg);
#pragma unroll
      for (int t = 0; t < 8; ++t) {
        uint4 v;
        v.x = pack_bf16x2(o[8 * t + 0] * inv, o[8 * t + 1] * inv);
        v.y = pack_bf16x2(o[8 * t + 2] * inv, o[8 * t + 3] * inv);
        v.z = pack_bf16x2(o[8 * t + 4] * inv, o[8 * t + 5] * inv);
        v.w = pack_bf16x2(o[8 * t + 6] * inv, o[8 * t + 7] * inv);
        d4[t] = v;
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
                     void *out, long long out_ld, int out_col, int heads, int *err) {
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
  p->err = err;
  return 0;
}

int attn_launch(const AttnParams *p, cudaStream_t stream) {
  dim3 grid((p->seq + TILE - 1) / TILE, p->heads, p->batch);
  attn_fwd_kernel<<<grid, ATT_THREADS, ATT_SMEM, stream>>>(*p);
  return cudaGetLastError() == cudaSuccess ? 0 : -8;
}

}  // namespace fx
