// K2, third generation: the attention2.cu pipeline with the softmax of every query tile spread over EIGHT warps.
//
//   O[q, head] = softmax(Q[q, head] . K[:, head]^T / sqrt(128)) . V[:, head]
//
// replaces the reference's mha_forward / joint_attention (flux_transformer.c:1249-1330, 1335-1460; flash variant
// flux_kernels.c:700-969), and with the causal / grouped-query / key-mask options qwen3_attention_forward
// (flux_qwen3.c:313-452).
//
// What the counters of attention2.cu said: tensor pipe and exponential unit both ~39 % busy, issue slots 34 %, the
// dominant stalls "long scoreboard" (waiting for TMEM loads) and "wait" (dependent arithmetic). With ONE warp per
// scheduler working on a tile, nothing hides that warp's own latencies: the tile's 128 x 128 exponentials took ~4300
// cycles where the exponential unit needs 1024, and the tensor pipe idled for the difference because the next S of
// a tile cannot be issued before its P V (P overwrites S in TMEM). Here two warps share every 32-row quarter of a
// tile, each taking 64 of the 128 key columns, so every scheduler has two warps of the SAME tile in flight: half the
// dependent chain per thread, twice the instruction-level parallelism per scheduler.
//
// One CTA = two tiles of 128 queries of one head (of one batch element) sharing every K/V tile. TMEM (512 columns):
// S_a, S_b (f32, 128 columns each; the 16-bit P overwrites the first 64 columns of its S), O_a, O_b (f32, 128 each).
//   warp 0       TMA producer: both Q tiles once, then K tiles and V tiles through two independent two-slot rings
//                (a K slot is free as soon as both tiles' S of that key tile completed, so the next K tile is in
//                flight a whole iteration before it is needed);
//   warp 1       MMA issuer: S_t = Q_t K^T, O_t += P_t V (P_t from TMEM, V as an MN-major shared-memory operand);
//   warps 2-9    softmax of tile a, warps 10-17 of tile b. Warp w may only touch TMEM lanes 32 (w % 4) .. +31, so the
//                two warps with equal w % 4 inside a tile own the same 32 query rows and split the key columns
//                (keys 0-63 / 64-127 of the tile). The two threads of a row agree on the row maximum through shared
//                memory (value + sequence flag, bounded poll); each keeps the sum of its own columns and they are
//                added once, after the last tile. Online softmax in base 2; the running maximum is raised only when a
//                tile exceeds it by more than 8, and then each thread rescales its half of the row's O columns.
#include "attention.cuh"
#include "gemm.cuh"
#include "launch.cuh"
#include "ptx.cuh"

namespace fx {

namespace a3 {
static constexpr int THREADS = 576;        // 18 warps
static constexpr int TILE = 128;           // queries per tile, keys per step, head dim
static constexpr int QTILES = 2;           // query tiles per CTA
static constexpr int CHUNK_BYTES = 16384;  // 128 rows x 64 16-bit elements
static constexpr int OFF_Q = 0;            // tile t at t * 32768
static constexpr int OFF_K = QTILES * 32768;   // slot s at OFF_K + s * 32768
static constexpr int OFF_V = OFF_K + 2 * 32768;
static constexpr int OFF_BAR = OFF_V + 2 * 32768;
static constexpr int OFF_X = OFF_BAR + 256;    // row-statistics exchange between the two column halves
static constexpr int X_BYTES = 2 * 2 * 128 * 8;  // one 8-byte slot per [tile][half][row]
static constexpr int SMEM = OFF_X + X_BYTES + 1024;
static constexpr float RESCALE_THRESHOLD = 8.0f;  // log2 units

struct Bars {
  uint64_t q_full;
  uint64_t k_full[2], v_full[2], k_empty[2], v_empty[2];
  uint64_t s_ready[QTILES], p_ready[QTILES], o_done[QTILES];
  uint32_t tmem_slot;
  int abort_flag;
};

struct Xchg {
  // [tile][half][row]: the thread's latest row maximum (low word) and its number, 1-based (high word), published
  // with ONE 8-byte store so that a reader never sees a number without its value
  unsigned long long slot[QTILES][2][TILE];
};

// p = 2^(s * scale - m) for this thread's 64 scores, packed to 16-bit pairs and written to 32 columns of TMEM;
// returns their sum. Laid out by hand like the loop of attention2.cu: every statement is a volatile asm, each
// exponential is followed by the multiply-add that forms the argument LEAD elements ahead and by the add / convert
// that consume the pair issued LAG pairs earlier.
template <bool F16>
__device__ __forceinline__ float exps64_lagged(const uint32_t (&s)[2][32], float scale, float neg_m, uint32_t p_addr) {
  constexpr int LEAD = 8, LAG = 4, NE = 64;
  float x[LEAD], p0[LAG], p1[LAG];
  float sum4[4] = {0.f, 0.f, 0.f, 0.f};
  uint32_t pk[16];
#pragma unroll
  for (int e = 0; e < LEAD; ++e) x[e] = fmaf_pinned(__uint_as_float(s[e >> 5][e & 31]), scale, neg_m);
#pragma unroll
  for (int i = 0; i < NE / 2 + LAG; ++i) {
    const int e = 2 * i;
    const int c = i - LAG;  // pair consumed in this slot
    float t = 0.f, q0 = 0.f, q1 = 0.f;
    if (c >= 0) {
      q0 = p0[c % LAG];
      q1 = p1[c % LAG];
    }
    if (i < NE / 2) {
      p0[i % LAG] = ex2f_pinned(x[e % LEAD]);
      if (e + LEAD < NE) x[e % LEAD] = fmaf_pinned(__uint_as_float(s[(e + LEAD) >> 5][(e + LEAD) & 31]), scale, neg_m);
    }
    if (c >= 0) t = addf_pinned(q0, q1);
    if (i < NE / 2) {
      p1[i % LAG] = ex2f_pinned(x[(e + 1) % LEAD]);
      if (e + 1 + LEAD < NE)
        x[(e + 1) % LEAD] = fmaf_pinned(__uint_as_float(s[(e + 1 + LEAD) >> 5][(e + 1 + LEAD) & 31]), scale, neg_m);
    }
    if (c >= 0) {
      sum4[c & 3] = addf_pinned(sum4[c & 3], t);
      pk[c & 15] = pack_16x2_pinned<F16>(q0, q1);
      if ((c & 15) == 15) tc_st_32x16(p_addr + (c >> 4) * 16, pk);
    }
  }
  return (sum4[0] + sum4[1]) + (sum4[2] + sum4[3]);
}

// 32 lanes x 32 consecutive f32 columns (ptx.cuh) is used for S and O; P is written 16 columns at a time.
}  // namespace a3

__global__ void __launch_bounds__(a3::THREADS, 1) attn3_fwd_kernel(const __grid_constant__ AttnParams P) {
  using namespace a3;
  extern __shared__ uint8_t smem_raw[];
  uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  Bars *B = reinterpret_cast<Bars *>(smem + OFF_BAR);
  Xchg *X = reinterpret_cast<Xchg *>(smem + OFF_X);
  volatile int *abort_flag = &B->abort_flag;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int q0 = blockIdx.x * (QTILES * TILE);
  const int head = blockIdx.y;
  const int batch = blockIdx.z;
  int T = (P.seq + TILE - 1) / TILE;  // key tiles
  if (P.causal) {  // no key beyond the last query of this CTA is visible
    const int t_causal = (q0 + QTILES * TILE + TILE - 1) / TILE;
    if (t_causal < T) T = t_causal;
  }
  const int kv_head = P.kv_group > 1 ? head / P.kv_group : head;

  if (threadIdx.x == 0) {
    mbar_init(&B->q_full, 1);
    for (int i = 0; i < 2; ++i) {
      mbar_init(&B->k_full[i], 1);
      mbar_init(&B->v_full[i], 1);
      mbar_init(&B->k_empty[i], 1);
      mbar_init(&B->v_empty[i], 1);
      mbar_init(&B->s_ready[i], 1);
      mbar_init(&B->p_ready[i], 8);
      mbar_init(&B->o_done[i], 1);
    }
    B->abort_flag = 0;
    mbar_fence_init();
  }
  for (int i = threadIdx.x; i < QTILES * 2 * TILE; i += THREADS) (&X->slot[0][0][0])[i] = 0ull;
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
  const bool traced = P.trace != nullptr && blockIdx.x == 0 && blockIdx.y == 0 && blockIdx.z == 0;
  auto stamp = [&](int j, int slot) {
    if (traced) P.trace[j * 16 + slot] = clock64();
  };

  if (warp == 0) {
    // ---------------------------------------------------------------- TMA producer
    if (lane == 0) {
      tma_prefetch_desc(&P.tm);
      mbar_arrive_expect_tx(&B->q_full, QTILES * 2 * CHUNK_BYTES);
      for (int t = 0; t < QTILES; ++t) {
        uint8_t *sq = smem + OFF_Q + t * 32768;
        tma_load_3d(sq, &P.tm, &B->q_full, P.q_col + head * 128, q0 + t * TILE, batch);
        tma_load_3d(sq + CHUNK_BYTES, &P.tm, &B->q_full, P.q_col + head * 128 + 64, q0 + t * TILE, batch);
      }
      for (int j = 0; j < T; ++j) {
        const int s = j & 1;
        const uint32_t ph = ((j >> 1) & 1) ^ 1;
        if (!mbar_wait(&B->k_empty[s], ph, abort_flag)) {
          fail();
          break;
        }
        uint8_t *sk = smem + OFF_K + s * 32768;
        mbar_arrive_expect_tx(&B->k_full[s], 2 * CHUNK_BYTES);
        tma_load_3d(sk, &P.tm, &B->k_full[s], P.k_col + kv_head * 128, j * TILE, batch);
        tma_load_3d(sk + CHUNK_BYTES, &P.tm, &B->k_full[s], P.k_col + kv_head * 128 + 64, j * TILE, batch);
        if (!mbar_wait(&B->v_empty[s], ph, abort_flag)) {
          fail();
          break;
        }
        uint8_t *sv = smem + OFF_V + s * 32768;
        mbar_arrive_expect_tx(&B->v_full[s], 2 * CHUNK_BYTES);
        tma_load_3d(sv, &P.tm, &B->v_full[s], P.v_col + kv_head * 128, j * TILE, batch);
        tma_load_3d(sv + CHUNK_BYTES, &P.tm, &B->v_full[s], P.v_col + kv_head * 128 + 64, j * TILE, batch);
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    // ---------------------------------------------------------------- MMA issuer
    // all 32 lanes run the loop, one elected lane issues (see gemm2_tcgen05.cu): descriptors stay warp-uniform
    const bool leader = elect_one();
    const uint32_t fmt = P.f16 ? FMT_F16 : FMT_BF16;
    const uint32_t idesc_s = make_idesc_16(128, 128, fmt, fmt, 0, 0);  // Q (K-major) x K (K-major)
    const uint32_t idesc_o = make_idesc_16(128, 128, fmt, fmt, 0, 1);  // P (TMEM)   x V (MN-major)
    const uint32_t smem_base = smem_u32(smem);
    auto issue_s = [&](int t, int j) {
      const uint32_t sq = smem_base + OFF_Q + t * 32768;
      const uint32_t sk = smem_base + OFF_K + (j & 1) * 32768;
      const uint32_t d = tmem + t * 128;
#pragma unroll
      for (int kc = 0; kc < 2; ++kc) {
        const uint64_t ad = make_smem_desc_sw128(sq + kc * CHUNK_BYTES, 16, 1024);
        const uint64_t bd = make_smem_desc_sw128(sk + kc * CHUNK_BYTES, 16, 1024);
#pragma unroll
        for (int k = 0; k < 4; ++k)
          if (leader) tc_mma_ss(d, ad + 2 * k, bd + 2 * k, idesc_s, (kc | k) ? 1u : 0u);
      }
      if (leader) {
        tc_commit(&B->s_ready[t]);
        if (t == QTILES - 1) tc_commit(&B->k_empty[j & 1]);  // both tiles have read this K tile
      }
    };
    bool ok = mbar_wait_warp(&B->q_full, 0, abort_flag) && mbar_wait_warp(&B->k_full[0], 0, abort_flag);
    if (ok) {
      tc_fence_after_sync();
      issue_s(0, 0);
      issue_s(1, 0);
    }
    for (int j = 0; ok && j < T; ++j) {
      const int st = j & 1;
      ok = mbar_wait_warp(&B->v_full[st], (j >> 1) & 1, abort_flag);
      if (leader) stamp(j, 0);
      // V tile: rows = keys (128 B each, one 64-wide half of d per chunk); 16 keys (2048 B) per MMA
      const uint64_t vd = make_smem_desc_sw128(smem_base + OFF_V + st * 32768, CHUNK_BYTES, 1024);
      for (int t = 0; ok && t < QTILES; ++t) {
        ok = mbar_wait_warp(&B->p_ready[t], j & 1, abort_flag);
        if (!ok) break;
        if (leader) stamp(j, 1 + 2 * t);
        tc_fence_after_sync();
        const uint32_t d = tmem + 256 + t * 128;
        const uint32_t pa = tmem + t * 128;
#pragma unroll
        for (int k = 0; k < 8; ++k)
          if (leader) tc_mma_ts(d, pa + k * 8, vd + static_cast<uint64_t>(k) * (2048 >> 4), idesc_o, (j | k) ? 1u : 0u);
        if (leader) {
          tc_commit(&B->o_done[t]);
          if (t == QTILES - 1) tc_commit(&B->v_empty[st]);
        }
        if (j + 1 < T) {
          if (t == 0) {
            ok = mbar_wait_warp(&B->k_full[(j + 1) & 1], ((j + 1) >> 1) & 1, abort_flag);
            if (!ok) break;
            tc_fence_after_sync();
          }
          issue_s(t, j + 1);  // overwrites P_t(j): issued after P_t V(j), executed after it
        }
        if (leader) stamp(j, 2 + 2 * t);
      }
    }
    if (!ok && lane == 0) fail();
    __syncwarp();
  } else {
    // ---------------------------------------------------------------- softmax + output (warps 2..17)
    const int sw = warp - 2;
    const int t = sw >> 3;          // query tile
    const int half = (sw >> 2) & 1; // key columns 64 half .. 64 half + 63 of every tile
    const int q = warp & 3;         // TMEM lane quarter this warp may access
    const int row = q * 32 + lane;  // row inside the tile = TMEM lane
    const uint32_t lane_base = static_cast<uint32_t>(q * 32) << 16;
    const uint32_t s_addr = tmem + lane_base + t * 128 + half * 64;        // this thread's 64 score columns
    const uint32_t p_addr = tmem + lane_base + t * 128 + half * 32;        // ... become 32 columns of 16-bit pairs
    const uint32_t o_addr = tmem + lane_base + 256 + t * 128 + half * 64;  // its half of the row's output columns
    const float scale = P.scale_log2;
    const bool f16 = P.f16 != 0;
    volatile unsigned long long *slot_mine = &X->slot[t][half][row];
    volatile unsigned long long *slot_other = &X->slot[t][half ^ 1][row];

    // Publishes `v` as this thread's value number n (1-based) and returns the partner's value number n. The partner
    // cannot publish number n + 1 before this thread has arrived on p_ready for step n, i.e. after this read.
    auto exchange = [&](float v, int n, bool &ok) -> float {
      *slot_mine = (static_cast<unsigned long long>(n) << 32) | __float_as_uint(v);
      unsigned long long o = *slot_other;
      if (static_cast<int>(o >> 32) < n) {
        const long long t0 = clock64();
        while (true) {
          o = *slot_other;
          if (static_cast<int>(o >> 32) >= n) break;
          if (*abort_flag || clock64() - t0 > WAIT_LIMIT_CYCLES) {
            ok = false;
            return v;
          }
        }
      }
      return __uint_as_float(static_cast<uint32_t>(o));
    };

    float m_ref = -1e30f, l = 0.f;
    uint32_t s[2][32];
    bool ok = true;

    for (int j = 0; j < T; ++j) {
      ok = mbar_wait_warp(&B->s_ready[t], j & 1, abort_flag);
      if (!ok) break;
      const bool tr = (sw & 7) == 0 && lane == 0;  // the first warp of each tile
      if (tr) stamp(j, 5 + 5 * t);
      tc_fence_after_sync();
      tc_ld_32x32(s_addr, s[0]);
      tc_ld_32x32(s_addr + 32, s[1]);
      tc_wait_ld();
      if (tr) stamp(j, 6 + 5 * t);
      // keys of this tile this row may see: inside the sequence, not after the query (causal), not masked out
      int limit = P.seq - j * TILE;
      if (P.causal) {
        const int lim_c = q0 + t * TILE + row - j * TILE + 1;
        if (lim_c < limit) limit = lim_c;
      }
      if (limit < TILE || P.key_mask) {
        uint32_t mw[2] = {0xffffffffu, 0xffffffffu};
        if (P.key_mask) {
          const int words = (P.seq + 31) / 32;
#pragma unroll
          for (int c = 0; c < 2; ++c)
            if (j * 4 + half * 2 + c < words)
              mw[c] = __ldg(P.key_mask + static_cast<size_t>(batch) * words + j * 4 + half * 2 + c);
        }
#pragma unroll
        for (int c = 0; c < 2; ++c)
#pragma unroll
          for (int i = 0; i < 32; ++i)
            if (half * 64 + c * 32 + i >= limit || !((mw[c] >> i) & 1u)) s[c][i] = __float_as_uint(-1e30f);
      }
      // four independent chains for the maximum of this thread's 64 scores
      float m4[4] = {-1e30f, -1e30f, -1e30f, -1e30f};
#pragma unroll
      for (int c = 0; c < 2; ++c)
#pragma unroll
        for (int i = 0; i < 32; ++i) m4[i & 3] = fmaxf(m4[i & 3], __uint_as_float(s[c][i]));
      float mloc = fmaxf(fmaxf(m4[0], m4[1]), fmaxf(m4[2], m4[3])) * scale;
      // the row's maximum over all 128 keys: the partner thread holds the other 64. The exchange also orders this
      // thread's stores of P below after the partner's loads of the S columns they overwrite.
      mloc = fmaxf(mloc, exchange(mloc, j + 1, ok));
      ok = __all_sync(0xffffffffu, ok);  // the lanes polled separately: agree, and reconverge for the TMEM accesses
      if (!ok) break;
      // Raise the reference maximum only when this tile exceeds it by more than the threshold.
      const bool raise = mloc > m_ref + RESCALE_THRESHOLD;
      if (j == 0) {
        m_ref = mloc;
      } else if (__any_sync(0xffffffffu, raise)) {
        // rescale this thread's half of the accumulator row in TMEM once P V(j-1) has completed
        ok = mbar_wait_warp(&B->o_done[t], (j - 1) & 1, abort_flag);
        if (!ok) break;
        tc_fence_after_sync();
        const float alpha = raise ? ex2f_(m_ref - mloc) : 1.0f;
        uint32_t o[16];  // 16 columns at a time: the 64 scores of this tile stay live in registers meanwhile
#pragma unroll 1
        for (int c = 0; c < 4; ++c) {
          tc_ld_32x16(o_addr + c * 16, o);
          tc_wait_ld();
#pragma unroll
          for (int i = 0; i < 16; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * alpha);
          tc_st_32x16(o_addr + c * 16, o);
        }
        tc_wait_st();
        if (raise) {
          l *= alpha;
          m_ref = mloc;
        }
      }
      if (tr) stamp(j, 7 + 5 * t);
      // p = 2^(s*scale - m_ref); 16-bit pairs: keys 2c, 2c+1 of the tile in column c of S
      l += f16 ? exps64_lagged<true>(s, scale, -m_ref, p_addr) : exps64_lagged<false>(s, scale, -m_ref, p_addr);
      if (tr) stamp(j, 8 + 5 * t);
      tc_wait_st();
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(&B->p_ready[t]);
      if (tr) stamp(j, 9 + 5 * t);
    }
    if (ok) {
      l += exchange(l, T + 1, ok);  // the row's sum over all keys
      ok = __all_sync(0xffffffffu, ok);
    }
    if (ok) ok = mbar_wait_warp(&B->o_done[t], (T - 1) & 1, abort_flag);
    if (!ok) {
      if (lane == 0) fail();
    } else {
      tc_fence_after_sync();
      const float inv = 1.0f / l;
      const int grow = q0 + t * TILE + row;
      __nv_bfloat16 *dstg = reinterpret_cast<__nv_bfloat16 *>(P.out) +
                            (static_cast<size_t>(batch) * P.seq + grow) * P.out_ld + P.out_col + head * 128 + half * 64;
      uint32_t o[32];
#pragma unroll 1
      for (int c = 0; c < 2; ++c) {
        tc_ld_32x32(o_addr + c * 32, o);
        tc_wait_ld();
        if (grow < P.seq) {
          uint4 *d4 = reinterpret_cast<uint4 *>(dstg + c * 32);
#pragma unroll
          for (int u = 0; u < 4; ++u) {
            uint4 v;
            v.x = pack_16x2(__uint_as_float(o[8 * u + 0]) * inv, __uint_as_float(o[8 * u + 1]) * inv, f16);
            v.y = pack_16x2(__uint_as_float(o[8 * u + 2]) * inv, __uint_as_float(o[8 * u + 3]) * inv, f16);
            v.z = pack_16x2(__uint_as_float(o[8 * u + 4]) * inv, __uint_as_float(o[8 * u + 5]) * inv, f16);
            v.w = pack_16x2(__uint_as_float(o[8 * u + 6]) * inv, __uint_as_float(o[8 * u + 7]) * inv, f16);
            d4[u] = v;
          }
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
int attn3_init() {
  return cudaFuncSetAttribute(attn3_fwd_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, a3::SMEM) == cudaSuccess
             ? 0
             : -2;
}

// Parameters are those of attn2_make_params (attention2.cu): same tensor map, same options.
int attn3_launch(const AttnParams *p, cudaStream_t stream) {
  dim3 grid((p->seq + a3::QTILES * a3::TILE - 1) / (a3::QTILES * a3::TILE), p->heads, p->batch);
  return launch_kernel(attn3_fwd_kernel, grid, dim3(a3::THREADS), a3::SMEM, stream, 1, *p) == cudaSuccess ? 0 : -8;
}

}  // namespace fx
