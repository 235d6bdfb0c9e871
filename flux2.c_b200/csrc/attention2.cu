// K2: joint text+image attention, flash style, on tcgen05.
//
//   O[q, head] = softmax(Q[q, head] . K[:, head]^T / sqrt(128)) . V[:, head]      no mask, all N keys
//
// replaces the reference's mha_forward / joint_attention (flux_transformer.c:1249-1330, 1335-1460;
// flash variant flux_kernels.c:700-969). Text and image tokens live in ONE [txt ; img ; refs] sequence
// in this engine, so the double-stream blocks' joint attention (both streams' queries against the
// concatenated keys) and the single-stream blocks' attention are the same launch.
//
// One CTA = TWO tiles of 128 queries of one head (of one batch element) that share every K/V tile and
// alternate on the tensor pipe, so that while the softmax warps of one tile exponentiate, the pipe
// works for the other. Q, K, V are read by TMA straight out of the fused projection output
// [B, N, ld] (16-bit, 128-byte swizzle, 64-column boxes). TMEM (512 columns): scores S_a, S_b (f32,
// 128 columns each; the 16-bit probabilities P overwrite the first 64 columns of their S) and the two
// output accumulators O_a, O_b (f32, 128 columns each). Roles:
//   warp 0      TMA producer: both Q tiles once, then a two-stage ring of K/V tiles (128 keys each);
//   warp 1      MMA issuer: S_t = Q_t K^T (both operands K-major in shared memory) and
//               O_t += P_t V (A = P_t from TMEM, B = V as an MN-major shared-memory operand);
//   warps 4-7   softmax of tile a, warps 8-11 of tile b: one thread per query row (its TMEM lane). Warps 2-3 only
//               give their registers to the softmax warps.
//               Online softmax in base 2 with f32 statistics. The reference maximum of a row is only raised when a
//               tile exceeds it by more than 8 (p stays below 2^8), so the accumulator in TMEM rarely has to be
//               rescaled; when it does, the row's thread multiplies its O row in place (tcgen05.ld / tcgen05.st)
//               before it releases P for the next P V. After the first tile the exponentials are taken against the
//               current reference right away and the tile's own maximum is not computed at all unless a partial sum
//               says that a probability may have left that range (then the tile is redone exactly from the scores
//               still in registers): the 128 comparisons per row and tile leave the serial chain
//               S -> softmax -> P V -> next S that bounds this kernel.
#include "attention.cuh"
#include "gemm.cuh"
#include "launch.cuh"
#include "ptx.cuh"

#include <cudaTypedefs.h>
#include <stdlib.h>

namespace fx {

static constexpr int ATT_THREADS = 384;
static constexpr int REGS_LAUNCH = 160;   // a floor of what 384 threads per block get at launch (ptxas reports 168)
static constexpr int REGS_ISSUE = 64;     // producer / MMA-issuer warp group after giving registers back
static constexpr int REGS_SOFTMAX = 208;  // the two softmax warp groups after taking them
static constexpr int TILE = 128;           // queries per tile, keys per step, head dim
static constexpr int QTILES = 2;           // query tiles per CTA
static constexpr int CHUNK_BYTES = 16384;  // 128 rows x 64 16-bit elements
static constexpr int OFF_Q = 0;            // tile t at t * 32768
static constexpr int OFF_KV = QTILES * 32768;  // stage s: K at OFF_KV + s*65536, V 32768 after it
static constexpr int OFF_BAR = OFF_KV + 2 * 65536;
static constexpr int ATT_SMEM = OFF_BAR + 256 + 1024;
static constexpr float RESCALE_THRESHOLD = 8.0f;  // log2 units

// p = 2^(s * scale - m) for the 128 scores of one row, packed to 16-bit pairs and written over the first 64 columns
// of S in TMEM; returns the row's sum. The special-function unit takes 8 cycles per warp instruction and its results
// come back tens of cycles later, so the instruction stream is laid out by hand (every statement below is a volatile
// asm, which keeps this order): each exponential is followed by the multiply-add that forms the argument LEAD
// elements ahead and by the add / convert that consume the pair issued LAG pairs earlier - never by an instruction
// that needs a result still in flight.
// `smax` returns the largest of the four partial sums (32 probabilities each): no single probability can be above it,
// which is the overflow check of the speculative pass at no cost inside the loop.
template <bool F16>
__device__ __forceinline__ float exps_row_lagged(const uint32_t (&s)[4][32], float scale, float neg_m, uint32_t s_addr,
                                                 float &smax) {
  constexpr int LEAD = 8, LAG = 4;
  float x[LEAD], p0[LAG], p1[LAG];
  float sum4[4] = {0.f, 0.f, 0.f, 0.f};
  uint32_t pk[32];
#pragma unroll
  for (int e = 0; e < LEAD; ++e) x[e] = fmaf_pinned(__uint_as_float(s[e >> 5][e & 31]), scale, neg_m);
#pragma unroll
  for (int i = 0; i < 64 + LAG; ++i) {
    const int e = 2 * i;
    float t = 0.f;
    const int c = i - LAG;  // pair consumed in this slot
    float q0 = 0.f, q1 = 0.f;
    if (c >= 0) {
      q0 = p0[c % LAG];
      q1 = p1[c % LAG];
    }
    if (i < 64) {
      p0[i % LAG] = ex2f_pinned(x[e % LEAD]);
      if (e + LEAD < 128) x[e % LEAD] = fmaf_pinned(__uint_as_float(s[(e + LEAD) >> 5][(e + LEAD) & 31]), scale, neg_m);
    }
    if (c >= 0) t = addf_pinned(q0, q1);
    if (i < 64) {
      p1[i % LAG] = ex2f_pinned(x[(e + 1) % LEAD]);
      if (e + 1 + LEAD < 128)
        x[(e + 1) % LEAD] = fmaf_pinned(__uint_as_float(s[(e + 1 + LEAD) >> 5][(e + 1 + LEAD) & 31]), scale, neg_m);
    }
    if (c >= 0) {
      sum4[c & 3] = addf_pinned(sum4[c & 3], t);
      pk[c & 31] = pack_16x2_pinned<F16>(q0, q1);
      if ((c & 31) == 31) tc_st_32x32(s_addr + (c >> 5) * 32, pk);
    }
  }
  smax = fmaxf(fmaxf(sum4[0], sum4[1]), fmaxf(sum4[2], sum4[3]));
  return (sum4[0] + sum4[1]) + (sum4[2] + sum4[3]);
}

struct Attn2Bars {
  uint64_t q_full;
  uint64_t k_full[2], v_full[2], kv_empty[2];
  uint64_t s_ready[QTILES], p_ready[QTILES], o_done[QTILES];
  uint32_t tmem_slot;
  int abort_flag;
};

__global__ void __launch_bounds__(ATT_THREADS, 1) attn2_fwd_kernel(const __grid_constant__ AttnParams P) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  Attn2Bars *B = reinterpret_cast<Attn2Bars *>(smem + OFF_BAR);
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
#ifdef FLUX_CUDA_DEBUG
  // Checked build: every TMA coordinate of this CTA must start on a 16-byte boundary and inside the row; otherwise
  // the CTA records the fact and leaves before anything is loaded.
  if (((P.q_col + head * 128) | (P.k_col + kv_head * 128) | (P.v_col + kv_head * 128) | P.out_col) & 7 || q0 < 0 ||
      q0 >= P.seq + QTILES * TILE || T < 1) {
    if (threadIdx.x == 0) atomicCAS(P.err, 0, KERR_BAD_INDEX);
    return;
  }
#endif

  if (threadIdx.x == 0) {
    mbar_init(&B->q_full, 1);
    for (int i = 0; i < 2; ++i) {
      mbar_init(&B->k_full[i], 1);
      mbar_init(&B->v_full[i], 1);
      mbar_init(&B->kv_empty[i], 1);
      mbar_init(&B->s_ready[i], 1);
      mbar_init(&B->p_ready[i], 4);
      mbar_init(&B->o_done[i], 1);
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
  const bool traced = P.trace != nullptr && blockIdx.x == 0 && blockIdx.y == 0 && blockIdx.z == 0;
  auto stamp = [&](int j, int slot) {
    if (traced) P.trace[j * 16 + slot] = clock64();
  };

  // Registers follow the work: the producer / issuer warp group gives registers back (64 per thread), the two
  // softmax groups, which hold a row's 128 scores plus the packed probabilities, take 216. The reallocation sits at
  // the top of each group's own branch, so that the compiler budgets each branch separately. The increase waits
  // (in hardware, without a bound) until the block's pool holds enough registers, so the sum after reallocation
  // must not exceed what the block was launched with - checked at compile time below.
  static_assert(128 * REGS_ISSUE + 256 * REGS_SOFTMAX <= ATT_THREADS * REGS_LAUNCH,
                "register reallocation asks for more than the block owns: setmaxnreg.inc would wait forever");
  if (warp < 4) {
    asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(REGS_ISSUE));
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
        if (!mbar_wait(&B->kv_empty[s], ((j >> 1) & 1) ^ 1, abort_flag)) {
          fail();
          break;
        }
        uint8_t *sk = smem + OFF_KV + s * 65536;
        uint8_t *sv = sk + 32768;
        stamp(j, 15);
        mbar_arrive_expect_tx(&B->k_full[s], 2 * CHUNK_BYTES);
        tma_load_3d(sk, &P.tm, &B->k_full[s], P.k_col + kv_head * 128, j * TILE, batch);
        tma_load_3d(sk + CHUNK_BYTES, &P.tm, &B->k_full[s], P.k_col + kv_head * 128 + 64, j * TILE, batch);
        mbar_arrive_expect_tx(&B->v_full[s], 2 * CHUNK_BYTES);
        tma_load_3d(sv, &P.tm, &B->v_full[s], P.v_col + kv_head * 128, j * TILE, batch);
        tma_load_3d(sv + CHUNK_BYTES, &P.tm, &B->v_full[s], P.v_col + kv_head * 128 + 64, j * TILE, batch);
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    // ---------------------------------------------------------------- MMA issuer
    // All 32 lanes run this loop and one elected lane issues each instruction: the operand descriptors and TMEM
    // addresses then stay warp-uniform values, which the compiler keeps in the uniform datapath the tcgen05
    // instructions read their operands from. (With the whole role inside `if (lane == 0)` every descriptor had to be
    // moved over from a per-thread register, and the issue of a 64-cycle MMA took ~100 cycles.)
    const bool leader = elect_one();
    const uint32_t fmt = P.f16 ? FMT_F16 : FMT_BF16;
    const uint32_t idesc_s = make_idesc_16(128, 128, fmt, fmt, 0, 0);  // Q (K-major) x K (K-major)
    const uint32_t idesc_o = make_idesc_16(128, 128, fmt, fmt, 0, 1);  // P (TMEM)   x V (MN-major)
    const uint32_t smem_base = smem_u32(smem);
    auto issue_s = [&](int t, int j) {
      const uint32_t d = tmem + t * 128;
      const uint32_t sq = smem_base + OFF_Q + t * 32768;
      const uint32_t sk = smem_base + OFF_KV + (j & 1) * 65536;
#pragma unroll
      for (int kc = 0; kc < 2; ++kc) {
        const uint64_t ad = make_smem_desc_sw128(sq + kc * CHUNK_BYTES, 16, 1024);
        const uint64_t bd = make_smem_desc_sw128(sk + kc * CHUNK_BYTES, 16, 1024);
#pragma unroll
        for (int k = 0; k < 4; ++k)
          if (leader) tc_mma_ss(d, ad + 2 * k, bd + 2 * k, idesc_s, (kc | k) ? 1u : 0u);
      }
      if (leader) tc_commit(&B->s_ready[t]);
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
      const uint64_t vd = make_smem_desc_sw128(smem_base + OFF_KV + st * 65536 + 32768, CHUNK_BYTES, 1024);
      for (int t = 0; ok && t < QTILES; ++t) {
        ok = mbar_wait_warp(&B->p_ready[t], j & 1, abort_flag);
        if (!ok) break;
        if (leader) stamp(j, 1 + 2 * t);
        tc_fence_after_sync();
        // O_t (+)= P_t V: P_t sits in the first 64 columns of S_t, 16 keys = 8 columns per MMA
        const uint32_t d = tmem + 256 + t * 128;
        const uint32_t pa = tmem + t * 128;
#pragma unroll
        for (int k = 0; k < 8; ++k)
          if (leader) tc_mma_ts(d, pa + k * 8, vd + static_cast<uint64_t>(k) * (2048 >> 4), idesc_o, (j | k) ? 1u : 0u);
        if (leader) {
          tc_commit(&B->o_done[t]);
          if (t == QTILES - 1) tc_commit(&B->kv_empty[st]);
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
  }
  } else {
    // ---------------------------------------------------------------- softmax + output (warps 4..11)
    asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(REGS_SOFTMAX));
    const int t = (warp - 4) >> 2;  // query tile
    const int q = warp & 3;         // TMEM lane quarter this warp may access
    const int row = q * 32 + lane;  // row inside the tile = TMEM lane
    const uint32_t lane_base = static_cast<uint32_t>(q * 32) << 16;
    const uint32_t s_addr = tmem + lane_base + t * 128;
    const uint32_t o_addr = tmem + lane_base + 256 + t * 128;
    const float scale = P.scale_log2;
    const bool f16 = P.f16 != 0;

    float m_ref = -1e30f, l = 0.f;
    uint32_t s[4][32];
    bool ok = true;

    for (int j = 0; j < T; ++j) {
      ok = mbar_wait_warp(&B->s_ready[t], j & 1, abort_flag);
      if (!ok) break;
      const bool tr = q == 0 && lane == 0;  // warps 4 and 8: the first warp of each tile
      if (tr) stamp(j, 5 + 5 * t);
      tc_fence_after_sync();
#pragma unroll
      for (int c = 0; c < 4; ++c) tc_ld_32x32(s_addr + c * 32, s[c]);
      tc_wait_ld();
      if (tr) stamp(j, 6 + 5 * t);
      // keys of this tile this row may see: inside the sequence, not after the query (causal), not masked out
      int limit = P.seq - j * TILE;
      if (P.causal) {
        const int lim_c = q0 + t * TILE + row - j * TILE + 1;
        if (lim_c < limit) limit = lim_c;
      }
      if (limit < TILE || P.key_mask) {
        uint32_t mw[4] = {0xffffffffu, 0xffffffffu, 0xffffffffu, 0xffffffffu};
        if (P.key_mask) {
          const int words = (P.seq + 31) / 32;
#pragma unroll
          for (int c = 0; c < 4; ++c)
            if (j * 4 + c < words) mw[c] = __ldg(P.key_mask + static_cast<size_t>(batch) * words + j * 4 + c);
        }
#pragma unroll
        for (int c = 0; c < 4; ++c)
#pragma unroll
          for (int i = 0; i < 32; ++i)
            if (c * 32 + i >= limit || !((mw[c] >> i) & 1u)) s[c][i] = __float_as_uint(-1e30f);
      }
      // Speculative pass: the exponentials are taken against the CURRENT reference maximum right away, and the row
      // maximum of this tile - which is only needed to decide whether the reference has to be raised - is not
      // computed at all unless some probability may have come out above 2^8 (the bound the lazy rescaling keeps: a
      // partial sum of 32 probabilities above 2^8 is the sign). In that
      // rare case, and for the first tile, the exact path below redoes the tile from the scores still in registers.
      float tile_sum = 0.f, smax = 0.f;
      bool exact = j == 0 || !P.spec;
      if (!exact) {
        tile_sum = f16 ? exps_row_lagged<true>(s, scale, -m_ref, s_addr, smax)
                       : exps_row_lagged<false>(s, scale, -m_ref, s_addr, smax);
        exact = __any_sync(0xffffffffu, !(smax <= 256.0f));  // also catches inf / NaN
        if (exact) tc_wait_st();  // the speculative P is overwritten below
      }
      if (exact) {
        // four independent chains for the maximum of the row's 128 scores (one chain would cost 128 dependent steps)
        float m4[4] = {-1e30f, -1e30f, -1e30f, -1e30f};
#pragma unroll
        for (int c = 0; c < 4; ++c)
#pragma unroll
          for (int i = 0; i < 32; ++i) m4[i & 3] = fmaxf(m4[i & 3], __uint_as_float(s[c][i]));
        const float mloc = fmaxf(fmaxf(m4[0], m4[1]), fmaxf(m4[2], m4[3])) * scale;
        // Raise the reference maximum only when this tile exceeds it by more than the threshold - or, when the
        // speculative pass sent us here, by anything at all: a tile whose scores sit a few bits above the reference
        // without reaching the threshold would otherwise fail the check of every following tile too.
        const bool raise = mloc > m_ref + ((P.spec && j > 0) ? 0.0f : RESCALE_THRESHOLD);
        if (j == 0) {
          m_ref = mloc;
        } else if (__any_sync(0xffffffffu, raise)) {
          // rescale the accumulator row in TMEM once P V(j-1) has completed
          ok = mbar_wait_warp(&B->o_done[t], (j - 1) & 1, abort_flag);
          if (!ok) break;
          tc_fence_after_sync();
          const float alpha = raise ? ex2f_(m_ref - mloc) : 1.0f;
          uint32_t o[32];
#pragma unroll 1
          for (int c = 0; c < 4; ++c) {
            tc_ld_32x32(o_addr + c * 32, o);
            tc_wait_ld();
#pragma unroll
            for (int i = 0; i < 32; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * alpha);
            tc_st_32x32(o_addr + c * 32, o);
          }
          tc_wait_st();
          if (raise) {
            l *= alpha;
            m_ref = mloc;
          }
        }
        if (tr) stamp(j, 7 + 5 * t);
        // p = 2^(s*scale - m_ref); 16-bit pairs into the first 64 columns of S (keys 2c, 2c+1 in column c)
        tile_sum = f16 ? exps_row_lagged<true>(s, scale, -m_ref, s_addr, smax)
                       : exps_row_lagged<false>(s, scale, -m_ref, s_addr, smax);
      }
      l += tile_sum;
      if (tr) stamp(j, 8 + 5 * t);
      tc_wait_st();
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(&B->p_ready[t]);
      if (tr) stamp(j, 9 + 5 * t);
    }
    if (ok) ok = mbar_wait_warp(&B->o_done[t], (T - 1) & 1, abort_flag);
    if (!ok) {
      if (lane == 0) fail();
    } else {
      tc_fence_after_sync();
      const float inv = 1.0f / l;
      const int grow = q0 + t * TILE + row;
      uint32_t o[32];
      if (P.tma_out) {
        // The Q tile of this query tile is no longer read by anything (its last MMA completed before o_done), so its
        // 32 KB hold the output on its way out: each warp packs its 32 rows x 128 columns into two swizzled blocks
        // of 32 rows x 64 columns and hands them to the TMA unit, which clips rows past the end of the sequence.
        uint8_t *stg = smem + OFF_Q + t * 32768 + q * 8192;
#pragma unroll 1
        for (int c = 0; c < 4; ++c) {
          tc_ld_32x32(o_addr + c * 32, o);
          tc_wait_ld();
          uint32_t w[16];
#pragma unroll
          for (int u = 0; u < 16; ++u)
            w[u] = pack_16x2(__uint_as_float(o[2 * u]) * inv, __uint_as_float(o[2 * u + 1]) * inv, f16);
          stage_pieces4(stg + (c >> 1) * 4096, lane, w, (c & 1) * 4);
        }
        fence_proxy_async_smem();
        __syncwarp();
        const int y0 = q0 + t * TILE + q * 32;
        if (lane == 0 && y0 < P.seq) {
          const int x0 = P.out_col + head * 128;
          tma_store_3d(&P.tm_out, stg, x0, y0, batch);
          tma_store_3d(&P.tm_out, stg + 4096, x0 + 64, y0, batch);
          bulk_commit();
          bulk_wait<0>();
        }
      } else {
        __nv_bfloat16 *dstg = reinterpret_cast<__nv_bfloat16 *>(P.out) +
                              (static_cast<size_t>(batch) * P.seq + grow) * P.out_ld + P.out_col + head * 128;
#pragma unroll 1
        for (int c = 0; c < 4; ++c) {
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
static PFN_cuTensorMapEncodeTiled_v12000 g_encode4 = nullptr;

int attn2_init() {
  if (!g_encode4) {
    void *fn = nullptr;
    cudaDriverEntryPointQueryResult qres;
    cudaError_t e = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &qres);
    if (e != cudaSuccess || qres != cudaDriverEntryPointSuccess || !fn) return -1;
    g_encode4 = reinterpret_cast<PFN_cuTensorMapEncodeTiled_v12000>(fn);
  }
  return cudaFuncSetAttribute(attn2_fwd_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, ATT_SMEM) == cudaSuccess
             ? 0
             : -2;
}

int attn2_make_params(AttnParams *p, const void *qkv, int batch, int seq, long long ld, int q_col, int k_col, int v_col,
                     void *out, long long out_ld, int out_col, int heads, int f16, int *err) {
  if (!g_encode4 && attn2_init() != 0) return -1;
  if (seq <= 0 || batch <= 0 || heads <= 0 || (ld % 8) || (q_col % 64) || (k_col % 64) || (v_col % 64) ||
      (out_ld % 8) || (out_col % 8) || (reinterpret_cast<uintptr_t>(qkv) & 15) ||
      (reinterpret_cast<uintptr_t>(out) & 15))
    return -3;
  cuuint64_t dims[3] = {static_cast<cuuint64_t>(ld), static_cast<cuuint64_t>(seq), static_cast<cuuint64_t>(batch)};
  cuuint64_t strides[2] = {static_cast<cuuint64_t>(ld) * 2, static_cast<cuuint64_t>(ld) * 2 * seq};
  cuuint32_t box[3] = {64, 128, 1};
  cuuint32_t estr[3] = {1, 1, 1};
  CUresult r = g_encode4(&p->tm, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void *>(qkv), dims, strides, box,
                         estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                         CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return -4;
  // The output as [batch, seq, out_ld] with a box of 32 rows x 64 columns: one warp's staging block. Opt out with
  // FLUX_CUDA_ATTN_TMA_OUT=0 (per-row 16-byte stores instead).
  static const int tma_out_env = [] {
    const char *e = getenv("FLUX_CUDA_ATTN_TMA_OUT");
    return e ? atoi(e) : 1;
  }();
  static const int spec_env = [] {
    const char *e = getenv("FLUX_CUDA_ATTN_SPEC");
    return e ? atoi(e) : 1;
  }();
  p->spec = spec_env;
  p->tma_out = 0;
  if (tma_out_env) {
    cuuint64_t odims[3] = {static_cast<cuuint64_t>(out_ld), static_cast<cuuint64_t>(seq),
                           static_cast<cuuint64_t>(batch)};
    cuuint64_t ostrides[2] = {static_cast<cuuint64_t>(out_ld) * 2, static_cast<cuuint64_t>(out_ld) * 2 * seq};
    cuuint32_t obox[3] = {64, 32, 1};
    r = g_encode4(&p->tm_out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, out, odims, ostrides, obox, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_NONE,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return -4;
    p->tma_out = 1;
  }
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
  p->trace = nullptr;
  return 0;
}

int attn2_launch(const AttnParams *p, cudaStream_t stream) {
  dim3 grid((p->seq + QTILES * TILE - 1) / (QTILES * TILE), p->heads, p->batch);
  return launch_kernel(attn2_fwd_kernel, grid, dim3(ATT_THREADS), ATT_SMEM, stream, 1, *p) == cudaSuccess ? 0 : -8;
}

}  // namespace fx
