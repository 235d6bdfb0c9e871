// Fused epilogues of the tcgen05 GEMM kernels: what one epilogue thread (one TMEM lane = one output row)
// does with a finished 128 x BN f32 accumulator tile. Shared by the 1-CTA and the 2-CTA kernel.
#pragma once
#include "gemm.cuh"
#include "ptx.cuh"

namespace fx {

__device__ __forceinline__ float silu_f(float x) { return x / (1.0f + __expf(-x)); }

// Shared-memory staging of the TMA-store epilogues: two 32 x 32 f32 blocks (4 KB each, 1024-byte aligned) per warp.
static constexpr int EPI_STAGE_BYTES_PER_WARP = 2 * 4096;

// One 32-column chunk of this warp's 32 rows goes out through the TMA unit: every lane writes its row's 32 floats
// into the staging block (16-byte pieces permuted as the 128-byte swizzle wants them, which also keeps the eight
// lanes of a store phase on different banks), then one lane hands the block to the TMA unit.
template <bool REDUCE>
__device__ __forceinline__ void stage_and_store_chunk(const CUtensorMap *tm, uint8_t *buf, const float (&v)[32], int lane,
                                                      int x, int y, bool issue) {
  const uint32_t base = smem_u32(buf) + static_cast<uint32_t>(lane) * 128u;
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    const uint32_t a = base + static_cast<uint32_t>((j ^ (lane & 7)) * 16);
    asm volatile("st.shared.v4.f32 [%0], {%1, %2, %3, %4};" ::"r"(a), "f"(v[4 * j]), "f"(v[4 * j + 1]),
                 "f"(v[4 * j + 2]), "f"(v[4 * j + 3])
                 : "memory");
  }
  fence_proxy_async_smem();
  __syncwarp();
  if (lane == 0 && issue) {
    if (REDUCE) tma_reduce_add_2d(tm, buf, x, y);
    else tma_store_2d(tm, buf, x, y);
    bulk_commit();
  }
}

// 16-bit outputs through the TMA unit: a staging block holds 32 rows x 64 columns (128 bytes per row), i.e. two
// 32-column chunks of the accumulator, written four 16-byte pieces at a time (stage_pieces4, ptx.cuh); the two blocks
// of a warp alternate so that one is being filled while the TMA unit still reads the other.
struct Stage16 {
  uint8_t *stage;
  int lane;
  int n;   // blocks handed to the TMA unit so far
  int nb;  // blocks available (a power of two)
  __device__ __forceinline__ uint8_t *acquire() {
    if (n >= nb) {  // every store but the latest has read its block, the one that last used this block among them
      if (lane == 0) bulk_wait_read<1>();
      __syncwarp();
    }
    return stage + (n & (nb - 1)) * 4096;
  }
  __device__ __forceinline__ void release(const CUtensorMap *tm, uint8_t *buf, int x, int y, bool issue) {
    fence_proxy_async_smem();
    __syncwarp();
    if (lane == 0 && issue) {
      tma_store_2d(tm, buf, x, y);
      bulk_commit();
    }
    ++n;
  }
  __device__ __forceinline__ void drain() {  // before anything else writes the blocks again
    if (lane == 0) bulk_wait_read<0>();
    __syncwarp();
  }
};

// stage: this warp's staging blocks (paired kernel) or nullptr (direct global stores); nblk: how many 4 KB blocks it
// holds (a power of two, at least 2). With two blocks a chunk waits for the TMA unit to have read the chunk before
// last; with eight (the operand ring, free during a CTA's last tile) a whole tile is staged without waiting.
template <int BN>
__device__ __forceinline__ void epilogue_tile(const GemmProblem &pb, int m0, int n0, uint32_t taddr, int lane_row,
                                              int *sat_counter, uint8_t *stage = nullptr, int nblk = 2) {
  const bool second = n0 >= pb.n_split;
  const EpiSeg &sg = second ? pb.seg[1] : pb.seg[0];
  const int nrel = n0 - (second ? pb.n_split : 0);  // segment-relative first column of this tile
  const int row = m0 + lane_row;
  const bool row_ok = row < pb.M;
  const bool f16 = sg.out_f16 != 0;
  float mx = 0.f;  // largest magnitude this thread converted to 16 bits (f16 stores saturate at 65504)
  uint32_t r[32];
#ifdef FLUX_CUDA_DEBUG
  {
    // Checked build: the tile must lie inside the problem and this row's destination inside the row pitch and on a
    // 16-byte boundary. A violation is recorded in the error word and the tile is skipped - nothing is accessed.
    const int width = sg.mode == EPI_SWIGLU_BF16 ? BN / 2 : BN;
    const int first = sg.mode == EPI_SWIGLU_BF16 ? sg.col0 + nrel / 2 : sg.col0 + nrel;
    const int esz = (sg.mode == EPI_STORE_BF16 || sg.mode == EPI_SWIGLU_BF16 || sg.mode == EPI_QKV_NORM_ROPE) ? 2 : 4;
    bool bad = m0 < 0 || n0 < 0 || n0 + BN > pb.N || m0 >= pb.M + 128 || nrel < 0 || sg.out == nullptr;
    if (sg.mode != EPI_STORE_F32_T) {
      bad = bad || first < 0 || static_cast<long long>(first) + width > sg.ld ||
            ((reinterpret_cast<uintptr_t>(sg.out) + (static_cast<size_t>(row_ok ? row : 0) * sg.ld + first) * esz) & 15);
    } else {
      bad = bad || sg.ld < pb.M;
    }
    if (bad) {
      if (sat_counter != nullptr) atomicCAS(sat_counter - 1, 0, KERR_BAD_INDEX);
      return;
    }
  }
#endif

  switch (sg.mode) {
    case EPI_STORE_BF16: {
      if (stage != nullptr && sg.tma_out) {
        const int lane = lane_row & 31, y = m0 + (lane_row & ~31);
        Stage16 st{stage, lane, 0, nblk};
        uint8_t *buf = nullptr;
        tc_ld_32x32(taddr, r);  // chunk c + 1 is loaded while chunk c is staged
#pragma unroll 1
        for (int c = 0; c < BN / 32; ++c) {
          if ((c & 1) == 0) buf = st.acquire();
          tc_wait_ld();
          uint32_t w[16];
#pragma unroll
          for (int j = 0; j < 16; ++j)
            w[j] = pack_16x2_t(__uint_as_float(r[2 * j]), __uint_as_float(r[2 * j + 1]), f16, mx);
          if (c + 1 < BN / 32) tc_ld_32x32(taddr + (c + 1) * 32, r);
          stage_pieces4(buf, lane, w, (c & 1) * 4);
          if (c & 1) st.release(&sg.tm_out, buf, sg.col0 + nrel + (c - 1) * 32, y, y < pb.M);
        }
        st.drain();
        break;
      }
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
            v.x = pack_16x2_t(__uint_as_float(r[8 * j + 0]), __uint_as_float(r[8 * j + 1]), f16, mx);
            v.y = pack_16x2_t(__uint_as_float(r[8 * j + 2]), __uint_as_float(r[8 * j + 3]), f16, mx);
            v.z = pack_16x2_t(__uint_as_float(r[8 * j + 4]), __uint_as_float(r[8 * j + 5]), f16, mx);
            v.w = pack_16x2_t(__uint_as_float(r[8 * j + 6]), __uint_as_float(r[8 * j + 7]), f16, mx);
            d4[j] = v;
          }
        }
      }
    } break;
    case EPI_STORE_F32: {
      if (stage != nullptr && sg.tma_out) {
        const int lane = lane_row & 31, y = m0 + (lane_row & ~31);
        // The TMEM load of chunk c + 1 is issued as soon as chunk c sits in `v`, so that it runs under the staging
        // stores, the proxy fence and the TMA issue of chunk c.
        tc_ld_32x32(taddr, r);
#pragma unroll 1
        for (int c = 0; c < BN / 32; ++c) {
          if (c >= nblk) {  // the store that last used this block has read it
            if (lane == 0) bulk_wait_read<1>();
            __syncwarp();
          }
          tc_wait_ld();
          float v[32];
#pragma unroll
          for (int j = 0; j < 32; ++j) v[j] = __uint_as_float(r[j]);
          if (c + 1 < BN / 32) tc_ld_32x32(taddr + (c + 1) * 32, r);
          stage_and_store_chunk<false>(&sg.tm_out, stage + (c & (nblk - 1)) * 4096, v, lane, sg.col0 + nrel + c * 32, y,
                                       y < pb.M);
        }
        if (lane == 0) bulk_wait_read<0>();  // the next tile's epilogue writes these blocks again
        __syncwarp();
        break;
      }
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
      if (stage != nullptr && sg.tma_out) {
        // out += gate * acc as a TMA reduce-add: the residual is read and updated in L2, the SM only sends gate * acc
        const int lane = lane_row & 31, y = m0 + (lane_row & ~31);
        const float4 *g4 = reinterpret_cast<const float4 *>(sg.gate + nrel);
        // Pipelined like the plain f32 store; the chunk's gate values are requested before the wait for its
        // accumulator, so that their latency runs under it.
        tc_ld_32x32(taddr, r);
#pragma unroll 1
        for (int c = 0; c < BN / 32; ++c) {
          float4 g[8];
#pragma unroll
          for (int j = 0; j < 8; ++j) g[j] = __ldg(g4 + c * 8 + j);
          if (c >= nblk) {
            if (lane == 0) bulk_wait_read<1>();
            __syncwarp();
          }
          tc_wait_ld();
          float v[32];
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            v[4 * j + 0] = g[j].x * __uint_as_float(r[4 * j + 0]);
            v[4 * j + 1] = g[j].y * __uint_as_float(r[4 * j + 1]);
            v[4 * j + 2] = g[j].z * __uint_as_float(r[4 * j + 2]);
            v[4 * j + 3] = g[j].w * __uint_as_float(r[4 * j + 3]);
          }
          if (c + 1 < BN / 32) tc_ld_32x32(taddr + (c + 1) * 32, r);
          stage_and_store_chunk<true>(&sg.tm_out, stage + (c & (nblk - 1)) * 4096, v, lane, sg.col0 + nrel + c * 32, y,
                                      y < pb.M);
        }
        if (lane == 0) bulk_wait_read<0>();
        __syncwarp();
        break;
      }
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
        uint32_t u[32];
        if (stage != nullptr && sg.tma_out) {
          const int lane = lane_row & 31, y = m0 + (lane_row & ~31);
          Stage16 st{stage, lane, 0, nblk};
          uint8_t *buf = nullptr;
#pragma unroll 1
          for (int c = 0; c < 4; ++c) {
            tc_ld_32x32(taddr + c * 32, r);
            tc_ld_32x32(taddr + 128 + c * 32, u);
            if ((c & 1) == 0) buf = st.acquire();
            tc_wait_ld();
            uint32_t w[16];
#pragma unroll
            for (int j = 0; j < 16; ++j)
              w[j] = pack_16x2_t(silu_f(__uint_as_float(r[2 * j])) * __uint_as_float(u[2 * j]),
                                 silu_f(__uint_as_float(r[2 * j + 1])) * __uint_as_float(u[2 * j + 1]), f16, mx);
            stage_pieces4(buf, lane, w, (c & 1) * 4);
            if (c & 1) st.release(&sg.tm_out, buf, sg.col0 + nrel / 2 + (c - 1) * 32, y, y < pb.M);
          }
          st.drain();
          break;
        }
        __nv_bfloat16 *dst =
            reinterpret_cast<__nv_bfloat16 *>(sg.out) + static_cast<size_t>(row) * sg.ld + sg.col0 + nrel / 2;
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
              v.x = pack_16x2_t(o[0], o[1], f16, mx);
              v.y = pack_16x2_t(o[2], o[3], f16, mx);
              v.z = pack_16x2_t(o[4], o[5], f16, mx);
              v.w = pack_16x2_t(o[6], o[7], f16, mx);
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
        const bool rotate = col < qk.q_cols + qk.k_cols;
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
          const bool is_k = col >= qk.q_cols;
          w = (pos < qk.n_txt) ? (is_k ? qk.wk_txt : qk.wq_txt) : (is_k ? qk.wk_img : qk.wq_img);
        }
        if (rotate && qk.half_split && stage != nullptr && sg.tma_out && qk.ang != nullptr) {
          // pairs (i, i + 64) with the pair angles read 16 bytes at a time, and both halves of the head leaving
          // through the TMA unit: staging block 0 collects columns 0..63 of the head, block 1 columns 64..127
          const int lane = lane_row & 31, y = m0 + (lane_row & ~31);
          uint32_t u[32];
          if (lane == 0) bulk_wait_read<0>();  // both blocks are free
          __syncwarp();
#pragma unroll 1
          for (int c = 0; c < 2; ++c) {
            tc_ld_32x32(th + c * 32, r);
            tc_ld_32x32(th + 64 + c * 32, u);
            float4 an4[8];
            const float4 *a4 = reinterpret_cast<const float4 *>(qk.ang + static_cast<size_t>(pos) * 64 + c * 32);
#pragma unroll
            for (int j = 0; j < 8; ++j) an4[j] = __ldg(a4 + j);
            tc_wait_ld();
            const float4 *wa4 = reinterpret_cast<const float4 *>(w + c * 32);
            const float4 *wb4 = reinterpret_cast<const float4 *>(w + 64 + c * 32);
            uint32_t oa[16], ob[16];
#pragma unroll
            for (int j = 0; j < 8; ++j) {
              const float4 wa = __ldg(wa4 + j), wb = __ldg(wb4 + j);
              const float av[4] = {an4[j].x, an4[j].y, an4[j].z, an4[j].w};
              const float wav[4] = {wa.x, wa.y, wa.z, wa.w}, wbv[4] = {wb.x, wb.y, wb.z, wb.w};
              float ya[4], yb[4];
#pragma unroll
              for (int k = 0; k < 4; ++k) {
                const float x0 = __uint_as_float(r[4 * j + k]) * rinv * wav[k];
                const float x1 = __uint_as_float(u[4 * j + k]) * rinv * wbv[k];
                float sn, cs;
                __sincosf(av[k], &sn, &cs);
                ya[k] = x0 * cs - x1 * sn;
                yb[k] = x0 * sn + x1 * cs;
              }
              oa[2 * j] = pack_16x2_t(ya[0], ya[1], f16, mx);
              oa[2 * j + 1] = pack_16x2_t(ya[2], ya[3], f16, mx);
              ob[2 * j] = pack_16x2_t(yb[0], yb[1], f16, mx);
              ob[2 * j + 1] = pack_16x2_t(yb[2], yb[3], f16, mx);
            }
            stage_pieces4(stage, lane, oa, c * 4);
            stage_pieces4(stage + 4096, lane, ob, c * 4);
          }
          fence_proxy_async_smem();
          __syncwarp();
          if (lane == 0) {
            if (y < pb.M) {
              tma_store_2d(&sg.tm_out, stage, sg.col0 + nrel + hd * 128, y);
              tma_store_2d(&sg.tm_out, stage + 4096, sg.col0 + nrel + hd * 128 + 64, y);
              bulk_commit();
            }
            bulk_wait_read<0>();  // whatever uses the blocks next finds them free
          }
          __syncwarp();
          continue;
        }
        if (rotate && qk.half_split) {
          // pairs (i, i + 64): chunk c of the first half rotates with chunk c of the second half
          uint32_t u[32];
#pragma unroll 1
          for (int c = 0; c < 2; ++c) {
            tc_ld_32x32(th + c * 32, r);
            tc_ld_32x32(th + 64 + c * 32, u);
            tc_wait_ld();
            if (row_ok) {
              const float *wa = w + c * 32, *wb = w + 64 + c * 32;
              const float *cs = qk.cos_t + static_cast<size_t>(pos) * 64 + c * 32;
              const float *sn = qk.sin_t + static_cast<size_t>(pos) * 64 + c * 32;
              uint4 *da = reinterpret_cast<uint4 *>(dst + hd * 128 + c * 32);
              uint4 *db = reinterpret_cast<uint4 *>(dst + hd * 128 + 64 + c * 32);
#pragma unroll
              for (int j = 0; j < 4; ++j) {
                uint32_t oa[4], ob[4];
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                  float ya[2], yb[2];
#pragma unroll
                  for (int k = 0; k < 2; ++k) {
                    const int i = 8 * j + 2 * e + k;
                    const float x0 = __uint_as_float(r[i]) * rinv * __ldg(wa + i);
                    const float x1 = __uint_as_float(u[i]) * rinv * __ldg(wb + i);
                    const float cc = __ldg(cs + i), ss = __ldg(sn + i);
                    ya[k] = x0 * cc - x1 * ss;
                    yb[k] = x0 * ss + x1 * cc;
                  }
                  oa[e] = pack_16x2_t(ya[0], ya[1], f16, mx);
                  ob[e] = pack_16x2_t(yb[0], yb[1], f16, mx);
                }
                da[j] = make_uint4(oa[0], oa[1], oa[2], oa[3]);
                db[j] = make_uint4(ob[0], ob[1], ob[2], ob[3]);
              }
            }
          }
          continue;
        }
        if (stage != nullptr && sg.tma_out) {
          const int lane = lane_row & 31, y = m0 + (lane_row & ~31);
          Stage16 st{stage, lane, 0, nblk};
          uint8_t *buf = nullptr;
#pragma unroll 1
          for (int c = 0; c < 4; ++c) {
            tc_ld_32x32(th + c * 32, r);
            // 16 pair angles of this row and chunk: four scattered 16-byte loads instead of sixteen, issued before
            // the wait for the accumulator so that the two latencies overlap
            float4 an4[4];
            if (rotate && qk.ang != nullptr) {
              const float4 *a4 = reinterpret_cast<const float4 *>(qk.ang + static_cast<size_t>(pos) * 64 + c * 16);
#pragma unroll
              for (int j4 = 0; j4 < 4; ++j4) an4[j4] = __ldg(a4 + j4);
            }
            if ((c & 1) == 0) buf = st.acquire();
            tc_wait_ld();
            uint32_t wv[16];
            if (rotate && qk.ang != nullptr) {
              const float4 *w4 = reinterpret_cast<const float4 *>(w + c * 32);
#pragma unroll
              for (int j4 = 0; j4 < 4; ++j4) {
                const float4 an = an4[j4];
                const float ang4[4] = {an.x, an.y, an.z, an.w};
#pragma unroll
                for (int e = 0; e < 2; ++e) {
                  const int j = 2 * j4 + e;  // float4 index inside the chunk: elements 4j .. 4j+3 = pairs 2j, 2j+1
                  const float4 ww = __ldg(w4 + j);
                  float s0, c0, s1, c1;
                  __sincosf(ang4[2 * e], &s0, &c0);
                  __sincosf(ang4[2 * e + 1], &s1, &c1);
                  const float x0 = __uint_as_float(r[4 * j + 0]) * rinv * ww.x;
                  const float x1 = __uint_as_float(r[4 * j + 1]) * rinv * ww.y;
                  const float x2 = __uint_as_float(r[4 * j + 2]) * rinv * ww.z;
                  const float x3 = __uint_as_float(r[4 * j + 3]) * rinv * ww.w;
                  wv[2 * j + 0] = pack_16x2_t(x0 * c0 - x1 * s0, x1 * c0 + x0 * s0, f16, mx);
                  wv[2 * j + 1] = pack_16x2_t(x2 * c1 - x3 * s1, x3 * c1 + x2 * s1, f16, mx);
                }
              }
            } else if (rotate) {
              const float4 *w4 = reinterpret_cast<const float4 *>(w + c * 32);
              const float4 *c4 = reinterpret_cast<const float4 *>(qk.cos_t + static_cast<size_t>(pos) * 128 + c * 32);
              const float4 *s4 = reinterpret_cast<const float4 *>(qk.sin_t + static_cast<size_t>(pos) * 128 + c * 32);
#pragma unroll
              for (int j = 0; j < 8; ++j) {
                const float4 ww = __ldg(w4 + j);
                const float4 cc = __ldg(c4 + j);
                const float4 sn = __ldg(s4 + j);
                const float x0 = __uint_as_float(r[4 * j + 0]) * rinv * ww.x;
                const float x1 = __uint_as_float(r[4 * j + 1]) * rinv * ww.y;
                const float x2 = __uint_as_float(r[4 * j + 2]) * rinv * ww.z;
                const float x3 = __uint_as_float(r[4 * j + 3]) * rinv * ww.w;
                wv[2 * j + 0] = pack_16x2_t(x0 * cc.x - x1 * sn.x, x1 * cc.x + x0 * sn.x, f16, mx);
                wv[2 * j + 1] = pack_16x2_t(x2 * cc.z - x3 * sn.z, x3 * cc.z + x2 * sn.z, f16, mx);
              }
            } else {
#pragma unroll
              for (int j = 0; j < 16; ++j)
                wv[j] = pack_16x2_t(__uint_as_float(r[2 * j]), __uint_as_float(r[2 * j + 1]), f16, mx);
            }
            stage_pieces4(buf, lane, wv, (c & 1) * 4);
            if (c & 1) st.release(&sg.tm_out, buf, sg.col0 + nrel + hd * 128 + (c - 1) * 32, y, y < pb.M);
          }
          st.drain();
          continue;
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
                  o[2 * e + 0] = pack_16x2_t(x0 * cc.x - x1 * sn.x, x1 * cc.x + x0 * sn.x, f16, mx);
                  o[2 * e + 1] = pack_16x2_t(x2 * cc.z - x3 * sn.z, x3 * cc.z + x2 * sn.z, f16, mx);
                }
                d4[j] = make_uint4(o[0], o[1], o[2], o[3]);
              }
            } else {
#pragma unroll
              for (int j = 0; j < 4; ++j) {
                uint4 v;
                v.x = pack_16x2_t(__uint_as_float(r[8 * j + 0]), __uint_as_float(r[8 * j + 1]), f16, mx);
                v.y = pack_16x2_t(__uint_as_float(r[8 * j + 2]), __uint_as_float(r[8 * j + 3]), f16, mx);
                v.z = pack_16x2_t(__uint_as_float(r[8 * j + 4]), __uint_as_float(r[8 * j + 5]), f16, mx);
                v.w = pack_16x2_t(__uint_as_float(r[8 * j + 6]), __uint_as_float(r[8 * j + 7]), f16, mx);
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
  sat_report(sat_counter, f16, mx);
}

}  // namespace fx
