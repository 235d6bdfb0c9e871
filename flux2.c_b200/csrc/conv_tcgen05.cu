// K8: 3x3 convolution as an implicit GEMM on the tcgen05 tensor cores, for the VAE.
//
// Activations are channels-last, so output pixel p and output channel co are
//     out[p, co] = bias[co] + sum over taps (ky, kx) and input channels ci of in[p + (ky-1, kx-1), ci] * w[co, tap, ci]
// i.e. a GEMM whose K dimension is (tap, ci). Nothing is materialised: for every k-slice (one tap, 64 input
// channels) the producer issues ONE 4-D TMA load of a pixel patch shifted by the tap's offset; pixels outside the
// image are filled with zeros by the TMA unit, which is exactly the convolution's zero padding. The rest is the
// paired GEMM of gemm2_tcgen05.cu: a cluster of two CTAs owns 256 pixels x BN output channels, each CTA stages its
// own 128-pixel patch and half of the weight slice, one thread of the leader issues tcgen05.mma cta_group::2 into
// both CTAs' TMEM, accumulators are double-buffered so the epilogue of one tile overlaps the MMAs of the next.
// With taps = 1 the same kernel is a plain GEMM with a bias (1x1 convolutions, the attention block's products).
#include <cudaTypedefs.h>

#include "conv.cuh"
#include "gemm.cuh"
#include "launch.cuh"
#include "ptx.cuh"

namespace fx {

static constexpr int C_BM = 128;
static constexpr int C_BK = 64;
static constexpr int C_STAGES = 6;
static constexpr int C_THREADS = 192;
template <int BN>
struct ConvCfg {
  static constexpr int A_BYTES = C_BM * C_BK * 2;
  static constexpr int B_BYTES = (BN / 2) * C_BK * 2;
  static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
  static constexpr int SMEM = C_STAGES * STAGE_BYTES + 256 + 1024;
  static constexpr int TMEM_COLS = 2 * BN;
};

__device__ __forceinline__ void tma_load_4d_pair(void *smem_dst, const CUtensorMap *m, uint32_t bar_cluster_addr,
                                                 int c0, int c1, int c2, int c3) {
  asm volatile(
      "cp.async.bulk.tensor.4d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, "
      "%5, %6}], [%2];" ::"r"(smem_u32(smem_dst)),
      "l"(reinterpret_cast<uint64_t>(m)), "r"(bar_cluster_addr), "r"(c0), "r"(c1), "r"(c2), "r"(c3)
      : "memory");
}

// Sums over the warp's 32 rows of N values per lane in N - 1 + 5 - log2(N) shuffles: at every step a lane hands
// one half of its values to its partner and adds the partner's other half, so the number of live values halves
// while the number of rows folded into each doubles. Afterwards lane L holds the total of value L >> (5 - log2 N).
template <int N>
__device__ __forceinline__ float warp_multi_sum(float (&a)[N], int lane) {
  int m = 16;
#pragma unroll
  for (int half = N / 2; half >= 1; half /= 2, m >>= 1) {
    const bool up = (lane & m) != 0;
#pragma unroll
    for (int j = 0; j < half; ++j) {
      const float send = up ? a[j] : a[j + half];
      const float recv = __shfl_xor_sync(0xffffffffu, send, m);
      a[j] = (up ? a[j + half] : a[j]) + recv;
    }
  }
  float t = a[0];
  for (; m >= 1; m >>= 1) t += __shfl_xor_sync(0xffffffffu, t, m);
  return t;
}

// v: this row's 32 consecutive output channels = 32 / CPG groups. Stores the warp's per-group sums and sums of
// squares (rows outside the image count as zero): group k of the chunk at dst[k * 2 * slots] (sum) and
// dst[(k * 2 + 1) * slots] (sum of squares).
template <int CPG>
__device__ __forceinline__ void gn_chunk_sums(const float (&v)[32], bool row_ok, float *dst, size_t slots) {
  constexpr int NG = 32 / CPG, N = 2 * NG;
  float a[N];
#pragma unroll
  for (int g = 0; g < NG; ++g) {
    float s = 0.f, ss = 0.f;
#pragma unroll
    for (int j = 0; j < CPG; ++j) {
      const float x = v[g * CPG + j];
      s += x;
      ss += x * x;
    }
    a[g] = row_ok ? s : 0.f;
    a[NG + g] = row_ok ? ss : 0.f;
  }
  const int lane = threadIdx.x & 31;
  const float t = warp_multi_sum<N>(a, lane);
  constexpr int SH = N == 16 ? 1 : (N == 8 ? 2 : 3);  // 5 - log2(N)
  if ((lane & ((1 << SH) - 1)) == 0) {
    const int k = lane >> SH;  // value index: k < NG sums, then NG sums of squares
    const int g = k < NG ? k : k - NG;
    dst[(static_cast<size_t>(g) * 2 + (k < NG ? 0 : 1)) * slots] = t;
  }
}

// One epilogue thread = one output row (pixel): reads its TMEM lane 32 columns at a time.
template <int BN>
__device__ __forceinline__ void conv_epilogue(const ConvParams &P, size_t row, bool row_ok, int n0, uint32_t taddr,
                                              size_t warp_slot) {
  uint32_t r[32];
  const bool f16 = P.out_f16 != 0;
  float mx = 0.f;
  if (P.mode == CONV_STORE_RGB8) {
    tc_ld_32x32(taddr, r);
    tc_wait_ld();
    if (row_ok && n0 == 0) {
      uint8_t *dst = reinterpret_cast<uint8_t *>(P.out) + row * 3;
#pragma unroll
      for (int c = 0; c < 3; ++c) {
        float v = __uint_as_float(r[c]) + (P.bias ? __ldg(P.bias + c) : 0.f);
        v = (v + 1.0f) * 0.5f * 255.0f;
        v = fminf(fmaxf(v, 0.f), 255.f);
        dst[c] = static_cast<uint8_t>(v);
      }
    }
    return;
  }
#pragma unroll 1
  for (int c = 0; c < BN / 32; ++c) {
    tc_ld_32x32(taddr + c * 32, r);
    tc_wait_ld();
    if (!row_ok && !P.gn_partial) continue;
    const int col = n0 + c * 32;
    float v[32];
    if (P.bias) {
      const float4 *b4 = reinterpret_cast<const float4 *>(P.bias + col);
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const float4 b = __ldg(b4 + j);
        v[4 * j + 0] = __uint_as_float(r[4 * j + 0]) + b.x;
        v[4 * j + 1] = __uint_as_float(r[4 * j + 1]) + b.y;
        v[4 * j + 2] = __uint_as_float(r[4 * j + 2]) + b.z;
        v[4 * j + 3] = __uint_as_float(r[4 * j + 3]) + b.w;
      }
    } else {
#pragma unroll
      for (int j = 0; j < 32; ++j) v[j] = __uint_as_float(r[j]);
    }
    if (P.mode == CONV_STORE_16) {
      if (row_ok) {
        uint4 *d4 = reinterpret_cast<uint4 *>(reinterpret_cast<uint16_t *>(P.out) + row * P.ld + col);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          uint4 o;
          o.x = pack_16x2_t(v[8 * j + 0], v[8 * j + 1], f16, mx);
          o.y = pack_16x2_t(v[8 * j + 2], v[8 * j + 3], f16, mx);
          o.z = pack_16x2_t(v[8 * j + 4], v[8 * j + 5], f16, mx);
          o.w = pack_16x2_t(v[8 * j + 6], v[8 * j + 7], f16, mx);
          d4[j] = o;
        }
      }
    } else if (row_ok) {
      float4 *d4 = reinterpret_cast<float4 *>(reinterpret_cast<float *>(P.out) + row * P.ld + col);
      const bool add = P.mode == CONV_ADD_F32;
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        if (add) {
          const float4 h = d4[j];
          v[4 * j + 0] += h.x;
          v[4 * j + 1] += h.y;
          v[4 * j + 2] += h.z;
          v[4 * j + 3] += h.w;
        }
        d4[j] = make_float4(v[4 * j + 0], v[4 * j + 1], v[4 * j + 2], v[4 * j + 3]);
      }
    }
    if (P.gn_partial) {  // statistics of what was just written, for the GroupNorm that reads it next
      // group-major layout: [group][sum | sum of squares][row slot], so that the fold reads contiguous floats
      const size_t slots = static_cast<size_t>(P.tiles_m) * 8;
      float *dst = P.gn_partial + static_cast<size_t>(col / P.gn_cpg) * 2 * slots + warp_slot;
      if (P.gn_cpg == 4) gn_chunk_sums<4>(v, row_ok, dst, slots);
      else if (P.gn_cpg == 8) gn_chunk_sums<8>(v, row_ok, dst, slots);
      else gn_chunk_sums<16>(v, row_ok, dst, slots);
    }
  }
  sat_report(P.err + 1, f16 && P.mode == CONV_STORE_16, mx);
}

template <int BN>
__global__ void __launch_bounds__(C_THREADS, 1) conv2_tn_kernel(const __grid_constant__ ConvParams P) {
  using Cfg = ConvCfg<BN>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t *bars = reinterpret_cast<uint64_t *>(smem + C_STAGES * Cfg::STAGE_BYTES);
  uint64_t *full = bars;                  // used in the leader only
  uint64_t *empty = bars + C_STAGES;      // both CTAs
  uint64_t *tfull = bars + 2 * C_STAGES;  // both CTAs
  uint64_t *tempty = tfull + 2;           // leader only, 8 arrivals
  uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(tempty + 2);
  volatile int *abort_flag = reinterpret_cast<volatile int *>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();  // 0 = leader
  const int pair = blockIdx.x >> 1;
  const int num_pairs = gridDim.x >> 1;
  const int total_tiles = P.tiles_m * P.tiles_n;
  const int KB = P.taps * (P.Cin / C_BK);

  if (threadIdx.x == 0) {
    for (int s = 0; s < C_STAGES; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(&tfull[a], 1);
      mbar_init(&tempty[a], 8);
    }
    *abort_flag = 0;
    mbar_fence_init();
  }
  if (warp == 1) tmem_alloc_pair(tmem_slot, Cfg::TMEM_COLS);
  tc_fence_before_sync();
  __syncthreads();
  cluster_sync_all();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;
  pdl_launch_dependents();
  pdl_wait();

  auto fail = [&](int code) {
    *abort_flag = 1;
    atomicCAS(P.err, 0, code);
  };

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer (both CTAs)
    if (lane == 0) {
      tma_prefetch_desc(&P.tmA);
      tma_prefetch_desc(&P.tmB);
      const int cb = P.Cin / C_BK;
      const int bw = 1 << P.bw_log2, bh = C_BM >> P.bw_log2;
      uint32_t kiter = 0;
      bool ok = true;
      for (int tile = pair; ok && tile < total_tiles; tile += num_pairs) {
        const int patch = (tile % P.tiles_m) * 2 + static_cast<int>(rank);
        const int n0 = (tile / P.tiles_m) * BN;
        // first pixel of this CTA's patch (3x3) or first row (plain GEMM)
        const int tx = patch % P.tiles_x, ty = (patch / P.tiles_x) % P.tiles_y, img = patch / (P.tiles_x * P.tiles_y);
        for (int kb = 0; kb < KB; ++kb, ++kiter) {
          const int s = kiter % C_STAGES;
          const uint32_t ph = (kiter / C_STAGES) & 1;
          if (!mbar_wait(&empty[s], ph ^ 1, abort_flag)) {
            fail(KERR_WAIT_EMPTY);
            ok = false;
            break;
          }
          uint8_t *sa = smem + s * Cfg::STAGE_BYTES;
          uint8_t *sb = sa + Cfg::A_BYTES;
          const uint32_t full_leader = map_to_cta(smem_u32(&full[s]), 0);
          if (rank == 0) mbar_arrive_expect_tx(&full[s], 2 * Cfg::STAGE_BYTES);
          if (P.taps == 9) {
            const int tap = kb / cb, c0 = (kb - tap * cb) * C_BK;
            const int ky = tap / 3, kx = tap - 3 * ky;
            if (P.stride2)
              tma_load_4d_pair(sa, &P.tmA, full_leader, c0, tx * bw + (kx >> 1), ty * bh + (ky >> 1),
                               img * 4 + (ky & 1) * 2 + (kx & 1));
            else
              tma_load_4d_pair(sa, &P.tmA, full_leader, c0, tx * bw + kx - 1, ty * bh + ky - 1, img);
          } else {
            tma_load_2d_pair(sa, &P.tmA, full_leader, kb * C_BK, patch * C_BM);
          }
          tma_load_2d_pair(sb, &P.tmB, full_leader, kb * C_BK, n0 + static_cast<int>(rank) * (BN / 2));
        }
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer (leader CTA only)
    // the whole warp runs the loop, one elected lane issues (see gemm2_tcgen05.cu): descriptors stay warp-uniform
    if (rank == 0) {
      const bool leader = elect_one();
      constexpr uint32_t idesc_bf16 = make_idesc_16(2 * C_BM, BN, FMT_BF16, FMT_BF16, 0, 0);
      constexpr uint32_t idesc_f16 = make_idesc_16(2 * C_BM, BN, FMT_F16, FMT_F16, 0, 0);
      const uint32_t idesc = P.x_f16 ? idesc_f16 : idesc_bf16;
      const uint32_t smem_base = smem_u32(smem);
      uint32_t kiter = 0, it = 0;
      bool ok = true;
      for (int tile = pair; ok && tile < total_tiles; tile += num_pairs, ++it) {
        const int acc = it & 1;
        if (!mbar_wait_warp(&tempty[acc], ((it >> 1) & 1) ^ 1, abort_flag)) {
          if (lane == 0) fail(KERR_WAIT_TMEM_EMPTY);
          break;
        }
        tc_fence_after_sync();
        const uint32_t d = tmem_base + acc * BN;
        for (int kb = 0; kb < KB; ++kb, ++kiter) {
          const int s = kiter % C_STAGES;
          const uint32_t ph = (kiter / C_STAGES) & 1;
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
            for (int k = 0; k < C_BK / 16; ++k) tc_mma_ss_pair(d, ad + 2 * k, bd + 2 * k, idesc, (kb | k) ? 1u : 0u);
            tc_commit_pair(&empty[s], 3);
          }
        }
        if (ok && leader) tc_commit_pair(&tfull[acc], 3);
      }
    }
    __syncwarp();
  } else {
    // ------------------------------------------------------------------ epilogue (warps 2..5 of both CTAs)
    const int q = warp & 3;
    const int r = q * 32 + lane;  // row of the CTA's patch = TMEM lane
    uint32_t it = 0;
    for (int tile = pair; tile < total_tiles; tile += num_pairs, ++it) {
      const int patch = (tile % P.tiles_m) * 2 + static_cast<int>(rank);
      const int n0 = (tile / P.tiles_m) * BN;
      size_t row;
      bool row_ok;
      if (P.taps == 9) {
        const int tx = patch % P.tiles_x, ty = (patch / P.tiles_x) % P.tiles_y, img = patch / (P.tiles_x * P.tiles_y);
        const int x = (tx << P.bw_log2) + (r & ((1 << P.bw_log2) - 1));
        const int y = ty * (C_BM >> P.bw_log2) + (r >> P.bw_log2);
        row_ok = x < P.W && y < P.H && img < P.n_img;
        row = (static_cast<size_t>(img) * P.H + y) * P.W + x;
      } else {
        row = static_cast<size_t>(patch) * C_BM + r;
        row_ok = row < static_cast<size_t>(P.M);
      }
      const int acc = it & 1;
      const bool ok = mbar_wait_warp(&tfull[acc], (it >> 1) & 1, abort_flag);
      if (!ok) {
        if (lane == 0) fail(KERR_WAIT_TMEM_FULL);
        break;
      }
      tc_fence_after_sync();
      const uint32_t taddr = tmem_base + acc * BN + (static_cast<uint32_t>(q * 32) << 16);
      conv_epilogue<BN>(P, row, row_ok, n0, taddr, (static_cast<size_t>(tile % P.tiles_m) * 2 + rank) * 4 + q);
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster(map_to_cta(smem_u32(&tempty[acc]), 0));
    }
  }

  // ------------------------------------------------------------------ teardown
  if (*abort_flag) {
    const long long t0 = clock64();
    while (clock64() - t0 < 2000000LL) __nanosleep(1000);
  }
  tc_fence_before_sync();
  __syncthreads();
  cluster_sync_all();
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc_pair(tmem_base, Cfg::TMEM_COLS);
  }
}

// One block per group: folds the epilogue warps' partial sums in a fixed order (per thread ascending, then a fixed
// shared-memory tree in double precision).
__global__ void __launch_bounds__(256) conv_gn_finalize_kernel(const float *__restrict__ partial, int tiles_m,
                                                               int cpg, long long pixels, float eps,
                                                               float *__restrict__ stats) {
  __shared__ double sa[256], sb[256];
  pdl_launch_dependents();
  pdl_wait();
  const int g = blockIdx.x;
  const long long slots = static_cast<long long>(tiles_m) * 8;  // (row tile, cta, warp) of the tiles covering this group
  const float *ps = partial + static_cast<size_t>(g) * 2 * slots, *pq = ps + slots;
  double a = 0.0, b = 0.0;
  for (long long e = threadIdx.x; e < slots; e += 256) {
    a += static_cast<double>(__ldcg(ps + e));
    b += static_cast<double>(__ldcg(pq + e));
  }
  sa[threadIdx.x] = a;
  sb[threadIdx.x] = b;
  __syncthreads();
  for (int o = 128; o > 0; o >>= 1) {
    if (threadIdx.x < o) {
      sa[threadIdx.x] += sa[threadIdx.x + o];
      sb[threadIdx.x] += sb[threadIdx.x + o];
    }
    __syncthreads();
  }
  if (threadIdx.x == 0) {
    const double n = static_cast<double>(pixels) * cpg;
    const double mean = sa[0] / n;
    double var = sb[0] / n - mean * mean;
    if (var < 0.0) var = 0.0;
    stats[2 * g] = static_cast<float>(mean);
    stats[2 * g + 1] = static_cast<float>(1.0 / sqrt(var + static_cast<double>(eps)));
  }
}

int conv_gn_finalize(const ConvParams &p, long long pixels, float eps, float *stats, cudaStream_t stream) {
  if (!p.gn_partial || (p.gn_cpg != 4 && p.gn_cpg != 8 && p.gn_cpg != 16) || p.Cout != 32 * p.gn_cpg) return -5;
  return launch_kernel(conv_gn_finalize_kernel, dim3(32), dim3(256), 0, stream, 1,
                       static_cast<const float *>(p.gn_partial), p.tiles_m, p.gn_cpg, pixels, eps, stats) ==
                 cudaSuccess
             ? 0
             : -8;
}

// ---------------------------------------------------------------------------------------------- host
static PFN_cuTensorMapEncodeTiled_v12000 g_conv_encode = nullptr;

int conv_init() {
  if (!g_conv_encode) {
    void *fn = nullptr;
    cudaDriverEntryPointQueryResult qres;
    cudaError_t e = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &qres);
    if (e != cudaSuccess || qres != cudaDriverEntryPointSuccess || !fn) return -1;
    g_conv_encode = reinterpret_cast<PFN_cuTensorMapEncodeTiled_v12000>(fn);
  }
  cudaError_t e1 = cudaFuncSetAttribute(conv2_tn_kernel<256>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                        ConvCfg<256>::SMEM);
  cudaError_t e2 = cudaFuncSetAttribute(conv2_tn_kernel<128>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                        ConvCfg<128>::SMEM);
  return (e1 == cudaSuccess && e2 == cudaSuccess) ? 0 : -2;
}

static int pick_bn(int Cout) { return Cout % 256 == 0 ? 256 : (Cout % 128 == 0 ? 128 : 0); }

static void finish_tiles(ConvParams *p) {
  p->tiles_m = (p->patches + 1) / 2;
  p->tiles_n = p->Cout / p->bn;
}

static int conv_make_3x3_impl(ConvParams *p, const void *x, int n_img, int H, int W, int Cin, const void *w, int Cout,
                              int planes_per_img);

int conv_make_3x3(ConvParams *p, const void *x, int n_img, int H, int W, int Cin, const void *w, int Cout) {
  return conv_make_3x3_impl(p, x, n_img, H, W, Cin, w, Cout, 1);
}

int conv_make_3x3_s2(ConvParams *p, const void *planes, int n_img, int Ho, int Wo, int Cin, const void *w, int Cout) {
  int rc = conv_make_3x3_impl(p, planes, n_img, Ho, Wo, Cin, w, Cout, 4);
  if (!rc) p->stride2 = 1;
  return rc;
}

static int conv_make_3x3_impl(ConvParams *p, const void *x, int n_img, int H, int W, int Cin, const void *w, int Cout,
                              int planes_per_img) {
  if (!g_conv_encode && conv_init() != 0) return -1;
  const int bn = pick_bn(Cout);
  if (n_img < 1 || H < 1 || W < 1 || Cin < 64 || (Cin % 64) || !bn) return -5;
  if ((reinterpret_cast<uintptr_t>(x) & 15) || (reinterpret_cast<uintptr_t>(w) & 15)) return -3;
  int bl = 7;  // patch width: the largest power of two <= min(W, 128), so that narrow images do not waste rows
  while (bl > 0 && (1 << bl) > W) --bl;
  const int bw = 1 << bl, bh = C_BM >> bl;
  cuuint64_t dims[4] = {static_cast<cuuint64_t>(Cin), static_cast<cuuint64_t>(W), static_cast<cuuint64_t>(H),
                        static_cast<cuuint64_t>(n_img) * planes_per_img};
  cuuint64_t strides[3] = {static_cast<cuuint64_t>(Cin) * 2, static_cast<cuuint64_t>(W) * Cin * 2,
                           static_cast<cuuint64_t>(H) * W * Cin * 2};
  cuuint32_t box[4] = {C_BK, static_cast<cuuint32_t>(bw), static_cast<cuuint32_t>(bh), 1};
  cuuint32_t estr[4] = {1, 1, 1, 1};
  CUresult r = g_conv_encode(&p->tmA, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, const_cast<void *>(x), dims, strides, box, estr,
                             CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                             CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return -4;
  int rc = make_tmap_2d_bf16(&p->tmB, w, Cout, 9ull * Cin, 9ull * Cin, bn / 2, C_BK);
  if (rc) return rc;
  p->taps = 9;
  p->stride2 = 0;
  p->n_img = n_img;
  p->H = H;
  p->W = W;
  p->bw_log2 = bl;
  p->tiles_x = (W + bw - 1) / bw;
  p->tiles_y = (H + bh - 1) / bh;
  p->M = n_img * H * W;
  p->Cin = Cin;
  p->Cout = Cout;
  p->bn = bn;
  p->patches = n_img * p->tiles_x * p->tiles_y;
  finish_tiles(p);
  return 0;
}

int conv_make_gemm(ConvParams *p, const void *X, long long ldx, const void *Wt, long long ldw, int M, int N, int K,
                   int w_rows) {
  if (!g_conv_encode && conv_init() != 0) return -1;
  const int bn = pick_bn(N);
  if (M < 1 || K < 64 || (K % 64) || !bn || ldx < K || ldw < K || w_rows < 1 || w_rows > N) return -5;
  int rc = make_tmap_2d_bf16(&p->tmA, X, M, K, ldx, C_BM, C_BK);
  if (rc) return rc;
  rc = make_tmap_2d_bf16(&p->tmB, Wt, w_rows, K, ldw, bn / 2, C_BK);
  if (rc) return rc;
  p->taps = 1;
  p->n_img = 1;
  p->H = p->W = 1;
  p->bw_log2 = 7;
  p->tiles_x = p->tiles_y = 1;
  p->M = M;
  p->Cin = K;
  p->Cout = N;
  p->bn = bn;
  p->patches = (M + C_BM - 1) / C_BM;
  // tiles_x * tiles_y = 1, so patch -> (0, 0, patch): only the row arithmetic of the GEMM branch is used
  finish_tiles(p);
  return 0;
}

int conv_launch(ConvParams *p, int num_sms, cudaStream_t stream) {
  const int total = p->tiles_m * p->tiles_n;
  if (total < 1 || !p->out || !p->err) return -5;
  if (p->mode == CONV_STORE_RGB8 && p->tiles_n != 1) return -6;
  if (p->gn_partial && (p->mode == CONV_STORE_RGB8 || p->Cout != 32 * p->gn_cpg ||
                        (p->gn_cpg != 4 && p->gn_cpg != 8 && p->gn_cpg != 16)))
    return -7;
  int pairs = num_sms / 2;
  if (total < pairs) pairs = total;
  cudaError_t e = p->bn == 256 ? launch_kernel(conv2_tn_kernel<256>, dim3(2 * pairs), dim3(C_THREADS), ConvCfg<256>::SMEM,
                                               stream, 2, *p)
                               : launch_kernel(conv2_tn_kernel<128>, dim3(2 * pairs), dim3(C_THREADS), ConvCfg<128>::SMEM,
                                               stream, 2, *p);
  return e == cudaSuccess ? 0 : -8;
}

}  // namespace fx
