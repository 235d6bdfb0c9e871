// Memory-bound kernels of the denoising step: AdaLN (K3), timestep/modulation projections (K4),
// QK-RMSNorm + 2-axis RoPE (K5), sampler updates (K6), layout/dtype changes at the edges (K7).
// All are bandwidth-bound: 128-bit accesses, warp-shuffle reductions, f32 statistics.
#include "elementwise.cuh"
#include "launch.cuh"
#include "ptx.cuh"

#include <cuda_fp16.h>

namespace fx {

// ------------------------------------------------------------------------------------------------
// K3  AdaLN:  out_bf16[r, :] = (1 + scale) * LayerNorm(x_f32[r, :]) + shift      (no affine, eps 1e-6,
// biased variance, two-pass like the reference: flux_transformer.c:1021-1046). One warp per row; the
// row stays in registers between the passes (VPL float4 per lane), so HBM sees one read and one write.
// Four rows per 128-thread block, three blocks per SM: the 1536-row launches of a 512x512 step fit in one wave.
// ------------------------------------------------------------------------------------------------
template <int VPL>
__global__ void __launch_bounds__(128, 3) adaln_kernel(const float *__restrict__ x, __nv_bfloat16 *__restrict__ out,
                                                    int row0, int rows, int hidden, int seq, int n_txt, int f16,
                                                    const float *__restrict__ shift_txt,
                                                    const float *__restrict__ scale_txt,
                                                    const float *__restrict__ shift_img,
                                                    const float *__restrict__ scale_img, int *sat) {
  pdl_launch_dependents();
  pdl_wait();
  const int local = blockIdx.x * 4 + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (local >= rows) return;
  const int row = row0 + local;
#ifdef FLUX_CUDA_DEBUG
  if (row < 0 || seq <= 0 || hidden != VPL * 128 || ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(out)) & 15)) {
    if (sat != nullptr && lane == 0) atomicCAS(sat - 1, 0, KERR_BAD_INDEX);  // checked build: record and skip
    return;
  }
#endif
  const bool is_txt = (row % seq) < n_txt;  // position inside the [txt ; img ; refs] sequence picks the stream
  const float *shift = is_txt ? shift_txt : shift_img;
  const float *scale = is_txt ? scale_txt : scale_img;
  const float4 *xr = reinterpret_cast<const float4 *>(x + static_cast<size_t>(row) * hidden);
  float4 v[VPL];
  float s = 0.f;
#pragma unroll
  for (int i = 0; i < VPL; ++i) {
    v[i] = xr[i * 32 + lane];
    s += (v[i].x + v[i].y) + (v[i].z + v[i].w);
  }
  const float mean = warp_sum(s) / static_cast<float>(hidden);
  float q = 0.f;
#pragma unroll
  for (int i = 0; i < VPL; ++i) {
    const float a = v[i].x - mean, b = v[i].y - mean, c = v[i].z - mean, d = v[i].w - mean;
    q += (a * a + b * b) + (c * c + d * d);
  }
  const float rstd = rsqrtf(warp_sum(q) / static_cast<float>(hidden) + 1e-6f);
  const float4 *sh4 = reinterpret_cast<const float4 *>(shift);
  const float4 *sc4 = reinterpret_cast<const float4 *>(scale);
  uint2 *o2 = reinterpret_cast<uint2 *>(out + static_cast<size_t>(row) * hidden);
  float mx = 0.f;
#pragma unroll
  for (int i = 0; i < VPL; ++i) {
    const float4 sh = __ldg(sh4 + i * 32 + lane);
    const float4 sc = __ldg(sc4 + i * 32 + lane);
    const float a = fmaf((v[i].x - mean) * rstd, 1.f + sc.x, sh.x);
    const float b = fmaf((v[i].y - mean) * rstd, 1.f + sc.y, sh.y);
    const float c = fmaf((v[i].z - mean) * rstd, 1.f + sc.z, sh.z);
    const float d = fmaf((v[i].w - mean) * rstd, 1.f + sc.w, sh.w);
    o2[i * 32 + lane] = make_uint2(pack_16x2_t(a, b, f16 != 0, mx), pack_16x2_t(c, d, f16 != 0, mx));
  }
  sat_report(sat, f16 != 0, mx);
}

int launch_adaln(const float *x, void *out, int row0, int rows, int hidden, int seq, int n_txt, int f16,
                 const float *shift_txt, const float *scale_txt, const float *shift_img, const float *scale_img,
                 cudaStream_t st, int *sat) {
  if (rows <= 0) return 0;
  const int grid = (rows + 3) / 4;
  __nv_bfloat16 *o = reinterpret_cast<__nv_bfloat16 *>(out);
#define FX_ADALN(V)                                                                                             \
  launch_kernel(adaln_kernel<V>, dim3(grid), dim3(128), 0, st, 1, x, o, row0, rows, hidden, seq, n_txt, f16, \
                shift_txt, scale_txt, shift_img, scale_img, sat)
  switch (hidden) {
    case 3072: FX_ADALN(24); break;
    case 256: FX_ADALN(2); break;
    case 512: FX_ADALN(4); break;
    case 1024: FX_ADALN(8); break;
    default: return -1;
  }
#undef FX_ADALN
  return cudaGetLastError() == cudaSuccess ? 0 : -8;
}

// ------------------------------------------------------------------------------------------------
// K5  per-head RMSNorm of Q and K followed by the consecutive-pair rotation (apply_qk_norm,
// flux_transformer.c:1083-1101; apply_rope_2d, 719-741), in place on the bf16 projection output.
// One warp per (token, head, q|k): lane l owns elements 4l..4l+3 = two rotation pairs. Rows below
// `n_txt` use the text stream's norm weights (double-stream blocks), the others the image stream's;
// cos/sin come from one table over the whole [txt ; img ; refs] sequence.
// ------------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(256) qk_norm_rope_kernel(__nv_bfloat16 *__restrict__ qkv, long long ld, int q_col,
                                                           int k_col, int seq, int batch, int heads, int n_txt,
                                                           const float *__restrict__ wq_txt,
                                                           const float *__restrict__ wk_txt,
                                                           const float *__restrict__ wq_img,
                                                           const float *__restrict__ wk_img,
                                                           const float *__restrict__ cos_t,
                                                           const float *__restrict__ sin_t) {
  const long long gw = static_cast<long long>(blockIdx.x) * 8 + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  const long long total = static_cast<long long>(batch) * seq * heads * 2;
  if (gw >= total) return;
  const int which = static_cast<int>(gw & 1);  // 0 = Q, 1 = K
  const int head = static_cast<int>((gw >> 1) % heads);
  const long long tok = (gw >> 1) / heads;  // batch * seq + position
  const int pos = static_cast<int>(tok % seq);
  __nv_bfloat16 *p = qkv + tok * ld + (which ? k_col : q_col) + head * 128 + lane * 4;
  const uint2 raw = *reinterpret_cast<const uint2 *>(p);
  float x0 = bf16_lo(raw.x), x1 = bf16_hi(raw.x), x2 = bf16_lo(raw.y), x3 = bf16_hi(raw.y);
  const float ss = warp_sum((x0 * x0 + x1 * x1) + (x2 * x2 + x3 * x3));
  const float rinv = rsqrtf(ss * (1.0f / 128.0f) + 1e-6f);
  const float *w = (pos < n_txt) ? (which ? wk_txt : wq_txt) : (which ? wk_img : wq_img);
  const float4 w4 = __ldg(reinterpret_cast<const float4 *>(w) + lane);
  x0 *= rinv * w4.x;
  x1 *= rinv * w4.y;
  x2 *= rinv * w4.z;
  x3 *= rinv * w4.w;
  const float4 c4 = __ldg(reinterpret_cast<const float4 *>(cos_t + static_cast<size_t>(pos) * 128) + lane);
  const float4 s4 = __ldg(reinterpret_cast<const float4 *>(sin_t + static_cast<size_t>(pos) * 128) + lane);
  const float y0 = x0 * c4.x - x1 * s4.x;
  const float y1 = x1 * c4.x + x0 * s4.x;
  const float y2 = x2 * c4.z - x3 * s4.z;
  const float y3 = x3 * c4.z + x2 * s4.z;
  *reinterpret_cast<uint2 *>(p) = make_uint2(pack_bf16x2(y0, y1), pack_bf16x2(y2, y3));
}

int launch_qk_norm_rope(void *qkv, long long ld, int q_col, int k_col, int seq, int batch, int heads, int n_txt,
                        const float *wq_txt, const float *wk_txt, const float *wq_img, const float *wk_img,
                        const float *cos_t, const float *sin_t, cudaStream_t st) {
  const long long total = static_cast<long long>(batch) * seq * heads * 2;
  if (total <= 0) return 0;
  const unsigned grid = static_cast<unsigned>((total + 7) / 8);
  qk_norm_rope_kernel<<<grid, 256, 0, st>>>(reinterpret_cast<__nv_bfloat16 *>(qkv), ld, q_col, k_col, seq, batch,
                                            heads, n_txt, wq_txt, wk_txt, wq_img, wk_img, cos_t, sin_t);
  return cudaGetLastError() == cudaSuccess ? 0 : -8;
}

// ------------------------------------------------------------------------------------------------
// K4  timestep embedding and modulation projections for up to GEMV_S timesteps at once
// (get_timestep_embedding + time_embed_forward, flux_transformer.c:940-969; modulation projections,
// 3226-3234, 3016-3024, 3523-3534). The schedule is known before the loop starts, so the weights
// (341 MB in bf16 for klein-4B) are streamed once per group of GEMV_S steps instead of once per step
// (and instead of once per single-stream block, as the reference does).
//   y[s, r] = act( sum_k W_bf16[r, k] * x_f32[s, k] ),   one warp per output row r.
// ------------------------------------------------------------------------------------------------
__global__ void timestep_sincos_kernel(const float *__restrict__ t, int S, int dim, float *__restrict__ out) {
  const int s = blockIdx.x;
  const int half = dim / 2;
  const float log_max = logf(10000.0f);
  for (int i = threadIdx.x; i < half; i += blockDim.x) {
    const float freq = expf(-log_max * static_cast<float>(i) / static_cast<float>(half));
    const float ang = t[s] * 1000.0f * freq;
    out[static_cast<size_t>(s) * dim + i] = cosf(ang);
    out[static_cast<size_t>(s) * dim + i + half] = sinf(ang);
  }
  (void)S;
}

// Four output rows per warp: the S x 8 activations a lane needs for its slice of K are read from shared memory ONCE
// and applied to four rows' weights, whose 16-byte loads are all in flight together - a quarter of the shared-memory
// traffic per weight byte of a one-row-per-warp kernel (which ran at 19 % of the HBM rate on the 320 MB modulation
// matrix) and four times the memory-level parallelism.
static constexpr int GEMV_ROWS = 4;

template <int S>
__global__ void __launch_bounds__(256) gemv_multi_kernel(const __nv_bfloat16 *__restrict__ W,
                                                         const float *__restrict__ x, float *__restrict__ y, int R,
                                                         int K, int silu_out, int f16) {
  extern __shared__ float xs[];  // [S, K]
  for (int i = threadIdx.x; i < S * K / 4; i += blockDim.x)
    reinterpret_cast<float4 *>(xs)[i] = reinterpret_cast<const float4 *>(x)[i];
  __syncthreads();
  const int lane = threadIdx.x & 31;
  // Persistent blocks: x is staged once per block, then the block walks over groups of 8 * GEMV_ROWS rows.
  for (int r0 = (blockIdx.x * 8 + (threadIdx.x >> 5)) * GEMV_ROWS; r0 < R; r0 += gridDim.x * 8 * GEMV_ROWS) {
  const uint4 *wr[GEMV_ROWS];
#pragma unroll
  for (int q = 0; q < GEMV_ROWS; ++q) {
    const int r = r0 + q < R ? r0 + q : R - 1;  // rows past the end repeat the last one; their results are dropped
    wr[q] = reinterpret_cast<const uint4 *>(W + static_cast<size_t>(r) * K);
  }
  float acc[GEMV_ROWS][S];
#pragma unroll
  for (int q = 0; q < GEMV_ROWS; ++q)
#pragma unroll
    for (int s = 0; s < S; ++s) acc[q][s] = 0.f;
  for (int i = lane; i < K / 8; i += 32) {
    uint4 w[GEMV_ROWS];
#pragma unroll
    for (int q = 0; q < GEMV_ROWS; ++q) w[q] = __ldg(wr[q] + i);
    float4 xa[S], xb[S];
#pragma unroll
    for (int s = 0; s < S; ++s) {
      xa[s] = *reinterpret_cast<const float4 *>(xs + s * K + i * 8);
      xb[s] = *reinterpret_cast<const float4 *>(xs + s * K + i * 8 + 4);
    }
#pragma unroll
    for (int q = 0; q < GEMV_ROWS; ++q) {
      float wf[8];
      if (f16) {
        const float2 a = __half22float2(*reinterpret_cast<const __half2 *>(&w[q].x));
        const float2 b = __half22float2(*reinterpret_cast<const __half2 *>(&w[q].y));
        const float2 c = __half22float2(*reinterpret_cast<const __half2 *>(&w[q].z));
        const float2 d = __half22float2(*reinterpret_cast<const __half2 *>(&w[q].w));
        wf[0] = a.x, wf[1] = a.y, wf[2] = b.x, wf[3] = b.y, wf[4] = c.x, wf[5] = c.y, wf[6] = d.x, wf[7] = d.y;
      } else {
        wf[0] = bf16_lo(w[q].x), wf[1] = bf16_hi(w[q].x), wf[2] = bf16_lo(w[q].y), wf[3] = bf16_hi(w[q].y);
        wf[4] = bf16_lo(w[q].z), wf[5] = bf16_hi(w[q].z), wf[6] = bf16_lo(w[q].w), wf[7] = bf16_hi(w[q].w);
      }
#pragma unroll
      for (int s = 0; s < S; ++s)
        acc[q][s] += (wf[0] * xa[s].x + wf[1] * xa[s].y) + (wf[2] * xa[s].z + wf[3] * xa[s].w) +
                     (wf[4] * xb[s].x + wf[5] * xb[s].y) + (wf[6] * xb[s].z + wf[7] * xb[s].w);
    }
  }
#pragma unroll
  for (int q = 0; q < GEMV_ROWS; ++q)
#pragma unroll
    for (int s = 0; s < S; ++s) {
      float v = warp_sum(acc[q][s]);
      if (silu_out) v = v / (1.0f + expf(-v));
      if (lane == 0 && r0 + q < R) y[static_cast<size_t>(s) * R + r0 + q] = v;
    }
  }
}

int launch_timestep_sincos(const float *t, int S, int dim, float *out, cudaStream_t st) {
  timestep_sincos_kernel<<<S, 128, 0, st>>>(t, S, dim, out);
  return cudaGetLastError() == cudaSuccess ? 0 : -8;
}

int elementwise_init() {
  cudaError_t e = cudaFuncSetAttribute(gemv_multi_kernel<GEMV_S>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                       GEMV_S * 12288 * 4);
  return e == cudaSuccess ? 0 : -2;
}

// x [S, K] f32 (S <= GEMV_S; unused rows are read as zero padding by the caller's buffer), y [S, R] f32.
int launch_gemv_multi(const void *W, const float *x, float *y, int R, int K, int silu_out, int f16, cudaStream_t st) {
  if (K % 8 || K > 12288) return -1;
  const size_t smem = static_cast<size_t>(GEMV_S) * K * 4;
  int dev = 0, sms = 148;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  const int groups = (R + 8 * GEMV_ROWS - 1) / (8 * GEMV_ROWS);
  const int grid = groups < 2 * sms ? groups : 2 * sms;  // two blocks per SM (registers), each staging x once
  gemv_multi_kernel<GEMV_S><<<grid, 256, smem, st>>>(reinterpret_cast<const __nv_bfloat16 *>(W), x, y, R, K,
                                                             silu_out, f16);
  return cudaGetLastError() == cudaSuccess ? 0 : -8;
}

// ------------------------------------------------------------------------------------------------
// K7  edges: channel-major f32 latents -> token-major bf16 (the NCHW -> NLC transpose of
// flux_transformer.c:3156-3161 / 3650-3664 fused with the cast), and f32 -> bf16 for the context.
// ------------------------------------------------------------------------------------------------
__global__ void pack_tokens_kernel(const float *__restrict__ z, uint16_t *__restrict__ tok, int C, int n, int f16,
                                   int *sat) {
  __shared__ float tile[32][33];
  pdl_launch_dependents();
  pdl_wait();
  const int p0 = blockIdx.x * 32, c0 = blockIdx.y * 32;
  const int tx = threadIdx.x, ty = threadIdx.y;  // 32 x 8
  for (int i = ty; i < 32; i += 8) {
    const int c = c0 + i, p = p0 + tx;
    tile[i][tx] = (c < C && p < n) ? z[static_cast<size_t>(c) * n + p] : 0.f;
  }
  __syncthreads();
  for (int i = ty; i < 32; i += 8) {
    const int p = p0 + i, c = c0 + tx;
    if (p < n && c < C) {
      const float v = tile[tx][i];
      tok[static_cast<size_t>(p) * C + c] = static_cast<uint16_t>(pack_16x2(v, 0.f, f16 != 0) & 0xFFFFu);
      sat_report(sat, f16 != 0, fabsf(v));
    }
  }
}

int launch_pack_tokens(const float *z, void *tok, int C, int n, int f16, cudaStream_t st, int *sat) {
  dim3 grid((n + 31) / 32, (C + 31) / 32);
  return launch_kernel(pack_tokens_kernel, grid, dim3(32, 8), 0, st, 1, z, reinterpret_cast<uint16_t *>(tok), C, n,
                       f16, sat) == cudaSuccess
             ? 0
             : -8;
}

__global__ void f32_to_bf16_kernel(const float4 *__restrict__ in, uint2 *__restrict__ out, long long n4, int f16,
                                   int *sat) {
  float mx = 0.f;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < n4;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const float4 v = in[i];
    out[i] = make_uint2(pack_16x2_t(v.x, v.y, f16 != 0, mx), pack_16x2_t(v.z, v.w, f16 != 0, mx));
  }
  sat_report(sat, f16 != 0, mx);
}

int launch_f32_to_bf16(const float *in, void *out, long long n, int f16, cudaStream_t st, int *sat) {
  if (n % 4) return -1;
  const long long n4 = n / 4;
  const int grid = static_cast<int>((n4 + 255) / 256 < 148 * 8 ? (n4 + 255) / 256 : 148 * 8);
  f32_to_bf16_kernel<<<grid, 256, 0, st>>>(reinterpret_cast<const float4 *>(in), reinterpret_cast<uint2 *>(out), n4,
                                           f16, sat);
  return cudaGetLastError() == cudaSuccess ? 0 : -8;
}

// ------------------------------------------------------------------------------------------------
// K7b  patchify / unpatchify: space-to-depth of p x p pixel blocks, [B, C, H, W] <-> [B, C p p, H/p, W/p] with the
// new channel index c p p + pi p + pj (flux_patchify / flux_unpatchify, flux_kernels.c:1038-1094). This is the
// layout change between VAE latents (32 channels) and the DiT's 128-channel latents. One thread per element of
// the PACKED tensor, so the packed side is read or written fully coalesced.
// ------------------------------------------------------------------------------------------------
__global__ void patchify_kernel(float *__restrict__ packed, float *__restrict__ plain, int C, int H, int W, int p,
                                long long total, int to_packed) {
  const int oh = H / p, ow = W / p;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const int pw = static_cast<int>(i % ow);
    long long r = i / ow;
    const int ph = static_cast<int>(r % oh);
    r /= oh;
    const int oc = static_cast<int>(r % (C * p * p));
    const long long b = r / (C * p * p);
    const int c = oc / (p * p), pi = (oc / p) % p, pj = oc % p;
    const long long j = ((b * C + c) * H + (ph * p + pi)) * W + (pw * p + pj);
    if (to_packed) packed[i] = plain[j];
    else plain[j] = packed[i];
  }
}

int launch_patchify(float *packed, float *plain, int batch, int C, int H, int W, int p, int to_packed, cudaStream_t st) {
  if (p <= 0 || H % p || W % p) return -1;
  const long long total = static_cast<long long>(batch) * C * H * W;
  if (total <= 0) return 0;
  long long blocks = (total + 255) / 256;
  if (blocks > 148 * 16) blocks = 148 * 16;
  patchify_kernel<<<static_cast<int>(blocks), 256, 0, st>>>(packed, plain, C, H, W, p, total, to_packed);
  return cudaGetLastError() == cudaSuccess ? 0 : -8;
}

// ------------------------------------------------------------------------------------------------
// K6  sampler updates: Euler  z += dt * v  (flux_axpy, flux_kernels.c:126-130; flux_sample.c:248) and
// the classifier-free-guidance combine  v = v_u + g (v_c - v_u); z += dt * v  (flux_sample.c:495-499).
// dt is read from the device-resident schedule so that a captured launch works for every step.
// ------------------------------------------------------------------------------------------------
__global__ void euler_kernel(float *__restrict__ z, const float *__restrict__ v, const float *__restrict__ sched,
                             int step, long long n) {
  pdl_launch_dependents();
  pdl_wait();
  const float dt = sched[step + 1] - sched[step];
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < n;
       i += static_cast<long long>(gridDim.x) * blockDim.x)
    z[i] = fmaf(dt, v[i], z[i]);
}

__global__ void cfg_euler_kernel(float *__restrict__ z, const float *__restrict__ v_cond,
                                 const float *__restrict__ v_uncond, float *__restrict__ v_out, float g,
                                 const float *__restrict__ sched, int step, long long n, int apply_update) {
  const float dt = sched[step + 1] - sched[step];
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < n;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const float vu = v_uncond[i];
    const float v = vu + g * (v_cond[i] - vu);
    if (v_out) v_out[i] = v;
    if (apply_update) z[i] = fmaf(dt, v, z[i]);
  }
}

__global__ void scale_copy_kernel(float *__restrict__ dst, const float *__restrict__ src, float a, long long n) {
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < n;
       i += static_cast<long long>(gridDim.x) * blockDim.x)
    dst[i] = a * src[i];
}

static int ew_grid(long long n) {
  long long b = (n + 255) / 256;
  return static_cast<int>(b < 148 * 4 ? (b > 0 ? b : 1) : 148 * 4);
}

int launch_euler(float *z, const float *v, const float *sched, int step, long long n, cudaStream_t st) {
  return launch_kernel(euler_kernel, dim3(ew_grid(n)), dim3(256), 0, st, 1, z, v, sched, step, n) == cudaSuccess ? 0
                                                                                                                   : -8;
}

int launch_scale_copy(float *dst, const float *src, float a, long long n, cudaStream_t st) {
  scale_copy_kernel<<<ew_grid(n), 256, 0, st>>>(dst, src, a, n);
  return cudaGetLastError() == cudaSuccess ? 0 : -8;
}

int launch_cfg_euler(float *z, const float *v_cond, const float *v_uncond, float *v_out, float g, const float *sched,
                     int step, long long n, int apply_update, cudaStream_t st) {
  cfg_euler_kernel<<<ew_grid(n), 256, 0, st>>>(z, v_cond, v_uncond, v_out, g, sched, step, n, apply_update);
  return cudaGetLastError() == cudaSuccess ? 0 : -8;
}

// Rotation angle of every consecutive pair from cos / sin tables that hold each value twice ([seq, 128] ->
// [seq, 64], in [-pi, pi]): the form the fused projection epilogue reads (gemm.cuh, QkvNormRope::ang).
__global__ void rope_angles_kernel(const float *__restrict__ cos_t, const float *__restrict__ sin_t,
                                   float *__restrict__ ang, long long pairs) {
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < pairs;
       i += static_cast<long long>(gridDim.x) * blockDim.x)
    ang[i] = atan2f(sin_t[2 * i], cos_t[2 * i]);
}

int launch_rope_angles(const float *cos_t, const float *sin_t, float *ang, long long pairs, cudaStream_t st) {
  if (pairs <= 0) return 0;
  rope_angles_kernel<<<ew_grid(pairs), 256, 0, st>>>(cos_t, sin_t, ang, pairs);
  return cudaGetLastError() == cudaSuccess ? 0 : -8;
}

// ------------------------------------------------------------------------------------------------ 16-bit formats
__device__ __forceinline__ uint32_t cvt16_pair(uint32_t u, bool to_f16) {
  if (to_f16) {
    const float lo = __uint_as_float(u << 16), hi = __uint_as_float(u & 0xFFFF0000u);
    return pack_f16x2(lo, hi);
  }
  const float lo = __half2float(__ushort_as_half(static_cast<unsigned short>(u & 0xFFFFu)));
  const float hi = __half2float(__ushort_as_half(static_cast<unsigned short>(u >> 16)));
  return pack_bf16x2(lo, hi);
}

__global__ void __launch_bounds__(256) convert16_kernel(uint16_t *__restrict__ p, long long n, int to_f16) {
  const long long n8 = n >> 3;
  uint4 *p4 = reinterpret_cast<uint4 *>(p);
  for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < n8;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    uint4 v = p4[i];
    v.x = cvt16_pair(v.x, to_f16 != 0);
    v.y = cvt16_pair(v.y, to_f16 != 0);
    v.z = cvt16_pair(v.z, to_f16 != 0);
    v.w = cvt16_pair(v.w, to_f16 != 0);
    p4[i] = v;
  }
  if (blockIdx.x == 0 && threadIdx.x == 0)
    for (long long i = n8 << 3; i < n; ++i) {  // at most seven trailing elements
      const uint32_t r = cvt16_pair(static_cast<uint32_t>(p[i]), to_f16 != 0);
      p[i] = static_cast<uint16_t>(r & 0xFFFFu);
    }
}

int launch_convert16_inplace(void *p, long long n, int to_f16, cudaStream_t st) {
  if (n <= 0) return 0;
  if (reinterpret_cast<uintptr_t>(p) & 15) return -1;
  long long nb = ((n >> 3) + 255) / 256;
  if (nb < 1) nb = 1;
  if (nb > 148 * 8) nb = 148 * 8;
  convert16_kernel<<<static_cast<unsigned>(nb), 256, 0, st>>>(reinterpret_cast<uint16_t *>(p), n, to_f16);
  return cudaGetLastError() == cudaSuccess ? 0 : -8;
}

}  // namespace fx
