// The VAE's memory-bound kernels: latent de-normalisation + depth-to-space + 1x1 convolution, GroupNorm(32)
// (statistics, then normalise + swish), nearest 2x upsampling, row softmax and a 16-bit transpose for the single
// attention block. Channels-last throughout, 16-byte vector accesses, two-stage deterministic reductions.
#include <cuda_fp16.h>

#include "launch.cuh"
#include "ptx.cuh"
#include "vae_kernels.cuh"

namespace fx {

__device__ __forceinline__ float half_bits_to_f32(uint16_t v, bool f16) {
  return f16 ? __half2float(__ushort_as_half(v)) : __uint_as_float(static_cast<uint32_t>(v) << 16);
}
__device__ __forceinline__ void unpack_16x2(uint32_t u, bool f16, float &lo, float &hi) {
  lo = half_bits_to_f32(static_cast<uint16_t>(u & 0xFFFFu), f16);
  hi = half_bits_to_f32(static_cast<uint16_t>(u >> 16), f16);
}

// ------------------------------------------------------------------------------------------------ prologue
__global__ void __launch_bounds__(128) vae_prologue_kernel(const float *__restrict__ latent, uint16_t *__restrict__ out,
                                                           int n_img, int h, int w, const float *__restrict__ bn_mean,
                                                           const float *__restrict__ bn_var, float eps,
                                                           const float *__restrict__ wq, const float *__restrict__ bq,
                                                           int f16) {
  __shared__ float sw[32 * 33];
  __shared__ float sb[32], sstd[128], smean[128];
  pdl_launch_dependents();
  pdl_wait();
  for (int i = threadIdx.x; i < 1024; i += blockDim.x) sw[(i >> 5) * 33 + (i & 31)] = wq[i];
  if (threadIdx.x < 32) sb[threadIdx.x] = bq ? bq[threadIdx.x] : 0.f;
  for (int i = threadIdx.x; i < 128; i += blockDim.x) {
    sstd[i] = sqrtf(bn_var[i] + eps);
    smean[i] = bn_mean[i];
  }
  __syncthreads();
  const int H = 2 * h, W = 2 * w;
  const long long total = static_cast<long long>(n_img) * H * W;
  const long long p = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (p >= total) return;
  const int X = static_cast<int>(p % W), Y = static_cast<int>((p / W) % H), img = static_cast<int>(p / (static_cast<long long>(W) * H));
  const int x = X >> 1, pj = X & 1, y = Y >> 1, pi = Y & 1;
  float in[32];
#pragma unroll
  for (int c = 0; c < 32; ++c) {
    const int lc = c * 4 + pi * 2 + pj;  // channel of the packed latent that holds (c, pi, pj)
    in[c] = latent[((static_cast<size_t>(img) * 128 + lc) * h + y) * w + x] * sstd[lc] + smean[lc];
  }
  uint32_t o[32];
#pragma unroll 4
  for (int co = 0; co < 32; co += 2) {
    float a0 = sb[co], a1 = sb[co + 1];
#pragma unroll
    for (int ci = 0; ci < 32; ++ci) {
      a0 = fmaf(sw[co * 33 + ci], in[ci], a0);
      a1 = fmaf(sw[(co + 1) * 33 + ci], in[ci], a1);
    }
    o[co >> 1] = pack_16x2(a0, a1, f16 != 0);
  }
  uint4 *dst = reinterpret_cast<uint4 *>(out + static_cast<size_t>(p) * 64);
#pragma unroll
  for (int j = 0; j < 4; ++j) dst[j] = make_uint4(o[4 * j], o[4 * j + 1], o[4 * j + 2], o[4 * j + 3]);
#pragma unroll
  for (int j = 4; j < 8; ++j) dst[j] = make_uint4(0u, 0u, 0u, 0u);
}

int launch_vae_prologue(const float *latent, void *out16, int n_img, int h, int w, const float *bn_mean,
                        const float *bn_var, float eps, const float *wq, const float *bq, int f16, cudaStream_t st) {
  const long long total = static_cast<long long>(n_img) * 4 * h * w;
  const dim3 grid(static_cast<unsigned>((total + 127) / 128)), block(128);
  return launch_kernel(vae_prologue_kernel, grid, block, 0, st, 1, latent, reinterpret_cast<uint16_t *>(out16), n_img, h,
                       w, bn_mean, bn_var, eps, wq, bq, f16) == cudaSuccess
             ? 0
             : -8;
}

// ------------------------------------------------------------------------------------------------ GroupNorm
// A thread owns 4 consecutive channels (one group or part of one: channels per group is 4, 8 or 16) and walks
// over pixels; per block the 256 partial (sum, sum of squares) pairs are folded per group in a fixed order, and
// the last block of an image to finish folds the blocks' partials, again in a fixed order, in double precision.
template <bool IN16>
__global__ void __launch_bounds__(256) gn_stats_kernel(const void *__restrict__ xv, int f16, long long pixels, int C,
                                                       float eps, float *__restrict__ partial,
                                                       unsigned int *__restrict__ counters, float *__restrict__ stats) {
  __shared__ float ps[256], pss[256];
  __shared__ bool last;
  pdl_launch_dependents();
  pdl_wait();
  const int img = blockIdx.y, nblk = gridDim.x;
  const int quads = C >> 2;              // threads per pixel
  const int lanes = 256 / quads;         // pixels per block iteration
  const int qd = threadIdx.x % quads, pl = threadIdx.x / quads;
  const size_t base = static_cast<size_t>(img) * pixels * C;
  float s = 0.f, ss = 0.f;
  auto load4 = [&](long long p) {
    float4 v;
    if (IN16) {
      const uint2 u = *reinterpret_cast<const uint2 *>(reinterpret_cast<const uint16_t *>(xv) + base + p * C + qd * 4);
      unpack_16x2(u.x, f16 != 0, v.x, v.y);
      unpack_16x2(u.y, f16 != 0, v.z, v.w);
    } else {
      v = *reinterpret_cast<const float4 *>(reinterpret_cast<const float *>(xv) + base + p * C + qd * 4);
    }
    return v;
  };
  auto add4 = [&](const float4 &v) {
    s += (v.x + v.y) + (v.z + v.w);
    ss += (v.x * v.x + v.y * v.y) + (v.z * v.z + v.w * v.w);
  };
  const long long stride = static_cast<long long>(nblk) * lanes;
  long long p = static_cast<long long>(blockIdx.x) * lanes + pl;
  for (; p + 3 * stride < pixels; p += 4 * stride) {  // four independent loads in flight per thread
    const float4 a = load4(p), b = load4(p + stride), c = load4(p + 2 * stride), d = load4(p + 3 * stride);
    add4(a);
    add4(b);
    add4(c);
    add4(d);
  }
  for (; p < pixels; p += stride) add4(load4(p));
  ps[threadIdx.x] = s;
  pss[threadIdx.x] = ss;
  __syncthreads();
  const int cpg = C / GN_GROUPS, qpg = cpg >> 2;  // quads per group: 1, 2 or 4
  float *mine = partial + (static_cast<size_t>(img) * GN_MAX_BLOCKS + blockIdx.x) * 64;
  if (threadIdx.x < GN_GROUPS) {
    const int g = threadIdx.x;
    float a = 0.f, b = 0.f;
    for (int l = 0; l < lanes; ++l)
      for (int k = 0; k < qpg; ++k) {
        a += ps[l * quads + g * qpg + k];
        b += pss[l * quads + g * qpg + k];
      }
    mine[2 * g] = a;
    mine[2 * g + 1] = b;
  }
  __threadfence();
  __syncthreads();
  if (threadIdx.x == 0) last = atomicAdd(&counters[img], 1u) == static_cast<unsigned>(nblk - 1);
  __syncthreads();
  if (!last) return;
  __threadfence();
  {
    // eight threads per group, each over every eighth block in ascending order, then a fixed-order shuffle fold
    const int g = threadIdx.x >> 3, sub = threadIdx.x & 7;
    double a = 0.0, b = 0.0;
    const float *pp = partial + static_cast<size_t>(img) * GN_MAX_BLOCKS * 64;
    for (int k = sub; k < nblk; k += 8) {
      a += static_cast<double>(__ldcg(pp + k * 64 + 2 * g));
      b += static_cast<double>(__ldcg(pp + k * 64 + 2 * g + 1));
    }
#pragma unroll
    for (int o = 4; o > 0; o >>= 1) {
      a += __shfl_xor_sync(0xffffffffu, a, o);
      b += __shfl_xor_sync(0xffffffffu, b, o);
    }
    if (sub == 0) {
      const double n = static_cast<double>(pixels) * cpg;
      const double mean = a / n;
      double var = b / n - mean * mean;
      if (var < 0.0) var = 0.0;
      stats[(img * GN_GROUPS + g) * 2] = static_cast<float>(mean);
      stats[(img * GN_GROUPS + g) * 2 + 1] = static_cast<float>(1.0 / sqrt(var + static_cast<double>(eps)));
    }
  }
  if (threadIdx.x == 0) counters[img] = 0;
}

int launch_gn_stats(const void *x, int in16, int f16, int n_img, long long pixels, int C, float eps, float *partial,
                    unsigned int *counters, float *stats, cudaStream_t st) {
  if (C % 128 || C > 1024 || 256 % (C >> 2) || pixels < 1) return -1;
  const int lanes = 256 / (C >> 2);
  long long nb = (pixels + lanes - 1) / lanes;
  const long long cap = n_img > 1 ? 296 : 592;  // four resident blocks per SM for one image
  if (nb > cap) nb = cap;
  if (nb > GN_MAX_BLOCKS) nb = GN_MAX_BLOCKS;
  const dim3 grid(static_cast<unsigned>(nb), n_img), block(256);
  cudaError_t e = in16 ? launch_kernel(gn_stats_kernel<true>, grid, block, 0, st, 1, x, f16, pixels, C, eps, partial,
                                       counters, stats)
                       : launch_kernel(gn_stats_kernel<false>, grid, block, 0, st, 1, x, f16, pixels, C, eps, partial,
                                       counters, stats);
  return e == cudaSuccess ? 0 : -8;
}

template <bool IN16>
__global__ void __launch_bounds__(256) gn_apply_kernel(const void *__restrict__ xv, uint16_t *__restrict__ out, int f16,
                                                       long long pixels, int C, const float *__restrict__ stats,
                                                       const float *__restrict__ gamma, const float *__restrict__ beta,
                                                       int swish, long long total8) {
  pdl_launch_dependents();
  pdl_wait();
  const int img = blockIdx.y;
  const int cpg = C / GN_GROUPS;
  const size_t base = static_cast<size_t>(img) * pixels * C;
  const float *st = stats + img * GN_GROUPS * 2;
  const unsigned cmask = static_cast<unsigned>(C) - 1u;  // C is a power of two (128 .. 1024)
  const int gshift = __ffs(cpg) - 1;
  for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < total8;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const size_t e = static_cast<size_t>(i) * 8;  // element offset inside the image
    const int c = static_cast<int>(static_cast<unsigned>(e) & cmask);
    float v[8];
    if (IN16) {
      const uint4 u = *reinterpret_cast<const uint4 *>(reinterpret_cast<const uint16_t *>(xv) + base + e);
      unpack_16x2(u.x, f16 != 0, v[0], v[1]);
      unpack_16x2(u.y, f16 != 0, v[2], v[3]);
      unpack_16x2(u.z, f16 != 0, v[4], v[5]);
      unpack_16x2(u.w, f16 != 0, v[6], v[7]);
    } else {
      const float4 a = *reinterpret_cast<const float4 *>(reinterpret_cast<const float *>(xv) + base + e);
      const float4 b = *reinterpret_cast<const float4 *>(reinterpret_cast<const float *>(xv) + base + e + 4);
      v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w;
      v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
    }
    const float4 g0 = __ldg(reinterpret_cast<const float4 *>(gamma + c)), g1 = __ldg(reinterpret_cast<const float4 *>(gamma + c + 4));
    const float4 b0 = __ldg(reinterpret_cast<const float4 *>(beta + c)), b1 = __ldg(reinterpret_cast<const float4 *>(beta + c + 4));
    const float gm[8] = {g0.x, g0.y, g0.z, g0.w, g1.x, g1.y, g1.z, g1.w};
    const float bt[8] = {b0.x, b0.y, b0.z, b0.w, b1.x, b1.y, b1.z, b1.w};
    const int ga = c >> gshift, gb = (c + 4) >> gshift;  // the two halves may sit in different groups when cpg == 4
    const float ma = __ldg(st + 2 * ga), ra = __ldg(st + 2 * ga + 1), mb = __ldg(st + 2 * gb), rb = __ldg(st + 2 * gb + 1);
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      float y = (v[j] - (j < 4 ? ma : mb)) * (j < 4 ? ra : rb) * gm[j] + bt[j];
      if (swish) y = __fdividef(y, 1.0f + __expf(-y));
      v[j] = y;
    }
    *reinterpret_cast<uint4 *>(out + base + e) =
        make_uint4(pack_16x2(v[0], v[1], f16 != 0), pack_16x2(v[2], v[3], f16 != 0), pack_16x2(v[4], v[5], f16 != 0),
                   pack_16x2(v[6], v[7], f16 != 0));
  }
}

int launch_gn_apply(const void *x, int in16, void *out16, int f16, int n_img, long long pixels, int C,
                    const float *stats, const float *gamma, const float *beta, int swish, cudaStream_t st) {
  if (C < 128 || C > 1024 || (C & (C - 1))) return -1;
  const long long total8 = pixels * C / 8;
  long long nb = (total8 + 255) / 256;
  if (nb > 148 * 8) nb = 148 * 8;
  const dim3 grid(static_cast<unsigned>(nb), n_img), block(256);
  uint16_t *o = reinterpret_cast<uint16_t *>(out16);
  cudaError_t e = in16 ? launch_kernel(gn_apply_kernel<true>, grid, block, 0, st, 1, x, o, f16, pixels, C, stats, gamma,
                                       beta, swish, total8)
                       : launch_kernel(gn_apply_kernel<false>, grid, block, 0, st, 1, x, o, f16, pixels, C, stats, gamma,
                                       beta, swish, total8);
  return e == cudaSuccess ? 0 : -8;
}

// ------------------------------------------------------------------------------------------------ upsample
__global__ void __launch_bounds__(256) upsample2x_kernel(const float *__restrict__ x, uint16_t *__restrict__ out, int f16,
                                                         int H, int W, int C, long long total8) {
  pdl_launch_dependents();
  pdl_wait();
  const int c8 = C >> 3;
  for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < total8;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const int cc = static_cast<int>(i % c8);
    const long long op = i / c8;  // output pixel over all images
    const int ox = static_cast<int>(op % (2 * W)), oy = static_cast<int>((op / (2 * W)) % (2 * H));
    const long long img = op / (4LL * W * H);
    const float *src = x + ((img * H + (oy >> 1)) * W + (ox >> 1)) * C + cc * 8;
    const float4 a = *reinterpret_cast<const float4 *>(src), b = *reinterpret_cast<const float4 *>(src + 4);
    *reinterpret_cast<uint4 *>(out + op * C + cc * 8) =
        make_uint4(pack_16x2(a.x, a.y, f16 != 0), pack_16x2(a.z, a.w, f16 != 0), pack_16x2(b.x, b.y, f16 != 0),
                   pack_16x2(b.z, b.w, f16 != 0));
  }
}

int launch_upsample2x(const float *x, void *out16, int f16, int n_img, int H, int W, int C, cudaStream_t st) {
  if (C % 8) return -1;
  const long long total8 = static_cast<long long>(n_img) * 4 * H * W * (C / 8);
  long long nb = (total8 + 255) / 256;
  if (nb > 148 * 8) nb = 148 * 8;
  return launch_kernel(upsample2x_kernel, dim3(static_cast<unsigned>(nb)), dim3(256), 0, st, 1, x,
                       reinterpret_cast<uint16_t *>(out16), f16, H, W, C, total8) == cudaSuccess
             ? 0
             : -8;
}

// ------------------------------------------------------------------------------------------------ encoder edges
__global__ void __launch_bounds__(256) parity_planes_kernel(const float *__restrict__ x, uint16_t *__restrict__ out,
                                                            int f16, int H, int W, int C, long long total8) {
  pdl_launch_dependents();
  pdl_wait();
  const int c8 = C >> 3, Ho = H >> 1, Wo = W >> 1;
  for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < total8;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const int cc = static_cast<int>(i % c8);
    const long long ip = i / c8;  // input pixel over all images
    const int ix = static_cast<int>(ip % W), iy = static_cast<int>((ip / W) % H);
    const long long img = ip / (static_cast<long long>(W) * H);
    const float *src = x + ip * C + cc * 8;
    const float4 a = *reinterpret_cast<const float4 *>(src), b = *reinterpret_cast<const float4 *>(src + 4);
    const long long plane = img * 4 + (iy & 1) * 2 + (ix & 1);
    uint16_t *dst = out + ((plane * Ho + (iy >> 1)) * Wo + (ix >> 1)) * C + cc * 8;
    *reinterpret_cast<uint4 *>(dst) = make_uint4(pack_16x2(a.x, a.y, f16 != 0), pack_16x2(a.z, a.w, f16 != 0),
                                                 pack_16x2(b.x, b.y, f16 != 0), pack_16x2(b.z, b.w, f16 != 0));
  }
}

int launch_parity_planes(const float *x, void *out16, int f16, int n_img, int H, int W, int C, cudaStream_t st) {
  if (C % 8 || (H & 1) || (W & 1)) return -1;
  const long long total8 = static_cast<long long>(n_img) * H * W * (C / 8);
  long long nb = (total8 + 255) / 256;
  if (nb > 148 * 8) nb = 148 * 8;
  return launch_kernel(parity_planes_kernel, dim3(static_cast<unsigned>(nb)), dim3(256), 0, st, 1, x,
                       reinterpret_cast<uint16_t *>(out16), f16, H, W, C, total8) == cudaSuccess
             ? 0
             : -8;
}

__global__ void __launch_bounds__(256) image_to_nhwc_kernel(const float *__restrict__ img, uint16_t *__restrict__ out,
                                                            int f16, long long pixels) {
  pdl_launch_dependents();
  pdl_wait();
  for (long long p = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; p < pixels;
       p += static_cast<long long>(gridDim.x) * blockDim.x) {
    const float r = img[p], g = img[pixels + p], b = img[2 * pixels + p];
    uint4 *dst = reinterpret_cast<uint4 *>(out + p * 64);
    dst[0] = make_uint4(pack_16x2(r, g, f16 != 0), pack_16x2(b, 0.f, f16 != 0), 0u, 0u);
#pragma unroll
    for (int j = 1; j < 8; ++j) dst[j] = make_uint4(0u, 0u, 0u, 0u);
  }
}

int launch_image_to_nhwc(const float *img, void *out16, int f16, int H, int W, cudaStream_t st) {
  const long long pixels = static_cast<long long>(H) * W;
  long long nb = (pixels + 255) / 256;
  if (nb > 148 * 8) nb = 148 * 8;
  return launch_kernel(image_to_nhwc_kernel, dim3(static_cast<unsigned>(nb)), dim3(256), 0, st, 1, img,
                       reinterpret_cast<uint16_t *>(out16), f16, pixels) == cudaSuccess
             ? 0
             : -8;
}

// one warp per latent-resolution pixel: lane = output channel of the mean half
__global__ void __launch_bounds__(128) vae_encode_tail_kernel(const float *__restrict__ y, int ld, float *__restrict__ latent,
                                                              int Hl, int Wl, const float *__restrict__ wq,
                                                              const float *__restrict__ bq, const float *__restrict__ bn_mean,
                                                              const float *__restrict__ bn_var, float eps) {
  pdl_launch_dependents();
  pdl_wait();
  const int lane = threadIdx.x & 31;
  const long long pix = static_cast<long long>(blockIdx.x) * 4 + (threadIdx.x >> 5);
  if (pix >= static_cast<long long>(Hl) * Wl) return;
  const float *row = y + pix * ld;
  const float v0 = row[lane], v1 = row[lane + 32];
  float acc = bq ? bq[lane] : 0.f;
  const float *wr = wq + lane * 64;
#pragma unroll 8
  for (int k = 0; k < 32; ++k) {
    acc = fmaf(wr[k], __shfl_sync(0xffffffffu, v0, k), acc);
    acc = fmaf(wr[k + 32], __shfl_sync(0xffffffffu, v1, k), acc);
  }
  const int Y = static_cast<int>(pix / Wl), X = static_cast<int>(pix % Wl);
  const int lc = lane * 4 + (Y & 1) * 2 + (X & 1);  // channel of the packed latent (flux_patchify, p = 2)
  const int h = Hl >> 1, w = Wl >> 1;
  latent[(static_cast<size_t>(lc) * h + (Y >> 1)) * w + (X >> 1)] = (acc - bn_mean[lc]) / sqrtf(bn_var[lc] + eps);
}

int launch_vae_encode_tail(const float *y, int ld, float *latent, int Hl, int Wl, const float *wq, const float *bq,
                           const float *bn_mean, const float *bn_var, float eps, cudaStream_t st) {
  if ((Hl & 1) || (Wl & 1) || ld < 64) return -1;
  const long long pixels = static_cast<long long>(Hl) * Wl;
  return launch_kernel(vae_encode_tail_kernel, dim3(static_cast<unsigned>((pixels + 3) / 4)), dim3(128), 0, st, 1, y, ld,
                       latent, Hl, Wl, wq, bq, bn_mean, bn_var, eps) == cudaSuccess
             ? 0
             : -8;
}

// ------------------------------------------------------------------------------------------------ softmax
__device__ __forceinline__ float block_reduce(float v, bool is_max, float *sm) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float t = __shfl_xor_sync(0xffffffffu, v, o);
    v = is_max ? fmaxf(v, t) : v + t;
  }
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  __syncthreads();
  if (lane == 0) sm[warp] = v;
  __syncthreads();
  v = sm[0];
  for (int i = 1; i < static_cast<int>(blockDim.x >> 5); ++i) v = is_max ? fmaxf(v, sm[i]) : v + sm[i];
  return v;
}

__global__ void __launch_bounds__(256) softmax_rows_kernel(const float *__restrict__ s, uint16_t *__restrict__ out,
                                                           int f16, int cols, int ld, float scale) {
  __shared__ float sm[8];
  pdl_launch_dependents();
  pdl_wait();
  const float *row = s + static_cast<size_t>(blockIdx.x) * ld;
  uint16_t *orow = out + static_cast<size_t>(blockIdx.x) * ld;
  const int n4 = cols >> 2;
  float m = -3.0e38f;
  for (int i = threadIdx.x; i < n4; i += blockDim.x) {
    const float4 v = reinterpret_cast<const float4 *>(row)[i];
    m = fmaxf(m, fmaxf(fmaxf(v.x, v.y), fmaxf(v.z, v.w)));
  }
  m = block_reduce(m, true, sm) * scale;
  float sum = 0.f;
  for (int i = threadIdx.x; i < n4; i += blockDim.x) {
    const float4 v = reinterpret_cast<const float4 *>(row)[i];
    sum += (__expf(v.x * scale - m) + __expf(v.y * scale - m)) + (__expf(v.z * scale - m) + __expf(v.w * scale - m));
  }
  sum = block_reduce(sum, false, sm);
  const float inv = 1.0f / sum;
  for (int i = threadIdx.x; i < n4; i += blockDim.x) {
    const float4 v = reinterpret_cast<const float4 *>(row)[i];
    reinterpret_cast<uint2 *>(orow)[i] =
        make_uint2(pack_16x2(__expf(v.x * scale - m) * inv, __expf(v.y * scale - m) * inv, f16 != 0),
                   pack_16x2(__expf(v.z * scale - m) * inv, __expf(v.w * scale - m) * inv, f16 != 0));
  }
  for (int i = n4 + threadIdx.x; i < (ld >> 2); i += blockDim.x) reinterpret_cast<uint2 *>(orow)[i] = make_uint2(0u, 0u);
}

int launch_softmax_rows(const float *s, void *out16, int f16, long long rows, int cols, int ld, float scale,
                        cudaStream_t st) {
  if (cols % 4 || ld % 4 || ld < cols || rows < 1 || scale <= 0.f) return -1;
  return launch_kernel(softmax_rows_kernel, dim3(static_cast<unsigned>(rows)), dim3(256), 0, st, 1, s,
                       reinterpret_cast<uint16_t *>(out16), f16, cols, ld, scale) == cudaSuccess
             ? 0
             : -8;
}

// ------------------------------------------------------------------------------------------------ transpose
__global__ void __launch_bounds__(256) transpose16_kernel(const uint16_t *__restrict__ in, long long ld_in,
                                                          uint16_t *__restrict__ out, long long ld_out, int rows,
                                                          int cols) {
  __shared__ uint16_t t[32][33];
  pdl_launch_dependents();
  pdl_wait();
  const int r0 = blockIdx.y * 32, c0 = blockIdx.x * 32;
  const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
  for (int j = ty; j < 32; j += 8)
    if (r0 + j < rows && c0 + tx < cols) t[j][tx] = in[static_cast<size_t>(r0 + j) * ld_in + c0 + tx];
  __syncthreads();
  for (int j = ty; j < 32; j += 8)
    if (c0 + j < cols && r0 + tx < rows) out[static_cast<size_t>(c0 + j) * ld_out + r0 + tx] = t[tx][j];
}

int launch_transpose16(const void *in16, long long ld_in, void *out16, long long ld_out, int rows, int cols,
                       cudaStream_t st) {
  const dim3 grid((cols + 31) / 32, (rows + 31) / 32), block(256);
  return launch_kernel(transpose16_kernel, grid, block, 0, st, 1, reinterpret_cast<const uint16_t *>(in16), ld_in,
                       reinterpret_cast<uint16_t *>(out16), ld_out, rows, cols) == cudaSuccess
             ? 0
             : -8;
}

// ------------------------------------------------------------------------------------------------ widen
__global__ void __launch_bounds__(256) widen16_kernel(const uint16_t *__restrict__ in, float *__restrict__ out, int f16,
                                                      long long n8) {
  pdl_launch_dependents();
  pdl_wait();
  for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < n8;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const uint4 u = reinterpret_cast<const uint4 *>(in)[i];
    float4 a, b;
    unpack_16x2(u.x, f16 != 0, a.x, a.y);
    unpack_16x2(u.y, f16 != 0, a.z, a.w);
    unpack_16x2(u.z, f16 != 0, b.x, b.y);
    unpack_16x2(u.w, f16 != 0, b.z, b.w);
    reinterpret_cast<float4 *>(out)[2 * i] = a;
    reinterpret_cast<float4 *>(out)[2 * i + 1] = b;
  }
}

int launch_widen16(const void *in16, float *out, int f16, long long n, cudaStream_t st) {
  if (n % 8) return -1;
  long long nb = (n / 8 + 255) / 256;
  if (nb > 148 * 8) nb = 148 * 8;
  return launch_kernel(widen16_kernel, dim3(static_cast<unsigned>(nb)), dim3(256), 0, st, 1,
                       reinterpret_cast<const uint16_t *>(in16), out, f16, n / 8) == cudaSuccess
             ? 0
             : -8;
}

}  // namespace fx
