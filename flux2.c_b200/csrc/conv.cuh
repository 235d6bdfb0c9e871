// Host-visible description of one launch of the tcgen05 implicit-GEMM convolution kernel (conv_tcgen05.cu):
// a 3x3, stride 1, zero-padded convolution over a channels-last (NHWC) 16-bit activation tensor, or - with
// taps = 1 - a plain GEMM over rows with a bias (1x1 convolutions, attention products). This is the engine's
// replacement for the reference's flux_conv2d call sites in the VAE (flux_vae.c:127-145, flux_kernels.c:342-505).
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace fx {

enum ConvEpi : int {
  CONV_STORE_16 = 0,    // out16[row, col] = acc + bias[col]
  CONV_STORE_F32 = 1,   // out32[row, col] = acc + bias[col]
  CONV_ADD_F32 = 2,     // out32[row, col] += acc + bias[col]   (residual connection of a ResNet block)
  CONV_STORE_RGB8 = 3,  // out8[row * 3 + c] = clamp((acc[c] + bias[c] + 1) * 127.5, 0, 255) truncated, c < 3
                        // (flux_vae.c:822-833: the decoder's last convolution and its conversion to an image)
};

struct alignas(64) ConvParams {
  CUtensorMap tmA;  // taps == 9: {C, W, H, N} channels-last, box {64, BW, BH, 1}; taps == 1: [M, K], box {64, 128}
  CUtensorMap tmB;  // weights [Cout, taps * Cin] (tap-major, input channel minor), box {64, BN / 2}
  int taps;         // 9 or 1
  int stride2;      // taps == 9 only: the input is stored as four parity planes (see conv_make_3x3_s2)
  int n_img, H, W;  // taps == 9
  int bw_log2;      // a CTA's 128 rows are a patch of 2^bw_log2 columns x (128 >> bw_log2) rows of pixels
  int tiles_x, tiles_y;
  int M;            // rows = pixels of all images
  int Cin, Cout;    // Cin % 64 == 0 (pad with zero channels), Cout % bn == 0
  int bn;           // 128 or 256 output columns per tile
  int patches, tiles_m, tiles_n;
  int x_f16;        // operands hold f16 instead of bf16
  int mode, out_f16;
  void *out;
  long long ld;       // destination row pitch in elements
  const float *bias;  // [Cout] or null
  // Optional GroupNorm statistics of the tensor being written (modes 0-2; Cout = 32 groups of gn_cpg channels, gn_cpg
  // 4, 8 or 16): every epilogue warp stores the sums and sums of squares of its 32 rows, per group, at
  // gn_partial[(group * 2 + {0: sum, 1: sum of squares}) * slots + slot], slot = (row tile * 2 + cta) * 4 + warp,
  // slots = tiles_m * 8; conv_gn_finalize folds them. No atomics: the result does not depend on scheduling.
  float *gn_partial;
  int gn_cpg;
  int *err;
};
// Floats of gn_partial a launch of `p` writes.
inline size_t conv_gn_partial_floats(const ConvParams &p) {
  return static_cast<size_t>(p.tiles_m) * 8 * 2 * 32;
}
// stats[g] = (mean, 1 / sqrt(var + eps)) of group g over `pixels` rows from the partial sums a launch of `p` wrote.
int conv_gn_finalize(const ConvParams &p, long long pixels, float eps, float *stats, cudaStream_t stream);

int conv_init();
// x: [n_img, H, W, Cin] 16-bit; w: [Cout, 9 * Cin] 16-bit.
int conv_make_3x3(ConvParams *p, const void *x, int n_img, int H, int W, int Cin, const void *w, int Cout);
// 3x3 convolution with stride 2 over an input padded by one zero row at the bottom and one zero column at the right
// (the VAE encoder's downsampling, flux_vae.c:146-171, 360-372): out[y, x] = sum in[2y + ky, 2x + kx]. The input is
// given as parity planes, planes[(n * 4 + py * 2 + px), y, x, c] = in[n, 2y + py, 2x + px, c], each Ho x Wo pixels,
// so that tap (ky, kx) is a stride-1 read of plane (ky & 1, kx & 1) shifted by (ky >> 1, kx >> 1); the shift past the
// last row / column is the zero padding. Ho, Wo: output size.
int conv_make_3x3_s2(ConvParams *p, const void *planes, int n_img, int Ho, int Wo, int Cin, const void *w, int Cout);
// Y[M, N] = X[M, K] (row pitch ldx) * Wt[N, K]^T (row pitch ldw). Only the first w_rows rows of Wt exist in memory
// (w_rows <= N): the columns of Y beyond them come out as the bias alone.
int conv_make_gemm(ConvParams *p, const void *X, long long ldx, const void *Wt, long long ldw, int M, int N, int K,
                   int w_rows);
// Fill mode / out / ld / bias / out_f16 / x_f16 / err before launching.
int conv_launch(ConvParams *p, int num_sms, cudaStream_t stream);

}  // namespace fx
