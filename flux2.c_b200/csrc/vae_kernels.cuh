// Launchers of the VAE's memory-bound kernels (vae_kernels.cu). Activations are channels-last: [pixels, C].
// All return 0 on success and are asynchronous on `st`. f16 != 0: 16-bit tensors hold f16, else bf16.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

namespace fx {

static constexpr int GN_GROUPS = 32;
static constexpr int GN_MAX_BLOCKS = 640;  // per image; size of the partial-sum scratch is n_img * this * 64 floats

// latent f32 [n_img, 128, h, w] -> per-channel de-normalisation x * sqrt(var + eps) + mean -> 2x2 depth-to-space
// -> 1x1 convolution 32 -> 32 (wq [32, 32] f32, bq [32]) -> out16 [n_img, 2h, 2w, 64], channels 32..63 zero
// (flux_vae.c:717-742: batch de-normalisation, flux_unpatchify, post_quant_conv).
int launch_vae_prologue(const float *latent, void *out16, int n_img, int h, int w, const float *bn_mean,
                        const float *bn_var, float eps, const float *wq, const float *bq, int f16, cudaStream_t st);
// GroupNorm(32) statistics of x ([n_img, pixels, C], f32 if in16 == 0 else 16-bit): stats[n_img, 32, 2] = (mean, rstd).
// partial: scratch of n_img * GN_MAX_BLOCKS * 64 floats; counters: n_img ints, zero before the first use (the kernel
// leaves them zero).
int launch_gn_stats(const void *x, int in16, int f16, int n_img, long long pixels, int C, float eps, float *partial,
                    unsigned int *counters, float *stats, cudaStream_t st);
// out16 = act((x - mean) * rstd * gamma + beta), act = x * sigmoid(x) if swish else identity (flux_kernels.c:511-553,
// flux_vae.c:174-177).
int launch_gn_apply(const void *x, int in16, void *out16, int f16, int n_img, long long pixels, int C,
                    const float *stats, const float *gamma, const float *beta, int swish, cudaStream_t st);
// Nearest-neighbour 2x upsampling, f32 [n_img, H, W, C] -> 16-bit [n_img, 2H, 2W, C] (flux_kernels.c:1017-1036).
int launch_upsample2x(const float *x, void *out16, int f16, int n_img, int H, int W, int C, cudaStream_t st);
// Parity planes for the stride-2 convolution: out16[(n * 4 + py * 2 + px), y, x, c] = x[n, 2y + py, 2x + px, c],
// f32 [n_img, H, W, C] -> 16-bit [4 n_img, H/2, W/2, C]; H and W even.
int launch_parity_planes(const float *x, void *out16, int f16, int n_img, int H, int W, int C, cudaStream_t st);
// Image f32 [3, H, W] (planar, as flux_image_to_tensor produces it) -> 16-bit channels-last [H, W, 64], channels 3..63 zero.
int launch_image_to_nhwc(const float *img, void *out16, int f16, int H, int W, cudaStream_t st);
// The encoder's tail (flux_vae.c:404-437): per latent-resolution pixel the first 32 rows of the 1x1 quant_conv
// (wq [64, 64] f32 row-major, bq [64]; only the mean half of the 64 outputs is used) applied to conv_out's 64
// channels (f32 [pixels, ld]), then 2x2 space-to-depth into [128, Hl/2, Wl/2] and (x - mean) / sqrt(var + eps).
int launch_vae_encode_tail(const float *y, int ld, float *latent, int Hl, int Wl, const float *wq, const float *bq,
                           const float *bn_mean, const float *bn_var, float eps, cudaStream_t st);
// out16[r, 0..cols) = softmax(scale * s[r, 0..cols)), out16[r, cols..ld) = 0; both with row pitch ld (flux_kernels.c:596-628).
int launch_softmax_rows(const float *s, void *out16, int f16, long long rows, int cols, int ld, float scale,
                        cudaStream_t st);
// out16[c, r] = in16[r, c] for r < rows, c < cols (in row pitch ld_in, out row pitch ld_out), 16-bit elements.
int launch_transpose16(const void *in16, long long ld_in, void *out16, long long ld_out, int rows, int cols,
                       cudaStream_t st);
// 16-bit [rows, C] -> f32 [rows, C] (the first residual stream of the decoder).
int launch_widen16(const void *in16, float *out, int f16, long long n, cudaStream_t st);

}  // namespace fx
