// Launchers of the memory-bound kernels (elementwise.cu). All return 0 on success and are asynchronous.
#pragma once
#include <cuda_runtime.h>

namespace fx {

static constexpr int GEMV_S = 4;  // timesteps handled per pass over the modulation weights

int elementwise_init();
// Rows row0 .. row0+rows-1 of x/out ([*, hidden]); a row whose position (row % seq) is below n_txt uses the
// text stream's (shift, scale), the others the image stream's.
// f16 != 0: 16-bit outputs of these launchers are f16 (saturating) instead of bf16.
// sat (may be null): device counter that receives one count per thread that clamped a value to the f16 range.
int launch_adaln(const float *x, void *out_16, int row0, int rows, int hidden, int seq, int n_txt, int f16,
                 const float *shift_txt, const float *scale_txt, const float *shift_img, const float *scale_img,
                 cudaStream_t st, int *sat = nullptr);
int launch_qk_norm_rope(void *qkv_bf16, long long ld, int q_col, int k_col, int seq, int batch, int heads, int n_txt,
                        const float *wq_txt, const float *wk_txt, const float *wq_img, const float *wk_img,
                        const float *cos_t, const float *sin_t, cudaStream_t st);
int launch_timestep_sincos(const float *t, int S, int dim, float *out, cudaStream_t st);
int launch_gemv_multi(const void *W_16, const float *x, float *y, int R, int K, int silu_out, int w_f16,
                      cudaStream_t st);
int launch_pack_tokens(const float *z, void *tok_16, int C, int n, int f16, cudaStream_t st, int *sat = nullptr);
int launch_f32_to_bf16(const float *in, void *out_16, long long n, int f16, cudaStream_t st, int *sat = nullptr);
// In place, n 16-bit elements: bf16 -> f16 (to_f16 != 0; round to nearest even, saturating at +-65504) or f16 -> bf16.
// The load-time format conversion of the weights, done on the device so that the host never walks over them.
int launch_convert16_inplace(void *p, long long n, int to_f16, cudaStream_t st);
// to_packed != 0: packed[B, C p p, H/p, W/p] = patchify(plain[B, C, H, W]); else the inverse.
int launch_patchify(float *packed, float *plain, int batch, int C, int H, int W, int p, int to_packed, cudaStream_t st);
// ang[i] = atan2(sin_t[2 i], cos_t[2 i]) for i < pairs
int launch_rope_angles(const float *cos_t, const float *sin_t, float *ang, long long pairs, cudaStream_t st);
int launch_euler(float *z, const float *v, const float *sched, int step, long long n, cudaStream_t st);
int launch_scale_copy(float *dst, const float *src, float a, long long n, cudaStream_t st);
int launch_cfg_euler(float *z, const float *v_cond, const float *v_uncond, float *v_out, float g, const float *sched,
                     int step, long long n, int apply_update, cudaStream_t st);

}  // namespace fx
