/*
 * flux_cuda_vae_seam.c - the reference's VAE decoder and encoder, served by the B200 engine.
 *
 * flux_vae.c stays in the build (it owns flux_vae_t, flux_image_to_tensor and the legacy loader); four of its
 * functions are redirected at link time:
 *
 *     -Wl,--wrap=flux_vae_load_safetensors -Wl,--wrap=flux_vae_decode -Wl,--wrap=flux_vae_encode
 *     -Wl,--wrap=flux_vae_free
 *
 * With these flags every call of flux_vae_decode from flux.c (flux.c:480, 569, 659, 846, 1052, 1104, 1226) and from
 * the sampler seam's step-image callback lands in __wrap_flux_vae_decode below, which decodes on the GPU through
 * flux_cuda_vae_decode (flux_cuda.h). The wrapped loader loads the file a second time into the engine (the decoder
 * half, 16-bit, ~100 MB) and remembers which engine decoder belongs to which flux_vae_t.
 *
 * Behaviour kept: flux_image ownership (caller frees with flux_image_free), NULL on failure with the reason on
 * stderr, the progress callback (reported as complete when the image is back), malloc ownership of the latent
 * flux_vae_encode returns. Calls the engine cannot serve (batch != 1, image sides that are not multiples of 16) go to
 * the reference's own code.
 */
#include <stdio.h>
#include <stdlib.h>

#include "flux.h"
#include "flux_cuda.h"
#include "flux_kernels.h"
#include "flux_safetensors.h"

typedef struct flux_vae flux_vae_t;
flux_vae_t *__real_flux_vae_load_safetensors(safetensors_file_t *sf);
flux_image *__real_flux_vae_decode(flux_vae_t *vae, const float *latent, int batch, int latent_h, int latent_w);
float *__real_flux_vae_encode(flux_vae_t *vae, const float *img, int batch, int H, int W, int *out_h, int *out_w);
void __real_flux_vae_free(flux_vae_t *vae);
flux_cuda_ctx *flux_cuda_seam_context(void); /* flux_cuda_seam.c */

#define MAX_VAES 8
static struct {
  flux_vae_t *cpu;
  flux_cuda_vae *gpu;
} g_vaes[MAX_VAES];

static flux_cuda_vae *find_gpu(flux_vae_t *vae) {
  for (int i = 0; i < MAX_VAES; ++i)
    if (g_vaes[i].cpu == vae && vae) return g_vaes[i].gpu;
  return NULL;
}

flux_vae_t *__wrap_flux_vae_load_safetensors(safetensors_file_t *sf) {
  flux_cuda_ctx *ctx = flux_cuda_seam_context();
  if (!ctx || !sf) return NULL;
  flux_vae_t *cpu = __real_flux_vae_load_safetensors(sf);
  if (!cpu) return NULL;
  int slot = -1;
  for (int i = 0; i < MAX_VAES && slot < 0; ++i)
    if (!g_vaes[i].cpu) slot = i;
  flux_cuda_vae *gpu = NULL;
  if (slot < 0 || flux_cuda_vae_load_safetensors(ctx, sf->path, &gpu) != FLUX_CUDA_OK) {
    fprintf(stderr, "flux_cuda: VAE decoder: %s\n", slot < 0 ? "too many VAEs are loaded" : flux_cuda_last_error());
    __real_flux_vae_free(cpu);
    return NULL;
  }
  g_vaes[slot].cpu = cpu;
  g_vaes[slot].gpu = gpu;
  return cpu;
}

flux_image *__wrap_flux_vae_decode(flux_vae_t *vae, const float *latent, int batch, int latent_h, int latent_w) {
  flux_cuda_vae *gpu = find_gpu(vae);
  if (!gpu || batch != 1) return __real_flux_vae_decode(vae, latent, batch, latent_h, latent_w);
  if (!latent || latent_h < 1 || latent_w < 1) return NULL;
  flux_image *img = flux_image_create(latent_w * 16, latent_h * 16, 3);
  if (!img) return NULL;
  if (flux_cuda_vae_decode(gpu, latent, latent_h, latent_w, img->data) != FLUX_CUDA_OK) {
    fprintf(stderr, "flux_vae_decode: %s\n", flux_cuda_last_error());
    flux_image_free(img);
    return NULL;
  }
  if (flux_vae_progress_callback) flux_vae_progress_callback(14, 15); /* 3 mid + 12 up blocks, flux_vae.c:750 */
  return img;
}

float *__wrap_flux_vae_encode(flux_vae_t *vae, const float *img, int batch, int H, int W, int *out_h, int *out_w) {
  flux_cuda_vae *gpu = find_gpu(vae);
  if (!gpu || batch != 1 || !flux_cuda_vae_has_encoder(gpu) || H < 16 || W < 16 || (H % 16) || (W % 16))
    return __real_flux_vae_encode(vae, img, batch, H, W, out_h, out_w);
  if (!img || !out_h || !out_w) return NULL;
  float *latent = (float *)malloc((size_t)128 * (H / 16) * (W / 16) * sizeof(float));
  if (!latent) return NULL;
  if (flux_cuda_vae_encode(gpu, img, H, W, latent) != FLUX_CUDA_OK) {
    fprintf(stderr, "flux_vae_encode: %s\n", flux_cuda_last_error());
    free(latent);
    return NULL;
  }
  *out_h = H / 16;
  *out_w = W / 16;
  if (flux_vae_progress_callback) flux_vae_progress_callback(10, 11); /* 8 down + 3 mid blocks, flux_vae.c:343 */
  return latent;
}

void __wrap_flux_vae_free(flux_vae_t *vae) {
  for (int i = 0; i < MAX_VAES; ++i)
    if (vae && g_vaes[i].cpu == vae) {
      flux_cuda_vae_free(g_vaes[i].gpu);
      g_vaes[i].cpu = NULL;
      g_vaes[i].gpu = NULL;
    }
  __real_flux_vae_free(vae);
}
