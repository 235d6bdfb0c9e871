/*
 * flux_cuda_seam.c - the reference's internal link seam, served by the B200 engine.
 *
 * The reference's flux.c declares its transformer and sampler as `extern` symbols (flux.c:36-119) and
 * flux_sample.c / flux_transformer.c define them. This file defines the same symbols on top of
 * flux_cuda.h, so that building the reference with this file (and libflux_cuda.so) IN PLACE OF
 * flux_transformer.c and flux_sample.c gives the unmodified CLI / library (main.c, flux.c, flux_cli.c,
 * flux_vae.c, flux_kernels.c, ...) a GPU denoising path (flux_cuda_qwen3_seam.c does the same for
 * flux_qwen3.c). It is compiled inside the
 * reference's source tree (it includes the reference's own flux_safetensors.h and flux_kernels.h for the
 * struct layouts and the global callback pointers those files own).
 *
 * Behaviour kept from the reference: argument meaning, malloc ownership of returned buffers (caller
 * frees), NULL on failure, input latent not modified, callback order (step callback before a step,
 * progress callback after it, 5 + 20 + 1 sub-step events per forward, step-image callback after every
 * step but the last), timing globals. Difference: there is no CPU fallback - a CUDA failure returns NULL
 * with the reason on stderr.
 */
#include <math.h>
#include <stdint.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>
#include <sys/time.h>

#include "flux.h"
#include "flux_cuda.h"
#include "flux_kernels.h"
#include "flux_safetensors.h"

typedef struct flux_vae flux_vae_t;
extern flux_image *flux_vae_decode(flux_vae_t *vae, const float *latent, int batch, int latent_h, int latent_w);

typedef struct flux_transformer {
  flux_cuda_model *model;
  safetensors_file_t *owned_sf; /* set by the _mmap loader, which takes ownership of the file */
  flux_cuda_dims dims;
  int grouped;                  /* the replicas belong to the GPU group (FLUX_CUDA_DEVICES=a,b) */
} flux_transformer_t;

typedef struct { /* flux.c:68-72 */
  const float *latent;
  int h, w;
  int t_offset;
} flux_ref_t;

float *flux_linear_schedule(int num_steps);
float *flux_init_noise(int batch, int channels, int h, int w, int64_t seed);
float *flux_transformer_forward(flux_transformer_t *tf, const float *img_latent, int img_h, int img_w,
                                const float *txt_emb, int txt_seq, float timestep);
float *flux_sample_euler(void *transformer, void *text_encoder, float *z, int batch, int channels, int h, int w,
                         const float *text_emb, int text_seq, const float *schedule, int num_steps,
                         void (*progress_callback)(int step, int total));

double flux_timing_transformer_total = 0.0;
double flux_timing_transformer_double = 0.0;
double flux_timing_transformer_single = 0.0;
double flux_timing_transformer_final = 0.0;

void flux_reset_timing(void) {
  flux_timing_transformer_total = flux_timing_transformer_double = 0.0;
  flux_timing_transformer_single = flux_timing_transformer_final = 0.0;
}

static flux_cuda_ctx *g_ctx = NULL;
static flux_cuda_group *g_group = NULL; /* FLUX_CUDA_DEVICES=a,b: guided sampling splits its two passes over a and b */

static double now_ms(void) {
  struct timeval tv;
  gettimeofday(&tv, NULL);
  return tv.tv_sec * 1000.0 + tv.tv_usec / 1000.0;
}

static flux_cuda_ctx *seam_ctx(void) {
  if (!g_ctx) {
    const char *list = getenv("FLUX_CUDA_DEVICES");
    int devs[2], n = 0;
    if (list && sscanf(list, "%d,%d", &devs[0], &devs[1]) == 2) n = 2;
    if (n == 2) {
      if (flux_cuda_group_create(2, devs, &g_group) == FLUX_CUDA_OK) {
        g_ctx = flux_cuda_group_context(g_group, 0);
      } else {
        fprintf(stderr, "flux_cuda: FLUX_CUDA_DEVICES=%s ignored: %s\n", list, flux_cuda_last_error());
        g_group = NULL;
      }
    }
    if (!g_ctx) {
      const char *dev = getenv("FLUX_CUDA_DEVICE");
      if (flux_cuda_ctx_create(dev ? atoi(dev) : 0, &g_ctx) != FLUX_CUDA_OK) {
        fprintf(stderr, "flux_cuda: %s\n", flux_cuda_last_error());
        g_ctx = NULL;
      }
    }
  }
  return g_ctx;
}

/* The seam's one context, for the other seam files (flux_cuda_qwen3_seam.c). */
flux_cuda_ctx *flux_cuda_seam_context(void) { return seam_ctx(); }

/* ------------------------------------------------------------------------------------------ loading */
static flux_transformer_t *load_from(safetensors_file_t *sf) {
  flux_cuda_ctx *ctx = seam_ctx();
  if (!ctx || !sf) return NULL;
  flux_transformer_t *tf = (flux_transformer_t *)calloc(1, sizeof(*tf));
  if (!tf) return NULL;
  /* the file is already open and mapped by the caller: hand the path to the engine's own validating loader */
  int rc;
  if (g_group) { /* one replica per GPU of the pair, loaded concurrently */
    rc = flux_cuda_group_load_safetensors(g_group, sf->path);
    tf->model = rc == FLUX_CUDA_OK ? flux_cuda_group_model(g_group, 0) : NULL;
    tf->grouped = 1;
  } else {
    rc = flux_cuda_model_load_safetensors(ctx, sf->path, &tf->model);
  }
  if (rc != FLUX_CUDA_OK) {
    fprintf(stderr, "flux_cuda: %s\n", flux_cuda_last_error());
    free(tf);
    return NULL;
  }
  flux_cuda_model_dims(tf->model, &tf->dims);
  return tf;
}

flux_transformer_t *flux_transformer_load_safetensors(safetensors_file_t *sf) { return load_from(sf); }

flux_transformer_t *flux_transformer_load_safetensors_mmap(safetensors_file_t *sf) {
  /* 7.75 GB of bf16 weights stay resident in HBM, so "mmap mode" is the same load; the ownership
   * contract is kept: the file now belongs to the transformer and is closed by flux_transformer_free. */
  flux_transformer_t *tf = load_from(sf);
  if (tf) tf->owned_sf = sf;
  return tf;
}

flux_transformer_t *flux_transformer_load(FILE *f) {
  (void)f; /* legacy binary format: declared by flux.c, never called */
  return NULL;
}

void flux_transformer_free(flux_transformer_t *tf) {
  if (!tf) return;
  if (tf->grouped) flux_cuda_group_unload(g_group);
  else flux_cuda_model_free(tf->model);
  if (tf->owned_sf) safetensors_close(tf->owned_sf);
  free(tf);
}

/* ------------------------------------------------------------------------------------------ forward */
static void fire_substeps(const flux_transformer_t *tf) {
  if (!flux_substep_callback) return;
  for (int i = 0; i < tf->dims.n_double; i++) flux_substep_callback(FLUX_SUBSTEP_DOUBLE_BLOCK, i, tf->dims.n_double);
  for (int i = 0; i < tf->dims.n_single; i++) flux_substep_callback(FLUX_SUBSTEP_SINGLE_BLOCK, i, tf->dims.n_single);
  flux_substep_callback(FLUX_SUBSTEP_FINAL_LAYER, 0, 1);
}

float *flux_transformer_forward_with_multi_refs(flux_transformer_t *tf, const float *img_latent, int img_h, int img_w,
                                                const flux_ref_t *refs, int num_refs, const float *txt_emb,
                                                int txt_seq, float timestep) {
  if (!tf || !img_latent || !txt_emb) return NULL;
  if (!refs) num_refs = 0;
  flux_cuda_ref cr[16];
  if (num_refs > 16) return NULL;
  for (int i = 0; i < num_refs; i++) {
    cr[i].latent = refs[i].latent;
    cr[i].h = refs[i].h;
    cr[i].w = refs[i].w;
    cr[i].t_offset = refs[i].t_offset;
  }
  const size_t n = (size_t)tf->dims.latent_ch * img_h * img_w;
  float *out = (float *)malloc(n * sizeof(float));
  if (!out) return NULL;
  const double t0 = now_ms();
  if (flux_cuda_forward(tf->model, img_latent, img_h, img_w, cr, num_refs, txt_emb, txt_seq, timestep, out) !=
      FLUX_CUDA_OK) {
    fprintf(stderr, "flux_cuda: %s\n", flux_cuda_last_error());
    free(out);
    return NULL;
  }
  flux_timing_transformer_total += now_ms() - t0;
  fire_substeps(tf);
  return out;
}

float *flux_transformer_forward(flux_transformer_t *tf, const float *img_latent, int img_h, int img_w,
                                const float *txt_emb, int txt_seq, float timestep) {
  return flux_transformer_forward_with_multi_refs(tf, img_latent, img_h, img_w, NULL, 0, txt_emb, txt_seq, timestep);
}

float *flux_transformer_forward_with_refs(flux_transformer_t *tf, const float *img_latent, int img_h, int img_w,
                                          const float *ref_latent, int ref_h, int ref_w, int t_offset,
                                          const float *txt_emb, int txt_seq, float timestep) {
  flux_ref_t r = {ref_latent, ref_h, ref_w, t_offset};
  return flux_transformer_forward_with_multi_refs(tf, img_latent, img_h, img_w, ref_latent ? &r : NULL,
                                                  ref_latent ? 1 : 0, txt_emb, txt_seq, timestep);
}

/* ------------------------------------------------------------------------------------------ samplers */
/* Adds the last run's device time per block group to the reference's timing globals (only when profiling is on). */
static void add_group_times(flux_cuda_sampler *s) {
  float g[FLUX_CUDA_BLOCK_GROUPS];
  if (!flux_verbose || flux_cuda_sampler_profile_groups(s, g) != FLUX_CUDA_OK) return;
  flux_timing_transformer_double += g[1];
  flux_timing_transformer_single += g[2];
  flux_timing_transformer_final += g[3];
}

/* The engine stores activations as f16 by default; a checkpoint whose activations leave that range is clamped, and
 * says so here instead of silently producing a wrong picture. */
static void warn_if_saturated(void) {
  long long n = 0;
  if (g_ctx && flux_cuda_ctx_saturated_stores(g_ctx, &n, 1) == FLUX_CUDA_OK && n > 0)
    fprintf(stderr,
            "flux_cuda: warning: %lld 16-bit stores were clamped to the f16 range (+-65504); "
            "run with FLUX_CUDA_BF16=1 for this checkpoint\n", n);
}

static float *sample_common(flux_transformer_t *tf, const float *z, int batch, int channels, int h, int w,
                            const flux_ref_t *refs, int num_refs, const float *emb_cond, int seq_cond,
                            const float *emb_uncond, int seq_uncond, float guidance, const float *schedule,
                            int num_steps, void (*progress_callback)(int, int)) {
  if (!tf || !z || !emb_cond || !schedule || num_steps < 1 || batch != 1 || channels != tf->dims.latent_ch ||
      num_refs > 16 || (emb_uncond && seq_uncond != seq_cond))
    return NULL;
  if (!refs) num_refs = 0;
  flux_cuda_ref_shape shapes[16];
  const float *lat[16];
  for (int i = 0; i < num_refs; i++) {
    shapes[i].h = refs[i].h;
    shapes[i].w = refs[i].w;
    shapes[i].t_offset = refs[i].t_offset;
    lat[i] = refs[i].latent;
  }
  const size_t n = (size_t)channels * h * w;
  float *out = (float *)malloc(n * sizeof(float));
  flux_cuda_sampler *s = NULL;
  int rc = out ? FLUX_CUDA_OK : FLUX_CUDA_ERR_NOMEM;
  if (!rc && emb_uncond && tf->grouped && g_group && !flux_verbose &&
      !(flux_step_callback || progress_callback || flux_substep_callback ||
        (flux_step_image_callback && flux_step_image_vae))) {
    /* two GPUs and nobody watching the steps: the conditional pass runs on one, the unconditional pass on the other
     * (the reference runs them one after the other, flux_sample.c:485-499) */
    flux_cuda_ref cr[16];
    for (int i = 0; i < num_refs; i++) {
      cr[i].latent = refs[i].latent;
      cr[i].h = refs[i].h;
      cr[i].w = refs[i].w;
      cr[i].t_offset = refs[i].t_offset;
    }
    flux_cuda_sample_params sp;
    memset(&sp, 0, sizeof(sp));
    sp.h = h;
    sp.w = w;
    sp.num_steps = num_steps;
    sp.schedule = schedule;
    sp.ctx = emb_cond;
    sp.ctx_uncond = emb_uncond;
    sp.txt_seq = seq_cond;
    sp.guidance = guidance;
    sp.refs = cr;
    sp.num_refs = num_refs;
    flux_reset_timing();
    const double t_pair = now_ms();
    rc = flux_cuda_group_sample_cfg_pair(g_group, &sp, z, out);
    flux_timing_transformer_total = now_ms() - t_pair;
    warn_if_saturated();
    if (rc) {
      fprintf(stderr, "flux_cuda: %s\n", flux_cuda_last_error());
      free(out);
      return NULL;
    }
    return out;
  }
  if (!rc) rc = flux_cuda_sampler_create(tf->model, h, w, seq_cond, shapes, num_refs, emb_uncond ? 2 : 1, num_steps, &s);
  if (!rc) rc = flux_cuda_sampler_upload(s, z, emb_cond, emb_uncond, lat);

  flux_reset_timing();
  const double t_start = now_ms();
  const int observed = flux_step_callback || progress_callback || flux_substep_callback ||
                       (flux_step_image_callback && flux_step_image_vae);
  double step_ms[FLUX_MAX_STEPS];
  /* -v: the reference prints wall-clock time per block group (flux_sample.c:270-287); here the same split comes
   * from CUDA events around every launch, which costs a few percent and is therefore off otherwise */
  if (!rc && flux_verbose) rc = flux_cuda_sampler_set_profiling(s, 1);
  if (!rc && !observed) {
    /* nobody watches the steps: the whole loop stays on the device */
    rc = flux_cuda_sampler_run(s, schedule, num_steps, guidance, 0, 1);
    if (!rc) rc = flux_cuda_sampler_download(s, out, NULL);
    if (!rc) add_group_times(s);
  } else {
    for (int step = 0; !rc && step < num_steps; step++) {
      const double t0 = now_ms();
      if (flux_step_callback) flux_step_callback(step + 1, num_steps);
      rc = flux_cuda_sampler_run_steps(s, schedule, num_steps, step, 1, guidance, 0);
      if (!rc) rc = flux_cuda_sampler_download(s, out, NULL); /* waits for the step; out = current latent */
      if (rc) break;
      add_group_times(s);
      fire_substeps(tf);
      if (emb_uncond) fire_substeps(tf); /* the reference runs two forwards per guided step */
      if (step < FLUX_MAX_STEPS) step_ms[step] = now_ms() - t0;
      if (progress_callback) progress_callback(step + 1, num_steps);
      if (flux_step_image_callback && flux_step_image_vae && step + 1 < num_steps) {
        flux_image *img = flux_vae_decode((flux_vae_t *)flux_step_image_vae, out, 1, h, w);
        if (img) {
          flux_step_image_callback(step + 1, num_steps, img);
          flux_image_free(img);
        }
      }
    }
  }
  flux_timing_transformer_total = now_ms() - t_start;
  if (!rc && flux_verbose) {
    fprintf(stderr, "\nDenoising timing breakdown:\n");
    if (observed)
      for (int step = 0; step < num_steps && step < FLUX_MAX_STEPS; step++)
        fprintf(stderr, "  Step %d: %.1f ms\n", step + 1, step_ms[step]);
    fprintf(stderr, "  Total denoising: %.1f ms (%.2f s)\n", flux_timing_transformer_total,
            flux_timing_transformer_total / 1000.0);
    if (flux_timing_transformer_double > 0 || flux_timing_transformer_single > 0) {
      const double tot = flux_timing_transformer_total;
      fprintf(stderr, "  Transformer breakdown (device time):\n");
      fprintf(stderr, "    Double blocks: %.1f ms (%.1f%%)\n", flux_timing_transformer_double,
              100.0 * flux_timing_transformer_double / tot);
      fprintf(stderr, "    Single blocks: %.1f ms (%.1f%%)\n", flux_timing_transformer_single,
              100.0 * flux_timing_transformer_single / tot);
      fprintf(stderr, "    Final layer:   %.1f ms (%.1f%%)\n", flux_timing_transformer_final,
              100.0 * flux_timing_transformer_final / tot);
      fprintf(stderr, "    Total:         %.1f ms\n", tot);
    }
  }
  warn_if_saturated();
  flux_cuda_sampler_free(s);
  if (rc) {
    fprintf(stderr, "flux_cuda: %s\n", flux_cuda_last_error());
    free(out);
    return NULL;
  }
  return out;
}

float *flux_sample_euler(void *transformer, void *text_encoder, float *z, int batch, int channels, int h, int w,
                         const float *text_emb, int text_seq, const float *schedule, int num_steps,
                         void (*progress_callback)(int step, int total)) {
  (void)text_encoder;
  return sample_common((flux_transformer_t *)transformer, z, batch, channels, h, w, NULL, 0, text_emb, text_seq, NULL,
                       0, 1.0f, schedule, num_steps, progress_callback);
}

float *flux_sample_euler_with_refs(void *transformer, void *text_encoder, float *z, int batch, int channels, int h,
                                   int w, const float *ref_latent, int ref_h, int ref_w, int t_offset,
                                   const float *text_emb, int text_seq, const float *schedule, int num_steps,
                                   void (*progress_callback)(int step, int total)) {
  (void)text_encoder;
  flux_ref_t r = {ref_latent, ref_h, ref_w, t_offset};
  return sample_common((flux_transformer_t *)transformer, z, batch, channels, h, w, ref_latent ? &r : NULL,
                       ref_latent ? 1 : 0, text_emb, text_seq, NULL, 0, 1.0f, schedule, num_steps, progress_callback);
}

float *flux_sample_euler_with_multi_refs(void *transformer, void *text_encoder, float *z, int batch, int channels,
                                         int h, int w, const flux_ref_t *refs, int num_refs, const float *text_emb,
                                         int text_seq, const float *schedule, int num_steps,
                                         void (*progress_callback)(int step, int total)) {
  (void)text_encoder;
  return sample_common((flux_transformer_t *)transformer, z, batch, channels, h, w, refs, num_refs, text_emb,
                       text_seq, NULL, 0, 1.0f, schedule, num_steps, progress_callback);
}

float *flux_sample_euler_cfg(void *transformer, void *text_encoder, float *z, int batch, int channels, int h, int w,
                             const float *text_emb_cond, int text_seq_cond, const float *text_emb_uncond,
                             int text_seq_uncond, float guidance_scale, const float *schedule, int num_steps,
                             void (*progress_callback)(int step, int total)) {
  (void)text_encoder;
  return sample_common((flux_transformer_t *)transformer, z, batch, channels, h, w, NULL, 0, text_emb_cond,
                       text_seq_cond, text_emb_uncond, text_seq_uncond, guidance_scale, schedule, num_steps,
                       progress_callback);
}

float *flux_sample_euler_cfg_with_refs(void *transformer, void *text_encoder, float *z, int batch, int channels, int h,
                                       int w, const float *ref_latent, int ref_h, int ref_w, int t_offset,
                                       const float *text_emb_cond, int text_seq_cond, const float *text_emb_uncond,
                                       int text_seq_uncond, float guidance_scale, const float *schedule,
                                       int num_steps, void (*progress_callback)(int step, int total)) {
  (void)text_encoder;
  flux_ref_t r = {ref_latent, ref_h, ref_w, t_offset};
  return sample_common((flux_transformer_t *)transformer, z, batch, channels, h, w, ref_latent ? &r : NULL,
                       ref_latent ? 1 : 0, text_emb_cond, text_seq_cond, text_emb_uncond, text_seq_uncond,
                       guidance_scale, schedule, num_steps, progress_callback);
}

float *flux_sample_euler_cfg_with_multi_refs(void *transformer, void *text_encoder, float *z, int batch, int channels,
                                             int h, int w, const flux_ref_t *refs, int num_refs,
                                             const float *text_emb_cond, int text_seq_cond,
                                             const float *text_emb_uncond, int text_seq_uncond, float guidance_scale,
                                             const float *schedule, int num_steps,
                                             void (*progress_callback)(int step, int total)) {
  (void)text_encoder;
  return sample_common((flux_transformer_t *)transformer, z, batch, channels, h, w, refs, num_refs, text_emb_cond,
                       text_seq_cond, text_emb_uncond, text_seq_uncond, guidance_scale, schedule, num_steps,
                       progress_callback);
}

/* ------------------------------------------------------------------------------------------ other samplers
 * Exported by flux_sample.c but called from nowhere in the reference (flux_sample.c:697-821, 891-930). They are
 * host loops over single forwards, kept for symbol completeness; the latent visits the host between steps. */
static void after_step(int step, int num_steps, const float *z, int h, int w, void (*progress_callback)(int, int)) {
  if (progress_callback) progress_callback(step + 1, num_steps);
  if (flux_step_image_callback && flux_step_image_vae && step + 1 < num_steps) {
    flux_image *img = flux_vae_decode((flux_vae_t *)flux_step_image_vae, z, 1, h, w);
    if (img) {
      flux_step_image_callback(step + 1, num_steps, img);
      flux_image_free(img);
    }
  }
}

/* Euler steps with fresh Gaussian noise of scale eta * sqrt(|dt|) added after every step but the last. */
float *flux_sample_euler_ancestral(void *transformer, float *z, int batch, int channels, int h, int w,
                                   const float *text_emb, int text_seq, const float *schedule, int num_steps,
                                   float eta, void (*progress_callback)(int step, int total)) {
  flux_transformer_t *tf = (flux_transformer_t *)transformer;
  if (!tf || !z || batch != 1) return NULL;
  const int n = channels * h * w;
  float *cur = (float *)malloc((size_t)n * sizeof(float));
  float *noise = (float *)malloc((size_t)n * sizeof(float));
  if (!cur || !noise) {
    free(cur);
    free(noise);
    return NULL;
  }
  memcpy(cur, z, (size_t)n * sizeof(float));
  for (int step = 0; step < num_steps; step++) {
    const float dt = schedule[step + 1] - schedule[step];
    float *v = flux_transformer_forward(tf, cur, h, w, text_emb, text_seq, schedule[step]);
    if (!v) {
      free(cur);
      free(noise);
      return NULL;
    }
    for (int i = 0; i < n; i++) cur[i] += dt * v[i];
    free(v);
    if (eta > 0.0f && step < num_steps - 1) {
      const float sigma = eta * sqrtf(fabsf(dt));
      flux_randn(noise, n);
      for (int i = 0; i < n; i++) cur[i] += sigma * noise[i];
    }
    after_step(step, num_steps, cur, h, w, progress_callback);
  }
  free(noise);
  return cur;
}

/* Heun (second order): predictor z + dt v(z, t), corrector with the mean of the two velocities; the last step
 * is a plain Euler step. */
float *flux_sample_heun(void *transformer, float *z, int batch, int channels, int h, int w, const float *text_emb,
                        int text_seq, const float *schedule, int num_steps,
                        void (*progress_callback)(int step, int total)) {
  flux_transformer_t *tf = (flux_transformer_t *)transformer;
  if (!tf || !z || batch != 1) return NULL;
  const int n = channels * h * w;
  float *cur = (float *)malloc((size_t)n * sizeof(float));
  float *pred = (float *)malloc((size_t)n * sizeof(float));
  if (!cur || !pred) {
    free(cur);
    free(pred);
    return NULL;
  }
  memcpy(cur, z, (size_t)n * sizeof(float));
  for (int step = 0; step < num_steps; step++) {
    const float dt = schedule[step + 1] - schedule[step];
    float *v1 = flux_transformer_forward(tf, cur, h, w, text_emb, text_seq, schedule[step]);
    float *v2 = NULL;
    if (v1 && step < num_steps - 1) {
      for (int i = 0; i < n; i++) pred[i] = cur[i] + dt * v1[i];
      v2 = flux_transformer_forward(tf, pred, h, w, text_emb, text_seq, schedule[step + 1]);
    }
    if (!v1 || (step < num_steps - 1 && !v2)) {
      free(v1);
      free(cur);
      free(pred);
      return NULL;
    }
    if (v2)
      for (int i = 0; i < n; i++) cur[i] += 0.5f * dt * (v1[i] + v2[i]);
    else
      for (int i = 0; i < n; i++) cur[i] += dt * v1[i];
    free(v1);
    free(v2);
    after_step(step, num_steps, cur, h, w, progress_callback);
  }
  free(pred);
  return cur;
}

/* Shifted-sigmoid and resolution-dependent schedules (flux_sample.c:75-116). */
float *flux_sigmoid_schedule(int num_steps, float shift) {
  float *s = (float *)malloc((num_steps + 1) * sizeof(float));
  if (!s) return NULL;
  for (int i = 0; i <= num_steps; i++) {
    const float x = ((float)i / (float)num_steps - 0.5f) * 10.0f + shift;
    s[i] = 1.0f - 1.0f / (1.0f + expf(-x));
  }
  s[0] = 1.0f;
  s[num_steps] = 0.0f;
  return s;
}

float *flux_resolution_schedule(int num_steps, int height, int width) {
  float *s = (float *)malloc((num_steps + 1) * sizeof(float));
  if (!s) return NULL;
  const long pixels = (long)height * width;
  const float shift = pixels >= 1024L * 1024L ? 1.0f : pixels >= 512L * 512L ? 0.5f : 0.0f;
  for (int i = 0; i <= num_steps; i++) s[i] = 1.0f - powf((float)i / (float)num_steps, 1.0f + 0.5f * shift);
  return s;
}

/* flux_generate_latent (flux_sample.c:891-919): noise from the seed, LINEAR schedule, plain Euler loop. */
float *flux_generate_latent(void *ctx_ptr, const float *text_emb, int text_seq, int height, int width, int num_steps,
                            int64_t seed, void (*progress_callback)(int step, int total)) {
  const int lh = height / 16, lw = width / 16;
  float *z = flux_init_noise(1, FLUX_LATENT_CHANNELS, lh, lw, seed);
  float *sched = flux_linear_schedule(num_steps);
  float *out = (z && sched) ? flux_sample_euler(ctx_ptr, NULL, z, 1, FLUX_LATENT_CHANNELS, lh, lw, text_emb, text_seq,
                                                sched, num_steps, progress_callback)
                            : NULL;
  free(z);
  free(sched);
  return out;
}

void (*flux_progress_callback)(int, int) = NULL;
void flux_set_progress_callback(void (*callback)(int, int)) { flux_progress_callback = callback; }

/* ------------------------------------------------------------------------------------------ host pieces */
float *flux_linear_schedule(int num_steps) {
  float *s = (float *)malloc((num_steps + 1) * sizeof(float));
  if (s) flux_cuda_linear_schedule(num_steps, s);
  return s;
}

float *flux_power_schedule(int num_steps, float alpha) {
  float *s = (float *)malloc((num_steps + 1) * sizeof(float));
  if (s) flux_cuda_power_schedule(num_steps, alpha, s);
  return s;
}

float *flux_official_schedule(int num_steps, int image_seq_len) {
  float *s = (float *)malloc((num_steps + 1) * sizeof(float));
  if (s) flux_cuda_official_schedule(num_steps, image_seq_len, s);
  return s;
}

float *flux_init_noise(int batch, int channels, int h, int w, int64_t seed) {
  if (batch != 1) return NULL; /* every call site of the reference passes 1 */
  float *n = (float *)malloc((size_t)channels * h * w * sizeof(float));
  if (!n) return NULL;
  if (seed < 0) seed = 0;
  flux_cuda_init_noise(channels, h, w, (long long)seed, n);
  return n;
}
