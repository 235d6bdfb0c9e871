/* Host-side pieces of the sampler: timestep schedules and the seeded initial noise. Plain C, no GPU.
 * Same results as the reference's flux_linear_schedule / flux_power_schedule / flux_official_schedule
 * (flux_sample.c:49-69, 122-155) and flux_init_noise (flux_sample.c:835-877) with its generator
 * (flux_kernels.c:45-102), so that a seed produces the same image through either implementation. */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>

#include "flux_cuda.h"

void flux_cuda_linear_schedule(int num_steps, float *out) {
  for (int i = 0; i <= num_steps; i++) out[i] = 1.0f - (float)i / (float)num_steps;
}

void flux_cuda_power_schedule(int num_steps, float alpha, float *out) {
  for (int i = 0; i <= num_steps; i++) out[i] = 1.0f - powf((float)i / (float)num_steps, alpha);
}

/* mu: two lines fitted in the image token count (one for 10 steps, one for 200), interpolated in the
 * step count; above 4300 tokens only the 200-step line is used. */
static float empirical_mu(int seq_len, int num_steps) {
  const float a1 = 8.73809524e-05f, b1 = 1.89833333f, a2 = 0.00016927f, b2 = 0.45666666f;
  const float m200 = a2 * (float)seq_len + b2;
  if (seq_len > 4300) return m200;
  const float m10 = a1 * (float)seq_len + b1;
  const float slope = (m200 - m10) / 190.0f;
  return slope * (float)num_steps + (m200 - 200.0f * slope);
}

void flux_cuda_official_schedule(int num_steps, int image_seq_len, float *out) {
  const float emu = expf(empirical_mu(image_seq_len, num_steps));
  for (int i = 0; i <= num_steps; i++) {
    const float t = 1.0f - (float)i / (float)num_steps;
    if (t <= 0.0f) out[i] = 0.0f;
    else if (t >= 1.0f) out[i] = 1.0f;
    else out[i] = emu / (emu + (1.0f / t - 1.0f));
  }
}

/* xoshiro256** seeded by four rounds of SplitMix64; one normal per two uniforms (Box-Muller, cosine branch). */
typedef struct { uint64_t s[4]; } fx_rng;

static uint64_t fx_rotl(uint64_t x, int k) { return (x << k) | (x >> (64 - k)); }

static void fx_rng_seed(fx_rng *r, uint64_t seed) {
  for (int i = 0; i < 4; i++) {
    seed += 0x9e3779b97f4a7c15ULL;
    uint64_t z = seed;
    z = (z ^ (z >> 30)) * 0xbf58476d1ce4e5b9ULL;
    z = (z ^ (z >> 27)) * 0x94d049bb133111ebULL;
    r->s[i] = z ^ (z >> 31);
  }
}

static uint64_t fx_rng_next(fx_rng *r) {
  uint64_t *s = r->s;
  const uint64_t out = fx_rotl(s[1] * 5, 7) * 9;
  const uint64_t t = s[1] << 17;
  s[2] ^= s[0];
  s[3] ^= s[1];
  s[1] ^= s[2];
  s[0] ^= s[3];
  s[2] ^= t;
  s[3] = fx_rotl(s[3], 45);
  return out;
}

static float fx_uniform(fx_rng *r) { return (float)((double)(fx_rng_next(r) >> 11) * (1.0 / 9007199254740992.0)); }

static float fx_normal(fx_rng *r) {
  float u1 = fx_uniform(r);
  const float u2 = fx_uniform(r);
  while (u1 == 0.0f) u1 = fx_uniform(r);
  return sqrtf(-2.0f * logf(u1)) * cosf(2.0f * 3.14159265358979323846f * u2);
}

#define FX_NOISE_MAX 112 /* 1792 / 16: the master field every smaller latent is sampled from */

void flux_cuda_init_noise(int channels, int h, int w, long long seed, float *out) {
  fx_rng r;
  fx_rng_seed(&r, (uint64_t)seed);
  if (h >= FX_NOISE_MAX && w >= FX_NOISE_MAX) {
    const long long n = (long long)channels * h * w;
    for (long long i = 0; i < n; i++) out[i] = fx_normal(&r);
    return;
  }
  /* The field is generated channel by channel in row-major order; only the rows and columns the
   * nearest-neighbour subsampling picks (sy = ty*112/h, sx = tx*112/w) are kept. */
  float *row = (float *)malloc(sizeof(float) * FX_NOISE_MAX);
  for (int c = 0; c < channels; c++) {
    int ty = 0;
    for (int sy = 0; sy < FX_NOISE_MAX; sy++) {
      for (int sx = 0; sx < FX_NOISE_MAX; sx++) row[sx] = fx_normal(&r);
      while (ty < h && ty * FX_NOISE_MAX / h == sy) {
        float *dst = out + ((long long)c * h + ty) * w;
        for (int tx = 0; tx < w; tx++) dst[tx] = row[tx * FX_NOISE_MAX / w];
        ty++;
      }
    }
  }
  free(row);
}
