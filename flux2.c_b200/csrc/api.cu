// extern "C" surface of the library (declared in include/flux_cuda.h): context management, error
// reporting and the kernel-level entry points.
#include "flux_cuda.h"

#include <stdarg.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#include <vector>

#include "attention.cuh"
#include "context.cuh"
#include "elementwise.cuh"
#include "engine.cuh"
#include "conv.cuh"
#include "gemm.cuh"
#include "launch.cuh"
#include "vae_kernels.cuh"

namespace fx {
static thread_local char g_err[512] = "";

void set_error(const char *fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_err, sizeof(g_err), fmt, ap);
  va_end(ap);
}
int check_cuda(cudaError_t e, const char *what) {
  if (e == cudaSuccess) return FLUX_CUDA_OK;
  set_error("%s: %s", what, cudaGetErrorString(e));
  return FLUX_CUDA_ERR_CUDA;
}
int ctx_sync_check(flux_cuda_ctx *ctx) {
  // word 0: first kernel error code; word 1: f16 stores that saturated since the last read
  int rc = check_cuda(cudaMemcpyAsync(ctx->err_host, ctx->err_dev, 2 * sizeof(int), cudaMemcpyDeviceToHost,
                                      ctx->stream),
                      "read kernel error word");
  if (rc) return rc;
  rc = check_cuda(cudaStreamSynchronize(ctx->stream), "stream synchronize");
  if (rc) return rc;
  if (ctx->err_host[1] != 0) {
    ctx->saturated += static_cast<unsigned int>(ctx->err_host[1]);
    cudaMemsetAsync(ctx->err_dev + 1, 0, sizeof(int), ctx->stream);
  }
  if (ctx->err_host[0] != 0) {
    const int code = ctx->err_host[0];
    cudaMemsetAsync(ctx->err_dev, 0, sizeof(int), ctx->stream);
    if (code == 8) {  // KERR_BAD_INDEX
      set_error("checked build: a kernel computed an address outside its buffer or off its alignment and skipped it");
      return FLUX_CUDA_ERR_KERNEL;
    }
    if (code == 9) {  // KERR_PEER_TIMEOUT
      set_error("the other GPU of the pair did not deliver its half of a step within the kernel's wait limit");
      return FLUX_CUDA_ERR_PEER_TIMEOUT;
    }
    set_error("a kernel gave up on a bounded wait (code %d)", code);
    return FLUX_CUDA_ERR_KERNEL;
  }
  return FLUX_CUDA_OK;
}
}  // namespace fx

using namespace fx;

extern "C" {

const char *flux_cuda_last_error(void) { return g_err; }

int flux_cuda_build_checked(void) {
#ifdef FLUX_CUDA_DEBUG
  return 1;
#else
  return 0;
#endif
}

int flux_cuda_ctx_create(int device, flux_cuda_ctx **out) {
  if (!out) return FLUX_CUDA_ERR_ARG;
  *out = nullptr;
  int n = 0;
  if (cudaGetDeviceCount(&n) != cudaSuccess || n == 0) {
    set_error("no CUDA device is visible: this library has no CPU path");
    return FLUX_CUDA_ERR_CUDA;
  }
  if (device < 0 || device >= n) {
    set_error("device %d out of range (have %d)", device, n);
    return FLUX_CUDA_ERR_ARG;
  }
  int rc = check_cuda(cudaSetDevice(device), "cudaSetDevice");
  if (rc) return rc;
  cudaDeviceProp prop;
  rc = check_cuda(cudaGetDeviceProperties(&prop, device), "cudaGetDeviceProperties");
  if (rc) return rc;
  if (prop.major != 10) {
    set_error("device %d is sm_%d%d; this library contains sm_100a code only", device, prop.major, prop.minor);
    return FLUX_CUDA_ERR_CUDA;
  }
  flux_cuda_ctx *c = new flux_cuda_ctx();
  c->device = device;
  c->num_sms = prop.multiProcessorCount;
  if ((rc = check_cuda(cudaStreamCreateWithFlags(&c->stream, cudaStreamNonBlocking), "cudaStreamCreate")) ||
      (rc = check_cuda(cudaMalloc(&c->err_dev, 2 * sizeof(int)), "cudaMalloc")) ||
      (rc = check_cuda(cudaMallocHost(&c->err_host, 2 * sizeof(int)), "cudaMallocHost")) ||
      (rc = check_cuda(cudaMemset(c->err_dev, 0, 2 * sizeof(int)), "cudaMemset"))) {
    flux_cuda_ctx_destroy(c);
    return rc;
  }
  if (const char *e = getenv("FLUX_CUDA_GEMM_PAIR")) c->gemm_pair = atoi(e) != 0;
  if (const char *e = getenv("FLUX_CUDA_BF16")) c->f16 = atoi(e) == 0;
  if (const char *e = getenv("FLUX_CUDA_ATTN")) c->attn_version = atoi(e) == 3 ? 3 : 2;
  if (gemm_init() != 0 || gemm2_init() != 0 || attn2_init() != 0 || attn3_init() != 0 || elementwise_init() != 0 ||
      conv_init() != 0) {
    set_error("could not resolve cuTensorMapEncodeTiled / configure shared memory");
    flux_cuda_ctx_destroy(c);
    return FLUX_CUDA_ERR_CUDA;
  }
  *out = c;
  return FLUX_CUDA_OK;
}

void flux_cuda_ctx_destroy(flux_cuda_ctx *ctx) {
  if (!ctx) return;
  cudaSetDevice(ctx->device);
  if (ctx->stream) {
    cudaStreamSynchronize(ctx->stream);
    cudaStreamDestroy(ctx->stream);
  }
  fx::upload_ring_release(ctx);
  if (ctx->copy_stream) {
    cudaStreamSynchronize(ctx->copy_stream);
    cudaStreamDestroy(ctx->copy_stream);
  }
  if (ctx->err_dev) cudaFree(ctx->err_dev);
  if (ctx->err_host) cudaFreeHost(ctx->err_host);
  if (ctx->gn_scratch) cudaFree(ctx->gn_scratch);
  if (ctx->rope_scratch) cudaFree(ctx->rope_scratch);
  delete ctx;
}

int flux_cuda_ctx_sync(flux_cuda_ctx *ctx) {
  if (!ctx) return FLUX_CUDA_ERR_ARG;
  return ctx_sync_check(ctx);
}

void *flux_cuda_ctx_stream(flux_cuda_ctx *ctx) { return ctx ? (void *)ctx->stream : nullptr; }

int flux_cuda_ctx_saturated_stores(flux_cuda_ctx *ctx, long long *count, int reset) {
  if (!ctx || !count) return FLUX_CUDA_ERR_ARG;
  *count = ctx->saturated;
  if (reset) ctx->saturated = 0;
  return FLUX_CUDA_OK;
}

int flux_cuda_ctx_set_half_format(flux_cuda_ctx *ctx, int dtype) {
  if (!ctx || (dtype != FLUX_CUDA_F16 && dtype != FLUX_CUDA_BF16)) return FLUX_CUDA_ERR_ARG;
  ctx->f16 = dtype == FLUX_CUDA_F16;
  return FLUX_CUDA_OK;
}

int flux_cuda_ctx_set_gemm_trace(flux_cuda_ctx *ctx, long long *stamps_dev) {
  if (!ctx) return FLUX_CUDA_ERR_ARG;
  ctx->gemm_trace = stamps_dev;
  return FLUX_CUDA_OK;
}

int flux_cuda_ctx_set_gemm_pair(flux_cuda_ctx *ctx, int on) {
  if (!ctx) return FLUX_CUDA_ERR_ARG;
  ctx->gemm_pair = on != 0;
  return FLUX_CUDA_OK;
}

int flux_cuda_gemm_bf16(flux_cuda_ctx *ctx, const void *x, const void *w, void *out, int M, int N, int K,
                        int epilogue, long long ld_out, const float *gate, int tile_n) {
  if (!ctx || !x || !w || !out) {
    set_error("gemm: null argument");
    return FLUX_CUDA_ERR_ARG;
  }
  const int x_f16 = (epilogue & FLUX_CUDA_EPI_X_F16) != 0, out_f16 = (epilogue & FLUX_CUDA_EPI_OUT_F16) != 0;
  epilogue &= 0xFF;
  if (epilogue < 0 || epilogue > 4 || (epilogue == EPI_GATED_RES_F32 && !gate)) {
    set_error("gemm: bad epilogue %d", epilogue);
    return FLUX_CUDA_ERR_ARG;
  }
  int bn = tile_n;
  if (bn == 0) bn = (N % 256 == 0) ? 256 : 128;
  const bool pair = bn == 512;  // 256-wide tiles computed by CTA pairs
  GemmParams P;
  memset(&P, 0, sizeof(P));
  int rc = pair ? gemm_make_problem_pair(&P.p[0], x, K, w, M, N, K) : gemm_make_problem(&P.p[0], x, K, w, M, N, K, bn);
  if (rc) {
    set_error("gemm: unsupported shape/alignment M=%d N=%d K=%d tile_n=%d (rc %d)", M, N, K, bn, rc);
    return FLUX_CUDA_ERR_ARG;
  }
  P.nprob = 1;
  P.err = ctx->err_dev;
  P.trace = ctx->gemm_trace;
  P.p[0].x_f16 = x_f16;
  P.p[0].seg[0].out_f16 = out_f16;
  P.p[0].seg[0].mode = epilogue;
  P.p[0].seg[0].col0 = 0;
  P.p[0].seg[0].ld = ld_out;
  P.p[0].seg[0].out = out;
  P.p[0].seg[0].gate = gate;
  rc = pair ? gemm2_launch(&P, ctx->num_sms, ctx->stream) : gemm_launch(&P, bn, ctx->num_sms, ctx->stream);
  if (rc) {
    set_error("gemm: launch failed (rc %d: %s)", rc, cudaGetErrorString(cudaGetLastError()));
    return rc <= -8 ? FLUX_CUDA_ERR_CUDA : FLUX_CUDA_ERR_ARG;
  }
  return FLUX_CUDA_OK;
}


int flux_cuda_gemm_qkv_norm_rope(flux_cuda_ctx *ctx, const void *x, const void *w, void *out, int M, int hidden, int K,
                                 const float *wq, const float *wk, const float *cos_t, const float *sin_t, int seq,
                                 int f16) {
  if (!ctx || !x || !w || !out || !wq || !wk || !cos_t || !sin_t || seq <= 0 || hidden % 128) {
    set_error("gemm_qkv_norm_rope: bad argument");
    return FLUX_CUDA_ERR_ARG;
  }
  GemmParams P;
  memset(&P, 0, sizeof(P));
  // the kernel the engine itself uses for this projection: CTA pairs unless the context was told otherwise
  const bool pair = ctx->gemm_pair && (3 * hidden) % 256 == 0;
  int rc = pair ? gemm_make_problem_pair(&P.p[0], x, K, w, M, 3 * hidden, K)
                : gemm_make_problem(&P.p[0], x, K, w, M, 3 * hidden, K, 256);
  if (rc) {
    set_error("gemm_qkv_norm_rope: unsupported shape/alignment M=%d hidden=%d K=%d (rc %d)", M, hidden, K, rc);
    return FLUX_CUDA_ERR_ARG;
  }
  P.nprob = 1;
  P.err = ctx->err_dev;
  P.p[0].x_f16 = f16 != 0;
  EpiSeg &sg = P.p[0].seg[0];
  sg.out_f16 = f16 != 0;
  sg.mode = EPI_QKV_NORM_ROPE;
  sg.ld = 3 * hidden;
  sg.out = out;
  sg.qk.wq_txt = sg.qk.wq_img = wq;
  sg.qk.wk_txt = sg.qk.wk_img = wk;
  sg.qk.cos_t = cos_t;
  sg.qk.sin_t = sin_t;
  {
    // the engine hands the epilogue pair angles instead of the two tables; derive them here so that this entry point
    // runs the epilogue the way the engine does
    const size_t pairs = static_cast<size_t>(seq) * 64;
    if (ctx->rope_scratch_floats < pairs) {
      cudaStreamSynchronize(ctx->stream);
      if (ctx->rope_scratch) cudaFree(ctx->rope_scratch);
      ctx->rope_scratch = nullptr;
      ctx->rope_scratch_floats = 0;
      if (check_cuda(cudaMalloc(&ctx->rope_scratch, pairs * sizeof(float)), "cudaMalloc")) return FLUX_CUDA_ERR_NOMEM;
      ctx->rope_scratch_floats = pairs;
    }
    if (launch_rope_angles(cos_t, sin_t, ctx->rope_scratch, static_cast<long long>(pairs), ctx->stream)) {
      set_error("gemm_qkv_norm_rope: angle table launch failed");
      return FLUX_CUDA_ERR_CUDA;
    }
    sg.qk.ang = ctx->rope_scratch;
  }
  sg.qk.seq = seq;
  sg.qk.q_cols = hidden;
  sg.qk.k_cols = hidden;
  sg.qk.half_split = 0;
  rc = pair ? gemm2_launch(&P, ctx->num_sms, ctx->stream) : gemm_launch(&P, 256, ctx->num_sms, ctx->stream);
  if (rc) {
    set_error("gemm_qkv_norm_rope: launch failed (rc %d)", rc);
    return FLUX_CUDA_ERR_CUDA;
  }
  return FLUX_CUDA_OK;
}

int flux_cuda_patchify(flux_cuda_ctx *ctx, float *out, const float *in, int batch, int channels, int H, int W,
                       int patch_size) {
  if (!ctx || !out || !in || batch <= 0 || channels <= 0 || H <= 0 || W <= 0) return FLUX_CUDA_ERR_ARG;
  int rc = launch_patchify(out, const_cast<float *>(in), batch, channels, H, W, patch_size, 1, ctx->stream);
  if (rc) set_error("patchify: H and W must be multiples of the patch size");
  return rc == 0 ? FLUX_CUDA_OK : rc == -1 ? FLUX_CUDA_ERR_ARG : FLUX_CUDA_ERR_CUDA;
}
int flux_cuda_unpatchify(flux_cuda_ctx *ctx, float *out, const float *in, int batch, int channels, int H, int W,
                         int patch_size) {
  if (!ctx || !out || !in || batch <= 0 || channels <= 0 || H <= 0 || W <= 0 || patch_size <= 0)
    return FLUX_CUDA_ERR_ARG;
  // the reference passes the PACKED height and width here; the kernel wants the plain ones
  int rc = launch_patchify(const_cast<float *>(in), out, batch, channels, H * patch_size, W * patch_size, patch_size, 0,
                           ctx->stream);
  if (rc) set_error("unpatchify: launch failed");
  return rc == 0 ? FLUX_CUDA_OK : FLUX_CUDA_ERR_CUDA;
}

int flux_cuda_attention(flux_cuda_ctx *ctx, const void *qkv, int batch, int seq, long long ld, int q_col, int k_col,
                        int v_col, int heads, void *out, long long out_ld, int out_col, int f16) {
  if (!ctx || !qkv || !out) return FLUX_CUDA_ERR_ARG;
  AttnParams A;
  int rc = attn2_make_params(&A, qkv, batch, seq, ld, q_col, k_col, v_col, out, out_ld, out_col, heads, f16,
                             ctx->err_dev);
  if (rc) {
    set_error("attention: unsupported shape/alignment (rc %d)", rc);
    return FLUX_CUDA_ERR_ARG;
  }
  A.trace = ctx->gemm_trace;  // measurement aid, normally null (flux_cuda_ctx_set_gemm_trace)
  rc = attn_launch_version(ctx->attn_version, &A, ctx->stream);
  if (rc) {
    set_error("attention: launch failed: %s", cudaGetErrorString(cudaGetLastError()));
    return FLUX_CUDA_ERR_CUDA;
  }
  return FLUX_CUDA_OK;
}

int flux_cuda_adaln(flux_cuda_ctx *ctx, const float *x, void *out, int rows, int hidden, const float *shift,
                    const float *scale, int f16) {
  if (!ctx || !x || !out || !shift || !scale) return FLUX_CUDA_ERR_ARG;
  int rc = launch_adaln(x, out, 0, rows, hidden, rows > 0 ? rows : 1, 0, f16, shift, scale, shift, scale, ctx->stream,
                        ctx->err_dev + 1);
  if (rc) {
    set_error("adaln: unsupported hidden size %d or launch failure", hidden);
    return rc == -1 ? FLUX_CUDA_ERR_ARG : FLUX_CUDA_ERR_CUDA;
  }
  return FLUX_CUDA_OK;
}

static int conv_finish(flux_cuda_ctx *ctx, ConvParams &P, const float *bias, int mode, void *out, long long ld, int f16,
                       const char *what) {
  if (mode < 0 || mode > 3 || !out) {
    set_error("%s: bad mode or output", what);
    return FLUX_CUDA_ERR_ARG;
  }
  P.mode = mode;
  P.out = out;
  P.ld = ld;
  P.bias = bias;
  P.out_f16 = P.x_f16 = f16 ? 1 : 0;
  P.err = ctx->err_dev;
  PdlOff plain_launches;  // plain stream order, as the VAE itself launches this kernel
  if (conv_launch(&P, ctx->num_sms, ctx->stream) != 0) {
    set_error("%s: launch failed: %s", what, cudaGetErrorString(cudaGetLastError()));
    return FLUX_CUDA_ERR_CUDA;
  }
  return FLUX_CUDA_OK;
}

int flux_cuda_conv3x3(flux_cuda_ctx *ctx, const void *x16, int n_img, int H, int W, int cin, const void *w16, int cout,
                      const float *bias, int mode, void *out, long long ld, int f16) {
  if (!ctx || !x16 || !w16) return FLUX_CUDA_ERR_ARG;
  cudaSetDevice(ctx->device);
  ConvParams P;
  memset(&P, 0, sizeof(P));
  if (conv_make_3x3(&P, x16, n_img, H, W, cin, w16, cout) != 0) {
    set_error("conv3x3: unsupported shape (cin %% 64, cout %% 128, 16-byte aligned pointers)");
    return FLUX_CUDA_ERR_ARG;
  }
  return conv_finish(ctx, P, bias, mode, out, ld, f16, "conv3x3");
}

int flux_cuda_conv3x3_stride2(flux_cuda_ctx *ctx, const void *planes16, int n_img, int Ho, int Wo, int cin,
                              const void *w16, int cout, const float *bias, int mode, void *out, long long ld, int f16) {
  if (!ctx || !planes16 || !w16) return FLUX_CUDA_ERR_ARG;
  cudaSetDevice(ctx->device);
  ConvParams P;
  memset(&P, 0, sizeof(P));
  if (conv_make_3x3_s2(&P, planes16, n_img, Ho, Wo, cin, w16, cout) != 0) {
    set_error("conv3x3_stride2: unsupported shape (cin %% 64, cout %% 128, 16-byte aligned pointers)");
    return FLUX_CUDA_ERR_ARG;
  }
  return conv_finish(ctx, P, bias, mode, out, ld, f16, "conv3x3_stride2");
}

int flux_cuda_gemm_bias(flux_cuda_ctx *ctx, const void *x16, long long ldx, const void *w16, long long ldw, int M, int N,
                        int K, int w_rows, const float *bias, int mode, void *out, long long ld, int f16) {
  if (!ctx || !x16 || !w16) return FLUX_CUDA_ERR_ARG;
  cudaSetDevice(ctx->device);
  ConvParams P;
  memset(&P, 0, sizeof(P));
  if (conv_make_gemm(&P, x16, ldx, w16, ldw, M, N, K, w_rows) != 0) {
    set_error("gemm_bias: unsupported shape (K %% 64, N %% 128, 16-byte aligned pointers and pitches)");
    return FLUX_CUDA_ERR_ARG;
  }
  return conv_finish(ctx, P, bias, mode, out, ld, f16, "gemm_bias");
}

int flux_cuda_group_norm(flux_cuda_ctx *ctx, const void *x, int in16, void *out16, int n_img, long long pixels, int C,
                         const float *gamma, const float *beta, float eps, int swish, int f16) {
  if (!ctx || !x || !out16 || !gamma || !beta || n_img < 1 || n_img > 8 || pixels < 1) {
    set_error("group_norm: bad argument (1 <= n_img <= 8)");
    return FLUX_CUDA_ERR_ARG;
  }
  if ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(out16) | reinterpret_cast<uintptr_t>(gamma) |
       reinterpret_cast<uintptr_t>(beta)) & 15) {
    set_error("group_norm: x, out16, gamma and beta must be 16-byte aligned");
    return FLUX_CUDA_ERR_ARG;
  }
  cudaSetDevice(ctx->device);
  PdlOff plain_launches;  // plain stream order, as the VAE itself launches these kernels
  const size_t part = static_cast<size_t>(8) * GN_MAX_BLOCKS * 64, stats = 8 * GN_GROUPS * 2;
  if (!ctx->gn_scratch) {
    int rc = check_cuda(cudaMalloc(&ctx->gn_scratch, (part + stats + 8) * 4), "cudaMalloc");
    if (rc) return rc;
    cudaMemsetAsync(ctx->gn_scratch, 0, (part + stats + 8) * 4, ctx->stream);
  }
  float *st = ctx->gn_scratch + part;
  unsigned int *counters = reinterpret_cast<unsigned int *>(st + stats);
  int rc = launch_gn_stats(x, in16, f16, n_img, pixels, C, eps, ctx->gn_scratch, counters, st, ctx->stream);
  if (!rc) rc = launch_gn_apply(x, in16, out16, f16, n_img, pixels, C, st, gamma, beta, swish, ctx->stream);
  if (rc) {
    set_error("group_norm: unsupported channel count %d or launch failure", C);
    return rc == -1 ? FLUX_CUDA_ERR_ARG : FLUX_CUDA_ERR_CUDA;
  }
  return FLUX_CUDA_OK;
}

int flux_cuda_qk_norm_rope(flux_cuda_ctx *ctx, void *qkv, long long ld, int q_col, int k_col, int seq, int batch,
                           int heads, const float *wq, const float *wk, const float *cos_t, const float *sin_t) {
  if (!ctx || !qkv || !wq || !wk || !cos_t || !sin_t) return FLUX_CUDA_ERR_ARG;
  int rc = launch_qk_norm_rope(qkv, ld, q_col, k_col, seq, batch, heads, 0, wq, wk, wq, wk, cos_t, sin_t, ctx->stream);
  if (rc) {
    set_error("qk_norm_rope: launch failed");
    return FLUX_CUDA_ERR_CUDA;
  }
  return FLUX_CUDA_OK;
}

// ------------------------------------------------------------------------------------------------ model
void flux_cuda_dims_klein4b(flux_cuda_dims *d) {
  if (!d) return;
  d->hidden = 3072;
  d->heads = 24;
  d->head_dim = 128;
  d->mlp = 9216;
  d->n_double = 5;
  d->n_single = 20;
  d->text_dim = 7680;
  d->latent_ch = 128;
  d->time_dim = 256;
  d->rope_theta = 2000.0f;
  d->axis_dim = 32;
}

static ModelDims to_dims(const flux_cuda_dims *d) {
  ModelDims m;
  m.hidden = d->hidden;
  m.heads = d->heads;
  m.head_dim = d->head_dim;
  m.mlp = d->mlp;
  m.n_double = d->n_double;
  m.n_single = d->n_single;
  m.text_dim = d->text_dim;
  m.latent_ch = d->latent_ch;
  m.time_dim = d->time_dim;
  m.rope_theta = d->rope_theta;
  m.axis_dim = d->axis_dim;
  return m;
}

int flux_cuda_model_create(flux_cuda_ctx *ctx, const flux_cuda_dims *dims, flux_cuda_model **out) {
  if (!ctx || !dims || !out) return FLUX_CUDA_ERR_ARG;
  return model_create(ctx, to_dims(dims), out);
}
int flux_cuda_model_set_tensor(flux_cuda_model *m, const char *name, const void *data, int dtype,
                               const long long *shape, int ndim) {
  return model_set_tensor(m, name, data, dtype, shape, ndim);
}
int flux_cuda_model_finalize(flux_cuda_model *m) { return model_finalize(m); }
void flux_cuda_model_free(flux_cuda_model *m) { model_free(m); }
int flux_cuda_model_load_safetensors(flux_cuda_ctx *ctx, const char *path, flux_cuda_model **out) {
  if (!out) return FLUX_CUDA_ERR_ARG;
  return model_load_safetensors(ctx, path, out);
}
int flux_cuda_model_dims(const flux_cuda_model *m, flux_cuda_dims *o) {
  if (!m || !o) return FLUX_CUDA_ERR_ARG;
  const ModelDims &d = m->d;
  o->hidden = d.hidden;
  o->heads = d.heads;
  o->head_dim = d.head_dim;
  o->mlp = d.mlp;
  o->n_double = d.n_double;
  o->n_single = d.n_single;
  o->text_dim = d.text_dim;
  o->latent_ch = d.latent_ch;
  o->time_dim = d.time_dim;
  o->rope_theta = d.rope_theta;
  o->axis_dim = d.axis_dim;
  return FLUX_CUDA_OK;
}

// ------------------------------------------------------------------------------------------------ sampler
int flux_cuda_sampler_create(flux_cuda_model *m, int h, int w, int txt_seq, const flux_cuda_ref_shape *refs,
                             int num_refs, int batch, int max_steps, flux_cuda_sampler **out) {
  if (!out) return FLUX_CUDA_ERR_ARG;
  std::vector<RefSpec> rs;
  for (int i = 0; i < num_refs && refs; ++i) rs.push_back(RefSpec{refs[i].h, refs[i].w, refs[i].t_offset});
  return sampler_create(m, h, w, txt_seq, rs.data(), num_refs, batch, max_steps, out);
}
void flux_cuda_sampler_free(flux_cuda_sampler *s) { sampler_free(s); }
int flux_cuda_sampler_upload(flux_cuda_sampler *s, const float *z0, const float *ctx, const float *ctx_uncond,
                             const float *const *ref_latents) {
  return sampler_upload(s, z0, ctx, ctx_uncond, ref_latents);
}
int flux_cuda_sampler_run(flux_cuda_sampler *s, const float *schedule, int num_steps, float guidance,
                          int record_velocities, int apply_update) {
  return sampler_run(s, schedule, num_steps, 0, num_steps, guidance, record_velocities, apply_update);
}
int flux_cuda_sampler_run_steps(flux_cuda_sampler *s, const float *schedule, int num_steps, int first, int count,
                                float guidance, int record_velocities) {
  return sampler_run(s, schedule, num_steps, first, count, guidance, record_velocities, 1);
}
int flux_cuda_sampler_predict(flux_cuda_sampler *s, const float *schedule, int num_steps, int step) {
  return sampler_run(s, schedule, num_steps, step, 1, 1.0f, 0, 0);
}
int flux_cuda_sampler_velocity(flux_cuda_sampler *s, float *dst_dev, float scale) {
  if (!s || !dst_dev) return FLUX_CUDA_ERR_ARG;
  if (s->ws->B != 1) {
    set_error("velocity: only for batch-1 samplers (one member of a guidance pair per GPU)");
    return FLUX_CUDA_ERR_ARG;
  }
  cudaSetDevice(s->model->ctx->device);
  const long long n = static_cast<long long>(s->model->d.latent_ch) * s->ws->n_img;
  if (launch_scale_copy(dst_dev, s->ws->v, scale, n, s->model->ctx->stream)) {
    set_error("velocity: launch failed");
    return FLUX_CUDA_ERR_CUDA;
  }
  return FLUX_CUDA_OK;
}
int flux_cuda_sampler_apply_velocity(flux_cuda_sampler *s, const float *v_dev, int step) {
  if (!s || !v_dev || step < 0 || step >= s->ws->last_steps) {
    set_error("apply_velocity: bad argument");
    return FLUX_CUDA_ERR_ARG;
  }
  cudaSetDevice(s->model->ctx->device);
  const long long n = static_cast<long long>(s->model->d.latent_ch) * s->ws->n_img;
  if (launch_euler(s->ws->z, v_dev, s->ws->sched, step, n, s->model->ctx->stream)) {
    set_error("apply_velocity: launch failed");
    return FLUX_CUDA_ERR_CUDA;
  }
  return FLUX_CUDA_OK;
}
int flux_cuda_sampler_download(flux_cuda_sampler *s, float *latent_out, float *velocities_out) {
  return sampler_download(s, latent_out, velocities_out);
}
int flux_cuda_sampler_stage_inputs(flux_cuda_sampler *s, const float *z0, const float *ctx, const float *ctx_uncond,
                                   const float *const *ref_latents) {
  return sampler_stage_inputs(s, z0, ctx, ctx_uncond, ref_latents);
}
int flux_cuda_sampler_download_async(flux_cuda_sampler *s, float *latent_out) {
  return sampler_download_async(s, latent_out);
}
int flux_cuda_sampler_latent_device(flux_cuda_sampler *s, const float **latent_dev) {
  if (!s || !latent_dev) return FLUX_CUDA_ERR_ARG;
  *latent_dev = s->ws->z;
  return FLUX_CUDA_OK;
}
int flux_cuda_sampler_last_run(flux_cuda_sampler *s, float *ms, long long *kernel_launches) {
  if (!s) return FLUX_CUDA_ERR_ARG;
  if (ms) {
    int rc = check_cuda(cudaEventElapsedTime(ms, s->ws->ev0, s->ws->ev1), "cudaEventElapsedTime");
    if (rc) return rc;
  }
  if (kernel_launches) *kernel_launches = s->ws->launches;
  return FLUX_CUDA_OK;
}

int flux_cuda_sampler_set_profiling(flux_cuda_sampler *s, int on) {
  if (!s) return FLUX_CUDA_ERR_ARG;
  s->ws->profiling = on != 0;
  return FLUX_CUDA_OK;
}
int flux_cuda_sampler_profile(flux_cuda_sampler *s, float *ms_by_class, long long *launches_by_class) {
  return sampler_profile(s, ms_by_class, launches_by_class);
}

int flux_cuda_sampler_profile_groups(flux_cuda_sampler *s, float *ms_by_group) {
  return sampler_profile_groups(s, ms_by_group);
}

int flux_cuda_sampler_profile_launches(flux_cuda_sampler *s, float *ms, int *kernel_class, int capacity, int *count) {
  if (!s || !ms || !kernel_class || !count) return FLUX_CUDA_ERR_ARG;
  Workspace *ws = s->ws;
  int n = 0;
  for (size_t i = 0; i < ws->prof_used && n < capacity; ++i, ++n) {
    if (cudaEventElapsedTime(&ms[n], ws->prof_events[2 * i], ws->prof_events[2 * i + 1]) != cudaSuccess) {
      set_error("profile: events not complete (synchronize first)");
      return FLUX_CUDA_ERR_CUDA;
    }
    kernel_class[n] = ws->prof_class[i];
  }
  *count = n;
  return FLUX_CUDA_OK;
}

static int run_once(flux_cuda_model *m, int h, int w, const flux_cuda_ref *refs, int num_refs, const float *ctx,
                    const float *ctx_uncond, int txt_seq, const float *schedule, int num_steps, float guidance,
                    const float *z0, float *latent_out, float *velocities_out, int apply_update) {
  if (!m || !z0 || !ctx || !schedule || (num_refs > 0 && !refs)) {
    set_error("null argument");
    return FLUX_CUDA_ERR_ARG;
  }
  std::vector<RefSpec> rs;
  std::vector<const float *> lat;
  for (int i = 0; i < num_refs; ++i) {
    rs.push_back(RefSpec{refs[i].h, refs[i].w, refs[i].t_offset});
    lat.push_back(refs[i].latent);
  }
  flux_cuda_sampler *s = nullptr;
  int rc = sampler_create(m, h, w, txt_seq, rs.data(), num_refs, ctx_uncond ? 2 : 1, num_steps, &s);
  if (rc) return rc;
  s->ws->use_graphs = false;  // a one-shot sampler would pay the capture for a single replay
  rc = sampler_upload(s, z0, ctx, ctx_uncond, lat.data());
  if (!rc) rc = sampler_run(s, schedule, num_steps, 0, num_steps, guidance, velocities_out != nullptr, apply_update);
  if (!rc) rc = sampler_download(s, latent_out, velocities_out);
  else ctx_sync_check(m->ctx);
  sampler_free(s);
  return rc;
}

int flux_cuda_forward(flux_cuda_model *m, const float *z, int h, int w, const flux_cuda_ref *refs, int num_refs,
                      const float *ctx, int txt_seq, float timestep, float *v_out) {
  if (!v_out) return FLUX_CUDA_ERR_ARG;
  const float sched[2] = {timestep, timestep};
  return run_once(m, h, w, refs, num_refs, ctx, nullptr, txt_seq, sched, 1, 1.0f, z, nullptr, v_out, 0);
}

int flux_cuda_sample(flux_cuda_model *m, const flux_cuda_sample_params *p, const float *z0, float *latent_out,
                     float *velocities_out) {
  if (!p || !latent_out) return FLUX_CUDA_ERR_ARG;
  return run_once(m, p->h, p->w, p->refs, p->num_refs, p->ctx, p->ctx_uncond, p->txt_seq, p->schedule, p->num_steps,
                  p->guidance, z0, latent_out, velocities_out, 1);
}

}  // extern "C"
