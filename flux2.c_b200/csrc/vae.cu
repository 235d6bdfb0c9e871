// The VAE on the GPU: the decoder, the stage right after the denoising loop, and the encoder, which turns img2img
// reference images into latents before it. Replaces the reference's flux_vae_load_safetensors / flux_vae_decode /
// flux_vae_encode / flux_vae_free (flux_vae.c:1232-1386, 690-837, 320-440, 1034-1104) with the same tensor names and the
// same outputs (uint8 RGB [16h, 16w, 3]; latent f32 [128, H/16, W/16]).
//
// Layout in HBM: activations channels-last; the residual stream x is f32 [pixels, C], everything a convolution reads is
// 16-bit [pixels, C] (GroupNorm+swish output, upsampled tensor, attention operands); 3x3 weights are re-laid from the
// file's [Cout, Cin, 3, 3] f32 to 16-bit [Cout, 9, Cin] (tap-major) so that the convolution is one GEMM over K = 9 Cin
// (conv_tcgen05.cu). ResNet block: GN+swish -> conv1(+bias) -> GN+swish -> conv2(+bias) accumulated onto x in the
// convolution's epilogue; a 1x1 shortcut, where channels change, writes the new x first. Upsampling writes the 2x
// tensor once in 16 bits and the following convolution writes x. The single attention block (one head of 512
// channels over all latent pixels) is three GEMMs around a row softmax. The encoder mirrors this; its stride-2
// convolutions read the input as four parity planes written by one 16-bit conversion pass (conv.cuh).
#include <math.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#include <map>
#include <set>
#include <string>
#include <vector>

#include "context.cuh"
#include "conv.cuh"
#include "elementwise.cuh"
#include "engine.cuh"
#include "flux_cuda.h"
#include "launch.cuh"
#include "vae_kernels.cuh"

using namespace fx;

namespace {

struct ConvW {
  uint16_t *w = nullptr;  // [cout_pad, taps * cin_pad]
  float *b = nullptr;     // [cout_pad]
  int cin = 0, cout = 0, cin_pad = 0, cout_pad = 0, taps = 0;
};
struct ResW {
  float *g1 = nullptr, *b1 = nullptr, *g2 = nullptr, *b2 = nullptr;
  ConvW c1, c2, skip;
  int cin = 0, cout = 0;
};

struct AttnW {
  float *g = nullptr, *b = nullptr;
  ConvW qkv, out;
};

struct Slot {  // where a named tensor of the file goes
  enum Kind { CONV_W, CONV_B, VEC, QKV_W, QKV_B, PQ_W } kind;
  ConvW *conv;
  float *vec;
  int n;      // VEC: length; QKV_*: which third
};

}  // namespace

struct flux_cuda_vae {
  flux_cuda_ctx *ctx = nullptr;
  bool f16 = true;
  float eps = 1e-4f;  // flux_vae.c:1247: used by the GroupNorms and by the latent de-normalisation
  float *bn_mean = nullptr, *bn_var = nullptr, *pq_w = nullptr, *pq_b = nullptr;
  ConvW conv_in, conv_out, ups[3];
  AttnW attn;
  float *out_g = nullptr, *out_b = nullptr;
  ResW mid[2], up[12];
  // encoder half (optional: decoding works without it)
  ConvW e_conv_in, e_conv_out, e_down[3];
  AttnW e_attn;
  float *e_out_g = nullptr, *e_out_b = nullptr, *q_w = nullptr, *q_b = nullptr;  // quant_conv [64, 64], [64] in f32
  ResW e_mid[2], e_res[8];
  bool has_encoder = false;
  std::map<std::string, Slot> slots;
  std::set<std::string> seen, optional;
  std::vector<void *> allocs;
  bool finalized = false;
  // workspace, grown on demand
  size_t cap_elems = 0, cap_tok = 0;
  float *xa = nullptr, *xb = nullptr, *scores = nullptr, *stats = nullptr, *partial = nullptr, *lat = nullptr;
  float *img_in = nullptr;  // the encoder's input image [3, 16h, 16w]
  float *gnp = nullptr;     // GroupNorm partial sums written by the convolution epilogues
  bool fused_gn = true;     // FLUX_CUDA_VAE_FUSED_GN=0: statistics by a separate pass over the tensor
  uint16_t *a16 = nullptr, *h16 = nullptr, *qkv16 = nullptr, *vt16 = nullptr, *p16 = nullptr, *o16 = nullptr;
  unsigned int *counters = nullptr;
  uint8_t *img = nullptr;
  std::vector<void *> ws_allocs;
  long long launches = 0;
};

namespace {

template <typename T>
int v_alloc(flux_cuda_vae *v, std::vector<void *> &list, T **p, size_t count, bool zero = false) {
  void *q = nullptr;
  const size_t bytes = count * sizeof(T);
  cudaError_t e = cudaMalloc(&q, bytes ? bytes : 16);
  if (e != cudaSuccess) {
    set_error("cudaMalloc of %zu bytes failed: %s", bytes, cudaGetErrorString(e));
    return FLUX_CUDA_ERR_NOMEM;
  }
  list.push_back(q);
  if (zero) cudaMemsetAsync(q, 0, bytes ? bytes : 16, v->ctx->stream);
  *p = reinterpret_cast<T *>(q);
  return 0;
}

int make_conv(flux_cuda_vae *v, ConvW *c, int cin, int cout, int taps) {
  c->cin = cin;
  c->cout = cout;
  c->taps = taps;
  c->cin_pad = (cin + 63) / 64 * 64;
  c->cout_pad = (cout + 127) / 128 * 128;
  int rc = v_alloc(v, v->allocs, &c->w, static_cast<size_t>(c->cout_pad) * taps * c->cin_pad, true);
  if (!rc) rc = v_alloc(v, v->allocs, &c->b, c->cout_pad, true);
  return rc;
}

int make_vec(flux_cuda_vae *v, float **p, int n) { return v_alloc(v, v->allocs, p, n, true); }

void reg_conv(flux_cuda_vae *v, const std::string &prefix, ConvW *c) {
  v->slots[prefix + ".weight"] = Slot{Slot::CONV_W, c, nullptr, 0};
  v->slots[prefix + ".bias"] = Slot{Slot::CONV_B, c, nullptr, 0};
}
void reg_vec(flux_cuda_vae *v, const std::string &name, float *p, int n) { v->slots[name] = Slot{Slot::VEC, nullptr, p, n}; }

int make_res(flux_cuda_vae *v, ResW *r, const std::string &prefix, int cin, int cout) {
  r->cin = cin;
  r->cout = cout;
  int rc = make_vec(v, &r->g1, cin);
  if (!rc) rc = make_vec(v, &r->b1, cin);
  if (!rc) rc = make_vec(v, &r->g2, cout);
  if (!rc) rc = make_vec(v, &r->b2, cout);
  if (!rc) rc = make_conv(v, &r->c1, cin, cout, 9);
  if (!rc) rc = make_conv(v, &r->c2, cout, cout, 9);
  if (!rc && cin != cout) rc = make_conv(v, &r->skip, cin, cout, 1);
  if (rc) return rc;
  reg_vec(v, prefix + ".norm1.weight", r->g1, cin);
  reg_vec(v, prefix + ".norm1.bias", r->b1, cin);
  reg_vec(v, prefix + ".norm2.weight", r->g2, cout);
  reg_vec(v, prefix + ".norm2.bias", r->b2, cout);
  reg_conv(v, prefix + ".conv1", &r->c1);
  reg_conv(v, prefix + ".conv2", &r->c2);
  if (cin != cout) reg_conv(v, prefix + ".conv_shortcut", &r->skip);
  return 0;
}

int make_attn(flux_cuda_vae *v, AttnW *a, const std::string &prefix, int ch) {
  int rc = make_vec(v, &a->g, ch);
  if (!rc) rc = make_vec(v, &a->b, ch);
  if (!rc) rc = make_conv(v, &a->qkv, ch, 3 * ch, 1);
  if (!rc) rc = make_conv(v, &a->out, ch, ch, 1);
  if (rc) return rc;
  reg_vec(v, prefix + ".group_norm.weight", a->g, ch);
  reg_vec(v, prefix + ".group_norm.bias", a->b, ch);
  const char *qkv[3] = {"to_q", "to_k", "to_v"};
  for (int i = 0; i < 3; ++i) {
    v->slots[prefix + "." + qkv[i] + ".weight"] = Slot{Slot::QKV_W, &a->qkv, nullptr, i};
    v->slots[prefix + "." + qkv[i] + ".bias"] = Slot{Slot::QKV_B, &a->qkv, nullptr, i};
  }
  reg_conv(v, prefix + ".to_out.0", &a->out);
  return 0;
}

int ensure_workspace(flux_cuda_vae *v, int h, int w) {
  const size_t tok = static_cast<size_t>(4) * h * w;            // latent-resolution pixels (2h x 2w)
  const size_t elems = static_cast<size_t>(256) * h * w * 256;  // 16h x 16w pixels x 256 channels
  if (elems <= v->cap_elems && tok <= v->cap_tok) return 0;
  cudaStreamSynchronize(v->ctx->stream);
  for (void *p : v->ws_allocs) cudaFree(p);
  v->ws_allocs.clear();
  v->cap_elems = v->cap_tok = 0;
  const size_t tpad = (tok + 127) / 128 * 128;
  const size_t chunk = tok < 8192 ? tpad : 8192;
  int rc = v_alloc(v, v->ws_allocs, &v->xa, elems);
  if (!rc) rc = v_alloc(v, v->ws_allocs, &v->xb, elems);
  if (!rc) rc = v_alloc(v, v->ws_allocs, &v->a16, elems);
  if (!rc) rc = v_alloc(v, v->ws_allocs, &v->h16, elems);
  if (!rc) rc = v_alloc(v, v->ws_allocs, &v->qkv16, tpad * 1536, true);
  if (!rc) rc = v_alloc(v, v->ws_allocs, &v->vt16, static_cast<size_t>(512) * tpad, true);
  if (!rc) rc = v_alloc(v, v->ws_allocs, &v->o16, tpad * 512, true);
  if (!rc) rc = v_alloc(v, v->ws_allocs, &v->scores, chunk * tpad);
  if (!rc) rc = v_alloc(v, v->ws_allocs, &v->p16, chunk * tpad, true);
  if (!rc) rc = v_alloc(v, v->ws_allocs, &v->lat, static_cast<size_t>(128) * h * w);
  if (!rc) rc = v_alloc(v, v->ws_allocs, &v->img, static_cast<size_t>(256) * h * w * 3);
  if (!rc && v->has_encoder) rc = v_alloc(v, v->ws_allocs, &v->img_in, static_cast<size_t>(256) * h * w * 3);
  if (!rc) rc = v_alloc(v, v->ws_allocs, &v->gnp, static_cast<size_t>(512) * h * w + 8192);
  if (!rc) rc = v_alloc(v, v->ws_allocs, &v->stats, GN_GROUPS * 2);
  if (!rc) rc = v_alloc(v, v->ws_allocs, &v->partial, static_cast<size_t>(GN_MAX_BLOCKS) * 64);
  if (!rc) rc = v_alloc(v, v->ws_allocs, &v->counters, 4, true);
  if (rc) return rc;
  v->cap_elems = elems;
  v->cap_tok = tok;
  return 0;
}

struct Runner {
  flux_cuda_vae *v;
  cudaStream_t st;
  int f16, sms;
  int rc = 0;
  // statistics of the tensor the last convolution wrote, still to be folded (gn_next launches)
  bool pending = false;
  ConvParams lastP;
  long long last_pixels = 0;

  void note(int r) {
    ++v->launches;
    if (r && !rc) rc = r;
  }
  // gn_next: the tensor written is normalised by a GroupNorm next, so the epilogue also leaves its statistics
  void conv3(const ConvW &c, const void *in16, int H, int W, int mode, void *out, long long ld, bool gn_next = false) {
    if (rc) return;
    ConvParams P;
    memset(&P, 0, sizeof(P));
    int r = conv_make_3x3(&P, in16, 1, H, W, c.cin_pad, c.w, c.cout_pad);
    if (r) return note(r);
    finish(P, c, mode, out, ld, gn_next);
  }
  void conv3_s2(const ConvW &c, const void *planes16, int Ho, int Wo, int mode, void *out, long long ld,
                bool gn_next = false) {
    if (rc) return;
    ConvParams P;
    memset(&P, 0, sizeof(P));
    int r = conv_make_3x3_s2(&P, planes16, 1, Ho, Wo, c.cin_pad, c.w, c.cout_pad);
    if (r) return note(r);
    finish(P, c, mode, out, ld, gn_next);
  }
  void gemm(const ConvW &c, const void *in16, long long ldx, long long M, int mode, void *out, long long ld,
            bool gn_next = false) {
    if (rc) return;
    ConvParams P;
    memset(&P, 0, sizeof(P));
    int r = conv_make_gemm(&P, in16, ldx, c.w, c.cin_pad, static_cast<int>(M), c.cout_pad, c.cin_pad, c.cout_pad);
    if (r) return note(r);
    finish(P, c, mode, out, ld, gn_next);
  }
  void finish(ConvParams &P, const ConvW &c, int mode, void *out, long long ld, bool gn_next = false) {
    P.mode = mode;
    P.out = out;
    P.ld = ld;
    P.bias = c.b;
    P.out_f16 = f16;
    P.x_f16 = f16;
    P.err = v->ctx->err_dev;
    const int cpg = c.cout / GN_GROUPS;
    pending = false;
    if (gn_next && v->fused_gn && c.cout == c.cout_pad && c.cout == cpg * GN_GROUPS && (cpg == 4 || cpg == 8 || cpg == 16)) {
      P.gn_partial = v->gnp;
      P.gn_cpg = cpg;
      pending = true;
      lastP = P;
      last_pixels = P.M;
    }
    note(conv_launch(&P, sms, st));
  }
  void gn(const void *x, int in16, long long pixels, int C, const float *g, const float *b, int swish, void *out16) {
    if (rc) return;
    if (pending && last_pixels == pixels && lastP.Cout == C)
      note(conv_gn_finalize(lastP, pixels, v->eps, v->stats, st));
    else
      note(launch_gn_stats(x, in16, f16, 1, pixels, C, v->eps, v->partial, v->counters, v->stats, st));
    pending = false;
    if (rc) return;
    note(launch_gn_apply(x, in16, out16, f16, 1, pixels, C, v->stats, g, b, swish, st));
  }
  // Attention over T pixels, one head of 512 channels (flux_vae.c:223-314): x += out(softmax(q k^T / sqrt(512)) v)
  void attention(const AttnW &a, float *x, long long T) {
    const long long tpad = (T + 127) / 128 * 128;
    gn(x, 0, T, 512, a.g, a.b, 0, v->a16);
    gemm(a.qkv, v->a16, 512, T, CONV_STORE_16, v->qkv16, 1536);
    if (!rc) note(check_cuda(cudaMemsetAsync(v->vt16, 0, static_cast<size_t>(512) * tpad * 2, st), "clear") ? -8 : 0);
    if (!rc) note(launch_transpose16(v->qkv16 + 1024, 1536, v->vt16, tpad, static_cast<int>(T), 512, st));
    const long long chunk = T < 8192 ? tpad : 8192;
    ConvW none;
    for (long long r0 = 0; r0 < T && !rc; r0 += chunk) {
      const long long rows = T - r0 < chunk ? T - r0 : chunk;
      ConvParams P;
      memset(&P, 0, sizeof(P));
      // scores[rows, tpad] = Q[r0.., :] K^T; key rows beyond T are read as zeros by the tensor map
      int r = conv_make_gemm(&P, v->qkv16 + r0 * 1536, 1536, v->qkv16 + 512, 1536, static_cast<int>(rows),
                             static_cast<int>(tpad), 512, static_cast<int>(T));
      if (r) return note(r);
      finish(P, none, CONV_STORE_F32, v->scores, tpad);
      if (!rc)
        note(launch_softmax_rows(v->scores, v->p16, f16, rows, static_cast<int>(T), static_cast<int>(tpad),
                                 1.0f / sqrtf(512.0f), st));
      memset(&P, 0, sizeof(P));
      r = conv_make_gemm(&P, v->p16, tpad, v->vt16, tpad, static_cast<int>(rows), 512, static_cast<int>(tpad), 512);
      if (r) return note(r);
      finish(P, none, CONV_STORE_16, v->o16 + r0 * 512, 512);
    }
    gemm(a.out, v->o16, 512, T, CONV_ADD_F32, x, 512, true);
  }
  // x (f32 [P, cin]) -> x (f32 [P, cout]); returns the buffer that holds the result
  float *res(const ResW &r, float *x, float *other, int H, int W) {
    const long long P = static_cast<long long>(H) * W;
    gn(x, 0, P, r.cin, r.g1, r.b1, 1, v->a16);
    conv3(r.c1, v->a16, H, W, CONV_STORE_16, v->h16, r.cout, true);
    gn(v->h16, 1, P, r.cout, r.g2, r.b2, 1, v->a16);
    if (r.cin != r.cout) {
      if (!rc) note(launch_f32_to_bf16(x, v->h16, P * r.cin, f16, st));
      gemm(r.skip, v->h16, r.cin, P, CONV_STORE_F32, other, r.cout);
      x = other;
    }
    conv3(r.c2, v->a16, H, W, CONV_ADD_F32, x, r.cout, true);
    return x;
  }
};

}  // namespace

extern "C" {

void flux_cuda_vae_free(flux_cuda_vae *v) {
  if (!v) return;
  cudaSetDevice(v->ctx->device);
  cudaStreamSynchronize(v->ctx->stream);
  for (void *p : v->allocs) cudaFree(p);
  for (void *p : v->ws_allocs) cudaFree(p);
  delete v;
}

int flux_cuda_vae_create(flux_cuda_ctx *ctx, flux_cuda_vae **out) {
  if (!ctx || !out) return FLUX_CUDA_ERR_ARG;
  *out = nullptr;
  cudaSetDevice(ctx->device);
  if (conv_init() != 0) {
    set_error("convolution kernels could not be initialised");
    return FLUX_CUDA_ERR_CUDA;
  }
  flux_cuda_vae *v = new flux_cuda_vae();
  v->ctx = ctx;
  v->f16 = ctx->f16;
  if (const char *e = getenv("FLUX_CUDA_VAE_FUSED_GN")) v->fused_gn = atoi(e) != 0;
  const int base = 128, mult[4] = {1, 2, 4, 4}, mid = base * mult[3];
  int rc = make_vec(v, &v->bn_mean, 128);
  if (!rc) rc = make_vec(v, &v->bn_var, 128);
  if (!rc) rc = make_vec(v, &v->pq_w, 32 * 32);
  if (!rc) rc = make_vec(v, &v->pq_b, 32);
  if (!rc) rc = make_conv(v, &v->conv_in, 32, mid, 9);
  if (!rc) rc = make_res(v, &v->mid[0], "decoder.mid_block.resnets.0", mid, mid);
  if (!rc) rc = make_res(v, &v->mid[1], "decoder.mid_block.resnets.1", mid, mid);
  if (!rc) rc = make_attn(v, &v->attn, "decoder.mid_block.attentions.0", mid);
  int bi = 0;
  for (int level = 3; !rc && level >= 0; --level) {  // flux_vae.c:1322-1334: up_blocks.0 is the deepest level
    const int ch = base * mult[level], prev = level == 3 ? mid : base * mult[level + 1];
    for (int r = 0; !rc && r < 3; ++r) {
      char name[96];
      snprintf(name, sizeof(name), "decoder.up_blocks.%d.resnets.%d", 3 - level, r);
      rc = make_res(v, &v->up[bi++], name, r == 0 ? prev : ch, ch);
    }
  }
  for (int i = 0; !rc && i < 3; ++i) {
    const int ch = base * mult[3 - i];
    rc = make_conv(v, &v->ups[i], ch, ch, 9);
    char name[96];
    snprintf(name, sizeof(name), "decoder.up_blocks.%d.upsamplers.0.conv", i);
    if (!rc) reg_conv(v, name, &v->ups[i]);
  }
  if (!rc) rc = make_vec(v, &v->out_g, base);
  if (!rc) rc = make_vec(v, &v->out_b, base);
  if (!rc) rc = make_conv(v, &v->conv_out, base, 3, 9);
  // encoder half (flux_vae.c:1255-1300)
  const size_t dec_slots = v->slots.size();
  if (!rc) rc = make_conv(v, &v->e_conv_in, 3, base, 9);
  int ei = 0;
  for (int level = 0; !rc && level < 4; ++level) {
    const int ch = base * mult[level], prev = level == 0 ? base : base * mult[level - 1];
    for (int r = 0; !rc && r < 2; ++r) {
      char name[96];
      snprintf(name, sizeof(name), "encoder.down_blocks.%d.resnets.%d", level, r);
      rc = make_res(v, &v->e_res[ei++], name, (r == 0 && level > 0) ? prev : ch, ch);
    }
    if (!rc && level < 3) {
      rc = make_conv(v, &v->e_down[level], ch, ch, 9);
      char name[96];
      snprintf(name, sizeof(name), "encoder.down_blocks.%d.downsamplers.0.conv", level);
      if (!rc) reg_conv(v, name, &v->e_down[level]);
    }
  }
  if (!rc) rc = make_res(v, &v->e_mid[0], "encoder.mid_block.resnets.0", mid, mid);
  if (!rc) rc = make_res(v, &v->e_mid[1], "encoder.mid_block.resnets.1", mid, mid);
  if (!rc) rc = make_attn(v, &v->e_attn, "encoder.mid_block.attentions.0", mid);
  if (!rc) rc = make_vec(v, &v->e_out_g, mid);
  if (!rc) rc = make_vec(v, &v->e_out_b, mid);
  if (!rc) rc = make_conv(v, &v->e_conv_out, mid, 64, 9);
  if (!rc) rc = make_vec(v, &v->q_w, 64 * 64);
  if (!rc) rc = make_vec(v, &v->q_b, 64);
  if (rc) {
    flux_cuda_vae_free(v);
    return rc;
  }
  reg_conv(v, "encoder.conv_in", &v->e_conv_in);
  reg_conv(v, "encoder.conv_out", &v->e_conv_out);
  reg_vec(v, "encoder.conv_norm_out.weight", v->e_out_g, mid);
  reg_vec(v, "encoder.conv_norm_out.bias", v->e_out_b, mid);
  v->slots["quant_conv.weight"] = Slot{Slot::PQ_W, nullptr, v->q_w, 64 * 64};
  reg_vec(v, "quant_conv.bias", v->q_b, 64);
  (void)dec_slots;
  reg_conv(v, "decoder.conv_in", &v->conv_in);
  reg_conv(v, "decoder.conv_out", &v->conv_out);
  reg_vec(v, "decoder.conv_norm_out.weight", v->out_g, base);
  reg_vec(v, "decoder.conv_norm_out.bias", v->out_b, base);
  v->slots["post_quant_conv.weight"] = Slot{Slot::PQ_W, nullptr, v->pq_w, 32 * 32};
  reg_vec(v, "post_quant_conv.bias", v->pq_b, 32);
  reg_vec(v, "bn.running_mean", v->bn_mean, 128);
  reg_vec(v, "bn.running_var", v->bn_var, 128);
  v->optional = {"bn.running_mean", "bn.running_var"};  // absent: mean 0, variance 1 (flux_vae.c:1352-1358)
  std::vector<float> ones(128, 1.0f);
  rc = check_cuda(upload_h2d(ctx->stream, v->bn_var, ones.data(), 128 * 4), "upload");
  if (rc) {
    flux_cuda_vae_free(v);
    return rc;
  }
  *out = v;
  return FLUX_CUDA_OK;
}

int flux_cuda_vae_set_tensor(flux_cuda_vae *v, const char *name, const void *data, int dtype, const long long *shape,
                             int ndim) {
  if (!v || !name || !data || !shape || dtype < 0 || dtype > 2 || ndim < 1 || ndim > 4) {
    set_error("vae set_tensor: bad argument");
    return FLUX_CUDA_ERR_ARG;
  }
  cudaSetDevice(v->ctx->device);
  const std::string n(name);
  auto it = v->slots.find(n);
  if (it == v->slots.end()) {
    if (n.rfind("encoder.", 0) == 0 || n.rfind("quant_conv.", 0) == 0) return FLUX_CUDA_OK;  // not used by decoding
    set_error("unknown VAE tensor %s", name);
    return FLUX_CUDA_ERR_MODEL;
  }
  size_t count = 1;
  for (int i = 0; i < ndim; ++i) count *= static_cast<size_t>(shape[i]);
  const Slot &s = it->second;
  auto f32_at = [&](size_t i) {
    return dtype == 0 ? reinterpret_cast<const float *>(data)[i]
                      : half_to_f32_host(reinterpret_cast<const uint16_t *>(data)[i], dtype);
  };
  auto bad_shape = [&](size_t want) {
    set_error("VAE tensor %s has %zu elements, expected %zu", name, count, want);
    return FLUX_CUDA_ERR_MODEL;
  };
  int rc = 0;
  cudaStream_t st = v->ctx->stream;
  switch (s.kind) {
    case Slot::VEC:
    case Slot::PQ_W: {
      if (count != static_cast<size_t>(s.n)) return bad_shape(s.n);
      std::vector<float> tmp(count);
      for (size_t i = 0; i < count; ++i) tmp[i] = f32_at(i);
      rc = check_cuda(upload_h2d(st, s.vec, tmp.data(), count * 4), "upload VAE vector");
    } break;
    case Slot::CONV_B:
    case Slot::QKV_B: {
      const ConvW &c = *s.conv;
      const size_t want = s.kind == Slot::QKV_B ? c.cout / 3 : c.cout;
      if (count != want) return bad_shape(want);
      std::vector<float> tmp(count);
      for (size_t i = 0; i < count; ++i) tmp[i] = f32_at(i);
      rc = check_cuda(upload_h2d(st, c.b + (s.kind == Slot::QKV_B ? s.n * want : 0), tmp.data(), count * 4),
                      "upload VAE bias");
    } break;
    case Slot::CONV_W:
    case Slot::QKV_W: {
      const ConvW &c = *s.conv;
      const int rows = s.kind == Slot::QKV_W ? c.cout / 3 : c.cout;
      const size_t want = static_cast<size_t>(rows) * c.cin * c.taps;
      if (count != want || shape[0] != rows) return bad_shape(want);
      std::vector<uint16_t> tmp;
      const uint16_t *src = to_half_host(data, dtype, count, tmp, v->f16);
      // file: [co][ci][tap]  ->  device: [co][tap][ci_pad], zero in the padding
      std::vector<uint16_t> re(static_cast<size_t>(rows) * c.taps * c.cin_pad, 0);
      for (int co = 0; co < rows; ++co)
        for (int ci = 0; ci < c.cin; ++ci)
          for (int t = 0; t < c.taps; ++t)
            re[(static_cast<size_t>(co) * c.taps + t) * c.cin_pad + ci] = src[(static_cast<size_t>(co) * c.cin + ci) * c.taps + t];
      uint16_t *dst = c.w + (s.kind == Slot::QKV_W ? static_cast<size_t>(s.n) * rows * c.taps * c.cin_pad : 0);
      rc = check_cuda(upload_h2d(st, dst, re.data(), re.size() * 2), "upload VAE weights");
    } break;
  }
  if (!rc) v->seen.insert(n);
  return rc;
}

int flux_cuda_vae_finalize(flux_cuda_vae *v) {
  if (!v) return FLUX_CUDA_ERR_ARG;
  bool enc_all = true, enc_any = false;
  std::string enc_missing;
  for (const auto &kv : v->slots) {
    const bool is_enc = kv.first.rfind("encoder.", 0) == 0 || kv.first.rfind("quant_conv.", 0) == 0;
    const bool have = v->seen.count(kv.first) != 0;
    if (is_enc) {
      enc_any |= have;
      if (!have) {
        enc_all = false;
        if (enc_missing.empty()) enc_missing = kv.first;
      }
    } else if (!have && !v->optional.count(kv.first)) {
      set_error("VAE incomplete: tensor %s was not provided", kv.first.c_str());
      return FLUX_CUDA_ERR_MODEL;
    }
  }
  if (enc_any && !enc_all) {  // a file with half an encoder is a broken file, not a decoder-only file
    set_error("VAE incomplete: encoder tensor %s was not provided", enc_missing.c_str());
    return FLUX_CUDA_ERR_MODEL;
  }
  v->has_encoder = enc_all;
  v->finalized = true;
  return FLUX_CUDA_OK;
}

int flux_cuda_vae_load_safetensors(flux_cuda_ctx *ctx, const char *path, flux_cuda_vae **out) {
  if (!ctx || !path || !out) return FLUX_CUDA_ERR_ARG;
  *out = nullptr;
  flux_cuda_vae *v = nullptr;
  int rc = flux_cuda_vae_create(ctx, &v);
  if (rc) return rc;
  rc = safetensors_for_each(path, [&](const char *name, const void *data, int dt, const long long *shape, int nd) {
    return flux_cuda_vae_set_tensor(v, name, data, dt, shape, nd);
  });
  if (!rc) rc = flux_cuda_vae_finalize(v);
  if (rc) {
    flux_cuda_vae_free(v);
    return rc;
  }
  *out = v;
  return FLUX_CUDA_OK;
}

// Queues the whole decoder on the context's stream: latent (host or device, f32 [128, h, w]) -> v->img (device).
static int vae_enqueue(flux_cuda_vae *v, const float *latent, int h, int w) {
  if (!v || !latent || h < 1 || w < 1) {
    set_error("vae_decode: bad argument");
    return FLUX_CUDA_ERR_ARG;
  }
  if (!v->finalized) {
    set_error("vae_decode: model is not finalized");
    return FLUX_CUDA_ERR_MODEL;
  }
  cudaSetDevice(v->ctx->device);
  int rc = ensure_workspace(v, h, w);
  if (rc) return rc;
  cudaStream_t st = v->ctx->stream;
  rc = check_cuda(cudaMemcpyAsync(v->lat, latent, static_cast<size_t>(128) * h * w * 4, cudaMemcpyDefault, st), "upload latent");
  if (rc) return rc;
  // Plain stream-ordered launches for the VAE: with programmatic dependent launch, repeated back-to-back decodes
  // whose GroupNorm statistics come from the convolution epilogue stopped making progress on the device in roughly
  // one run out of three (never without it, never with the separate statistics pass); the overlap it buys here is
  // below 1 % of a decode.
  PdlOff no_pdl;
  Runner R{v, st, v->f16 ? 1 : 0, v->ctx->num_sms};
  v->launches = 0;
  int H = 2 * h, W = 2 * w;
  const long long T = static_cast<long long>(H) * W;
  R.note(launch_vae_prologue(v->lat, v->a16, 1, h, w, v->bn_mean, v->bn_var, v->eps, v->pq_w, v->pq_b, R.f16, st));
  float *x = v->xa, *other = v->xb;
  auto swap_to = [&](float *now) {
    if (now != x) {
      other = x;
      x = now;
    }
  };
  R.conv3(v->conv_in, v->a16, H, W, CONV_STORE_F32, x, 512, true);
  swap_to(R.res(v->mid[0], x, other, H, W));
  R.attention(v->attn, x, T);
  swap_to(R.res(v->mid[1], x, other, H, W));
  int bi = 0;
  for (int level = 3; level >= 0; --level) {
    for (int r = 0; r < 3; ++r) swap_to(R.res(v->up[bi++], x, other, H, W));
    if (level > 0) {
      const ConvW &c = v->ups[3 - level];
      if (!R.rc) R.note(launch_upsample2x(x, v->a16, R.f16, 1, H, W, c.cin, st));
      H *= 2;
      W *= 2;
      R.conv3(c, v->a16, H, W, CONV_STORE_F32, x, c.cout, true);
    }
  }
  R.gn(x, 0, static_cast<long long>(H) * W, 128, v->out_g, v->out_b, 1, v->a16);
  R.conv3(v->conv_out, v->a16, H, W, CONV_STORE_RGB8, v->img, 3);
  if (R.rc) {
    set_error("vae_decode: kernel launch failed (rc %d, cuda: %s)", R.rc, cudaGetErrorString(cudaGetLastError()));
    ctx_sync_check(v->ctx);
    return R.rc == -1 || R.rc == -5 ? FLUX_CUDA_ERR_ARG : FLUX_CUDA_ERR_CUDA;
  }
  return FLUX_CUDA_OK;
}

// Queues the whole encoder: image f32 [3, H, W] (host or device; H, W multiples of 16) -> v->lat (device, f32
// [128, H/16, W/16]).
static int vae_encode_enqueue(flux_cuda_vae *v, const float *image, int H, int W) {
  if (!v || !image || H < 16 || W < 16 || (H % 16) || (W % 16)) {
    set_error("vae_encode: bad argument (image sides must be multiples of 16)");
    return FLUX_CUDA_ERR_ARG;
  }
  if (!v->finalized || !v->has_encoder) {
    set_error("vae_encode: the encoder tensors were not loaded");
    return FLUX_CUDA_ERR_MODEL;
  }
  cudaSetDevice(v->ctx->device);
  const int h = H / 16, w = W / 16;
  if (!v->img_in) {  // the workspace was sized before the encoder was known to be needed
    v->cap_elems = 0;
  }
  int rc = ensure_workspace(v, h, w);
  if (rc) return rc;
  cudaStream_t st = v->ctx->stream;
  rc = check_cuda(cudaMemcpyAsync(v->img_in, image, static_cast<size_t>(3) * H * W * 4, cudaMemcpyDefault, st), "upload image");
  if (rc) return rc;
  PdlOff no_pdl;  // see vae_enqueue
  Runner R{v, st, v->f16 ? 1 : 0, v->ctx->num_sms};
  v->launches = 0;
  R.note(launch_image_to_nhwc(v->img_in, v->a16, R.f16, H, W, st));
  float *x = v->xa, *other = v->xb;
  auto swap_to = [&](float *now) {
    if (now != x) {
      other = x;
      x = now;
    }
  };
  R.conv3(v->e_conv_in, v->a16, H, W, CONV_STORE_F32, x, 128, true);
  int ei = 0;
  for (int level = 0; level < 4; ++level) {
    for (int r = 0; r < 2; ++r) swap_to(R.res(v->e_res[ei++], x, other, H, W));
    if (level < 3) {
      const ConvW &c = v->e_down[level];
      if (!R.rc) R.note(launch_parity_planes(x, v->a16, R.f16, 1, H, W, c.cin, st));
      H /= 2;
      W /= 2;
      R.conv3_s2(c, v->a16, H, W, CONV_STORE_F32, x, c.cout, true);
    }
  }
  const long long T = static_cast<long long>(H) * W;
  swap_to(R.res(v->e_mid[0], x, other, H, W));
  R.attention(v->e_attn, x, T);
  swap_to(R.res(v->e_mid[1], x, other, H, W));
  R.gn(x, 0, T, 512, v->e_out_g, v->e_out_b, 1, v->a16);
  R.conv3(v->e_conv_out, v->a16, H, W, CONV_STORE_F32, other, 128);  // 64 channels of 128 columns are real
  if (!R.rc)
    R.note(launch_vae_encode_tail(other, 128, v->lat, H, W, v->q_w, v->q_b, v->bn_mean, v->bn_var, v->eps, st));
  if (R.rc) {
    set_error("vae_encode: kernel launch failed (rc %d, cuda: %s)", R.rc, cudaGetErrorString(cudaGetLastError()));
    ctx_sync_check(v->ctx);
    return R.rc == -1 || R.rc == -5 ? FLUX_CUDA_ERR_ARG : FLUX_CUDA_ERR_CUDA;
  }
  return FLUX_CUDA_OK;
}

int flux_cuda_vae_encode(flux_cuda_vae *v, const float *image, int H, int W, float *latent_out) {
  if (!latent_out) {
    set_error("vae_encode: bad argument");
    return FLUX_CUDA_ERR_ARG;
  }
  int rc = vae_encode_enqueue(v, image, H, W);
  if (rc) return rc;
  rc = check_cuda(cudaMemcpyAsync(latent_out, v->lat, static_cast<size_t>(128) * (H / 16) * (W / 16) * 4,
                                  cudaMemcpyDeviceToHost, v->ctx->stream),
                  "download latent");
  if (!rc) rc = ctx_sync_check(v->ctx);
  return rc;
}

int flux_cuda_vae_has_encoder(const flux_cuda_vae *v) { return v && v->has_encoder ? 1 : 0; }

int flux_cuda_vae_decode(flux_cuda_vae *v, const float *latent, int h, int w, unsigned char *rgb_out) {
  if (!rgb_out) {
    set_error("vae_decode: bad argument");
    return FLUX_CUDA_ERR_ARG;
  }
  int rc = vae_enqueue(v, latent, h, w);
  if (rc) return rc;
  rc = check_cuda(cudaMemcpyAsync(rgb_out, v->img, static_cast<size_t>(256) * h * w * 3, cudaMemcpyDeviceToHost, v->ctx->stream),
                  "download image");
  if (!rc) rc = ctx_sync_check(v->ctx);
  return rc;
}

int flux_cuda_vae_decode_device(flux_cuda_vae *v, const float *latent, int h, int w, const unsigned char **rgb_dev) {
  if (!rgb_dev) {
    set_error("vae_decode_device: bad argument");
    return FLUX_CUDA_ERR_ARG;
  }
  *rgb_dev = nullptr;
  int rc = vae_enqueue(v, latent, h, w);
  if (rc) return rc;
  *rgb_dev = v->img;
  return FLUX_CUDA_OK;
}

long long flux_cuda_vae_last_launches(const flux_cuda_vae *v) { return v ? v->launches : 0; }

}  // extern "C"
