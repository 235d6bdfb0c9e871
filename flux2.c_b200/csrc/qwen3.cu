// The Qwen3 text encoder on the GPU: the stage right before the denoising loop. Replaces the reference's
// qwen3_model_load / qwen3_forward / qwen3_model_free (flux_qwen3.c:1329-1430, 1041-1156, 1529-1590) with the same
// tensor names and the same output (hidden states after layers 8, 17 and 26 concatenated, f32 [seq, 3 * hidden]).
// It reuses the DiT's kernels: the tcgen05 GEMM (fused Q|K|V projection with per-head RMSNorm and half-split RoPE in
// the epilogue, SwiGLU epilogue, residual-add epilogue) and the attention kernel in its grouped-query, causal,
// key-masked mode. Only the layers the output depends on are kept and run (27 of 36; the reference's CPU path runs
// all 36, its GPU path stops at the same layer).
#include <math.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#include <set>
#include <string>
#include <vector>

#include "attention.cuh"
#include "context.cuh"
#include "elementwise.cuh"
#include "engine.cuh"
#include "flux_cuda.h"
#include "gemm.cuh"
#include "launch.cuh"
#include "ptx.cuh"

#include <cuda_fp16.h>

namespace fx {

// ------------------------------------------------------------------------------------------------ kernels
// hidden[s, :] = embed[ids[s], :] as f32; ids outside the vocabulary give a zero row (flux_qwen3.c:1047-1057).
__global__ void embed_gather_kernel(const uint16_t *__restrict__ table, const int *__restrict__ ids,
                                    float *__restrict__ out, int hidden, int vocab, int f16) {
  const int s = blockIdx.x;
  const int tok = ids[s];
  const bool ok = tok >= 0 && tok < vocab;
  const uint16_t *row = table + static_cast<size_t>(ok ? tok : 0) * hidden;
  for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
    float v = 0.f;
    if (ok) v = f16 ? __half2float(__ushort_as_half(row[i])) : __uint_as_float(static_cast<uint32_t>(row[i]) << 16);
    out[static_cast<size_t>(s) * hidden + i] = v;
  }
}

// RMSNorm: out_16[r, :] = x[r, :] * rsqrt(mean(x^2) + 1e-6) * w (qwen3_rms_norm, flux_qwen3.c:176-196).
// One warp per row, the row stays in registers between the two passes. With nsplit > 0 the row first receives the
// partial products of the preceding split-K projection, x[r, :] += sum_s part[s][r, :] (in ascending s, so the
// result does not depend on scheduling), and is written back: the residual add of that projection. out == nullptr
// stops after the add.
template <int VPL>
__global__ void __launch_bounds__(128, 3) rmsnorm_kernel(float *__restrict__ x, uint16_t *__restrict__ out,
                                                         const float *__restrict__ w, int rows, int hidden, int f16,
                                                         const float *__restrict__ part, int nsplit, long long pstride) {
  pdl_launch_dependents();
  pdl_wait();
  const int row = blockIdx.x * 4 + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (row >= rows) return;
  float4 *xr = reinterpret_cast<float4 *>(x + static_cast<size_t>(row) * hidden);
  float4 v[VPL];
  float ss = 0.f;
#pragma unroll
  for (int i = 0; i < VPL; ++i) v[i] = xr[i * 32 + lane];
  if (nsplit > 0) {
    for (int s = 0; s < nsplit; ++s) {
      const float4 *pr = reinterpret_cast<const float4 *>(part + s * pstride + static_cast<size_t>(row) * hidden);
#pragma unroll
      for (int i = 0; i < VPL; ++i) {
        const float4 a = pr[i * 32 + lane];
        v[i].x += a.x;
        v[i].y += a.y;
        v[i].z += a.z;
        v[i].w += a.w;
      }
    }
#pragma unroll
    for (int i = 0; i < VPL; ++i) xr[i * 32 + lane] = v[i];
    if (!out) return;
  }
#pragma unroll
  for (int i = 0; i < VPL; ++i) ss += (v[i].x * v[i].x + v[i].y * v[i].y) + (v[i].z * v[i].z + v[i].w * v[i].w);
  const float rinv = rsqrtf(warp_sum(ss) / static_cast<float>(hidden) + 1e-6f);
  const float4 *w4 = reinterpret_cast<const float4 *>(w);
  uint2 *o2 = reinterpret_cast<uint2 *>(out + static_cast<size_t>(row) * hidden);
#pragma unroll
  for (int i = 0; i < VPL; ++i) {
    const float4 ww = __ldg(w4 + i * 32 + lane);
    o2[i * 32 + lane] = make_uint2(pack_16x2(v[i].x * rinv * ww.x, v[i].y * rinv * ww.y, f16 != 0),
                                   pack_16x2(v[i].z * rinv * ww.z, v[i].w * rinv * ww.w, f16 != 0));
  }
}

static int launch_rmsnorm(float *x, void *out, const float *w, int rows, int hidden, int f16, const float *part,
                          int nsplit, long long pstride, cudaStream_t st) {
  const dim3 grid((rows + 3) / 4), block(128);
  uint16_t *o = reinterpret_cast<uint16_t *>(out);
  cudaError_t e;
  // Plain stream order: this small grid always follows a paired (cluster) GEMM, and a small grid launched with
  // programmatic dependent launch directly behind such a kernel is the one pattern a device stall was traced to.
  PdlOff plain_launch;
#define RMS_LAUNCH(V) launch_kernel(rmsnorm_kernel<V>, grid, block, 0, st, 1, x, o, w, rows, hidden, f16, part, nsplit, pstride)
  switch (hidden) {
    case 2560: e = RMS_LAUNCH(20); break;
    case 256: e = RMS_LAUNCH(2); break;
    case 512: e = RMS_LAUNCH(4); break;
    case 1024: e = RMS_LAUNCH(8); break;
    default: return -1;
  }
#undef RMS_LAUNCH
  return e == cudaSuccess ? 0 : -8;
}

}  // namespace fx

using namespace fx;

// ------------------------------------------------------------------------------------------------ model
struct QwenLayer {
  uint16_t *qkv = nullptr, *o = nullptr, *gateup = nullptr, *down = nullptr;
  float *ln1 = nullptr, *ln2 = nullptr, *qn = nullptr, *kn = nullptr;
};

struct flux_cuda_qwen3 {
  flux_cuda_ctx *ctx = nullptr;
  flux_cuda_qwen3_dims d{};
  bool f16 = true;
  int run_layers = 0, max_seq = 0;
  uint16_t *embed = nullptr;
  std::vector<QwenLayer> layers;
  std::vector<void *> allocs;
  void *staging = nullptr;
  size_t staging_bytes = 0;
  std::set<std::string> seen;
  size_t expected = 0;
  bool finalized = false;
  // workspace for max_seq tokens
  float *hidden = nullptr, *out = nullptr, *ones = nullptr, *cos_t = nullptr, *sin_t = nullptr, *ang_t = nullptr, *part = nullptr;
  bool split_k = true;  // FLUX_CUDA_QWEN_SPLITK=0: every projection as one problem
  uint16_t *norm = nullptr, *qkv = nullptr, *attn = nullptr, *act = nullptr;
  int *ids = nullptr;
  uint32_t *mask = nullptr;
};

template <typename T>
static int q_alloc(flux_cuda_qwen3 *m, T **p, size_t count) {
  void *q = nullptr;
  const size_t bytes = count * sizeof(T);
  cudaError_t e = cudaMalloc(&q, bytes > 0 ? bytes : 16);
  if (e != cudaSuccess) {
    set_error("cudaMalloc of %zu bytes failed: %s", count * sizeof(T), cudaGetErrorString(e));
    return FLUX_CUDA_ERR_NOMEM;
  }
  m->allocs.push_back(q);
  *p = reinterpret_cast<T *>(q);
  return 0;
}

extern "C" {

void flux_cuda_qwen3_dims_4b(flux_cuda_qwen3_dims *d) {
  if (!d) return;
  d->hidden = 2560;
  d->heads = 32;
  d->kv_heads = 8;
  d->head_dim = 128;
  d->inter = 9728;
  d->layers = 36;
  d->vocab = 151936;
  d->rope_theta = 1000000.0f;
  d->out_layers[0] = 8;
  d->out_layers[1] = 17;
  d->out_layers[2] = 26;
}

void flux_cuda_qwen3_free(flux_cuda_qwen3 *m) {
  if (!m) return;
  cudaSetDevice(m->ctx->device);
  cudaStreamSynchronize(m->ctx->stream);
  for (void *p : m->allocs) cudaFree(p);
  delete m;
}

int flux_cuda_qwen3_create(flux_cuda_ctx *ctx, const flux_cuda_qwen3_dims *dims, int max_seq, flux_cuda_qwen3 **out) {
  if (!ctx || !dims || !out) return FLUX_CUDA_ERR_ARG;
  *out = nullptr;
  const flux_cuda_qwen3_dims &d = *dims;
  const int qkv_n = (d.heads + 2 * d.kv_heads) * d.head_dim;
  if (d.head_dim != 128 || d.heads % d.kv_heads || qkv_n % 256 || d.hidden % 256 || d.inter % 128 ||
      (2 * d.inter) % 256 || (d.heads * d.head_dim) % 64 || d.layers < 1 || max_seq < 1 ||
      !(d.hidden == 256 || d.hidden == 512 || d.hidden == 1024 || d.hidden == 2560)) {
    set_error("unsupported text-encoder dimensions");
    return FLUX_CUDA_ERR_ARG;
  }
  int last = 0;
  for (int i = 0; i < 3; ++i) {
    if (d.out_layers[i] < 0 || d.out_layers[i] >= d.layers || (i && d.out_layers[i] <= d.out_layers[i - 1])) {
      set_error("output layers must be increasing and inside the model");
      return FLUX_CUDA_ERR_ARG;
    }
    last = d.out_layers[i];
  }
  cudaSetDevice(ctx->device);
  flux_cuda_qwen3 *m = new flux_cuda_qwen3();
  m->ctx = ctx;
  m->d = d;
  m->f16 = ctx->f16;
  m->run_layers = last + 1;
  m->max_seq = max_seq;
  m->layers.resize(m->run_layers);
  const size_t h = d.hidden, hd = d.head_dim, qd = static_cast<size_t>(d.heads) * hd, it = d.inter, S = max_seq;
  int rc = q_alloc(m, &m->embed, static_cast<size_t>(d.vocab) * h);
  for (QwenLayer &l : m->layers) {
    if (!rc) rc = q_alloc(m, &l.qkv, static_cast<size_t>(qkv_n) * h);
    if (!rc) rc = q_alloc(m, &l.o, h * qd);
    if (!rc) rc = q_alloc(m, &l.gateup, 2 * it * h);
    if (!rc) rc = q_alloc(m, &l.down, h * it);
    if (!rc) rc = q_alloc(m, &l.ln1, h);
    if (!rc) rc = q_alloc(m, &l.ln2, h);
    if (!rc) rc = q_alloc(m, &l.qn, hd);
    if (!rc) rc = q_alloc(m, &l.kn, hd);
  }
  m->staging_bytes = it * h * 2;
  uint16_t *stg = nullptr;
  if (!rc) rc = q_alloc(m, &stg, it * h);
  m->staging = stg;
  if (!rc) rc = q_alloc(m, &m->hidden, S * h);
  if (!rc) rc = q_alloc(m, &m->out, S * 3 * h);
  if (!rc) rc = q_alloc(m, &m->part, GEMM_MAX_PROBLEMS * S * h);
  if (const char *e = getenv("FLUX_CUDA_QWEN_SPLITK")) m->split_k = atoi(e) != 0;
  if (!rc) rc = q_alloc(m, &m->ones, h);
  if (!rc) rc = q_alloc(m, &m->cos_t, S * 64);
  if (!rc) rc = q_alloc(m, &m->sin_t, S * 64);
  if (!rc) rc = q_alloc(m, &m->ang_t, S * 64);
  if (!rc) rc = q_alloc(m, &m->norm, S * h);
  if (!rc) rc = q_alloc(m, &m->qkv, S * static_cast<size_t>(qkv_n));
  if (!rc) rc = q_alloc(m, &m->attn, S * qd);
  if (!rc) rc = q_alloc(m, &m->act, S * it);
  if (!rc) rc = q_alloc(m, &m->ids, S);
  if (!rc) rc = q_alloc(m, &m->mask, S / 32 + S + 4);  // [batch, ceil(seq / 32)] words for any split of S tokens
  if (!rc) {
    std::vector<float> ones(h, 1.0f), cs(S * 64), sn(S * 64), an(S * 64);
    for (size_t p = 0; p < S; ++p)
      for (int i = 0; i < 64; ++i) {  // compute_rope_freqs, flux_qwen3.c:253-262, in float like the reference
        const float freq = 1.0f / powf(d.rope_theta, static_cast<float>(2 * i) / static_cast<float>(hd));
        const float ang = static_cast<float>(p) * freq;
        cs[p * 64 + i] = cosf(ang);
        sn[p * 64 + i] = sinf(ang);
        // the same angle reduced to [-pi, pi] (in double): what the fused projection epilogue reads, taking cos and
        // sin from the special-function unit in its accurate range
        an[p * 64 + i] = static_cast<float>(remainder(static_cast<double>(ang), 6.283185307179586476925286766559));
      }
    rc = check_cuda(upload_h2d(ctx->stream, m->ones, ones.data(), h * 4), "upload");
    if (!rc) rc = check_cuda(upload_h2d(ctx->stream, m->cos_t, cs.data(), cs.size() * 4), "upload");
    if (!rc) rc = check_cuda(upload_h2d(ctx->stream, m->sin_t, sn.data(), sn.size() * 4), "upload");
    if (!rc) rc = check_cuda(upload_h2d(ctx->stream, m->ang_t, an.data(), an.size() * 4), "upload");
  }
  if (rc) {
    flux_cuda_qwen3_free(m);
    return rc;
  }
  m->expected = 1 + static_cast<size_t>(m->run_layers) * 11;  // the embedding and the layers the output depends on
  *out = m;
  return FLUX_CUDA_OK;
}

int flux_cuda_qwen3_set_tensor(flux_cuda_qwen3 *m, const char *name, const void *data, int dtype,
                               const long long *shape, int ndim) {
  if (!m || !name || !data || !shape || dtype < 0 || dtype > 2 || ndim < 1 || ndim > 2) {
    set_error("set_tensor: bad argument");
    return FLUX_CUDA_ERR_ARG;
  }
  cudaSetDevice(m->ctx->device);
  const flux_cuda_qwen3_dims &d = m->d;
  const long long h = d.hidden, hd = d.head_dim, qd = static_cast<long long>(d.heads) * hd,
                  kd = static_cast<long long>(d.kv_heads) * hd, it = d.inter;
  const long long r = shape[0], c = ndim == 2 ? shape[1] : 1;
  const size_t count = static_cast<size_t>(r) * c;
  std::vector<uint16_t> tmp;
  auto want = [&](long long er, long long ec) -> int {
    if (r != er || c != ec) {
      set_error("tensor %s has shape [%lld, %lld], expected [%lld, %lld]", name, r, c, er, ec);
      return FLUX_CUDA_ERR_MODEL;
    }
    return 0;
  };
  auto plain = [&](uint16_t *dst, long long er, long long ec) -> int {
    int rc = want(er, ec);
    if (rc) return rc;
    return upload_16(m->ctx, dst, data, dtype, 0, count, m->f16, tmp);
  };
  auto vec = [&](float *dst, long long n) -> int {
    if (ndim != 1 || r != n) {
      set_error("tensor %s must have shape [%lld]", name, n);
      return FLUX_CUDA_ERR_MODEL;
    }
    std::vector<float> v(n);
    for (long long i = 0; i < n; ++i)
      v[i] = dtype == 0 ? reinterpret_cast<const float *>(data)[i]
                        : half_to_f32_host(reinterpret_cast<const uint16_t *>(data)[i], dtype);
    return check_cuda(upload_h2d(m->ctx->stream, dst, v.data(), n * 4), "upload norm weights");
  };
  // gate (half 0) or up (half 1) rows into the 128-row interleaved [gate | up] layout of the SwiGLU epilogue
  auto interleave = [&](uint16_t *dst, int half) -> int {
    int rc = want(it, h);
    if (rc) return rc;
    rc = upload_16(m->ctx, m->staging, data, dtype, 0, count, m->f16, tmp);
    if (rc) return rc;
    const size_t blk = 128 * h * 2;
    for (long long b = 0; b < it / 128; ++b)
      cudaMemcpyAsync(reinterpret_cast<char *>(dst) + (2 * b + half) * blk,
                      reinterpret_cast<const char *>(m->staging) + b * blk, blk, cudaMemcpyDeviceToDevice, m->ctx->stream);
    return check_cuda(cudaStreamSynchronize(m->ctx->stream), "interleave weights");
  };

  int rc = FLUX_CUDA_ERR_MODEL, idx = -1;
  char rest[128] = "";
  std::string n(name);
  if (n == "model.embed_tokens.weight") rc = plain(m->embed, d.vocab, h);
  else if (n == "model.norm.weight") rc = (ndim == 1 && r == h) ? 0 : want(h, 1);  // final norm: not part of the output
  else if (sscanf(name, "model.layers.%d.%127s", &idx, rest) == 2 && idx >= 0 && idx < d.layers) {
    std::string t(rest);
    static const char *known[] = {"input_layernorm.weight", "post_attention_layernorm.weight",
                                  "self_attn.q_proj.weight", "self_attn.k_proj.weight", "self_attn.v_proj.weight",
                                  "self_attn.o_proj.weight", "self_attn.q_norm.weight", "self_attn.k_norm.weight",
                                  "mlp.gate_proj.weight", "mlp.up_proj.weight", "mlp.down_proj.weight"};
    bool is_known = false;
    for (const char *k : known) is_known |= t == k;
    if (!is_known) {
      set_error("unknown tensor %s", name);
    } else if (idx >= m->run_layers) {
      rc = 0;  // layers after the last output layer do not influence the result: accepted, not kept
    } else {
      QwenLayer &l = m->layers[idx];
      if (t == "input_layernorm.weight") rc = vec(l.ln1, h);
      else if (t == "post_attention_layernorm.weight") rc = vec(l.ln2, h);
      else if (t == "self_attn.q_norm.weight") rc = vec(l.qn, hd);
      else if (t == "self_attn.k_norm.weight") rc = vec(l.kn, hd);
      else if (t == "self_attn.q_proj.weight") rc = plain(l.qkv, qd, h);
      else if (t == "self_attn.k_proj.weight") rc = plain(l.qkv + qd * h, kd, h);
      else if (t == "self_attn.v_proj.weight") rc = plain(l.qkv + (qd + kd) * h, kd, h);
      else if (t == "self_attn.o_proj.weight") rc = plain(l.o, h, qd);
      else if (t == "mlp.down_proj.weight") rc = plain(l.down, h, it);
      else if (t == "mlp.gate_proj.weight") rc = interleave(l.gateup, 0);
      else rc = interleave(l.gateup, 1);
    }
  } else {
    set_error("unknown tensor %s", name);
  }
  // completeness is judged on what the output depends on: the final norm and later layers are accepted, not required
  if (rc == 0 && (n == "model.embed_tokens.weight" || (idx >= 0 && idx < m->run_layers))) m->seen.insert(n);
  return rc;
}

int flux_cuda_qwen3_finalize(flux_cuda_qwen3 *m) {
  if (!m) return FLUX_CUDA_ERR_ARG;
  if (m->seen.size() != m->expected) {
    set_error("text encoder incomplete: %zu of %zu tensors were provided", m->seen.size(), m->expected);
    return FLUX_CUDA_ERR_MODEL;
  }
  int rc = check_cuda(cudaStreamSynchronize(m->ctx->stream), "upload weights");  // uploads are stream-ordered
  if (rc) return rc;
  m->finalized = true;
  return FLUX_CUDA_OK;
}

int flux_cuda_qwen3_load_dir(flux_cuda_ctx *ctx, const char *model_dir, int max_seq, flux_cuda_qwen3 **out) {
  if (!ctx || !model_dir || !out) return FLUX_CUDA_ERR_ARG;
  *out = nullptr;
  flux_cuda_qwen3_dims d;
  flux_cuda_qwen3_dims_4b(&d);
  flux_cuda_qwen3 *m = nullptr;
  int rc = flux_cuda_qwen3_create(ctx, &d, max_seq, &m);
  for (int f = 1; !rc && f <= 2; ++f) {  // both shards must exist; a tensor may live in either
    char path[1024];
    snprintf(path, sizeof(path), "%s/model-%05d-of-00002.safetensors", model_dir, f);
    rc = safetensors_for_each(path, [&](const char *name, const void *data, int dt, const long long *shape, int nd) {
      return flux_cuda_qwen3_set_tensor(m, name, data, dt, shape, nd);
    });
  }
  if (!rc) rc = flux_cuda_qwen3_finalize(m);
  if (rc) {
    flux_cuda_qwen3_free(m);
    return rc;
  }
  *out = m;
  return FLUX_CUDA_OK;
}

// One GEMM of the encoder: out = epilogue(X[M, K] * W[N, K]^T).
static int q_gemm(flux_cuda_qwen3 *m, const void *X, long long ldx, const void *W, int M, int N, int K, const EpiSeg &s0,
                  int n_split = 0, const EpiSeg *s1 = nullptr) {
  GemmParams P;
  memset(&P, 0, sizeof(P));
  const bool pair = m->ctx->gemm_pair;
  int rc = pair ? gemm_make_problem_pair(&P.p[0], X, ldx, W, M, N, K) : gemm_make_problem(&P.p[0], X, ldx, W, M, N, K, 256);
  if (rc) return rc;
  P.nprob = 1;
  P.err = m->ctx->err_dev;
  P.p[0].x_f16 = m->f16;
  P.p[0].seg[0] = s0;
  if (s1 && n_split > 0 && n_split < N) {
    P.p[0].n_split = n_split;
    P.p[0].seg[1] = *s1;
  }
  return pair ? gemm2_launch(&P, m->ctx->num_sms, m->ctx->stream) : gemm_launch(&P, 256, m->ctx->num_sms, m->ctx->stream);
}

// Residual projection hidden += X[M, K] * W[h, K]^T. A plain launch has only ceil(M / 256) * h / 256 output tiles
// (20 at 512 tokens) for 74 SM pairs, each with a long K loop. When at least two K-slices fit on the idle pairs, K is
// cut into up to four slices that run as independent problems of ONE launch and store f32 partial products; the next
// RMSNorm pass adds them to the residual stream in slice order (deterministic, no atomics). Returns the number of
// slices written to m->part (0: accumulated directly), or a negative launch error.
static int q_residual_gemm(flux_cuda_qwen3 *m, const void *X, long long ldx, const uint16_t *W, int M, int K) {
  const int h = m->d.hidden;
  const bool pair = m->ctx->gemm_pair;
  const int units = pair ? m->ctx->num_sms / 2 : m->ctx->num_sms;
  const int tiles = ((M + (pair ? 255 : 127)) / (pair ? 256 : 128)) * (h / 256);
  const int KB = K / 64;
  int S = m->split_k ? units / tiles : 1;
  if (S > GEMM_MAX_PROBLEMS) S = GEMM_MAX_PROBLEMS;
  if (S > KB) S = KB;
  EpiSeg sg;
  memset(&sg, 0, sizeof(sg));
  sg.out_f16 = m->f16;
  sg.ld = h;
  if (S < 2) {
    sg.mode = EPI_GATED_RES_F32;
    sg.out = m->hidden;
    sg.gate = m->ones;
    int rc = q_gemm(m, X, ldx, W, M, h, K, sg);
    return rc ? (rc < 0 ? rc : -rc) : 0;
  }
  GemmParams P;
  memset(&P, 0, sizeof(P));
  P.nprob = S;
  P.err = m->ctx->err_dev;
  int kb0 = 0;
  for (int s = 0; s < S; ++s) {
    const int kbs = KB / S + (s < KB % S ? 1 : 0);
    const uint16_t *Xs = reinterpret_cast<const uint16_t *>(X) + static_cast<size_t>(kb0) * 64;
    const uint16_t *Ws = W + static_cast<size_t>(kb0) * 64;
    int rc = pair ? gemm_make_problem_pair(&P.p[s], Xs, ldx, Ws, M, h, kbs * 64, K)
                  : gemm_make_problem(&P.p[s], Xs, ldx, Ws, M, h, kbs * 64, 256, K);
    if (rc) return rc < 0 ? rc : -rc;
    P.p[s].x_f16 = m->f16;
    sg.mode = EPI_STORE_F32;
    sg.out = m->part + static_cast<size_t>(s) * m->max_seq * h;
    P.p[s].seg[0] = sg;
    kb0 += kbs;
  }
  int rc = pair ? gemm2_launch(&P, m->ctx->num_sms, m->ctx->stream) : gemm_launch(&P, 256, m->ctx->num_sms, m->ctx->stream);
  return rc ? (rc < 0 ? rc : -rc) : S;
}

// Queues the whole pass on the context's stream; the result is m->out ([seq, 3 * hidden] f32, device).
// `batch` prompts of `seq` tokens each (ids and mask [batch, seq]); rows of all prompts go through the layers together,
// attention sees each prompt on its own.
static int qwen3_enqueue(flux_cuda_qwen3 *m, const int *input_ids, const int *attention_mask, int seq, int batch) {
  if (!m || !input_ids || seq < 1 || batch < 1) {
    set_error("qwen3_forward: bad argument");
    return FLUX_CUDA_ERR_ARG;
  }
  if (!m->finalized) {
    set_error("qwen3_forward: model is not finalized");
    return FLUX_CUDA_ERR_MODEL;
  }
  if (static_cast<long long>(seq) * batch > m->max_seq) {
    set_error("qwen3_forward: %d x %d tokens exceed the capacity of %d", batch, seq, m->max_seq);
    return FLUX_CUDA_ERR_ARG;
  }
  cudaSetDevice(m->ctx->device);
  cudaStream_t st = m->ctx->stream;
  const flux_cuda_qwen3_dims &d = m->d;
  const int h = d.hidden, hd = d.head_dim, qd = d.heads * hd, kd = d.kv_heads * hd, it = d.inter;
  const int qkv_n = qd + 2 * kd, f16 = m->f16 ? 1 : 0;
  const int rows = seq * batch;
  const int words = (seq + 31) / 32;
  std::vector<uint32_t> bits(static_cast<size_t>(words) * batch, 0u);
  for (int b = 0; b < batch; ++b)
    for (int j = 0; j < seq; ++j)
      if (!attention_mask || attention_mask[b * seq + j]) bits[static_cast<size_t>(b) * words + (j >> 5)] |= 1u << (j & 31);
  int rc = check_cuda(cudaMemcpyAsync(m->ids, input_ids, rows * sizeof(int), cudaMemcpyHostToDevice, st), "upload ids");
  if (!rc) rc = check_cuda(cudaMemcpyAsync(m->mask, bits.data(), bits.size() * 4, cudaMemcpyHostToDevice, st), "upload mask");
  if (rc) return rc;
  embed_gather_kernel<<<rows, 256, 0, st>>>(m->embed, m->ids, m->hidden, h, d.vocab, f16);
  rc = check_cuda(cudaGetLastError(), "embedding lookup");
  if (rc) return rc;

  auto seg = [&](int mode, void *dst, long long ld, int col0, const float *gate) {
    EpiSeg s;
    memset(&s, 0, sizeof(s));
    s.mode = mode;
    s.out_f16 = f16;
    s.col0 = col0;
    s.ld = ld;
    s.out = dst;
    s.gate = gate;
    return s;
  };
  int gr = 0;
  int next_out = 0;
  int pending = 0;  // K-slices of the last residual projection still to be added to the residual stream
  const long long pstride = static_cast<long long>(m->max_seq) * h;
  for (int l = 0; l < m->run_layers && !gr; ++l) {
    const QwenLayer &w = m->layers[l];
    gr = launch_rmsnorm(m->hidden, m->norm, w.ln1, rows, h, f16, m->part, pending, pstride, st);
    pending = 0;
    if (gr) break;
    EpiSeg sq = seg(EPI_QKV_NORM_ROPE, m->qkv, qkv_n, 0, nullptr);
    sq.qk.wq_txt = sq.qk.wq_img = w.qn;
    sq.qk.wk_txt = sq.qk.wk_img = w.kn;
    sq.qk.cos_t = m->cos_t;
    sq.qk.sin_t = m->sin_t;
    sq.qk.ang = m->ang_t;
    sq.qk.pos0 = 0;
    sq.qk.seq = seq;
    sq.qk.n_txt = 0;
    sq.qk.q_cols = qd;
    sq.qk.k_cols = kd;
    sq.qk.half_split = 1;
    gr = q_gemm(m, m->norm, h, w.qkv, rows, qkv_n, h, sq);
    if (gr) break;
    AttnParams A;
    gr = attn2_make_params(&A, m->qkv, batch, seq, qkv_n, 0, qd, qd + kd, m->attn, qd, 0, d.heads, f16, m->ctx->err_dev);
    if (gr) break;
    A.kv_group = d.heads / d.kv_heads;
    A.causal = 1;
    A.key_mask = m->mask;
    gr = attn_launch_version(m->ctx->attn_version, &A, st);
    if (gr) break;
    pending = q_residual_gemm(m, m->attn, qd, w.o, rows, qd);
    if (pending < 0) {
      gr = pending;
      break;
    }
    gr = launch_rmsnorm(m->hidden, m->norm, w.ln2, rows, h, f16, m->part, pending, pstride, st);
    pending = 0;
    if (gr) break;
    gr = q_gemm(m, m->norm, h, w.gateup, rows, 2 * it, h, seg(EPI_SWIGLU_BF16, m->act, it, 0, nullptr));
    if (gr) break;
    pending = q_residual_gemm(m, m->act, it, w.down, rows, it);
    if (pending < 0) {
      gr = pending;
      break;
    }
    const bool collect = next_out < 3 && l == d.out_layers[next_out];
    if (pending > 0 && (collect || l + 1 == m->run_layers)) {  // nobody after this layer folds the slices: do it now
      gr = launch_rmsnorm(m->hidden, nullptr, w.ln1, rows, h, f16, m->part, pending, pstride, st);
      pending = 0;
      if (gr) break;
    }
    if (collect) {
      rc = check_cuda(cudaMemcpy2DAsync(m->out + static_cast<size_t>(next_out) * h, 3 * h * sizeof(float), m->hidden,
                                        h * sizeof(float), h * sizeof(float), rows, cudaMemcpyDeviceToDevice, st),
                      "collect layer output");
      if (rc) return rc;
      ++next_out;
    }
  }
  if (gr) {
    set_error("qwen3_forward: kernel launch failed (rc %d, cuda: %s)", gr, cudaGetErrorString(cudaGetLastError()));
    ctx_sync_check(m->ctx);
    return (gr == -1 || gr == -5) ? FLUX_CUDA_ERR_ARG : FLUX_CUDA_ERR_CUDA;
  }
  return FLUX_CUDA_OK;
}

int flux_cuda_qwen3_forward(flux_cuda_qwen3 *m, const int *input_ids, const int *attention_mask, int seq, float *out) {
  if (!out) {
    set_error("qwen3_forward: bad argument");
    return FLUX_CUDA_ERR_ARG;
  }
  return flux_cuda_qwen3_forward_batch(m, input_ids, attention_mask, 1, seq, out);
}

int flux_cuda_qwen3_forward_batch(flux_cuda_qwen3 *m, const int *input_ids, const int *attention_mask, int batch, int seq,
                                  float *out) {
  if (!out) {
    set_error("qwen3_forward: bad argument");
    return FLUX_CUDA_ERR_ARG;
  }
  int rc = qwen3_enqueue(m, input_ids, attention_mask, seq, batch);
  if (rc) return rc;
  rc = check_cuda(cudaMemcpyAsync(out, m->out, static_cast<size_t>(seq) * batch * 3 * m->d.hidden * sizeof(float),
                                  cudaMemcpyDeviceToHost, m->ctx->stream),
                  "download embeddings");
  if (!rc) rc = ctx_sync_check(m->ctx);
  return rc;
}

int flux_cuda_qwen3_forward_device(flux_cuda_qwen3 *m, const int *input_ids, const int *attention_mask, int seq,
                                   const float **out_dev) {
  if (!out_dev) {
    set_error("qwen3_forward_device: bad argument");
    return FLUX_CUDA_ERR_ARG;
  }
  return flux_cuda_qwen3_forward_batch_device(m, input_ids, attention_mask, 1, seq, out_dev);
}

int flux_cuda_qwen3_forward_batch_device(flux_cuda_qwen3 *m, const int *input_ids, const int *attention_mask, int batch,
                                         int seq, const float **out_dev) {
  if (!out_dev) {
    set_error("qwen3_forward_device: bad argument");
    return FLUX_CUDA_ERR_ARG;
  }
  *out_dev = nullptr;
  int rc = qwen3_enqueue(m, input_ids, attention_mask, seq, batch);
  if (rc) return rc;
  *out_dev = m->out;
  return FLUX_CUDA_OK;
}

}  // extern "C"
