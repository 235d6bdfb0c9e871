// Model residency, the DiT forward pass and the on-device sampler loop.
//
// Replaces, behind the C ABI, the reference's flux_transformer_load_safetensors (flux_transformer.c:4411-4656),
// flux_transformer_forward / _with_refs / _with_multi_refs (3115-3577, 3605-4043) and the Euler samplers
// flux_sample_euler* / flux_sample_euler_cfg* (flux_sample.c:212-691). The whole loop (steps x forward +
// update) is queued on one stream; the host sees only the inputs it uploads and the latent it downloads.
#include "engine.cuh"

#include <math.h>
#include <stdint.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>
#include <algorithm>
#include <thread>

#include "attention.cuh"
#include "elementwise.cuh"
#include "flux_cuda.h"
#include "gemm.cuh"
#include "launch.cuh"

namespace fx {

typedef __nv_bfloat16 bf16;

// ------------------------------------------------------------------------------------------------ helpers
static uint16_t f32_to_bf16_host(float f) {
  uint32_t u;
  memcpy(&u, &f, 4);
  if ((u & 0x7F800000u) == 0x7F800000u && (u & 0x007FFFFFu)) return static_cast<uint16_t>((u >> 16) | 0x40);
  u += 0x7FFFu + ((u >> 16) & 1u);
  return static_cast<uint16_t>(u >> 16);
}
static float bf16_to_f32_host(uint16_t b) {
  uint32_t u = static_cast<uint32_t>(b) << 16;
  float f;
  memcpy(&f, &u, 4);
  return f;
}
// f32 -> f16 bits, round to nearest even, saturating at +-65504, subnormals handled.
static uint16_t f32_to_f16_host(float f) {
  uint32_t u;
  memcpy(&u, &f, 4);
  const uint16_t sign = static_cast<uint16_t>((u >> 16) & 0x8000u);
  const uint32_t a = u & 0x7FFFFFFFu;
  if (a >= 0x7F800000u) return static_cast<uint16_t>(sign | (a > 0x7F800000u ? 0x7E00u : 0x7BFFu));
  if (a >= 0x477FF000u) return static_cast<uint16_t>(sign | 0x7BFFu);  // rounds to >= 65520: saturate
  if (a < 0x33000001u) return sign;                                   // below half of the smallest subnormal
  int exp = static_cast<int>(a >> 23) - 127;
  uint32_t man = (a & 0x7FFFFFu) | 0x800000u;  // 24-bit significand
  int shift;                                   // bits to drop
  uint32_t base;
  if (exp < -14) {  // subnormal result: value = man * 2^(exp-23), unit 2^-24
    shift = -exp - 14 + 13;  // = 23 - (exp + 24)
    base = 0;
  } else {
    shift = 13;
    base = static_cast<uint32_t>(exp + 15) << 10;
    man &= 0x7FFFFFu;
  }
  uint32_t q = man >> shift;
  const uint32_t rem = man & ((1u << shift) - 1u), half = 1u << (shift - 1);
  if (rem > half || (rem == half && (q & 1u))) ++q;  // may carry into the exponent: still correct
  return static_cast<uint16_t>(sign | (base + q));
}
static float f16_to_f32_host(uint16_t h) {
  const uint32_t sign = (h & 0x8000u) << 16;
  int exp = (h >> 10) & 0x1F;
  uint32_t man = h & 0x3FFu;
  uint32_t u;
  if (exp == 0) {
    if (man == 0) {
      u = sign;
    } else {
      exp = 127 - 15 + 1;
      while (!(man & 0x400u)) {
        man <<= 1;
        --exp;
      }
      man &= 0x3FFu;
      u = sign | (static_cast<uint32_t>(exp) << 23) | (man << 13);
    }
  } else if (exp == 31) {
    u = sign | 0x7F800000u | (man << 13);
  } else {
    u = sign | (static_cast<uint32_t>(exp - 15 + 127) << 23) | (man << 13);
  }
  float f;
  memcpy(&f, &u, 4);
  return f;
}

template <typename T>
static int dev_alloc(std::vector<void *> &bag, T **p, size_t count) {
  void *q = nullptr;
  const size_t bytes = count * sizeof(T);
  cudaError_t e = cudaMalloc(&q, bytes ? bytes : 16);
  if (e != cudaSuccess) {
    set_error("cudaMalloc of %zu bytes failed: %s", bytes, cudaGetErrorString(e));
    return FLUX_CUDA_ERR_NOMEM;
  }
  bag.push_back(q);
  *p = reinterpret_cast<T *>(q);
  return 0;
}

// ------------------------------------------------------------------------------------------------ model
int model_create(flux_cuda_ctx *ctx, const ModelDims &d, flux_cuda_model **out) {
  *out = nullptr;
  if (d.head_dim != 128 || d.heads * d.head_dim != d.hidden || d.hidden % 256 || d.mlp % 128 || (2 * d.mlp) % 256 ||
      d.text_dim % 64 || d.latent_ch % 64 || d.latent_ch % 128 || d.time_dim % 8 || d.axis_dim * 4 != d.head_dim ||
      d.n_double < 0 || d.n_single < 0 ||
      !(d.hidden == 256 || d.hidden == 512 || d.hidden == 1024 || d.hidden == 3072)) {
    set_error("unsupported model dimensions (head_dim must be 128, hidden in {256,512,1024,3072}, mlp %% 128 == 0)");
    return FLUX_CUDA_ERR_ARG;
  }
  cudaSetDevice(ctx->device);
  flux_cuda_model *m = new flux_cuda_model();
  m->ctx = ctx;
  m->d = d;
  m->f16 = ctx->f16;
  const size_t h = d.hidden, mlp = d.mlp;
  int rc = 0;
  auto A = [&](bf16 **p, size_t n) {
    if (!rc) {
      rc = dev_alloc(m->allocs, p, n);
      m->weight_bytes += n * 2;
    }
  };
  auto AF = [&](float **p, size_t n) {
    if (!rc) rc = dev_alloc(m->allocs, p, n);
  };
  A(&m->x_emb, h * d.latent_ch);
  A(&m->ctx_emb, h * d.text_dim);
  A(&m->t1, h * d.time_dim);
  A(&m->t2, h * h);
  A(&m->mod_all, 17 * h * h);
  A(&m->proj_out, static_cast<size_t>(d.latent_ch) * h);
  m->dbl.resize(d.n_double);
  m->sgl.resize(d.n_single);
  for (auto &b : m->dbl)
    for (int s = 0; s < 2; ++s) {
      A(&b.qkv[s], 3 * h * h);
      A(&b.out[s], h * h);
      A(&b.ffin[s], 2 * mlp * h);
      A(&b.ffout[s], h * mlp);
      AF(&b.nq[s], 128);
      AF(&b.nk[s], 128);
    }
  for (auto &b : m->sgl) {
    A(&b.lin1, (3 * h + 2 * mlp) * h);
    A(&b.lin2, h * (h + mlp));
    AF(&b.nq, 128);
    AF(&b.nk, 128);
  }
  m->staging_bytes = (3 * h + 2 * mlp) * h * 2;
  if (!rc) {
    bf16 *st = nullptr;
    rc = dev_alloc(m->allocs, &st, m->staging_bytes / 2);
    m->staging = st;
  }
  if (rc) {
    model_free(m);
    return rc;
  }
  m->expected = 9 + static_cast<size_t>(d.n_double) * 16 + static_cast<size_t>(d.n_single) * 4;
  *out = m;
  return 0;
}

void model_free(flux_cuda_model *m) {
  if (!m) return;
  cudaSetDevice(m->ctx->device);
  cudaStreamSynchronize(m->ctx->stream);
  for (void *p : m->allocs) cudaFree(p);
  delete m;
}

// Converts `count` elements of the source dtype (0 = F32, 1 = F16, 2 = BF16) to the model's 16-bit weight format
// on the host. bf16 -> f16 is exact for 6.1e-5 <= |w| <= 65504 (bf16 has fewer mantissa bits); smaller weights
// land on f16 subnormals with an absolute error below 3e-8.
float half_to_f32_host(uint16_t bits, int dtype) {
  return dtype == 1 ? f16_to_f32_host(bits) : bf16_to_f32_host(bits);
}

const uint16_t *to_half_host(const void *data, int dtype, size_t count, std::vector<uint16_t> &tmp, bool want_f16) {
  if ((dtype == 2 && !want_f16) || (dtype == 1 && want_f16)) return reinterpret_cast<const uint16_t *>(data);
  tmp.resize(count);
  const float *f = reinterpret_cast<const float *>(data);
  const uint16_t *hh = reinterpret_cast<const uint16_t *>(data);
  for (size_t i = 0; i < count; ++i) {
    const float v = dtype == 0 ? f[i] : dtype == 1 ? f16_to_f32_host(hh[i]) : bf16_to_f32_host(hh[i]);
    tmp[i] = want_f16 ? f32_to_f16_host(v) : f32_to_bf16_host(v);
  }
  return tmp.data();
}

// ---- pinned, multi-threaded weight upload
// A cudaMemcpy from pageable memory is staged by the driver through one bounce buffer on one thread (7.6 GB/s measured
// for the 7.75 GB transformer file). Here several host threads fill 32 MB pinned slots while earlier slots are in
// flight, so the copy runs at the smaller of the hosts' memcpy rate and the PCIe rate.
static void parallel_memcpy(void *dst, const void *src, size_t bytes, int threads) {
  if (threads <= 1 || bytes < (4u << 20)) {
    memcpy(dst, src, bytes);
    return;
  }
  const size_t per = ((bytes + threads - 1) / threads + 4095) & ~static_cast<size_t>(4095);
  std::vector<std::thread> pool;
  size_t handed = std::min(per, bytes);  // bytes [0, handed) are this thread's own part
  for (int t = 1; t < threads; ++t) {
    const size_t o = per * t;
    if (o >= bytes) break;
    const size_t n = std::min(per, bytes - o);
    try {
      pool.emplace_back([=] { memcpy(static_cast<char *>(dst) + o, static_cast<const char *>(src) + o, n); });
    } catch (...) {  // no thread to be had: this thread copies the rest itself (nothing may throw through the C ABI)
      break;
    }
    handed = o + n;
  }
  memcpy(dst, src, std::min(per, bytes));
  if (handed < bytes) memcpy(static_cast<char *>(dst) + handed, static_cast<const char *>(src) + handed, bytes - handed);
  for (auto &th : pool) th.join();
}

int upload_pipelined(flux_cuda_ctx *ctx, void *dst, const void *src, size_t bytes) {
  UploadRing &r = ctx->upload;
  if (r.state == 0) {
    const char *e = getenv("FLUX_CUDA_UPLOAD_THREADS");
    const int hw = static_cast<int>(std::thread::hardware_concurrency());
    r.threads = e ? atoi(e) : std::max(1, std::min(8, hw / 2));
    r.state = r.threads >= 1 ? 1 : -1;  // FLUX_CUDA_UPLOAD_THREADS=0: plain pageable copies
    for (int i = 0; i < UploadRing::SLOTS && r.state == 1; ++i) {
      if (cudaHostAlloc(&r.buf[i], UploadRing::SLOT_BYTES, cudaHostAllocDefault) != cudaSuccess ||
          cudaEventCreateWithFlags(&r.drained[i], cudaEventDisableTiming) != cudaSuccess) {
        cudaGetLastError();
        r.state = -1;
      }
    }
    if (r.state != 1) upload_ring_release(ctx), r.state = -1;
  }
  if (r.state != 1) return check_cuda(upload_h2d(ctx->stream, dst, src, bytes), "upload weights");
  for (size_t off = 0; off < bytes; off += UploadRing::SLOT_BYTES) {
    const size_t n = std::min(UploadRing::SLOT_BYTES, bytes - off);
    const int slot = r.next;
    r.next = (r.next + 1) % UploadRing::SLOTS;
    int rc = check_cuda(cudaEventSynchronize(r.drained[slot]), "upload weights");  // never recorded: returns at once
    if (rc) return rc;
    parallel_memcpy(r.buf[slot], static_cast<const char *>(src) + off, n, r.threads);
    rc = check_cuda(cudaMemcpyAsync(static_cast<char *>(dst) + off, r.buf[slot], n, cudaMemcpyHostToDevice, ctx->stream),
                    "upload weights");
    if (!rc) rc = check_cuda(cudaEventRecord(r.drained[slot], ctx->stream), "upload weights");
    if (rc) return rc;
  }
  return 0;
}

void upload_ring_release(flux_cuda_ctx *ctx) {
  UploadRing &r = ctx->upload;
  for (int i = 0; i < UploadRing::SLOTS; ++i) {
    if (r.drained[i]) cudaEventDestroy(r.drained[i]);
    if (r.buf[i]) cudaFreeHost(r.buf[i]);
    r.drained[i] = nullptr;
    r.buf[i] = nullptr;
  }
  r.state = 0;
  r.next = 0;
}

// 16-bit weights: copy, then convert in place on the device if the file's format is not the context's. Returns once
// the host data has been read; the device side completes in stream order (model_finalize synchronises).
int upload_16(flux_cuda_ctx *ctx, void *dst, const void *data, int dtype, size_t off, size_t count, bool want_f16,
              std::vector<uint16_t> &tmp) {
  if (dtype == 0) {
    const uint16_t *src = to_half_host(reinterpret_cast<const float *>(data) + off, 0, count, tmp, want_f16);
    return check_cuda(upload_h2d(ctx->stream, dst, src, count * 2), "upload weights");
  }
  int rc = upload_pipelined(ctx, dst, reinterpret_cast<const uint16_t *>(data) + off, count * 2);
  if (rc) return rc;
  const bool is_f16 = dtype == 1;
  if (is_f16 != want_f16 && launch_convert16_inplace(dst, static_cast<long long>(count), want_f16 ? 1 : 0, ctx->stream)) {
    set_error("weight format conversion could not be launched");
    return FLUX_CUDA_ERR_CUDA;
  }
  return 0;
}

// dst rows [0, 2*half): per block of 128 output columns, 128 rows of the first half then the matching 128 of the second.
// The source is elements [off, off + 2 * half_rows * cols) of `data`.
static int upload_interleaved(flux_cuda_model *m, bf16 *dst, const void *data, int dtype, size_t off, size_t half_rows,
                              size_t cols, std::vector<uint16_t> &tmp) {
  const size_t bytes = 2 * half_rows * cols * 2;
  if (bytes > m->staging_bytes) return FLUX_CUDA_ERR_ARG;
  int rc = upload_16(m->ctx, m->staging, data, dtype, off, 2 * half_rows * cols, m->f16, tmp);
  if (rc) return rc;
  const char *st = reinterpret_cast<const char *>(m->staging);
  const size_t blk = 128 * cols * 2;
  for (size_t b = 0; b < half_rows / 128; ++b) {
    char *d = reinterpret_cast<char *>(dst) + 2 * b * blk;
    cudaMemcpyAsync(d, st + b * blk, blk, cudaMemcpyDeviceToDevice, m->ctx->stream);
    cudaMemcpyAsync(d + blk, st + (half_rows / 128 + b) * blk, blk, cudaMemcpyDeviceToDevice, m->ctx->stream);
  }
  return check_cuda(cudaGetLastError(), "interleave weights");  // m->staging is reused in stream order
}

int model_set_tensor(flux_cuda_model *m, const char *name, const void *data, int dtype, const long long *shape,
                     int ndim) {
  if (!m || !name || !data || !shape || dtype < 0 || dtype > 2 || ndim < 1 || ndim > 2) {
    set_error("set_tensor: bad argument");
    return FLUX_CUDA_ERR_ARG;
  }
  cudaSetDevice(m->ctx->device);
  const ModelDims &d = m->d;
  const long long h = d.hidden, mlp = d.mlp;
  const long long r = shape[0], c = ndim == 2 ? shape[1] : 1;
  const size_t count = static_cast<size_t>(r) * c;
  std::vector<uint16_t> tmp;
  std::string n(name);

  auto want = [&](long long er, long long ec) -> int {
    if (r != er || c != ec) {
      set_error("tensor %s has shape [%lld, %lld], expected [%lld, %lld]", name, r, c, er, ec);
      return FLUX_CUDA_ERR_MODEL;
    }
    return 0;
  };
  auto plain = [&](bf16 *dst, long long er, long long ec) -> int {
    int rc = want(er, ec);
    if (rc) return rc;
    return upload_16(m->ctx, dst, data, dtype, 0, count, m->f16, tmp);
  };
  auto vec_f32 = [&](float *dst) -> int {
    if (ndim != 1 || r != 128) {
      set_error("tensor %s must have shape [128]", name);
      return FLUX_CUDA_ERR_MODEL;
    }
    float v[128];
    for (int i = 0; i < 128; ++i) {
      if (dtype == 0) v[i] = reinterpret_cast<const float *>(data)[i];
      else if (dtype == 1) v[i] = f16_to_f32_host(reinterpret_cast<const uint16_t *>(data)[i]);
      else v[i] = bf16_to_f32_host(reinterpret_cast<const uint16_t *>(data)[i]);
    }
    return check_cuda(upload_h2d(m->ctx->stream, dst, v, sizeof(v)), "upload norm weights");
  };

  int rc = FLUX_CUDA_ERR_MODEL;
  int idx = -1;
  char rest[128] = "";
  if (n == "x_embedder.weight") rc = plain(m->x_emb, h, d.latent_ch);
  else if (n == "context_embedder.weight") rc = plain(m->ctx_emb, h, d.text_dim);
  else if (n == "time_guidance_embed.timestep_embedder.linear_1.weight") rc = plain(m->t1, h, d.time_dim);
  else if (n == "time_guidance_embed.timestep_embedder.linear_2.weight") rc = plain(m->t2, h, h);
  else if (n == "double_stream_modulation_img.linear.weight") rc = plain(m->mod_all, 6 * h, h);
  else if (n == "double_stream_modulation_txt.linear.weight") rc = plain(m->mod_all + 6 * h * h, 6 * h, h);
  else if (n == "single_stream_modulation.linear.weight") rc = plain(m->mod_all + 12 * h * h, 3 * h, h);
  else if (n == "norm_out.linear.weight") rc = plain(m->mod_all + 15 * h * h, 2 * h, h);
  else if (n == "proj_out.weight") rc = plain(m->proj_out, d.latent_ch, h);
  else if (sscanf(name, "transformer_blocks.%d.%127s", &idx, rest) == 2 && idx >= 0 && idx < d.n_double) {
    DoubleW &b = m->dbl[idx];
    std::string t(rest);
    if (t == "attn.norm_q.weight") rc = vec_f32(b.nq[1]);
    else if (t == "attn.norm_k.weight") rc = vec_f32(b.nk[1]);
    else if (t == "attn.norm_added_q.weight") rc = vec_f32(b.nq[0]);
    else if (t == "attn.norm_added_k.weight") rc = vec_f32(b.nk[0]);
    else if (t == "attn.to_q.weight") rc = plain(b.qkv[1], h, h);
    else if (t == "attn.to_k.weight") rc = plain(b.qkv[1] + h * h, h, h);
    else if (t == "attn.to_v.weight") rc = plain(b.qkv[1] + 2 * h * h, h, h);
    else if (t == "attn.add_q_proj.weight") rc = plain(b.qkv[0], h, h);
    else if (t == "attn.add_k_proj.weight") rc = plain(b.qkv[0] + h * h, h, h);
    else if (t == "attn.add_v_proj.weight") rc = plain(b.qkv[0] + 2 * h * h, h, h);
    else if (t == "attn.to_out.0.weight") rc = plain(b.out[1], h, h);
    else if (t == "attn.to_add_out.weight") rc = plain(b.out[0], h, h);
    else if (t == "ff.linear_out.weight") rc = plain(b.ffout[1], h, mlp);
    else if (t == "ff_context.linear_out.weight") rc = plain(b.ffout[0], h, mlp);
    else if (t == "ff.linear_in.weight" || t == "ff_context.linear_in.weight") {
      // rows [0, mlp) = gate, [mlp, 2 mlp) = up (flux_transformer.c:4503-4523)
      if (!(rc = want(2 * mlp, h)))
        rc = upload_interleaved(m, b.ffin[t == "ff.linear_in.weight" ? 1 : 0], data, dtype, 0, mlp, h, tmp);
    } else {
      set_error("unknown tensor %s", name);
    }
  } else if (sscanf(name, "single_transformer_blocks.%d.%127s", &idx, rest) == 2 && idx >= 0 && idx < d.n_single) {
    SingleW &b = m->sgl[idx];
    std::string t(rest);
    if (t == "attn.norm_q.weight") rc = vec_f32(b.nq);
    else if (t == "attn.norm_k.weight") rc = vec_f32(b.nk);
    else if (t == "attn.to_out.weight") rc = plain(b.lin2, h, h + mlp);
    else if (t == "attn.to_qkv_mlp_proj.weight") {
      // rows [Q | K | V | gate | up] (flux_transformer.c:3051-3058): Q, K, V stay; gate/up are interleaved
      if (!(rc = want(3 * h + 2 * mlp, h))) {
        rc = upload_16(m->ctx, b.lin1, data, dtype, 0, 3 * h * h, m->f16, tmp);
        if (!rc) rc = upload_interleaved(m, b.lin1 + 3 * h * h, data, dtype, 3 * h * h, mlp, h, tmp);
      }
    } else {
      set_error("unknown tensor %s", name);
    }
  } else {
    set_error("unknown tensor %s", name);
  }
  if (rc == 0) m->seen.insert(n);
  return rc;
}

int model_finalize(flux_cuda_model *m) {
  if (!m) return FLUX_CUDA_ERR_ARG;
  if (m->seen.size() != m->expected) {
    set_error("model incomplete: %zu of %zu tensors were provided", m->seen.size(), m->expected);
    return FLUX_CUDA_ERR_MODEL;
  }
  int rc = check_cuda(cudaStreamSynchronize(m->ctx->stream), "upload weights");  // uploads are stream-ordered
  if (rc) return rc;
  m->finalized = true;
  return 0;
}

// ------------------------------------------------------------------------------------------------ workspace
static void build_rope(const ModelDims &d, const Workspace &ws, std::vector<float> &cs, std::vector<float> &sn,
                       std::vector<float> &ang) {
  // cos/sin [N, 128] over [txt ; img ; refs]; 4 axes (T, Y, X, L) x 16 frequencies, each duplicated over its
  // (even, odd) pair (flux_transformer.c:591-779), evaluated in float like the reference.
  const int ax = d.axis_dim, half = ax / 2, hd = d.head_dim;
  std::vector<float> fr(half);
  for (int k = 0; k < half; ++k) fr[k] = 1.0f / powf(d.rope_theta, static_cast<float>(2 * k) / static_cast<float>(ax));
  cs.assign(static_cast<size_t>(ws.N) * hd, 1.0f);
  sn.assign(static_cast<size_t>(ws.N) * hd, 0.0f);
  ang.assign(static_cast<size_t>(ws.N) * (hd / 2), 0.0f);
  auto put = [&](int row, int axis, int pos) {
    for (int k = 0; k < half; ++k) {
      const float a = static_cast<float>(pos) * fr[k];
      const float c = cosf(a), s = sinf(a);
      const size_t o = static_cast<size_t>(row) * hd + axis * ax + 2 * k;
      cs[o] = cs[o + 1] = c;
      sn[o] = sn[o + 1] = s;
      // the same angle (the float product the reference forms), reduced in double to [-pi, pi] so that the device's
      // fast sine / cosine work in their accurate range
      ang[static_cast<size_t>(row) * (hd / 2) + (axis * ax) / 2 + k] =
          static_cast<float>(remainder(static_cast<double>(a), 6.283185307179586476925286766559));
    }
  };
  for (int i = 0; i < ws.n_txt; ++i) put(i, 3, i);
  int row = ws.n_txt;
  for (int y = 0; y < ws.h; ++y)
    for (int x = 0; x < ws.w; ++x, ++row) {
      put(row, 1, y);
      put(row, 2, x);
    }
  for (const RefSpec &r : ws.refs)
    for (int y = 0; y < r.h; ++y)
      for (int x = 0; x < r.w; ++x, ++row) {
        put(row, 0, r.t_offset);
        put(row, 1, y);
        put(row, 2, x);
      }
}

void sampler_free(flux_cuda_sampler *s) {
  if (!s) return;
  if (s->ws) {
    cudaSetDevice(s->model->ctx->device);
    cudaStreamSynchronize(s->model->ctx->stream);
    if (s->model->ctx->copy_stream) cudaStreamSynchronize(s->model->ctx->copy_stream);
    for (void *p : s->ws->allocs) cudaFree(p);
    for (cudaEvent_t e : s->ws->prof_events) cudaEventDestroy(e);
    for (auto &g : s->ws->graphs) cudaGraphExecDestroy(g.exec);
    if (s->ws->ev0) cudaEventDestroy(s->ws->ev0);
    if (s->ws->ev1) cudaEventDestroy(s->ws->ev1);
    if (s->ws->ev_staged) cudaEventDestroy(s->ws->ev_staged);
    if (s->ws->ev_stage_free) cudaEventDestroy(s->ws->ev_stage_free);
    delete s->ws;
  }
  delete s;
}

int sampler_create(flux_cuda_model *m, int h, int w, int txt_seq, const RefSpec *refs, int num_refs, int batch,
                   int max_steps, flux_cuda_sampler **out) {
  *out = nullptr;
  if (!m || !m->finalized) {
    set_error("sampler: model is not finalized");
    return FLUX_CUDA_ERR_MODEL;
  }
  if (h <= 0 || w <= 0 || txt_seq <= 0 || num_refs < 0 || (num_refs && !refs) || batch < 1 || batch > 2 ||
      max_steps < 1) {
    set_error("sampler: bad shape h=%d w=%d txt=%d refs=%d batch=%d steps=%d", h, w, txt_seq, num_refs, batch,
              max_steps);
    return FLUX_CUDA_ERR_ARG;
  }
  cudaSetDevice(m->ctx->device);
  const ModelDims &d = m->d;
  flux_cuda_sampler *s = new flux_cuda_sampler();
  s->model = m;
  Workspace *ws = s->ws = new Workspace();
  ws->h = h;
  ws->w = w;
  ws->n_txt = txt_seq;
  ws->n_img = h * w;
  ws->B = batch;
  ws->max_steps = (max_steps + GEMV_S - 1) / GEMV_S * GEMV_S;
  for (int i = 0; i < num_refs; ++i) {
    if (refs[i].h <= 0 || refs[i].w <= 0) {
      sampler_free(s);
      set_error("sampler: bad reference shape");
      return FLUX_CUDA_ERR_ARG;
    }
    ws->refs.push_back(refs[i]);
    ws->n_ref += refs[i].h * refs[i].w;
  }
  ws->N = ws->n_txt + ws->n_img + ws->n_ref;
  const size_t rows = static_cast<size_t>(ws->B) * ws->N, hid = d.hidden, C = d.latent_ch;
  const size_t S = ws->max_steps;
  int rc = 0;
#define WS_ALLOC(ptr, count) \
  if (!rc) rc = dev_alloc(ws->allocs, &ws->ptr, (count))
  WS_ALLOC(hs, rows * hid);
  WS_ALLOC(txt0, static_cast<size_t>(ws->B) * ws->n_txt * hid);
  WS_ALLOC(norm, rows * hid);
  WS_ALLOC(qkv, rows * 3 * hid);
  WS_ALLOC(cat, rows * (hid + d.mlp));
  WS_ALLOC(tok, static_cast<size_t>(ws->n_img + ws->n_ref) * C);
  WS_ALLOC(ctx_bf, static_cast<size_t>(ws->B) * ws->n_txt * d.text_dim);
  WS_ALLOC(z, C * ws->n_img);
  WS_ALLOC(v, static_cast<size_t>(ws->B) * C * ws->n_img);
  WS_ALLOC(vcomb, C * ws->n_img);
  WS_ALLOC(vel_rec, S * C * ws->n_img);
  WS_ALLOC(z_in, C * ws->n_img);
  WS_ALLOC(ctx_in, static_cast<size_t>(ws->B) * ws->n_txt * d.text_dim);
  WS_ALLOC(ref_in, C * static_cast<size_t>(ws->n_ref ? ws->n_ref : 1));
  WS_ALLOC(sched, S + 1);
  WS_ALLOC(tsin, S * d.time_dim);
  WS_ALLOC(th, S * hid);
  WS_ALLOC(svec, S * hid);
  WS_ALLOC(mod, S * 17 * hid);
  WS_ALLOC(rope_cos, static_cast<size_t>(ws->N) * d.head_dim);
  WS_ALLOC(rope_sin, static_cast<size_t>(ws->N) * d.head_dim);
  WS_ALLOC(rope_ang, static_cast<size_t>(ws->N) * (d.head_dim / 2));
#undef WS_ALLOC
  if (!rc) rc = check_cuda(cudaEventCreate(&ws->ev0), "cudaEventCreate");
  if (!rc) rc = check_cuda(cudaEventCreate(&ws->ev1), "cudaEventCreate");
  if (!rc) {
    // zero what kernels read before anyone writes it (padding rows of the timestep buffers)
    cudaMemsetAsync(ws->sched, 0, (S + 1) * 4, m->ctx->stream);
    cudaMemsetAsync(ws->tsin, 0, S * d.time_dim * 4, m->ctx->stream);
    cudaMemsetAsync(ws->th, 0, S * hid * 4, m->ctx->stream);
    cudaMemsetAsync(ws->svec, 0, S * hid * 4, m->ctx->stream);
    std::vector<float> cs, sn, ang;
    build_rope(d, *ws, cs, sn, ang);
    rc = check_cuda(upload_h2d(m->ctx->stream, ws->rope_cos, cs.data(), cs.size() * 4), "upload rope");
    if (!rc) rc = check_cuda(upload_h2d(m->ctx->stream, ws->rope_sin, sn.data(), sn.size() * 4), "upload rope");
    if (!rc) rc = check_cuda(upload_h2d(m->ctx->stream, ws->rope_ang, ang.data(), ang.size() * 4), "upload rope");
  }
  if (rc) {
    sampler_free(s);
    return rc;
  }
  *out = s;
  return 0;
}

int sampler_upload(flux_cuda_sampler *s, const float *z0, const float *ctx0, const float *ctx1,
                   const float *const *ref_latents) {
  if (!s || !z0 || !ctx0) {
    set_error("upload: null argument");
    return FLUX_CUDA_ERR_ARG;
  }
  Workspace *ws = s->ws;
  const ModelDims &d = s->model->d;
  cudaStream_t st = s->model->ctx->stream;
  cudaSetDevice(s->model->ctx->device);
  if (ws->B == 2 && !ctx1) {
    set_error("upload: a batch-2 sampler needs two contexts");
    return FLUX_CUDA_ERR_ARG;
  }
  if (ws->refs.size() && !ref_latents) {
    set_error("upload: reference latents missing");
    return FLUX_CUDA_ERR_ARG;
  }
  const size_t C = d.latent_ch, ctx_n = static_cast<size_t>(ws->n_txt) * d.text_dim;
  int rc = check_cuda(cudaMemcpyAsync(ws->z_in, z0, C * ws->n_img * 4, cudaMemcpyDefault, st), "upload z");
  if (!rc) rc = check_cuda(cudaMemcpyAsync(ws->ctx_in, ctx0, ctx_n * 4, cudaMemcpyDefault, st), "upload ctx");
  if (!rc && ws->B == 2)
    rc = check_cuda(cudaMemcpyAsync(ws->ctx_in + ctx_n, ctx1, ctx_n * 4, cudaMemcpyDefault, st), "upload ctx");
  size_t off = 0;
  for (size_t i = 0; !rc && i < ws->refs.size(); ++i) {
    const size_t n = static_cast<size_t>(ws->refs[i].h) * ws->refs[i].w;
    if (!ref_latents[i]) {
      set_error("upload: reference latent %zu is null", i);
      return FLUX_CUDA_ERR_ARG;
    }
    rc = check_cuda(cudaMemcpyAsync(ws->ref_in + off * C, ref_latents[i], C * n * 4, cudaMemcpyDefault, st),
                    "upload ref");
    off += n;
  }
  return rc;
}

// ------------------------------------------------------------------------------------------------ forward
// 16-bit tensors are f16 by default (model->f16): same tensor-core rate as bf16, 3 more mantissa bits where the
// rounding error of the step comes from (the GEMM A operands). The guidance pair needs them:
// v_u + g (v_c - v_u) multiplies per-pass errors by up to g + |1 - g|.
#define ACT_F16 (m->f16 ? 1 : 0)

struct Launcher {
  flux_cuda_model *m;
  Workspace *ws;
  cudaStream_t st;
  int rc = 0;
  int group = BG_EDGE;  // part of the forward the next launches belong to

  void fail(const char *what, int code) {
    if (!rc) {
      rc = code <= -8 ? FLUX_CUDA_ERR_CUDA : FLUX_CUDA_ERR_ARG;
      set_error("%s failed (rc %d, cuda: %s)", what, code, cudaGetErrorString(cudaGetLastError()));
    }
  }
  // begin(cls) ... launch ... count(): counts the launch and, when profiling, brackets it with an event pair
  void begin(int cls) {
    if (!ws->profiling) return;
    if (ws->prof_used * 2 + 2 > ws->prof_events.size()) {
      cudaEvent_t a, b;
      if (cudaEventCreate(&a) != cudaSuccess || cudaEventCreate(&b) != cudaSuccess) return;
      ws->prof_events.push_back(a);
      ws->prof_events.push_back(b);
      ws->prof_class.push_back(cls);
      ws->prof_group.push_back(group);
    }
    ws->prof_class[ws->prof_used] = cls;
    ws->prof_group[ws->prof_used] = group;
    cudaEventRecord(ws->prof_events[ws->prof_used * 2], st);
    open = true;
  }
  void count() {
    ws->launches++;
    if (open) {
      cudaEventRecord(ws->prof_events[ws->prof_used * 2 + 1], st);
      ws->prof_used++;
      open = false;
    }
  }
  bool open = false;

  // [Q|K|V] projection with the per-head RMSNorm and the rotation applied in the epilogue
  EpiSeg seg_qkv(void *out, int pos0, const float *nq_t, const float *nk_t, const float *nq_i, const float *nk_i) {
    EpiSeg s = seg(EPI_QKV_NORM_ROPE, out, 3 * m->d.hidden, 0);
    s.out_f16 = ACT_F16;
    s.qk.wq_txt = nq_t;
    s.qk.wk_txt = nk_t;
    s.qk.wq_img = nq_i;
    s.qk.wk_img = nk_i;
    s.qk.cos_t = ws->rope_cos;
    s.qk.sin_t = ws->rope_sin;
    s.qk.ang = ws->rope_ang;
    s.qk.pos0 = pos0;
    s.qk.seq = ws->N;
    s.qk.n_txt = ws->n_txt;
    s.qk.q_cols = m->d.hidden;
    s.qk.k_cols = m->d.hidden;
    s.qk.half_split = 0;
    return s;
  }
  EpiSeg seg(int mode, void *out, long long ld, int col0, const float *gate = nullptr) {
    EpiSeg s;
    memset(&s, 0, sizeof(s));
    s.out_f16 = ACT_F16;
    s.mode = mode;
    s.col0 = col0;
    s.ld = ld;
    s.out = out;
    s.gate = gate;
    return s;
  }
  // One problem per entry; launched together.
  struct Prob {
    const void *X;
    long long ldx;
    const void *W;
    int M, N, K;
    EpiSeg s0;
    int n_split;
    EpiSeg s1;
  };
  void gemm(const Prob *pr, int n, int bn) {
    if (rc) return;
    GemmParams P;
    memset(&P, 0, sizeof(P));
    P.nprob = n;
    P.err = m->ctx->err_dev;
    const bool pair = bn == 256 && m->ctx->gemm_pair;
    for (int i = 0; i < n; ++i) {
      int r = pair ? gemm_make_problem_pair(&P.p[i], pr[i].X, pr[i].ldx, pr[i].W, pr[i].M, pr[i].N, pr[i].K)
                   : gemm_make_problem(&P.p[i], pr[i].X, pr[i].ldx, pr[i].W, pr[i].M, pr[i].N, pr[i].K, bn);
      if (r) return fail("gemm_make_problem", r);
      P.p[i].x_f16 = ACT_F16;
      P.p[i].seg[0] = pr[i].s0;
      if (pr[i].n_split > 0 && pr[i].n_split < pr[i].N) {
        P.p[i].n_split = pr[i].n_split;
        P.p[i].seg[1] = pr[i].s1;
      }
    }
    begin(KC_GEMM);
    int r = pair ? gemm2_launch(&P, m->ctx->num_sms, st) : gemm_launch(&P, bn, m->ctx->num_sms, st);
    count();
    if (r) return fail("gemm_launch", r);
  }
  void adaln(int row0, int rows, const float *sh_t, const float *sc_t, const float *sh_i, const float *sc_i) {
    if (rc) return;
    begin(KC_ADALN);
    // This launch always follows a paired (cluster) GEMM. A small grid launched with programmatic dependent launch
    // directly behind such a kernel is the one pattern a device stall was ever traced to (in the VAE, cause not
    // found), so it goes out in plain stream order; the GEMM behind it still overlaps its prologue with this kernel.
    PdlOff plain_launch;
    int r = launch_adaln(ws->hs, ws->norm, row0, rows, m->d.hidden, ws->N, ws->n_txt, ACT_F16, sh_t, sc_t, sh_i, sc_i,
                         st, m->ctx->err_dev + 1);
    count();
    if (r) return fail("adaln", r);
  }
  void qknorm(const float *nq_t, const float *nk_t, const float *nq_i, const float *nk_i) {
    if (rc) return;
    const int h = m->d.hidden;
    begin(KC_QKNORM);
    int r = launch_qk_norm_rope(ws->qkv, 3 * h, 0, h, ws->N, ws->B, m->d.heads, ws->n_txt, nq_t, nk_t, nq_i, nk_i,
                                ws->rope_cos, ws->rope_sin, st);
    count();
    if (r) return fail("qk_norm_rope", r);
  }
  void attention() {
    if (rc) return;
    const int h = m->d.hidden;
    AttnParams A;
    int r = attn2_make_params(&A, ws->qkv, ws->B, ws->N, 3 * h, 0, h, 2 * h, ws->cat, h + m->d.mlp, 0, m->d.heads,
                              ACT_F16, m->ctx->err_dev);
    if (r) return fail("attn_make_params", r);
    begin(KC_ATTN);
    r = attn_launch_version(m->ctx->attn_version, &A, st);
    count();
    if (r) return fail("attn_launch", r);
  }
};

// One DiT forward over the workspace's current tokens, using modulation row `step` (ws->mod + step*17h).
// Writes the velocity of batch element b to ws->v + b*C*n_img (channel-major, like the reference's output).
static int forward_step(flux_cuda_model *m, Workspace *ws, int step, cudaStream_t st) {
  const ModelDims &d = m->d;
  const int h = d.hidden, mlp = d.mlp, N = ws->N, B = ws->B, n_txt = ws->n_txt, n_it = ws->n_img + ws->n_ref;
  const int C = d.latent_ch;
  const long long cat_ld = h + mlp;
  Launcher L{m, ws, st};
  const float *mod = ws->mod + static_cast<size_t>(step) * 17 * h;
  const float *mi = mod, *mt = mod + 6 * h, *ms = mod + 12 * h, *mf = mod + 15 * h;

  // target tokens of the current latent: NCHW f32 -> NLC bf16 (reference tokens were packed once per sample)
  L.begin(KC_OTHER);
  if (launch_pack_tokens(ws->z, ws->tok, C, ws->n_img, ACT_F16, st, m->ctx->err_dev + 1)) L.fail("pack_tokens", -8);
  L.count();
  // embedders: image tokens every step; the text projection is step-invariant and was computed once
  {
    Launcher::Prob pr[2];
    for (int b = 0; b < B; ++b)
      pr[b] = {ws->tok, C, m->x_emb, n_it, h, C,
               L.seg(EPI_STORE_F32, ws->hs + (static_cast<size_t>(b) * N + n_txt) * h, h, 0), 0, {}};
    L.gemm(pr, B, 256);
    if (!L.rc &&
        cudaMemcpy2DAsync(ws->hs, static_cast<size_t>(N) * h * 4, ws->txt0, static_cast<size_t>(n_txt) * h * 4,
                          static_cast<size_t>(n_txt) * h * 4, B, cudaMemcpyDeviceToDevice, st) != cudaSuccess)
      L.fail("copy text stream", -8);
  }

  // ---- double-stream blocks (flux_transformer.c:1774-1986)
  L.group = BG_DOUBLE;
  for (int blk = 0; blk < d.n_double; ++blk) {
    const DoubleW &w = m->dbl[blk];
    Launcher::Prob pr[4];
    auto per_stream = [&](auto make) {
      int n = 0;
      for (int b = 0; b < B; ++b)
        for (int s = 0; s < 2; ++s) pr[n++] = make(b, s, static_cast<size_t>(b) * N + (s ? n_txt : 0), s ? n_it : n_txt);
      return n;
    };
    L.adaln(0, B * N, mt + 0 * h, mt + 1 * h, mi + 0 * h, mi + 1 * h);
    int n = per_stream([&](int, int s, size_t row, int M) {
      return Launcher::Prob{ws->norm + row * h, h, w.qkv[s], M, 3 * h, h,
                            L.seg_qkv(ws->qkv + row * 3 * h, s ? n_txt : 0, w.nq[0], w.nk[0], w.nq[1], w.nk[1]), 0, {}};
    });
    L.gemm(pr, n, 256);
    L.attention();
    n = per_stream([&](int, int s, size_t row, int M) {
      return Launcher::Prob{ws->cat + row * cat_ld, cat_ld, w.out[s], M, h, h,
                            L.seg(EPI_GATED_RES_F32, ws->hs + row * h, h, 0, (s ? mi : mt) + 2 * h), 0, {}};
    });
    L.gemm(pr, n, 256);
    L.adaln(0, B * N, mt + 3 * h, mt + 4 * h, mi + 3 * h, mi + 4 * h);
    n = per_stream([&](int, int s, size_t row, int M) {
      return Launcher::Prob{ws->norm + row * h, h, w.ffin[s], M, 2 * mlp, h,
                            L.seg(EPI_SWIGLU_BF16, ws->cat + row * cat_ld, cat_ld, h), 0, {}};
    });
    L.gemm(pr, n, 256);
    n = per_stream([&](int, int s, size_t row, int M) {
      return Launcher::Prob{ws->cat + row * cat_ld + h, cat_ld, w.ffout[s], M, h, mlp,
                            L.seg(EPI_GATED_RES_F32, ws->hs + row * h, h, 0, (s ? mi : mt) + 5 * h), 0, {}};
    });
    L.gemm(pr, n, 256);
  }

  // ---- single-stream blocks (flux_transformer.c:2992-3109)
  L.group = BG_SINGLE;
  for (int blk = 0; blk < d.n_single; ++blk) {
    const SingleW &w = m->sgl[blk];
    L.adaln(0, B * N, ms, ms + h, ms, ms + h);
    Launcher::Prob p1{ws->norm, h, w.lin1, B * N, 3 * h + 2 * mlp, h,
                      L.seg_qkv(ws->qkv, 0, w.nq, w.nk, w.nq, w.nk), 3 * h,
                      L.seg(EPI_SWIGLU_BF16, ws->cat, cat_ld, h)};
    L.gemm(&p1, 1, 256);
    L.attention();
    Launcher::Prob p2{ws->cat, cat_ld, w.lin2, B * N, h, h + mlp,
                      L.seg(EPI_GATED_RES_F32, ws->hs, h, 0, ms + 2 * h), 0, {}};
    L.gemm(&p2, 1, 256);
  }

  // ---- final layer on the target tokens only: modulation is (scale, shift) (flux_transformer.c:3523-3552)
  L.group = BG_FINAL;
  {
    Launcher::Prob pr[2];
    for (int b = 0; b < B; ++b) {
      const size_t row = static_cast<size_t>(b) * N + n_txt;
      L.adaln(static_cast<int>(row), ws->n_img, mf + h, mf, mf + h, mf);
      pr[b] = {ws->norm + row * h, h, m->proj_out, ws->n_img, C, h,
               L.seg(EPI_STORE_F32_T, ws->v + static_cast<size_t>(b) * C * ws->n_img, ws->n_img, 0), 0, {}};
    }
    L.gemm(pr, B, 128);
  }
  return L.rc;
}

// Everything that depends on the inputs but not on the step: bf16 context and its projection, reference
// tokens, and the timestep MLP + modulation vectors of ALL steps (the schedule is known up front).
static int prepare(flux_cuda_model *m, Workspace *ws, int num_steps, cudaStream_t st) {
  const ModelDims &d = m->d;
  const int h = d.hidden, C = d.latent_ch;
  Launcher L{m, ws, st};
  const long long ctx_n = static_cast<long long>(ws->B) * ws->n_txt * d.text_dim;
  L.begin(KC_OTHER);
  if (launch_f32_to_bf16(ws->ctx_in, ws->ctx_bf, ctx_n, ACT_F16, st, m->ctx->err_dev + 1)) L.fail("f32_to_bf16", -8);
  L.count();
  Launcher::Prob pc{ws->ctx_bf, d.text_dim, m->ctx_emb, ws->B * ws->n_txt, h, d.text_dim,
                    L.seg(EPI_STORE_F32, ws->txt0, h, 0), 0, {}};
  L.gemm(&pc, 1, 256);
  size_t off = 0;
  for (const RefSpec &r : ws->refs) {
    const int n = r.h * r.w;
    L.begin(KC_OTHER);
    if (launch_pack_tokens(ws->ref_in + off * C, ws->tok + (ws->n_img + off) * C, C, n, ACT_F16, st,
                           m->ctx->err_dev + 1))
      L.fail("pack refs", -8);
    L.count();
    off += n;
  }
  L.begin(KC_OTHER);
  if (launch_timestep_sincos(ws->sched, num_steps, d.time_dim, ws->tsin, st)) L.fail("timestep_sincos", -8);
  L.count();
  for (int s0 = 0; s0 < num_steps && !L.rc; s0 += GEMV_S) {
    L.begin(KC_OTHER);  // the three projections of this group of steps share one event pair
    int r = launch_gemv_multi(m->t1, ws->tsin + static_cast<size_t>(s0) * d.time_dim,
                              ws->th + static_cast<size_t>(s0) * h, h, d.time_dim, 1, ACT_F16, st);
    if (!r)  // svec = silu(t_emb): every consumer of t_emb applies SiLU first (flux_transformer.c:3227-3230)
      r = launch_gemv_multi(m->t2, ws->th + static_cast<size_t>(s0) * h, ws->svec + static_cast<size_t>(s0) * h, h, h,
                            1, ACT_F16, st);
    if (!r)
      r = launch_gemv_multi(m->mod_all, ws->svec + static_cast<size_t>(s0) * h,
                            ws->mod + static_cast<size_t>(s0) * 17 * h, 17 * h, h, 0, ACT_F16, st);
    L.count();
    if (r) L.fail("modulation gemv", r);
    ws->launches += 2;
  }
  return L.rc;
}

// Queues steps [first, first + count) on `st` (directly, or into a stream capture).
static int enqueue_steps(flux_cuda_model *m, Workspace *ws, int num_steps, int first, int count, float guidance,
                         int record_velocities, int apply_update, cudaStream_t st) {
  const size_t n = static_cast<size_t>(m->d.latent_ch) * ws->n_img;
  int rc = 0;
  if (first == 0) {
    rc = check_cuda(cudaMemcpyAsync(ws->z, ws->z_in, n * 4, cudaMemcpyDeviceToDevice, st), "init latent");
    if (!rc) rc = prepare(m, ws, num_steps, st);
  }
  for (int i = first; !rc && i < first + count; ++i) {
    rc = forward_step(m, ws, i, st);
    if (rc) break;
    const float *v = ws->v;
    if (ws->B == 2) {
      // row 0 = conditional, row 1 = unconditional: v = v_u + g (v_c - v_u) (flux_sample.c:495-499)
      if (launch_cfg_euler(ws->z, ws->v, ws->v + n, ws->vcomb, guidance, ws->sched, i, static_cast<long long>(n),
                           apply_update, st))
        rc = FLUX_CUDA_ERR_CUDA;
      v = ws->vcomb;
      ws->launches++;
    } else if (apply_update) {
      if (launch_euler(ws->z, ws->v, ws->sched, i, static_cast<long long>(n), st)) rc = FLUX_CUDA_ERR_CUDA;
      ws->launches++;
    }
    if (!rc && record_velocities)
      rc = check_cuda(cudaMemcpyAsync(ws->vel_rec + static_cast<size_t>(i) * n, v, n * 4, cudaMemcpyDeviceToDevice, st),
                      "record velocity");
  }
  return rc;
}

// Inputs of the NEXT image: host -> device on the context's copy stream into staging buffers, so that the PCIe
// transfer runs under the image that is being computed. The next run(first = 0) waits for the transfer and moves
// the staged inputs into place with device-to-device copies on the context's stream.
int sampler_stage_inputs(flux_cuda_sampler *s, const float *z0, const float *ctx0, const float *ctx1,
                         const float *const *ref_latents) {
  if (!s || !z0 || !ctx0) {
    set_error("stage_inputs: null argument");
    return FLUX_CUDA_ERR_ARG;
  }
  Workspace *ws = s->ws;
  flux_cuda_ctx *c = s->model->ctx;
  const ModelDims &d = s->model->d;
  cudaSetDevice(c->device);
  if ((ws->B == 2 && !ctx1) || (ws->refs.size() && !ref_latents)) {
    set_error("stage_inputs: a context or the reference latents are missing");
    return FLUX_CUDA_ERR_ARG;
  }
  const size_t C = d.latent_ch, ctx_n = static_cast<size_t>(ws->n_txt) * d.text_dim;
  int rc = 0;
  if (!c->copy_stream) rc = check_cuda(cudaStreamCreateWithFlags(&c->copy_stream, cudaStreamNonBlocking), "copy stream");
  if (!rc && !ws->stage_z) {
    rc = dev_alloc(ws->allocs, &ws->stage_z, C * ws->n_img);
    if (!rc) rc = dev_alloc(ws->allocs, &ws->stage_ctx, static_cast<size_t>(ws->B) * ctx_n);
    if (!rc) rc = dev_alloc(ws->allocs, &ws->stage_ref, C * static_cast<size_t>(ws->n_ref ? ws->n_ref : 1));
    if (!rc) rc = check_cuda(cudaEventCreateWithFlags(&ws->ev_staged, cudaEventDisableTiming), "cudaEventCreate");
    if (!rc) rc = check_cuda(cudaEventCreateWithFlags(&ws->ev_stage_free, cudaEventDisableTiming), "cudaEventCreate");
  }
  if (rc) return rc;
  cudaStream_t cs = c->copy_stream;
  // the staging buffers are free once the previous staged inputs have been moved into place
  if (ws->stage_used) rc = check_cuda(cudaStreamWaitEvent(cs, ws->ev_stage_free, 0), "stage wait");
  if (!rc) rc = check_cuda(cudaMemcpyAsync(ws->stage_z, z0, C * ws->n_img * 4, cudaMemcpyDefault, cs), "stage z");
  if (!rc) rc = check_cuda(cudaMemcpyAsync(ws->stage_ctx, ctx0, ctx_n * 4, cudaMemcpyDefault, cs), "stage ctx");
  if (!rc && ws->B == 2)
    rc = check_cuda(cudaMemcpyAsync(ws->stage_ctx + ctx_n, ctx1, ctx_n * 4, cudaMemcpyDefault, cs), "stage ctx");
  size_t off = 0;
  for (size_t i = 0; !rc && i < ws->refs.size(); ++i) {
    const size_t n = static_cast<size_t>(ws->refs[i].h) * ws->refs[i].w;
    if (!ref_latents[i]) {
      set_error("stage_inputs: reference latent %zu is null", i);
      return FLUX_CUDA_ERR_ARG;
    }
    rc = check_cuda(cudaMemcpyAsync(ws->stage_ref + off * C, ref_latents[i], C * n * 4, cudaMemcpyDefault, cs), "stage ref");
    off += n;
  }
  if (!rc) rc = check_cuda(cudaEventRecord(ws->ev_staged, cs), "stage record");
  if (!rc) ws->staged_pending = true;
  return rc;
}

// Moves staged inputs into place (called by run at first == 0), ordered on the context's stream.
static int consume_staged(flux_cuda_sampler *s) {
  Workspace *ws = s->ws;
  if (!ws->staged_pending) return 0;
  const ModelDims &d = s->model->d;
  cudaStream_t st = s->model->ctx->stream;
  const size_t C = d.latent_ch, ctx_n = static_cast<size_t>(ws->B) * ws->n_txt * d.text_dim;
  int rc = check_cuda(cudaStreamWaitEvent(st, ws->ev_staged, 0), "staged wait");
  if (!rc) rc = check_cuda(cudaMemcpyAsync(ws->z_in, ws->stage_z, C * ws->n_img * 4, cudaMemcpyDeviceToDevice, st), "staged z");
  if (!rc) rc = check_cuda(cudaMemcpyAsync(ws->ctx_in, ws->stage_ctx, ctx_n * 4, cudaMemcpyDeviceToDevice, st), "staged ctx");
  if (!rc && ws->n_ref)
    rc = check_cuda(cudaMemcpyAsync(ws->ref_in, ws->stage_ref, C * ws->n_ref * 4, cudaMemcpyDeviceToDevice, st), "staged ref");
  if (!rc) rc = check_cuda(cudaEventRecord(ws->ev_stage_free, st), "staged record");
  ws->staged_pending = false;
  ws->stage_used = true;
  return rc;
}

// Device -> host copy of the latent, ordered on the context's stream; does not wait (flux_cuda_ctx_sync does).
int sampler_download_async(flux_cuda_sampler *s, float *latent_out) {
  if (!s || !latent_out) return FLUX_CUDA_ERR_ARG;
  flux_cuda_model *m = s->model;
  cudaSetDevice(m->ctx->device);
  const size_t n = static_cast<size_t>(m->d.latent_ch) * s->ws->n_img;
  return check_cuda(cudaMemcpyAsync(latent_out, s->ws->z, n * 4, cudaMemcpyDeviceToHost, m->ctx->stream), "download");
}

int sampler_run(flux_cuda_sampler *s, const float *schedule, int num_steps, int first, int count, float guidance,
                int record_velocities, int apply_update) {
  if (!s || !schedule || num_steps < 1 || first < 0 || count < 1 || first + count > num_steps) {
    set_error("run: bad argument");
    return FLUX_CUDA_ERR_ARG;
  }
  flux_cuda_model *m = s->model;
  Workspace *ws = s->ws;
  if (num_steps > ws->max_steps) {
    set_error("run: %d steps exceed the sampler's capacity of %d", num_steps, ws->max_steps);
    return FLUX_CUDA_ERR_ARG;
  }
  cudaSetDevice(m->ctx->device);
  cudaStream_t st = m->ctx->stream;
  ws->launches = 0;
  ws->prof_used = 0;
  ws->last_steps = num_steps;
  cudaEventRecord(ws->ev0, st);
  int rc = 0;
  if (first == 0) rc = consume_staged(s);
  if (rc) return rc;
  if (first == 0)
    // A copy from pageable memory returns once the source has been staged, so `schedule` is free on return and
    // no host synchronisation is needed between consecutive runs. It stays outside the captured graph because a
    // graph would bake the caller's pointer in.
    rc = check_cuda(cudaMemcpyAsync(ws->sched, schedule, (num_steps + 1) * 4, cudaMemcpyHostToDevice, st), "schedule");
  if (rc) return rc;

  if (ws->profiling || !ws->use_graphs || first != 0 || count != num_steps) {
    rc = enqueue_steps(m, ws, num_steps, first, count, guidance, record_velocities, apply_update, st);
  } else {
    // The loop is ~150 launches per step: replay it as one CUDA graph so that launch gaps do not add up.
    Workspace::GraphEntry *hit = nullptr;
    for (auto &g : ws->graphs)
      if (g.num_steps == num_steps && g.first == first && g.count == count && g.record == record_velocities &&
          g.apply == apply_update && g.guidance == guidance)
        hit = &g;
    if (!hit) {
      cudaGraph_t graph = nullptr;
      rc = check_cuda(cudaStreamBeginCapture(st, cudaStreamCaptureModeThreadLocal), "begin capture");
      if (rc) return rc;
      rc = enqueue_steps(m, ws, num_steps, first, count, guidance, record_velocities, apply_update, st);
      cudaError_t e = cudaStreamEndCapture(st, &graph);
      if (!rc && e != cudaSuccess) rc = check_cuda(e, "end capture");
      cudaGraphExec_t exec = nullptr;
      if (!rc) rc = check_cuda(cudaGraphInstantiate(&exec, graph, 0), "graph instantiate");
      if (graph) cudaGraphDestroy(graph);
      if (rc) return rc;
      if (ws->graphs.size() >= 16) {  // bounded cache: drop the oldest
        cudaGraphExecDestroy(ws->graphs.front().exec);
        ws->graphs.erase(ws->graphs.begin());
      }
      ws->graphs.push_back({num_steps, first, count, record_velocities, apply_update, guidance, exec, ws->launches});
      hit = &ws->graphs.back();
    }
    ws->launches = hit->launches;
    rc = check_cuda(cudaGraphLaunch(hit->exec, st), "graph launch");
  }
  cudaEventRecord(ws->ev1, st);
  return rc;
}

int sampler_download(flux_cuda_sampler *s, float *latent_out, float *velocities_out) {
  if (!s) return FLUX_CUDA_ERR_ARG;
  flux_cuda_model *m = s->model;
  Workspace *ws = s->ws;
  cudaSetDevice(m->ctx->device);
  cudaStream_t st = m->ctx->stream;
  const size_t n = static_cast<size_t>(m->d.latent_ch) * ws->n_img;
  int rc = 0;
  if (latent_out) rc = check_cuda(cudaMemcpyAsync(latent_out, ws->z, n * 4, cudaMemcpyDeviceToHost, st), "download");
  if (!rc && velocities_out)
    rc = check_cuda(cudaMemcpyAsync(velocities_out, ws->vel_rec, n * 4 * ws->last_steps, cudaMemcpyDeviceToHost, st),
                    "download velocities");
  if (!rc) rc = ctx_sync_check(m->ctx);
  return rc;
}

int sampler_profile(flux_cuda_sampler *s, float *ms_by_class, long long *launches_by_class) {
  if (!s || !ms_by_class || !launches_by_class) return FLUX_CUDA_ERR_ARG;
  Workspace *ws = s->ws;
  for (int c = 0; c < KC_COUNT; ++c) {
    ms_by_class[c] = 0.f;
    launches_by_class[c] = 0;
  }
  for (size_t i = 0; i < ws->prof_used; ++i) {
    float ms = 0.f;
    if (cudaEventElapsedTime(&ms, ws->prof_events[2 * i], ws->prof_events[2 * i + 1]) != cudaSuccess) {
      set_error("profile: events not complete (synchronize first)");
      return FLUX_CUDA_ERR_CUDA;
    }
    ms_by_class[ws->prof_class[i]] += ms;
    launches_by_class[ws->prof_class[i]]++;
  }
  return 0;
}

int sampler_profile_groups(flux_cuda_sampler *s, float *ms_by_group) {
  if (!s || !ms_by_group) return FLUX_CUDA_ERR_ARG;
  Workspace *ws = s->ws;
  for (int g = 0; g < BG_COUNT; ++g) ms_by_group[g] = 0.f;
  for (size_t i = 0; i < ws->prof_used; ++i) {
    float ms = 0.f;
    if (cudaEventElapsedTime(&ms, ws->prof_events[2 * i], ws->prof_events[2 * i + 1]) != cudaSuccess) {
      set_error("profile: events not complete (synchronize first)");
      return FLUX_CUDA_ERR_CUDA;
    }
    ms_by_group[ws->prof_group[i]] += ms;
  }
  return 0;
}

}  // namespace fx
