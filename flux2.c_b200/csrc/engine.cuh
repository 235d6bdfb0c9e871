// Device-resident model and sampler state of the denoising engine.
//
// Layout in HBM (all row-major):
//   weights       bf16, [out, in] as in the file; Q/K/V of a stream concatenated to one [3h, h] matrix;
//                 gate/up halves of every SwiGLU input projection interleaved in 128-row blocks so that
//                 one 256-column GEMM tile holds matching gate and up columns; the four modulation
//                 projections concatenated to one [17h, h] matrix; QK-norm vectors f32.
//   activations   one sequence [txt ; img ; refs] per batch element (batch = 2 only for the
//                 classifier-free-guidance pair), residual stream f32 [B*N, h]; AdaLN output, fused
//                 Q|K|V and [attention | mlp] buffers bf16.
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <functional>
#include <set>
#include <string>
#include <vector>

#include "context.cuh"

namespace fx {

struct ModelDims {
  int hidden, heads, head_dim, mlp, n_double, n_single, text_dim, latent_ch, time_dim;
  float rope_theta;
  int axis_dim;
};

struct DoubleW {  // index 0 = text stream, 1 = image stream
  __nv_bfloat16 *qkv[2], *out[2], *ffin[2], *ffout[2];
  float *nq[2], *nk[2];
};
struct SingleW {
  __nv_bfloat16 *lin1, *lin2;
  float *nq, *nk;
};

struct RefSpec {
  int h, w, t_offset;
};

struct Workspace;

}  // namespace fx

struct flux_cuda_model {
  flux_cuda_ctx *ctx = nullptr;
  fx::ModelDims d{};
  __nv_bfloat16 *x_emb = nullptr, *ctx_emb = nullptr, *t1 = nullptr, *t2 = nullptr, *mod_all = nullptr,
                *proj_out = nullptr;
  std::vector<fx::DoubleW> dbl;
  std::vector<fx::SingleW> sgl;
  std::vector<void *> allocs;
  void *staging = nullptr;
  size_t staging_bytes = 0;
  std::set<std::string> seen;
  size_t expected = 0;
  bool finalized = false;
  bool f16 = true;  // weights were converted to f16 at upload (else kept bf16); activations follow
  size_t weight_bytes = 0;
};

struct flux_cuda_sampler {
  flux_cuda_model *model = nullptr;
  fx::Workspace *ws = nullptr;
};

namespace fx {

struct Workspace {
  int h = 0, w = 0, n_txt = 0, n_img = 0, n_ref = 0, N = 0, B = 1, max_steps = 0;
  std::vector<RefSpec> refs;
  std::vector<void *> allocs;
  float *hs = nullptr, *txt0 = nullptr;
  __nv_bfloat16 *norm = nullptr, *qkv = nullptr, *cat = nullptr, *tok = nullptr, *ctx_bf = nullptr;
  float *z = nullptr, *v = nullptr, *vcomb = nullptr, *vel_rec = nullptr;
  float *z_in = nullptr, *ctx_in = nullptr, *ref_in = nullptr;  // raw uploads
  // inputs of the NEXT image, copied in on the context's copy stream while the current image runs
  float *stage_z = nullptr, *stage_ctx = nullptr, *stage_ref = nullptr;
  cudaEvent_t ev_staged = nullptr, ev_stage_free = nullptr;
  bool staged_pending = false, stage_used = false;
  float *sched = nullptr, *tsin = nullptr, *th = nullptr, *svec = nullptr, *mod = nullptr;
  float *rope_cos = nullptr, *rope_sin = nullptr;
  float *rope_ang = nullptr;  // [N, 64]: rotation angle of every consecutive pair, reduced to [-pi, pi]
  cudaEvent_t ev0 = nullptr, ev1 = nullptr;
  int last_steps = 0;
  long long launches = 0;  // kernels launched by the last run
  // captured CUDA graphs of the run loop, one per distinct (steps, range, guidance, flags)
  struct GraphEntry {
    int num_steps, first, count, record, apply;
    float guidance;
    cudaGraphExec_t exec;
    long long launches;
  };
  std::vector<GraphEntry> graphs;
  bool use_graphs = true;
  // optional per-kernel-class timing of a run: one CUDA event pair per launch
  bool profiling = false;
  std::vector<cudaEvent_t> prof_events;  // pairs: [2i] before, [2i+1] after launch i
  std::vector<int> prof_class;
  std::vector<int> prof_group;  // BlockGroup of each profiled launch
  size_t prof_used = 0;
};

enum KernelClass : int { KC_GEMM = 0, KC_ATTN = 1, KC_ADALN = 2, KC_QKNORM = 3, KC_OTHER = 4, KC_COUNT = 5 };
// Which part of the forward a launch belongs to: the reference keeps wall-clock totals per part
// (flux_timing_transformer_double / _single / _final, flux_sample.c:22-39).
enum BlockGroup : int { BG_EDGE = 0, BG_DOUBLE = 1, BG_SINGLE = 2, BG_FINAL = 3, BG_COUNT = 4 };

int model_create(flux_cuda_ctx *ctx, const ModelDims &d, flux_cuda_model **out);
int model_set_tensor(flux_cuda_model *m, const char *name, const void *data, int dtype, const long long *shape,
                     int ndim);
int model_finalize(flux_cuda_model *m);
void model_free(flux_cuda_model *m);
int model_load_safetensors(flux_cuda_ctx *ctx, const char *path, flux_cuda_model **out);
int safetensors_for_each(const char *path,
                         const std::function<int(const char *, const void *, int, const long long *, int)> &visit);
// Host-side conversion of `count` elements (dtype 0/1/2 = F32/F16/BF16) to 16-bit words in the wanted format;
// returns `data` itself when no conversion is needed, else a pointer into `tmp`.
const uint16_t *to_half_host(const void *data, int dtype, size_t count, std::vector<uint16_t> &tmp, bool want_f16);
float half_to_f32_host(uint16_t bits, int dtype);
// Puts elements [off, off + count) of `data` (dtype 0/1/2) at `dst` (device, 16-byte aligned) in the wanted 16-bit
// format, complete on return. 16-bit sources are copied as they are and, if they hold the other 16-bit format,
// converted in place by a kernel; only f32 sources are converted on the host (tmp is its scratch).
int upload_16(flux_cuda_ctx *ctx, void *dst, const void *data, int dtype, size_t off, size_t count, bool want_f16,
              std::vector<uint16_t> &tmp);

int sampler_create(flux_cuda_model *m, int h, int w, int txt_seq, const RefSpec *refs, int num_refs, int batch,
                   int max_steps, flux_cuda_sampler **out);
void sampler_free(flux_cuda_sampler *s);
int sampler_upload(flux_cuda_sampler *s, const float *z0, const float *ctx0, const float *ctx1,
                   const float *const *ref_latents);
// guidance is used only when the sampler was created with batch 2 (row 0 = conditional context).
// Runs steps [first, first + count) of a num_steps schedule. first == 0 (re)starts from the uploaded latent and
// prepares the step-invariant inputs; first > 0 continues from the current latent.
int sampler_run(flux_cuda_sampler *s, const float *schedule, int num_steps, int first, int count, float guidance,
                int record_velocities, int apply_update);
int sampler_download(flux_cuda_sampler *s, float *latent_out, float *velocities_out);
int sampler_stage_inputs(flux_cuda_sampler *s, const float *z0, const float *ctx0, const float *ctx1,
                         const float *const *ref_latents);
int sampler_download_async(flux_cuda_sampler *s, float *latent_out);
// Sums the event pairs of the last profiled run per kernel class (call after a sync).
int sampler_profile(flux_cuda_sampler *s, float *ms_by_class, long long *launches_by_class);
// The same event pairs summed per BlockGroup.
int sampler_profile_groups(flux_cuda_sampler *s, float *ms_by_group);

}  // namespace fx
