/*
 * flux_cuda.h - C ABI of the B200 (sm_100a) denoising engine for FLUX.2-klein.
 *
 * Plain C: opaque handles, POD structs, int status codes (0 = success, negative = error; the text
 * of the last error of the calling thread is returned by flux_cuda_last_error()). Nothing here
 * throws, exits or falls back to the CPU. Host buffers are borrowed for the duration of a call.
 * A context and the objects created from it must be used from one host thread at a time;
 * different contexts (different GPUs) are independent.
 */
#ifndef FLUX_CUDA_H
#define FLUX_CUDA_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define FLUX_CUDA_OK 0
#define FLUX_CUDA_ERR_ARG (-1)     /* bad argument / shape / alignment */
#define FLUX_CUDA_ERR_CUDA (-2)    /* a CUDA runtime or driver call failed */
#define FLUX_CUDA_ERR_KERNEL (-3)  /* a kernel gave up on a bounded wait and reported it */
#define FLUX_CUDA_ERR_IO (-4)      /* file missing / truncated / malformed */
#define FLUX_CUDA_ERR_MODEL (-5)   /* tensor missing, wrong shape or dtype */
#define FLUX_CUDA_ERR_NOMEM (-6)
#define FLUX_CUDA_ERR_PEER_TIMEOUT (-7) /* the other GPU of a pair did not show up in time (host rendezvous or kernel wait) */

typedef struct flux_cuda_ctx flux_cuda_ctx;

const char *flux_cuda_last_error(void);
/* 1 for the checked build of the library (compiled with -DFLUX_CUDA_DEBUG: libflux_cuda_debug.so), whose kernels verify
 * the tile, row and alignment arithmetic of what they are about to access and, on a violation, record it in the
 * context's error word (reported as FLUX_CUDA_ERR_KERNEL by the next synchronising call) and skip the access - they
 * never trap. 0 for the normal build. The reference's counterpart is its -fsanitize=address debug target. */
int flux_cuda_build_checked(void);

/* One context per GPU: creates the stream all work of this context is issued on. */
int flux_cuda_ctx_create(int device, flux_cuda_ctx **out);
void flux_cuda_ctx_destroy(flux_cuda_ctx *ctx);
/* Waits for all queued work; returns FLUX_CUDA_ERR_KERNEL if any kernel reported a failed wait. */
int flux_cuda_ctx_sync(flux_cuda_ctx *ctx);
/* The context's cudaStream_t, for callers that time with their own CUDA events. */
void *flux_cuda_ctx_stream(flux_cuda_ctx *ctx);
/*
 * Range check of the f16 format. Every 16-bit store saturates at +-65504 instead of overflowing; the GEMM and
 * convolution epilogues, AdaLN, the context conversion and the token packing count the threads that clamped a value,
 * and every synchronising call (flux_cuda_ctx_sync, the sampler / encoder / VAE calls that return host data) adds
 * that count to the context. *count = saturating stores seen so far (0 = the f16 range held); reset != 0 clears it.
 * A non-zero count with a real checkpoint means: switch to FLUX_CUDA_BF16. No counterpart in the reference, which
 * computes in f32.
 */
int flux_cuda_ctx_saturated_stores(flux_cuda_ctx *ctx, long long *count, int reset);

/*
 * Exercises the failure path of the kernels' bounded waits without touching a tensor kernel: queues a one-warp kernel
 * that waits on a barrier nobody arrives on, gives up after limit_cycles SM clock cycles (1 .. 2e9; 2e6 is about a
 * millisecond), records the failure in the context's error word and returns normally. The next flux_cuda_ctx_sync
 * therefore returns FLUX_CUDA_ERR_KERNEL once, and the context stays usable. waited_cycles_dev (device pointer, may
 * be NULL) receives the cycles the wait really took. No counterpart in the reference (a CPU path has no waits to
 * bound).
 */
int flux_cuda_selftest_wait_timeout(flux_cuda_ctx *ctx, long long limit_cycles, long long *waited_cycles_dev);

/*
 * 16-bit storage format of models created afterwards from this context: FLUX_CUDA_F16 (default) or FLUX_CUDA_BF16
 * (also: environment variable FLUX_CUDA_BF16=1 before the context is created). Weights arrive as bf16 in the
 * file and are converted once at upload (exact for 6.1e-5 <= |w| <= 65504, absolute error below 3e-8 under
 * that); activations use the same format because tcgen05 kind::f16 needs both operands in one format. f16 has
 * three more mantissa bits than bf16 at the same tensor-core rate; every 16-bit store saturates at +-65504.
 */
int flux_cuda_ctx_set_half_format(flux_cuda_ctx *ctx, int dtype);

/* Chooses how the 256-column GEMM tiles are computed: 0 = one CTA per 128 x 256 tile, 1 = a pair of CTAs on
 * neighbouring SMs per 256 x 256 tile (tcgen05 cta_group::2; each CTA stages half of the weight tile). Also
 * settable with the environment variable FLUX_CUDA_GEMM_PAIR before the context is created. */
int flux_cuda_ctx_set_gemm_pair(flux_cuda_ctx *ctx, int on);
/* Measurement aid: while stamps_dev (device memory, int64) is set, kernels launched through the kernel-level entry
 * points write the SM clock of their first CTA at fixed points of its life. flux_cuda_gemm_bf16 (paired kernel),
 * 8 stamps: 0 entry, 1 prologue done, 2 first operands landed, 3 last MMA issued, 4 first accumulator ready, 5 last
 * epilogue done, 6 before teardown, 7 TMEM freed. flux_cuda_attention, 16 stamps per key tile j at [16 j + ..]:
 * 0-4 MMA issuer (V landed, P of tile a seen, a's MMAs issued, P of tile b seen, b's MMAs issued), 5-9 first softmax
 * warp of tile a (S ready, S loaded, maximum known, P computed, P released), 10-14 the same for tile b, 15 producer
 * (K/V tile j requested); the buffer must hold 16 x ceil(seq / 128) values. NULL switches it off. No counterpart in
 * the reference. */
int flux_cuda_ctx_set_gemm_trace(flux_cuda_ctx *ctx, long long *stamps_dev);

/* ------------------------------------------------------------------------------------------------
 * Model: the FLUX.2-klein diffusion transformer resident on one GPU (bf16 weights).
 * ---------------------------------------------------------------------------------------------- */
typedef struct flux_cuda_model flux_cuda_model;

typedef struct flux_cuda_dims {
  int hidden, heads, head_dim, mlp, n_double, n_single, text_dim, latent_ch, time_dim;
  float rope_theta;
  int axis_dim;
} flux_cuda_dims;

/* The shape the reference hard-codes (flux_transformer.c:4418-4434). */
void flux_cuda_dims_klein4b(flux_cuda_dims *d);

#define FLUX_CUDA_F32 0
#define FLUX_CUDA_F16 1
#define FLUX_CUDA_BF16 2

/*
 * Loads `transformer/diffusion_pytorch_model.safetensors`. Replaces
 * flux_transformer_load_safetensors / _mmap (flux_transformer.c:4411-4656, 4659-4786): same tensor
 * names, but every tensor's shape is checked, dimensions are inferred from the file, and weights
 * stay bf16 on the device (the mmap streaming mode has no equivalent: 7.75 GB fit in HBM).
 */
int flux_cuda_model_load_safetensors(flux_cuda_ctx *ctx, const char *path, flux_cuda_model **out);
/* The same, tensor by tensor from host memory (dtype FLUX_CUDA_F32 / F16 / BF16; data is copied). */
int flux_cuda_model_create(flux_cuda_ctx *ctx, const flux_cuda_dims *dims, flux_cuda_model **out);
int flux_cuda_model_set_tensor(flux_cuda_model *m, const char *name, const void *data, int dtype,
                               const long long *shape, int ndim);
int flux_cuda_model_finalize(flux_cuda_model *m); /* fails if a tensor is missing */
/* flux_transformer_free (flux_transformer.c:4189-4312); NULL-safe. */
void flux_cuda_model_free(flux_cuda_model *m);
int flux_cuda_model_dims(const flux_cuda_model *m, flux_cuda_dims *out);

/* ------------------------------------------------------------------------------------------------
 * Forward pass and samplers with HOST buffers (the calls the reference's link seam maps onto).
 * Latents / velocities are f32 [latent_ch, h, w]; contexts f32 [txt_seq, text_dim]; h, w in latent
 * pixels (image size / 16).
 * ---------------------------------------------------------------------------------------------- */
typedef struct flux_cuda_ref { /* flux_ref_t, flux.c:68-72 */
  const float *latent;         /* [latent_ch, h, w] */
  int h, w;
  int t_offset;                /* RoPE T coordinate: 10, 20, ... */
} flux_cuda_ref;

/*
 * One velocity prediction. Replaces flux_transformer_forward (flux_transformer.c:3115-3577),
 * flux_transformer_forward_with_refs (3605-3799) and _with_multi_refs (3815-4043): num_refs == 0
 * is the plain forward. v_out receives f32 [latent_ch, h, w].
 */
int flux_cuda_forward(flux_cuda_model *m, const float *z, int h, int w, const flux_cuda_ref *refs, int num_refs,
                      const float *ctx, int txt_seq, float timestep, float *v_out);

typedef struct flux_cuda_sample_params {
  int h, w;                 /* latent size */
  int num_steps;
  const float *schedule;    /* num_steps + 1 timesteps, 1 -> 0 */
  const float *ctx;         /* conditional context [txt_seq, text_dim] */
  const float *ctx_uncond;  /* NULL: no guidance (flux_sample_euler*); else flux_sample_euler_cfg* */
  int txt_seq;
  float guidance;           /* used only with ctx_uncond */
  const flux_cuda_ref *refs;
  int num_refs;
} flux_cuda_sample_params;

/*
 * The whole Euler loop on the device. Replaces flux_sample_euler (flux_sample.c:212-290),
 * _with_refs (303-375), _with_multi_refs (381-444), flux_sample_euler_cfg (457-529), _cfg_with_refs
 * (534-610), _cfg_with_multi_refs (615-691). With guidance the conditional and unconditional passes
 * run as one batch of two. z0 is not modified; latent_out receives the final latent;
 * velocities_out (may be NULL) receives the num_steps velocities the loop used, [num_steps, C, h, w].
 */
int flux_cuda_sample(flux_cuda_model *m, const flux_cuda_sample_params *p, const float *z0, float *latent_out,
                     float *velocities_out);

/* ------------------------------------------------------------------------------------------------
 * The same loop in three phases, for callers that keep a shape's buffers alive across images and
 * for measuring the device time without the PCIe copies.
 * ---------------------------------------------------------------------------------------------- */
typedef struct flux_cuda_sampler flux_cuda_sampler;
typedef struct flux_cuda_ref_shape { int h, w, t_offset; } flux_cuda_ref_shape;

/* batch = 1, or 2 for the guidance pair (element 0 conditional, element 1 unconditional). */
int flux_cuda_sampler_create(flux_cuda_model *m, int h, int w, int txt_seq, const flux_cuda_ref_shape *refs,
                             int num_refs, int batch, int max_steps, flux_cuda_sampler **out);
void flux_cuda_sampler_free(flux_cuda_sampler *s);
/* Asynchronous copies of the raw f32 inputs into the sampler's buffers, ordered on the context's stream. Each
 * pointer may be host memory (pinned host memory makes the copies overlap) or memory of the context's device. */
int flux_cuda_sampler_upload(flux_cuda_sampler *s, const float *z0, const float *ctx, const float *ctx_uncond,
                             const float *const *ref_latents);
/* Queues input preparation + num_steps x (forward, update) on the context's stream; does not wait.
 * apply_update = 0 leaves the latent untouched (velocity of the uploaded latent at schedule[i]). */
int flux_cuda_sampler_run(flux_cuda_sampler *s, const float *schedule, int num_steps, float guidance,
                          int record_velocities, int apply_update);
/* Steps [first, first + count) of the same loop, for callers that must observe the latent between steps (the
 * reference's per-step callbacks, flux_sample.c:240-266). first == 0 starts from the uploaded latent; a later
 * call with first > 0 continues from where the previous one stopped. */
int flux_cuda_sampler_run_steps(flux_cuda_sampler *s, const float *schedule, int num_steps, int first, int count,
                                float guidance, int record_velocities);
/*
 * Guidance pair split across two GPUs (the reference runs the two passes one after the other on one device,
 * flux_sample.c:485-499). Each GPU holds a replica and a batch-1 sampler with ITS context (conditional on one
 * rank, unconditional on the other) and the same latent. Per step: flux_cuda_sampler_predict computes this
 * rank's velocity without touching the latent; flux_cuda_sampler_velocity writes scale * v to a device buffer
 * (scale = g on the conditional rank, 1 - g on the other); the caller sums the two buffers across the pair (one
 * all-reduce of latent_ch*h*w floats over NVLink); flux_cuda_sampler_apply_velocity adds dt * v_sum to the
 * latent on both ranks, which therefore stay bit-identical. All calls are asynchronous on the context's stream.
 */
int flux_cuda_sampler_predict(flux_cuda_sampler *s, const float *schedule, int num_steps, int step);
int flux_cuda_sampler_velocity(flux_cuda_sampler *s, float *dst_dev, float scale);
int flux_cuda_sampler_apply_velocity(flux_cuda_sampler *s, const float *v_dev, int step);
/* Device -> host copy of the latent (and recorded velocities), then waits and checks for kernel errors. */
int flux_cuda_sampler_download(flux_cuda_sampler *s, float *latent_out, float *velocities_out);
/*
 * Pipelined generation of many images with one sampler (no counterpart in the reference, which generates one image
 * per call): flux_cuda_sampler_stage_inputs copies the inputs of the NEXT image to the device on a second stream
 * while the current image is being computed (pinned host memory makes that a real overlap; the buffers must stay
 * valid until the next run has been queued and the stream synchronised past it); the next flux_cuda_sampler_run
 * picks them up. flux_cuda_sampler_download_async queues the device -> host copy of the latent behind the run
 * and returns; flux_cuda_ctx_sync waits for everything and reports kernel errors. Arguments as for
 * flux_cuda_sampler_upload.
 */
int flux_cuda_sampler_stage_inputs(flux_cuda_sampler *s, const float *z0, const float *ctx, const float *ctx_uncond,
                                   const float *const *ref_latents);
int flux_cuda_sampler_download_async(flux_cuda_sampler *s, float *latent_out);
/* CUDA-event time of the last flux_cuda_sampler_run in ms (valid after a sync), and its kernel count. */
int flux_cuda_sampler_last_run(flux_cuda_sampler *s, float *ms, long long *kernel_launches);

/* Per-kernel-class device time of a run: when on, every launch of the next runs is bracketed by a CUDA
 * event pair. Classes: 0 GEMM, 1 attention, 2 AdaLN, 3 QK-norm+RoPE, 4 everything else. The reference's
 * counterpart is its flux_timing_transformer_* wall-clock globals (flux_sample.c:22-39). */
#define FLUX_CUDA_KERNEL_CLASSES 5
int flux_cuda_sampler_set_profiling(flux_cuda_sampler *s, int on);
int flux_cuda_sampler_profile(flux_cuda_sampler *s, float *ms_by_class, long long *launches_by_class);
/* The same event pairs summed per part of the forward: 0 input/output edges, 1 double-stream blocks, 2 single-stream
 * blocks, 3 final layer - the split of the reference's flux_timing_transformer_double / _single / _final
 * (flux_sample.c:22-39; accumulated at flux_transformer.c:3558-3564), as device time instead of wall-clock time. */
#define FLUX_CUDA_BLOCK_GROUPS 4
int flux_cuda_sampler_profile_groups(flux_cuda_sampler *s, float *ms_by_group);
/* The same per launch, in launch order: ms[i] and kernel_class[i] for up to `capacity` launches. */
int flux_cuda_sampler_profile_launches(flux_cuda_sampler *s, float *ms, int *kernel_class, int capacity, int *count);

/* ------------------------------------------------------------------------------------------------
 * Several GPUs of one machine. The reference drives one device and runs the two passes of a guided step one after
 * the other (flux_sample_euler_cfg, flux_sample.c:485-499); these calls let a plain C host use more than one GPU:
 * one internal host thread per GPU, a full replica of the model on each.
 * ---------------------------------------------------------------------------------------------- */
typedef struct flux_cuda_group flux_cuda_group;

/* One context per listed device (devices == NULL: 0 .. n_gpus-1). Members 0 and 1 get access to each other's memory
 * when the hardware allows it (needed by flux_cuda_group_sample_cfg_pair only). FLUX_CUDA_PEER_TIMEOUT_MS overrides
 * the 20 s the host threads of a pair wait for each other. */
int flux_cuda_group_create(int n_gpus, const int *devices, flux_cuda_group **out);
void flux_cuda_group_destroy(flux_cuda_group *g);
int flux_cuda_group_size(const flux_cuda_group *g);
/* The member's context, e.g. to create a model on it from tensors. Owned by the group. */
flux_cuda_ctx *flux_cuda_group_context(flux_cuda_group *g, int member);
/* A replica on every member, loaded concurrently (flux_transformer_load_safetensors, once per GPU); owned by the
 * group. Or: hand the group models the caller created on the members' contexts (the caller keeps ownership). */
int flux_cuda_group_load_safetensors(flux_cuda_group *g, const char *path);
int flux_cuda_group_set_models(flux_cuda_group *g, flux_cuda_model *const *models);
/* The member's replica (NULL before a load), and: drop the replicas (frees the ones the group loaded itself). */
flux_cuda_model *flux_cuda_group_model(flux_cuda_group *g, int member);
void flux_cuda_group_unload(flux_cuda_group *g);
/*
 * n_images independent images, image i on member i % n_gpus: z0[i], ctx[i] (host f32, shapes as in `p`; p->ctx,
 * p->ctx_uncond and p->guidance are ignored, p->refs are shared by all images) -> latent_out[i]. No data moves
 * between the GPUs. The loop per image is flux_sample_euler / _with_multi_refs (flux_sample.c:212-290, 381-444).
 */
int flux_cuda_group_sample_batch(flux_cuda_group *g, const flux_cuda_sample_params *p, int n_images,
                                 const float *const *z0, const float *const *ctx, float *const *latent_out);
/*
 * One guided image on members 0 and 1: member 0 runs the conditional pass, member 1 the unconditional one, every
 * step; each stores its pre-scaled velocity (g v_c, (1 - g) v_u) into the other's memory with plain stores, waits for
 * the other's, and adds both into its own latent (one kernel per step and GPU; 128 h w floats cross NVLink each
 * way). Same result as flux_cuda_sample with ctx_uncond set (flux_sample_euler_cfg*, flux_sample.c:457-691), in
 * about half the time. The two host threads meet before every step; if one of them failed or does not arrive in
 * time the other returns FLUX_CUDA_ERR_PEER_TIMEOUT without having launched anything that waits, and the wait inside
 * the kernel is bounded too (reported by the same code).
 */
int flux_cuda_group_sample_cfg_pair(flux_cuda_group *g, const flux_cuda_sample_params *p, const float *z0,
                                    float *latent_out);

/* The rendezvous the pair's host threads use, on its own (plain host code, no GPU involved): `parties` threads call
 * arrive_and_wait with the same growing sequence number; it returns once every other party has announced a number
 * >= seq, or FLUX_CUDA_ERR_PEER_TIMEOUT after timeout_ms, or at once if a missing party has called abandon. */
typedef struct flux_cuda_rendezvous flux_cuda_rendezvous;
int flux_cuda_rendezvous_create(int parties, flux_cuda_rendezvous **out);
void flux_cuda_rendezvous_destroy(flux_cuda_rendezvous *r);
int flux_cuda_rendezvous_arrive_and_wait(flux_cuda_rendezvous *r, int party, long long seq, int timeout_ms);
void flux_cuda_rendezvous_abandon(flux_cuda_rendezvous *r, int party);

/* ------------------------------------------------------------------------------------------------
 * Host-side pieces of the sampler (plain C, no GPU involved).
 * ---------------------------------------------------------------------------------------------- */
/* flux_official_schedule (flux_sample.c:122-155); out has num_steps + 1 entries. */
void flux_cuda_official_schedule(int num_steps, int image_seq_len, float *out);
/* flux_linear_schedule / flux_power_schedule (flux_sample.c:49-69). */
void flux_cuda_linear_schedule(int num_steps, float *out);
void flux_cuda_power_schedule(int num_steps, float alpha, float *out);
/* flux_init_noise (flux_sample.c:835-877) with its xoshiro256** / Box-Muller stream
 * (flux_kernels.c:45-102): out is f32 [channels, h, w] (batch 1). */
void flux_cuda_init_noise(int channels, int h, int w, long long seed, float *out);

/* ------------------------------------------------------------------------------------------------
 * Text encoder (Qwen3): the stage right before the denoising loop. Replaces qwen3_model_load / qwen3_forward /
 * qwen3_model_free (flux_qwen3.c:1329-1430, 1041-1156, 1529-1590): same tensor names, same output.
 * ---------------------------------------------------------------------------------------------- */
typedef struct flux_cuda_qwen3 flux_cuda_qwen3;

typedef struct flux_cuda_qwen3_dims {
  int hidden, heads, kv_heads, head_dim, inter, layers, vocab;
  float rope_theta;
  int out_layers[3]; /* hidden states after these layers (0-based) are concatenated */
} flux_cuda_qwen3_dims;

/* The Qwen3-4B shape the reference hard-codes (flux_qwen3.h:21-40): outputs after layers 8, 17, 26. */
void flux_cuda_qwen3_dims_4b(flux_cuda_qwen3_dims *d);
/* Loads `text_encoder/` (both model-0000{1,2}-of-00002.safetensors must exist, flux_qwen3.c:1341-1356). Only the
 * layers the output depends on are kept on the device (and only those must be present in the files). max_seq: largest
 * token count of a later forward (batch * seq for a batched one). */
int flux_cuda_qwen3_load_dir(flux_cuda_ctx *ctx, const char *model_dir, int max_seq, flux_cuda_qwen3 **out);
int flux_cuda_qwen3_create(flux_cuda_ctx *ctx, const flux_cuda_qwen3_dims *dims, int max_seq, flux_cuda_qwen3 **out);
int flux_cuda_qwen3_set_tensor(flux_cuda_qwen3 *m, const char *name, const void *data, int dtype,
                               const long long *shape, int ndim);
int flux_cuda_qwen3_finalize(flux_cuda_qwen3 *m);
void flux_cuda_qwen3_free(flux_cuda_qwen3 *m);
/* input_ids, attention_mask (may be NULL = all ones): host int[seq]; out: host f32 [seq, 3 * hidden]. Causal,
 * grouped-query attention with the key padding mask, as the reference's CPU path (flux_qwen3.c:313-452). */
int flux_cuda_qwen3_forward(flux_cuda_qwen3 *m, const int *input_ids, const int *attention_mask, int seq, float *out);
/* Several prompts in one pass: input_ids and attention_mask are [batch, seq] (every prompt padded to the same seq),
 * out is host f32 [batch, seq, 3 * hidden]; batch * seq must not exceed the max_seq given at creation. The projections
 * of all prompts run as one GEMM each (the weights are read once for the batch), attention per prompt. */
int flux_cuda_qwen3_forward_batch(flux_cuda_qwen3 *m, const int *input_ids, const int *attention_mask, int batch, int seq,
                                  float *out);
int flux_cuda_qwen3_forward_batch_device(flux_cuda_qwen3 *m, const int *input_ids, const int *attention_mask, int batch,
                                         int seq, const float **out_dev);
/* The same pass, queued on the context's stream without waiting and without the device -> host copy: *out_dev is the
 * encoder's own device buffer, f32 [seq, 3 * hidden], valid (in stream order) until the next forward on this
 * encoder. Hand it to flux_cuda_sampler_upload as the context: prompt -> latent then never leaves the device. No
 * counterpart in the reference, whose encoder and transformer exchange host buffers (flux.c:330-360). */
int flux_cuda_qwen3_forward_device(flux_cuda_qwen3 *m, const int *input_ids, const int *attention_mask, int seq,
                                   const float **out_dev);

/* ------------------------------------------------------------------------------------------------
 * The stage after the loop: the VAE decoder (latent -> RGB image). Mirrors flux_vae_load_safetensors /
 * flux_vae_decode / flux_vae_free (flux_vae.c:1232-1386, 690-837, 1034-1104) for the decoder half: channel
 * configuration 128 x (1, 2, 4, 4), two + one ResNet blocks per level, GroupNorm(32), one attention block.
 * Tensor names are the file's own ("decoder.*", "post_quant_conv.*", optional "bn.running_mean/var"); the encoder
 * half ("encoder.*", "quant_conv.*") is optional as a whole.
 * ---------------------------------------------------------------------------------------------- */
typedef struct flux_cuda_vae flux_cuda_vae;
int flux_cuda_vae_load_safetensors(flux_cuda_ctx *ctx, const char *path, flux_cuda_vae **out);
int flux_cuda_vae_create(flux_cuda_ctx *ctx, flux_cuda_vae **out);
/* dtype as flux_cuda_model_set_tensor; convolution weights in the file's [out, in, kh, kw] order. */
int flux_cuda_vae_set_tensor(flux_cuda_vae *v, const char *name, const void *data, int dtype, const long long *shape,
                             int ndim);
int flux_cuda_vae_finalize(flux_cuda_vae *v);
void flux_cuda_vae_free(flux_cuda_vae *v);
/* latent: f32 [128, h, w], host memory or memory of the context's device (e.g. flux_cuda_sampler_latent_device);
 * rgb_out: host uint8 [16h, 16w, 3], values (x + 1) * 127.5 clamped to [0, 255] and truncated like the reference's
 * conversion (flux_vae.c:822-833). Buffers grow to the largest size decoded so far. */
int flux_cuda_vae_decode(flux_cuda_vae *v, const float *latent, int h, int w, unsigned char *rgb_out);
/* The same, queued without waiting; *rgb_dev is the decoder's own device buffer (valid until the next decode). */
int flux_cuda_vae_decode_device(flux_cuda_vae *v, const float *latent, int h, int w, const unsigned char **rgb_dev);
/* The encoder (flux_vae_encode, flux_vae.c:320-440): image f32 [3, H, W] planar, values in [-1, 1] as
 * flux_image_to_tensor produces them, host or device memory, H and W multiples of 16 -> latent_out: host f32
 * [128, H/16, W/16] (mean of the posterior, 2x2 packed, batch-normalised with the file's running statistics).
 * Needs the file's "encoder.*" and "quant_conv.*" tensors: a model created without them decodes only
 * (flux_cuda_vae_has_encoder returns 0 and this call FLUX_CUDA_ERR_MODEL). */
int flux_cuda_vae_encode(flux_cuda_vae *v, const float *image, int H, int W, float *latent_out);
int flux_cuda_vae_has_encoder(const flux_cuda_vae *v);
/* Kernels launched by the last decode or encode. */
long long flux_cuda_vae_last_launches(const flux_cuda_vae *v);
/* Device address of a sampler's current latent (f32 [128, h, w]; batch 2: the shared latent), in stream order
 * after the last run. */
int flux_cuda_sampler_latent_device(flux_cuda_sampler *s, const float **latent_dev);

/* ------------------------------------------------------------------------------------------------
 * Kernel-level entry points on DEVICE pointers (unit tests, microbenchmarks). Asynchronous on the
 * context's stream.
 * ---------------------------------------------------------------------------------------------- */

#define FLUX_CUDA_EPI_STORE_BF16 0
#define FLUX_CUDA_EPI_STORE_F32 1
#define FLUX_CUDA_EPI_GATED_RES_F32 2
#define FLUX_CUDA_EPI_SWIGLU_BF16 3
#define FLUX_CUDA_EPI_STORE_F32_T 4
/* or-ed into `epilogue`: x AND w hold f16 instead of bf16 / 16-bit outputs are written as f16 (saturating at
 * +-65504) instead of bf16. */
#define FLUX_CUDA_EPI_X_F16 0x100
#define FLUX_CUDA_EPI_OUT_F16 0x200

/*
 * out = epilogue(x[M,K] * w[N,K]^T), x and w bf16 row-major, f32 accumulation.
 * Replaces flux_linear_nobias / flux_linear_nobias_bf16 (flux_kernels.c:210-320, called through
 * LINEAR_BF16_OR_F32 in flux_transformer.c) plus, depending on `epilogue`:
 *   STORE_BF16 / STORE_F32   out[M, ld_out] row-major;
 *   GATED_RES_F32            out_f32[r, c] += gate[c] * acc      (gated_add, flux_transformer.c:90-97);
 *   SWIGLU_BF16              w rows interleaved per 256 as [128 gate rows | 128 up rows];
 *                            out_bf16[M, N/2] = silu(gate) * up   (flux_transformer.c:1737-1763);
 *   STORE_F32_T              out_f32[c * ld_out + r] = acc        (flux_transformer.c:3547-3552).
 * K % 64 == 0, N % tile_n == 0, tile_n in {128, 256} (0 = choose); tile_n = 512 selects the paired kernel
 * (256-column tiles, two CTAs per 256 x 256 tile, N % 256 == 0).
 */
int flux_cuda_gemm_bf16(flux_cuda_ctx *ctx, const void *x, const void *w, void *out, int M, int N, int K,
                        int epilogue, long long ld_out, const float *gate, int tile_n);

/*
 * The fused [Q|K|V] projection as the engine runs it: out_bf16[M, 3*hidden] = x[M,K] * w[3*hidden,K]^T with the
 * per-head RMSNorm (weights wq / wk, f32 [128]) and the consecutive-pair rotation (cos/sin f32 [seq,128], row r at
 * position r % seq) applied to the Q and K thirds inside the GEMM epilogue, V stored unchanged. Replaces the three
 * flux_linear_nobias calls + apply_qk_norm + apply_rope_2d of flux_transformer.c:1826-1841 / 3051-3079.
 * hidden % 256 == 0 (two 128-wide heads per output tile), K % 64 == 0.
 */
int flux_cuda_gemm_qkv_norm_rope(flux_cuda_ctx *ctx, const void *x, const void *w, void *out, int M, int hidden, int K,
                                 const float *wq, const float *wk, const float *cos_t, const float *sin_t, int seq,
                                 int f16 /* x and out in f16 instead of bf16 */);

/*
 * Joint attention over a fused projection buffer qkv[batch*seq, ld] (bf16): for every head,
 * out[:, out_col + 128*head ..] = softmax(Q K^T / sqrt(128)) V with Q/K/V at columns q_col/k_col/v_col
 * (+128*head). Replaces mha_forward / joint_attention (flux_transformer.c:1249-1330, 1335-1460).
 */
int flux_cuda_attention(flux_cuda_ctx *ctx, const void *qkv, int batch, int seq, long long ld, int q_col, int k_col,
                        int v_col, int heads, void *out, long long out_ld, int out_col,
                        int f16 /* qkv and out hold f16 instead of bf16 */);
/* apply_adaln (flux_transformer.c:979-1048): out_16 = (1 + scale) * LayerNorm(x_f32) + shift, rows x hidden. */
int flux_cuda_adaln(flux_cuda_ctx *ctx, const float *x, void *out, int rows, int hidden, const float *shift,
                    const float *scale, int f16 /* out in f16 instead of bf16 */);
/* K8, the VAE's convolution (flux_conv2d, flux_kernels.c:342-505, for 3x3 / stride 1 / padding 1): channels-last
 * x16 [n_img, H, W, cin] (cin a multiple of 64), w16 [cout, 9, cin] (tap-major; cout a multiple of 128), bias f32
 * [cout] or NULL. mode 0: out16[pixel, co]; 1: out32[pixel, co]; 2: out32[pixel, co] += ...; 3: uint8 RGB from
 * output channels 0..2 as (v + 1) * 127.5 clamped and truncated. ld: row pitch of out in elements. */
int flux_cuda_conv3x3(flux_cuda_ctx *ctx, const void *x16, int n_img, int H, int W, int cin, const void *w16, int cout,
                      const float *bias, int mode, void *out, long long ld, int f16);
/* The encoder's downsampling convolution (flux_vae.c:146-171, 360-372): 3x3, stride 2, over the input extended by one
 * zero row at the bottom and one zero column at the right. planes16 holds the input as four parity planes,
 * [(n * 4 + py * 2 + px), Ho, Wo, cin] = in[n, 2y + py, 2x + px, :]; Ho x Wo is the output size. Otherwise as above. */
int flux_cuda_conv3x3_stride2(flux_cuda_ctx *ctx, const void *planes16, int n_img, int Ho, int Wo, int cin,
                              const void *w16, int cout, const float *bias, int mode, void *out, long long ld, int f16);
/* The same kernel as a plain GEMM with a bias: out[M, N] = x16[M, K] * w16[N, K]^T + bias (modes 0-2). Only the first
 * w_rows rows of w16 are read; the rest count as zero. 1x1 convolutions and the VAE attention block's products. */
int flux_cuda_gemm_bias(flux_cuda_ctx *ctx, const void *x16, long long ldx, const void *w16, long long ldw, int M, int N,
                        int K, int w_rows, const float *bias, int mode, void *out, long long ld, int f16);
/* GroupNorm with 32 groups over channels-last x [n_img, pixels, C] (f32, or 16-bit when in16 != 0), optional swish,
 * 16-bit result (flux_group_norm, flux_kernels.c:511-553; swish_inplace, flux_vae.c:174-177). n_img <= 8; x, out16,
 * gamma and beta 16-byte aligned (else FLUX_CUDA_ERR_ARG); x and out16 must hold n_img * pixels * C elements - the
 * call cannot check the extent of the caller's buffers. */
int flux_cuda_group_norm(flux_cuda_ctx *ctx, const void *x, int in16, void *out16, int n_img, long long pixels, int C,
                         const float *gamma, const float *beta, float eps, int swish, int f16);
/* The same operation for callers that must not allocate: hosts that gave all device memory to their own pool at
 * start-up, or loops that cannot tolerate an allocation's device-wide synchronisation. No counterpart in the
 * reference (it has no device memory to manage). The reduction scratch is a fixed array inside the library image
 * (641 KB per device), so after the first call on a device this call performs no allocation, on the device or
 * through any library. The FIRST call on a device is different: it looks the array's address up
 * (cudaGetSymbolAddress), which makes the CUDA runtime load this part of the library image - code plus the 641 KB
 * array - and that load takes device memory from the driver. Make one warm-up call per device before the host hands
 * the remaining memory to its own pool and before any stream capture begins.
 * Limits: n_img <= 4 per call (larger is rejected with FLUX_CUDA_ERR_ARG); pointers 16-byte aligned as above; the
 * scratch is one per device and shared by every call on it, so calls that overlap in time (other streams or threads)
 * race - serialise them. */
int flux_cuda_group_norm_noalloc(flux_cuda_ctx *ctx, const void *x, int in16, void *out16, int n_img, long long pixels,
                                 int C, const float *gamma, const float *beta, float eps, int swish, int f16);
/* apply_qk_norm + apply_rope_2d (flux_transformer.c:1052-1106, 719-741) in place on bf16 Q and K. */
int flux_cuda_qk_norm_rope(flux_cuda_ctx *ctx, void *qkv, long long ld, int q_col, int k_col, int seq, int batch,
                           int heads, const float *wq, const float *wk, const float *cos_t, const float *sin_t);

/*
 * flux_patchify / flux_unpatchify (flux_kernels.c:1038-1094), device pointers, f32: p x p space-to-depth between
 * VAE latents [B, C, H, W] and DiT latents [B, C p p, H/p, W/p] (new channel = c p p + pi p + pj). Arguments as in
 * the reference: patchify takes the plain H, W; unpatchify takes the packed H, W.
 */
int flux_cuda_patchify(flux_cuda_ctx *ctx, float *out, const float *in, int batch, int channels, int H, int W,
                       int patch_size);
int flux_cuda_unpatchify(flux_cuda_ctx *ctx, float *out, const float *in, int batch, int channels, int H, int W,
                         int patch_size);

#ifdef __cplusplus
}
#endif
#endif /* FLUX_CUDA_H */
