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

typedef struct flux_cuda_ctx flux_cuda_ctx;

const char *flux_cuda_last_error(void);

/* One context per GPU: creates the stream all work of this context is issued on. */
int flux_cuda_ctx_create(int device, flux_cuda_ctx **out);
void flux_cuda_ctx_destroy(flux_cuda_ctx *ctx);
/* Waits for all queued work; returns FLUX_CUDA_ERR_KERNEL if any kernel reported a failed wait. */
int flux_cuda_ctx_sync(flux_cuda_ctx *ctx);
/* The context's cudaStream_t, for callers that time with their own CUDA events. */
void *flux_cuda_ctx_stream(flux_cuda_ctx *ctx);

/* ------------------------------------------------------------------------------------------------
 * Kernel-level entry points on DEVICE pointers (unit tests, microbenchmarks). Asynchronous on the
 * context's stream.
 * ---------------------------------------------------------------------------------------------- */

#define FLUX_CUDA_EPI_STORE_BF16 0
#define FLUX_CUDA_EPI_STORE_F32 1
#define FLUX_CUDA_EPI_GATED_RES_F32 2
#define FLUX_CUDA_EPI_SWIGLU_BF16 3
#define FLUX_CUDA_EPI_STORE_F32_T 4

/*
 * out = epilogue(x[M,K] * w[N,K]^T), x and w bf16 row-major, f32 accumulation.
 * Replaces flux_linear_nobias / flux_linear_nobias_bf16 (flux_kernels.c:210-320, called through
 * LINEAR_BF16_OR_F32 in flux_transformer.c) plus, depending on `epilogue`:
 *   STORE_BF16 / STORE_F32   out[M, ld_out] row-major;
 *   GATED_RES_F32            out_f32[r, c] += gate[c] * acc      (gated_add, flux_transformer.c:90-97);
 *   SWIGLU_BF16              w rows interleaved per 256 as [128 gate rows | 128 up rows];
 *                            out_bf16[M, N/2] = silu(gate) * up   (flux_transformer.c:1737-1763);
 *   STORE_F32_T              out_f32[c * ld_out + r] = acc        (flux_transformer.c:3547-3552).
 * K % 64 == 0, N % tile_n == 0, tile_n in {128, 256} (0 = choose).
 */
int flux_cuda_gemm_bf16(flux_cuda_ctx *ctx, const void *x, const void *w, void *out, int M, int N, int K,
                        int epilogue, long long ld_out, const float *gate, int tile_n);

#ifdef __cplusplus
}
#endif
#endif /* FLUX_CUDA_H */
