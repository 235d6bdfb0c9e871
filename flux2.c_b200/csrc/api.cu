// extern "C" surface of the library (declared in include/flux_cuda.h): context management, error
// reporting and the kernel-level entry points.
#include "flux_cuda.h"

#include <stdarg.h>
#include <stdio.h>
#include <string.h>

#include "context.cuh"
#include "gemm.cuh"

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
  int rc = check_cuda(cudaMemcpyAsync(ctx->err_host, ctx->err_dev, sizeof(int), cudaMemcpyDeviceToHost, ctx->stream),
                      "read kernel error word");
  if (rc) return rc;
  rc = check_cuda(cudaStreamSynchronize(ctx->stream), "stream synchronize");
  if (rc) return rc;
  if (*ctx->err_host != 0) {
    const int code = *ctx->err_host;
    cudaMemsetAsync(ctx->err_dev, 0, sizeof(int), ctx->stream);
    set_error("a kernel gave up on a bounded wait (code %d)", code);
    return FLUX_CUDA_ERR_KERNEL;
  }
  return FLUX_CUDA_OK;
}
}  // namespace fx

using namespace fx;

extern "C" {

const char *flux_cuda_last_error(void) { return g_err; }

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
      (rc = check_cuda(cudaMalloc(&c->err_dev, sizeof(int)), "cudaMalloc")) ||
      (rc = check_cuda(cudaMallocHost(&c->err_host, sizeof(int)), "cudaMallocHost")) ||
      (rc = check_cuda(cudaMemset(c->err_dev, 0, sizeof(int)), "cudaMemset"))) {
    flux_cuda_ctx_destroy(c);
    return rc;
  }
  if (gemm_init() != 0) {
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
  if (ctx->err_dev) cudaFree(ctx->err_dev);
  if (ctx->err_host) cudaFreeHost(ctx->err_host);
  delete ctx;
}

int flux_cuda_ctx_sync(flux_cuda_ctx *ctx) {
  if (!ctx) return FLUX_CUDA_ERR_ARG;
  return ctx_sync_check(ctx);
}

void *flux_cuda_ctx_stream(flux_cuda_ctx *ctx) { return ctx ? (void *)ctx->stream : nullptr; }

int flux_cuda_gemm_bf16(flux_cuda_ctx *ctx, const void *x, const void *w, void *out, int M, int N, int K,
                        int epilogue, long long ld_out, const float *gate, int tile_n) {
  if (!ctx || !x || !w || !out) {
    set_error("gemm: null argument");
    return FLUX_CUDA_ERR_ARG;
  }
  if (epilogue < 0 || epilogue > 4 || (epilogue == EPI_GATED_RES_F32 && !gate)) {
    set_error("gemm: bad epilogue %d", epilogue);
    return FLUX_CUDA_ERR_ARG;
  }
  int bn = tile_n;
  if (bn == 0) bn = (N % 256 == 0) ? 256 : 128;
  GemmParams P;
  memset(&P, 0, sizeof(P));
  int rc = gemm_make_problem(&P.p[0], x, w, M, N, K, bn);
  if (rc) {
    set_error("gemm: unsupported shape/alignment M=%d N=%d K=%d tile_n=%d (rc %d)", M, N, K, bn, rc);
    return FLUX_CUDA_ERR_ARG;
  }
  P.nprob = 1;
  P.err = ctx->err_dev;
  P.p[0].seg[0].mode = epilogue;
  P.p[0].seg[0].col0 = 0;
  P.p[0].seg[0].ld = ld_out;
  P.p[0].seg[0].out = out;
  P.p[0].seg[0].gate = gate;
  rc = gemm_launch(&P, bn, ctx->num_sms, ctx->stream);
  if (rc) {
    set_error("gemm: launch failed (rc %d: %s)", rc, cudaGetErrorString(cudaGetLastError()));
    return rc <= -8 ? FLUX_CUDA_ERR_CUDA : FLUX_CUDA_ERR_ARG;
  }
  return FLUX_CUDA_OK;
}

}  // extern "C"
