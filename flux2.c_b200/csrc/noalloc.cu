// GroupNorm for callers that must not allocate device memory.
//
// flux_cuda_group_norm keeps its reduction scratch in a buffer it obtains from cudaMalloc the first time it runs.
// Some hosts cannot afford that: a server that has handed every byte of the device to its own pool at start-up and
// treats a later driver allocation as a fault, or a latency-critical loop in which an allocation (which may
// synchronise the whole device) is not acceptable. For them the same two kernels run here on scratch that is part of
// the library image itself: a fixed, file-scope __device__ array, so that once the library image is on the device the
// entry point below performs no allocation of any kind, on the device or through a library. The one exception is the
// first call on a device: the CUDA runtime loads this file's module (its code and the 641 KB array) lazily, at that
// first cudaGetSymbolAddress, and that load takes device memory from the driver. A host that is about to give the
// remaining memory to its own pool makes one warm-up call first.
//
// The price is a fixed capacity and shared state: the array is one per device, every call on that device uses it, and
// two calls that overlap in time (different streams or threads) race on it.
#include <cuda_runtime.h>

#include <stdint.h>

#include "context.cuh"
#include "flux_cuda.h"
#include "launch.cuh"
#include "vae_kernels.cuh"

namespace {

constexpr int NA_MAX_IMAGES = 4;  // capacity: at most this many images per call
constexpr size_t NA_PARTIAL = static_cast<size_t>(NA_MAX_IMAGES) * fx::GN_MAX_BLOCKS * 64;  // per-block partial sums
constexpr size_t NA_STATS = static_cast<size_t>(NA_MAX_IMAGES) * fx::GN_GROUPS * 2;         // (mean, rstd) per group
constexpr size_t NA_COUNTERS = 8;                                                           // one per image, padded
constexpr size_t NA_FLOATS = NA_PARTIAL + NA_STATS + NA_COUNTERS;                           // 164,104 floats = 641 KB

static __device__ __align__(256) float g_na_scratch[NA_FLOATS];

constexpr int NA_MAX_DEVICES = 64;
float *g_na_ptr[NA_MAX_DEVICES] = {};  // device address of the array, per device, filled by the first call there

}  // namespace

extern "C" int flux_cuda_group_norm_noalloc(flux_cuda_ctx *ctx, const void *x, int in16, void *out16, int n_img,
                                            long long pixels, int C, const float *gamma, const float *beta, float eps,
                                            int swish, int f16) {
  using namespace fx;
  if (!ctx || !x || !out16 || !gamma || !beta || n_img < 1 || pixels < 1) {
    set_error("group_norm_noalloc: bad argument");
    return FLUX_CUDA_ERR_ARG;
  }
  if ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(out16) | reinterpret_cast<uintptr_t>(gamma) |
       reinterpret_cast<uintptr_t>(beta)) & 15) {
    set_error("group_norm_noalloc: x, out16, gamma and beta must be 16-byte aligned");
    return FLUX_CUDA_ERR_ARG;
  }
  if (n_img > NA_MAX_IMAGES) {
    set_error("group_norm_noalloc: %d images exceed the built-in scratch, which holds at most %d per call", n_img,
              NA_MAX_IMAGES);
    return FLUX_CUDA_ERR_ARG;
  }
  if (ctx->device < 0 || ctx->device >= NA_MAX_DEVICES) {
    set_error("group_norm_noalloc: device index %d is outside the supported range", ctx->device);
    return FLUX_CUDA_ERR_ARG;
  }
  int rc = check_cuda(cudaSetDevice(ctx->device), "cudaSetDevice");
  if (rc) return rc;
  if (!g_na_ptr[ctx->device]) {  // set-up, once per device, with that device current
    float *p = nullptr;
    cudaError_t e = cudaGetSymbolAddress(reinterpret_cast<void **>(&p), g_na_scratch);
    if (e != cudaSuccess || !p) {
      set_error("group_norm_noalloc: cudaGetSymbolAddress failed: %s", cudaGetErrorString(e));
      return FLUX_CUDA_ERR_CUDA;
    }
    g_na_ptr[ctx->device] = p;
  }
  float *partial = g_na_ptr[ctx->device];
  float *stats = partial + NA_PARTIAL;
  unsigned int *counters = reinterpret_cast<unsigned int *>(stats + NA_STATS);
  // the block counters are the one part that has to start at zero; a finished call leaves them so, this covers a call
  // that was cut short
  rc = check_cuda(cudaMemsetAsync(counters, 0, NA_COUNTERS * sizeof(unsigned int), ctx->stream), "clear counters");
  if (rc) return rc;
  PdlOff plain_launches;  // plain stream order, as the VAE itself launches these kernels
  int lr = launch_gn_stats(x, in16, f16, n_img, pixels, C, eps, partial, counters, stats, ctx->stream);
  if (!lr) lr = launch_gn_apply(x, in16, out16, f16, n_img, pixels, C, stats, gamma, beta, swish, ctx->stream);
  if (lr) {
    set_error("group_norm_noalloc: unsupported channel count %d or launch failure", C);
    return lr == -1 ? FLUX_CUDA_ERR_ARG : FLUX_CUDA_ERR_CUDA;
  }
  return FLUX_CUDA_OK;
}
