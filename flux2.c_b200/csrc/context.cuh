// Per-device context shared by every entry point of the library: the stream work is issued on, the
// device error word the kernels' bounded waits report through, and the SM count used to size
// persistent grids.
#pragma once
#include <cuda_runtime.h>
#include <string>

// Ring of pinned staging buffers for weight uploads: host threads copy the next piece of a (pageable, usually
// memory-mapped) tensor into one slot while the DMA engine drains the previous slots.
struct UploadRing {
  static constexpr int SLOTS = 3;
  static constexpr size_t SLOT_BYTES = 32u << 20;
  void *buf[SLOTS] = {nullptr, nullptr, nullptr};
  cudaEvent_t drained[SLOTS] = {nullptr, nullptr, nullptr};
  int next = 0;
  int state = 0;  // 0 not tried, 1 ready, -1 pinned memory unavailable (uploads fall back to pageable copies)
  int threads = 1;
};

struct flux_cuda_ctx {
  int device = 0;
  int num_sms = 0;
  cudaStream_t stream = nullptr;  // owned
  cudaStream_t copy_stream = nullptr;  // owned; created by the first staged upload (inputs of the next image)
  int *err_dev = nullptr;         // two device words: [0] first kernel error (0 = none), [1] saturated f16 stores
  int *err_host = nullptr;        // pinned mirror of both
  long long saturated = 0;        // saturated f16 stores seen by the synchronisations so far
  bool f16 = true;                // 16-bit tensors (weights and activations) are f16; false: bf16
  int attn_version = 2;           // 2: attention2.cu (default), 3: attention3.cu (FLUX_CUDA_ATTN=3, measured slower)
  bool gemm_pair = true;          // 256-wide GEMM tiles computed by CTA pairs (tcgen05 cta_group::2)
  float *gn_scratch = nullptr;    // lazily allocated scratch of the kernel-level GroupNorm entry point
  float *rope_scratch = nullptr;  // lazily allocated pair-angle table of flux_cuda_gemm_qkv_norm_rope
  size_t rope_scratch_floats = 0;
  UploadRing upload;              // created by the first weight upload, released with the context
  long long *gemm_trace = nullptr;  // device buffer for the paired GEMM's timeline stamps (measurements only)
};

namespace fx {
void set_error(const char *fmt, ...);
int check_cuda(cudaError_t e, const char *what);
// Synchronises the context's stream and returns FLUX_CUDA_ERR_KERNEL if a kernel recorded an error.
int ctx_sync_check(flux_cuda_ctx *ctx);
// Host-to-device copy ordered on the context's (non-blocking) stream, complete on return. A plain cudaMemcpy from
// pageable memory may return while the DMA is still in flight and is not ordered against a non-blocking stream,
// so work queued on that stream right after it could read the old contents.
inline cudaError_t upload_h2d(cudaStream_t st, void *dst, const void *src, size_t bytes) {
  cudaError_t e = cudaMemcpyAsync(dst, src, bytes, cudaMemcpyHostToDevice, st);
  return e != cudaSuccess ? e : cudaStreamSynchronize(st);
}
// Copies `bytes` of pageable host memory to the device through the context's pinned ring, ordered on the context's
// stream. The host memory has been read completely when this returns; the device copy completes in stream order.
int upload_pipelined(flux_cuda_ctx *ctx, void *dst, const void *src, size_t bytes);
void upload_ring_release(flux_cuda_ctx *ctx);
}  // namespace fx
