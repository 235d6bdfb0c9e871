// Parameters of the fused joint-attention kernels (attention2.cu, attention3.cu).
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace fx {

struct alignas(64) AttnParams {
  CUtensorMap tm;          // [batch, seq, ld] bf16 view of the fused projection output; box 64 x 128 x 1
  CUtensorMap tm_out;      // [batch, seq, out_ld] view of the output; box 64 x 32 x 1 (attention2.cu, when tma_out)
  int tma_out;
  int spec;                // attention2.cu: exponentials against the current reference maximum first (see there)
  int seq, batch, heads;
  int q_col, k_col, v_col; // first column of head 0 of Q / K / V inside a row of that buffer
  void *out;               // bf16 [batch*seq, out_ld]; head h goes to columns out_col + 128*h ..
  long long out_ld;
  int out_col;
  float scale_log2;        // log2(e) / sqrt(head_dim)
  int f16;                 // Q, K, V, P and the output are f16 instead of bf16
  // Options used by the text encoder (all zero for the DiT):
  int kv_group;            // query heads per K/V head (grouped-query attention); 0 or 1 = one K/V head per query head
  int causal;              // key j is visible to query i only if j <= i
  const uint32_t *key_mask;  // [batch, ceil(seq/32)] bit j%32 of word j/32 set = key j is valid; NULL = all valid
  int *err;
  long long *trace;        // optional (attention2.cu): clock64 stamps of CTA (0,0,0), 16 per key tile, for timeline
                           // measurements: 0-4 MMA issuer, 5-9 softmax warp of tile a, 10-14 of tile b, 15 producer
};

// Second-generation kernel (attention2.cu): two query tiles per CTA, P and the output accumulator in TMEM.
int attn2_init();
int attn2_make_params(AttnParams *p, const void *qkv, int batch, int seq, long long ld, int q_col, int k_col, int v_col,
                      void *out, long long out_ld, int out_col, int heads, int f16, int *err);
int attn2_launch(const AttnParams *p, cudaStream_t stream);
// Third generation (attention3.cu): the same pipeline with eight softmax warps per query tile. Takes the parameters
// attn2_make_params fills.
int attn3_init();
int attn3_launch(const AttnParams *p, cudaStream_t stream);
// version 2 or 3 (the context's attn_version)
inline int attn_launch_version(int version, const AttnParams *p, cudaStream_t stream) {
  return version == 2 ? attn2_launch(p, stream) : attn3_launch(p, stream);
}

}  // namespace fx
