// Host-visible description of one launch of the tcgen05 GEMM  Y[M,N] = X[M,K] * W[N,K]^T
// (both operands bf16, K contiguous, f32 accumulation in TMEM) and of what its epilogue does with
// the accumulator. This is the engine's replacement for the reference's flux_linear_nobias /
// cblas_sgemm call sites (flux_kernels.c:210-320) together with the elementwise passes the
// reference runs right after each of them.
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace fx {

enum EpiMode : int {
  EPI_STORE_BF16 = 0,     // out_bf16[row, col] = acc
  EPI_STORE_F32 = 1,      // out_f32[row, col] = acc
  EPI_GATED_RES_F32 = 2,  // out_f32[row, col] += gate[col] * acc   (reference: gated_add, flux_transformer.c:90-97)
  EPI_SWIGLU_BF16 = 3,    // tile columns [0,128) = gate, [128,256) = up; out_bf16[row, col/2..] = silu(g)*u
  EPI_STORE_F32_T = 4,    // out_f32[col * ld + row] = acc          (token-major -> channel-major, NLC -> NCHW)
  EPI_QKV_NORM_ROPE = 5,  // fused [Q|K|V] projection: per-head RMSNorm * w and pair rotation on the Q and K columns
                          // (apply_qk_norm + apply_rope_2d, flux_transformer.c:1052-1106, 719-741), V stored as is; bf16
};

// Extra operands of EPI_QKV_NORM_ROPE. Segment-relative column c: c < q_cols is Q, c < q_cols + k_cols is K, else
// V (heads of 128 columns). Row r of the problem sits at sequence position (pos0 + r) % seq; positions below n_txt
// use the text stream's norm weights. Two rotation conventions:
//   half_split = 0 (DiT): consecutive pairs (2j, 2j+1), cos/sin f32 [seq, 128] with one value per element;
//   half_split = 1 (Qwen3 encoder, flux_qwen3.c:264-307): pairs (i, i + 64), cos/sin f32 [seq, 64].
struct QkvNormRope {
  const float *wq_txt, *wk_txt, *wq_img, *wk_img;
  const float *cos_t, *sin_t;
  // half_split = 0 only, optional: the rotation ANGLE of every consecutive pair, f32 [seq, 64], reduced to [-pi, pi].
  // When set it replaces the cos/sin tables: a row's 64 angles are a quarter of the bytes of its 2 x 128 table values
  // (the tables hold every value twice), and an epilogue thread - which owns a whole row, so that its 32 lanes read 32
  // different rows - issues a quarter of the scattered loads; cos and sin come from the special-function unit, which
  // has nothing else to do in a GEMM.
  const float *ang;
  int pos0, seq, n_txt, q_cols, k_cols, half_split;
};

struct alignas(64) EpiSeg {
  CUtensorMap tm_out;  // paired kernel, f32 store modes: f32 view [M, col0 + width] of `out`, box 32 x 32, 128-byte swizzle
  int tma_out;         // tm_out is valid: the epilogue stages 32 x 32 blocks in shared memory and lets the TMA unit
                       // store them (STORE_F32) or add them to the destination in L2 (GATED_RES_F32)
  int mode;
  int out_f16;        // 16-bit outputs are written as f16 (saturating) instead of bf16
  int col0;           // first destination column of this segment
  long long ld;       // destination leading dimension in elements
  void *out;
  const float *gate;  // EPI_GATED_RES_F32 only; indexed by the segment-relative column
  QkvNormRope qk;     // EPI_QKV_NORM_ROPE only
};

struct alignas(64) GemmProblem {
  CUtensorMap tmA;  // X  [M, K] bf16, box 64 x 128, 128B swizzle
  CUtensorMap tmB;  // W  [N, K] bf16, box 64 x BN,  128B swizzle
  int M, N, K;
  int x_f16;        // X and W hold f16 instead of bf16 (tcgen05 kind::f16 needs both operands in one format)
  int n_split;      // output columns [0, n_split) go to seg[0], [n_split, N) to seg[1]
  EpiSeg seg[2];
  int tiles_m, tiles_n;
};

static constexpr int GEMM_MAX_PROBLEMS = 4;

struct alignas(64) GemmParams {
  GemmProblem p[GEMM_MAX_PROBLEMS];  // independent problems sharing one persistent launch (e.g. the text and
                                     // image streams of a double-stream block, per batch element)
  int nprob;
  int tile_end[GEMM_MAX_PROBLEMS];   // exclusive prefix sums of the problems' tile counts
  int total_tiles;
  int *err;          // device words: [0] first failing role's KernelError, [1] count of saturated f16 stores
  long long *trace;  // optional (paired kernel only): 8 clock64 stamps of CTA 0's roles, for timeline measurements:
                     // 0 entry, 1 prologue done, 2 first operands landed, 3 last MMA issued, 4 first accumulator
                     // ready, 5 last epilogue done, 6 before teardown, 7 TMEM freed
};

// Fills the tensor maps and tile counts of `p` for tile width bn (128 or 256). Returns 0 on success.
// ldx = row pitch of X in elements (>= K), so X may be a column slice of a wider buffer.
// ldw = row pitch of W in elements (0: K), so W may be a K-slice of a wider matrix (split-K).
int gemm_make_problem(GemmProblem *p, const void *X, long long ldx, const void *W, int M, int N, int K, int bn,
                      long long ldw = 0);
// Launches the persistent kernel over P.nprob problems. bn must match gemm_make_problem.
int gemm_launch(GemmParams *P, int bn, int num_sms, cudaStream_t stream);
// Paired variant (gemm2_tcgen05.cu): two CTAs per 256 x 256 tile, tile width fixed at 256.
int gemm2_init();
int gemm_make_problem_pair(GemmProblem *p, const void *X, long long ldx, const void *W, int M, int N, int K,
                           long long ldw = 0);
int gemm2_launch(GemmParams *P, int num_sms, cudaStream_t stream);
int gemm_init();  // resolves cuTensorMapEncodeTiled and opts the kernels into large shared memory

// Tensor-map helper shared with the attention kernel: rank-2 bf16 tensor [rows, cols], cols contiguous,
// row pitch `ld` elements, box = box_cols x box_rows, 128-byte swizzle.
int make_tmap_2d_bf16(CUtensorMap *m, const void *base, uint64_t rows, uint64_t cols, uint64_t ld, uint32_t box_rows,
                      uint32_t box_cols);
// The same for f32 elements (box_cols * 4 bytes must be 128: one swizzle span).
int make_tmap_2d_f32(CUtensorMap *m, const void *base, uint64_t rows, uint64_t cols, uint64_t ld, uint32_t box_rows,
                     uint32_t box_cols);

}  // namespace fx
