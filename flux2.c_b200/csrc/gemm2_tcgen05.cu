// K1 (paired variant): the same GEMM as gemm_tcgen05.cu, computed by PAIRS of CTAs on neighbouring SMs
// (a cluster of two, tcgen05 cta_group::2). A pair owns a 256 x 256 output tile: each CTA stages its own 128
// rows of X and only HALF of the W tile (128 of the 256 output columns' rows); one thread of the leader CTA
// issues tcgen05.mma M256 N256 K16, which reads both CTAs' shared memory and writes each CTA's half of the
// accumulator into that CTA's TMEM. Per k-slice a CTA therefore pulls 32 KB through L2 instead of 48 KB for the
// same 128 x 256 x 64 of work, which matters because the single-CTA kernel is limited by operand delivery
// (~16 TB/s of L2->SM traffic), not by the tensor pipe. No multicast is used: every CTA issues its own loads.
//
// Synchronisation: "full" barriers live in the leader (both CTAs' TMA loads complete bytes on them); "empty"
// and "accumulator full" barriers exist in both CTAs and are signalled by one multicast tcgen05.commit;
// "accumulator drained" lives in the leader and collects the arrivals of all eight epilogue warps of the pair.
#include <cudaTypedefs.h>
#include <stdlib.h>

#include "gemm.cuh"
#include "gemm_epilogue.cuh"
#include "launch.cuh"
#include "ptx.cuh"

namespace fx {

static constexpr int P_BM = 128;  // rows per CTA (256 per pair)
static constexpr int P_BN = 256;
static constexpr int P_BK = 64;
static constexpr int P_STAGES = 6;
static constexpr int P_A_BYTES = P_BM * P_BK * 2;        // 16 KB
static constexpr int P_B_BYTES = (P_BN / 2) * P_BK * 2;  // 16 KB: this CTA's half of the W tile
static constexpr int P_STAGE_BYTES = P_A_BYTES + P_B_BYTES;
static constexpr int P_EPI_STAGE = 4 * EPI_STAGE_BYTES_PER_WARP;  // staging blocks of the four epilogue warps
static constexpr int P_SMEM = P_STAGES * P_STAGE_BYTES + P_EPI_STAGE + 256 + 1024;
static_assert(4 * 8 * 4096 <= P_STAGES * P_STAGE_BYTES, "the last tile's staging must fit the operand ring");
static_assert(P_SMEM <= 232448, "shared memory of the paired GEMM exceeds what an SM offers");
static_assert(sizeof(GemmParams) <= 4096, "kernel parameters must stay within the classic 4 KB limit");
static constexpr int P_THREADS = 192;

__global__ void __launch_bounds__(P_THREADS, 1) gemm2_bf16_tn_kernel(const __grid_constant__ GemmParams P) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t *epi_stage = smem + P_STAGES * P_STAGE_BYTES;  // 1024-byte aligned
  uint64_t *bars = reinterpret_cast<uint64_t *>(epi_stage + P_EPI_STAGE);
  uint64_t *full = bars;                  // used in the leader only
  uint64_t *empty = bars + P_STAGES;      // both CTAs
  uint64_t *tfull = bars + 2 * P_STAGES;  // both CTAs
  uint64_t *tempty = tfull + 2;           // leader only, 8 arrivals
  uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(tempty + 2);
  volatile int *abort_flag = reinterpret_cast<volatile int *>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();  // 0 = leader
  const int pair = blockIdx.x >> 1;
  const int num_pairs = gridDim.x >> 1;
  const bool traced = P.trace != nullptr && blockIdx.x == 0;
  auto stamp = [&](int slot) {
    if (traced) P.trace[slot] = clock64();
  };
  if (threadIdx.x == 0) stamp(0);

  if (threadIdx.x == 0) {
    for (int s = 0; s < P_STAGES; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(&tfull[a], 1);
      mbar_init(&tempty[a], 8);
    }
    *abort_flag = 0;
    mbar_fence_init();
  }
  if (warp == 1) tmem_alloc_pair(tmem_slot, 512);
  tc_fence_before_sync();
  __syncthreads();
  cluster_sync_all();  // the partner's barriers exist before anything can arrive on them
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;
  pdl_launch_dependents();
  pdl_wait();  // everything above touched only shared memory and TMEM
  if (threadIdx.x == 0) stamp(1);

  auto fail = [&](int code) {
    *abort_flag = 1;
    atomicCAS(P.err, 0, code);
  };
  // pair-level tile -> (problem, first row of the PAIR's tile, first column)
  auto decode = [&](int tile, int &prob, int &m0, int &n0) {
    prob = 0;
    while (prob + 1 < P.nprob && tile >= P.tile_end[prob]) ++prob;
    const int local = tile - (prob ? P.tile_end[prob - 1] : 0);
    const int tm = P.p[prob].tiles_m;
    m0 = (local % tm) * (2 * P_BM);
    n0 = (local / tm) * P_BN;
  };

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer (both CTAs)
    if (lane == 0) {
      for (int i = 0; i < P.nprob; ++i) {
        tma_prefetch_desc(&P.p[i].tmA);
        tma_prefetch_desc(&P.p[i].tmB);
      }
      uint32_t kiter = 0;
      bool ok = true;
      for (int tile = pair; ok && tile < P.total_tiles; tile += num_pairs) {
        int prob, m0, n0;
        decode(tile, prob, m0, n0);
        const GemmProblem &pb = P.p[prob];
        const int KB = pb.K / P_BK;
        for (int kb = 0; kb < KB; ++kb, ++kiter) {
          const int s = kiter % P_STAGES;
          const uint32_t ph = (kiter / P_STAGES) & 1;
          if (!mbar_wait(&empty[s], ph ^ 1, abort_flag)) {
            fail(KERR_WAIT_EMPTY);
            ok = false;
            break;
          }
          uint8_t *sa = smem + s * P_STAGE_BYTES;
          uint8_t *sb = sa + P_A_BYTES;
          const uint32_t full_leader = map_to_cta(smem_u32(&full[s]), 0);
          if (rank == 0) mbar_arrive_expect_tx(&full[s], 2 * P_STAGE_BYTES);  // both CTAs' bytes
          tma_load_2d_pair(sa, &pb.tmA, full_leader, kb * P_BK, m0 + rank * P_BM);
          tma_load_2d_pair(sb, &pb.tmB, full_leader, kb * P_BK, n0 + rank * (P_BN / 2));
        }
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer (leader CTA only)
    // The whole warp runs the loop and one elected lane issues: descriptors, TMEM addresses and loop state are then
    // warp-uniform values that stay in the uniform datapath the tcgen05 instructions take their operands from.
    // (With the role inside `if (lane == 0)` each descriptor is a per-thread value that has to be moved across for
    // every instruction; measured on the attention kernel that made the issue of one MMA cost ~100 cycles.)
    if (rank == 0) {
      const bool leader = elect_one();
      constexpr uint32_t idesc_bf16 = make_idesc_16(2 * P_BM, P_BN, FMT_BF16, FMT_BF16, 0, 0);
      constexpr uint32_t idesc_f16 = make_idesc_16(2 * P_BM, P_BN, FMT_F16, FMT_F16, 0, 0);
      const uint32_t smem_base = smem_u32(smem);
      uint32_t kiter = 0, it = 0;
      bool ok = true;
      for (int tile = pair; ok && tile < P.total_tiles; tile += num_pairs, ++it) {
        int prob, m0, n0;
        decode(tile, prob, m0, n0);
        const int KB = P.p[prob].K / P_BK;
        const uint32_t idesc = P.p[prob].x_f16 ? idesc_f16 : idesc_bf16;
        const int acc = it & 1;
        if (!mbar_wait_warp(&tempty[acc], ((it >> 1) & 1) ^ 1, abort_flag)) {
          if (lane == 0) fail(KERR_WAIT_TMEM_EMPTY);
          break;
        }
        tc_fence_after_sync();
        const uint32_t d = tmem_base + acc * P_BN;
        for (int kb = 0; kb < KB; ++kb, ++kiter) {
          const int s = kiter % P_STAGES;
          const uint32_t ph = (kiter / P_STAGES) & 1;
          if (!mbar_wait_warp(&full[s], ph, abort_flag)) {
            if (lane == 0) fail(KERR_WAIT_FULL);
            ok = false;
            break;
          }
          tc_fence_after_sync();
          if (kiter == 0 && leader) stamp(2);
          const uint32_t sa = smem_base + s * P_STAGE_BYTES;
          const uint64_t ad = make_smem_desc_sw128(sa, 16, 1024);
          const uint64_t bd = make_smem_desc_sw128(sa + P_A_BYTES, 16, 1024);
          if (leader) {
#pragma unroll
            for (int k = 0; k < P_BK / 16; ++k) tc_mma_ss_pair(d, ad + 2 * k, bd + 2 * k, idesc, (kb | k) ? 1u : 0u);
            tc_commit_pair(&empty[s], 3);  // frees the stage in both CTAs
          }
        }
        if (ok && leader) tc_commit_pair(&tfull[acc], 3);
      }
      if (leader) stamp(3);
    }
    __syncwarp();
  } else {
    // ------------------------------------------------------------------ epilogue (warps 2..5 of both CTAs)
    const int q = warp & 3;
    uint32_t it = 0;
    for (int tile = pair; tile < P.total_tiles; tile += num_pairs, ++it) {
      int prob, m0, n0;
      decode(tile, prob, m0, n0);
      const int acc = it & 1;
      const bool ok = mbar_wait_warp(&tfull[acc], (it >> 1) & 1, abort_flag);
      if (!ok) {
        if (lane == 0) fail(KERR_WAIT_TMEM_FULL);
        break;
      }
      tc_fence_after_sync();
      if (it == 0 && warp == 2 && lane == 0) stamp(4);
      const uint32_t taddr = tmem_base + acc * P_BN + (static_cast<uint32_t>(q * 32) << 16);
      // During this CTA's last tile nothing reads or fills the operand ring any more (the accumulator barrier says
      // every MMA of the pair has completed), so each warp stages its whole 32 x 256 part of the tile there (eight
      // blocks) and all of its TMA stores are in flight at once. This part of a launch is never hidden by a next tile.
      const bool last = tile + num_pairs >= P.total_tiles;
      uint8_t *stage = last ? smem + q * (8 * 4096) : epi_stage + q * EPI_STAGE_BYTES_PER_WARP;
      epilogue_tile<P_BN>(P.p[prob], m0 + static_cast<int>(rank) * P_BM, n0, taddr, q * 32 + lane, P.err + 1, stage,
                          last ? 8 : 2);
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster(map_to_cta(smem_u32(&tempty[acc]), 0));
    }
    if (lane == 0) bulk_wait<0>();  // this warp's TMA stores have been performed before the CTA leaves
    if (warp == 2 && lane == 0) stamp(5);
  }

  // ------------------------------------------------------------------ teardown
  if (threadIdx.x == 0) stamp(6);
  if (*abort_flag) {
    const long long t0 = clock64();
    while (clock64() - t0 < 2000000LL) __nanosleep(1000);
  }
  tc_fence_before_sync();
  __syncthreads();
  cluster_sync_all();  // neither CTA leaves while the other may still read its shared memory or signal its barriers
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc_pair(tmem_base, 512);
    if (lane == 0) stamp(7);
  }
}

int gemm2_init() {
  cudaError_t e = cudaFuncSetAttribute(gemm2_bf16_tn_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, P_SMEM);
  return e == cudaSuccess ? 0 : -2;
}

// Same contract as gemm_launch for bn = 256, but problems must have been made with gemm_make_problem_pair.
int gemm2_launch(GemmParams *P, int num_sms, cudaStream_t stream) {
  if (P->nprob < 1 || P->nprob > GEMM_MAX_PROBLEMS) return -5;
  int acc = 0;
  for (int i = 0; i < P->nprob; ++i) {
    const GemmProblem &pb = P->p[i];
    if (pb.n_split % P_BN) return -6;
    acc += pb.tiles_m * pb.tiles_n;
    P->tile_end[i] = acc;
  }
  P->total_tiles = acc;
  // Outputs leave through the TMA unit when the destination allows it (16-byte aligned base and pitch). For
  // comparisons: FLUX_CUDA_EPI_TMA=0 keeps the direct global stores everywhere, =1 uses the TMA unit for the f32
  // outputs only.
  static const int tma_level = getenv("FLUX_CUDA_EPI_TMA") ? atoi(getenv("FLUX_CUDA_EPI_TMA")) : 2;
  const bool tma_epilogue = tma_level >= 1;
  for (int i = 0; i < P->nprob; ++i) {
    GemmProblem &pb = P->p[i];
    for (int sgi = 0; sgi < 2; ++sgi) {
      EpiSeg &sg = pb.seg[sgi];
      sg.tma_out = 0;
      const int width = sgi == 0 ? pb.n_split : pb.N - pb.n_split;
      if (!tma_epilogue || width <= 0 || !sg.out) continue;
      if (sg.mode == EPI_STORE_F32 || sg.mode == EPI_GATED_RES_F32) {
        if (!(sg.col0 & 3) &&
            make_tmap_2d_f32(&sg.tm_out, sg.out, pb.M, static_cast<uint64_t>(sg.col0) + width, sg.ld, 32, 32) == 0)
          sg.tma_out = 1;
      } else if (tma_level >= 2 && (sg.mode == EPI_STORE_BF16 || sg.mode == EPI_SWIGLU_BF16 ||
                                    (sg.mode == EPI_QKV_NORM_ROPE && (!sg.qk.half_split || sg.qk.ang != nullptr)))) {
        // 16-bit outputs: blocks of 32 rows x 64 columns (SwiGLU writes half as many columns as it computes)
        const int out_cols = sg.mode == EPI_SWIGLU_BF16 ? width / 2 : width;
        if (!(sg.col0 & 7) && make_tmap_2d_bf16(&sg.tm_out, sg.out, pb.M, static_cast<uint64_t>(sg.col0) + out_cols,
                                                sg.ld, 32, 64) == 0)
          sg.tma_out = 1;
      }
    }
  }
  int pairs = num_sms / 2;
  if (acc < pairs) pairs = acc;
  return launch_kernel(gemm2_bf16_tn_kernel, dim3(2 * pairs), dim3(P_THREADS), P_SMEM, stream, 2, *P) == cudaSuccess
             ? 0
             : -8;
}

int gemm_make_problem_pair(GemmProblem *p, const void *X, long long ldx, const void *W, int M, int N, int K,
                           long long ldw) {
  if (ldw == 0) ldw = K;
  if (M <= 0 || N <= 0 || K <= 0 || (K % P_BK) || (N % P_BN) || ldx < K || ldw < K) return -5;
  int rc = make_tmap_2d_bf16(&p->tmA, X, M, K, ldx, P_BM, P_BK);
  if (rc) return rc;
  rc = make_tmap_2d_bf16(&p->tmB, W, N, K, ldw, P_BN / 2, P_BK);
  if (rc) return rc;
  p->M = M;
  p->N = N;
  p->K = K;
  p->x_f16 = 0;
  p->n_split = N;
  p->tiles_m = (M + 2 * P_BM - 1) / (2 * P_BM);
  p->tiles_n = N / P_BN;
  return 0;
}

}  // namespace fx
