// Self-test of the error path every kernel of this library shares: a bounded mbarrier wait that runs out, the error
// word, and the host-side report. The kernel below waits on a barrier nobody will ever arrive on, with a limit the
// caller chooses (milliseconds instead of the ~2 s the production kernels allow), records KERR_SELFTEST exactly the
// way a GEMM or attention role records its failure, and returns normally: no trap, no device assert, nothing left
// behind on the device. flux_cuda_ctx_sync then reports FLUX_CUDA_ERR_KERNEL and clears the word, and the context
// stays usable.
#include <cuda_runtime.h>

#include "context.cuh"
#include "flux_cuda.h"
#include "ptx.cuh"

namespace fx {

__global__ void __launch_bounds__(32) wait_timeout_kernel(int *err, long long limit_cycles, long long *waited_cycles) {
  __shared__ uint64_t bar;
  __shared__ int abort_flag;
  if (threadIdx.x == 0) {
    mbar_init(&bar, 1);
    abort_flag = 0;
    mbar_fence_init();
  }
  __syncwarp();
  if (threadIdx.x == 0) {
    const long long t0 = clock64();
    const bool ok = mbar_wait(&bar, 0, &abort_flag, limit_cycles);  // phase 0 never completes: nobody arrives
    if (waited_cycles) *waited_cycles = clock64() - t0;
    if (!ok) {
      abort_flag = 1;
      atomicCAS(err, 0, KERR_SELFTEST);
    }
  }
  __syncwarp();
}

}  // namespace fx

extern "C" int flux_cuda_selftest_wait_timeout(flux_cuda_ctx *ctx, long long limit_cycles, long long *waited_cycles_dev) {
  using namespace fx;
  if (!ctx || limit_cycles < 1 || limit_cycles > 2000000000LL) {
    set_error("selftest_wait_timeout: the limit must lie in [1, 2e9] clock cycles");
    return FLUX_CUDA_ERR_ARG;
  }
  int rc = check_cuda(cudaSetDevice(ctx->device), "cudaSetDevice");
  if (rc) return rc;
  wait_timeout_kernel<<<1, 32, 0, ctx->stream>>>(ctx->err_dev, limit_cycles, waited_cycles_dev);
  return check_cuda(cudaGetLastError(), "selftest launch");
}
