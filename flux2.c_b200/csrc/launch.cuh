// Kernel launch helper: every kernel of the step is launched with programmatic dependent launch allowed, so
// that the next kernel's CTAs can be scheduled and run their prologue (barrier init, TMEM allocation, tensor-map
// prefetch) while the previous kernel drains. Each kernel calls pdl_launch_dependents() early and pdl_wait()
// before it first touches global memory (ptx.cuh). FLUX_CUDA_PDL=0 turns the attribute off.
#pragma once
#include <cuda_runtime.h>
#include <stdlib.h>

#include <utility>

namespace fx {

inline bool pdl_enabled() {
  static int on = -1;
  if (on < 0) {
    const char *e = getenv("FLUX_CUDA_PDL");
    on = (e && atoi(e) == 0) ? 0 : 1;
  }
  return on != 0;
}

// Launches made while a PdlOff object is alive on this thread do not ask for programmatic dependent launch.
inline int &pdl_off_depth() {
  static thread_local int depth = 0;
  return depth;
}
struct PdlOff {
  PdlOff() { ++pdl_off_depth(); }
  ~PdlOff() { --pdl_off_depth(); }
  PdlOff(const PdlOff &) = delete;
  PdlOff &operator=(const PdlOff &) = delete;
};

template <typename... KArgs, typename... Args>
inline cudaError_t launch_kernel(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t st,
                                 int cluster_x, Args &&...args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = st;
  cudaLaunchAttribute attr[2];
  unsigned n = 0;
  if (pdl_enabled() && pdl_off_depth() == 0) {
    attr[n].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[n].val.programmaticStreamSerializationAllowed = 1;
    ++n;
  }
  if (cluster_x > 1) {
    attr[n].id = cudaLaunchAttributeClusterDimension;
    attr[n].val.clusterDim.x = cluster_x;
    attr[n].val.clusterDim.y = 1;
    attr[n].val.clusterDim.z = 1;
    ++n;
  }
  cfg.attrs = attr;
  cfg.numAttrs = n;
  return cudaLaunchKernelEx(&cfg, kernel, std::forward<Args>(args)...);
}

}  // namespace fx
