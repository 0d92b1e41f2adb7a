// Launch helper: thread-block clusters and programmatic dependent launch.
//
// With programmatic dependent launch a kernel's blocks may start while the kernel before
// it in the stream still runs.  Such a kernel does what does not depend on its predecessor
// first (the matrix products prefetch their weights), then executes `ms_pdl_wait()`, which
// returns when the predecessor has finished and its writes are visible.  `ms_pdl_trigger()`
// tells the hardware that the blocks of the NEXT kernel may be started early; every kernel
// here calls it at its top.  Both are no-ops in a kernel launched the ordinary way.
#pragma once
#include "common.cuh"

__device__ __forceinline__ void ms_pdl_wait() { asm volatile("griddepcontrol.wait;\n" ::: "memory"); }
__device__ __forceinline__ void ms_pdl_trigger() { asm volatile("griddepcontrol.launch_dependents;\n" ::); }

extern int g_ms_pdl;  // 1: kernels that support it are launched as programmatic dependents

template <typename... KArgs, typename... Args>
static cudaError_t ms_launch(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                             int cluster, bool pdl, Args... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[2];
  int n = 0;
  if (cluster > 1) {
    attr[n].id = cudaLaunchAttributeClusterDimension;
    attr[n].val.clusterDim.x = cluster;
    attr[n].val.clusterDim.y = 1;
    attr[n].val.clusterDim.z = 1;
    ++n;
  }
  if (pdl && g_ms_pdl) {
    attr[n].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[n].val.programmaticStreamSerializationAllowed = 1;
    ++n;
  }
  cfg.attrs = attr;
  cfg.numAttrs = n;
  return cudaLaunchKernelEx(&cfg, kernel, KArgs(args)...);
}

#define MS_LAUNCH_RESULT(name, call)                                        \
  do {                                                                      \
    cudaError_t e_ = (call);                                                \
    if (e_ != cudaSuccess) {                                                \
      ms_set_error("%s: launch failed: %s", name, cudaGetErrorString(e_));  \
      return 2;                                                             \
    }                                                                       \
  } while (0)
