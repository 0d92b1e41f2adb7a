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

// Diagnostics, compiled only with -DMS_TIMELINE: every block stamps the device clock when it starts, when its
// wait for the preceding kernel returns and when it ends, into the record of its launch: [id, first start, first
// wait return, first end, last end, then five marks of block 0 after its wait] in nanoseconds.  The record's index is a counter that block 0 advances when
// it ends; a block reads it after its wait, when the preceding kernel has advanced it and block 0 of its own
// kernel, with its work still ahead, has not.  Each translation unit has its own pointer, set from the host.
#ifdef MS_TIMELINE
static __device__ unsigned long long* g_ms_tl;  // [0]: counter, then records of 10
struct MsTimeline {
  unsigned long long t0, t1;
  int id, slot;
  bool on;
  __device__ __forceinline__ static unsigned long long now() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
    return t;
  }
  __device__ __forceinline__ MsTimeline(int id_) : t0(0), t1(0), id(id_), slot(-1) {
    on = g_ms_tl != nullptr && threadIdx.x == 0 && threadIdx.y == 0 && threadIdx.z == 0;
    if (on) t0 = now();
  }
  __device__ __forceinline__ void waited() {
    if (!on) return;
    t1 = now();
    slot = (int)*reinterpret_cast<volatile unsigned long long*>(g_ms_tl);
  }
  __device__ __forceinline__ void mark(int i) {  // block 0 only: nanoseconds since its wait returned
    if (!on || slot < 0 || slot >= 4096 || blockIdx.x || blockIdx.y || blockIdx.z) return;
    g_ms_tl[1 + (size_t)slot * 10 + 5 + i] = now() - t1;
  }
  __device__ __forceinline__ ~MsTimeline() {
    if (!on || slot < 0 || slot >= 4096) return;
    const unsigned long long t2 = now();
    unsigned long long* r = g_ms_tl + 1 + (size_t)slot * 10;
    r[0] = (unsigned long long)id;
    atomicMin(r + 1, t0);
    atomicMin(r + 2, t1);
    atomicMin(r + 3, t2);
    atomicMax(r + 4, t2);
    if (blockIdx.x == 0 && blockIdx.y == 0 && blockIdx.z == 0) {
      __threadfence();
      atomicAdd(g_ms_tl, 1ull);
    }
  }
};
#define MS_TIMELINE_BEGIN(id) MsTimeline ms_tl_(id)
#define MS_TIMELINE_WAITED() ms_tl_.waited()
#define MS_TIMELINE_MARK(i) ms_tl_.mark(i)
#define MS_TIMELINE_SETTER(name) \
  MS_API int name(void* p) { return cudaMemcpyToSymbol(g_ms_tl, &p, sizeof(p)) == cudaSuccess ? 0 : 2; }
#else
#define MS_TIMELINE_BEGIN(id)
#define MS_TIMELINE_WAITED()
#define MS_TIMELINE_MARK(i)
#define MS_TIMELINE_SETTER(name)
#endif

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
