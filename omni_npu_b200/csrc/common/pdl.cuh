// Programmatic dependent launch: a kernel launched with the attribute below may begin
// (block scheduling, prologue, loads of data that no earlier kernel writes) while the
// kernel before it in the stream is still draining.  Inside the kernel,
//   pdl_trigger()  lets the NEXT kernel of the stream start launching once every block of
//                  this grid has called it (or exited);
//   pdl_wait()     returns when all kernels this one depends on have finished and their
//                  writes are visible.  Everything that reads or overwrites data touched
//                  by earlier kernels must come after it.
// Both are no-ops in a kernel launched without the attribute, so a kernel that uses
// them may still be launched the plain way.  Works under stream capture: the graph gets
// a programmatic edge instead of a full one.
//
// OMNI_B200_PDL=0 turns the attribute off (plain stream order).
#pragma once

#include <cuda_runtime.h>

#include <cstdlib>

namespace b200 {

__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_trigger() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

inline bool pdl_enabled() {
  static const bool on = [] {
    const char* e = getenv("OMNI_B200_PDL");
    return e == nullptr || atoi(e) != 0;
  }();
  return on;
}

// Launches `kern` with the programmatic-serialization attribute (and a cluster dimension
// when cluster_x > 1).  Returns the CUDA error of the launch.
template <typename... KArgs, typename... Args>
inline cudaError_t launch_pdl(void (*kern)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                              int cluster_x, Args&&... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[2];
  unsigned n = 0;
  if (cluster_x > 1) {
    attr[n].id = cudaLaunchAttributeClusterDimension;
    attr[n].val.clusterDim.x = static_cast<unsigned>(cluster_x);
    attr[n].val.clusterDim.y = 1;
    attr[n].val.clusterDim.z = 1;
    ++n;
  }
  if (pdl_enabled()) {
    attr[n].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[n].val.programmaticStreamSerializationAllowed = 1;
    ++n;
  }
  cfg.attrs = attr;
  cfg.numAttrs = n;
  return cudaLaunchKernelEx(&cfg, kern, static_cast<KArgs>(args)...);
}

}  // namespace b200
