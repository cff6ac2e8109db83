// Kernel launches with programmatic dependent launch: a kernel launched through launch_pdl is
// queued behind the previous kernel of the stream with a programmatic dependency instead of a full
// one: its blocks may be scheduled as soon as every block of the previous kernel has exited (or
// has executed griddepcontrol.launch_dependents, which these kernels do not do by default, see
// ptx.cuh), so its launch latency overlaps the previous kernel. Inside the kernel,
// griddepcontrol.wait blocks until the previous kernel has completed and its writes are visible;
// every kernel launched this way calls it before its first dependent global access and before its
// first global write (the GEMM starts its weight stream before it: weights are never written).
// The attribute is also honoured inside CUDA-graph capture (programmatic edges).
// XV_PDL=0 turns the attribute off; the device-side instructions are then no-ops.
#pragma once

#include <cuda_runtime.h>

#include <cstdlib>

namespace xv {

inline bool pdl_enabled() {
  static const bool on = [] {
    const char* e = std::getenv("XV_PDL");
    return !(e != nullptr && e[0] == '0');
  }();
  return on;
}

template <typename... KArgs, typename... Args>
inline cudaError_t launch_pdl(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                              Args&&... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = pdl_enabled() ? 1 : 0;
  return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

// Same, with the grid cut into thread-block clusters of `cluster_x` consecutive CTAs (for kernels that
// are not compiled with a fixed cluster shape).
template <typename... KArgs, typename... Args>
inline cudaError_t launch_pdl_cluster(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                                      unsigned cluster_x, Args&&... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = cluster_x;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[1].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = pdl_enabled() ? 2 : 1;
  return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

}  // namespace xv
