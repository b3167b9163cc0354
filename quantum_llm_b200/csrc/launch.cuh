// Programmatic dependent launch: a kernel launched through launch_pdl() may be scheduled
// while its predecessor in the stream is still running.  It must call pdl_wait() before it
// reads anything an earlier kernel wrote or overwrites anything an earlier kernel reads;
// what it does before that (barrier set-up, tensor-memory allocation, prefetching weights)
// overlaps the predecessor.  pdl_trigger() lets the NEXT kernel in the stream be scheduled.
// Both instructions are no-ops for kernels launched the ordinary way.
#pragma once

#include <cuda_runtime.h>

#include <utility>

namespace qllm {

bool pdl_enabled();
void set_pdl_enabled(bool enabled);

__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_trigger() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

// cluster_x > 1: grid.x is a multiple of cluster_x and consecutive CTAs along x form a
// thread-block cluster (distributed shared memory between them).
template <typename... KArgs, typename... Args>
cudaError_t launch_pdl_cluster(void (*kernel)(KArgs...), dim3 grid, dim3 block, unsigned cluster_x, size_t smem,
                               cudaStream_t stream, Args&&... args) {
  cudaLaunchConfig_t config{};
  config.gridDim = grid;
  config.blockDim = block;
  config.dynamicSmemBytes = smem;
  config.stream = stream;
  cudaLaunchAttribute attribute[2];
  attribute[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attribute[0].val.programmaticStreamSerializationAllowed = pdl_enabled() ? 1 : 0;
  config.numAttrs = 1;
  if (cluster_x > 1U) {
    attribute[1].id = cudaLaunchAttributeClusterDimension;
    attribute[1].val.clusterDim.x = cluster_x;
    attribute[1].val.clusterDim.y = 1;
    attribute[1].val.clusterDim.z = 1;
    config.numAttrs = 2;
  }
  config.attrs = attribute;
  return cudaLaunchKernelEx(&config, kernel, std::forward<Args>(args)...);
}

// Ordinary stream order (the kernel starts after everything before it has finished) for a
// kernel that contains the dependency instructions.
template <typename... KArgs, typename... Args>
cudaError_t launch_ordered(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                           Args&&... args) {
  cudaLaunchConfig_t config{};
  config.gridDim = grid;
  config.blockDim = block;
  config.dynamicSmemBytes = smem;
  config.stream = stream;
  return cudaLaunchKernelEx(&config, kernel, std::forward<Args>(args)...);
}

template <typename... KArgs, typename... Args>
cudaError_t launch_pdl(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                       Args&&... args) {
  return launch_pdl_cluster(kernel, grid, block, 1U, smem, stream, std::forward<Args>(args)...);
}

}  // namespace qllm
