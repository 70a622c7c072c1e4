// Kernel launches with programmatic dependent launch (PDL).
//
// A training step here is a chain of several hundred short kernels on one stream.  Launched the ordinary way,
// kernel N+1 is only scheduled once kernel N has drained, so every boundary costs a launch latency plus the new
// kernel's prologue (barrier initialisation, TMEM allocation, tensor-map fetch) with the GPU idle.  With the
// programmatic-stream-serialization attribute the next kernel's blocks are scheduled as soon as every block of the
// current one has called pdl_launch_dependents() (all kernels of this library do so first thing), run their prologue
// while the current kernel's last blocks finish, and stop at pdl_wait() until the current kernel has completed and its
// writes are visible.  Rules kept by every kernel launched through tb::launch:
//   * every thread calls pdl_wait() before its first access to global memory (read or write) -- unconditionally, on
//     every path, so that completion of a kernel implies completion of everything before it in the stream;
//   * nothing before pdl_wait() touches global memory.
// Both instructions do nothing in a kernel launched without the attribute, and stream capture records the
// dependency as a programmatic edge, so the same code runs eagerly and inside CUDA graphs.
#pragma once
#include <cuda_runtime.h>

namespace tb {

__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_enter() {
  pdl_launch_dependents();
  pdl_wait();
}

// 1 (default): launch with the attribute; 0: plain launches.  One switch for the whole library (tb_set_pdl).
inline int& pdl_enabled() {
  static int on = 1;
  return on;
}

template <typename... KArgs, typename... Args>
inline cudaError_t launch(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream, Args&&... args) {
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

}  // namespace tb
