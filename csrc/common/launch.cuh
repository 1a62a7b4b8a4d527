// Kernel launch with programmatic dependent launch (PDL).
//
// A kernel launched through launch_pdl may be scheduled while the kernel before it in the stream is still running:
// its CTAs do their private set-up (barrier init, TMEM allocation, tensor-map prefetch) and then block in
// pdl_wait() until the previous kernel has completed and its memory is visible.  The previous kernel opens that
// window with pdl_launch_dependents().  Rules that every kernel using these helpers follows:
//   * no global memory access before pdl_wait() (kernel parameters, tensor maps passed by value and shared memory are fine);
//   * a kernel that allocates TMEM calls pdl_launch_dependents() only after its allocation has succeeded, so a CTA of
//     the next kernel can never take the columns an already-running CTA of this kernel is still waiting for.
// Launched without the attribute (the default; UB_PDL=1 switches it on) both calls are no-ops and the stream order
// is the usual one.  The launches are captured into CUDA graphs as programmatic edges.
#pragma once
#include <cuda_runtime.h>
#include <stdlib.h>

#include <utility>

namespace ub {

__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

inline bool pdl_enabled() {
  static int v = -1;
  if (v < 0) {
    const char* e = getenv("UB_PDL");
    v = e ? atoi(e) : 0;       // off by default: on the serving step it measured 3 % slower than plain stream order
  }
  return v != 0;
}

// Fills `attr` with the PDL attribute and returns how many attributes were written (0 when disabled).
inline int pdl_attr(cudaLaunchAttribute* attr) {
  if (!pdl_enabled()) return 0;
  attr->id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr->val.programmaticStreamSerializationAllowed = 1;
  return 1;
}

template <typename... P, typename... A>
inline cudaError_t launch_pdl(void (*kern)(P...), dim3 grid, dim3 block, size_t smem, cudaStream_t st, A&&... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = st;
  cudaLaunchAttribute attr[1];
  cfg.attrs = attr;
  cfg.numAttrs = pdl_attr(attr);
  return cudaLaunchKernelEx(&cfg, kern, std::forward<A>(args)...);
}

}  // namespace ub
