// Programmatic dependent launch (sm_90+): a kernel launched with the stream-serialisation attribute may be
// scheduled while its predecessor in the stream is still running - once every CTA of the predecessor has called
// pdl_trigger() or exited - and must call pdl_wait() before touching anything the predecessor writes (the wait
// returns when the predecessor has completed and its writes are visible). This hides the launch gap between the
// short kernels of one operation. Both instructions do nothing in a kernel that was launched normally.
#pragma once
#include <cuda_runtime.h>
#include <stdlib.h>

namespace gcow {

__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_trigger() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

// Launch `kernel` so that it may overlap the tail of its predecessor in the stream. The kernel must start with
// pdl_wait(). GCOW_PDL=0 falls back to ordinary launches.
template <typename... KArgs, typename... Args>
static void launch_dependent(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t s, Args... args) {
  static const bool enabled = [] { const char* e = getenv("GCOW_PDL"); return !(e && e[0] == '0'); }();
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid; cfg.blockDim = block; cfg.dynamicSmemBytes = smem; cfg.stream = s;
  cudaLaunchAttribute attr;
  attr.id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr.val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = &attr; cfg.numAttrs = enabled ? 1 : 0;
  cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

}  // namespace gcow
