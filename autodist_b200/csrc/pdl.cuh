// Programmatic dependent launch: a kernel launched through `launch_pdl` may be scheduled while the kernel before it
// in the stream is still draining, which hides its launch latency and whatever it does before `pdl_sync()`. Every
// kernel launched this way calls `pdl_sync()` before its first access to global memory: the call lets the kernel
// after it start its own launch (`griddepcontrol.launch_dependents`) and then waits until every kernel before it
// in the stream has completed and its writes are visible (`griddepcontrol.wait`). In a kernel that was launched without
// the attribute both instructions do nothing. AUTODIST_PDL=0 turns the attribute off (plain stream order).
#pragma once
#include <cuda_runtime.h>

#include <cstdlib>
#include <utility>

namespace adb200 {

inline bool pdl_enabled() {
  static const bool on = [] {
    const char* e = std::getenv("AUTODIST_PDL");
    return e == nullptr || e[0] != '0';
  }();
  return on;
}

template <typename... KArgs, typename... Args>
inline cudaError_t launch_pdl(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream, Args&&... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = pdl_enabled() ? 1 : 0;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(std::forward<Args>(args))...);
}

#ifdef __CUDACC__
__device__ __forceinline__ void pdl_sync() {
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  asm volatile("griddepcontrol.wait;" ::: "memory");
}
#endif

}  // namespace adb200
