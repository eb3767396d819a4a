// Kernel launches with programmatic dependent launch (PDL).
//
// A step is a chain of several hundred short kernels, each depending on the one before, so the
// gap between "previous grid drained" and "next grid's CTAs running their main loop" is paid
// hundreds of times. With PDL the next grid may become resident as soon as every CTA of the
// previous grid has passed its `launch_dependents` point; it then runs everything that does not
// depend on the previous grid (barrier and TMEM set-up, tensor-map fetches, and for the linears
// the first weight tiles, which are static) and blocks in `grid_dependency_wait()` until the
// previous grid has completed and its writes are visible.
//
// Rule for every kernel launched through this helper: no load or store of data another kernel of
// the chain writes or reads may precede grid_dependency_wait().
#pragma once

#include <cuda_runtime.h>

#include <cstdlib>

namespace carat_b200 {

#ifdef __CUDACC__
__device__ __forceinline__ void grid_dependency_wait() {
  asm volatile("griddepcontrol.wait;" ::: "memory");
}

__device__ __forceinline__ void grid_dependency_launch() {
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
}
#endif

// CARAT_B200_PDL=0 turns the attribute off (the device-side calls then do nothing).
inline bool pdl_enabled() {
  static const bool enabled = [] {
    const char *configured = std::getenv("CARAT_B200_PDL");
    return configured == nullptr || configured[0] != '0';
  }();
  return enabled;
}

template <typename... KernelArgs, typename... Args>
cudaError_t launch_chained(void (*kernel)(KernelArgs...), dim3 grid, dim3 block,
                           size_t shared_bytes, cudaStream_t stream, bool cooperative,
                           Args... args) {
  cudaLaunchConfig_t config{};
  config.gridDim = grid;
  config.blockDim = block;
  config.dynamicSmemBytes = shared_bytes;
  config.stream = stream;
  cudaLaunchAttribute attributes[2];
  unsigned int count = 0;
  if (pdl_enabled()) {
    attributes[count].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attributes[count].val.programmaticStreamSerializationAllowed = 1;
    ++count;
  }
  if (cooperative) {
    attributes[count].id = cudaLaunchAttributeCooperative;
    attributes[count].val.cooperative = 1;
    ++count;
  }
  config.attrs = attributes;
  config.numAttrs = count;
  return cudaLaunchKernelEx(&config, kernel, static_cast<KernelArgs>(args)...);
}

} // namespace carat_b200
