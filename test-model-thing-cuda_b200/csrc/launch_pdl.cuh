// Programmatic dependent launch for chains of short kernels (the sampler step is five launches of a few
// microseconds each): a kernel launched with the attribute may be scheduled, and run whatever precedes its
// `pdl_wait()`, while the kernel before it in the stream is still running; `pdl_wait()` returns once that kernel
// has completed and its writes are visible. Every kernel of such a chain calls `pdl_begin()` first (lets its own
// successor be scheduled early) and touches nothing another kernel reads or writes before `pdl_wait()`. Without the
// attribute both calls do nothing. TMT_MOE_PDL=0 launches the chain the ordinary way.
#pragma once
#include <cuda_runtime.h>

#include <cstdlib>
#include <utility>

namespace tmt {

__device__ __forceinline__ void pdl_begin() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }

inline bool pdl_enabled() {
    const char* s = getenv("TMT_MOE_PDL");
    return !(s && *s == '0');
}

template <class... KArgs, class... Args>
cudaError_t launch_pdl(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream, Args&&... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid; cfg.blockDim = block; cfg.dynamicSmemBytes = smem; cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = pdl_enabled() ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, kernel, std::forward<Args>(args)...);
}

}  // namespace tmt
