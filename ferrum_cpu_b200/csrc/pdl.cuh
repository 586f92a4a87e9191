// Programmatic dependent launch: a kernel launched with launch_pdl may begin (be scheduled, run
// its preamble) before the kernel ahead of it in the stream has finished. Inside such a kernel
// pdl_wait() blocks until the kernel ahead has completed and its writes are visible; everything
// that reads or writes data another kernel of the chain touches comes after it, on every path,
// so completion stays transitive along the chain. pdl_trigger() lets the kernel behind start.
// Both are no-ops in a kernel that was launched the ordinary way.
#pragma once
#include "fc_common.cuh"

namespace fc {

__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_trigger() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

template <class... KArgs, class... Args>
cudaError_t launch_pdl(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t st, Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, kernel, KArgs(args)...);
}

}  // namespace fc
