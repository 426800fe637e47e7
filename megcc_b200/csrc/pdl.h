// Programmatic dependent launch: a kernel launched with launch_pdl() may be scheduled while the
// kernel before it on the stream is still running. Its CTAs take the SMs the predecessor's CTAs
// leave, run their set-up (barrier initialisation, tensor-memory allocation, descriptor
// prefetch) and then block in pdl_start() until the predecessor has completed and its writes
// are visible. That hides the launch latency and the ramp of each of the 20-odd kernels of a
// network behind the tail of the previous one. Every kernel launched this way calls
// pdl_start() before it reads or writes global memory; a kernel launched without the
// attribute executes the two instructions as no-ops.
#pragma once
#include <cuda_runtime.h>

#include <utility>

#include "tuning.h"

namespace mb200 {

#if defined(__CUDACC__)
// Releases the NEXT kernel for scheduling (it still waits for this one to complete before it
// touches memory), then waits for the PREVIOUS kernel's completion.
__device__ __forceinline__ void pdl_release() {
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
}
__device__ __forceinline__ void pdl_wait() {
    asm volatile("griddepcontrol.wait;" ::: "memory");
}
__device__ __forceinline__ void pdl_start() {
    pdl_release();
    pdl_wait();
}
#endif

template <class... KArgs, class... Args>
inline cudaError_t launch_pdl(
        void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t st,
        Args&&... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = tuning().pdl ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, kernel, std::forward<Args>(args)...);
}

}  // namespace mb200
