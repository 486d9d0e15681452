// Host-side launch helper: programmatic dependent launch (PDL).
//
// A kernel launched through `launch_pdl` may be scheduled while its predecessor in the stream is still running: as soon
// as every CTA of the predecessor has executed `griddepcontrol.launch_dependents` (or exited), the CTAs of this kernel
// start, run their prologue (shared-memory carve-up, barrier init, TMEM allocation) and block in `griddepcontrol.wait`
// until the predecessor has finished and its writes are visible.  That hides the launch gap and the prologue of the
// many small kernels of a decode step, inside CUDA graphs as well.  Kernels launched this way call `pdl_trigger()` first
// and `pdl_wait()` before they touch global memory (common.cuh).  A predecessor that never triggers (any other kernel)
// simply keeps the ordinary stream order.
#pragma once
#include <cuda_runtime.h>

#include <utility>

namespace llm {

inline bool& pdl_enabled() {
    static bool on = true;
    return on;
}

template <class... KArgs, class... Args>
inline cudaError_t launch_pdl(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t st, Args&&... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = pdl_enabled() ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(std::forward<Args>(args))...);
}

}  // namespace llm
