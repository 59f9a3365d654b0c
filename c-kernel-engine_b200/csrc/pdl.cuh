// Programmatic dependent launch helpers.
//
// A kernel launched through launch_pdl() may start while the previous kernel on the stream is still
// running.  Inside such a kernel: pdl_trigger() lets the next kernel start early, pdl_wait() blocks
// until the previous kernel has completed and its writes are visible.  Everything before pdl_wait()
// may only read data that no kernel writes (weights) and must not write global memory.
#pragma once

#include <cuda_runtime.h>

#include "launch.h"
#include "runtime.h"

namespace ckb {

__device__ __forceinline__ void pdl_trigger() { asm volatile("griddepcontrol.launch_dependents;"); }
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }

template <typename... KArgs, typename... Args>
inline int launch_pdl(const char *what, void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t st, Args... args)
{
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = ckb_tune_get("pdl", 1) ? 1 : 0;
    if (ckb_check_cuda((int)cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...), what)) return CKB_ERR_CUDA;
    return ckb_check_launch(what);
}

}  // namespace ckb
