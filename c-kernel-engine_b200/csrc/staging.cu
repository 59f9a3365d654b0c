// Copies from device memory to pinned host memory issued from the SMs instead of the copy engine.
//
// A host-pointer call of a small kernel (one GEMV: a few microseconds) is dominated by fixed latencies, and one avoidable part is
// the hand-over from the compute engine to the copy engine behind the kernel: measured on B200, fetching a 16-57 KB result row by
// cudaMemcpyAsync costs 4-6 us more than letting a kernel in the same stream write it across PCIe (pinned host memory is mapped
// into the device's address space).  The bytes still cross the bus inside the call; only the engine switch is gone.  Used for
// destinations inside ranges handed out by ckb200_host_alloc (known to be pinned and mapped); any other host pointer, and every
// input (where the engine's copy measured faster than reads from the SMs), keeps the copy engine.
#include <cstdint>

#include "launch.h"
#include "pdl.cuh"
#include "runtime.h"

namespace ckb {

__global__ void __launch_bounds__(256) staging_copy_kernel(uint8_t *__restrict__ dst, const uint8_t *__restrict__ src, size_t bytes)
{
    pdl_trigger();
    pdl_wait();
    const size_t tid = (size_t)blockIdx.x * blockDim.x + threadIdx.x, nthreads = (size_t)gridDim.x * blockDim.x;
    if ((((uintptr_t)dst | (uintptr_t)src) & 15) == 0) {
        const size_t n16 = bytes / 16;
        const uint4 *s = reinterpret_cast<const uint4 *>(src);
        uint4 *d = reinterpret_cast<uint4 *>(dst);
        for (size_t i = tid; i < n16; i += nthreads) d[i] = s[i];
        for (size_t i = n16 * 16 + tid; i < bytes; i += nthreads) dst[i] = src[i];
    } else {
        for (size_t i = tid; i < bytes; i += nthreads) dst[i] = src[i];
    }
}

}  // namespace ckb

extern "C" int ckb_staging_copy(void *dst, const void *src, size_t bytes, cudaStream_t st)
{
    if (!bytes) return 0;
    size_t blocks = (bytes / 16 + 255) / 256;
    if (blocks < 1) blocks = 1;
    if (blocks > 592) blocks = 592;                     // four CTAs per SM keep enough stores in flight for the bus
    return ckb::launch_pdl("staging_copy", ckb::staging_copy_kernel, dim3((unsigned)blocks), dim3(256), 0, st, (uint8_t *)dst, (const uint8_t *)src, bytes);
}
