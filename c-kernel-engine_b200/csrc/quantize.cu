// Activation quantisers: fp32 -> Q8_K (256-element superblocks) and fp32 -> Q8_0 (32-element blocks).
//
// Bit-exact with the reference's quantize_row_q8_k (src/kernels/gemm_kernels_q4k_q8k.c:53-103,
// src/kernels/quantize_row_q8_k_sse.c:22-82) and quantize_row_q8_0
// (src/kernels/gemm_kernels_q8_0.c:70-175):
//   * the scale comes from the SIGNED value of the first element holding the largest |x|
//     (the warp reduction compares (|x|, index) so that the lowest index wins ties);
//   * iscale = -127/max and d = 1/iscale use IEEE division; the product iscale*x is rounded
//     to fp32 before the round-to-nearest-even integer conversion (no FMA contraction).
#include "q8k_block.cuh"
#include "pdl.cuh"
#include "launch.h"
#include "runtime.h"

namespace ckb {

// One warp per 256-element block; lane l owns elements 8l..8l+7.
__global__ void __launch_bounds__(128) quantize_q8_k_kernel(const float *__restrict__ x, uint8_t *__restrict__ y,
                                                            long long nblocks)
{
    const int lane = threadIdx.x & 31;
    const long long blk = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    pdl_trigger();
    pdl_wait();
    if (blk >= nblocks) return;

    // written by the previous kernel, which may still have been running when this one started:
    // read through L2 (the read-only path is not coherent across a programmatic launch)
    const float4 *src = reinterpret_cast<const float4 *>(x + blk * QK_K) + 2 * lane;
    const float4 a = __ldcg(src), b = __ldcg(src + 1);
    const float v[8] = {a.x, a.y, a.z, a.w, b.x, b.y, b.z, b.w};

    quantize_block_q8k(v, y + blk * Q8K_BYTES, lane);
}

// One warp per 32-element block; lane l owns element l.
__global__ void __launch_bounds__(128) quantize_q8_0_kernel(const float *__restrict__ x, uint8_t *__restrict__ y,
                                                            long long nblocks)
{
    const int lane = threadIdx.x & 31;
    const long long blk = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (blk >= nblocks) return;
    const float v = x[blk * QK8_0 + lane];
    float amax = fabsf(v);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
    const float d = __fdiv_rn(amax, 127.0f);
    const float id = amax != 0.0f ? __fdiv_rn(127.0f, amax) : 0.0f;
    const int q = __float2int_rn(__fmul_rn(v, id));
    const int qn = __shfl_down_sync(0xffffffffu, q, 1);
    uint8_t *out = y + blk * Q80_BYTES;
    if (lane == 0) *reinterpret_cast<unsigned short *>(out) = __half_as_ushort(__float2half_rn(d));
    if ((lane & 1) == 0)
        *reinterpret_cast<unsigned short *>(out + 2 + lane) = (unsigned short)((q & 255) | ((qn & 255) << 8));
}

}  // namespace ckb

extern "C" int ckb200_dev_quantize_q8_k(const float *x, void *y, int rows, int k, void *stream)
{
    if (!x || !y || rows <= 0 || k <= 0) return 0;
    if (k % ckb::QK_K) return ckb_fail(CKB_ERR_SHAPE, "quantize_q8_k: k=%d is not a multiple of 256", k);
    if (((uintptr_t)x & 15) || ((uintptr_t)y & 3))
        return ckb_fail(CKB_ERR_ALIGN, "quantize_q8_k: x must be 16-byte and y 4-byte aligned");
    if (ckb_ensure_init()) return CKB_ERR_NO_DEVICE;
    const long long nblocks = (long long)rows * (k / ckb::QK_K);
    const unsigned grid = (unsigned)((nblocks + 3) / 4);
    return ckb::launch_pdl("quantize_q8_k", ckb::quantize_q8_k_kernel, dim3(grid), dim3(128), 0, ckb_stream(stream), x, (uint8_t *)y, nblocks);
}

extern "C" int ckb200_dev_quantize_q8_0(const float *x, void *y, int rows, int k, void *stream)
{
    if (!x || !y || rows <= 0 || k <= 0) return 0;
    if (k % ckb::QK8_0) return ckb_fail(CKB_ERR_SHAPE, "quantize_q8_0: k=%d is not a multiple of 32", k);
    if ((uintptr_t)y & 1) return ckb_fail(CKB_ERR_ALIGN, "quantize_q8_0: y must be 2-byte aligned");
    if (ckb_ensure_init()) return CKB_ERR_NO_DEVICE;
    const long long nblocks = (long long)rows * (k / ckb::QK8_0);
    const unsigned grid = (unsigned)((nblocks + 3) / 4);
    ckb::quantize_q8_0_kernel<<<grid, 128, 0, ckb_stream(stream)>>>(x, (uint8_t *)y, nblocks);
    return ckb_check_launch("quantize_q8_0");
}
