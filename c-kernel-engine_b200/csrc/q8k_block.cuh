// One warp quantises one 256-element block to Q8_K; lane l holds elements 8l..8l+7 in v[].
// Bit-exact with the reference's quantize_row_q8_k (src/kernels/gemm_kernels_q4k_q8k.c:53-103):
// the SIGNED value of the first element with the largest |x| sets the scale (the reduction compares
// (|x|, index) so the lowest index wins ties), iscale = -127/max and d = 1/iscale are IEEE divisions,
// and iscale*x is rounded to fp32 before the round-to-nearest-even conversion.
#pragma once

#include "device_common.cuh"

namespace ckb {

__device__ __forceinline__ void quantize_block_q8k(const float (&v)[8], uint8_t *out, int lane)
{
    float best = 0.0f;
    int best_i = 8 * lane;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
        const float ax = fabsf(v[j]);
        if (ax > best) { best = ax; best_i = 8 * lane + j; }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ob = __shfl_xor_sync(0xffffffffu, best, o);
        const int oi = __shfl_xor_sync(0xffffffffu, best_i, o);
        if (ob > best || (ob == best && oi < best_i)) { best = ob; best_i = oi; }
    }
    float cand = 0.0f;
#pragma unroll
    for (int j = 0; j < 8; ++j) if ((best_i & 7) == j) cand = v[j];
    const float vmax = __shfl_sync(0xffffffffu, cand, best_i >> 3);

    if (best == 0.0f) {
        if (lane == 0) *reinterpret_cast<float *>(out) = 0.0f;
        reinterpret_cast<uint32_t *>(out + 4)[2 * lane] = 0u;
        reinterpret_cast<uint32_t *>(out + 4)[2 * lane + 1] = 0u;
        if (lane < 8) reinterpret_cast<uint32_t *>(out + 260)[lane] = 0u;
        return;
    }
    const float iscale = __fdiv_rn(-127.0f, vmax);
    int q[8], s = 0;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
        int r = __float2int_rn(__fmul_rn(iscale, v[j]));
        r = max(-128, min(127, r));
        q[j] = r;
        s += r;
    }
    const uint32_t w0 = (q[0] & 255) | ((q[1] & 255) << 8) | ((q[2] & 255) << 16) | ((uint32_t)(q[3] & 255) << 24);
    const uint32_t w1 = (q[4] & 255) | ((q[5] & 255) << 8) | ((q[6] & 255) << 16) | ((uint32_t)(q[7] & 255) << 24);
    reinterpret_cast<uint32_t *>(out + 4)[2 * lane] = w0;
    reinterpret_cast<uint32_t *>(out + 4)[2 * lane + 1] = w1;
    s += __shfl_xor_sync(0xffffffffu, s, 1);   // the 16-element sum lives in both lanes of a pair
    if ((lane & 1) == 0) reinterpret_cast<int16_t *>(out + 260)[lane >> 1] = (int16_t)s;
    if (lane == 0) *reinterpret_cast<float *>(out) = __fdiv_rn(1.0f, iscale);
}

}  // namespace ckb
