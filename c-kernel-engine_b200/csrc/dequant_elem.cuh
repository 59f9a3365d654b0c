// Element-wise dequantisation of the weight formats (src/kernels/dequant_kernels.c:276-430):
// the same rounding sequence as the reference (separate fp32 multiplies and subtraction, no FMA).
#pragma once

#include "device_common.cuh"

namespace ckb {

enum { DQ_Q4K = 0, DQ_Q6K = 1, DQ_Q80 = 2, DQ_Q50 = 3 };

__device__ __forceinline__ void q4k_scale_min(const uint8_t *s, int j, int &sc, int &mn)
{
    if (j < 4) {
        sc = s[j] & 63;
        mn = s[j + 4] & 63;
    } else {
        sc = (s[j + 4] & 15) | ((s[j - 4] >> 6) << 4);
        mn = (s[j + 4] >> 4) | ((s[j] >> 6) << 4);
    }
}

// weight value of element e of the block at p
template <int FMT>
__device__ __forceinline__ float dequant_elem(const uint8_t *p, int e)
{
    if constexpr (FMT == DQ_Q4K) {
        const float d = half_bits_to_float(p[0] | (p[1] << 8)), dmin = half_bits_to_float(p[2] | (p[3] << 8));
        const int j = e >> 5, l = e & 31;
        int sc, mn;
        q4k_scale_min(p + 4, j, sc, mn);
        const uint8_t byte = p[16 + 32 * (j >> 1) + l];
        const int q = (j & 1) ? (byte >> 4) : (byte & 15);
        return __fsub_rn(__fmul_rn(__fmul_rn(d, (float)sc), (float)q), __fmul_rn(dmin, (float)mn));
    } else if constexpr (FMT == DQ_Q6K) {
        const int half = e >> 7, r = e & 127, quarter = r >> 5, l = r & 31;
        const uint8_t lo = p[64 * half + l + 32 * (quarter & 1)];
        const uint8_t h = p[128 + 32 * half + l];
        const int nib = quarter >= 2 ? (lo >> 4) : (lo & 15);
        const int q = (nib | (((h >> (2 * quarter)) & 3) << 4)) - 32;
        const float d = half_bits_to_float(p[208] | (p[209] << 8));
        const int sc = (int)(int8_t)p[192 + (e >> 4)];
        return __fmul_rn(__fmul_rn(d, (float)sc), (float)q);
    } else if constexpr (FMT == DQ_Q50) {
        // block_q5_0 (src/kernels/dequant_kernels.c:160-193): element j < 16: low nibble of qs[j] and bit j of qh; j + 16: high nibble, bit j + 16
        const float d = half_bits_to_float(p[0] | (p[1] << 8));
        const uint32_t qh = p[2] | (p[3] << 8) | (p[4] << 16) | ((uint32_t)p[5] << 24);
        const int j = e & 15, nib = e < 16 ? (p[6 + j] & 15) : (p[6 + j] >> 4);
        return __fmul_rn(d, (float)((nib | (int)(((qh >> e) & 1u) << 4)) - 16));
    } else {
        const float d = half_bits_to_float(p[0] | (p[1] << 8));
        return __fmul_rn(d, (float)(int8_t)p[2 + e]);
    }
}

template <int FMT> struct DqTraits;
template <> struct DqTraits<DQ_Q4K> { static constexpr int BS = Q4K_BYTES, BE = 256; };
template <> struct DqTraits<DQ_Q6K> { static constexpr int BS = Q6K_BYTES, BE = 256; };
template <> struct DqTraits<DQ_Q80> { static constexpr int BS = Q80_BYTES, BE = 32; };
template <> struct DqTraits<DQ_Q50> { static constexpr int BS = Q50_BYTES, BE = 32; };

}  // namespace ckb
