// Element-wise dequantisation of the weight formats (src/kernels/dequant_kernels.c:276-430):
// the same rounding sequence as the reference (separate fp32 multiplies and subtraction, no FMA).
#pragma once

#include "device_common.cuh"

namespace ckb {

// DQ_Q40 / Q41 / Q51: the 32-element formats in the element order of the reference's row dequantisers (element j in the low nibble of
// qs[j], element j + 16 in the high nibble); the ..._G forms are the order of its fp32-activation GEMVs (the nibbles of qs[i] are elements 2i
// and 2i + 1); DQ_Q5K_F is Q5_K as the fp32 fall-back of gemv_q5_k reads it.  The reference is not consistent between the two orders, and
// each entry point follows the function it replaces.
enum { DQ_Q4K = 0, DQ_Q6K = 1, DQ_Q80 = 2, DQ_Q50 = 3, DQ_Q40 = 4, DQ_Q41 = 5, DQ_Q51 = 6, DQ_Q40_G = 7, DQ_Q41_G = 8, DQ_Q51_G = 9, DQ_Q5K_F = 10 };

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
    } else if constexpr (FMT == DQ_Q40 || FMT == DQ_Q40_G) {
        // block_q4_0: fp16 d, qs[16] (src/kernels/dequant_kernels.c:40-56; GEMV order src/kernels/gemm_kernels_q4_0.c:49-78)
        const float d = half_bits_to_float(p[0] | (p[1] << 8));
        const int bi = FMT == DQ_Q40 ? (e & 15) : (e >> 1), hi = FMT == DQ_Q40 ? (e >> 4) : (e & 1);
        const int q = (hi ? (p[2 + bi] >> 4) : (p[2 + bi] & 15)) - 8;
        return __fmul_rn(d, (float)q);
    } else if constexpr (FMT == DQ_Q41 || FMT == DQ_Q41_G) {
        // block_q4_1: fp16 d, fp16 m, qs[16]: w = d * q + m (src/kernels/dequant_kernels.c:119-139, src/kernels/gemm_kernels_q4_1.c:50-84)
        const float d = half_bits_to_float(p[0] | (p[1] << 8)), m = half_bits_to_float(p[2] | (p[3] << 8));
        const int bi = FMT == DQ_Q41 ? (e & 15) : (e >> 1), hi = FMT == DQ_Q41 ? (e >> 4) : (e & 1);
        const int q = hi ? (p[4 + bi] >> 4) : (p[4 + bi] & 15);
        return __fadd_rn(__fmul_rn(d, (float)q), m);
    } else if constexpr (FMT == DQ_Q51 || FMT == DQ_Q51_G) {
        // block_q5_1: fp16 d, fp16 m, qh[4], qs[16] (src/kernels/dequant_kernels.c:220-252, src/kernels/gemm_kernels_q5_1.c:52-100)
        const float d = half_bits_to_float(p[0] | (p[1] << 8)), m = half_bits_to_float(p[2] | (p[3] << 8));
        const uint32_t qh = p[4] | (p[5] << 8) | (p[6] << 16) | ((uint32_t)p[7] << 24);
        const int bi = FMT == DQ_Q51 ? (e & 15) : (e >> 1), hi = FMT == DQ_Q51 ? (e >> 4) : (e & 1);
        const int bit = FMT == DQ_Q51 ? (hi ? bi + 16 : bi) : e;
        const int q = (hi ? (p[8 + bi] >> 4) : (p[8 + bi] & 15)) | (int)(((qh >> bit) & 1u) << 4);
        return __fadd_rn(__fmul_rn(d, (float)q), m);
    } else if constexpr (FMT == DQ_Q5K_F) {
        // block_q5_K as gemv_q5_k's fp32 fall-back reads it (src/kernels/gemm_kernels_q5_k.c:229-241): (d * sc) * q - dmin * m
        const float d = half_bits_to_float(p[0] | (p[1] << 8)), dmin = half_bits_to_float(p[2] | (p[3] << 8));
        const int sb = e >> 5, i = e & 31;
        int sc, mn;
        q4k_scale_min(p + 4, sb, sc, mn);
        const int q = ((p[48 + sb * 16 + (i >> 1)] >> (4 * (i & 1))) & 15) | (((p[16 + sb * 4 + (i >> 3)] >> (i & 7)) & 1) << 4);
        return __fsub_rn(__fmul_rn(__fmul_rn(d, (float)sc), (float)q), __fmul_rn(dmin, (float)mn));
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
template <> struct DqTraits<DQ_Q40> { static constexpr int BS = 18, BE = 32; };
template <> struct DqTraits<DQ_Q41> { static constexpr int BS = 20, BE = 32; };
template <> struct DqTraits<DQ_Q51> { static constexpr int BS = 24, BE = 32; };
template <> struct DqTraits<DQ_Q40_G> { static constexpr int BS = 18, BE = 32; };
template <> struct DqTraits<DQ_Q41_G> { static constexpr int BS = 20, BE = 32; };
template <> struct DqTraits<DQ_Q51_G> { static constexpr int BS = 24, BE = 32; };
template <> struct DqTraits<DQ_Q5K_F> { static constexpr int BS = 176, BE = 256; };

}  // namespace ckb
