// Activation vector staging shared by the ring GEMV kernels (gemv.cu) and the planar Q6_K GEMV (gemv_q6k_planar.cu):
// the quantised vector is read once per CTA through L2 and repacked into conflict-free shared-memory layouts.
#pragma once
#include "quant_units.cuh"

namespace ckb {

enum Fmt : int { FMT_Q4K = 0, FMT_Q6K = 1, FMT_Q80 = 2, FMT_Q50 = 3 };   // Q5_0 weights take Q8_0 activations, like Q8_0

// Q8_K vector for Q6_K weights: q8 data in the HP = 2 padded layout, fp32 d per block, and per
// (block, half n, l-half h) the four 16-element sums bsums[8n + 2t + h], t = 0..3, split as 128*hi + lo
// and packed 4 x s8, so that sum_t sc_t * bsum_t is two dp4a.
struct RingX {
    uint32_t q, d, lo, hi;   // shared addresses (Q8_K)   | q80: q = 48-byte slots
};

__host__ __device__ inline int ringx_smem_bytes(int fmt, int nb)
{
    const int raw = (fmt == FMT_Q80 || fmt == FMT_Q50) ? nb * 48 : (fmt == FMT_Q6K ? nb * (20 * 16 + 4 + 32) : nb * (18 * 16 + 4 + 32));
    return (raw + 127) & ~127;
}

// Batched loads through L2 (__ldcg): the vector may have been written by a kernel that overlaps this one.
// LOCAL_SRC (Q8_K only): the vector was just built by this CTA in shared memory and is read with plain loads.
template <int FMT, bool LOCAL_SRC = false>
__device__ __forceinline__ RingX ring_stage_x(const uint8_t *xg, int nb, uint8_t *smem)
{
    RingX r;
    if constexpr (FMT == FMT_Q80 || FMT == FMT_Q50) {
        const int total = nb * 17;
        for (int base = 0; base < total; base += 8 * blockDim.x) {
            uint32_t v[8];
#pragma unroll
            for (int u = 0; u < 8; ++u) {
                const int i = base + u * blockDim.x + threadIdx.x;
                v[u] = 0;
                if (i < total) {
                    unsigned short t;
                    asm volatile("ld.global.cg.u16 %0, [%1];" : "=h"(t) : "l"(xg + 2 * (size_t)i));
                    v[u] = t;
                }
            }
#pragma unroll
            for (int u = 0; u < 8; ++u) {
                const int i = base + u * blockDim.x + threadIdx.x;
                if (i < total) {
                    const int b = i / 17, h = i - b * 17;
                    if (h == 0) *reinterpret_cast<float *>(smem + b * 48 + 32) = half_bits_to_float(v[u]);
                    else *reinterpret_cast<unsigned short *>(smem + b * 48 + 2 * (h - 1)) = (unsigned short)v[u];
                }
            }
        }
        r.q = smem_u32(smem);
        r.d = r.lo = r.hi = 0;
    } else {
        constexpr int SLOTS = FMT == FMT_Q6K ? 20 : 18, HP = FMT == FMT_Q6K ? 2 : 1;
        uint32_t *xq = reinterpret_cast<uint32_t *>(smem);
        float *xd = reinterpret_cast<float *>(smem + nb * SLOTS * 16);
        int8_t *lo = reinterpret_cast<int8_t *>(smem + nb * (SLOTS * 16 + 4));
        int8_t *hi = lo + nb * 16;
        const uint32_t *src = reinterpret_cast<const uint32_t *>(xg);
        const int total = nb * 73;
        for (int base = 0; base < total; base += 8 * blockDim.x) {
            uint32_t v[8];
#pragma unroll
            for (int u = 0; u < 8; ++u) {
                const int i = base + u * blockDim.x + threadIdx.x;
                if constexpr (LOCAL_SRC) v[u] = i < total ? src[i] : 0u;
                else v[u] = i < total ? __ldcg(src + i) : 0u;
            }
#pragma unroll
            for (int u = 0; u < 8; ++u) {
                const int i = base + u * blockDim.x + threadIdx.x;
                if (i >= total) break;
                const int b = i / 73, w = i - b * 73;
                if (w == 0) {
                    xd[b] = __uint_as_float(v[u]);
                } else if (w <= 64) {
                    const int c = (w - 1) >> 2;
                    xq[b * SLOTS * 4 + (c + HP * (c >> 3)) * 4 + ((w - 1) & 3)] = v[u];
                } else if constexpr (FMT == FMT_Q6K) {
                    const int j = w - 65, n = j >> 2, t = j & 3;               // bsums[2j] (h = 0), bsums[2j+1] (h = 1)
                    const int s0 = (int)(short)(v[u] & 0xffffu), s1 = (int)(short)(v[u] >> 16);
                    lo[(b * 4 + n * 2 + 0) * 4 + t] = (int8_t)(s0 & 127);
                    hi[(b * 4 + n * 2 + 0) * 4 + t] = (int8_t)(s0 >> 7);
                    lo[(b * 4 + n * 2 + 1) * 4 + t] = (int8_t)(s1 & 127);
                    hi[(b * 4 + n * 2 + 1) * 4 + t] = (int8_t)(s1 >> 7);
                } else {
                    reinterpret_cast<int *>(lo)[b * 8 + (w - 65)] = (int)(short)(v[u] & 0xffffu) + (int)(short)(v[u] >> 16);
                }
            }
        }
        r.q = smem_u32(xq);
        r.d = smem_u32(xd);
        r.lo = smem_u32(lo);
        r.hi = smem_u32(hi);
    }
    return r;
}

}  // namespace ckb
