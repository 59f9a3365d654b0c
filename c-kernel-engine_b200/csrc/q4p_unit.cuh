// The unit of the Q4_K x Q8_K "pair" GEMV (gemv_q4k.cu) and what it needs from shared memory: two lanes per
// superblock, lane p takes the nibble bytes of quarters p and p+2, i.e. sub-blocks 2p, 2p+1 (6-bit scales stored
// directly) and 2p+4, 2p+5 (scales split over two bytes).  Kept in a header because the fused step kernels and the
// integer-stage dump (subblock_sums.cu) run the very same functions.
// Reference arithmetic: dot_q4_k_q8_k_ref, src/kernels/gemm_kernels_q4k_q8k.c:121-181.
#pragma once

#include "quant_units.cuh"

namespace ckb {

// shared-memory layout of the activations for this kernel:
//   q8 data: 17 slots of 16 B per superblock (16 data + 1 pad: 8 consecutive lanes then hit 8 distinct bank groups)
//   d[nb] fp32
//   per (superblock, p): the four 32-element sums of sub-blocks {2p, 2p+1, 2p+4, 2p+5}, split as
//   sum = 128 * hi + lo with lo in [0, 127] and hi in [-32, 31], packed as 4 x s8 (lo word, hi word),
//   so that sum_j m_j * bsum_j is two dp4a
constexpr int Q4P_SLOTS = 17;
__host__ __device__ inline int q4p_smem_bytes(int nb) { return ((nb * (Q4P_SLOTS * 16 + 4 + 16)) + 127) & ~127; }

struct Q4pX { uint32_t q, d, lo, hi; };

// LOCAL_SRC: the Q8_K vector was just built by this CTA in shared memory (a fused quantising prologue) and is read with plain
// loads; otherwise it is global memory written by an earlier kernel and comes through L2.
template <bool LOCAL_SRC = false>
__device__ __forceinline__ Q4pX q4p_stage_x(const uint8_t *xg, int nb, uint8_t *smem)
{
    uint32_t *xq = reinterpret_cast<uint32_t *>(smem);
    float *xd = reinterpret_cast<float *>(smem + nb * Q4P_SLOTS * 16);
    int8_t *lo = reinterpret_cast<int8_t *>(smem + nb * (Q4P_SLOTS * 16 + 4));
    int8_t *hi = lo + nb * 8;
    const uint32_t *src = reinterpret_cast<const uint32_t *>(xg);
    // eight independent loads per thread are issued before the first one is used: the staging costs about
    // one L2 round trip, which matters because it sits between the dependency wait and the first multiply
    const int total = nb * 73;
    for (int base = 0; base < total; base += 8 * blockDim.x) {
        uint32_t v[8];
#pragma unroll
        for (int u = 0; u < 8; ++u) {
            const int i = base + u * blockDim.x + threadIdx.x;
            if constexpr (LOCAL_SRC) v[u] = i < total ? src[i] : 0u;
            else v[u] = i < total ? __ldcg(src + i) : 0u;  // through L2: the producer may overlap this kernel (programmatic launch)
        }
#pragma unroll
        for (int u = 0; u < 8; ++u) {
            const int i = base + u * blockDim.x + threadIdx.x;
            if (i >= total) break;
            const int b = i / 73, w = i - b * 73;
            if (w == 0) {
                xd[b] = __uint_as_float(v[u]);
            } else if (w <= 64) {
                xq[b * Q4P_SLOTS * 4 + (w - 1)] = v[u];
            } else {
                const int j = w - 65;                                  // 32-element sub-block
                const int sum = (int)(short)(v[u] & 0xffffu) + (int)(short)(v[u] >> 16);
                const int p = (j >> 1) & 1, byte = (j & 1) | ((j >> 2) << 1);
                lo[(b * 2 + p) * 4 + byte] = (int8_t)(sum & 127);
                hi[(b * 2 + p) * 4 + byte] = (int8_t)(sum >> 7);
            }
        }
    }
    Q4pX r;
    r.q = smem_u32(xq);
    r.d = smem_u32(xd);
    r.lo = smem_u32(lo);
    r.hi = smem_u32(hi);
    return r;
}

struct Q4pW { uint4 hdr, a0, a1, b0, b1; };     // header, quarter p (32 B), quarter p+2 (32 B)

__device__ __forceinline__ void q4p_nibble_dots(const uint4 &w0, const uint4 &w1, uint32_t xa, int &s_lo, int &s_hi16)
{
    // xa: shared address of the 64 activations of this quarter (32 for the low nibbles, then 32 for the high ones)
    const uint4 l0 = lds_u4(xa), l1 = lds_u4(xa + 16), h0 = lds_u4(xa + 32), h1 = lds_u4(xa + 48);
    const uint32_t ml = 0x0F0F0F0Fu, mh = 0xF0F0F0F0u;
    int lo = 0, hi = 0;
    lo = dp4a_us(w0.x & ml, l0.x, lo); hi = dp4a_us(w0.x & mh, h0.x, hi);
    lo = dp4a_us(w0.y & ml, l0.y, lo); hi = dp4a_us(w0.y & mh, h0.y, hi);
    lo = dp4a_us(w0.z & ml, l0.z, lo); hi = dp4a_us(w0.z & mh, h0.z, hi);
    lo = dp4a_us(w0.w & ml, l0.w, lo); hi = dp4a_us(w0.w & mh, h0.w, hi);
    lo = dp4a_us(w1.x & ml, l1.x, lo); hi = dp4a_us(w1.x & mh, h1.x, hi);
    lo = dp4a_us(w1.y & ml, l1.y, lo); hi = dp4a_us(w1.y & mh, h1.y, hi);
    lo = dp4a_us(w1.z & ml, l1.z, lo); hi = dp4a_us(w1.z & mh, h1.z, hi);
    lo = dp4a_us(w1.w & ml, l1.w, lo); hi = dp4a_us(w1.w & mh, h1.w, hi);
    s_lo = lo;
    s_hi16 = hi;          // 16 x the high-nibble sum (the nibbles were left in place)
}

// Integer stage of (superblock b, lane half p): the 32-element sums of nibble x q8 of sub-blocks 2p (a_lo), 2p+1
// (a_hi16 / 16), 2p+4 (b_lo) and 2p+5 (b_hi16 / 16) - sum_q4q8_lo / sum_q4q8_hi of the reference (:144-167).
__device__ __forceinline__ void q4p_isums(const Q4pW &w, const Q4pX &x, int b, int p, int &a_lo, int &a_hi16, int &b_lo, int &b_hi16)
{
    const uint32_t xa = x.q + (uint32_t)(b * Q4P_SLOTS + 4 * p) * 16u;
    q4p_nibble_dots(w.a0, w.a1, xa, a_lo, a_hi16);             // sub-blocks 2p, 2p+1
    q4p_nibble_dots(w.b0, w.b1, xa + 128, b_lo, b_hi16);       // sub-blocks 2p+4, 2p+5
}

// contribution of (superblock b, lane half p) of one row
__device__ __forceinline__ float q4p_unit(const Q4pW &w, const Q4pX &x, int b, int p)
{
    int a_lo, a_hi16, b_lo, b_hi16;
    q4p_isums(w, x, b, p, a_lo, a_hi16, b_lo, b_hi16);
    const int t = 16 * p;
    const uint32_t a = w.hdr.y >> t, bb = w.hdr.z >> t, c = w.hdr.w >> t;
    const uint32_t scA = a & 0x3F3Fu, mA = bb & 0x3F3Fu;                               // include/ckernel_quant.h:230-238
    const uint32_t scB = (c & 0x0F0Fu) | ((a >> 2) & 0x3030u);                         // :242-245
    const uint32_t mB = ((c >> 4) & 0x0F0Fu) | ((bb >> 2) & 0x3030u);                  // :247-250
    const int isum = (int)(scA & 255u) * a_lo + (int)(scB & 255u) * b_lo +
                     (((int)(scA >> 8) * a_hi16 + (int)(scB >> 8) * b_hi16) >> 4);   // exact: both terms are multiples of 16
    const uint32_t m4 = mA | (mB << 16);
    const uint32_t blo = lds_u32(x.lo + 4u * (2 * b + p)), bhi = lds_u32(x.hi + 4u * (2 * b + p));
    const int imin = dp4a_us(m4, blo, 0) + 128 * dp4a_us(m4, bhi, 0);
    const float xd = __uint_as_float(lds_u32(x.d + 4u * b));
    const float2 dd = __half22float2(*reinterpret_cast<const __half2 *>(&w.hdr.x));
    return (dd.x * xd) * (float)isum - (dd.y * xd) * (float)imin;
}

}  // namespace ckb
