// The unit of the planar Q6_K x Q8_K GEMV (gemv_q6k_planar.cu): one quarter (n, h) of one superblock of one row, fetched with
// aligned loads from the row-planar layout, multiplied in the exact-integer bit-plane form.  In a header because the fused
// step kernels (step_fused.cu) run the same functions.  Reference arithmetic: src/kernels/gemm_kernels_q6k_q8k.c:86-116.
#pragma once

#include "ring_x.cuh"

namespace ckb {

__host__ __device__ inline size_t q6p_row_bytes(int nb) { return ((size_t)nb * Q6K_BYTES + 15) & ~(size_t)15; }

struct Q6pW {              // one quarter of one superblock of one row
    uint4 qa, qb, qh;
    uint2 sc;              // the 8 scale bytes of half n
    uint32_t d;            // fp16 bits
};

__device__ __forceinline__ float q6p_unit(const Q6pW &w, int b, int u, const RingX &x)
{
    const int n = u >> 1, h = u & 1;
    const uint32_t xa = x.q + (uint32_t)(b * 80 + (10 * n + h) * 4) * 4u;
    const uint4 x0 = lds_u4(xa), x1 = lds_u4(xa + 32), x2 = lds_u4(xa + 64), x3 = lds_u4(xa + 96);
    int S1, S2, S3, S4;
    q6k_plane_sums(w.qa, w.qb, w.qh, x0, x1, x2, x3, S1, S2, S3, S4);
    // scales of groups 8n + h + {0, 2, 4, 6}: bytes h, h + 2 of each scale word
    const uint32_t sc4 = h ? __byte_perm(w.sc.x, w.sc.y, 0x7531) : __byte_perm(w.sc.x, w.sc.y, 0x6420);
    const int s0 = (int)(int8_t)(sc4 & 255u), s1 = (int)(int8_t)((sc4 >> 8) & 255u), s2 = (int)(int8_t)((sc4 >> 16) & 255u), s3 = (int)sc4 >> 24;
    const uint32_t lo4 = lds_u32(x.lo + 4u * (b * 4 + u)), hi4 = lds_u32(x.hi + 4u * (b * 4 + u));
    const int center = dp4a_ss(sc4, lo4, 0) + 128 * dp4a_ss(sc4, hi4, 0);          // sum_t sc_t * bsum_t
    const int tot = s0 * S1 + s1 * S2 + s2 * S3 + s3 * S4 - 32 * center;
    const float xd = __uint_as_float(lds_u32(x.d + 4u * b));
    return (half_bits_to_float(w.d) * xd) * (float)tot;
}

// the five aligned loads of quarter u = (n, h) of superblock b of a planar row
__device__ __forceinline__ void q6p_load(Q6pW &w, const uint8_t *row, int nb, int b, int n, int h)
{
    const size_t off_qh = (size_t)nb * 128, off_sc = (size_t)nb * 192, off_d = (size_t)nb * 208;
    w.qa = __ldg(reinterpret_cast<const uint4 *>(row + (size_t)b * 128 + 64 * n + 16 * h));
    w.qb = __ldg(reinterpret_cast<const uint4 *>(row + (size_t)b * 128 + 64 * n + 32 + 16 * h));
    w.qh = __ldg(reinterpret_cast<const uint4 *>(row + off_qh + (size_t)b * 64 + 32 * n + 16 * h));
    w.sc = __ldg(reinterpret_cast<const uint2 *>(row + off_sc + (size_t)b * 16 + 8 * n));
    w.d = ldg_nc_u16(row + off_d + (size_t)b * 2);
}

}  // namespace ckb
