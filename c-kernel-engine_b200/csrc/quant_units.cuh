// Per-lane "work units" of the dequant-dot GEMVs.  A unit is the piece of one weight block
// that one lane multiplies against the matching activation bytes with dp4a:
//
//   Q4_K  unit = quarter q (0..3) of a 144-byte superblock: 32 bytes of nibbles = sub-block 2q
//         (low nibbles) and 2q+1 (high nibbles), 64 activations.  Integer stage = the two
//         32-element sums the reference calls sum_q4q8_lo / sum_q4q8_hi
//         (src/kernels/gemm_kernels_q4k_q8k.c:144-173).
//   Q6_K  unit = quarter (n, h) of a 210-byte superblock: l = 16h..16h+15 of 128-half n, i.e. four
//         16-element scale groups (src/kernels/gemm_kernels_q6k_q8k.c:86-116), 64 activations.
//   Q8_0  unit = one 34-byte block, 32 activations (src/kernels/gemm_kernels_q8_0.c:968-989).
//
// Activations are repacked once per CTA into shared memory in a bank-conflict-free layout:
//   Q8_K: per superblock 16 + 2*HP 16-byte slots (chunk c lives in slot c + HP * (c >> 3)); the pad
//         HP is 1 for the Q4_K access pattern and 2 for the Q6_K one; then fp32 d per block,
//         then eight int32 sums of 32 elements per block.
//   Q8_0: per block 48 bytes = 32 int8 + fp32 d + pad.
#pragma once

#include "device_common.cuh"

namespace ckb {

template <int HP> struct XQ8KLayout { static constexpr int SLOT_WORDS = (16 + 2 * HP) * 4; };

struct XQ8K {                            // shared-memory view of a repacked Q8_K vector
    uint32_t q;                          // shared address of the padded int8 data
    uint32_t d;                          // shared address of fp32 d[nb]
    uint32_t bs;                         // shared address of int32 sums[nb][8]
};

__host__ __device__ inline int xq8k_smem_bytes(int nb, int hp) { return nb * ((16 + 2 * hp) * 16 + 4 + 32); }
__host__ __device__ inline int xq80_smem_bytes(int nblk) { return nblk * 48; }

// Repack `nb` Q8_K blocks (global, 4-byte aligned) into shared memory.  Whole CTA cooperates.
template <int HP>
__device__ __forceinline__ XQ8K load_x_q8k(const uint8_t *xg, int nb, uint8_t *smem)
{
    constexpr int XQ8K_SLOT_WORDS = XQ8KLayout<HP>::SLOT_WORDS;
    uint32_t *xq = reinterpret_cast<uint32_t *>(smem);
    float *xd = reinterpret_cast<float *>(smem + nb * XQ8K_SLOT_WORDS * 4);
    int *xbs = reinterpret_cast<int *>(smem + nb * (XQ8K_SLOT_WORDS * 4 + 4));
    const uint32_t *src = reinterpret_cast<const uint32_t *>(xg);
    for (int i = threadIdx.x; i < nb * 73; i += blockDim.x) {
        const int b = i / 73, w = i - b * 73;
        const uint32_t v = __ldg(src + i);
        if (w == 0) {
            xd[b] = __uint_as_float(v);
        } else if (w <= 64) {
            const int c = (w - 1) >> 2;
            xq[b * XQ8K_SLOT_WORDS + (c + HP * (c >> 3)) * 4 + ((w - 1) & 3)] = v;
        } else {
            xbs[b * 8 + (w - 65)] = (int)(short)(v & 0xffffu) + (int)(short)(v >> 16);
        }
    }
    XQ8K r;
    r.q = smem_u32(xq);
    r.d = smem_u32(xd);
    r.bs = smem_u32(xbs);
    return r;
}

// Repack `nblk` Q8_0 blocks (global, 2-byte aligned) into 48-byte shared slots.
__device__ __forceinline__ uint32_t load_x_q80(const uint8_t *xg, int nblk, uint8_t *smem)
{
    for (int i = threadIdx.x; i < nblk * 17; i += blockDim.x) {
        const int b = i / 17, h = i - b * 17;
        const uint32_t v = ldg_nc_u16(xg + (size_t)b * Q80_BYTES + 2 * h);
        if (h == 0) *reinterpret_cast<float *>(smem + b * 48 + 32) = half_bits_to_float(v);
        else *reinterpret_cast<unsigned short *>(smem + b * 48 + 2 * (h - 1)) = (unsigned short)v;
    }
    return smem_u32(smem);
}

// ---------------------------------------------------------------- Q4_K

// The two 6-bit scales and two 6-bit mins of sub-blocks 2q and 2q+1, from the three packed
// scale words (include/ckernel_quant.h:227-251): returns sc pair and m pair as two bytes each.
__device__ __forceinline__ void q4k_scales(uint32_t s0, uint32_t s1, uint32_t s2, int q, uint32_t &sc2, uint32_t &m2)
{
    const int t = (q & 1) * 16;
    const uint32_t a = s0 >> t, b = s1 >> t, c = s2 >> t;
    if (q < 2) {
        sc2 = a & 0x3F3Fu;
        m2 = b & 0x3F3Fu;
    } else {
        sc2 = (c & 0x0F0Fu) | ((a & 0xC0C0u) >> 2);
        m2 = ((c >> 4) & 0x0F0Fu) | ((b & 0xC0C0u) >> 2);
    }
}

struct Q4kX {            // activations of one unit, in registers
    uint4 lo0, lo1, hi0, hi1;
    float d;
    int bs_lo, bs_hi;
};

__device__ __forceinline__ Q4kX q4k_load_x(const XQ8K &x, int b, int q)
{
    Q4kX r;
    const uint32_t a = x.q + (uint32_t)(b * XQ8KLayout<1>::SLOT_WORDS + (4 * q + (q >> 1)) * 4) * 4u;
    r.lo0 = lds_u4(a);
    r.lo1 = lds_u4(a + 16);
    r.hi0 = lds_u4(a + 32);
    r.hi1 = lds_u4(a + 48);
    r.d = __uint_as_float(lds_u32(x.d + 4u * b));
    r.bs_lo = (int)lds_u32(x.bs + 4u * (8 * b + 2 * q));
    r.bs_hi = (int)lds_u32(x.bs + 4u * (8 * b + 2 * q + 1));
    return r;
}

// Integer stage: the 32-element sums of (low nibble)*q8 and (high nibble)*q8.
__device__ __forceinline__ void q4k_isums(const uint4 &qa, const uint4 &qb, const Q4kX &x, int &sum_lo, int &sum_hi)
{
    const uint32_t m = 0x0F0F0F0Fu;
    int lo = 0, hi = 0;
    lo = dp4a_us(qa.x & m, x.lo0.x, lo); hi = dp4a_us((qa.x >> 4) & m, x.hi0.x, hi);
    lo = dp4a_us(qa.y & m, x.lo0.y, lo); hi = dp4a_us((qa.y >> 4) & m, x.hi0.y, hi);
    lo = dp4a_us(qa.z & m, x.lo0.z, lo); hi = dp4a_us((qa.z >> 4) & m, x.hi0.z, hi);
    lo = dp4a_us(qa.w & m, x.lo0.w, lo); hi = dp4a_us((qa.w >> 4) & m, x.hi0.w, hi);
    lo = dp4a_us(qb.x & m, x.lo1.x, lo); hi = dp4a_us((qb.x >> 4) & m, x.hi1.x, hi);
    lo = dp4a_us(qb.y & m, x.lo1.y, lo); hi = dp4a_us((qb.y >> 4) & m, x.hi1.y, hi);
    lo = dp4a_us(qb.z & m, x.lo1.z, lo); hi = dp4a_us((qb.z >> 4) & m, x.hi1.z, hi);
    lo = dp4a_us(qb.w & m, x.lo1.w, lo); hi = dp4a_us((qb.w >> 4) & m, x.hi1.w, hi);
    sum_lo = lo;
    sum_hi = hi;
}

// fp32 contribution of one unit: d*xd*(sc_lo*sum_lo + sc_hi*sum_hi) - dmin*xd*(m_lo*bs_lo + m_hi*bs_hi).
// The scale-weighted integer sums are exact in int32 (|.| < 2^25).
__device__ __forceinline__ float q4k_unit(const uint4 &hdr, const uint4 &qa, const uint4 &qb, const Q4kX &x, int q)
{
    int sum_lo, sum_hi;
    q4k_isums(qa, qb, x, sum_lo, sum_hi);
    uint32_t sc2, m2;
    q4k_scales(hdr.y, hdr.z, hdr.w, q, sc2, m2);
    const int isum = (int)(sc2 & 255u) * sum_lo + (int)(sc2 >> 8) * sum_hi;
    const int imin = (int)(m2 & 255u) * x.bs_lo + (int)(m2 >> 8) * x.bs_hi;
    const float2 dd = __half22float2(*reinterpret_cast<const __half2 *>(&hdr.x));
    return (dd.x * x.d) * (float)isum - (dd.y * x.d) * (float)imin;
}

// ---------------------------------------------------------------- Q6_K

struct Q6kX {            // activations of one (n, h) quarter
    uint4 x0, x1, x2, x3;   // q8[128n + 32t + 16h .. +15] for t = 0..3
    float d;
};

__device__ __forceinline__ Q6kX q6k_load_x(const XQ8K &x, int b, int n, int h)
{
    Q6kX r;
    // element offset 128n + 32t + 16h -> 16-byte chunk c = 8n + 2t + h -> slot c + 2 * (c >> 3) = 10n + 2t + h
    const uint32_t a = x.q + (uint32_t)(b * XQ8KLayout<2>::SLOT_WORDS + (10 * n + h) * 4) * 4u;
    r.x0 = lds_u4(a);
    r.x1 = lds_u4(a + 32);
    r.x2 = lds_u4(a + 64);
    r.x3 = lds_u4(a + 96);
    r.d = __uint_as_float(lds_u32(x.d + 4u * b));
    return r;
}

// (q6 - 32) for four packed values: low 4 bits from `lo4` (already masked), 2 high bits from
// `hi2` (already in bits 4-5 of each byte); the subtraction is done per byte without borrow.
__device__ __forceinline__ uint32_t q6k_center(uint32_t lo4, uint32_t hi2)
{
    return (((lo4 | hi2) | 0x80808080u) - 0x20202020u) ^ 0x80808080u;
}

__device__ __forceinline__ int q6k_dot4(const uint32_t qa, const uint32_t qb, const uint32_t qh, uint32_t xa, uint32_t xb,
                                        uint32_t xc, uint32_t xd, int &s0, int &s1, int &s2, int &s3)
{
    const uint32_t m4 = 0x0F0F0F0Fu, m2 = 0x30303030u;
    s0 = dp4a_ss(q6k_center(qa & m4, (qh << 4) & m2), xa, s0);
    s1 = dp4a_ss(q6k_center(qb & m4, (qh << 2) & m2), xb, s1);
    s2 = dp4a_ss(q6k_center((qa >> 4) & m4, qh & m2), xc, s2);
    s3 = dp4a_ss(q6k_center((qb >> 4) & m4, (qh >> 2) & m2), xd, s3);
    return 0;
}

// Integer stage of one quarter: four 16-element sums of (q6-32)*q8, for scale groups
// 8n + h + {0, 2, 4, 6}.  ql_a = ql[64n+16h ..], ql_b = ql[64n+32+16h ..], qh = qh[32n+16h ..].
__device__ __forceinline__ void q6k_isums(const uint4 &ql_a, const uint4 &ql_b, const uint4 &qh, const Q6kX &x, int s[4])
{
    s[0] = s[1] = s[2] = s[3] = 0;
    q6k_dot4(ql_a.x, ql_b.x, qh.x, x.x0.x, x.x1.x, x.x2.x, x.x3.x, s[0], s[1], s[2], s[3]);
    q6k_dot4(ql_a.y, ql_b.y, qh.y, x.x0.y, x.x1.y, x.x2.y, x.x3.y, s[0], s[1], s[2], s[3]);
    q6k_dot4(ql_a.z, ql_b.z, qh.z, x.x0.z, x.x1.z, x.x2.z, x.x3.z, s[0], s[1], s[2], s[3]);
    q6k_dot4(ql_a.w, ql_b.w, qh.w, x.x0.w, x.x1.w, x.x2.w, x.x3.w, s[0], s[1], s[2], s[3]);
}

__device__ __forceinline__ float q6k_unit(const uint4 &ql_a, const uint4 &ql_b, const uint4 &qh, int sc0, int sc1, int sc2,
                                          int sc3, uint32_t d_bits, const Q6kX &x)
{
    int s[4];
    q6k_isums(ql_a, ql_b, qh, x, s);
    const int tot = sc0 * s[0] + sc1 * s[1] + sc2 * s[2] + sc3 * s[3];   // |tot| < 2^23, exact
    return (half_bits_to_float(d_bits) * x.d) * (float)tot;
}

// Integer stage of a Q6_K quarter (n, h) without assembling any 6-bit value: the nibble planes and the 2-bit planes are
// multiplied in place (masked, not shifted) by the activation bytes and the place values are applied to the int32 sums.
// S_t = sum over the 16 elements of scale group 8n + h + 2t of q6 * q8 with q6 in 0..63, t = 0..3; the reference's
// sum of (q6 - 32) * q8 (src/kernels/gemm_kernels_q6k_q8k.c:92-111) is S_t - 32 * bsums[8n + h + 2t].
// qa = ql[64n + 16h ..], qb = ql[64n + 32 + 16h ..], qh = qh[32n + 16h ..]; x_t = q8[128n + 32t + 16h ..].
__device__ __forceinline__ void q6k_plane_sums(const uint4 &qa, const uint4 &qb, const uint4 &qh, const uint4 &x0, const uint4 &x1,
                                               const uint4 &x2, const uint4 &x3, int &S1, int &S2, int &S3, int &S4)
{
    int A1 = 0, A2 = 0, A3 = 0, A4 = 0, B1 = 0, B2 = 0, B3 = 0, B4 = 0;
#define CKB_Q6_STEP(QA, QB, QH, X0, X1, X2, X3)                      \
    A1 = dp4a_us((QA) & 0x0F0F0F0Fu, X0, A1); B1 = dp4a_us((QH) & 0x03030303u, X0, B1); \
    A2 = dp4a_us((QB) & 0x0F0F0F0Fu, X1, A2); B2 = dp4a_us((QH) & 0x0C0C0C0Cu, X1, B2); \
    A3 = dp4a_us((QA) & 0xF0F0F0F0u, X2, A3); B3 = dp4a_us((QH) & 0x30303030u, X2, B3); \
    A4 = dp4a_us((QB) & 0xF0F0F0F0u, X3, A4); B4 = dp4a_us((QH) & 0xC0C0C0C0u, X3, B4);
    CKB_Q6_STEP(qa.x, qb.x, qh.x, x0.x, x1.x, x2.x, x3.x)
    CKB_Q6_STEP(qa.y, qb.y, qh.y, x0.y, x1.y, x2.y, x3.y)
    CKB_Q6_STEP(qa.z, qb.z, qh.z, x0.z, x1.z, x2.z, x3.z)
    CKB_Q6_STEP(qa.w, qb.w, qh.w, x0.w, x1.w, x2.w, x3.w)
#undef CKB_Q6_STEP
    S1 = A1 + 16 * B1; S2 = A2 + 4 * B2; S3 = (A3 >> 4) + B3; S4 = (A4 >> 4) + (B4 >> 2);   // all exact
}

// ---------------------------------------------------------------- unaligned 16-byte reads

// 16 bytes starting at a 2-byte-aligned shared address: five aligned words + funnel shifts.
__device__ __forceinline__ uint4 lds_u4_align2(uint32_t addr)
{
    const uint32_t a = addr & ~3u, sh = (addr & 3u) * 8u;
    const uint32_t w0 = lds_u32(a), w1 = lds_u32(a + 4), w2 = lds_u32(a + 8), w3 = lds_u32(a + 12), w4 = lds_u32(a + 16);
    uint4 r;
    r.x = __funnelshift_r(w0, w1, sh);
    r.y = __funnelshift_r(w1, w2, sh);
    r.z = __funnelshift_r(w2, w3, sh);
    r.w = __funnelshift_r(w3, w4, sh);
    return r;
}

// Same from global memory, built from 2-byte loads (no over-read past the 16 bytes).
__device__ __forceinline__ uint4 ldg_u4_align2(const uint8_t *p)
{
    uint4 r;
    r.x = ldg_nc_u16(p) | (ldg_nc_u16(p + 2) << 16);
    r.y = ldg_nc_u16(p + 4) | (ldg_nc_u16(p + 6) << 16);
    r.z = ldg_nc_u16(p + 8) | (ldg_nc_u16(p + 10) << 16);
    r.w = ldg_nc_u16(p + 12) | (ldg_nc_u16(p + 14) << 16);
    return r;
}

// One block_q5_0 against one Q8_0 activation block (vec_dot_q5_0_q8_0_ref, src/kernels/gemm_kernels_q5_0.c:901-939): element j
// (j < 16) is the low nibble of qs[j] with bit j of qh as its fifth bit, element j + 16 the high nibble with bit j + 16, both
// minus 16; int32 dot with the activation bytes, times d_w * d_x.  Four bits of qh are spread to bit 4 of four bytes with
// one multiply (t * 0x00204081 puts bit i of t at bit 8 i), and v - 16 becomes a signed byte without borrows between bytes.
__device__ __forceinline__ uint32_t q50_s8x4(uint32_t nibbles, uint32_t qh_bits4)
{
    const uint32_t v = nibbles | ((((qh_bits4 & 15u) * 0x00204081u) & 0x01010101u) << 4);      // 0 .. 31 per byte
    return ((v | 0x80808080u) - 0x10101010u) ^ 0x80808080u;                                    // v - 16 as int8
}
__device__ __forceinline__ float q50_unit(uint32_t dbits, uint32_t qh, const uint4 &qs, uint32_t xa)
{
    const uint4 x0 = lds_u4(xa), x1 = lds_u4(xa + 16);
    const float xd = __uint_as_float(lds_u32(xa + 32));
    const uint32_t w[4] = {qs.x, qs.y, qs.z, qs.w}, xl[4] = {x0.x, x0.y, x0.z, x0.w}, xh[4] = {x1.x, x1.y, x1.z, x1.w};
    int s = 0;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        s = dp4a_ss(q50_s8x4(w[i] & 0x0F0F0F0Fu, qh >> (4 * i)), xl[i], s);
        s = dp4a_ss(q50_s8x4((w[i] >> 4) & 0x0F0F0F0Fu, qh >> (16 + 4 * i)), xh[i], s);
    }
    return (float)s * (half_bits_to_float(dbits) * xd);
}

// The same block with the -16 taken out of the bytes: sum (v - 16) x = sum nibble x + 16 sum fifth-bit x - 16 sum x, where
// sum x of the activation block was stored once per CTA at byte 36 of the block's 48-byte slot (q50_store_xsums).  Nibbles
// and spread fifth bits go into unsigned x signed dp4a as they are: about 6 integer instructions per 4 weights instead of 10.
__device__ __forceinline__ float q50_unit_presum(uint32_t dbits, uint32_t qh, const uint4 &qs, uint32_t xa)
{
    const uint4 x0 = lds_u4(xa), x1 = lds_u4(xa + 16);
    const float xd = __uint_as_float(lds_u32(xa + 32));
    const int xsum = (int)lds_u32(xa + 36);
    const uint32_t w[4] = {qs.x, qs.y, qs.z, qs.w}, xl[4] = {x0.x, x0.y, x0.z, x0.w}, xh[4] = {x1.x, x1.y, x1.z, x1.w};
    int s = 0, hb = 0;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        s = dp4a_us(w[i] & 0x0F0F0F0Fu, xl[i], s);
        s = dp4a_us((w[i] >> 4) & 0x0F0F0F0Fu, xh[i], s);
        hb = dp4a_us((((qh >> (4 * i)) & 15u) * 0x00204081u) & 0x01010101u, xl[i], hb);
        hb = dp4a_us((((qh >> (16 + 4 * i)) & 15u) * 0x00204081u) & 0x01010101u, xh[i], hb);
    }
    return (float)(s + 16 * (hb - xsum)) * (half_bits_to_float(dbits) * xd);
}

// one thread per activation block: the sum of its 32 bytes into the spare word of the slot (call between two __syncthreads)
__device__ __forceinline__ void q50_store_xsums(uint32_t xq, int nb)
{
    for (int b = threadIdx.x; b < nb; b += blockDim.x) {
        const uint32_t xa = xq + 48u * b;
        const uint4 x0 = lds_u4(xa), x1 = lds_u4(xa + 16);
        int t = 0;
        t = dp4a_ss(0x01010101u, x0.x, t); t = dp4a_ss(0x01010101u, x0.y, t); t = dp4a_ss(0x01010101u, x0.z, t); t = dp4a_ss(0x01010101u, x0.w, t);
        t = dp4a_ss(0x01010101u, x1.x, t); t = dp4a_ss(0x01010101u, x1.y, t); t = dp4a_ss(0x01010101u, x1.z, t); t = dp4a_ss(0x01010101u, x1.w, t);
        asm volatile("st.shared.u32 [%0], %1;" ::"r"(xa + 36), "r"(t) : "memory");
    }
}

}  // namespace ckb
