/*
 * ck_oracle.c - CPU restatement of the C-Kernel-Engine quantised decode/prefill hot path.
 *
 * TEST INFRASTRUCTURE ONLY.  This file is the checker for the CUDA kernels: the
 * parity tests, the smoke check and the bench's cpu_baseline leg load it; the
 * product library never links, loads or calls it.
 *
 * Every function restates the arithmetic of one reference function (cited as
 * file:line inside the reference project) in plain scalar C, keeping the
 * reference's fp32 evaluation order so that a build with -ffp-contract=off is
 * bit-identical to the reference's scalar (_ref) functions.  Parity is pinned:
 * tests/golden/ holds outputs of the reference itself (built unmodified into
 * oracle/_ref/libck_ref.so) and tests/test_oracle.py checks this file against
 * them byte for byte.
 */
#include <math.h>
#include <stddef.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#define ORC_QK_K 256
#define ORC_QK8_0 32

/* Block layouts: include/ckernel_quant.h:104-107, :124-129, :139-144, :153-157 */
#pragma pack(push, 1)
typedef struct { uint16_t d; int8_t qs[32]; } orc_q8_0;                              /* 34 B  */
typedef struct { uint16_t d, dmin; uint8_t scales[12]; uint8_t qs[128]; } orc_q4_K;   /* 144 B */
typedef struct { uint8_t ql[128]; uint8_t qh[64]; int8_t scales[16]; uint16_t d; } orc_q6_K; /* 210 B */
typedef struct { float d; int8_t qs[256]; int16_t bsums[16]; } orc_q8_K;              /* 292 B */
#pragma pack(pop)

_Static_assert(sizeof(orc_q8_0) == 34, "q8_0");
_Static_assert(sizeof(orc_q4_K) == 144, "q4_K");
_Static_assert(sizeof(orc_q6_K) == 210, "q6_K");
_Static_assert(sizeof(orc_q8_K) == 292, "q8_K");

/* ---- fp16 <-> fp32 (include/ckernel_quant.h:265-294, :311-336; IEEE, RNE) ---- */

float oracle_fp16_to_fp32(uint16_t h)
{
    const uint32_t sgn = (uint32_t)(h >> 15) << 31;
    int e = (h >> 10) & 31;
    uint32_t f = h & 1023u;
    uint32_t bits;
    if (e == 31) {
        bits = sgn | 0x7F800000u | (f << 13);
    } else if (e != 0) {
        bits = sgn | ((uint32_t)(e + 112) << 23) | (f << 13);
    } else if (f == 0) {
        bits = sgn;
    } else {
        e = 113;
        do { f <<= 1; --e; } while (!(f & 1024u));
        bits = sgn | ((uint32_t)e << 23) | ((f & 1023u) << 13);
    }
    float out;
    memcpy(&out, &bits, 4);
    return out;
}

uint16_t oracle_fp32_to_fp16(float v)
{
    uint32_t u;
    memcpy(&u, &v, 4);
    const uint16_t sgn = (uint16_t)((u >> 16) & 0x8000u);
    const uint32_t a = u & 0x7FFFFFFFu;
    if (a > 0x7F800000u) return (uint16_t)(sgn | 0x7E00u);          /* NaN */
    if (a >= 0x477FF000u) return (uint16_t)(sgn | 0x7C00u);         /* >= 65520 rounds to infinity */
    if (a < 0x33000001u) return sgn;                                /* <= 2^-25: to zero (tie goes to even = 0) */
    int e = (int)(a >> 23) - 127;
    uint32_t m = (a & 0x7FFFFFu) | 0x800000u;
    int shift;
    uint32_t base;
    if (e < -14) { shift = 13 + (-14 - e); base = 0; }               /* subnormal half */
    else { shift = 13; base = (uint32_t)(e + 15) << 10; m &= 0x7FFFFFu; }
    uint32_t q = m >> shift;
    const uint32_t rem = m & ((1u << shift) - 1u);
    const uint32_t half = 1u << (shift - 1);
    if (rem > half || (rem == half && (q & 1u))) ++q;
    return (uint16_t)(sgn | (base + q));
}

/* ---- Q4_K 6-bit scale/min unpack (include/ckernel_quant.h:227-251) ---- */

void oracle_unpack_q4_k_scales(const uint8_t *s, uint8_t *sc, uint8_t *mn)
{
    for (int j = 0; j < 4; ++j) {
        sc[j] = s[j] & 63;
        mn[j] = s[j + 4] & 63;
        sc[j + 4] = (uint8_t)((s[j + 8] & 15) | ((s[j] >> 6) << 4));
        mn[j + 4] = (uint8_t)((s[j + 8] >> 4) | ((s[j + 4] >> 6) << 4));
    }
}

/* ---- Q8_K activation quantiser (src/kernels/gemm_kernels_q4k_q8k.c:45-103;
 *      same contract as src/kernels/quantize_row_q8_k_sse.c:22-82) ----
 * Signed value of the first element with the strictly largest |x| picks the
 * scale; iscale = -127/max; q = RNE(iscale*x) with the product rounded to fp32
 * first; bsums over 16 elements; d = 1/iscale. */

static int orc_rne(float v)
{
    /* |v| <= 128 here, so nearbyintf under the default rounding mode is the
     * same integer as the reference's add-magic-constant trick. */
    return (int)nearbyintf(v);
}

void oracle_quantize_row_q8_k(const float *x, void *vy, int k)
{
    if (!x || !vy || k <= 0) return;
    orc_q8_K *y = (orc_q8_K *)vy;
    const int nb = k / ORC_QK_K;
    for (int b = 0; b < nb; ++b, x += ORC_QK_K) {
        float best = 0.0f, pick = 0.0f;
        for (int j = 0; j < ORC_QK_K; ++j) {
            const float a = fabsf(x[j]);
            if (a > best) { best = a; pick = x[j]; }
        }
        if (best == 0.0f) {
            memset(&y[b], 0, sizeof(orc_q8_K));
            continue;
        }
        const float iscale = -127.0f / pick;
        for (int j = 0; j < ORC_QK_K; ++j) {
            const float p = iscale * x[j];
            int q = orc_rne(p);
            q = q > 127 ? 127 : (q < -128 ? -128 : q);
            y[b].qs[j] = (int8_t)q;
        }
        for (int g = 0; g < 16; ++g) {
            int s = 0;
            for (int j = 0; j < 16; ++j) s += y[b].qs[16 * g + j];
            y[b].bsums[g] = (int16_t)s;
        }
        y[b].d = 1.0f / iscale;
    }
}

/* quantize_batch_q8_k: src/kernels/gemm_kernels_q8_0.c:221-239 (rows are independent) */
void oracle_quantize_batch_q8_k(const float *x, void *vy, int rows, int k)
{
    uint8_t *out = (uint8_t *)vy;
    for (int r = 0; r < rows; ++r)
        oracle_quantize_row_q8_k(x + (size_t)r * k, out + (size_t)r * (k / ORC_QK_K) * sizeof(orc_q8_K), k);
}

/* ---- Q8_0 activation quantiser (src/kernels/gemm_kernels_q8_0.c:70-175) ----
 * amax over 32; d = amax/127 stored as fp16; id = 127/amax from the fp32 amax;
 * q = RNE(x*id).  The vector path of the reference does not clamp (|q| <= 127
 * by construction); neither does this. */
void oracle_quantize_row_q8_0(const float *x, void *vy, int k)
{
    orc_q8_0 *y = (orc_q8_0 *)vy;
    const int nb = k / ORC_QK8_0;
    for (int b = 0; b < nb; ++b, x += ORC_QK8_0) {
        float amax = 0.0f;
        for (int j = 0; j < ORC_QK8_0; ++j) {
            const float a = fabsf(x[j]);
            if (a > amax) amax = a;
        }
        const float d = amax / 127.0f;
        const float id = amax != 0.0f ? 127.0f / amax : 0.0f;
        y[b].d = oracle_fp32_to_fp16(d);
        for (int j = 0; j < ORC_QK8_0; ++j) {
            const float p = x[j] * id;
            y[b].qs[j] = (int8_t)orc_rne(p);
        }
    }
}

void oracle_quantize_batch_q8_0(const float *x, void *vy, int rows, int k)
{
    uint8_t *out = (uint8_t *)vy;
    for (int r = 0; r < rows; ++r)
        oracle_quantize_row_q8_0(x + (size_t)r * k, out + (size_t)r * (k / ORC_QK8_0) * sizeof(orc_q8_0), k);
}

/* ---- Q4_K x Q8_K (src/kernels/gemm_kernels_q4k_q8k.c:121-200) ---- */

/* Integer stage: the eight 32-element sums of nibble*q8 of one superblock. */
static void orc_q4k_isums(const orc_q4_K *w, const orc_q8_K *x, int32_t out[8])
{
    for (int g = 0; g < 4; ++g) {
        int32_t lo = 0, hi = 0;
        for (int l = 0; l < 32; ++l) {
            const uint8_t byte = w->qs[32 * g + l];
            lo += (int32_t)(byte & 15) * x->qs[64 * g + l];
            hi += (int32_t)(byte >> 4) * x->qs[64 * g + 32 + l];
        }
        out[2 * g] = lo;
        out[2 * g + 1] = hi;
    }
}

void oracle_q4_k_q8_k_subblock_sums(const void *w_row, const void *x_q8, int K, int32_t *out)
{
    const orc_q4_K *w = (const orc_q4_K *)w_row;
    const orc_q8_K *x = (const orc_q8_K *)x_q8;
    for (int b = 0; b < K / ORC_QK_K; ++b) orc_q4k_isums(&w[b], &x[b], out + 8 * b);
}

static float orc_dot_q4k_q8k(const orc_q4_K *w, const orc_q8_K *x, int nb)
{
    float acc = 0.0f;
    for (int b = 0; b < nb; ++b) {
        uint8_t sc[8], mn[8];
        int32_t is[8];
        oracle_unpack_q4_k_scales(w[b].scales, sc, mn);
        orc_q4k_isums(&w[b], &x[b], is);
        const float d = oracle_fp16_to_fp32(w[b].d) * x[b].d;
        const float dm = oracle_fp16_to_fp32(w[b].dmin) * x[b].d;
        for (int j = 0; j < 8; ++j) {
            const int32_t bs = (int32_t)x[b].bsums[2 * j] + (int32_t)x[b].bsums[2 * j + 1];
            acc += d * (float)sc[j] * (float)is[j];
            acc -= dm * (float)mn[j] * (float)bs;
        }
    }
    return acc;
}

void oracle_gemv_q4_k_q8_k(float *y, const void *W, const void *x_q8, int M, int K)
{
    if (!y || !W || !x_q8 || M <= 0 || K <= 0) return;
    const int nb = K / ORC_QK_K;
    const orc_q4_K *w = (const orc_q4_K *)W;
    for (int r = 0; r < M; ++r) y[r] = orc_dot_q4k_q8k(w + (size_t)r * nb, (const orc_q8_K *)x_q8, nb);
}

/* gemm_nt_q4_k_q8_k: src/kernels/gemm_kernels_q4k_q8k.c:301-326 - C[m][n] = dot(B row n, A row m) + bias[n] */
void oracle_gemm_nt_q4_k_q8_k(const void *A_q8, const void *B, const float *bias, float *C, int M, int N, int K)
{
    if (!A_q8 || !B || !C || M <= 0 || N <= 0 || K <= 0) return;
    const int nb = K / ORC_QK_K;
    const orc_q8_K *a = (const orc_q8_K *)A_q8;
    for (int m = 0; m < M; ++m) {
        oracle_gemv_q4_k_q8_k(C + (size_t)m * N, B, a + (size_t)m * nb, N, K);
        if (bias) for (int n = 0; n < N; ++n) C[(size_t)m * N + n] += bias[n];
    }
}

/* fp32-activation Q4_K GEMV: src/kernels/gemm_kernels_q4k.c:53-101 (dequantise then multiply,
 * weight = d*sc*q - dmin*m as in src/kernels/dequant_kernels.c:336-366) */
void oracle_dequant_q4_k_row(const void *src, float *dst, size_t n)
{
    const orc_q4_K *w = (const orc_q4_K *)src;
    for (size_t b = 0; b < n / ORC_QK_K; ++b) {
        uint8_t sc[8], mn[8];
        oracle_unpack_q4_k_scales(w[b].scales, sc, mn);
        const float d = oracle_fp16_to_fp32(w[b].d), dm = oracle_fp16_to_fp32(w[b].dmin);
        float *o = dst + b * ORC_QK_K;
        for (int g = 0; g < 4; ++g) {
            const float d1 = d * (float)sc[2 * g], m1 = dm * (float)mn[2 * g];
            const float d2 = d * (float)sc[2 * g + 1], m2 = dm * (float)mn[2 * g + 1];
            for (int l = 0; l < 32; ++l) {
                const uint8_t byte = w[b].qs[32 * g + l];
                o[64 * g + l] = d1 * (float)(byte & 15) - m1;
                o[64 * g + 32 + l] = d2 * (float)(byte >> 4) - m2;
            }
        }
    }
}

/* ---- Q6_K x Q8_K (src/kernels/gemm_kernels_q6k_q8k.c:70-120, :197-214) ---- */

/* 6-bit value (already minus 32) of element e (0..255) of a superblock. */
static int orc_q6_value(const orc_q6_K *w, int e)
{
    const int half = e >> 7, r = e & 127, quarter = r >> 5, l = r & 31;
    const uint8_t *ql = w->ql + 64 * half;
    const uint8_t h = w->qh[32 * half + l];
    const uint8_t lo = ql[l + 32 * (quarter & 1)];
    const int nib = quarter >= 2 ? (lo >> 4) : (lo & 15);
    return (nib | (((h >> (2 * quarter)) & 3) << 4)) - 32;
}

/* Integer stage: sixteen 16-element sums of (q6-32)*q8 of one superblock; sum j
 * covers elements 16j..16j+15 and is scaled by scales[j]. */
static void orc_q6k_isums(const orc_q6_K *w, const orc_q8_K *x, int32_t out[16])
{
    for (int j = 0; j < 16; ++j) {
        int32_t s = 0;
        for (int i = 0; i < 16; ++i) s += orc_q6_value(w, 16 * j + i) * (int32_t)x->qs[16 * j + i];
        out[j] = s;
    }
}

void oracle_q6_k_q8_k_subblock_sums(const void *w_row, const void *x_q8, int K, int32_t *out)
{
    const orc_q6_K *w = (const orc_q6_K *)w_row;
    const orc_q8_K *x = (const orc_q8_K *)x_q8;
    for (int b = 0; b < K / ORC_QK_K; ++b) orc_q6k_isums(&w[b], &x[b], out + 16 * b);
}

/* The reference's scalar order: per element, fp32, l-major over four strided streams. */
static float orc_dot_q6k_q8k(const orc_q6_K *w, const orc_q8_K *x, int nb)
{
    float acc = 0.0f;
    for (int b = 0; b < nb; ++b) {
        const float d = oracle_fp16_to_fp32(w[b].d) * x[b].d;
        for (int half = 0; half < 2; ++half) {
            const int8_t *sc = w[b].scales + 8 * half;
            const int8_t *q8 = x[b].qs + 128 * half;
            for (int l = 0; l < 32; ++l) {
                const int is = l >> 4;
                for (int qt = 0; qt < 4; ++qt) {
                    const int e = 128 * half + 32 * qt + l;
                    acc += d * (float)sc[is + 2 * qt] * (float)orc_q6_value(&w[b], e) * (float)q8[32 * qt + l];
                }
            }
        }
    }
    return acc;
}

void oracle_gemv_q6_k_q8_k(float *y, const void *W, const void *x_q8, int M, int K)
{
    if (!y || !W || !x_q8 || M <= 0 || K <= 0) return;
    const int nb = K / ORC_QK_K;
    const orc_q6_K *w = (const orc_q6_K *)W;
    for (int r = 0; r < M; ++r) y[r] = orc_dot_q6k_q8k(w + (size_t)r * nb, (const orc_q8_K *)x_q8, nb);
}

/* The reference's vector paths (src/kernels/gemm_kernels_q6k_q8k.c:601-695, :887-1002)
 * sum scale*isum in int32 per superblock and apply d once; same value up to fp32 rounding. */
void oracle_gemv_q6_k_q8_k_intorder(float *y, const void *W, const void *x_q8, int M, int K)
{
    if (!y || !W || !x_q8 || M <= 0 || K <= 0) return;
    const int nb = K / ORC_QK_K;
    const orc_q6_K *w = (const orc_q6_K *)W;
    const orc_q8_K *x = (const orc_q8_K *)x_q8;
    for (int r = 0; r < M; ++r) {
        float acc = 0.0f;
        for (int b = 0; b < nb; ++b) {
            int32_t is[16], tot = 0;
            const orc_q6_K *wb = &w[(size_t)r * nb + b];
            orc_q6k_isums(wb, &x[b], is);
            for (int j = 0; j < 16; ++j) tot += (int32_t)wb->scales[j] * is[j];
            acc += oracle_fp16_to_fp32(wb->d) * x[b].d * (float)tot;
        }
        y[r] = acc;
    }
}

void oracle_gemm_nt_q6_k_q8_k(const void *A_q8, const void *B, const float *bias, float *C, int M, int N, int K)
{
    if (!A_q8 || !B || !C || M <= 0 || N <= 0 || K <= 0) return;
    const int nb = K / ORC_QK_K;
    const orc_q8_K *a = (const orc_q8_K *)A_q8;
    for (int m = 0; m < M; ++m) {
        oracle_gemv_q6_k_q8_k(C + (size_t)m * N, B, a + (size_t)m * nb, N, K);
        if (bias) for (int n = 0; n < N; ++n) C[(size_t)m * N + n] += bias[n];
    }
}

/* src/kernels/dequant_kernels.c:391-430 */
void oracle_dequant_q6_k_row(const void *src, float *dst, size_t n)
{
    const orc_q6_K *w = (const orc_q6_K *)src;
    for (size_t b = 0; b < n / ORC_QK_K; ++b) {
        const float d = oracle_fp16_to_fp32(w[b].d);
        for (int e = 0; e < ORC_QK_K; ++e)
            dst[b * ORC_QK_K + e] = d * (float)w[b].scales[e >> 4] * (float)orc_q6_value(&w[b], e);
    }
}

/* ---- Q8_0 (src/kernels/gemm_kernels_q8_0.c:254-277, :968-989, :1237-1251) ---- */

void oracle_gemv_q8_0(float *y, const void *W, const float *x, int M, int K)
{
    const orc_q8_0 *w = (const orc_q8_0 *)W;
    const int nb = K / ORC_QK8_0;
    for (int r = 0; r < M; ++r) {
        float acc = 0.0f;
        for (int b = 0; b < nb; ++b) {
            const orc_q8_0 *blk = &w[(size_t)r * nb + b];
            const float d = oracle_fp16_to_fp32(blk->d);
            for (int i = 0; i < ORC_QK8_0; ++i) acc += d * (float)blk->qs[i] * x[b * ORC_QK8_0 + i];
        }
        y[r] = acc;
    }
}

void oracle_vec_dot_q8_0_q8_0(int n, float *s, const void *vx, const void *vy)
{
    const orc_q8_0 *a = (const orc_q8_0 *)vx, *b = (const orc_q8_0 *)vy;
    float acc = 0.0f;
    for (int ib = 0; ib < n / ORC_QK8_0; ++ib) {
        int32_t si = 0;
        for (int j = 0; j < ORC_QK8_0; ++j) si += (int32_t)a[ib].qs[j] * (int32_t)b[ib].qs[j];
        acc += (float)si * (oracle_fp16_to_fp32(a[ib].d) * oracle_fp16_to_fp32(b[ib].d));
    }
    *s = acc;
}

void oracle_q8_0_q8_0_block_sums(const void *w_row, const void *x_q8, int K, int32_t *out)
{
    const orc_q8_0 *a = (const orc_q8_0 *)w_row, *b = (const orc_q8_0 *)x_q8;
    for (int ib = 0; ib < K / ORC_QK8_0; ++ib) {
        int32_t si = 0;
        for (int j = 0; j < ORC_QK8_0; ++j) si += (int32_t)a[ib].qs[j] * (int32_t)b[ib].qs[j];
        out[ib] = si;
    }
}

void oracle_gemv_q8_0_q8_0(float *y, const void *W, const void *x_q8, int M, int K)
{
    const orc_q8_0 *w = (const orc_q8_0 *)W;
    const int nb = K / ORC_QK8_0;
    for (int r = 0; r < M; ++r) oracle_vec_dot_q8_0_q8_0(K, &y[r], w + (size_t)r * nb, x_q8);
}

/* gemm_nt_q8_0_q8_0: src/kernels/gemm_batch_int8.c:87-120 */
void oracle_gemm_nt_q8_0_q8_0(const void *A_q8, const void *B, const float *bias, float *C, int M, int N, int K)
{
    const orc_q8_0 *a = (const orc_q8_0 *)A_q8;
    const int nb = K / ORC_QK8_0;
    for (int m = 0; m < M; ++m) {
        oracle_gemv_q8_0_q8_0(C + (size_t)m * N, B, a + (size_t)m * nb, N, K);
        if (bias) for (int n = 0; n < N; ++n) C[(size_t)m * N + n] += bias[n];
    }
}

/* src/kernels/dequant_kernels.c:276-296 */
void oracle_dequant_q8_0_row(const void *src, float *dst, size_t n)
{
    const orc_q8_0 *w = (const orc_q8_0 *)src;
    for (size_t b = 0; b < n / ORC_QK8_0; ++b) {
        const float d = oracle_fp16_to_fp32(w[b].d);
        for (int i = 0; i < ORC_QK8_0; ++i) dst[b * ORC_QK8_0 + i] = d * (float)w[b].qs[i];
    }
}

/* ---- Decode attention over the head-major KV cache
 *      (src/kernels/attention_kernels.c:3365-3406 -> src/kernels/attention_flash_true.c:142-230) ----
 * One query token; per Q head an online softmax over key tiles of 32 (d<=64),
 * 16 (d<=128) or 8 keys (attention_flash_true.c:88-106). */
static int orc_tile_k(int d) { return d > 128 ? 8 : (d > 64 ? 16 : 32); }

static void orc_flash_decode_head(float *out, const float *q, const float *k, const float *v, int T, int D, float scale)
{
    const int tile = orc_tile_k(D);
    float run_max = -INFINITY, run_sum = 0.0f, sc[32];
    for (int i = 0; i < D; ++i) out[i] = 0.0f;
    for (int t0 = 0; t0 < T; t0 += tile) {
        const int n = T - t0 < tile ? T - t0 : tile;
        float blk_max = -INFINITY;
        for (int j = 0; j < n; ++j) {
            const float *kr = k + (size_t)(t0 + j) * D;
            float dot = 0.0f;
            for (int i = 0; i < D; ++i) dot += q[i] * kr[i];
            sc[j] = dot * scale;
            if (sc[j] > blk_max) blk_max = sc[j];
        }
        if (blk_max > run_max) {
            const float f = run_max == -INFINITY ? 0.0f : expf(run_max - blk_max);
            run_sum *= f;
            for (int i = 0; i < D; ++i) out[i] *= f;
            run_max = blk_max;
        }
        for (int j = 0; j < n; ++j) {
            const float *vr = v + (size_t)(t0 + j) * D;
            const float p = expf(sc[j] - run_max);
            run_sum += p;
            for (int i = 0; i < D; ++i) out[i] += p * vr[i];
        }
    }
    if (run_sum > 0.0f) {
        const float inv = 1.0f / run_sum;
        for (int i = 0; i < D; ++i) out[i] *= inv;
    } else {
        for (int i = 0; i < D; ++i) out[i] = 0.0f;
    }
}

void oracle_attention_forward_decode_head_major_gqa_flash(const float *q_token, const float *k_cache,
                                                          const float *v_cache, float *out_token,
                                                          int num_heads, int num_kv_heads, int kv_tokens,
                                                          int cache_capacity, int head_dim, int aligned_head_dim)
{
    if (!q_token || !k_cache || !v_cache || !out_token) return;
    if (num_heads <= 0 || num_kv_heads <= 0 || kv_tokens <= 0 || cache_capacity <= 0) return;
    if (kv_tokens > cache_capacity || head_dim <= 0 || aligned_head_dim <= 0) return;
    const float scale = 1.0f / sqrtf((float)head_dim);
    const size_t hs = (size_t)cache_capacity * (size_t)aligned_head_dim;
    for (int h = 0; h < num_heads; ++h) {
        const int kvh = (int)((long long)h * num_kv_heads / num_heads);
        orc_flash_decode_head(out_token + (size_t)h * aligned_head_dim, q_token + (size_t)h * aligned_head_dim,
                              k_cache + kvh * hs, v_cache + kvh * hs, kv_tokens, aligned_head_dim, scale);
    }
}

/* ---- Q5_0 x Q8_0 (src/kernels/gemm_kernels_q5_0.c:901-939 vec_dot, :1637-1651 gemv, :1725-1752 gemm_nt) ----
 * block_q5_0 = { fp16 d; u8 qh[4]; u8 qs[16] } (include/ckernel_quant.h:70-74): element j < 16 is the low nibble of qs[j]
 * with bit j of qh as bit 4, element j + 16 the high nibble with bit j + 16, both minus 16. */
typedef struct { uint16_t d; uint8_t qh[4]; uint8_t qs[16]; } orc_q5_0;
typedef struct { uint16_t d; int8_t qs[32]; } orc_q8_0_blk;

void oracle_vec_dot_q5_0_q8_0(int n, float *s, const void *vx, const void *vy)
{
    const orc_q5_0 *x = (const orc_q5_0 *)vx;
    const orc_q8_0_blk *y = (const orc_q8_0_blk *)vy;
    float sumf = 0.0f;
    for (int ib = 0; ib < n / 32; ++ib) {
        uint32_t qh;
        memcpy(&qh, x[ib].qh, 4);
        int sumi0 = 0, sumi1 = 0;
        for (int j = 0; j < 16; ++j) {
            const int x0 = (int)((x[ib].qs[j] & 15) | (((qh >> j) & 1u) << 4)) - 16;
            const int x1 = (int)((x[ib].qs[j] >> 4) | (((qh >> (j + 16)) & 1u) << 4)) - 16;
            sumi0 += x0 * y[ib].qs[j];
            sumi1 += x1 * y[ib].qs[j + 16];
        }
        sumf += (oracle_fp16_to_fp32(x[ib].d) * oracle_fp16_to_fp32(y[ib].d)) * (float)(sumi0 + sumi1);
    }
    *s = sumf;
}

/* dequant_q5_0_row (src/kernels/dequant_kernels.c:160-206) and gemv_q5_0_ref (src/kernels/gemm_kernels_q5_0.c:67-111):
 * weight = d * (q5 - 16); the GEMV adds d * q * x element by element in block order */
void oracle_dequant_q5_0_row(const void *src, float *dst, size_t n)
{
    const orc_q5_0 *b = (const orc_q5_0 *)src;
    for (size_t ib = 0; ib < n / 32; ++ib) {
        const float d = oracle_fp16_to_fp32(b[ib].d);
        uint32_t qh;
        memcpy(&qh, b[ib].qh, 4);
        for (int j = 0; j < 16; ++j) {
            const int q0 = (int)((b[ib].qs[j] & 15) | (((qh >> j) & 1u) << 4)) - 16;
            const int q1 = (int)((b[ib].qs[j] >> 4) | (((qh >> (j + 16)) & 1u) << 4)) - 16;
            dst[ib * 32 + j] = d * (float)q0;
            dst[ib * 32 + j + 16] = d * (float)q1;
        }
    }
}

void oracle_gemv_q5_0(float *y, const void *W, const float *x, int M, int K)
{
    if (!y || !W || !x || M <= 0 || K <= 0) return;
    const orc_q5_0 *w = (const orc_q5_0 *)W;
    float tmp[32];
    for (int r = 0; r < M; ++r) {
        float sum = 0.0f;
        for (int b = 0; b < K / 32; ++b) {
            oracle_dequant_q5_0_row(&w[(size_t)r * (K / 32) + b], tmp, 32);
            for (int j = 0; j < 16; ++j) {           /* the reference walks the packed bytes: elements j and j + 16 together */
                sum += tmp[j] * x[b * 32 + j];
                sum += tmp[j + 16] * x[b * 32 + j + 16];
            }
        }
        y[r] = sum;
    }
}

void oracle_gemv_q5_0_q8_0(float *y, const void *W, const void *x_q8, int M, int K)
{
    if (!y || !W || !x_q8 || M <= 0 || K <= 0) return;
    const orc_q5_0 *w = (const orc_q5_0 *)W;
    for (int r = 0; r < M; ++r) oracle_vec_dot_q5_0_q8_0(K, &y[r], w + (size_t)r * (K / 32), x_q8);
}

void oracle_gemm_nt_q5_0_q8_0(const void *A_q8, const void *B, const float *bias, float *C, int M, int N, int K)
{
    if (!A_q8 || !B || !C || M <= 0 || N <= 0 || K <= 0) return;
    const orc_q5_0 *w = (const orc_q5_0 *)B;
    const orc_q8_0_blk *a = (const orc_q8_0_blk *)A_q8;
    for (int m = 0; m < M; ++m)
        for (int n = 0; n < N; ++n) {
            float *out = &C[(size_t)m * N + n];
            oracle_vec_dot_q5_0_q8_0(K, out, w + (size_t)n * (K / 32), a + (size_t)m * (K / 32));
            if (bias) *out += bias[n];
        }
}

/* ---- prefill attention (src/kernels/attention_kernels.c:2847-3005; per-query online softmax :1546-1602) ----
 * q, out [H][T][ad]; k, v [Hkv][kv_stride_tokens][ad]; query token i of head h sees keys 0 .. i (causal) or all T of
 * kv head h * Hkv / H; key by key: a new maximum rescales the running sum and output, otherwise exp(score - max). */
static void orc_flash_query(const float *q, const float *k, const float *v, int kv_tokens, int hd, int ad, float scale, float *out)
{
    float m = -INFINITY, s = 0.0f;
    for (int d = 0; d < hd; ++d) out[d] = 0.0f;
    for (int j = 0; j < kv_tokens; ++j) {
        const float *kr = k + (size_t)j * ad, *vr = v + (size_t)j * ad;
        float dot = 0.0f;
        for (int d = 0; d < hd; ++d) dot += q[d] * kr[d];
        const float score = dot * scale;
        if (score > m) {
            const float f = m == -INFINITY ? 0.0f : expf(m - score);
            s *= f;
            for (int d = 0; d < hd; ++d) out[d] *= f;
            s += 1.0f;
            for (int d = 0; d < hd; ++d) out[d] += vr[d];
            m = score;
        } else {
            const float e = expf(score - m);
            s += e;
            for (int d = 0; d < hd; ++d) out[d] += e * vr[d];
        }
    }
    const float inv = 1.0f / s;
    for (int d = 0; d < hd; ++d) out[d] *= inv;
    for (int d = hd; d < ad; ++d) out[d] = 0.0f;
}

static void orc_attention_prefill(const float *q, const float *k, const float *v, float *output, int num_heads, int num_kv_heads, int num_tokens,
                                  int head_dim, int aligned_head_dim, int kv_stride_tokens, int causal, int window)
{
    if (!q || !k || !v || !output) return;
    if (num_heads <= 0 || num_kv_heads <= 0 || num_tokens <= 0 || kv_stride_tokens < num_tokens) return;
    const float scale = 1.0f / sqrtf((float)head_dim);
    const size_t hs = (size_t)kv_stride_tokens * (size_t)aligned_head_dim;
    for (int h = 0; h < num_heads; ++h) {
        const int kvh = (int)((long long)h * num_kv_heads / num_heads);
        for (int i = 0; i < num_tokens; ++i) {
            const size_t row = ((size_t)h * num_tokens + i) * aligned_head_dim;
            /* sliding window (src/kernels/attention_kernels_sliding.c:391-402): keys max(0, i - window + 1) .. i */
            const int start = causal && window > 0 && i - window + 1 > 0 ? i - window + 1 : 0;
            const size_t skip = (size_t)start * aligned_head_dim;
            orc_flash_query(q + row, k + kvh * hs + skip, v + kvh * hs + skip, (causal ? i + 1 : num_tokens) - start, head_dim, aligned_head_dim, scale,
                            output + row);
        }
    }
}

void oracle_attention_forward_causal_head_major_gqa_flash_strided(const float *q, const float *k, const float *v, float *output, int num_heads,
                                                                  int num_kv_heads, int num_tokens, int head_dim, int aligned_head_dim,
                                                                  int kv_stride_tokens)
{
    orc_attention_prefill(q, k, v, output, num_heads, num_kv_heads, num_tokens, head_dim, aligned_head_dim, kv_stride_tokens, 1, 0);
}

void oracle_attention_forward_full_head_major_gqa_flash_strided(const float *q, const float *k, const float *v, float *output, int num_heads,
                                                                int num_kv_heads, int num_tokens, int head_dim, int aligned_head_dim,
                                                                int kv_stride_tokens)
{
    orc_attention_prefill(q, k, v, output, num_heads, num_kv_heads, num_tokens, head_dim, aligned_head_dim, kv_stride_tokens, 0, 0);
}

void oracle_attention_forward_causal_head_major_gqa_flash_strided_sliding(const float *q, const float *k, const float *v, float *output, int num_heads,
                                                                          int num_kv_heads, int num_tokens, int head_dim, int aligned_head_dim,
                                                                          int kv_stride_tokens, int sliding_window)
{
    orc_attention_prefill(q, k, v, output, num_heads, num_kv_heads, num_tokens, head_dim, aligned_head_dim, kv_stride_tokens, 1, sliding_window);
}

/* decode with a window (src/kernels/attention_kernels_sliding.c:528-600): the last min(kv_tokens, window) rows of every kv head */
void oracle_attention_forward_decode_head_major_gqa_flash_sliding(const float *q_token, const float *k_cache, const float *v_cache, float *out_token,
                                                                  int num_heads, int num_kv_heads, int kv_tokens, int cache_capacity, int head_dim,
                                                                  int aligned_head_dim, int sliding_window)
{
    if (!q_token || !k_cache || !v_cache || !out_token) return;
    if (num_heads <= 0 || num_kv_heads <= 0 || cache_capacity <= 0) return;
    if (kv_tokens <= 0 || kv_tokens > cache_capacity || head_dim <= 0 || aligned_head_dim <= 0) return;
    const int eff = sliding_window > 0 && sliding_window < kv_tokens ? sliding_window : kv_tokens;
    const size_t hs = (size_t)cache_capacity * aligned_head_dim, skip = (size_t)(kv_tokens - eff) * aligned_head_dim;
    const float scale = 1.0f / sqrtf((float)head_dim);
    for (int h = 0; h < num_heads; ++h) {
        const int kvh = (int)((long long)h * num_kv_heads / num_heads);
        orc_flash_query(q_token + (size_t)h * aligned_head_dim, k_cache + kvh * hs + skip, v_cache + kvh * hs + skip, eff, head_dim, aligned_head_dim,
                        scale, out_token + (size_t)h * aligned_head_dim);
    }
}

/* ---- "Llama-parity" attention (src/kernels/attention_kernels.c:1673-1744): q, k and v pass through fp16 before use and the
 * output accumulator is rounded to fp16 after every update, key by key, with the online max / sum recurrence.  The result depends
 * on the order of the keys, so a device kernel has to walk them in the same order. ---- */
static float orc_r16(float x) { return oracle_fp16_to_fp32(oracle_fp32_to_fp16(x)); }

static void orc_flash_query_f16kv(const float *q, const float *kh, const float *vh, int kv_tokens, int hd, int ad, float scale, float *out)
{
    for (int d = 0; d < ad; ++d) out[d] = 0.0f;
    if (kv_tokens <= 0) return;
    float sum = 0.0f, mx = -INFINITY;
    for (int j = 0; j < kv_tokens; ++j) {
        const float *k = kh + (size_t)j * ad, *v = vh + (size_t)j * ad;
        float dot = 0.0f;
        for (int d = 0; d < hd; ++d) dot += orc_r16(q[d]) * orc_r16(k[d]);
        const float score = dot * scale, prev = mx;
        float max_scale = 1.0f, value_scale = 1.0f;
        if (score > mx) {
            mx = score;
            max_scale = isfinite(prev) ? expf(prev - mx) : 0.0f;
            for (int d = 0; d < hd; ++d) out[d] = orc_r16(out[d] * max_scale);
        } else {
            value_scale = expf(score - mx);
        }
        for (int d = 0; d < hd; ++d) out[d] = orc_r16(out[d] + value_scale * orc_r16(v[d]));
        sum = sum * max_scale + value_scale;
    }
    if (sum > 0.0f) {
        const float inv = 1.0f / sum;
        for (int d = 0; d < hd; ++d) out[d] *= inv;
    } else {
        for (int d = 0; d < hd; ++d) out[d] = 0.0f;
    }
}

/* src/kernels/attention_kernels.c:3408-3448 */
void oracle_attention_forward_decode_head_major_gqa_flash_f16kv(const float *q_token, const float *k_cache, const float *v_cache, float *out_token,
                                                                int num_heads, int num_kv_heads, int kv_tokens, int cache_capacity, int head_dim,
                                                                int aligned_head_dim)
{
    if (!q_token || !k_cache || !v_cache || !out_token) return;
    if (num_heads <= 0 || num_kv_heads <= 0 || kv_tokens <= 0 || cache_capacity <= 0) return;
    if (kv_tokens > cache_capacity || head_dim <= 0 || aligned_head_dim <= 0) return;
    const float scale = 1.0f / sqrtf((float)head_dim);
    const size_t hs = (size_t)cache_capacity * aligned_head_dim;
    for (int h = 0; h < num_heads; ++h) {
        const int kvh = (int)((long long)h * num_kv_heads / num_heads);
        orc_flash_query_f16kv(q_token + (size_t)h * aligned_head_dim, k_cache + kvh * hs, v_cache + kvh * hs, kv_tokens, head_dim, aligned_head_dim, scale,
                              out_token + (size_t)h * aligned_head_dim);
    }
}

/* src/kernels/attention_kernels.c:3006-3046: query i of a prompt sees keys 0..i */
void oracle_attention_forward_causal_head_major_gqa_flash_strided_f16kv(const float *q, const float *k, const float *v, float *output, int num_heads,
                                                                        int num_kv_heads, int num_tokens, int head_dim, int aligned_head_dim,
                                                                        int kv_stride_tokens)
{
    if (!q || !k || !v || !output) return;
    if (num_heads <= 0 || num_kv_heads <= 0 || num_tokens <= 0 || kv_stride_tokens < num_tokens) return;
    const float scale = 1.0f / sqrtf((float)head_dim);
    const size_t hs = (size_t)kv_stride_tokens * aligned_head_dim;
    for (int h = 0; h < num_heads; ++h) {
        const int kvh = (int)((long long)h * num_kv_heads / num_heads);
        for (int i = 0; i < num_tokens; ++i) {
            const size_t row = ((size_t)h * num_tokens + i) * aligned_head_dim;
            orc_flash_query_f16kv(q + row, k + kvh * hs, v + kvh * hs, i + 1, head_dim, aligned_head_dim, scale, output + row);
        }
    }
}

/* ---- KV cache store (src/kernels/kv_cache_kernels.c:70-129) ---- */
void oracle_kv_cache_store(float *kc, float *vc, const float *k, const float *v, int layer, int pos,
                           int num_kv_heads, int head_dim, int max_seq_len)
{
    (void)layer;
    if (!k || !v || !kc || !vc || num_kv_heads <= 0 || pos < 0 || pos >= max_seq_len || head_dim <= 0) return;
    for (int h = 0; h < num_kv_heads; ++h) {
        const size_t dst = ((size_t)h * max_seq_len + pos) * head_dim;
        memcpy(kc + dst, k + (size_t)h * head_dim, sizeof(float) * head_dim);
        memcpy(vc + dst, v + (size_t)h * head_dim, sizeof(float) * head_dim);
    }
}

/* ---- fp16 KV cache (src/kernels/kv_cache_kernels.c:131-163 store; src/kernels/attention_kernels.c:3450-3557 decode:
 * every kv head's rows are widened to fp32 and attended exactly like the fp32 cache) ---- */
void oracle_kv_cache_store_f16(uint16_t *kc, uint16_t *vc, const float *k, const float *v, int layer, int pos,
                               int num_kv_heads, int head_dim, int max_seq_len)
{
    (void)layer;
    if (!k || !v || !kc || !vc || num_kv_heads <= 0 || pos < 0 || pos >= max_seq_len || head_dim <= 0) return;
    for (int h = 0; h < num_kv_heads; ++h) {
        const size_t dst = ((size_t)h * max_seq_len + pos) * head_dim;
        for (int d = 0; d < head_dim; ++d) {
            kc[dst + d] = oracle_fp32_to_fp16(k[(size_t)h * head_dim + d]);
            vc[dst + d] = oracle_fp32_to_fp16(v[(size_t)h * head_dim + d]);
        }
    }
}

void oracle_attention_forward_decode_head_major_gqa_flash_f16cache(const float *q_token, const uint16_t *k_cache, const uint16_t *v_cache,
                                                                   float *out_token, int num_heads, int num_kv_heads, int kv_tokens,
                                                                   int cache_capacity, int head_dim, int aligned_head_dim)
{
    if (!q_token || !k_cache || !v_cache || !out_token) return;
    if (num_heads <= 0 || num_kv_heads <= 0 || kv_tokens <= 0 || cache_capacity <= 0) return;
    if (kv_tokens > cache_capacity || head_dim <= 0 || aligned_head_dim <= 0) return;
    const float scale = 1.0f / sqrtf((float)head_dim);
    const size_t hs = (size_t)cache_capacity * (size_t)aligned_head_dim, n = (size_t)kv_tokens * aligned_head_dim;
    float *kf = (float *)malloc(n * sizeof(float)), *vf = (float *)malloc(n * sizeof(float));
    if (!kf || !vf) { free(kf); free(vf); return; }
    for (int kvh = 0; kvh < num_kv_heads; ++kvh) {
        for (size_t i = 0; i < n; ++i) {
            kf[i] = oracle_fp16_to_fp32(k_cache[kvh * hs + i]);
            vf[i] = oracle_fp16_to_fp32(v_cache[kvh * hs + i]);
        }
        const int h0 = (int)((long long)kvh * num_heads / num_kv_heads), h1 = (int)((long long)(kvh + 1) * num_heads / num_kv_heads);
        for (int h = h0; h < h1; ++h)
            orc_flash_decode_head(out_token + (size_t)h * aligned_head_dim, q_token + (size_t)h * aligned_head_dim, kf, vf, kv_tokens,
                                  aligned_head_dim, scale);
    }
    free(kf);
    free(vf);
}

/* ---- RoPE (src/kernels/rope_kernels.c:221-243 cache, :320-417 rotate-half, :806-819 q+k) ---- */
void oracle_rope_precompute_cache_split(float *cos_cache, float *sin_cache, int max_seq_len, int head_dim, float base)
{
    const int half = head_dim / 2;
    const long double lb = logl((long double)base);
    for (int p = 0; p < max_seq_len; ++p)
        for (int i = 0; i < half; ++i) {
            const float freq = (float)expl(-((long double)(2 * i) / (long double)head_dim) * lb);
            const float ang = (float)p * freq;
            cos_cache[(size_t)p * half + i] = cosf(ang);
            sin_cache[(size_t)p * half + i] = sinf(ang);
        }
}

static void orc_rope_heads(float *x, const float *cc, const float *ss, int heads, int tokens, int hd, int ahd, int pos0)
{
    const int half = hd / 2;
    for (int h = 0; h < heads; ++h)
        for (int t = 0; t < tokens; ++t) {
            float *r = x + ((size_t)h * tokens + t) * ahd;
            const float *c = cc + (size_t)(pos0 + t) * half, *s = ss + (size_t)(pos0 + t) * half;
            for (int i = 0; i < half; ++i) {
                const float a = r[i], b = r[i + half];
                r[i] = a * c[i] - b * s[i];
                r[i + half] = a * s[i] + b * c[i];
            }
        }
}

void oracle_rope_forward_qk(float *q, float *k, const float *cos_cache, const float *sin_cache, int num_heads,
                            int num_kv_heads, int num_tokens, int head_dim, int aligned_head_dim, int pos_offset)
{
    orc_rope_heads(q, cos_cache, sin_cache, num_heads, num_tokens, head_dim, aligned_head_dim, pos_offset);
    orc_rope_heads(k, cos_cache, sin_cache, num_kv_heads, num_tokens, head_dim, aligned_head_dim, pos_offset);
}

/* rope_forward_qk_with_rotary_dim (src/kernels/rope_kernels.c:320-417, :821-837): pairs (i, i + rotary_dim / 2), rows of rotary_dim / 2 */
void oracle_rope_forward_qk_with_rotary_dim(float *q, float *k, const float *cos_cache, const float *sin_cache, int num_heads, int num_kv_heads,
                                            int num_tokens, int head_dim, int aligned_head_dim, int pos_offset, int rotary_dim)
{
    if (rotary_dim <= 0 || rotary_dim > head_dim) rotary_dim = head_dim;
    orc_rope_heads(q, cos_cache, sin_cache, num_heads, num_tokens, rotary_dim, aligned_head_dim, pos_offset);
    orc_rope_heads(k, cos_cache, sin_cache, num_kv_heads, num_tokens, rotary_dim, aligned_head_dim, pos_offset);
}

/* ---- RMSNorm (src/kernels/rmsnorm_kernels.c:38-71 scalar form; :245-248 zero pad) ---- */
void oracle_rmsnorm_forward(const float *in, const float *gamma, float *out, float *rstd_cache, int tokens,
                            int d_model, int aligned, float eps)
{
    for (int t = 0; t < tokens; ++t) {
        const float *x = in + (size_t)t * aligned;
        float *y = out + (size_t)t * aligned;
        float ss = 0.0f;
        for (int i = 0; i < d_model; ++i) ss += x[i] * x[i];
        const float rstd = 1.0f / sqrtf(ss * (1.0f / (float)d_model) + eps);
        if (rstd_cache) rstd_cache[t] = rstd;
        for (int i = 0; i < d_model; ++i) y[i] = x[i] * rstd * gamma[i];
        for (int i = d_model; i < aligned; ++i) y[i] = 0.0f;
    }
}

/* ---- SwiGLU (src/kernels/swiglu_kernels.c:358-379 exact form; sigmoid_kernels.c:26-29) ---- */
void oracle_swiglu_forward(const float *in, float *out, int tokens, int dim)
{
    for (int t = 0; t < tokens; ++t)
        for (int i = 0; i < dim; ++i) {
            const float g = in[(size_t)t * 2 * dim + i], u = in[(size_t)t * 2 * dim + dim + i];
            const float sg = 1.0f / (1.0f + expf(-g));
            out[(size_t)t * dim + i] = g * sg * u;
        }
}

/* ---- residual add (src/ckernel_orchestration.c:139-149) ---- */
void oracle_residual_add_token_major(const float *a, const float *b, float *out, int tokens, int aligned)
{
    const size_t n = (size_t)tokens * aligned;
    for (size_t i = 0; i < n; ++i) out[i] = a[i] + b[i];
}

void oracle_ck_residual_add_token_major(const float *a, const float *b, float *out, int tokens, int aligned)      /* the reference's symbol */
{
    oracle_residual_add_token_major(a, b, out, tokens, aligned);
}

/* ---- embedding lookup (src/kernels/embedding_kernels.c:76-129 q4_k, :131-184 q8_0, :186-239 q6_k) ---- */
static void orc_embed(const int32_t *ids, int count, int vocab, const void *table, const float *pos, float *out,
                      int embed, int aligned, int ctx, int add_pos, size_t row_bytes,
                      void (*deq)(const void *, float *, size_t))
{
    if (!ids || !table || !out) return;
    int n = count < 0 ? 0 : (count > ctx ? ctx : count);
    for (int t = 0; t < n; ++t) {
        int id = ids[t];
        if (id < 0 || id >= vocab) id = 0;
        float *o = out + (size_t)t * aligned;
        deq((const uint8_t *)table + (size_t)id * row_bytes, o, (size_t)aligned);
        if (add_pos && pos) for (int i = 0; i < embed; ++i) o[i] += pos[(size_t)t * aligned + i];
        for (int i = embed; i < aligned; ++i) o[i] = 0.0f;
    }
    for (int t = n; t < ctx; ++t) memset(out + (size_t)t * aligned, 0, sizeof(float) * aligned);
}

void oracle_embedding_forward_q4_k(const int32_t *ids, int count, int vocab, const void *table, const float *pos,
                                   float *out, int embed, int aligned, int ctx, int add_pos)
{
    orc_embed(ids, count, vocab, table, pos, out, embed, aligned, ctx, add_pos, (size_t)(aligned / 256) * 144,
              oracle_dequant_q4_k_row);
}
void oracle_embedding_forward_q6_k(const int32_t *ids, int count, int vocab, const void *table, const float *pos,
                                   float *out, int embed, int aligned, int ctx, int add_pos)
{
    orc_embed(ids, count, vocab, table, pos, out, embed, aligned, ctx, add_pos, (size_t)(aligned / 256) * 210,
              oracle_dequant_q6_k_row);
}
void oracle_embedding_forward_q8_0(const int32_t *ids, int count, int vocab, const void *table, const float *pos,
                                   float *out, int embed, int aligned, int ctx, int add_pos)
{
    orc_embed(ids, count, vocab, table, pos, out, embed, aligned, ctx, add_pos, (size_t)(aligned / 32) * 34,
              oracle_dequant_q8_0_row);
}

/* ---- fp32-activation products of the reference's debug path ----
 * gemv_q4_k_ref: src/kernels/gemm_kernels_q4k.c:53-101 (per element (d*sc*q - dmin*m) * x, in element order);
 * gemv_q6_k -> dot_q6_k_ref: src/kernels/gemm_kernels_q6k.c:80-118, :169-193 (l-major over the four strided streams). */
void oracle_gemv_q4_k(float *y, const void *W, const float *x, int M, int K)
{
    if (!y || !W || !x || M <= 0 || K <= 0) return;
    const orc_q4_K *w = (const orc_q4_K *)W;
    const int nb = K / ORC_QK_K;
    for (int r = 0; r < M; ++r) {
        float sum = 0.0f;
        for (int b = 0; b < nb; ++b) {
            const orc_q4_K *blk = &w[(size_t)r * nb + b];
            const float d = oracle_fp16_to_fp32(blk->d), dmin = oracle_fp16_to_fp32(blk->dmin);
            uint8_t sc[8], mn[8];
            oracle_unpack_q4_k_scales(blk->scales, sc, mn);
            for (int g = 0; g < 4; ++g) {
                const float d1 = d * (float)sc[2 * g], m1 = dmin * (float)mn[2 * g];
                const float d2 = d * (float)sc[2 * g + 1], m2 = dmin * (float)mn[2 * g + 1];
                const uint8_t *qs = blk->qs + 32 * g;
                const float *xp = x + (size_t)b * ORC_QK_K + 64 * g;
                for (int l = 0; l < 32; ++l) sum += (d1 * (float)(qs[l] & 15) - m1) * xp[l];
                for (int l = 0; l < 32; ++l) sum += (d2 * (float)(qs[l] >> 4) - m2) * xp[l + 32];
            }
        }
        y[r] = sum;
    }
}

void oracle_gemv_q6_k(float *y, const void *W, const float *x, int M, int K)
{
    if (!y || !W || !x || M <= 0 || K <= 0) return;
    const orc_q6_K *w = (const orc_q6_K *)W;
    const int nb = K / ORC_QK_K;
    for (int r = 0; r < M; ++r) {
        float sum = 0.0f;
        for (int b = 0; b < nb; ++b) {
            const orc_q6_K *blk = &w[(size_t)r * nb + b];
            const float d = oracle_fp16_to_fp32(blk->d);
            for (int half = 0; half < 2; ++half)
                for (int l = 0; l < 32; ++l)
                    for (int qt = 0; qt < 4; ++qt) {
                        const int e = 128 * half + 32 * qt + l;
                        sum += d * (float)blk->scales[8 * half + (l >> 4) + 2 * qt] * (float)orc_q6_value(blk, e) * x[(size_t)b * ORC_QK_K + e];
                    }
        }
        y[r] = sum;
    }
}

/* gemm_nt_<fmt>(A fp32 [M][K], B [N][K], bias, C [M][N]): one fp32-activation GEMV per token, then the bias
 * (src/kernels/gemm_kernels_q4k.c:683-711, src/kernels/gemm_kernels_q6k.c:212-238, src/kernels/gemm_kernels_q8_0.c:683-696);
 * gemm_<fmt>(Y [N][M], W [M][K], X [N][K]) is the same loop (gemm_kernels_q4k.c:316-326, gemm_kernels_q6k.c:195-210,
 * gemm_kernels_q8_0.c:658-666). */
typedef void (*orc_gemv_f32_fn)(float *, const void *, const float *, int, int);
static void orc_gemm_nt_f32(orc_gemv_f32_fn gemv, const float *A, const void *B, const float *bias, float *C, int M, int N, int K)
{
    if (!A || !B || !C || M <= 0 || N <= 0 || K <= 0) return;
    for (int m = 0; m < M; ++m) {
        gemv(C + (size_t)m * N, B, A + (size_t)m * K, N, K);
        if (bias) for (int n = 0; n < N; ++n) C[(size_t)m * N + n] += bias[n];
    }
}
void oracle_gemm_nt_q4_k(const float *A, const void *B, const float *bias, float *C, int M, int N, int K) { orc_gemm_nt_f32(oracle_gemv_q4_k, A, B, bias, C, M, N, K); }
void oracle_gemm_nt_q6_k(const float *A, const void *B, const float *bias, float *C, int M, int N, int K) { orc_gemm_nt_f32(oracle_gemv_q6_k, A, B, bias, C, M, N, K); }
void oracle_gemm_nt_q8_0(const float *A, const void *B, const float *bias, float *C, int M, int N, int K) { orc_gemm_nt_f32(oracle_gemv_q8_0, A, B, bias, C, M, N, K); }
void oracle_gemm_q4_k(float *Y, const void *W, const float *X, int M, int N, int K) { orc_gemm_nt_f32(oracle_gemv_q4_k, X, W, NULL, Y, N, M, K); }
void oracle_gemm_q6_k(float *Y, const void *W, const float *X, int M, int N, int K) { orc_gemm_nt_f32(oracle_gemv_q6_k, X, W, NULL, Y, N, M, K); }
void oracle_gemm_q8_0(float *Y, const void *W, const float *X, int M, int N, int K) { orc_gemm_nt_f32(oracle_gemv_q8_0, X, W, NULL, Y, N, M, K); }

/* gemm_nt_q6_k_sse (src/kernels/gemm_kernels_q6k_sse.c:66-97): A rows quantised to Q8_K, then Q6_K x Q8_K dots */
void oracle_gemm_nt_q6_k_sse(const float *A, const void *B, const float *bias, float *C, int M, int N, int K)
{
    if (!A || !B || !C || M <= 0 || N <= 0 || K <= 0 || K % ORC_QK_K) return;
    orc_q8_K *aq = (orc_q8_K *)malloc((size_t)M * (K / ORC_QK_K) * sizeof(orc_q8_K));
    if (!aq) return;
    oracle_quantize_batch_q8_k(A, aq, M, K);
    oracle_gemm_nt_q6_k_q8_k(aq, B, bias, C, M, N, K);
    free(aq);
}

/* gemv_q8_0_q8_0_contract / gemm_nt_q8_0_q8_0_contract (src/kernels/gemm_kernels_q8_0_q8_0_contract.c:377-406, :408-486, the
 * non-strict path): x quantised to Q8_0 when a row has at most 1024 blocks, else the fp32-activation GEMV */
void oracle_gemv_q8_0_q8_0_contract(float *y, const void *W, const float *x, int M, int K)
{
    if (!y || !W || !x || M <= 0 || K <= 0) return;
    if (K % ORC_QK8_0 || K / ORC_QK8_0 > 1024) { oracle_gemv_q8_0(y, W, x, M, K); return; }
    orc_q8_0 xq[1024];
    oracle_quantize_row_q8_0(x, xq, K);
    oracle_gemv_q8_0_q8_0(y, W, xq, M, K);
}
void oracle_gemm_nt_q8_0_q8_0_contract(const float *A, const void *B, const float *bias, float *C, int M, int N, int K)
{
    orc_gemm_nt_f32(oracle_gemv_q8_0_q8_0_contract, A, B, bias, C, M, N, K);
}

/* ---- RoPE, general table and pairwise rotation (src/kernels/rope_kernels.c:270-316, :419-451, :839-866) ---- */
void oracle_rope_precompute_cache(float *cos_cache, float *sin_cache, int max_seq_len, int head_dim, float base, int rotary_dim,
                                  const char *scaling_type, float scaling_factor)
{
    if (rotary_dim <= 0 || rotary_dim > head_dim) rotary_dim = head_dim;
    const int linear = scaling_type && !strcmp(scaling_type, "linear") && scaling_factor > 0.0f && scaling_factor != 1.0f;
    const int half = rotary_dim / 2;
    const long double lb = logl((long double)base);
    for (int p = 0; p < max_seq_len; ++p) {
        const float epos = linear ? (float)p / scaling_factor : (float)p;
        for (int i = 0; i < half; ++i) {
            const float freq = (float)expl(-((long double)(2 * i) / (long double)rotary_dim) * lb);
            const float ang = epos * freq;
            cos_cache[(size_t)p * half + i] = cosf(ang);
            sin_cache[(size_t)p * half + i] = sinf(ang);
        }
    }
}

static void orc_rope_heads_pairwise(float *x, const float *cc, const float *ss, int heads, int tokens, int rot, int ahd, int pos0)
{
    const int half = rot / 2;
    for (int h = 0; h < heads; ++h)
        for (int t = 0; t < tokens; ++t) {
            float *r = x + ((size_t)h * tokens + t) * ahd;
            const float *c = cc + (size_t)(pos0 + t) * half, *s = ss + (size_t)(pos0 + t) * half;
            for (int i = 0; i < half; ++i) {
                const float a = r[2 * i], b = r[2 * i + 1];
                r[2 * i] = a * c[i] - b * s[i];
                r[2 * i + 1] = a * s[i] + b * c[i];
            }
        }
}

void oracle_rope_forward_qk_pairwise_with_rotary_dim(float *q, float *k, const float *cos_cache, const float *sin_cache, int num_heads,
                                                     int num_kv_heads, int num_tokens, int head_dim, int aligned_head_dim, int pos_offset,
                                                     int rotary_dim)
{
    if (rotary_dim <= 0 || rotary_dim > head_dim) rotary_dim = head_dim;
    orc_rope_heads_pairwise(q, cos_cache, sin_cache, num_heads, num_tokens, rotary_dim, aligned_head_dim, pos_offset);
    orc_rope_heads_pairwise(k, cos_cache, sin_cache, num_kv_heads, num_tokens, rotary_dim, aligned_head_dim, pos_offset);
}

/* ---- add_inplace_f32 (src/kernels/add_kernels_bf16.c:304-335), logits_copy_to_position (src/kernels/kv_cache_kernels.c:178-191) ---- */
void oracle_add_inplace_f32(float *a, const float *b, size_t n)
{
    if (!a || !b) return;
    for (size_t i = 0; i < n; ++i) a[i] = a[i] + b[i];
}
void oracle_logits_copy_to_position(const float *src, float *dst, int position, int vocab_size)
{
    if (!src || !dst || position < 0 || vocab_size <= 0) return;
    memmove(dst + (size_t)position * (size_t)vocab_size, src, (size_t)vocab_size * sizeof(float));
}

/* =====================================================================================================================
 * Further weight formats of the reference: Q5_K, and the 32-element formats Q4_0, Q4_1, Q5_1 (with Q8_1 activations).
 * Block layouts: Q5_K 176 B = fp16 d, fp16 dmin, scales[12], qh[32], qs[128] (src/kernels/gemm_kernels_q5_k.c:49-55);
 * Q4_0 18 B = fp16 d, qs[16]; Q4_1 20 B = fp16 d, fp16 m, qs[16]; Q5_1 24 B = fp16 d, fp16 m, qh[4], qs[16]
 * (include/ckernel_quant.h:33-92); Q8_1 36 B = fp16 d, fp16 s = d * sum(q), qs[32] (src/kernels/gemm_kernels_q5_1_q8_1.c:21-25).
 * ===================================================================================================================== */

static float orc_h(const uint8_t *p) { return oracle_fp16_to_fp32((uint16_t)(p[0] | (p[1] << 8))); }

/* the 6-bit scale / min pairs of Q4_K and Q5_K (src/kernels/gemm_kernels_q5_k.c:59-81) */
static void orc_k_scales(const uint8_t *s, uint8_t sc[8], uint8_t mn[8])
{
    for (int j = 0; j < 4; ++j) {
        sc[j] = s[j] & 63;
        mn[j] = s[j + 4] & 63;
        sc[j + 4] = (uint8_t)((s[j + 8] & 15) | ((s[j] >> 6) << 4));
        mn[j + 4] = (uint8_t)((s[j + 8] >> 4) | ((s[j + 4] >> 6) << 4));
    }
}

/* one 256-element block, Q5_K x Q8_K (src/kernels/gemm_kernels_q5_k.c:128-208): groups of 64 elements share 32 nibble bytes (low
 * nibbles first), bit 2j / 2j + 1 of qh[l] is the fifth bit; integer sums, then d * dot - dmin * sum(mins * bsums) */
static float orc_dot_q5_k_q8_k_block(const uint8_t *w, const uint8_t *x)
{
    uint8_t sc[8], mn[8];
    orc_k_scales(w + 4, sc, mn);
    const uint8_t *qh = w + 16, *qs = w + 48;
    const int8_t *q8 = (const int8_t *)(x + 4);
    const int16_t *bsums = (const int16_t *)(x + 260);
    float xd;
    memcpy(&xd, x, 4);
    int sumi = 0, doti = 0;
    for (int j = 0; j < 16; ++j) sumi += (int)bsums[j] * (int)mn[j / 2];
    for (int sb = 0; sb < 8; ++sb) {
        int s = 0;
        for (int l = 0; l < 32; ++l) {
            const uint8_t byte = qs[32 * (sb >> 1) + l];
            const int a = ((sb & 1) ? (byte >> 4) : (byte & 15)) + (((qh[l] >> sb) & 1) ? 16 : 0);
            s += a * (int)q8[32 * sb + l];
        }
        doti += (int)sc[sb] * s;
    }
    const float d = orc_h(w) * xd, dmin = orc_h(w + 2) * xd;
    return d * (float)doti - dmin * (float)sumi;
}

void oracle_gemv_q5_k_q8_k(float *y, const void *W, const void *x_q8, int M, int K)
{
    if (!y || !W || !x_q8 || M <= 0 || K <= 0 || K % 256) return;
    const int nb = K / 256;
    for (int m = 0; m < M; ++m) {
        float sum = 0.0f;
        for (int b = 0; b < nb; ++b) sum += orc_dot_q5_k_q8_k_block((const uint8_t *)W + ((size_t)m * nb + b) * 176, (const uint8_t *)x_q8 + (size_t)b * 292);
        y[m] = sum;
    }
}

void oracle_gemm_nt_q5_k_q8_k(const void *A_q8, const void *B, const float *bias, float *C, int M, int N, int K)
{
    if (!A_q8 || !B || !C || M <= 0 || N <= 0 || K <= 0 || K % 256) return;
    const int nb = K / 256;
    for (int m = 0; m < M; ++m)
        for (int n = 0; n < N; ++n) {
            float sum = 0.0f;
            for (int b = 0; b < nb; ++b)
                sum += orc_dot_q5_k_q8_k_block((const uint8_t *)B + ((size_t)n * nb + b) * 176, (const uint8_t *)A_q8 + ((size_t)m * nb + b) * 292);
            C[(size_t)m * N + n] = sum + (bias ? bias[n] : 0.0f);
        }
}

/* the fp32 fall-back of gemv_q5_k / gemm_nt_q5_k (src/kernels/gemm_kernels_q5_k.c:211-283) reads the block differently: sub-block sb
 * takes nibble i % 2 of qs[16 sb + i / 2] and bit i % 8 of qh[4 sb + i / 8] */
static float orc_q5_k_elem_fp32_layout(const uint8_t *w, int e)
{
    uint8_t sc[8], mn[8];
    orc_k_scales(w + 4, sc, mn);
    const int sb = e >> 5, i = e & 31;
    const uint8_t q = (uint8_t)(((w[48 + sb * 16 + i / 2] >> (4 * (i % 2))) & 15) | (((w[16 + sb * 4 + i / 8] >> (i % 8)) & 1) << 4));
    return orc_h(w) * (float)sc[sb] * (float)q - orc_h(w + 2) * (float)mn[sb];
}

static void orc_gemm_nt_q5_k_fp32(const float *A, const void *B, const float *bias, float *C, int M, int N, int K)
{
    const int nb = K / 256;            /* whole blocks only; rows of A are K floats apart */
    for (int m = 0; m < M; ++m)
        for (int n = 0; n < N; ++n) {
            float sum = 0.0f;
            for (int b = 0; b < nb; ++b)
                for (int e = 0; e < 256; ++e) sum += orc_q5_k_elem_fp32_layout((const uint8_t *)B + ((size_t)n * nb + b) * 176, e) * A[(size_t)m * K + b * 256 + e];
            C[(size_t)m * N + n] = sum + (bias ? bias[n] : 0.0f);
        }
}

/* gemm_nt_q5_k / gemv_q5_k (src/kernels/gemm_kernels_q5_k.c:369-434): fp32 activations are quantised to Q8_K per row (rows of up to 128
 * blocks), longer rows take the fp32 fall-back */
void oracle_gemm_nt_q5_k(const float *A, const void *B, const float *bias, float *C, int M, int N, int K)
{
    if (!A || !B || !C || M <= 0 || N <= 0 || K <= 0) return;
    if (K % 256 || K / 256 > 128) { orc_gemm_nt_q5_k_fp32(A, B, bias, C, M, N, K); return; }
    uint8_t *q = (uint8_t *)malloc((size_t)(K / 256) * 292);
    for (int m = 0; m < M; ++m) {
        oracle_quantize_row_q8_k(A + (size_t)m * K, q, K);
        oracle_gemm_nt_q5_k_q8_k(q, B, bias, C + (size_t)m * N, 1, N, K);
    }
    free(q);
}

void oracle_gemv_q5_k(float *y, const void *W, const float *x, int M, int K) { oracle_gemm_nt_q5_k(x, W, NULL, y, 1, M, K); }

/* ---- Q8_1 activations and Q5_1 x Q8_1 (src/kernels/gemm_kernels_q5_1_q8_1.c:27-122) ---- */
void oracle_quantize_row_q8_1(const float *x, void *vy, int k)
{
    uint8_t *y = (uint8_t *)vy;
    for (int b = 0; b < k / 32; ++b) {
        const float *xb = x + (size_t)b * 32;
        float amax = 0.0f;
        for (int j = 0; j < 32; ++j) { const float av = xb[j] >= 0.0f ? xb[j] : -xb[j]; if (av > amax) amax = av; }
        const float d = amax / 127.0f, id = d != 0.0f ? 1.0f / d : 0.0f;
        const uint16_t dh = oracle_fp32_to_fp16(d);
        int sum = 0;
        for (int j = 0; j < 32; ++j) { const int q = (int)roundf(xb[j] * id); ((int8_t *)(y + 4))[j] = (int8_t)q; sum += q; }
        const uint16_t sh = oracle_fp32_to_fp16((float)sum * d);
        y[0] = (uint8_t)dh; y[1] = (uint8_t)(dh >> 8); y[2] = (uint8_t)sh; y[3] = (uint8_t)(sh >> 8);
        y += 36;
    }
}

static float orc_dot_q5_1_q8_1_block(const uint8_t *w, const uint8_t *x)
{
    uint32_t qh;
    memcpy(&qh, w + 4, 4);
    const uint8_t *qs = w + 8;
    const int8_t *q8 = (const int8_t *)(x + 4);
    int s0 = 0, s1 = 0;
    for (int j = 0; j < 16; ++j) {
        const int q0 = (qs[j] & 15) | (int)(((qh >> j) << 4) & 0x10), q1 = (qs[j] >> 4) | (int)((qh >> (j + 12)) & 0x10);
        s0 += q0 * (int)q8[j];
        s1 += q1 * (int)q8[j + 16];
    }
    return (orc_h(w) * orc_h(x)) * (float)(s0 + s1) + orc_h(w + 2) * orc_h(x + 2);
}

void oracle_gemm_nt_q5_1_q8_1_ref(const void *A_q8, const void *B, const float *bias, float *C, int M, int N, int K)
{
    if (!A_q8 || !B || !C || M <= 0 || N <= 0 || K <= 0 || K % 32) return;
    const int nb = K / 32;
    for (int m = 0; m < M; ++m)
        for (int n = 0; n < N; ++n) {
            float sum = 0.0f;
            for (int b = 0; b < nb; ++b) sum += orc_dot_q5_1_q8_1_block((const uint8_t *)B + ((size_t)n * nb + b) * 24, (const uint8_t *)A_q8 + ((size_t)m * nb + b) * 36);
            C[(size_t)m * N + n] = sum + (bias ? bias[n] : 0.0f);
        }
}

void oracle_gemv_q5_1_q8_1_ref(float *y, const void *W, const void *x_q8, int M, int K) { oracle_gemm_nt_q5_1_q8_1_ref(x_q8, W, NULL, y, 1, M, K); }

/* fp32 in, quantised inside, rows of at most 256 blocks (src/kernels/gemm_kernels_q5_1_q8_1.c:125-175) */
void oracle_gemm_nt_q5_1_q8_1(const float *A, const void *B, const float *bias, float *C, int M, int N, int K)
{
    if (!A || !B || !C || M <= 0 || N <= 0 || K <= 0 || K % 32 || K / 32 > 256) return;
    uint8_t *q = (uint8_t *)malloc((size_t)(K / 32) * 36);
    for (int m = 0; m < M; ++m) {
        oracle_quantize_row_q8_1(A + (size_t)m * K, q, K);
        oracle_gemm_nt_q5_1_q8_1_ref(q, B, bias, C + (size_t)m * N, 1, N, K);
    }
    free(q);
}

void oracle_gemv_q5_1_q8_1(float *y, const void *W, const float *x, int M, int K) { oracle_gemm_nt_q5_1_q8_1(x, W, NULL, y, 1, M, K); }

/* ---- Q4_0 / Q4_1 / Q5_1 with fp32 activations.  Row dequantisers put element j in the low nibble of qs[j] and element j + 16 in the high
 * nibble (src/kernels/dequant_kernels.c:40-56, :119-139, :220-252); the GEMVs pair the nibbles of qs[i] with x[2i] and x[2i + 1]
 * (src/kernels/gemm_kernels_q4_0.c:49-78, gemm_kernels_q4_1.c:50-84, gemm_kernels_q5_1.c:52-100).  Both are restated as they are. ---- */
enum { ORC_Q40 = 0, ORC_Q41 = 1, ORC_Q51 = 2 };
static const int orc_legacy_bytes[3] = { 18, 20, 24 };

static float orc_legacy_elem(int fmt, const uint8_t *p, int e, int gemv_order)
{
    const float d = orc_h(p);
    const int byte_i = gemv_order ? e >> 1 : e & 15, hi = gemv_order ? e & 1 : e >> 4;
    if (fmt == ORC_Q40) {
        const uint8_t b = p[2 + byte_i];
        return d * (float)(int8_t)((hi ? (b >> 4) : (b & 15)) - 8);
    }
    const float m = orc_h(p + 2);
    if (fmt == ORC_Q41) {
        const uint8_t b = p[4 + byte_i];
        return d * (float)(hi ? (b >> 4) : (b & 15)) + m;
    }
    uint32_t qh;
    memcpy(&qh, p + 4, 4);
    const uint8_t b = p[8 + byte_i];
    const int fifth = gemv_order ? (int)((qh >> e) & 1) : (int)((qh >> (hi ? byte_i + 16 : byte_i)) & 1);
    return d * (float)((hi ? (b >> 4) : (b & 15)) | (fifth << 4)) + m;
}

static void orc_legacy_dequant(int fmt, const void *src, float *dst, size_t n)
{
    for (size_t i = 0; i < n; ++i) dst[i] = orc_legacy_elem(fmt, (const uint8_t *)src + (i / 32) * orc_legacy_bytes[fmt], (int)(i % 32), 0);
}
void oracle_dequant_q4_0_row(const void *src, float *dst, size_t n) { orc_legacy_dequant(ORC_Q40, src, dst, n); }
void oracle_dequant_q4_1_row(const void *src, float *dst, size_t n) { orc_legacy_dequant(ORC_Q41, src, dst, n); }
void oracle_dequant_q5_1_row(const void *src, float *dst, size_t n) { orc_legacy_dequant(ORC_Q51, src, dst, n); }

static void orc_legacy_gemv(int fmt, float *y, const void *W, const float *x, int M, int K)
{
    const int nb = K / 32;
    for (int r = 0; r < M; ++r) {
        float sum = 0.0f;
        for (int b = 0; b < nb; ++b) {
            const uint8_t *p = (const uint8_t *)W + ((size_t)r * nb + b) * orc_legacy_bytes[fmt];
            for (int e = 0; e < 32; ++e) {
                if (fmt == ORC_Q40) {      /* d * q * x, left to right (gemm_kernels_q4_0.c:71-72) */
                    const uint8_t bt = p[2 + (e >> 1)];
                    sum += orc_h(p) * (float)(int8_t)(((e & 1) ? (bt >> 4) : (bt & 15)) - 8) * x[b * 32 + e];
                } else {
                    sum += orc_legacy_elem(fmt, p, e, 1) * x[b * 32 + e];
                }
            }
        }
        y[r] = sum;
    }
}
void oracle_gemv_q4_0_ref(float *y, const void *W, const float *x, int M, int K) { orc_legacy_gemv(ORC_Q40, y, W, x, M, K); }
void oracle_gemv_q4_1_ref(float *y, const void *W, const float *x, int M, int K) { orc_legacy_gemv(ORC_Q41, y, W, x, M, K); }
void oracle_gemv_q5_1_ref(float *y, const void *W, const float *x, int M, int K) { orc_legacy_gemv(ORC_Q51, y, W, x, M, K); }
