/* Reference-named entry points (HOST pointers, conventions of host_api.c) for the further weight formats:
 *   Q5_K   gemv_q5_k_q8_k[_ref], gemm_nt_q5_k_q8_k[_ref], gemv_q5_k[_ref], gemm_nt_q5_k[_ref]      src/kernels/gemm_kernels_q5_k.c:305-520
 *   Q5_1 x Q8_1   gemv_q5_1_q8_1[_ref], gemm_nt_q5_1_q8_1[_ref]                                    src/kernels/gemm_kernels_q5_1_q8_1.c:75-175
 *   Q4_0, Q4_1, Q5_1 with fp32 activations: dequant_*_row, gemv_*[_ref], gemm_*, gemm_nt_*, dot_*   src/kernels/gemm_kernels_q4_0.c,
 *                                                                                  gemm_kernels_q4_1.c, gemm_kernels_q5_1.c, dequant_kernels.c
 * Activations are copied in once, quantised rows stay on the device, results are copied back. */
#include <stdint.h>
#include <stdlib.h>

#include "../../include/ckb200.h"
#include "../../include/ckb200_kernels.h"
#include "launch.h"
#include "runtime.h"

enum { L_Q40 = 0, L_Q41 = 1, L_Q51 = 2, L_Q5K = 3 };
static const int l_block_bytes[4] = { 18, 20, 24, 176 }, l_block_elems[4] = { 32, 32, 32, 256 };

static int l_gemv_f32(int fmt, float *y, const void *W, const float *x, int M, int K)
{
    switch (fmt) {
        case L_Q40: return ckb200_dev_gemv_q4_0(y, W, x, M, K, NULL);
        case L_Q41: return ckb200_dev_gemv_q4_1(y, W, x, M, K, NULL);
        case L_Q51: return ckb200_dev_gemv_q5_1(y, W, x, M, K, NULL);
        default: return ckb200_dev_gemv_q5_k_f32(y, W, x, M, K, NULL);
    }
}

/* C[m][n] = A[m] . B[n] (+ bias[n]) with fp32 activations: one dequantise-and-multiply GEMV per token */
static void host_f32_gemm_nt(int fmt, const float *A, const void *B, const float *bias, float *C, int M, int N, int K)
{
    if (!A || !B || !C || M <= 0 || N <= 0 || K <= 0) return;
    if (ckb_ensure_init()) return;
    const int Kb = K - K % l_block_elems[fmt];          /* whole blocks only, as the reference's loops */
    if (Kb <= 0) return;
    const size_t a_b = (size_t)M * K * sizeof(float), b_b = (size_t)N * (Kb / l_block_elems[fmt]) * l_block_bytes[fmt], c_b = (size_t)M * N * sizeof(float);
    const float *dA = (const float *)ckb_stage_in(A, a_b, CKB_SLOT_A, 0);
    const void *dB = ckb_stage_in(B, b_b, CKB_SLOT_W, 1);
    const float *dbias = bias ? (const float *)ckb_stage_in(bias, (size_t)N * sizeof(float), CKB_SLOT_B, 1) : NULL;
    int back;
    float *dC = (float *)ckb_stage_out(C, c_b, CKB_SLOT_C, &back);
    if (!dA || !dB || !dC || (bias && !dbias)) return;
    for (int m = 0; m < M; ++m)
        if (l_gemv_f32(fmt, dC + (size_t)m * N, dB, dA + (size_t)m * K, N, Kb) != 0) return;
    if (dbias && ckb200_dev_add_bias_rows(dC, dbias, M, N, NULL) != 0) return;
    ckb_finish_out(C, dC, c_b, back);
}

#define LEGACY_F32(fmt, tag)                                                                                                                              \
    void gemv_##fmt##_ref(float *y, const void *W, const float *x, int M, int K) { host_f32_gemm_nt(tag, x, W, NULL, y, 1, M, K); }                     \
    void gemv_##fmt(float *y, const void *W, const float *x, int M, int K) { host_f32_gemm_nt(tag, x, W, NULL, y, 1, M, K); }                           \
    void gemm_##fmt(float *Y, const void *W, const float *X, int M, int N, int K) { host_f32_gemm_nt(tag, X, W, NULL, Y, N, M, K); }                    \
    void gemm_nt_##fmt(const float *A, const void *B, const float *bias, float *C, int M, int N, int K) { host_f32_gemm_nt(tag, A, B, bias, C, M, N, K); } \
    float dot_##fmt(const void *w, const float *x, int K) { float r = 0.0f; host_f32_gemm_nt(tag, x, w, NULL, &r, 1, 1, K); return r; }

LEGACY_F32(q4_0, L_Q40)
LEGACY_F32(q4_1, L_Q41)
LEGACY_F32(q5_1, L_Q51)

static void host_dequant(int (*fn)(const void *, float *, size_t, void *), const void *src, float *dst, size_t n, int block_bytes)
{
    if (!src || !dst || n == 0 || n % 32) return;
    if (ckb_ensure_init()) return;
    const void *ds = ckb_stage_in(src, n / 32 * (size_t)block_bytes, CKB_SLOT_W, 1);
    int back;
    float *dd = (float *)ckb_stage_out(dst, n * sizeof(float), CKB_SLOT_C, &back);
    if (!ds || !dd || fn(ds, dd, n, NULL) != 0) return;
    ckb_finish_out(dst, dd, n * sizeof(float), back);
}
void dequant_q4_0_row(const void *src, float *dst, size_t n) { host_dequant(ckb200_dev_dequant_q4_0_row, src, dst, n, 18); }
void dequant_q4_1_row(const void *src, float *dst, size_t n) { host_dequant(ckb200_dev_dequant_q4_1_row, src, dst, n, 20); }
void dequant_q5_1_row(const void *src, float *dst, size_t n) { host_dequant(ckb200_dev_dequant_q5_1_row, src, dst, n, 24); }

/* ------------------------------------------------------------------ quantised products */

/* kind 0: Q5_K x Q8_K, kind 1: Q5_1 x Q8_1.  `quantise`: A is fp32 and is quantised on the device first. */
static void host_q_gemm_nt(int kind, int quantise, const void *A, const void *B, const float *bias, float *C, int M, int N, int K)
{
    if (!A || !B || !C || M <= 0 || N <= 0 || K <= 0) return;
    const int be = kind ? 32 : 256, wb = kind ? 24 : 176, xb = kind ? 36 : 292;
    if (K % be) return;
    if (ckb_ensure_init()) return;
    const size_t aq_b = (size_t)M * (K / be) * xb, b_b = (size_t)N * (K / be) * wb, c_b = (size_t)M * N * sizeof(float);
    const void *dQ;
    if (quantise) {
        const float *dA = (const float *)ckb_stage_in(A, (size_t)M * K * sizeof(float), CKB_SLOT_X, 0);
        void *q = ckb_scratch(CKB_SLOT_A, aq_b);
        if (!dA || !q) return;
        if ((kind ? ckb200_dev_quantize_q8_1(dA, q, M, K, NULL) : ckb200_dev_quantize_q8_k(dA, q, M, K, NULL)) != 0) return;
        dQ = q;
    } else {
        dQ = ckb_stage_in(A, aq_b, CKB_SLOT_A, 0);
    }
    const void *dB = ckb_stage_in(B, b_b, CKB_SLOT_W, 1);
    const float *dbias = bias ? (const float *)ckb_stage_in(bias, (size_t)N * sizeof(float), CKB_SLOT_B, 1) : NULL;
    int back;
    float *dC = (float *)ckb_stage_out(C, c_b, CKB_SLOT_C, &back);
    if (!dQ || !dB || !dC || (bias && !dbias)) return;
    const int rc = kind ? ckb200_dev_gemm_nt_q5_1_q8_1(dQ, dB, dbias, dC, M, N, K, NULL) : ckb200_dev_gemm_nt_q5_k_q8_k(dQ, dB, dbias, dC, M, N, K, NULL);
    if (rc != 0) return;
    ckb_finish_out(C, dC, c_b, back);
}

void gemv_q5_k_q8_k(float *y, const void *W, const void *x_q8, int M, int K) { host_q_gemm_nt(0, 0, x_q8, W, NULL, y, 1, M, K); }
void gemv_q5_k_q8_k_ref(float *y, const void *W, const void *x_q8, int M, int K) { host_q_gemm_nt(0, 0, x_q8, W, NULL, y, 1, M, K); }
void gemm_nt_q5_k_q8_k(const void *A_q8, const void *B, const float *bias, float *C, int M, int N, int K) { host_q_gemm_nt(0, 0, A_q8, B, bias, C, M, N, K); }
void gemm_nt_q5_k_q8_k_ref(const void *A_q8, const void *B, const float *bias, float *C, int M, int N, int K) { host_q_gemm_nt(0, 0, A_q8, B, bias, C, M, N, K); }

/* fp32 in: rows of whole superblocks, at most 128 of them, are quantised to Q8_K; anything else takes the fp32 path, which reads the block
 * in the order of the reference's fall-back (src/kernels/gemm_kernels_q5_k.c:369-434) */
#define Q5K_MAX_Q8_BLOCKS 128
void gemm_nt_q5_k(const float *A, const void *B, const float *bias, float *C, int M, int N, int K)
{
    if (K > 0 && (K % 256 || K / 256 > Q5K_MAX_Q8_BLOCKS)) { host_f32_gemm_nt(L_Q5K, A, B, bias, C, M, N, K); return; }
    host_q_gemm_nt(0, 1, A, B, bias, C, M, N, K);
}
void gemm_nt_q5_k_ref(const float *A, const void *B, const float *bias, float *C, int M, int N, int K) { gemm_nt_q5_k(A, B, bias, C, M, N, K); }
void gemv_q5_k(float *y, const void *W, const float *x, int M, int K) { gemm_nt_q5_k(x, W, NULL, y, 1, M, K); }
void gemv_q5_k_ref(float *y, const void *W, const float *x, int M, int K) { gemm_nt_q5_k(x, W, NULL, y, 1, M, K); }

void gemv_q5_1_q8_1_ref(float *y, const void *W, const void *x_q8, int M, int K) { host_q_gemm_nt(1, 0, x_q8, W, NULL, y, 1, M, K); }
void gemm_nt_q5_1_q8_1_ref(const void *A_q8, const void *B, const float *bias, float *C, int M, int N, int K) { host_q_gemm_nt(1, 0, A_q8, B, bias, C, M, N, K); }
/* fp32 in, rows of at most 256 blocks (src/kernels/gemm_kernels_q5_1_q8_1.c:125-175: longer rows are left untouched there too) */
void gemm_nt_q5_1_q8_1(const float *A, const void *B, const float *bias, float *C, int M, int N, int K)
{
    if (K <= 0 || K % 32 || K / 32 > 256) return;
    host_q_gemm_nt(1, 1, A, B, bias, C, M, N, K);
}
void gemv_q5_1_q8_1(float *y, const void *W, const float *x, int M, int K) { gemm_nt_q5_1_q8_1(x, W, NULL, y, 1, M, K); }
