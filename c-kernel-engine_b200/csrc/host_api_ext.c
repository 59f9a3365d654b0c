/* More reference-named entry points with HOST pointers (same conventions as host_api.c): the fp32-activation GEMMs
 * of the reference's debug path, the "contract" forms that quantise their fp32 input themselves, pairwise RoPE and the
 * general RoPE table, two small copies, and the flat ck_test_* wrappers of the reference's parity API.
 *
 * Everything here is a composition of device kernels the library already has: activations are copied in once, the
 * intermediate (quantised rows) stays on the device, results are copied back.
 */
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#include "../../include/ckb200.h"
#include "../../include/ckb200_kernels.h"
#include "launch.h"
#include "runtime.h"

enum { F_Q4K = 0, F_Q6K = 1, F_Q80 = 2, F_Q50 = 3 };

static int fmt_block32(int fmt) { return fmt == F_Q80 || fmt == F_Q50; }
static size_t w_row_bytes(int fmt, int K)
{
    switch (fmt) {
        case F_Q4K: return (size_t)(K / 256) * 144;
        case F_Q6K: return (size_t)(K / 256) * 210;
        case F_Q50: return (size_t)(K / 32) * 22;
        default: return (size_t)(K / 32) * 34;
    }
}
static size_t xq_row_bytes(int fmt, int K) { return fmt_block32(fmt) ? (size_t)(K / 32) * 34 : (size_t)(K / 256) * 292; }

/* ------------------------------------------------------------------ fp32-activation GEMMs (debug path of the reference)
 * gemm_nt_<fmt>(A fp32 [M][K], B [N][K] blocks, bias, C [M][N]) = one fp32-activation GEMV per token
 * (src/kernels/gemm_kernels_q4k.c:683-711, src/kernels/gemm_kernels_q6k.c:212-250, src/kernels/gemm_kernels_q8_0.c:683-696);
 * gemm_<fmt>(Y [N][M], W [M][K], X [N][K]) is the same loop with the roles named the other way round
 * (src/kernels/gemm_kernels_q4k.c:316-326, :461-469, src/kernels/gemm_kernels_q6k.c:195-210, src/kernels/gemm_kernels_q8_0.c:658-666). */
static void host_gemm_nt_f32(int fmt, const float *A, const void *B, const float *bias, float *C, int M, int N, int K)
{
    if (!A || !B || !C || M <= 0 || N <= 0 || K <= 0) return;
    if (ckb_ensure_init()) return;
    const size_t a_b = (size_t)M * K * sizeof(float), b_b = (size_t)N * w_row_bytes(fmt, K), c_b = (size_t)M * N * sizeof(float);
    const float *dA = (const float *)ckb_stage_in(A, a_b, CKB_SLOT_A, 0);
    const void *dB = ckb_stage_in(B, b_b, CKB_SLOT_W, 1);
    const float *dbias = bias ? (const float *)ckb_stage_in(bias, (size_t)N * sizeof(float), CKB_SLOT_B, 1) : NULL;
    int back;
    float *dC = (float *)ckb_stage_out(C, c_b, CKB_SLOT_C, &back);
    if (!dA || !dB || !dC || (bias && !dbias)) return;
    for (int m = 0; m < M; ++m) {
        int rc;
        float *y = dC + (size_t)m * N;
        const float *x = dA + (size_t)m * K;
        switch (fmt) {
            case F_Q4K: rc = ckb200_dev_gemv_q4_k(y, dB, x, N, K, NULL); break;
            case F_Q6K: rc = ckb200_dev_gemv_q6_k(y, dB, x, N, K, NULL); break;
            default: rc = ckb200_dev_gemv_q8_0(y, dB, x, N, K, NULL); break;
        }
        if (rc != 0) return;
    }
    if (dbias && ckb200_dev_add_bias_rows(dC, dbias, M, N, NULL) != 0) return;
    ckb_finish_out(C, dC, c_b, back);
}

void gemm_nt_q4_k(const float *A, const void *B, const float *bias, float *C, int M, int N, int K) { host_gemm_nt_f32(F_Q4K, A, B, bias, C, M, N, K); }
void gemm_nt_q6_k(const float *A, const void *B, const float *bias, float *C, int M, int N, int K) { host_gemm_nt_f32(F_Q6K, A, B, bias, C, M, N, K); }
void gemm_nt_q6_k_ref(const float *A, const void *B, const float *bias, float *C, int M, int N, int K) { host_gemm_nt_f32(F_Q6K, A, B, bias, C, M, N, K); }
void gemm_nt_q8_0(const float *A, const void *B, const float *bias, float *C, int M, int N, int K) { host_gemm_nt_f32(F_Q80, A, B, bias, C, M, N, K); }
void gemm_q4_k(float *Y, const void *W, const float *X, int M, int N, int K) { host_gemm_nt_f32(F_Q4K, X, W, NULL, Y, N, M, K); }
void gemm_q4_k_ref(float *Y, const void *W, const float *X, int M, int N, int K) { host_gemm_nt_f32(F_Q4K, X, W, NULL, Y, N, M, K); }
void gemm_q6_k(float *Y, const void *W, const float *X, int M, int N, int K) { host_gemm_nt_f32(F_Q6K, X, W, NULL, Y, N, M, K); }
void gemm_q8_0(float *Y, const void *W, const float *X, int M, int N, int K) { host_gemm_nt_f32(F_Q80, X, W, NULL, Y, N, M, K); }

/* ------------------------------------------------------------------ fp32 in, quantised inside
 * C[m][n] = dot(B row n, quantise(A row m)) + bias[n]: the activations are quantised on the device (Q8_K for the
 * K-quants, Q8_0 for the 32-element formats) and fed to the quantised GEMV / GEMM; nothing but fp32 crosses the bus. */
static void host_quant_gemm_nt(int fmt, const float *A, const void *B, const float *bias, float *C, int M, int N, int K)
{
    if (!A || !B || !C || M <= 0 || N <= 0 || K <= 0) return;
    if (ckb_ensure_init()) return;
    if (K % (fmt_block32(fmt) ? 32 : 256)) { ckb_fail(CKB_ERR_SHAPE, "quantised product: K=%d is not a whole number of blocks", K); return; }
    const size_t a_b = (size_t)M * K * sizeof(float), b_b = (size_t)N * w_row_bytes(fmt, K), c_b = (size_t)M * N * sizeof(float);
    const float *dA = (const float *)ckb_stage_in(A, a_b, CKB_SLOT_X, 0);
    const void *dB = ckb_stage_in(B, b_b, CKB_SLOT_W, 1);
    const float *dbias = bias ? (const float *)ckb_stage_in(bias, (size_t)N * sizeof(float), CKB_SLOT_B, 1) : NULL;
    void *dQ = ckb_scratch(CKB_SLOT_A, (size_t)M * xq_row_bytes(fmt, K));
    int back;
    float *dC = (float *)ckb_stage_out(C, c_b, CKB_SLOT_C, &back);
    if (!dA || !dB || !dQ || !dC || (bias && !dbias)) return;
    int rc = fmt_block32(fmt) ? ckb200_dev_quantize_q8_0(dA, dQ, M, K, NULL) : ckb200_dev_quantize_q8_k(dA, dQ, M, K, NULL);
    if (rc != 0) return;
    switch (fmt) {
        case F_Q4K: rc = ckb200_dev_gemm_nt_q4_k_q8_k(dQ, dB, dbias, dC, M, N, K, NULL); break;
        case F_Q6K: rc = ckb200_dev_gemm_nt_q6_k_q8_k(dQ, dB, dbias, dC, M, N, K, NULL); break;
        case F_Q50: rc = ckb200_dev_gemm_nt_q5_0_q8_0(dQ, dB, dbias, dC, M, N, K, NULL); break;
        default: rc = ckb200_dev_gemm_nt_q8_0_q8_0(dQ, dB, dbias, dC, M, N, K, NULL); break;
    }
    if (rc != 0) return;
    ckb_finish_out(C, dC, c_b, back);
}

/* gemm_nt_q6_k_sse (src/kernels/gemm_kernels_q6k_sse.c:66-97): quantises each A row to Q8_K, then Q6_K x Q8_K dots */
void gemm_nt_q6_k_sse(const float *A, const void *B, const float *bias, float *C, int M, int N, int K)
{
    if (K % 256) { host_gemm_nt_f32(F_Q6K, A, B, bias, C, M, N, K); return; }
    host_quant_gemm_nt(F_Q6K, A, B, bias, C, M, N, K);
}

/* gemv_q8_0_q8_0_contract / gemm_nt_q8_0_q8_0_contract (src/kernels/gemm_kernels_q8_0_q8_0_contract.c:377-406, :408-486):
 * rows of up to 1024 blocks are quantised to Q8_0 and go through the integer kernel, longer ones (and K not a multiple
 * of 32) through the fp32-activation GEMV, as in the reference. */
#define CONTRACT_MAX_BLOCKS 1024
void gemv_q8_0_q8_0_contract(float *y, const void *W, const float *x, int M, int K)
{
    if (!y || !W || !x || M <= 0 || K <= 0) return;
    if (K % 32 || K / 32 > CONTRACT_MAX_BLOCKS) { gemv_q8_0(y, W, x, M, K); return; }
    host_quant_gemm_nt(F_Q80, x, W, NULL, y, 1, M, K);
}
void gemm_nt_q8_0_q8_0_contract(const float *A, const void *B, const float *bias, float *C, int M, int N, int K)
{
    if (!A || !B || !C || M <= 0 || N <= 0 || K <= 0) return;
    if (K % 32 || K / 32 > CONTRACT_MAX_BLOCKS) { host_gemm_nt_f32(F_Q80, A, B, bias, C, M, N, K); return; }
    host_quant_gemm_nt(F_Q80, A, B, bias, C, M, N, K);
}

/* ------------------------------------------------------------------ RoPE: general table and the pairwise (interleaved) rotation */

void rope_precompute_cache(float *cos_cache, float *sin_cache, int max_seq_len, int head_dim, float base, int rotary_dim,
                           const char *scaling_type, float scaling_factor)
{
    if (!cos_cache || !sin_cache || max_seq_len <= 0 || head_dim <= 1) return;
    if (ckb_ensure_init()) return;
    if (rotary_dim <= 0 || rotary_dim > head_dim) rotary_dim = head_dim;
    const size_t b = (size_t)max_seq_len * (rotary_dim / 2) * sizeof(float);
    if (b == 0) return;
    const int linear = scaling_type && !strcmp(scaling_type, "linear");
    int bc, bs;
    float *dc = (float *)ckb_stage_out(cos_cache, b, CKB_SLOT_A, &bc);
    float *ds = (float *)ckb_stage_out(sin_cache, b, CKB_SLOT_B, &bs);
    if (!dc || !ds) return;
    if (ckb200_dev_rope_precompute_cache(dc, ds, max_seq_len, head_dim, base, rotary_dim, linear, scaling_factor, NULL) != 0) return;
    if (bc) cudaMemcpyAsync(cos_cache, dc, b, cudaMemcpyDeviceToHost, ckb_stream(NULL));
    ckb_finish_out(sin_cache, ds, b, bs);
}

void rope_forward_qk_pairwise_with_rotary_dim(float *q, float *k, const float *cos_cache, const float *sin_cache, int num_heads,
                                              int num_kv_heads, int num_tokens, int head_dim, int aligned_head_dim, int pos_offset,
                                              int rotary_dim)
{
    if (!q || !k || !cos_cache || !sin_cache || num_heads <= 0 || num_kv_heads <= 0 || num_tokens <= 0 || head_dim <= 1) return;
    if (ckb_ensure_init()) return;
    if (rotary_dim <= 0 || rotary_dim > head_dim) rotary_dim = head_dim;
    const size_t qb = (size_t)num_heads * num_tokens * aligned_head_dim * sizeof(float);
    const size_t kb = (size_t)num_kv_heads * num_tokens * aligned_head_dim * sizeof(float);
    const size_t cb = (size_t)(pos_offset + num_tokens) * (rotary_dim / 2) * sizeof(float);
    float *dq = (float *)ckb_stage_in(q, qb, CKB_SLOT_X, 0);
    float *dk = (float *)ckb_stage_in(k, kb, CKB_SLOT_Y, 0);
    const float *dc = (const float *)ckb_stage_in(cos_cache, cb, CKB_SLOT_A, 1);
    const float *ds = (const float *)ckb_stage_in(sin_cache, cb, CKB_SLOT_B, 1);
    if (!dq || !dk || !dc || !ds) return;
    if (ckb200_dev_rope_forward_qk_pairwise(dq, dk, dc, ds, num_heads, num_kv_heads, num_tokens, head_dim, aligned_head_dim, pos_offset,
                                            rotary_dim, NULL, NULL) != 0) return;
    if (dq != q) cudaMemcpyAsync(q, dq, qb, cudaMemcpyDeviceToHost, ckb_stream(NULL));
    ckb_finish_out(k, dk, kb, dk != k);
}

/* rope_forward_qk_with_rotary_dim (src/kernels/rope_kernels.c:821-837): half-split pairs over the first rotary_dim channels */
void rope_forward_qk_with_rotary_dim(float *q, float *k, const float *cos_cache, const float *sin_cache, int num_heads, int num_kv_heads,
                                     int num_tokens, int head_dim, int aligned_head_dim, int pos_offset, int rotary_dim)
{
    if (!q || !k || !cos_cache || !sin_cache || num_heads <= 0 || num_kv_heads <= 0 || num_tokens <= 0 || head_dim <= 1) return;
    if (ckb_ensure_init()) return;
    if (rotary_dim <= 0 || rotary_dim > head_dim) rotary_dim = head_dim;
    const size_t qb = (size_t)num_heads * num_tokens * aligned_head_dim * sizeof(float);
    const size_t kb = (size_t)num_kv_heads * num_tokens * aligned_head_dim * sizeof(float);
    const size_t cb = (size_t)(pos_offset + num_tokens) * (rotary_dim / 2) * sizeof(float);
    float *dq = (float *)ckb_stage_in(q, qb, CKB_SLOT_X, 0);
    float *dk = (float *)ckb_stage_in(k, kb, CKB_SLOT_Y, 0);
    const float *dc = (const float *)ckb_stage_in(cos_cache, cb, CKB_SLOT_A, 1);
    const float *ds = (const float *)ckb_stage_in(sin_cache, cb, CKB_SLOT_B, 1);
    if (!dq || !dk || !dc || !ds) return;
    if (ckb200_dev_rope_forward_qk_with_rotary_dim(dq, dk, dc, ds, num_heads, num_kv_heads, num_tokens, head_dim, aligned_head_dim, pos_offset, rotary_dim, NULL,
                                                   NULL) != 0) return;
    if (dq != q) cudaMemcpyAsync(q, dq, qb, cudaMemcpyDeviceToHost, ckb_stream(NULL));
    ckb_finish_out(k, dk, kb, dk != k);
}

/* ------------------------------------------------------------------ small copies */

/* add_inplace_f32 (include/ckernel_engine.h:1894, src/kernels/add_kernels_bf16.c:304): a[i] += b[i] */
void add_inplace_f32(float *a, const float *b, size_t n)
{
    if (!a || !b || n == 0) return;
    if (ckb_ensure_init()) return;
    float *da = (float *)ckb_stage_in(a, n * sizeof(float), CKB_SLOT_X, 0);
    const float *db = (const float *)ckb_stage_in(b, n * sizeof(float), CKB_SLOT_A, 0);
    if (!da || !db) return;
    if (ckb200_dev_add_inplace(da, db, (long long)n, NULL) != 0) return;
    ckb_finish_out(a, da, n * sizeof(float), da != a);
}

/* logits_copy_to_position (src/kernels/kv_cache_kernels.c:178-191): dst[position][0:vocab] = src; the buffers may be
 * device memory, host memory, or one of each, and may overlap (the reference uses memmove). */
void logits_copy_to_position(const float *src, float *dst, int position, int vocab_size)
{
    if (!src || !dst || position < 0 || vocab_size <= 0) return;
    float *to = dst + (size_t)position * (size_t)vocab_size;
    const size_t bytes = (size_t)vocab_size * sizeof(float);
    if (!ckb_is_device_ptr(src) && !ckb_is_device_ptr(to)) { memmove(to, src, bytes); return; }
    if (ckb_ensure_init()) return;
    cudaStream_t st = ckb_stream(NULL);
    if (ckb_check_cuda((int)cudaMemcpyAsync(to, src, bytes, cudaMemcpyDefault, st), "logits_copy_to_position")) return;
    ckb_check_cuda((int)cudaStreamSynchronize(st), "sync");
}

/* ------------------------------------------------------------------ the reference's flat parity API
 * ck_test_* (src/ck_parity_api.c:189-694): what the reference's kernel-parity scripts bind.  Same argument order and
 * meaning; each is the composition the reference wrapper performs (quantise the fp32 input, run the quantised kernel). */

void ck_test_dequant_q4_k(const void *src, float *dst, int n) { if (n > 0) dequant_q4_k_row(src, dst, (size_t)n); }
void ck_test_dequant_q6_k(const void *src, float *dst, int n) { if (n > 0) dequant_q6_k_row(src, dst, (size_t)n); }
void ck_test_quantize_q8_k(const float *src, void *dst, int n) { quantize_row_q8_k(src, dst, n); }

void ck_test_gemv_q4_k(const void *weight_q4k, const float *input_f32, float *output, int cols) { host_quant_gemm_nt(F_Q4K, input_f32, weight_q4k, NULL, output, 1, 1, cols); }
void ck_test_gemv_q6_k(const void *weight_q6k, const float *input_f32, float *output, int cols) { host_quant_gemm_nt(F_Q6K, input_f32, weight_q6k, NULL, output, 1, 1, cols); }
void ck_test_gemv_q5_0(const void *weight_q5_0, const float *input_f32, float *output, int rows, int cols) { host_quant_gemm_nt(F_Q50, input_f32, weight_q5_0, NULL, output, 1, rows, cols); }
void ck_test_gemv_q8_0(const void *weight_q8_0, const float *input_f32, float *output, int rows, int cols) { host_quant_gemm_nt(F_Q80, input_f32, weight_q8_0, NULL, output, 1, rows, cols); }
void ck_test_gemv_q5_0_q8_0(const void *weight_q5_0, const float *input_f32, float *output, int rows, int cols) { host_quant_gemm_nt(F_Q50, input_f32, weight_q5_0, NULL, output, 1, rows, cols); }
void ck_test_gemv_q8_0_q8_0(const void *weight_q8_0, const float *input_f32, float *output, int rows, int cols) { host_quant_gemm_nt(F_Q80, input_f32, weight_q8_0, NULL, output, 1, rows, cols); }
void ck_test_vec_dot_q5_0_q8_0(const void *weight_q5_0, const void *input_q8_0, float *output, int cols) { vec_dot_q5_0_q8_0(cols, output, weight_q5_0, input_q8_0); }
void ck_test_vec_dot_q8_0_q8_0(const void *weight_q8_0, const void *input_q8_0, float *output, int cols) { vec_dot_q8_0_q8_0(cols, output, weight_q8_0, input_q8_0); }
/* output [n_tokens][rows] = input [n_tokens][cols] . weight [rows][cols]^T */
void ck_test_gemm_q4_k(const void *weight_q4k, const float *input_f32, float *output, int rows, int cols, int n_tokens) { host_quant_gemm_nt(F_Q4K, input_f32, weight_q4k, NULL, output, n_tokens, rows, cols); }
void ck_test_gemm_q6_k(const void *weight_q6k, const float *input_f32, float *output, int rows, int cols, int n_tokens) { host_quant_gemm_nt(F_Q6K, input_f32, weight_q6k, NULL, output, n_tokens, rows, cols); }
void ck_test_gemm_q8_0(const void *weight_q8_0, const float *input_f32, float *output, int rows, int cols, int n_tokens) { host_quant_gemm_nt(F_Q80, input_f32, weight_q8_0, NULL, output, n_tokens, rows, cols); }
void ck_test_gemm_q5_0(const void *weight_q5_0, const float *input_f32, float *output, int rows, int cols, int n_tokens) { host_quant_gemm_nt(F_Q50, input_f32, weight_q5_0, NULL, output, n_tokens, rows, cols); }

void ck_test_rmsnorm(const float *input, const float *weight, float *output, int n_tokens, int dim, float eps)
{
    rmsnorm_forward(input, weight, output, NULL, n_tokens, dim, dim, eps);
}
void ck_test_swiglu(const float *gate_up, float *output, int n_tokens, int intermediate_dim) { swiglu_forward(gate_up, output, n_tokens, intermediate_dim); }

/* q [T][H*D], k [T][Hkv*D] token-major, rotate-half with a table built for theta: the wrapper transposes to the kernels'
 * head-major layout and back (src/ck_parity_api.c:552-628) */
static void test_rope_common(int pairwise, float *q, float *k, int n_tokens, int n_heads, int n_heads_kv, int head_dim, int pos_offset, float theta)
{
    if (!q || !k || n_tokens <= 0 || n_heads <= 0 || n_heads_kv <= 0 || head_dim <= 1 || pos_offset < 0) return;
    const int half = head_dim / 2, max_seq = pos_offset + n_tokens;
    float *cs = (float *)malloc((size_t)2 * max_seq * half * sizeof(float));
    float *qr = (float *)malloc((size_t)n_heads * n_tokens * head_dim * sizeof(float));
    float *kr = (float *)malloc((size_t)n_heads_kv * n_tokens * head_dim * sizeof(float));
    if (cs && qr && kr) {
        float *sn = cs + (size_t)max_seq * half;
        rope_precompute_cache(cs, sn, max_seq, head_dim, theta, head_dim, "none", 1.0f);
        for (int t = 0; t < n_tokens; ++t) {
            for (int h = 0; h < n_heads; ++h)
                memcpy(qr + ((size_t)h * n_tokens + t) * head_dim, q + ((size_t)t * n_heads + h) * head_dim, (size_t)head_dim * sizeof(float));
            for (int h = 0; h < n_heads_kv; ++h)
                memcpy(kr + ((size_t)h * n_tokens + t) * head_dim, k + ((size_t)t * n_heads_kv + h) * head_dim, (size_t)head_dim * sizeof(float));
        }
        if (pairwise) rope_forward_qk_pairwise_with_rotary_dim(qr, kr, cs, sn, n_heads, n_heads_kv, n_tokens, head_dim, head_dim, pos_offset, head_dim);
        else rope_forward_qk(qr, kr, cs, sn, n_heads, n_heads_kv, n_tokens, head_dim, head_dim, pos_offset);
        for (int t = 0; t < n_tokens; ++t) {
            for (int h = 0; h < n_heads; ++h)
                memcpy(q + ((size_t)t * n_heads + h) * head_dim, qr + ((size_t)h * n_tokens + t) * head_dim, (size_t)head_dim * sizeof(float));
            for (int h = 0; h < n_heads_kv; ++h)
                memcpy(k + ((size_t)t * n_heads_kv + h) * head_dim, kr + ((size_t)h * n_tokens + t) * head_dim, (size_t)head_dim * sizeof(float));
        }
    }
    free(cs);
    free(qr);
    free(kr);
}

void ck_test_rope(float *q, float *k, int n_tokens, int n_heads, int n_heads_kv, int head_dim, int pos_offset, float theta)
{
    test_rope_common(0, q, k, n_tokens, n_heads, n_heads_kv, head_dim, pos_offset, theta);
}

/* the interleaved (pair-rotated) form with the same arguments (src/ck_parity_api.c:630-687) */
void ck_test_rope_interleaved(float *q, float *k, int n_tokens, int n_heads, int n_heads_kv, int head_dim, int pos_offset, float theta)
{
    test_rope_common(1, q, k, n_tokens, n_heads, n_heads_kv, head_dim, pos_offset, theta);
}

/* src/ck_parity_api.c:199-202 and :861-881 */
void ck_test_dequant_q4_0(const void *src, float *dst, int n) { dequant_q4_0_row(src, dst, (size_t)n); }
void ck_test_attention_causal(const float *q, const float *k, const float *v, float *out, int num_heads, int num_kv_heads, int tokens, int seq_len, int head_dim)
{
    attention_forward_causal_head_major_gqa_flash_strided(q, k, v, out, num_heads, num_kv_heads, tokens, head_dim, head_dim, seq_len);
}
