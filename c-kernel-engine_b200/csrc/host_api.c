/* Reference-named entry points: the reference's own C symbols and signatures, HOST pointers in
 * and out, executed by the CUDA kernels.  This is what generated libmodel.so code, the
 * *_parallel_dispatch seam and the reference's ctypes unit tests bind
 * (prototypes: include/ckernel_engine.h:192-363, :1209-1257, :1635-1697 and include/ckernel_quant.h:398-410
 * in the reference).
 *
 * Per call: weights are looked up in the resident registry (else copied in), activations are
 * copied in, the kernels run on the library stream, results are copied back, the stream is
 * synchronised.  A pointer that already is device memory is used as is.  Like the reference
 * these functions are void and return silently on NULL / non-positive arguments; anything a
 * GPU adds (no device, alignment, launch failure) goes to ckb200_last_error().
 */
#include <stdint.h>
#include <string.h>

#include "../../include/ckb200.h"
#include "../../include/ckb200_kernels.h"
#include "launch.h"
#include "runtime.h"

#define Q4K_B 144
#define Q6K_B 210
#define Q80_B 34
#define Q8K_B 292

enum { F_Q4K = 0, F_Q6K = 1, F_Q80 = 2, F_Q50 = 3 };     /* F_Q50: Q5_0 weights (22-byte blocks) with Q8_0 activations */

int ckb_gemm_nt_q80_tc(const void *A_raw, const void *B_raw, const void *B_planar, const float *bias, float *C, int M, int N, int K, void *stream);   /* gemm.cu */

static size_t w_row_bytes(int fmt, int K)
{
    switch (fmt) {
        case F_Q4K: return (size_t)(K / 256) * Q4K_B;
        case F_Q6K: return (size_t)(K / 256) * Q6K_B;
        case F_Q50: return (size_t)(K / 32) * 22;
        default: return (size_t)(K / 32) * Q80_B;
    }
}
static size_t xq_bytes(int fmt, int K) { return (fmt == F_Q80 || fmt == F_Q50) ? (size_t)(K / 32) * Q80_B : (size_t)(K / 256) * Q8K_B; }

/* ------------------------------------------------------------------ quantisers */

static void host_quantize(int q80, const float *x, void *y, int rows, int k)
{
    if (!x || !y || rows <= 0 || k <= 0) return;
    if (ckb_ensure_init()) return;
    const size_t in_b = (size_t)rows * k * sizeof(float);
    const size_t out_b = (size_t)rows * xq_bytes(q80 ? F_Q80 : F_Q4K, k);
    const float *dx = (const float *)ckb_stage_in(x, in_b, CKB_SLOT_X, 0);
    int back;
    void *dy = ckb_stage_out(y, out_b, CKB_SLOT_Y, &back);
    if (!dx || !dy) return;
    if ((q80 ? ckb200_dev_quantize_q8_0(dx, dy, rows, k, NULL) : ckb200_dev_quantize_q8_k(dx, dy, rows, k, NULL)) != 0) return;
    ckb_finish_out(y, dy, out_b, back);
}

void quantize_row_q8_k(const float *x, void *y, int k) { host_quantize(0, x, y, 1, k); }
void quantize_row_q8_k_ref(const float *x, void *y, int k) { host_quantize(0, x, y, 1, k); }
void quantize_batch_q8_k(const float *x, void *y, int num_rows, int k) { host_quantize(0, x, y, num_rows, k); }
void quantize_row_q8_0(const float *x, void *y, int k) { host_quantize(1, x, y, 1, k); }
void quantize_batch_q8_0(const float *x, void *y, int num_rows, int k) { host_quantize(1, x, y, num_rows, k); }

/* ------------------------------------------------------------------ GEMV (quantised activations) */

static int dev_gemv(int fmt, float *y, const void *W, const void *xq, int M, int K)
{
    switch (fmt) {
        case F_Q4K: return ckb200_dev_gemv_q4_k_q8_k(y, W, xq, M, K, NULL);
        case F_Q6K: return ckb200_dev_gemv_q6_k_q8_k(y, W, xq, M, K, NULL);
        case F_Q50: return ckb200_dev_gemv_q5_0_q8_0(y, W, xq, M, K, NULL);
        default: return ckb200_dev_gemv_q8_0_q8_0(y, W, xq, M, K, NULL);
    }
}

/* rows [r0, r1) of y = W . x; the whole call when r0 = 0, r1 = M */
static void host_gemv_rows(int fmt, float *y, const void *W, const void *x_q8, int M, int K, int r0, int r1)
{
    if (!y || !W || !x_q8 || M <= 0 || K <= 0 || r0 >= r1) return;
    if (ckb_ensure_init()) return;
    const size_t rb = w_row_bytes(fmt, K);
    const uint8_t *Wr = (const uint8_t *)W + (size_t)r0 * rb;
    const int rows = r1 - r0;
    const void *dW = ckb_stage_in(Wr, (size_t)rows * rb, CKB_SLOT_W, 1);
    const void *dX = ckb_stage_in(x_q8, xq_bytes(fmt, K), CKB_SLOT_X, 0);
    int back;
    float *dY = (float *)ckb_stage_out(y + r0, (size_t)rows * sizeof(float), CKB_SLOT_Y, &back);
    if (!dW || !dX || !dY) return;
    /* resident weights in one of the 2-byte-aligned formats: the row-planar copy (built once) streams at aligned 16-byte loads */
    const void *planar = (fmt != F_Q4K && ckb200_device_ptr(Wr) == dW) ? ckb_planar_shadow(fmt, dW, rows, K) : NULL;
    int rc;
    if (planar) {
        switch (fmt) {
            case F_Q6K: rc = ckb200_dev_gemv_q6_k_planar_q8_k(dY, planar, dX, rows, K, NULL); break;
            case F_Q50: rc = ckb200_dev_gemv_q5_0_planar_q8_0(dY, planar, dX, rows, K, NULL); break;
            default: rc = ckb200_dev_gemv_q8_0_planar_q8_0(dY, planar, dX, rows, K, NULL); break;
        }
    } else {
        rc = dev_gemv(fmt, dY, dW, dX, rows, K);
    }
    if (rc != 0) return;
    /* the Q4_K kernels (unless the ring variant was asked for) and the planar kernels have no bounded wait; the ring kernels that
     * read the other formats in the reference layout do */
    if ((fmt == F_Q4K && ckb200_tune_get("gemv_q4_k", 0) != 1) || planar) ckb_finish_out_nowait(y + r0, dY, (size_t)rows * sizeof(float), back);
    else ckb_finish_out(y + r0, dY, (size_t)rows * sizeof(float), back);
}

static void host_gemv(int fmt, float *y, const void *W, const void *x_q8, int M, int K)
{
    host_gemv_rows(fmt, y, W, x_q8, M, K, 0, M);
}

/* The reference's thread-split variants compute rows [dr*ith, min(dr*(ith+1), M)), dr = ceil(M/nth)
 * (src/kernels/gemm_kernels_q4k_q8k.c:212-243).  Same row range here; the GPU does the splitting inside. */
static void host_gemv_part(int fmt, float *y, const void *W, const void *x_q8, int M, int K, int ith, int nth)
{
    if (M <= 0 || ith < 0 || nth <= 0 || ith >= nth) return;
    const int dr = (M + nth - 1) / nth, r0 = dr * ith;
    if (r0 >= M) return;
    const int r1 = r0 + dr < M ? r0 + dr : M;
    host_gemv_rows(fmt, y, W, x_q8, M, K, r0, r1);
}

#define GEMV_FAMILY(fmt, base)                                                                                           \
    void base(float *y, const void *W, const void *x_q8, int M, int K) { host_gemv(fmt, y, W, x_q8, M, K); }             \
    void base##_parallel_dispatch(float *y, const void *W, const void *x_q8, int M, int K) { host_gemv(fmt, y, W, x_q8, M, K); } \
    void base##_parallel(float *y, const void *W, const void *x_q8, int M, int K, int ith, int nth)                      \
    { host_gemv_part(fmt, y, W, x_q8, M, K, ith, nth); }                                                                 \
    void base##_parallel_simd(float *y, const void *W, const void *x_q8, int M, int K, int ith, int nth)                 \
    { host_gemv_part(fmt, y, W, x_q8, M, K, ith, nth); }

GEMV_FAMILY(F_Q4K, gemv_q4_k_q8_k)
GEMV_FAMILY(F_Q6K, gemv_q6_k_q8_k)
GEMV_FAMILY(F_Q80, gemv_q8_0_q8_0)

/* ISA-named variants of the reference all compute the same function */
void gemv_q4_k_q8_k_ref(float *y, const void *W, const void *x_q8, int M, int K) { host_gemv(F_Q4K, y, W, x_q8, M, K); }
void gemv_q4_k_q8_k_avx(float *y, const void *W, const void *x_q8, int M, int K) { host_gemv(F_Q4K, y, W, x_q8, M, K); }
void gemv_q4_k_q8_k_avx2(float *y, const void *W, const void *x_q8, int M, int K) { host_gemv(F_Q4K, y, W, x_q8, M, K); }
void gemv_q4_k_q8_k_vnni(float *y, const void *W, const void *x_q8, int M, int K) { host_gemv(F_Q4K, y, W, x_q8, M, K); }
void gemv_q4_k_q8_k_sse(float *y, const void *W, const void *x_q8, int M, int K) { host_gemv(F_Q4K, y, W, x_q8, M, K); }
void gemv_q6_k_q8_k_ref(float *y, const void *W, const void *x_q8, int M, int K) { host_gemv(F_Q6K, y, W, x_q8, M, K); }

void vec_dot_q6_k_q8_k(int n, float *s, const void *vx, const void *vy)
{
    if (!s || !vx || !vy || n <= 0) return;
    host_gemv(F_Q6K, s, vx, vy, 1, n);
}
/* Q5_0 x Q8_0 (src/kernels/gemm_kernels_q5_0.c:901-939, :1602-1720): the reference has no plain _parallel form for this pair */
void gemv_q5_0_q8_0(float *y, const void *W, const void *x_q8, int M, int K) { host_gemv(F_Q50, y, W, x_q8, M, K); }
void gemv_q5_0_q8_0_parallel_simd(float *y, const void *W, const void *x_q8, int M, int K, int ith, int nth)
{ host_gemv_part(F_Q50, y, W, x_q8, M, K, ith, nth); }
void gemv_q5_0_q8_0_parallel_dispatch(float *y, const void *W, const void *x_q8, int M, int K) { host_gemv(F_Q50, y, W, x_q8, M, K); }
void vec_dot_q5_0_q8_0(int n, float *s, const void *vx, const void *vy)
{
    if (!s || !vx || !vy || n <= 0) return;
    host_gemv(F_Q50, s, vx, vy, 1, n);
}
void vec_dot_q5_0_q8_0_ref(int n, float *s, const void *vx, const void *vy) { vec_dot_q5_0_q8_0(n, s, vx, vy); }

void vec_dot_q8_0_q8_0(int n, float *s, const void *vx, const void *vy)
{
    if (!s || !vx || !vy || n <= 0) return;
    host_gemv(F_Q80, s, vx, vy, 1, n);
}

void ck_parallel_decode_init(void) { ckb_ensure_init(); }
void ck_parallel_decode_shutdown(void) {}
void ck_parallel_prefill_init(void) { ckb_ensure_init(); }
void ck_parallel_prefill_shutdown(void) {}

/* ------------------------------------------------------------------ GEMM (batched GEMV semantics) */

/* gemm_nt: C[m][n] = dot(B row n, A_q8 row m) + bias[n]   (src/kernels/gemm_kernels_q4k_q8k.c:301-326)
 * gemm:    Y[n][m] = dot(W row m, X_q8 row n)             (:283-299) - same thing with the roles named differently. */
static void host_gemm_nt(int fmt, const void *A_q8, const void *B, const float *bias, float *C, int M, int N, int K)
{
    if (!A_q8 || !B || !C || M <= 0 || N <= 0 || K <= 0) return;
    if (ckb_ensure_init()) return;
    const size_t a_b = (size_t)M * xq_bytes(fmt, K), b_b = (size_t)N * w_row_bytes(fmt, K), c_b = (size_t)M * N * sizeof(float);
    const void *dA = ckb_stage_in(A_q8, a_b, CKB_SLOT_A, 0);
    const void *dB = ckb_stage_in(B, b_b, CKB_SLOT_W, 1);
    const float *dbias = bias ? (const float *)ckb_stage_in(bias, (size_t)N * sizeof(float), CKB_SLOT_B, 1) : NULL;
    int back;
    float *dC = (float *)ckb_stage_out(C, c_b, CKB_SLOT_C, &back);
    if (!dA || !dB || !dC || (bias && !dbias)) return;
    int rc;
    switch (fmt) {
        case F_Q4K: rc = ckb200_dev_gemm_nt_q4_k_q8_k(dA, dB, dbias, dC, M, N, K, NULL); break;
        case F_Q6K: {
            /* resident weights: the tensor-core kernel over their row-planar copy; others are re-laid per call inside the device entry */
            const void *planar = ckb200_device_ptr(B) == dB ? ckb_planar_shadow(F_Q6K, dB, N, K) : NULL;
            rc = planar ? ckb200_dev_gemm_nt_q6_k_planar_q8_k(dA, planar, dbias, dC, M, N, K, NULL) : ckb200_dev_gemm_nt_q6_k_q8_k(dA, dB, dbias, dC, M, N, K, NULL);
            break;
        }
        case F_Q50: rc = ckb200_dev_gemm_nt_q5_0_q8_0(dA, dB, dbias, dC, M, N, K, NULL); break;
        default: {
            const void *planar = ckb200_device_ptr(B) == dB ? ckb_planar_shadow(F_Q80, dB, N, K) : NULL;
            rc = planar ? ckb_gemm_nt_q80_tc(dA, NULL, planar, dbias, dC, M, N, K, NULL) : -1;
            if (rc < 0) rc = ckb200_dev_gemm_nt_q8_0_q8_0(dA, dB, dbias, dC, M, N, K, NULL);
            break;
        }
    }
    if (rc != 0) return;
    ckb_finish_out(C, dC, c_b, back);
}

void gemm_nt_q4_k_q8_k(const void *A_q8, const void *B, const float *bias, float *C, int M, int N, int K) { host_gemm_nt(F_Q4K, A_q8, B, bias, C, M, N, K); }
void gemm_nt_q6_k_q8_k(const void *A_q8, const void *B, const float *bias, float *C, int M, int N, int K) { host_gemm_nt(F_Q6K, A_q8, B, bias, C, M, N, K); }
void gemm_nt_q8_0_q8_0(const void *A_q8, const void *B, const float *bias, float *C, int M, int N, int K) { host_gemm_nt(F_Q80, A_q8, B, bias, C, M, N, K); }
void gemm_nt_q5_0_q8_0(const void *A_q8, const void *B, const float *bias, float *C, int M, int N, int K) { host_gemm_nt(F_Q50, A_q8, B, bias, C, M, N, K); }
void gemm_nt_q6_k_q8_k_parallel_dispatch(const void *A_q8, const void *B, const float *bias, float *C, int M, int N, int K) { host_gemm_nt(F_Q6K, A_q8, B, bias, C, M, N, K); }
void gemm_nt_q8_0_q8_0_parallel_dispatch(const void *A_q8, const void *B, const float *bias, float *C, int M, int N, int K) { host_gemm_nt(F_Q80, A_q8, B, bias, C, M, N, K); }
void gemm_q4_k_q8_k(float *Y, const void *W, const void *X_q8, int M, int N, int K) { host_gemm_nt(F_Q4K, X_q8, W, NULL, Y, N, M, K); }
void gemm_q4_k_q8_k_ref(float *Y, const void *W, const void *X_q8, int M, int N, int K) { host_gemm_nt(F_Q4K, X_q8, W, NULL, Y, N, M, K); }
void gemm_q6_k_q8_k(float *Y, const void *W, const void *X_q8, int M, int N, int K) { host_gemm_nt(F_Q6K, X_q8, W, NULL, Y, N, M, K); }

/* ------------------------------------------------------------------ fp32-activation GEMV + row dequant */

static void host_gemv_f32(int fmt, float *y, const void *W, const float *x, int M, int K)
{
    if (!y || !W || !x || M <= 0 || K <= 0) return;
    if (ckb_ensure_init()) return;
    const void *dW = ckb_stage_in(W, (size_t)M * w_row_bytes(fmt, K), CKB_SLOT_W, 1);
    const float *dX = (const float *)ckb_stage_in(x, (size_t)K * sizeof(float), CKB_SLOT_X, 0);
    int back;
    float *dY = (float *)ckb_stage_out(y, (size_t)M * sizeof(float), CKB_SLOT_Y, &back);
    if (!dW || !dX || !dY) return;
    int rc;
    switch (fmt) {
        case F_Q4K: rc = ckb200_dev_gemv_q4_k(dY, dW, dX, M, K, NULL); break;
        case F_Q6K: rc = ckb200_dev_gemv_q6_k(dY, dW, dX, M, K, NULL); break;
        case F_Q50: rc = ckb200_dev_gemv_q5_0(dY, dW, dX, M, K, NULL); break;
        default: rc = ckb200_dev_gemv_q8_0(dY, dW, dX, M, K, NULL); break;
    }
    if (rc != 0) return;
    ckb_finish_out(y, dY, (size_t)M * sizeof(float), back);
}

void gemv_q4_k(float *y, const void *W, const float *x, int M, int K) { host_gemv_f32(F_Q4K, y, W, x, M, K); }
void gemv_q6_k(float *y, const void *W, const float *x, int M, int K) { host_gemv_f32(F_Q6K, y, W, x, M, K); }
void gemv_q8_0(float *y, const void *W, const float *x, int M, int K) { host_gemv_f32(F_Q80, y, W, x, M, K); }
void gemv_q8_0_ref(float *y, const void *W, const float *x, int M, int K) { host_gemv_f32(F_Q80, y, W, x, M, K); }
/* fp32-activation Q5_0 (src/kernels/gemm_kernels_q5_0.c:67-111, :550-567) */
void gemv_q5_0(float *y, const void *W, const float *x, int M, int K) { host_gemv_f32(F_Q50, y, W, x, M, K); }
void gemv_q5_0_ref(float *y, const void *W, const float *x, int M, int K) { host_gemv_f32(F_Q50, y, W, x, M, K); }

static void host_dequant(int fmt, const void *src, float *dst, size_t n)
{
    if (!src || !dst || n == 0) return;
    if (ckb_ensure_init()) return;
    const size_t in_b = fmt == F_Q80 ? (n / 32) * Q80_B : (fmt == F_Q50 ? (n / 32) * 22 : (n / 256) * (fmt == F_Q4K ? Q4K_B : Q6K_B));
    const void *ds = ckb_stage_in(src, in_b, CKB_SLOT_W, 1);
    int back;
    float *dd = (float *)ckb_stage_out(dst, n * sizeof(float), CKB_SLOT_Y, &back);
    if (!ds || !dd) return;
    int rc;
    switch (fmt) {
        case F_Q4K: rc = ckb200_dev_dequant_q4_k_row(ds, dd, n, NULL); break;
        case F_Q6K: rc = ckb200_dev_dequant_q6_k_row(ds, dd, n, NULL); break;
        case F_Q50: rc = ckb200_dev_dequant_q5_0_row(ds, dd, n, NULL); break;
        default: rc = ckb200_dev_dequant_q8_0_row(ds, dd, n, NULL); break;
    }
    if (rc != 0) return;
    ckb_finish_out(dst, dd, n * sizeof(float), back);
}

void dequant_q4_k_row(const void *src, float *dst, size_t n_elements) { host_dequant(F_Q4K, src, dst, n_elements); }
void dequant_q6_k_row(const void *src, float *dst, size_t n_elements) { host_dequant(F_Q6K, src, dst, n_elements); }
void dequant_q8_0_row(const void *src, float *dst, size_t n_elements) { host_dequant(F_Q80, src, dst, n_elements); }
void dequant_q5_0_row(const void *src, float *dst, size_t n_elements) { host_dequant(F_Q50, src, dst, n_elements); }   /* src/kernels/dequant_kernels.c:198-206 */

/* ------------------------------------------------------------------ attention + KV cache */

void attention_forward_decode_head_major_gqa_flash(const float *q_token, const float *k_cache, const float *v_cache,
                                                   float *out_token, int num_heads, int num_kv_heads, int kv_tokens,
                                                   int cache_capacity, int head_dim, int aligned_head_dim)
{
    if (!q_token || !k_cache || !v_cache || !out_token) return;
    if (num_heads <= 0 || num_kv_heads <= 0 || kv_tokens <= 0 || cache_capacity <= 0) return;
    if (kv_tokens > cache_capacity || head_dim <= 0 || aligned_head_dim <= 0) return;
    if (ckb_ensure_init()) return;
    const size_t q_b = (size_t)num_heads * aligned_head_dim * sizeof(float);
    const size_t kv_b = (size_t)num_kv_heads * cache_capacity * aligned_head_dim * sizeof(float);
    const float *dq = (const float *)ckb_stage_in(q_token, q_b, CKB_SLOT_X, 0);
    const float *dk = (const float *)ckb_stage_in(k_cache, kv_b, CKB_SLOT_A, 0);
    const float *dv = (const float *)ckb_stage_in(v_cache, kv_b, CKB_SLOT_B, 0);
    int back;
    float *dout = (float *)ckb_stage_out(out_token, q_b, CKB_SLOT_Y, &back);
    if (!dq || !dk || !dv || !dout) return;
    if (ckb200_dev_attention_decode(dq, dk, dv, dout, 1, 0, num_heads, num_kv_heads, kv_tokens, cache_capacity, head_dim,
                                    aligned_head_dim, NULL) != 0) return;
    ckb_finish_out(out_token, dout, q_b, back);
}

/* Prefill attention, host pointers (src/kernels/attention_kernels.c:2924-3005): q/out [H][T][ad], k/v [Hkv][stride][ad]. */
static void host_attention_prefill(const float *q, const float *k, const float *v, float *output, int num_heads, int num_kv_heads,
                                   int num_tokens, int head_dim, int aligned_head_dim, int kv_stride_tokens, int causal, int window)
{
    if (!q || !k || !v || !output) return;
    if (num_heads <= 0 || num_kv_heads <= 0 || num_tokens <= 0 || kv_stride_tokens < num_tokens) return;
    if (head_dim <= 0 || aligned_head_dim < head_dim) return;
    if (ckb_ensure_init()) return;
    const size_t q_b = (size_t)num_heads * num_tokens * aligned_head_dim * sizeof(float);
    const size_t kv_b = (size_t)num_kv_heads * kv_stride_tokens * aligned_head_dim * sizeof(float);
    const float *dq = (const float *)ckb_stage_in(q, q_b, CKB_SLOT_X, 0);
    const float *dk = (const float *)ckb_stage_in(k, kv_b, CKB_SLOT_A, 0);
    const float *dv = (const float *)ckb_stage_in(v, kv_b, CKB_SLOT_B, 0);
    int back;
    float *dout = (float *)ckb_stage_out(output, q_b, CKB_SLOT_Y, &back);
    if (!dq || !dk || !dv || !dout) return;
    if (ckb200_dev_attention_prefill_window(dq, dk, dv, dout, num_heads, num_kv_heads, num_tokens, head_dim, aligned_head_dim, kv_stride_tokens, causal,
                                            window, NULL) != 0) return;
    ckb_finish_out(output, dout, q_b, back);
}

void attention_forward_causal_head_major_gqa_flash(const float *q, const float *k, const float *v, float *output, int num_heads,
                                                   int num_kv_heads, int num_tokens, int head_dim, int aligned_head_dim)
{
    host_attention_prefill(q, k, v, output, num_heads, num_kv_heads, num_tokens, head_dim, aligned_head_dim, num_tokens, 1, 0);
}
void attention_forward_causal_head_major_gqa_flash_strided(const float *q, const float *k, const float *v, float *output, int num_heads,
                                                           int num_kv_heads, int num_tokens, int head_dim, int aligned_head_dim,
                                                           int kv_stride_tokens)
{
    host_attention_prefill(q, k, v, output, num_heads, num_kv_heads, num_tokens, head_dim, aligned_head_dim, kv_stride_tokens, 1, 0);
}
void attention_forward_full_head_major_gqa_flash(const float *q, const float *k, const float *v, float *output, int num_heads,
                                                 int num_kv_heads, int num_tokens, int head_dim, int aligned_head_dim)
{
    host_attention_prefill(q, k, v, output, num_heads, num_kv_heads, num_tokens, head_dim, aligned_head_dim, num_tokens, 0, 0);
}
void attention_forward_full_head_major_gqa_flash_strided(const float *q, const float *k, const float *v, float *output, int num_heads,
                                                         int num_kv_heads, int num_tokens, int head_dim, int aligned_head_dim,
                                                         int kv_stride_tokens)
{
    host_attention_prefill(q, k, v, output, num_heads, num_kv_heads, num_tokens, head_dim, aligned_head_dim, kv_stride_tokens, 0, 0);
}

/* sliding window (src/kernels/attention_kernels_sliding.c:450-600); a window <= 0 means no limit */
void attention_forward_causal_head_major_gqa_flash_strided_sliding(const float *q, const float *k, const float *v, float *output, int num_heads,
                                                                   int num_kv_heads, int num_tokens, int head_dim, int aligned_head_dim,
                                                                   int kv_stride_tokens, int sliding_window)
{
    host_attention_prefill(q, k, v, output, num_heads, num_kv_heads, num_tokens, head_dim, aligned_head_dim, kv_stride_tokens, 1, sliding_window);
}

void attention_forward_decode_head_major_gqa_flash_sliding(const float *q_token, const float *k_cache, const float *v_cache, float *out_token,
                                                           int num_heads, int num_kv_heads, int kv_tokens, int cache_capacity, int head_dim,
                                                           int aligned_head_dim, int sliding_window)
{
    if (!q_token || !k_cache || !v_cache || !out_token) return;
    if (num_heads <= 0 || num_kv_heads <= 0 || cache_capacity <= 0) return;
    if (kv_tokens <= 0 || kv_tokens > cache_capacity || head_dim <= 0 || aligned_head_dim <= 0) return;
    if (ckb_ensure_init()) return;
    const size_t q_b = (size_t)num_heads * aligned_head_dim * sizeof(float);
    const size_t kv_b = (size_t)num_kv_heads * cache_capacity * aligned_head_dim * sizeof(float);
    const float *dq = (const float *)ckb_stage_in(q_token, q_b, CKB_SLOT_X, 0);
    const float *dk = (const float *)ckb_stage_in(k_cache, kv_b, CKB_SLOT_A, 0);
    const float *dv = (const float *)ckb_stage_in(v_cache, kv_b, CKB_SLOT_B, 0);
    int back;
    float *dout = (float *)ckb_stage_out(out_token, q_b, CKB_SLOT_Y, &back);
    if (!dq || !dk || !dv || !dout) return;
    if (ckb200_dev_attention_decode_sliding(dq, dk, dv, dout, 1, 0, num_heads, num_kv_heads, kv_tokens, cache_capacity, head_dim, aligned_head_dim,
                                            sliding_window, NULL) != 0) return;
    ckb_finish_out(out_token, dout, q_b, back);
}

/* the llama template's attention (src/kernels/attention_kernels.c:3006-3046, :3408-3448) */
void attention_forward_decode_head_major_gqa_flash_f16kv(const float *q_token, const float *k_cache, const float *v_cache, float *out_token,
                                                         int num_heads, int num_kv_heads, int kv_tokens, int cache_capacity, int head_dim,
                                                         int aligned_head_dim)
{
    if (!q_token || !k_cache || !v_cache || !out_token) return;
    if (num_heads <= 0 || num_kv_heads <= 0 || kv_tokens <= 0 || cache_capacity <= 0) return;
    if (kv_tokens > cache_capacity || head_dim <= 0 || aligned_head_dim <= 0) return;
    if (ckb_ensure_init()) return;
    const size_t q_b = (size_t)num_heads * aligned_head_dim * sizeof(float);
    const size_t kv_b = (size_t)num_kv_heads * cache_capacity * aligned_head_dim * sizeof(float);
    const float *dq = (const float *)ckb_stage_in(q_token, q_b, CKB_SLOT_X, 0);
    const float *dk = (const float *)ckb_stage_in(k_cache, kv_b, CKB_SLOT_A, 0);
    const float *dv = (const float *)ckb_stage_in(v_cache, kv_b, CKB_SLOT_B, 0);
    int back;
    float *dout = (float *)ckb_stage_out(out_token, q_b, CKB_SLOT_Y, &back);
    if (!dq || !dk || !dv || !dout) return;
    if (ckb200_dev_attention_decode_f16kv(dq, dk, dv, dout, num_heads, num_kv_heads, kv_tokens, cache_capacity, head_dim, aligned_head_dim, NULL, NULL) != 0)
        return;
    ckb_finish_out(out_token, dout, q_b, back);
}

void attention_forward_causal_head_major_gqa_flash_strided_f16kv(const float *q, const float *k, const float *v, float *output, int num_heads,
                                                                 int num_kv_heads, int num_tokens, int head_dim, int aligned_head_dim,
                                                                 int kv_stride_tokens)
{
    if (!q || !k || !v || !output) return;
    if (num_heads <= 0 || num_kv_heads <= 0 || num_tokens <= 0 || kv_stride_tokens < num_tokens) return;
    if (head_dim <= 0 || aligned_head_dim < head_dim) return;
    if (ckb_ensure_init()) return;
    const size_t q_b = (size_t)num_heads * num_tokens * aligned_head_dim * sizeof(float);
    const size_t kv_b = (size_t)num_kv_heads * kv_stride_tokens * aligned_head_dim * sizeof(float);
    const float *dq = (const float *)ckb_stage_in(q, q_b, CKB_SLOT_X, 0);
    const float *dk = (const float *)ckb_stage_in(k, kv_b, CKB_SLOT_A, 0);
    const float *dv = (const float *)ckb_stage_in(v, kv_b, CKB_SLOT_B, 0);
    int back;
    float *dout = (float *)ckb_stage_out(output, q_b, CKB_SLOT_Y, &back);
    if (!dq || !dk || !dv || !dout) return;
    if (ckb200_dev_attention_prefill_f16kv(dq, dk, dv, dout, num_heads, num_kv_heads, num_tokens, head_dim, aligned_head_dim, kv_stride_tokens, NULL) != 0) return;
    ckb_finish_out(output, dout, q_b, back);
}

/* attention_flash_decode(out, q, k, v, T_q, T_k, H, D_h, scale) (src/kernels/attention_flash_true.c:696-722) for the
 * decode case T_q = 1: out/q [H][D_h], k/v [T_k][H][D_h] token-major.  With H = 1 this is exactly one head of the
 * head-major cache, which is how the reference's decode entry point calls it. */
void attention_flash_decode(float *out, const float *q, const float *k, const float *v, int T_q, int T_k, int H, int D_h, float scale)
{
    if (!out || !q || !k || !v || T_q != 1 || T_k <= 0 || H != 1 || D_h <= 0) {
        if (out && q && k && v && (T_q != 1 || H != 1))
            ckb_fail(CKB_ERR_SHAPE, "attention_flash_decode: only T_q = 1, H = 1 (the decode call shape) is implemented");
        return;
    }
    /* scale = 1/sqrt(head_dim) -> head_dim = round(1/scale^2) */
    const float hd = 1.0f / (scale * scale);
    const int head_dim = (int)(hd + 0.5f);
    attention_forward_decode_head_major_gqa_flash(q, k, v, out, 1, 1, T_k, T_k, head_dim, D_h);
}

void kv_cache_write_head_major(const float *k_token, const float *v_token, float *k_cache, float *v_cache, int num_kv_heads,
                               int token_index, int cache_capacity, int head_dim, int aligned_head_dim)
{
    if (!k_token || !v_token || !k_cache || !v_cache) return;
    if (num_kv_heads <= 0 || token_index < 0 || cache_capacity <= 0) return;
    if (token_index >= cache_capacity || head_dim <= 0 || aligned_head_dim <= 0) return;
    if (ckb_ensure_init()) return;
    /* The cache lives on the host in this calling convention, so this is a strided host write:
     * only the touched rows travel (one aligned_head_dim row per head), through the device kernel. */
    const size_t tok_b = (size_t)num_kv_heads * aligned_head_dim * sizeof(float);
    float *stage = (float *)ckb_scratch(CKB_SLOT_T, 4 * tok_b);
    if (!stage) return;
    float *dk = stage, *dv = stage + num_kv_heads * aligned_head_dim;
    float *dkc = dv + num_kv_heads * aligned_head_dim, *dvc = dkc + num_kv_heads * aligned_head_dim;
    cudaStream_t st = ckb_stream(NULL);
    /* source rows are [h][aligned_head_dim]; only head_dim of each is meaningful, the rest is written as zero */
    if (ckb_check_cuda((int)cudaMemsetAsync(stage, 0, 4 * tok_b, st), "memset")) return;
    if (ckb_check_cuda((int)cudaMemcpy2DAsync(dk, aligned_head_dim * sizeof(float), k_token, aligned_head_dim * sizeof(float),
                                              head_dim * sizeof(float), num_kv_heads, cudaMemcpyHostToDevice, st), "H2D k")) return;
    if (ckb_check_cuda((int)cudaMemcpy2DAsync(dv, aligned_head_dim * sizeof(float), v_token, aligned_head_dim * sizeof(float),
                                              head_dim * sizeof(float), num_kv_heads, cudaMemcpyHostToDevice, st), "H2D v")) return;
    /* device-side store into a one-token cache [Hkv][1][ad], then scatter the rows back to the host cache */
    if (ckb200_dev_kv_cache_store(dkc, dvc, dk, dv, 0, NULL, num_kv_heads, aligned_head_dim, 1, NULL) != 0) return;
    const size_t head_stride = (size_t)cache_capacity * aligned_head_dim;
    if (ckb_check_cuda((int)cudaMemcpy2DAsync(k_cache + (size_t)token_index * aligned_head_dim, head_stride * sizeof(float), dkc,
                                              aligned_head_dim * sizeof(float), aligned_head_dim * sizeof(float), num_kv_heads,
                                              cudaMemcpyDeviceToHost, st), "D2H k")) return;
    if (ckb_check_cuda((int)cudaMemcpy2DAsync(v_cache + (size_t)token_index * aligned_head_dim, head_stride * sizeof(float), dvc,
                                              aligned_head_dim * sizeof(float), aligned_head_dim * sizeof(float), num_kv_heads,
                                              cudaMemcpyDeviceToHost, st), "D2H v")) return;
    ckb_check_cuda((int)cudaStreamSynchronize(st), "sync");
}

void kv_cache_store(float *kv_cache_k, float *kv_cache_v, const float *k, const float *v, int layer, int pos, int num_kv_heads,
                    int head_dim, int max_seq_len)
{
    (void)layer;
    kv_cache_write_head_major(k, v, kv_cache_k, kv_cache_v, num_kv_heads, pos, max_seq_len, head_dim, head_dim);
}

/* fp16 KV cache (src/kernels/kv_cache_kernels.c:131-163, src/kernels/attention_kernels.c:3450-3557): k, v [Hkv][head_dim]
 * fp32 -> cache[Hkv][max_seq_len][head_dim] IEEE half at pos; only the touched rows travel. */
void kv_cache_store_f16(uint16_t *kv_cache_k, uint16_t *kv_cache_v, const float *k, const float *v, int layer, int pos, int num_kv_heads,
                        int head_dim, int max_seq_len)
{
    (void)layer;
    if (!kv_cache_k || !kv_cache_v || !k || !v) return;
    if (num_kv_heads <= 0 || pos < 0 || head_dim <= 0 || max_seq_len <= 0 || pos >= max_seq_len) return;
    if (ckb_ensure_init()) return;
    const size_t tok_b = (size_t)num_kv_heads * head_dim * sizeof(float);
    const float *dk = (const float *)ckb_stage_in(k, tok_b, CKB_SLOT_X, 0);
    const float *dv = (const float *)ckb_stage_in(v, tok_b, CKB_SLOT_A, 0);
    uint16_t *stage = (uint16_t *)ckb_scratch(CKB_SLOT_T, tok_b);            /* two one-token fp16 caches [Hkv][1][d] */
    if (!dk || !dv || !stage) return;
    uint16_t *dkc = stage, *dvc = stage + (size_t)num_kv_heads * head_dim;
    if (ckb200_dev_kv_cache_store_f16(dkc, dvc, dk, dv, 0, NULL, num_kv_heads, head_dim, 1, NULL) != 0) return;
    cudaStream_t st = ckb_stream(NULL);
    const size_t row = (size_t)head_dim * sizeof(uint16_t), pitch = (size_t)max_seq_len * row;
    if (ckb_check_cuda((int)cudaMemcpy2DAsync(kv_cache_k + (size_t)pos * head_dim, pitch, dkc, row, row, num_kv_heads, cudaMemcpyDefault, st), "fp16 k rows")) return;
    if (ckb_check_cuda((int)cudaMemcpy2DAsync(kv_cache_v + (size_t)pos * head_dim, pitch, dvc, row, row, num_kv_heads, cudaMemcpyDefault, st), "fp16 v rows")) return;
    ckb_check_cuda((int)cudaStreamSynchronize(st), "sync");
}

void attention_forward_decode_head_major_gqa_flash_f16cache(const float *q_token, const uint16_t *k_cache, const uint16_t *v_cache,
                                                            float *out_token, int num_heads, int num_kv_heads, int kv_tokens,
                                                            int cache_capacity, int head_dim, int aligned_head_dim)
{
    if (!q_token || !k_cache || !v_cache || !out_token) return;
    if (num_heads <= 0 || num_kv_heads <= 0 || kv_tokens <= 0 || cache_capacity <= 0) return;
    if (kv_tokens > cache_capacity || head_dim <= 0 || aligned_head_dim <= 0) return;
    if (ckb_ensure_init()) return;
    const size_t q_b = (size_t)num_heads * aligned_head_dim * sizeof(float);
    const size_t kv_b = (size_t)num_kv_heads * cache_capacity * aligned_head_dim * sizeof(uint16_t);
    const float *dq = (const float *)ckb_stage_in(q_token, q_b, CKB_SLOT_X, 0);
    const uint16_t *dk = (const uint16_t *)ckb_stage_in(k_cache, kv_b, CKB_SLOT_A, 0);
    const uint16_t *dv = (const uint16_t *)ckb_stage_in(v_cache, kv_b, CKB_SLOT_B, 0);
    int back;
    float *dout = (float *)ckb_stage_out(out_token, q_b, CKB_SLOT_Y, &back);
    if (!dq || !dk || !dv || !dout) return;
    if (ckb200_dev_attention_decode_f16cache(dq, dk, dv, dout, 1, 0, num_heads, num_kv_heads, kv_tokens, cache_capacity, head_dim,
                                             aligned_head_dim, NULL) != 0) return;
    ckb_finish_out(out_token, dout, q_b, back);
}

/* ------------------------------------------------------------------ glue ops */

void rmsnorm_forward(const float *input, const float *gamma, float *output, float *rstd_cache, int tokens, int d_model,
                     int aligned_embed_dim, float eps)
{
    if (!input || !gamma || !output || tokens <= 0 || d_model <= 0) return;
    if (ckb_ensure_init()) return;
    const size_t b = (size_t)tokens * aligned_embed_dim * sizeof(float);
    const float *din = (const float *)ckb_stage_in(input, b, CKB_SLOT_X, 0);
    const float *dg = (const float *)ckb_stage_in(gamma, (size_t)d_model * sizeof(float), CKB_SLOT_B, 1);
    int back, back_r = 0;
    float *dout = (float *)ckb_stage_out(output, b, CKB_SLOT_Y, &back);
    float *dr = rstd_cache ? (float *)ckb_stage_out(rstd_cache, (size_t)tokens * sizeof(float), CKB_SLOT_T, &back_r) : NULL;
    if (!din || !dg || !dout) return;
    if (ckb200_dev_rmsnorm_forward(din, dg, dout, dr, tokens, d_model, aligned_embed_dim, eps, NULL) != 0) return;
    if (dr && back_r) cudaMemcpyAsync(rstd_cache, dr, (size_t)tokens * sizeof(float), cudaMemcpyDeviceToHost, ckb_stream(NULL));
    ckb_finish_out(output, dout, b, back);
}

void rope_precompute_cache_split(float *cos_cache, float *sin_cache, int max_seq_len, int head_dim, float base)
{
    if (!cos_cache || !sin_cache || max_seq_len <= 0 || head_dim <= 1) return;
    if (ckb_ensure_init()) return;
    const size_t b = (size_t)max_seq_len * (head_dim / 2) * sizeof(float);
    int bc, bs;
    float *dc = (float *)ckb_stage_out(cos_cache, b, CKB_SLOT_A, &bc);
    float *ds = (float *)ckb_stage_out(sin_cache, b, CKB_SLOT_B, &bs);
    if (!dc || !ds) return;
    if (ckb200_dev_rope_precompute_cache_split(dc, ds, max_seq_len, head_dim, base, NULL) != 0) return;
    if (bc) cudaMemcpyAsync(cos_cache, dc, b, cudaMemcpyDeviceToHost, ckb_stream(NULL));
    ckb_finish_out(sin_cache, ds, b, bs);
}

void rope_forward_qk(float *q, float *k, const float *cos_cache, const float *sin_cache, int num_heads, int num_kv_heads,
                     int num_tokens, int head_dim, int aligned_head_dim, int pos_offset)
{
    if (!q || !k || !cos_cache || !sin_cache || num_heads <= 0 || num_kv_heads <= 0 || num_tokens <= 0 || head_dim <= 1) return;
    if (ckb_ensure_init()) return;
    const size_t qb = (size_t)num_heads * num_tokens * aligned_head_dim * sizeof(float);
    const size_t kb = (size_t)num_kv_heads * num_tokens * aligned_head_dim * sizeof(float);
    const size_t cb = (size_t)(pos_offset + num_tokens) * (head_dim / 2) * sizeof(float);
    float *dq = (float *)ckb_stage_in(q, qb, CKB_SLOT_X, 0);
    float *dk = (float *)ckb_stage_in(k, kb, CKB_SLOT_Y, 0);
    const float *dc = (const float *)ckb_stage_in(cos_cache, cb, CKB_SLOT_A, 1);
    const float *ds = (const float *)ckb_stage_in(sin_cache, cb, CKB_SLOT_B, 1);
    if (!dq || !dk || !dc || !ds) return;
    if (ckb200_dev_rope_forward_qk(dq, dk, dc, ds, num_heads, num_kv_heads, num_tokens, head_dim, aligned_head_dim, pos_offset,
                                   NULL, NULL) != 0) return;
    if (dq != q) cudaMemcpyAsync(q, dq, qb, cudaMemcpyDeviceToHost, ckb_stream(NULL));
    ckb_finish_out(k, dk, kb, dk != k);
}

void swiglu_forward(const float *input, float *output, int tokens, int dim)
{
    if (!input || !output || tokens <= 0 || dim <= 0) return;
    if (ckb_ensure_init()) return;
    const size_t ib = (size_t)tokens * 2 * dim * sizeof(float), ob = (size_t)tokens * dim * sizeof(float);
    const float *din = (const float *)ckb_stage_in(input, ib, CKB_SLOT_X, 0);
    int back;
    float *dout = (float *)ckb_stage_out(output, ob, CKB_SLOT_Y, &back);
    if (!din || !dout) return;
    if (ckb200_dev_swiglu_forward(din, dout, tokens, dim, NULL) != 0) return;
    ckb_finish_out(output, dout, ob, back);
}

void ck_residual_add_token_major(const float *a, const float *b, float *out, int tokens, int aligned_embed_dim)
{
    if (!a || !b || !out || tokens <= 0 || aligned_embed_dim <= 0) return;
    if (ckb_ensure_init()) return;
    const size_t n = (size_t)tokens * aligned_embed_dim * sizeof(float);
    const float *da = (const float *)ckb_stage_in(a, n, CKB_SLOT_A, 0);
    const float *db = (const float *)ckb_stage_in(b, n, CKB_SLOT_B, 0);
    int back;
    float *dout = (float *)ckb_stage_out(out, n, CKB_SLOT_Y, &back);
    if (!da || !db || !dout) return;
    if (ckb200_dev_residual_add(da, db, dout, tokens, aligned_embed_dim, NULL) != 0) return;
    ckb_finish_out(out, dout, n, back);
}

static void host_embedding(int fmt, const int32_t *ids, int count, int vocab, const void *table, const float *pos_emb,
                           float *out, int embed, int aligned, int ctx, int add_pos)
{
    if (!ids || !table || !out || ctx <= 0 || aligned <= 0) return;
    if (ckb_ensure_init()) return;
    int n = count < 0 ? 0 : (count > ctx ? ctx : count);
    const size_t blk = fmt == F_Q80 ? 32 : 256;
    const size_t row_b = ((aligned + blk - 1) / blk) * (fmt == F_Q4K ? Q4K_B : (fmt == F_Q6K ? Q6K_B : Q80_B));
    const size_t ob = (size_t)ctx * aligned * sizeof(float);
    const void *dt = ckb_stage_in(table, (size_t)vocab * row_b, CKB_SLOT_W, 1);
    const int32_t *di = (const int32_t *)ckb_stage_in(ids, (size_t)(n > 0 ? n : 1) * sizeof(int32_t), CKB_SLOT_X, 0);
    const float *dp = (add_pos && pos_emb) ? (const float *)ckb_stage_in(pos_emb, (size_t)n * aligned * sizeof(float), CKB_SLOT_A, 1) : NULL;
    int back;
    float *dout = (float *)ckb_stage_out(out, ob, CKB_SLOT_Y, &back);
    if (!dt || !di || !dout) return;
    int rc;
    switch (fmt) {
        case F_Q4K: rc = ckb200_dev_embedding_forward_q4_k(di, n, vocab, dt, dp, dout, embed, aligned, ctx, add_pos, NULL); break;
        case F_Q6K: rc = ckb200_dev_embedding_forward_q6_k(di, n, vocab, dt, dp, dout, embed, aligned, ctx, add_pos, NULL); break;
        default: rc = ckb200_dev_embedding_forward_q8_0(di, n, vocab, dt, dp, dout, embed, aligned, ctx, add_pos, NULL); break;
    }
    if (rc != 0) return;
    ckb_finish_out(out, dout, ob, back);
}

void embedding_forward_q4_k(const int32_t *token_ids, int token_count, int vocab_size, const void *token_embeddings,
                            const float *pos_embeddings, float *output, int embed_dim, int aligned_embed_dim, int context_window, int add_pos)
{ host_embedding(F_Q4K, token_ids, token_count, vocab_size, token_embeddings, pos_embeddings, output, embed_dim, aligned_embed_dim, context_window, add_pos); }
void embedding_forward_q6_k(const int32_t *token_ids, int token_count, int vocab_size, const void *token_embeddings,
                            const float *pos_embeddings, float *output, int embed_dim, int aligned_embed_dim, int context_window, int add_pos)
{ host_embedding(F_Q6K, token_ids, token_count, vocab_size, token_embeddings, pos_embeddings, output, embed_dim, aligned_embed_dim, context_window, add_pos); }
void embedding_forward_q8_0(const int32_t *token_ids, int token_count, int vocab_size, const void *token_embeddings,
                            const float *pos_embeddings, float *output, int embed_dim, int aligned_embed_dim, int context_window, int add_pos)
{ host_embedding(F_Q80, token_ids, token_count, vocab_size, token_embeddings, pos_embeddings, output, embed_dim, aligned_embed_dim, context_window, add_pos); }
