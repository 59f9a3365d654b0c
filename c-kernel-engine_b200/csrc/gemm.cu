// Batched quantised GEMM C[M,N] = A_q8[M,K] . B[N,K]^T (+ bias): the prefill form of the dequant-dot
// kernels.  Replaces gemm_nt_q4_k_q8_k / gemm_nt_q6_k_q8_k / gemm_nt_q8_0_q8_0
// (src/kernels/gemm_kernels_q4k_q8k.c:301-326, src/kernels/gemm_kernels_q6k_q8k.c:1243-1268,
// src/kernels/gemm_batch_int8.c:87-120), which the reference computes as one GEMV per token.
//
// Small M (decode batches) runs the GEMV kernel once per token; weights then come from L2 after the
// first token when they fit.  Large M uses the tensor-core kernel in gemm_tc.cu when it applies.
#include "device_common.cuh"
#include "launch.h"
#include "runtime.h"

extern "C" int ckb200_dev_gemv_q4_k_q8_k(float *, const void *, const void *, int, int, void *);
extern "C" int ckb200_dev_gemv_q6_k_q8_k(float *, const void *, const void *, int, int, void *);
extern "C" int ckb200_dev_gemv_q8_0_q8_0(float *, const void *, const void *, int, int, void *);
extern "C" int ckb200_dev_add_bias_rows(float *, const float *, int, int, void *);
extern "C" int ckb_launch_gemm_q4k_tc(const void *, const void *, const float *, float *, int, int, int, void *);

typedef int (*gemv_fn)(float *, const void *, const void *, int, int, void *);

static int gemm_nt_by_rows(gemv_fn fn, size_t a_row_bytes, const void *A_q8, const void *B, const float *bias, float *C, int M,
                           int N, int K, void *stream)
{
    if (!A_q8 || !B || !C || M <= 0 || N <= 0 || K <= 0) return 0;
    for (int m = 0; m < M; ++m) {
        const int rc = fn(C + (size_t)m * N, B, (const uint8_t *)A_q8 + (size_t)m * a_row_bytes, N, K, stream);
        if (rc) return rc;
    }
    return bias ? ckb200_dev_add_bias_rows(C, bias, M, N, stream) : 0;
}

// Up to 64 tokens: the integer-MMA kernel that streams the weights through registers (gemm_q4k_mma.cu); above that the tcgen05 kernel.
extern "C" int ckb_launch_gemm_q4k_mma(const void *A_q8, const void *B, const float *bias, float *C, int ldc, int M, int N, int K, void *stream);
extern "C" int ckb200_dev_gemm_nt_q4_k_q8_k(const void *A_q8, const void *B, const float *bias, float *C, int M, int N, int K, void *stream)
{
    if (A_q8 && B && C && M > 0 && N > 0 && K > 0) {
        int rc = ckb_launch_gemm_q4k_mma(A_q8, B, bias, C, N, M, N, K, stream);
        if (rc >= 0) return rc;
        rc = ckb_launch_gemm_q4k_tc(A_q8, B, bias, C, M, N, K, stream);
        if (rc >= 0) return rc;
    }
    return gemm_nt_by_rows(ckb200_dev_gemv_q4_k_q8_k, (size_t)(K / 256) * ckb::Q8K_BYTES, A_q8, B, bias, C, M, N, K, stream);
}
// From 16 tokens up the reference's 210-byte rows are re-laid row-planar into the library's scratch (one pass over B, a few
// microseconds against the product itself) and the tensor-core kernel runs over that copy; the scratch belongs to the library's
// pool, so a caller that records its launches in a CUDA graph keeps its own planar copy and calls ckb200_dev_gemm_nt_q6_k_planar_q8_k.
extern "C" size_t ckb200_q6_k_planar_bytes(int rows, int cols);
extern "C" int ckb200_dev_q6_k_to_planar(void *dst, const void *src, int rows, int cols, void *stream);
extern "C" int ckb200_dev_gemm_nt_q6_k_planar_q8_k(const void *A_q8, const void *B_planar, const float *bias, float *C, int M, int N, int K, void *stream);
extern "C" int ckb200_dev_gemm_nt_q6_k_q8_k(const void *A_q8, const void *B, const float *bias, float *C, int M, int N, int K, void *stream)
{
    if (A_q8 && B && C && N > 0 && K > 0 && K % 256 == 0 && M >= ckb_tune_get("gemm_tc_min_tokens", 16) && ckb_tune_get("gemm_tc", 1) && !((uintptr_t)B & 1)) {
        const size_t bytes = ckb200_q6_k_planar_bytes(N, K);
        void *planar = bytes ? ckb_scratch(CKB_SLOT_P, bytes) : nullptr;
        if (planar) {
            const int rc = ckb200_dev_q6_k_to_planar(planar, B, N, K, stream);
            if (rc) return rc;
            return ckb200_dev_gemm_nt_q6_k_planar_q8_k(A_q8, planar, bias, C, M, N, K, stream);
        }
    }
    return gemm_nt_by_rows(ckb200_dev_gemv_q6_k_q8_k, (size_t)(K / 256) * ckb::Q8K_BYTES, A_q8, B, bias, C, M, N, K, stream);
}
// Q8_0 x Q8_0 from 16 tokens up: both operands are re-laid row-planar (the activations always, the weights unless the caller
// already has a planar copy) and the integer tensor-core kernel of gemm_q80_mma.cu reads every weight tile once per 128 tokens.
extern "C" size_t ckb200_q8_0_planar_bytes(int rows, int cols);
extern "C" int ckb200_dev_q8_0_to_planar(void *dst, const void *src, int rows, int cols, void *stream);
extern "C" int ckb_launch_gemm_q80_mma(const void *A_planar, const void *B_planar, const float *bias, float *C, int M, int N, int K, void *stream);

// B_planar may be NULL (then B_raw is converted into the library's scratch).  Returns -1 when the tensor-core path does not apply.
extern "C" int ckb_gemm_nt_q80_tc(const void *A_raw, const void *B_raw, const void *B_planar, const float *bias, float *C, int M, int N, int K, void *stream)
{
    if (!A_raw || !C || M < ckb_tune_get("gemm_tc_min_tokens", 16) || N <= 0 || K <= 0 || K % 128 || !ckb_tune_get("gemm_tc", 1)) return -1;
    if (((uintptr_t)A_raw & 1) || (!B_planar && (!B_raw || ((uintptr_t)B_raw & 1)))) return -1;
    const size_t a_bytes = (ckb200_q8_0_planar_bytes(M, K) + 255) & ~(size_t)255, b_bytes = B_planar ? 0 : ckb200_q8_0_planar_bytes(N, K);
    uint8_t *ws = (uint8_t *)ckb_scratch(CKB_SLOT_P, a_bytes + b_bytes);
    if (!ws) return CKB_ERR_CUDA;
    int rc = ckb200_dev_q8_0_to_planar(ws, A_raw, M, K, stream);
    if (!rc && !B_planar) {
        rc = ckb200_dev_q8_0_to_planar(ws + a_bytes, B_raw, N, K, stream);
        B_planar = ws + a_bytes;
    }
    if (rc) return rc;
    return ckb_launch_gemm_q80_mma(ws, B_planar, bias, C, M, N, K, stream);
}

extern "C" int ckb200_dev_gemm_nt_q8_0_q8_0(const void *A_q8, const void *B, const float *bias, float *C, int M, int N, int K, void *stream)
{
    if (A_q8 && B && C) {
        const int rc = ckb_gemm_nt_q80_tc(A_q8, B, nullptr, bias, C, M, N, K, stream);
        if (rc >= 0) return rc;
    }
    return gemm_nt_by_rows(ckb200_dev_gemv_q8_0_q8_0, (size_t)(K / 32) * ckb::Q80_BYTES, A_q8, B, bias, C, M, N, K, stream);
}

// gemm_nt_q5_0_q8_0 (src/kernels/gemm_kernels_q5_0.c:1725-1752): one GEMV per token, as the reference
extern "C" int ckb200_dev_gemv_q5_0_q8_0(float *, const void *, const void *, int, int, void *);
extern "C" int ckb200_dev_gemm_nt_q5_0_q8_0(const void *A_q8, const void *B, const float *bias, float *C, int M, int N, int K, void *stream)
{
    return gemm_nt_by_rows(ckb200_dev_gemv_q5_0_q8_0, (size_t)(K / 32) * ckb::Q80_BYTES, A_q8, B, bias, C, M, N, K, stream);
}
