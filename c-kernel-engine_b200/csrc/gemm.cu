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

extern "C" int ckb200_dev_gemm_nt_q4_k_q8_k(const void *A_q8, const void *B, const float *bias, float *C, int M, int N, int K, void *stream)
{
    if (A_q8 && B && C && M > 0 && N > 0 && K > 0) {
        const int rc = ckb_launch_gemm_q4k_tc(A_q8, B, bias, C, M, N, K, stream);
        if (rc >= 0) return rc;
    }
    return gemm_nt_by_rows(ckb200_dev_gemv_q4_k_q8_k, (size_t)(K / 256) * ckb::Q8K_BYTES, A_q8, B, bias, C, M, N, K, stream);
}
extern "C" int ckb200_dev_gemm_nt_q6_k_q8_k(const void *A_q8, const void *B, const float *bias, float *C, int M, int N, int K, void *stream)
{
    return gemm_nt_by_rows(ckb200_dev_gemv_q6_k_q8_k, (size_t)(K / 256) * ckb::Q8K_BYTES, A_q8, B, bias, C, M, N, K, stream);
}
extern "C" int ckb200_dev_gemm_nt_q8_0_q8_0(const void *A_q8, const void *B, const float *bias, float *C, int M, int N, int K, void *stream)
{
    return gemm_nt_by_rows(ckb200_dev_gemv_q8_0_q8_0, (size_t)(K / 32) * ckb::Q80_BYTES, A_q8, B, bias, C, M, N, K, stream);
}

// gemm_nt_q5_0_q8_0 (src/kernels/gemm_kernels_q5_0.c:1725-1752): one GEMV per token, as the reference
extern "C" int ckb200_dev_gemv_q5_0_q8_0(float *, const void *, const void *, int, int, void *);
extern "C" int ckb200_dev_gemm_nt_q5_0_q8_0(const void *A_q8, const void *B, const float *bias, float *C, int M, int N, int K, void *stream)
{
    return gemm_nt_by_rows(ckb200_dev_gemv_q5_0_q8_0, (size_t)(K / 32) * ckb::Q80_BYTES, A_q8, B, bias, C, M, N, K, stream);
}
