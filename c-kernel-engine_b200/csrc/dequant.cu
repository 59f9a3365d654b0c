// Row dequantisers and the fp32-activation GEMVs built on them.
//
// dequant_q4_k_row / dequant_q6_k_row / dequant_q8_0_row follow src/kernels/dequant_kernels.c:276-430
// with the same rounding sequence (products and the Q4_K min subtraction are separate fp32
// operations, no FMA), so the rows are bit-identical to the reference's.
//
// gemv_q4_k / gemv_q6_k / gemv_q8_0 with fp32 activations (src/kernels/gemm_kernels_q4k.c:53-101,
// src/kernels/gemm_kernels_q6k.c:169-193, src/kernels/gemm_kernels_q8_0.c:254-277) are the
// reference's debug path; here they are a warp-per-row dequantise-and-FMA kernel, not tuned.
#include "dequant_elem.cuh"
#include "launch.h"
#include "runtime.h"

namespace ckb {

template <int FMT>
__global__ void dequant_rows_kernel(const uint8_t *__restrict__ src, float *__restrict__ dst, long long n)
{
    constexpr int BS = DqTraits<FMT>::BS, BE = DqTraits<FMT>::BE;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
        const long long b = i / BE;
        dst[i] = dequant_elem<FMT>(src + b * BS, (int)(i - b * BE));
    }
}

// y[row] = sum_e w(row, e) * x[e]; one warp per row, lanes stride the elements
template <int FMT>
__global__ void __launch_bounds__(256) gemv_f32_kernel(const uint8_t *__restrict__ W, const float *__restrict__ x,
                                                       float *__restrict__ y, int M, int K)
{
    constexpr int BS = DqTraits<FMT>::BS, BE = DqTraits<FMT>::BE;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = blockDim.x >> 5;
    const size_t rb = (size_t)(K / BE) * BS;
    for (int row = blockIdx.x * nw + warp; row < M; row += gridDim.x * nw) {
        const uint8_t *wr = W + row * rb;
        float acc = 0.0f;
        for (int e = lane; e < K; e += 32) {
            const int b = e / BE;
            acc = fmaf(dequant_elem<FMT>(wr + (size_t)b * BS, e - b * BE), x[e], acc);
        }
        acc = group_sum<32>(acc);
        if (lane == 0) y[row] = acc;
    }
}

__global__ void add_bias_rows_kernel(float *__restrict__ c, const float *__restrict__ bias, long long total, int n)
{
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x)
        c[i] += bias[i % n];
}

}  // namespace ckb

using namespace ckb;

template <int FMT>
static int launch_dequant(const void *src, float *dst, size_t n, void *stream)
{
    if (!src || !dst || n == 0) return 0;
    if (n % DqTraits<FMT>::BE) return ckb_fail(CKB_ERR_SHAPE, "dequant row: n=%zu is not a whole number of blocks", n);
    if (ckb_ensure_init()) return CKB_ERR_NO_DEVICE;
    const unsigned grid = (unsigned)((n + 255) / 256 < 4096 ? (n + 255) / 256 : 4096);
    dequant_rows_kernel<FMT><<<grid, 256, 0, ckb_stream(stream)>>>((const uint8_t *)src, dst, (long long)n);
    return ckb_check_launch("dequant_row");
}

extern "C" int ckb200_dev_dequant_q4_k_row(const void *src, float *dst, size_t n, void *stream) { return launch_dequant<DQ_Q4K>(src, dst, n, stream); }
extern "C" int ckb200_dev_dequant_q6_k_row(const void *src, float *dst, size_t n, void *stream) { return launch_dequant<DQ_Q6K>(src, dst, n, stream); }
extern "C" int ckb200_dev_dequant_q8_0_row(const void *src, float *dst, size_t n, void *stream) { return launch_dequant<DQ_Q80>(src, dst, n, stream); }
extern "C" int ckb200_dev_dequant_q5_0_row(const void *src, float *dst, size_t n, void *stream) { return launch_dequant<DQ_Q50>(src, dst, n, stream); }
extern "C" int ckb200_dev_dequant_q4_0_row(const void *src, float *dst, size_t n, void *stream) { return launch_dequant<DQ_Q40>(src, dst, n, stream); }
extern "C" int ckb200_dev_dequant_q4_1_row(const void *src, float *dst, size_t n, void *stream) { return launch_dequant<DQ_Q41>(src, dst, n, stream); }
extern "C" int ckb200_dev_dequant_q5_1_row(const void *src, float *dst, size_t n, void *stream) { return launch_dequant<DQ_Q51>(src, dst, n, stream); }

template <int FMT>
static int launch_gemv_f32(float *y, const void *W, const float *x, int M, int K, void *stream)
{
    if (!y || !W || !x || M <= 0 || K <= 0) return 0;
    if (K % DqTraits<FMT>::BE) return ckb_fail(CKB_ERR_SHAPE, "gemv (fp32 activations): K=%d is not a whole number of blocks", K);
    if (ckb_ensure_init()) return CKB_ERR_NO_DEVICE;
    const int grid = (M + 7) / 8 < 148 * 8 ? (M + 7) / 8 : 148 * 8;
    gemv_f32_kernel<FMT><<<grid, 256, 0, ckb_stream(stream)>>>((const uint8_t *)W, x, y, M, K);
    return ckb_check_launch("gemv_f32");
}

extern "C" int ckb200_dev_gemv_q4_k(float *y, const void *W, const float *x, int M, int K, void *stream) { return launch_gemv_f32<DQ_Q4K>(y, W, x, M, K, stream); }
extern "C" int ckb200_dev_gemv_q6_k(float *y, const void *W, const float *x, int M, int K, void *stream) { return launch_gemv_f32<DQ_Q6K>(y, W, x, M, K, stream); }
extern "C" int ckb200_dev_gemv_q8_0(float *y, const void *W, const float *x, int M, int K, void *stream) { return launch_gemv_f32<DQ_Q80>(y, W, x, M, K, stream); }
extern "C" int ckb200_dev_gemv_q5_0(float *y, const void *W, const float *x, int M, int K, void *stream) { return launch_gemv_f32<DQ_Q50>(y, W, x, M, K, stream); }
// gemv_q4_0 / gemv_q4_1 / gemv_q5_1 (src/kernels/gemm_kernels_q4_0.c:49-145, gemm_kernels_q4_1.c:50-152, gemm_kernels_q5_1.c:52-200) and the fp32
// fall-back of gemv_q5_k for rows that are not quantised (src/kernels/gemm_kernels_q5_k.c:211-245), each in its function's element order
extern "C" int ckb200_dev_gemv_q4_0(float *y, const void *W, const float *x, int M, int K, void *stream) { return launch_gemv_f32<DQ_Q40_G>(y, W, x, M, K, stream); }
extern "C" int ckb200_dev_gemv_q4_1(float *y, const void *W, const float *x, int M, int K, void *stream) { return launch_gemv_f32<DQ_Q41_G>(y, W, x, M, K, stream); }
extern "C" int ckb200_dev_gemv_q5_1(float *y, const void *W, const float *x, int M, int K, void *stream) { return launch_gemv_f32<DQ_Q51_G>(y, W, x, M, K, stream); }
extern "C" int ckb200_dev_gemv_q5_k_f32(float *y, const void *W, const float *x, int M, int K, void *stream) { return launch_gemv_f32<DQ_Q5K_F>(y, W, x, M, K, stream); }

extern "C" int ckb200_dev_add_bias_rows(float *c, const float *bias, int rows, int n, void *stream)
{
    if (!c || !bias || rows <= 0 || n <= 0) return 0;
    if (ckb_ensure_init()) return CKB_ERR_NO_DEVICE;
    const long long total = (long long)rows * n;
    const unsigned grid = (unsigned)((total + 255) / 256 < 2048 ? (total + 255) / 256 : 2048);
    add_bias_rows_kernel<<<grid, 256, 0, ckb_stream(stream)>>>(c, bias, total, n);
    return ckb_check_launch("add_bias_rows");
}
