// Quantised products of two further weight formats, each as the reference computes it:
//   Q5_K x Q8_K   gemv_q5_k_q8_k / gemm_nt_q5_k_q8_k   src/kernels/gemm_kernels_q5_k.c:128-208, :305-367
//   Q5_1 x Q8_1   gemv_q5_1_q8_1_ref / gemm_nt_q5_1_q8_1_ref, quantize to Q8_1   src/kernels/gemm_kernels_q5_1_q8_1.c:27-122
//
// Both are sums over blocks of (integer dot) x (fp32 scales) added in block order.  The integer parts are exact in any order; the fp32 part
// is done by one lane per row, block after block, with the reference's operations (no FMA), so the results are bit-identical to the scalar
// loops.  One warp per (row, token).  These formats are off the measured path: the kernels are written for parity, not for bandwidth (byte
// loads, one shuffle reduction per block).
#include "device_common.cuh"
#include "launch.h"
#include "runtime.h"

namespace ckb {

constexpr int Q5K_BYTES = 176, Q51_BYTES = 24, Q81_BYTES = 36;

// the 6-bit (scale, min) pair j of a K-quant scale field (src/kernels/gemm_kernels_q5_k.c:59-81)
__device__ __forceinline__ void k_scale_min(const uint8_t *s, int j, int &sc, int &mn)
{
    if (j < 4) {
        sc = s[j] & 63;
        mn = s[j + 4] & 63;
    } else {
        sc = (s[j + 4] & 15) | ((s[j - 4] >> 6) << 4);
        mn = (s[j + 4] >> 4) | ((s[j] >> 6) << 4);
    }
}

__device__ __forceinline__ int warp_sum_int(int v)
{
#pragma unroll
    for (int o = 16; o; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

// grid (row groups, tokens).  y[t * ldy + row] = sum_b d_b dx_b doti_b - dmin_b dx_b sumi_b (+ bias[row])
__global__ void __launch_bounds__(256) gemv_q5k_q8k_kernel(const uint8_t *__restrict__ W, const uint8_t *__restrict__ xq, const float *__restrict__ bias,
                                                           float *__restrict__ y, int ldy, int M, int nb)
{
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = blockDim.x >> 5;
    const uint8_t *xrow = xq + (size_t)blockIdx.y * nb * Q8K_BYTES;
    for (int row = blockIdx.x * nw + warp; row < M; row += gridDim.x * nw) {
        float acc = 0.0f;
        for (int b = 0; b < nb; ++b) {
            const uint8_t *w = W + ((size_t)row * nb + b) * Q5K_BYTES, *x = xrow + (size_t)b * Q8K_BYTES;
            const uint8_t *qh = w + 16, *qs = w + 48;
            const int8_t *q8 = reinterpret_cast<const int8_t *>(x + 4);
            // lane l is column l of every 32-element sub-block: sub-block sb = low (even) or high (odd) nibbles of qs[32 (sb / 2) + l], fifth bit = bit sb of qh[l]
            const uint32_t hbits = qh[lane];
            int part = 0;
#pragma unroll
            for (int sb = 0; sb < 8; ++sb) {
                int sc, mn;
                k_scale_min(w + 4, sb, sc, mn);
                const uint32_t byte = qs[32 * (sb >> 1) + lane];
                const int a = (int)((sb & 1) ? (byte >> 4) : (byte & 15u)) + (int)(((hbits >> sb) & 1u) << 4);
                part += sc * a * (int)q8[32 * sb + lane];
            }
            int mpart = 0;
            if (lane < 16) {
                int sc, mn;
                k_scale_min(w + 4, lane >> 1, sc, mn);
                mpart = (int)reinterpret_cast<const int16_t *>(x + 260)[lane] * mn;
            }
            const int doti = warp_sum_int(part), sumi = warp_sum_int(mpart);
            if (lane == 0) {
                const float xd = *reinterpret_cast<const float *>(x);
                const float d = __fmul_rn(half_bits_to_float(w[0] | (w[1] << 8)), xd), dmin = __fmul_rn(half_bits_to_float(w[2] | (w[3] << 8)), xd);
                acc = __fadd_rn(acc, __fsub_rn(__fmul_rn(d, (float)doti), __fmul_rn(dmin, (float)sumi)));
            }
        }
        if (lane == 0) y[(size_t)blockIdx.y * ldy + row] = bias ? __fadd_rn(acc, bias[row]) : acc;
    }
}

// one warp per 32-element block: d = amax / 127, q = roundf(x / d) (half away from zero), s = fp16(sum(q) * d)
__global__ void __launch_bounds__(256) quantize_q8_1_kernel(const float *__restrict__ x, uint8_t *__restrict__ y, long long nblocks)
{
    const int lane = threadIdx.x & 31;
    for (long long b = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5); b < nblocks; b += (long long)gridDim.x * (blockDim.x >> 5)) {
        const float v = x[b * 32 + lane];
        float amax = fabsf(v);
#pragma unroll
        for (int o = 16; o; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
        const float d = __fdiv_rn(amax, 127.0f), id = d != 0.0f ? __fdiv_rn(1.0f, d) : 0.0f;
        const int q = (int)roundf(__fmul_rn(v, id));
        const int sum = warp_sum_int(q);
        uint8_t *o = y + b * Q81_BYTES;
        reinterpret_cast<int8_t *>(o + 4)[lane] = (int8_t)q;
        if (lane == 0) {
            reinterpret_cast<uint16_t *>(o)[0] = __half_as_ushort(__float2half_rn(d));
            reinterpret_cast<uint16_t *>(o)[1] = __half_as_ushort(__float2half_rn(__fmul_rn((float)sum, d)));
        }
    }
}

// grid (row groups, tokens).  Lane b % 32 computes block b's value; lane 0 adds the values in block order.
__global__ void __launch_bounds__(256) gemv_q51_q81_kernel(const uint8_t *__restrict__ W, const uint8_t *__restrict__ xq, const float *__restrict__ bias,
                                                           float *__restrict__ y, int ldy, int M, int nb)
{
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = blockDim.x >> 5;
    const uint8_t *xrow = xq + (size_t)blockIdx.y * nb * Q81_BYTES;
    for (int row = blockIdx.x * nw + warp; row < M; row += gridDim.x * nw) {
        float acc = 0.0f;
        for (int b0 = 0; b0 < nb; b0 += 32) {
            const int b = b0 + lane;
            float val = 0.0f;
            if (b < nb) {
                const uint8_t *w = W + ((size_t)row * nb + b) * Q51_BYTES, *x = xrow + (size_t)b * Q81_BYTES;
                const uint32_t qh = w[4] | (w[5] << 8) | (w[6] << 16) | ((uint32_t)w[7] << 24);
                const int8_t *q8 = reinterpret_cast<const int8_t *>(x + 4);
                int si = 0;
#pragma unroll
                for (int j = 0; j < 16; ++j) {
                    const int q0 = (w[8 + j] & 15) | (int)(((qh >> j) & 1u) << 4), q1 = (w[8 + j] >> 4) | (int)(((qh >> (j + 16)) & 1u) << 4);
                    si += q0 * (int)q8[j] + q1 * (int)q8[j + 16];
                }
                const float wd = half_bits_to_float(w[0] | (w[1] << 8)), wm = half_bits_to_float(w[2] | (w[3] << 8));
                const float xd = half_bits_to_float(x[0] | (x[1] << 8)), xs = half_bits_to_float(x[2] | (x[3] << 8));
                val = __fadd_rn(__fmul_rn(__fmul_rn(wd, xd), (float)si), __fmul_rn(wm, xs));
            }
            const int cnt = min(32, nb - b0);
            for (int j = 0; j < cnt; ++j) {
                const float v = __shfl_sync(0xffffffffu, val, j);
                acc = __fadd_rn(acc, v);
            }
        }
        if (lane == 0) y[(size_t)blockIdx.y * ldy + row] = bias ? __fadd_rn(acc, bias[row]) : acc;
    }
}

}  // namespace ckb

using namespace ckb;

static dim3 row_token_grid(int rows, int tokens) { return dim3((unsigned)((rows + 7) / 8 < 148 * 4 ? (rows + 7) / 8 : 148 * 4), (unsigned)tokens); }

// C[m * N + n] = A_q8k[m] . W_q5k[n] (+ bias[n]); M = 1 is gemv_q5_k_q8_k
extern "C" int ckb200_dev_gemm_nt_q5_k_q8_k(const void *A_q8, const void *B, const float *bias, float *C, int M, int N, int K, void *stream)
{
    if (!A_q8 || !B || !C || M <= 0 || N <= 0 || K <= 0) return 0;
    if (K % 256) return ckb_fail(CKB_ERR_SHAPE, "gemm_nt_q5_k_q8_k: K=%d is not a multiple of 256", K);
    if (M > 65535) return ckb_fail(CKB_ERR_SHAPE, "gemm_nt_q5_k_q8_k: %d tokens per call", M);
    if (ckb_ensure_init()) return CKB_ERR_NO_DEVICE;
    gemv_q5k_q8k_kernel<<<row_token_grid(N, M), 256, 0, ckb_stream(stream)>>>((const uint8_t *)B, (const uint8_t *)A_q8, bias, C, N, N, K / 256);
    return ckb_check_launch("gemm_nt_q5_k_q8_k");
}
extern "C" int ckb200_dev_gemv_q5_k_q8_k(float *y, const void *W, const void *x_q8, int M, int K, void *stream)
{
    return ckb200_dev_gemm_nt_q5_k_q8_k(x_q8, W, NULL, y, 1, M, K, stream);
}

extern "C" int ckb200_dev_quantize_q8_1(const float *x, void *y, int rows, int k, void *stream)
{
    if (!x || !y || rows <= 0 || k <= 0) return 0;
    if (k % 32) return ckb_fail(CKB_ERR_SHAPE, "quantize_q8_1: k=%d is not a multiple of 32", k);
    if (ckb_ensure_init()) return CKB_ERR_NO_DEVICE;
    const long long nblocks = (long long)rows * (k / 32);
    const unsigned grid = (unsigned)((nblocks + 7) / 8 < 4096 ? (nblocks + 7) / 8 : 4096);
    quantize_q8_1_kernel<<<grid, 256, 0, ckb_stream(stream)>>>(x, (uint8_t *)y, nblocks);
    return ckb_check_launch("quantize_q8_1");
}

extern "C" int ckb200_dev_gemm_nt_q5_1_q8_1(const void *A_q8, const void *B, const float *bias, float *C, int M, int N, int K, void *stream)
{
    if (!A_q8 || !B || !C || M <= 0 || N <= 0 || K <= 0) return 0;
    if (K % 32) return ckb_fail(CKB_ERR_SHAPE, "gemm_nt_q5_1_q8_1: K=%d is not a multiple of 32", K);
    if (M > 65535) return ckb_fail(CKB_ERR_SHAPE, "gemm_nt_q5_1_q8_1: %d tokens per call", M);
    if (ckb_ensure_init()) return CKB_ERR_NO_DEVICE;
    gemv_q51_q81_kernel<<<row_token_grid(N, M), 256, 0, ckb_stream(stream)>>>((const uint8_t *)B, (const uint8_t *)A_q8, bias, C, N, N, K / 32);
    return ckb_check_launch("gemm_nt_q5_1_q8_1");
}
