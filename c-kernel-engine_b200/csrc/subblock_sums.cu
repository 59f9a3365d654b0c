// Integer stage of the K-quant dot products, dumped as it is computed by the GEMV kernels' own unit functions.
//
// The reference's scalar dot products accumulate, per superblock, int32 sums of (weight code x activation byte) before
// any floating point happens: eight 32-element sums of nibble x q8 for Q4_K (sum_q4q8_lo / sum_q4q8_hi,
// src/kernels/gemm_kernels_q4k_q8k.c:144-167) and sixteen 16-element sums of (q6 - 32) x q8 for Q6_K
// (src/kernels/gemm_kernels_q6k_q8k.c:92-111).  No reference API returns them, and neither do the GEMVs here (they fold the
// sums into fp32 at once), so these two entry points exist for one purpose: a test can compare the integer stage bit for bit.
// They call the SAME device functions the production kernels call -
//
//   Q4_K  variant 0: q4p_stage_x + q4p_isums      (pair kernel gemv_q4k.cu; the register-activation kernel runs the same dp4a chain)
//         variant 1: load_x_q8k<1> + q4k_isums    (direct and ring kernels, gemv.cu)
//   Q6_K  variant 0: ring_stage_x<Q6_K> + q6k_plane_sums, minus 32 x the staged block sums   (planar kernel and ring kernel)
//         variant 1: load_x_q8k<2> + q6k_isums    (direct kernel)
//
// - on weights in the reference's own row layout.  One warp per row; not a fast path.
#include "q4p_unit.cuh"
#include "ring_x.cuh"
#include "launch.h"
#include "runtime.h"

namespace ckb {

// out[row][b][j], j = 0..7: sum over the 32 elements of sub-block j of (4-bit code) x q8
template <int VARIANT>
__global__ void __launch_bounds__(256) subblock_sums_q4k_kernel(const uint8_t *__restrict__ W, const uint8_t *__restrict__ xg, int32_t *__restrict__ out, int M, int nb)
{
    extern __shared__ __align__(128) uint8_t smem[];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = blockDim.x >> 5;
    if constexpr (VARIANT == 0) {
        const Q4pX x = q4p_stage_x(xg, nb, smem);
        __syncthreads();
        for (int row = blockIdx.x * nw + warp; row < M; row += gridDim.x * nw) {
            for (int i = lane; i < 2 * nb; i += 32) {
                const int b = i >> 1, p = i & 1;
                const uint8_t *pb = W + ((size_t)row * nb + b) * Q4K_BYTES;
                Q4pW w;
                w.hdr = ldg_stream_u4(pb);
                w.a0 = ldg_stream_u4(pb + 16 + 32 * p);
                w.a1 = ldg_stream_u4(pb + 32 + 32 * p);
                w.b0 = ldg_stream_u4(pb + 80 + 32 * p);
                w.b1 = ldg_stream_u4(pb + 96 + 32 * p);
                int a_lo, a_hi16, b_lo, b_hi16;
                q4p_isums(w, x, b, p, a_lo, a_hi16, b_lo, b_hi16);
                int32_t *o = out + ((size_t)row * nb + b) * 8;
                o[2 * p] = a_lo;
                o[2 * p + 1] = a_hi16 >> 4;          // the kernel leaves the high nibbles in place: 16 x the sum, exactly
                o[2 * p + 4] = b_lo;
                o[2 * p + 5] = b_hi16 >> 4;
            }
        }
    } else {
        const XQ8K x = load_x_q8k<1>(xg, nb, smem);
        __syncthreads();
        for (int row = blockIdx.x * nw + warp; row < M; row += gridDim.x * nw) {
            for (int i = lane; i < 4 * nb; i += 32) {
                const int b = i >> 2, q = i & 3;
                const uint8_t *pb = W + ((size_t)row * nb + b) * Q4K_BYTES;
                const uint4 qa = ldg_stream_u4(pb + 16 + 32 * q), qb = ldg_stream_u4(pb + 32 + 32 * q);
                const Q4kX xr = q4k_load_x(x, b, q);
                int lo, hi;
                q4k_isums(qa, qb, xr, lo, hi);
                int32_t *o = out + ((size_t)row * nb + b) * 8;
                o[2 * q] = lo;
                o[2 * q + 1] = hi;
            }
        }
    }
}

// out[row][b][j], j = 0..15: sum over elements 16j .. 16j+15 of (q6 - 32) x q8
template <int VARIANT>
__global__ void __launch_bounds__(256) subblock_sums_q6k_kernel(const uint8_t *__restrict__ W, const uint8_t *__restrict__ xg, int32_t *__restrict__ out, int M, int nb)
{
    extern __shared__ __align__(128) uint8_t smem[];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = blockDim.x >> 5;
    RingX rx = {};
    XQ8K kx = {};
    if constexpr (VARIANT == 0) rx = ring_stage_x<FMT_Q6K>(xg, nb, smem);
    else kx = load_x_q8k<2>(xg, nb, smem);
    __syncthreads();
    for (int row = blockIdx.x * nw + warp; row < M; row += gridDim.x * nw) {
        for (int i = lane; i < 4 * nb; i += 32) {
            const int b = i >> 2, u = i & 3, n = u >> 1, h = u & 1;
            const uint8_t *p = W + ((size_t)row * nb + b) * Q6K_BYTES;             // 2-byte aligned
            const uint4 qa = ldg_u4_align2(p + 64 * n + 16 * h);
            const uint4 qb = ldg_u4_align2(p + 64 * n + 32 + 16 * h);
            const uint4 qh = ldg_u4_align2(p + 128 + 32 * n + 16 * h);
            int s[4];
            if constexpr (VARIANT == 0) {
                const uint32_t xa = rx.q + (uint32_t)(b * 80 + (10 * n + h) * 4) * 4u;
                const uint4 x0 = lds_u4(xa), x1 = lds_u4(xa + 32), x2 = lds_u4(xa + 64), x3 = lds_u4(xa + 96);
                q6k_plane_sums(qa, qb, qh, x0, x1, x2, x3, s[0], s[1], s[2], s[3]);
                // the staged block sums of scale groups 8n + h + 2t, split as 128 * hi + lo (what the GEMV multiplies by the scales)
                const uint32_t lo4 = lds_u32(rx.lo + 4u * (b * 4 + u)), hi4 = lds_u32(rx.hi + 4u * (b * 4 + u));
#pragma unroll
                for (int t = 0; t < 4; ++t) {
                    const int bsum = (int)(int8_t)((lo4 >> (8 * t)) & 255u) + 128 * (int)(int8_t)((hi4 >> (8 * t)) & 255u);
                    s[t] -= 32 * bsum;
                }
            } else {
                const Q6kX xr = q6k_load_x(kx, b, n, h);
                q6k_isums(qa, qb, qh, xr, s);
            }
            int32_t *o = out + ((size_t)row * nb + b) * 16 + 8 * n + h;
#pragma unroll
            for (int t = 0; t < 4; ++t) o[2 * t] = s[t];
        }
    }
}

template <typename K>
static int launch_sums(const char *what, K kernel, int smem, const void *W, const void *xq, int32_t *out, int M, int nb, cudaStream_t st)
{
    if (smem > 200 * 1024) return ckb_fail(CKB_ERR_LIMIT, "%s: K too large for the shared activation buffer", what);
    if (smem > 48 * 1024 && ckb_check_cuda((int)cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem), "smem attr")) return CKB_ERR_CUDA;
    const int grid = M < 8 * 296 ? (M + 7) / 8 : 296;
    kernel<<<grid, 256, smem, st>>>((const uint8_t *)W, (const uint8_t *)xq, out, M, nb);
    return ckb_check_launch(what);
}

}  // namespace ckb

using namespace ckb;

extern "C" int ckb200_dev_subblock_sums_q4_k_q8_k(const void *W, const void *x_q8, int M, int K, int32_t *out, int variant, void *stream)
{
    if (!W || !x_q8 || !out || M <= 0 || K <= 0) return 0;
    if (K % QK_K) return ckb_fail(CKB_ERR_SHAPE, "subblock_sums_q4_k_q8_k: K=%d is not a multiple of 256", K);
    if (((uintptr_t)W & 15) || ((uintptr_t)x_q8 & 3) || ((uintptr_t)out & 3)) return ckb_fail(CKB_ERR_ALIGN, "subblock_sums_q4_k_q8_k: W 16-byte, x_q8 and out 4-byte aligned");
    if (ckb_ensure_init()) return CKB_ERR_NO_DEVICE;
    const int nb = K / QK_K;
    cudaStream_t st = ckb_stream(stream);
    if (variant == 0) return launch_sums("subblock_sums_q4k", subblock_sums_q4k_kernel<0>, q4p_smem_bytes(nb), W, x_q8, out, M, nb, st);
    if (variant == 1) return launch_sums("subblock_sums_q4k", subblock_sums_q4k_kernel<1>, (xq8k_smem_bytes(nb, 1) + 127) & ~127, W, x_q8, out, M, nb, st);
    return ckb_fail(CKB_ERR_STATE, "subblock_sums_q4_k_q8_k: unknown variant %d", variant);
}

extern "C" int ckb200_dev_subblock_sums_q6_k_q8_k(const void *W, const void *x_q8, int M, int K, int32_t *out, int variant, void *stream)
{
    if (!W || !x_q8 || !out || M <= 0 || K <= 0) return 0;
    if (K % QK_K) return ckb_fail(CKB_ERR_SHAPE, "subblock_sums_q6_k_q8_k: K=%d is not a multiple of 256", K);
    if (((uintptr_t)W & 1) || ((uintptr_t)x_q8 & 3) || ((uintptr_t)out & 3)) return ckb_fail(CKB_ERR_ALIGN, "subblock_sums_q6_k_q8_k: W 2-byte, x_q8 and out 4-byte aligned");
    if (ckb_ensure_init()) return CKB_ERR_NO_DEVICE;
    const int nb = K / QK_K;
    cudaStream_t st = ckb_stream(stream);
    if (variant == 0) return launch_sums("subblock_sums_q6k", subblock_sums_q6k_kernel<0>, ringx_smem_bytes(FMT_Q6K, nb), W, x_q8, out, M, nb, st);
    if (variant == 1) return launch_sums("subblock_sums_q6k", subblock_sums_q6k_kernel<1>, (xq8k_smem_bytes(nb, 2) + 127) & ~127, W, x_q8, out, M, nb, st);
    return ckb_fail(CKB_ERR_STATE, "subblock_sums_q6_k_q8_k: unknown variant %d", variant);
}
