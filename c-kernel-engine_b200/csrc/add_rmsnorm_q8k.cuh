// Pieces of the fused residual-add + RMSNorm + Q8_K quantisation row kernel that its two forms share: the single-GPU
// kernel (step_kernels.cu) and the tensor-parallel one that first sums the residual delta over the ranks (tp_p2p.cu).
#pragma once

#include "q8k_block.cuh"

namespace ckb {

constexpr int ARQ_MAX_V4 = 4;      // float4 pieces per thread: rows up to 1024 * 4 * 4 = 16384 elements

// piece i of the updated row: zero beyond d_model, kept in shared memory, squares accumulated
__device__ __forceinline__ void arq_keep_piece(float4 v, int i, int d_model, float *row, float &ss)
{
    const int e = 4 * i;
    if (e + 0 >= d_model) v.x = 0.f;
    if (e + 1 >= d_model) v.y = 0.f;
    if (e + 2 >= d_model) v.z = 0.f;
    if (e + 3 >= d_model) v.w = 0.f;
    ss = fmaf(v.x, v.x, ss); ss = fmaf(v.y, v.y, ss); ss = fmaf(v.z, v.z, ss); ss = fmaf(v.w, v.w, ss);
    reinterpret_cast<float4 *>(row)[i] = v;
}

// block-wide sum of squares -> rstd; one warp per 256-element block scales by gamma and quantises (row t of the output)
__device__ __forceinline__ void arq_norm_quant(float ss, const float *row, float *red, const float *__restrict__ gamma, uint8_t *__restrict__ out_q8,
                                               float *__restrict__ norm_out, int t, int d_model, int aligned, float eps)
{
    ss = group_sum<32>(ss);
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = blockDim.x >> 5;
    if (lane == 0) red[warp] = ss;
    __syncthreads();
    float tot = 0.0f;
    for (int w = 0; w < nw; ++w) tot += red[w];
    const float mean = __fmul_rn(tot, __fdiv_rn(1.0f, (float)d_model));
    const float rstd = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(mean, eps)));
    const int nb = aligned / QK_K;
    for (int b = warp; b < nb; b += nw) {
        float v[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            const int i = b * QK_K + 8 * lane + j;
            v[j] = i < d_model ? __fmul_rn(__fmul_rn(row[i], rstd), gamma[i]) : 0.0f;
            if (norm_out) norm_out[(size_t)t * aligned + i] = v[j];
        }
        quantize_block_q8k(v, out_q8 + ((size_t)t * nb + b) * Q8K_BYTES, lane);
    }
}

}  // namespace ckb
