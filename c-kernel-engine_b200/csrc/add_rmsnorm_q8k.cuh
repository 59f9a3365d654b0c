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

// gamma of the first block a warp will quantise (block `warp`), fetched before the dependency wait: the norm weights are
// constants, and a load issued after the row statistics are known would put an L2 round trip on the critical path
struct ArqGamma { float4 g0, g1; bool valid; };
__device__ __forceinline__ ArqGamma arq_prefetch_gamma(const float *__restrict__ gamma, int d_model)
{
    ArqGamma g;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    g.g0 = g.g1 = make_float4(0.f, 0.f, 0.f, 0.f);
    g.valid = warp * QK_K + 8 * lane + 8 <= d_model && (reinterpret_cast<uintptr_t>(gamma) & 15) == 0;      // gamma holds d_model values
    if (g.valid) {
        const float4 *p = reinterpret_cast<const float4 *>(gamma + (size_t)warp * QK_K) + 2 * lane;
        g.g0 = __ldg(p);
        g.g1 = __ldg(p + 1);
    }
    return g;
}

// block-wide sum of squares -> rstd; one warp per 256-element block scales by gamma and quantises (row t of the output)
__device__ __forceinline__ void arq_norm_quant(float ss, const float *row, float *red, const float *__restrict__ gamma, uint8_t *__restrict__ out_q8,
                                               float *__restrict__ norm_out, int t, int d_model, int aligned, float eps, const ArqGamma *pre = nullptr)
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
    const bool have_pre = pre != nullptr && pre->valid;
    for (int b = warp; b < nb; b += nw) {
        float gv[8];
        if (have_pre && b == warp) {
            gv[0] = pre->g0.x; gv[1] = pre->g0.y; gv[2] = pre->g0.z; gv[3] = pre->g0.w;
            gv[4] = pre->g1.x; gv[5] = pre->g1.y; gv[6] = pre->g1.z; gv[7] = pre->g1.w;
        } else {
#pragma unroll
            for (int j = 0; j < 8; ++j) gv[j] = b * QK_K + 8 * lane + j < d_model ? gamma[b * QK_K + 8 * lane + j] : 0.0f;
        }
        float v[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            const int i = b * QK_K + 8 * lane + j;
            v[j] = i < d_model ? __fmul_rn(__fmul_rn(row[i], rstd), gv[j]) : 0.0f;
            if (norm_out) norm_out[(size_t)t * aligned + i] = v[j];
        }
        quantize_block_q8k(v, out_q8 + ((size_t)t * nb + b) * Q8K_BYTES, lane);
    }
}

// The same tail for a consumer with 32-element blocks (Q8_0 / Q5_0 weights): the first `cols` elements of the normalised row
// (a multiple of 32) go to Q8_0 blocks with the arithmetic of quantize_row_q8_0 (src/kernels/gemm_kernels_q8_0.c:70-175;
// quantize.cu): one warp per block, amax over the 32 lanes, d = amax / 127 as fp16, q = rint(x * (127 / amax)).
__device__ __forceinline__ void arq_norm_quant_q80(float ss, const float *row, float *red, const float *__restrict__ gamma, uint8_t *__restrict__ out_q80,
                                                   int t, int d_model, int cols, float eps)
{
    ss = group_sum<32>(ss);
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = blockDim.x >> 5;
    if (lane == 0) red[warp] = ss;
    __syncthreads();
    float tot = 0.0f;
    for (int w = 0; w < nw; ++w) tot += red[w];
    const float mean = __fmul_rn(tot, __fdiv_rn(1.0f, (float)d_model));
    const float rstd = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(mean, eps)));
    const int nb = cols / 32;
    for (int b = warp; b < nb; b += nw) {
        const int i = b * 32 + lane;
        const float v = i < d_model ? __fmul_rn(__fmul_rn(row[i], rstd), gamma[i]) : 0.0f;
        float amax = fabsf(v);
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
        const float d = __fdiv_rn(amax, 127.0f);
        const float id = amax != 0.0f ? __fdiv_rn(127.0f, amax) : 0.0f;
        const int q = __float2int_rn(__fmul_rn(v, id));
        const int qn = __shfl_down_sync(0xffffffffu, q, 1);
        uint8_t *out = out_q80 + ((size_t)t * nb + b) * Q80_BYTES;
        if (lane == 0) *reinterpret_cast<unsigned short *>(out) = __half_as_ushort(__float2half_rn(d));
        if ((lane & 1) == 0) *reinterpret_cast<unsigned short *>(out + 2 + lane) = (unsigned short)((q & 255) | ((qn & 255) << 8));
    }
}

}  // namespace ckb
