// Layout glue of the batched prefill step.  The projections of a prompt are batched GEMMs whose outputs are token-major
// ([T][heads * d]), the prefill attention kernel (attention_prefill.cu; attention_forward_causal_head_major_gqa_flash_strided,
// src/kernels/attention_kernels.c:2968-2985) reads head-major tensors ([heads][T][d]) and the KV cache is head-major too
// ([Hkv][max_seq][d], src/kernels/kv_cache_kernels.c:17-20).  Two kernels move between the two, each fused with the op that sits
// at that point of the reference's generated prefill (version/v7/scripts/codegen_prefill_v7.py:194-208):
//
//   prefill_rope_scatter   rope_forward_qk (rotate-half, src/kernels/rope_kernels.c:320-417) on q and k of every token,
//                          q -> [H][T][d], k and v -> cache rows pos0 .. pos0 + T - 1 (kv_cache_store per token)
//   prefill_gather_q8k     attention output [H][T][d] -> token rows, quantised to Q8_K for the o projection (quantize_row_q8_k)
#include "launch.h"
#include "q8k_block.cuh"
#include "runtime.h"

namespace ckb {

__global__ void __launch_bounds__(256) prefill_rope_scatter_kernel(const float *__restrict__ q_tm, const float *__restrict__ k_tm, const float *__restrict__ v_tm,
                                                                   float *__restrict__ q_hm, float *__restrict__ kc, float *__restrict__ vc,
                                                                   const float *__restrict__ cos_cache, const float *__restrict__ sin_cache, int T, int H,
                                                                   int Hkv, int d, int max_seq, int pos0)
{
    const int half = d / 2;
    const long long per_tok = (long long)(H + 2 * Hkv) * half, n = (long long)T * per_tok;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
        const int t = (int)(i / per_tok), r = (int)(i - (long long)t * per_tok);
        const int h = r / half, j = r - h * half, pos = pos0 + t;
        if (pos >= max_seq) continue;
        const float c = cos_cache[(size_t)pos * half + j], sn = sin_cache[(size_t)pos * half + j];
        if (h < H) {
            const float *src = q_tm + ((size_t)t * H + h) * d;
            float *dst = q_hm + ((size_t)h * T + t) * d;
            const float a = src[j], b = src[j + half];
            dst[j] = __fsub_rn(__fmul_rn(a, c), __fmul_rn(b, sn));
            dst[j + half] = __fadd_rn(__fmul_rn(a, sn), __fmul_rn(b, c));
        } else if (h < H + Hkv) {
            const int hk = h - H;
            const float *src = k_tm + ((size_t)t * Hkv + hk) * d;
            float *dst = kc + ((size_t)hk * max_seq + pos) * d;
            const float a = src[j], b = src[j + half];
            dst[j] = __fsub_rn(__fmul_rn(a, c), __fmul_rn(b, sn));
            dst[j + half] = __fadd_rn(__fmul_rn(a, sn), __fmul_rn(b, c));
        } else {
            const int hk = h - H - Hkv;
            const float *src = v_tm + ((size_t)t * Hkv + hk) * d;
            float *dst = vc + ((size_t)hk * max_seq + pos) * d;
            dst[j] = src[j];
            dst[j + half] = src[j + half];
        }
    }
}

// The same with four rotation pairs per thread (16-byte accesses): d a multiple of 8, all pointers 16-byte aligned.
__global__ void __launch_bounds__(256) prefill_rope_scatter_v4_kernel(const float *__restrict__ q_tm, const float *__restrict__ k_tm, const float *__restrict__ v_tm,
                                                                      float *__restrict__ q_hm, float *__restrict__ kc, float *__restrict__ vc,
                                                                      const float *__restrict__ cos_cache, const float *__restrict__ sin_cache, int T, int H,
                                                                      int Hkv, int d, int max_seq, int pos0)
{
    const int half = d / 2, q4 = half / 4;
    const long long per_tok = (long long)(H + 2 * Hkv) * q4, n = (long long)T * per_tok;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
        const int t = (int)(i / per_tok), r = (int)(i - (long long)t * per_tok);
        const int h = r / q4, j = 4 * (r - h * q4), pos = pos0 + t;
        if (pos >= max_seq) continue;
        const float *src;
        float *dst;
        if (h < H) {
            src = q_tm + ((size_t)t * H + h) * d;
            dst = q_hm + ((size_t)h * T + t) * d;
        } else if (h < H + Hkv) {
            src = k_tm + ((size_t)t * Hkv + (h - H)) * d;
            dst = kc + ((size_t)(h - H) * max_seq + pos) * d;
        } else {
            src = v_tm + ((size_t)t * Hkv + (h - H - Hkv)) * d;
            dst = vc + ((size_t)(h - H - Hkv) * max_seq + pos) * d;
        }
        const float4 a = *reinterpret_cast<const float4 *>(src + j), b = *reinterpret_cast<const float4 *>(src + j + half);
        if (h >= H + Hkv) {
            *reinterpret_cast<float4 *>(dst + j) = a;
            *reinterpret_cast<float4 *>(dst + j + half) = b;
            continue;
        }
        const float4 c = *reinterpret_cast<const float4 *>(cos_cache + (size_t)pos * half + j), sn = *reinterpret_cast<const float4 *>(sin_cache + (size_t)pos * half + j);
        float4 lo, hi;
        lo.x = __fsub_rn(__fmul_rn(a.x, c.x), __fmul_rn(b.x, sn.x)); hi.x = __fadd_rn(__fmul_rn(a.x, sn.x), __fmul_rn(b.x, c.x));
        lo.y = __fsub_rn(__fmul_rn(a.y, c.y), __fmul_rn(b.y, sn.y)); hi.y = __fadd_rn(__fmul_rn(a.y, sn.y), __fmul_rn(b.y, c.y));
        lo.z = __fsub_rn(__fmul_rn(a.z, c.z), __fmul_rn(b.z, sn.z)); hi.z = __fadd_rn(__fmul_rn(a.z, sn.z), __fmul_rn(b.z, c.z));
        lo.w = __fsub_rn(__fmul_rn(a.w, c.w), __fmul_rn(b.w, sn.w)); hi.w = __fadd_rn(__fmul_rn(a.w, sn.w), __fmul_rn(b.w, c.w));
        *reinterpret_cast<float4 *>(dst + j) = lo;
        *reinterpret_cast<float4 *>(dst + j + half) = hi;
    }
}

// one warp per (token, 256-element block): lane l takes elements 8l .. 8l+7 of the block (d is a multiple of 8, so they lie in one head)
__global__ void __launch_bounds__(256) prefill_gather_q8k_kernel(const float *__restrict__ out_hm, uint8_t *__restrict__ aq, int T, int H, int d, int cols)
{
    const int lane = threadIdx.x & 31, nb = cols / QK_K;
    const long long blk = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (blk >= (long long)T * nb) return;
    const int t = (int)(blk / nb), b = (int)(blk - (long long)t * nb);
    const int e0 = b * QK_K + 8 * lane;                      // column of the token row
    float v[8];
    if (e0 < H * d) {
        const int h = e0 / d, e = e0 - h * d;
        const float4 lo = *reinterpret_cast<const float4 *>(out_hm + ((size_t)h * T + t) * d + e), hi = *reinterpret_cast<const float4 *>(out_hm + ((size_t)h * T + t) * d + e + 4);
        v[0] = lo.x; v[1] = lo.y; v[2] = lo.z; v[3] = lo.w; v[4] = hi.x; v[5] = hi.y; v[6] = hi.z; v[7] = hi.w;
    } else {
#pragma unroll
        for (int j = 0; j < 8; ++j) v[j] = 0.0f;             // the zero tail of a row narrower than its 256-aligned width
    }
    quantize_block_q8k(v, aq + (size_t)blk * Q8K_BYTES, lane);
}

}  // namespace ckb

using namespace ckb;

extern "C" int ckb200_dev_prefill_rope_scatter(const float *q_tm, const float *k_tm, const float *v_tm, float *q_hm, float *k_cache, float *v_cache,
                                               const float *cos_cache, const float *sin_cache, int tokens, int num_heads, int num_kv_heads, int head_dim,
                                               int max_seq_len, int pos0, void *stream)
{
    if (!q_tm || !k_tm || !v_tm || !q_hm || !k_cache || !v_cache || !cos_cache || !sin_cache || tokens <= 0 || num_heads <= 0 || num_kv_heads <= 0) return 0;
    if (head_dim % 2 || pos0 < 0) return ckb_fail(CKB_ERR_SHAPE, "prefill_rope_scatter: head_dim %d, pos0 %d", head_dim, pos0);
    if (ckb_ensure_init()) return CKB_ERR_NO_DEVICE;
    const long long n = (long long)tokens * (num_heads + 2 * num_kv_heads) * (head_dim / 2);
    const uintptr_t all = (uintptr_t)q_tm | (uintptr_t)k_tm | (uintptr_t)v_tm | (uintptr_t)q_hm | (uintptr_t)k_cache | (uintptr_t)v_cache | (uintptr_t)cos_cache |
                          (uintptr_t)sin_cache;
    if (head_dim % 8 == 0 && (all & 15) == 0) {
        const long long n4 = n / 4;
        const unsigned g4 = (unsigned)((n4 + 255) / 256 < 4736 ? (n4 + 255) / 256 : 4736);
        prefill_rope_scatter_v4_kernel<<<g4, 256, 0, ckb_stream(stream)>>>(q_tm, k_tm, v_tm, q_hm, k_cache, v_cache, cos_cache, sin_cache, tokens, num_heads,
                                                                           num_kv_heads, head_dim, max_seq_len, pos0);
        return ckb_check_launch("prefill_rope_scatter");
    }
    const unsigned grid = (unsigned)((n + 255) / 256 < 4736 ? (n + 255) / 256 : 4736);
    prefill_rope_scatter_kernel<<<grid, 256, 0, ckb_stream(stream)>>>(q_tm, k_tm, v_tm, q_hm, k_cache, v_cache, cos_cache, sin_cache, tokens, num_heads, num_kv_heads,
                                                                      head_dim, max_seq_len, pos0);
    return ckb_check_launch("prefill_rope_scatter");
}

extern "C" int ckb200_dev_prefill_gather_q8k(const float *out_hm, void *out_q8, int tokens, int num_heads, int head_dim, int cols, void *stream)
{
    if (!out_hm || !out_q8 || tokens <= 0 || num_heads <= 0) return 0;
    if (head_dim % 8 || cols % QK_K || cols < num_heads * head_dim || ((uintptr_t)out_hm & 15))
        return ckb_fail(CKB_ERR_SHAPE, "prefill_gather_q8k: head_dim %d, cols %d", head_dim, cols);
    if (ckb_ensure_init()) return CKB_ERR_NO_DEVICE;
    const long long blocks = (long long)tokens * (cols / QK_K);
    prefill_gather_q8k_kernel<<<(unsigned)((blocks + 7) / 8), 256, 0, ckb_stream(stream)>>>(out_hm, (uint8_t *)out_q8, tokens, num_heads, head_dim, cols);
    return ckb_check_launch("prefill_gather_q8k");
}
