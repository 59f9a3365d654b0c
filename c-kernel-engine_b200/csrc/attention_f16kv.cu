// The reference's "Llama-parity" attention: attention_forward_decode_head_major_gqa_flash_f16kv and
// attention_forward_causal_head_major_gqa_flash_strided_f16kv (src/kernels/attention_kernels.c:1673-1744, :3006-3046, :3408-3448).
//
// q, k and v pass through fp16 before use and the output accumulator is rounded to fp16 after EVERY key's update, with the online
// max / sum recurrence.  Rounding after each update makes the result depend on the order of the keys, so split-K over the context
// (what the other decode kernels do) would give a different answer: the accumulator has to walk the keys in order.  What can
// still run in parallel is everything that does not touch the accumulator:
//   1. all scores  s_j = scale * sum_d r16(q_d) r16(k_jd)            - warps over keys, lanes over d
//   2. the running max before key j (a prefix maximum) and from it the pair the reference derives per key:
//        new maximum:  max_scale_j = exp(prev - s_j) (0 for the first key), value_scale_j = 1
//        otherwise:    max_scale_j = 1,                                     value_scale_j = exp(s_j - prev)
//      - one warp, 32 keys per step with a shuffle scan
//   3. per output element d (one thread each), key by key:  o = r16(o * max_scale_j) when key j set a new maximum, then
//      o = r16(o + value_scale_j * r16(v_jd));  and  sum = sum * max_scale_j + value_scale_j
//      - the only serial part: three dependent operations per key, the v loads run ahead of it
//      - the only serial part; the value rows arrive through a four-deep cp.async ring in shared memory, so the walk never waits for DRAM
// One CTA of 256 threads per (query head, query token).  Scores and the per-key pairs live in shared memory (8 bytes per key).
// Against the reference the dot products are summed in another order and expf is the device's, so parity is by tolerance; the
// rounding sequence itself is the reference's.
#include <cuda_fp16.h>

#include "device_common.cuh"
#include "launch.h"
#include "pdl.cuh"
#include "runtime.h"

namespace ckb {

constexpr int FK_THREADS = 256;
constexpr int FK_MAX_SMEM = 220 * 1024;
constexpr int FK_CHUNK = 32, FK_STAGES = 4;        // value rows per staged chunk, chunks in flight

__device__ __forceinline__ float r16(float x) { return __half2float(__float2half_rn(x)); }
__device__ __forceinline__ void fk_cp16(uint32_t dst, const void *src) { asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src) : "memory"); }
__device__ __forceinline__ void fk_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void fk_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

// q/out: rows of `ad` floats at (h * q_tokens + i); k/v: [Hkv][kv_stride][ad].  kv_tokens of query i = base_tokens + i, where
// base_tokens comes from *pos_dev + 1 when pos_dev is given.  VEC: ad % 4 == 0 and 16-byte-aligned rows (float4 score loads, value rows
// staged through shared memory by cp.async four chunks ahead of the walk); otherwise plain loads.
template <bool VEC>
__global__ void __launch_bounds__(FK_THREADS) attn_f16kv_kernel(const float *__restrict__ q, const float *__restrict__ k, const float *__restrict__ v,
                                                                float *__restrict__ out, int num_heads, int num_kv_heads, int q_tokens, int base_tokens,
                                                                const int *__restrict__ pos_dev, int kv_stride, int hd, int ad, int max_keys)
{
    extern __shared__ __align__(16) float fk_smem[];
    pdl_wait();
    pdl_trigger();
    const int h = blockIdx.x, i = blockIdx.y;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    constexpr int NW = FK_THREADS / 32;
    int T = (pos_dev ? __ldcg(pos_dev) + 1 : base_tokens) + i;
    T = min(T, min(kv_stride, max_keys));
    float *vs = fk_smem, *ms = fk_smem + max_keys;            // scores, then value_scale; max_scale (-1 = no new maximum at this key)
    float *stage = fk_smem + 2 * max_keys;                    // VEC: FK_STAGES chunks of FK_CHUNK value rows
    const int kvh = (int)((long long)h * num_kv_heads / num_heads);
    const float *qr = q + ((size_t)h * q_tokens + i) * ad;
    const float *kh = k + (size_t)kvh * kv_stride * ad, *vh = v + (size_t)kvh * kv_stride * ad;
    float *orow = out + ((size_t)h * q_tokens + i) * ad;
    const float scale = 1.0f / sqrtf((float)hd);

    // value rows are contiguous: chunk c = rows [c * FK_CHUNK, ...) = one block of FK_CHUNK * ad floats; start the first chunks now
    const int nchunks = (T + FK_CHUNK - 1) / FK_CHUNK, chunk_f4 = FK_CHUNK * ad / 4;
    auto issue_chunk = [&](int c) {
        if (c < nchunks) {
            const int rows = min(FK_CHUNK, T - c * FK_CHUNK), n4 = rows * ad / 4;
            const float4 *src = reinterpret_cast<const float4 *>(vh + (size_t)c * FK_CHUNK * ad);
            const uint32_t dst = smem_u32(stage + (size_t)(c % FK_STAGES) * FK_CHUNK * ad);
            for (int x = tid; x < n4; x += FK_THREADS) fk_cp16(dst + 16u * (uint32_t)x, src + x);
        }
        fk_commit();
    };
    if constexpr (VEC) {
        (void)chunk_f4;
        for (int c = 0; c < FK_STAGES - 1; ++c) issue_chunk(c);
    }

    // 1. scores
    if constexpr (VEC) {
        // lane holds q elements 4 lane .. 4 lane + 3 (and + 128 for heads wider than 128); eight keys per warp step, one float4 per key in flight
        const int n4 = hd / 4;
        float4 q0 = make_float4(0.f, 0.f, 0.f, 0.f), q1 = q0;
        if (lane < n4) { const float4 t = __ldcg(reinterpret_cast<const float4 *>(qr) + lane); q0 = make_float4(r16(t.x), r16(t.y), r16(t.z), r16(t.w)); }
        if (lane + 32 < n4) { const float4 t = __ldcg(reinterpret_cast<const float4 *>(qr) + lane + 32); q1 = make_float4(r16(t.x), r16(t.y), r16(t.z), r16(t.w)); }
        for (int j0 = warp * 8; j0 < T; j0 += 8 * NW) {
            float4 kv0[8], kv1[8];
#pragma unroll
            for (int u = 0; u < 8; ++u) {
                const float4 *kr = reinterpret_cast<const float4 *>(kh + (size_t)min(j0 + u, T - 1) * ad);
                kv0[u] = lane < n4 ? __ldcg(kr + lane) : make_float4(0.f, 0.f, 0.f, 0.f);
                kv1[u] = lane + 32 < n4 ? __ldcg(kr + lane + 32) : make_float4(0.f, 0.f, 0.f, 0.f);
            }
#pragma unroll
            for (int u = 0; u < 8; ++u) {
                float dot = q0.x * r16(kv0[u].x);
                dot = fmaf(q0.y, r16(kv0[u].y), dot);
                dot = fmaf(q0.z, r16(kv0[u].z), dot);
                dot = fmaf(q0.w, r16(kv0[u].w), dot);
                dot = fmaf(q1.x, r16(kv1[u].x), dot);
                dot = fmaf(q1.y, r16(kv1[u].y), dot);
                dot = fmaf(q1.z, r16(kv1[u].z), dot);
                dot = fmaf(q1.w, r16(kv1[u].w), dot);
#pragma unroll
                for (int o = 16; o; o >>= 1) dot += __shfl_xor_sync(0xffffffffu, dot, o);
                if (lane == 0 && j0 + u < T) vs[j0 + u] = dot * scale;
            }
        }
    } else {
        float qv[8];
#pragma unroll
        for (int e = 0; e < 8; ++e) qv[e] = lane + 32 * e < hd ? r16(__ldcg(qr + lane + 32 * e)) : 0.0f;
        for (int j0 = warp * 4; j0 < T; j0 += 4 * NW) {
            float dot[4] = {0.0f, 0.0f, 0.0f, 0.0f};
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                const int j = min(j0 + u, T - 1);
#pragma unroll
                for (int e = 0; e < 8; ++e)
                    if (lane + 32 * e < hd) dot[u] = fmaf(qv[e], r16(__ldcg(kh + (size_t)j * ad + lane + 32 * e)), dot[u]);
            }
#pragma unroll
            for (int u = 0; u < 4; ++u) {
#pragma unroll
                for (int o = 16; o; o >>= 1) dot[u] += __shfl_xor_sync(0xffffffffu, dot[u], o);
                if (lane == 0 && j0 + u < T) vs[j0 + u] = dot[u] * scale;
            }
        }
    }
    __syncthreads();

    // 2. prefix maximum and the per-key pairs
    if (warp == 0) {
        float carry = -INFINITY;
        for (int j0 = 0; j0 < T; j0 += 32) {
            const int j = j0 + lane;
            const float s = j < T ? vs[j] : -INFINITY;
            float incl = s;
#pragma unroll
            for (int o = 1; o < 32; o <<= 1) {
                const float other = __shfl_up_sync(0xffffffffu, incl, o);
                if (lane >= o) incl = fmaxf(incl, other);
            }
            float prev = __shfl_up_sync(0xffffffffu, incl, 1);
            prev = lane == 0 ? carry : fmaxf(prev, carry);
            if (j < T) {
                if (s > prev) {
                    ms[j] = isfinite(prev) ? expf(prev - s) : 0.0f;
                    vs[j] = 1.0f;
                } else {
                    ms[j] = -1.0f;
                    vs[j] = expf(s - prev);
                }
            }
            carry = fmaxf(carry, __shfl_sync(0xffffffffu, incl, 31));
        }
    }
    __syncthreads();

    // 3. the ordered walk: thread d owns output element d
    if constexpr (VEC) {
        float o = 0.0f, sum = 0.0f;
        for (int c = 0; c < nchunks; ++c) {
            issue_chunk(c + FK_STAGES - 1);                   // into the stage that chunk c - 1 has just left (the barrier at the loop's end)
            fk_wait<FK_STAGES - 1>();
            __syncthreads();                                  // chunk c has landed for every thread
            if (tid < hd) {
                const float *vrow = stage + (size_t)(c % FK_STAGES) * FK_CHUNK * ad + tid;
                const int j0 = c * FK_CHUNK, rows = min(FK_CHUNK, T - j0);
                int u = 0;
                for (; u + 8 <= rows; u += 8) {               // the factors and products of eight keys first, then the dependent chain
                    float m8[8], w8[8], p8[8];
#pragma unroll
                    for (int e = 0; e < 8; ++e) {
                        m8[e] = ms[j0 + u + e];
                        w8[e] = vs[j0 + u + e];
                        p8[e] = __fmul_rn(w8[e], r16(vrow[(size_t)(u + e) * ad]));
                    }
#pragma unroll
                    for (int e = 0; e < 8; ++e) {
                        if (m8[e] >= 0.0f) { o = r16(__fmul_rn(o, m8[e])); sum = __fmul_rn(sum, m8[e]); }
                        o = r16(__fadd_rn(o, p8[e]));
                        sum = __fadd_rn(sum, w8[e]);
                    }
                }
                for (; u < rows; ++u) {
                    const float m = ms[j0 + u], w = vs[j0 + u], vv = r16(vrow[(size_t)u * ad]);
                    if (m >= 0.0f) { o = r16(__fmul_rn(o, m)); sum = __fmul_rn(sum, m); }
                    o = r16(__fadd_rn(o, __fmul_rn(w, vv)));
                    sum = __fadd_rn(sum, w);
                }
            }
            __syncthreads();                                  // everyone is done with this stage before it is refilled
        }
        fk_wait<0>();
        for (int d = tid; d < ad; d += FK_THREADS) {
            if (d >= hd) orow[d] = 0.0f;
            else if (d == tid) orow[d] = sum > 0.0f ? __fmul_rn(o, __fdiv_rn(1.0f, sum)) : 0.0f;
        }
    } else {
        for (int d = tid; d < ad; d += FK_THREADS) {
            if (d >= hd) { orow[d] = 0.0f; continue; }
            float o = 0.0f, sum = 0.0f;
            const float *vp = vh + d;
            for (int j = 0; j < T; ++j) {
                const float m = ms[j], w = vs[j], vv = r16(__ldcg(vp + (size_t)j * ad));
                if (m >= 0.0f) { o = r16(__fmul_rn(o, m)); sum = __fmul_rn(sum, m); }
                o = r16(__fadd_rn(o, __fmul_rn(w, vv)));
                sum = __fadd_rn(sum, w);
            }
            orow[d] = sum > 0.0f ? __fmul_rn(o, __fdiv_rn(1.0f, sum)) : 0.0f;
        }
    }
}

static int launch_f16kv(const float *q, const float *k, const float *v, float *out, int num_heads, int num_kv_heads, int q_tokens, int base_tokens,
                        const int *pos_dev, int kv_stride, int hd, int ad, int max_keys, cudaStream_t st, const char *what)
{
    if (hd <= 0 || hd > 256 || ad < hd || num_heads <= 0 || num_kv_heads <= 0 || q_tokens <= 0) return ckb_fail(CKB_ERR_SHAPE, "%s: head size %d / %d not handled", what, hd, ad);
    max_keys = (max_keys + 3) & ~3;                           /* the arrays behind the per-key pairs start on 16-byte boundaries */
    const bool vec = ad % 4 == 0 && hd % 4 == 0 && hd <= FK_THREADS && !((((uintptr_t)q | (uintptr_t)k | (uintptr_t)v) & 15));
    const size_t smem = (size_t)max_keys * 2 * sizeof(float) + (vec ? (size_t)FK_STAGES * FK_CHUNK * ad * sizeof(float) : 0);
    if (smem > FK_MAX_SMEM)
        return ckb_fail(CKB_ERR_LIMIT, "%s: %d keys need %zu bytes of shared memory for the ordered walk (limit about %d keys)", what, max_keys, smem,
                        (int)((FK_MAX_SMEM - FK_STAGES * FK_CHUNK * ad * 4) / 8));
    static int attr_set = 0;
    if (!attr_set) {
        if (ckb_check_cuda((int)cudaFuncSetAttribute(attn_f16kv_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, FK_MAX_SMEM), "attn_f16kv smem attr") ||
            ckb_check_cuda((int)cudaFuncSetAttribute(attn_f16kv_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, FK_MAX_SMEM), "attn_f16kv smem attr"))
            return CKB_ERR_CUDA;
        attr_set = 1;
    }
    if (vec)
        return launch_pdl(what, attn_f16kv_kernel<true>, dim3(num_heads, q_tokens), dim3(FK_THREADS), smem, st, q, k, v, out, num_heads, num_kv_heads, q_tokens, base_tokens,
                          pos_dev, kv_stride, hd, ad, max_keys);
    return launch_pdl(what, attn_f16kv_kernel<false>, dim3(num_heads, q_tokens), dim3(FK_THREADS), smem, st, q, k, v, out, num_heads, num_kv_heads, q_tokens, base_tokens,
                      pos_dev, kv_stride, hd, ad, max_keys);
}

}  // namespace ckb

using namespace ckb;

// q/out [H][ad], caches [Hkv][cache_capacity][ad]; with pos_dev the context length is *pos_dev + 1, read on the device (the shared
// memory is then sized for the whole cache).
extern "C" int ckb200_dev_attention_decode_f16kv(const float *q, const float *k_cache, const float *v_cache, float *out, int num_heads, int num_kv_heads,
                                                 int kv_tokens, int cache_capacity, int head_dim, int aligned_head_dim, const int *pos_dev, void *stream)
{
    if (!q || !k_cache || !v_cache || !out) return 0;
    if (!pos_dev && (kv_tokens <= 0 || kv_tokens > cache_capacity)) return 0;
    if (cache_capacity <= 0) return 0;
    return launch_f16kv(q, k_cache, v_cache, out, num_heads, num_kv_heads, 1, kv_tokens, pos_dev, cache_capacity, head_dim, aligned_head_dim,
                        pos_dev ? cache_capacity : kv_tokens, ckb_stream(stream), "attention_decode_f16kv");
}

// q/out [H][T][ad], k/v [Hkv][kv_stride][ad]; query i sees keys 0..i
extern "C" int ckb200_dev_attention_prefill_f16kv(const float *q, const float *k, const float *v, float *out, int num_heads, int num_kv_heads, int num_tokens,
                                                  int head_dim, int aligned_head_dim, int kv_stride_tokens, void *stream)
{
    if (!q || !k || !v || !out) return 0;
    if (num_tokens <= 0 || kv_stride_tokens < num_tokens) return 0;
    return launch_f16kv(q, k, v, out, num_heads, num_kv_heads, num_tokens, 1, NULL, kv_stride_tokens, head_dim, aligned_head_dim, num_tokens,
                        ckb_stream(stream), "attention_prefill_f16kv");
}
