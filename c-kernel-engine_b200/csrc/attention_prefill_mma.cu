// Prefill attention (attention_forward_causal_head_major_gqa_flash[_strided], attention_forward_full_head_major_gqa_flash[_strided],
// src/kernels/attention_kernels.c:2924-3005) on the tensor cores at fp32 accuracy.
//
// The trick of attention_f16mma.cu applied to a block of 16 query tokens: a product of two fp16 numbers is exact in the fp32
// accumulator, so every fp32 operand is split into two fp16 pieces (x = x_hi + x_lo, 22 significant bits) and a product a x b becomes
// three instructions, a_hi b_hi + a_lo b_hi + a_hi b_lo (the fourth term is below fp32 resolution).  A CTA is one kv head and one
// block of 16 queries, one warp per query head of the kv head: the warps share each 64-key tile, which all threads convert once,
// while loading it, into four fp16 tiles in shared memory (K hi, K lo, V hi, V lo; rows padded by 16 bytes so that ldmatrix meets no
// bank conflicts).  Scores, online softmax (base 2, the scale folded into the query) and probabilities x values follow
// mma.sync.m16n8k16's fragment layouts, so the probabilities go from the score registers straight into the A operand of the next
// product.  Causal blocks are dealt heaviest first; key tiles of 8 that lie wholly behind the diagonal are skipped.
// The pieces live in fp16's range: key and value magnitudes of 65504 or more are not supported by this form (the CUDA-core kernel
// of attention_prefill.cu is; tune attn_prefill_mma = 0).
#include <cuda_fp16.h>

#include "device_common.cuh"
#include "launch.h"
#include "pdl.cuh"
#include "runtime.h"

namespace ckb {

constexpr int PM_BQ = 16, PM_BK = 64;
constexpr float PM_QSCALE = 256.0f, PM_PSCALE = 16384.0f;    // powers of two that keep the lo pieces out of fp16's subnormal range

__device__ __forceinline__ void pm_ldmatrix(uint32_t (&r)[4], uint32_t addr)
{
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void pm_ldmatrix_t(uint32_t (&r)[4], uint32_t addr)
{
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void pm_mma(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1)
{
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3]) : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void pm_split2(float a, float b, uint32_t &hi, uint32_t &lo)
{
    const __half2 h = __floats2half2_rn(a, b);
    const float2 hf = __half22float2(h);
    const __half2 l = __floats2half2_rn(a - hf.x, b - hf.y);
    hi = *reinterpret_cast<const uint32_t *>(&h);
    lo = *reinterpret_cast<const uint32_t *>(&l);
}

// Keys and values as the four fp16 tiles want them, once per call: kv16 = K hi | K lo | V hi | V lo, each [Hkv][T][AD] (columns
// past the head are zeros).  Every query block of a kv head reads the same keys, so the split is done here and not per block.
template <int AD>
__global__ void __launch_bounds__(256) pm_split_kv_kernel(const float *__restrict__ k, const float *__restrict__ v, __half *__restrict__ kv16, int Hkv, int T, int hd,
                                                          int kv_stride)
{
    pdl_trigger();
    pdl_wait();
    const size_t n4 = (size_t)Hkv * T * (AD / 4), arr = (size_t)Hkv * T * AD;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n4; i += (size_t)gridDim.x * blockDim.x) {
        const int c4 = (int)(i % (AD / 4));
        const size_t row = i / (AD / 4);
        const int tok = (int)(row % T), h = (int)(row / T), d = 4 * c4;
        const size_t src = ((size_t)h * kv_stride + tok) * AD + d;
        float4 kx = __ldcg(reinterpret_cast<const float4 *>(k + src)), vx = __ldcg(reinterpret_cast<const float4 *>(v + src));
        if (d + 3 >= hd) {
            if (d >= hd) { kx.x = 0.f; vx.x = 0.f; }
            if (d + 1 >= hd) { kx.y = 0.f; vx.y = 0.f; }
            if (d + 2 >= hd) { kx.z = 0.f; vx.z = 0.f; }
            kx.w = 0.f; vx.w = 0.f;
        }
        uint2 hi, lo;
        __half *dst = kv16 + row * AD + d;
        pm_split2(kx.x, kx.y, hi.x, lo.x);
        pm_split2(kx.z, kx.w, hi.y, lo.y);
        *reinterpret_cast<uint2 *>(dst) = hi;
        *reinterpret_cast<uint2 *>(dst + arr) = lo;
        pm_split2(vx.x, vx.y, hi.x, lo.x);
        pm_split2(vx.z, vx.w, hi.y, lo.y);
        *reinterpret_cast<uint2 *>(dst + 2 * arr) = hi;
        *reinterpret_cast<uint2 *>(dst + 3 * arr) = lo;
    }
}

__device__ __forceinline__ void pm_cp16(uint32_t dst, const void *src, uint32_t bytes)     // bytes = 0: sixteen zeros
{
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(bytes) : "memory");
}
__device__ __forceinline__ void pm_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
__device__ __forceinline__ void pm_wait1() { asm volatile("cp.async.wait_group 1;" ::: "memory"); }

// q, out: [H][T][AD]; kv16 as written by pm_split_kv_kernel.  grid (kv heads, query blocks), block = 32 * KH * (H / Hkv) threads:
// warp = key part * G + query head of the kv head.  With KH = 2 (up to four query heads per kv head) two warps share a head and
// take 32 keys of each 64-key tile each, with their own running maximum; they are merged at the end.  The tiles of the next step
// are copied (cp.async, rows padded to PITCH) while this step multiplies.
template <int AD, int KH>
__global__ void __launch_bounds__(256) attn_prefill_mma_kernel(const float *__restrict__ q, const __half *__restrict__ kv16, float *__restrict__ out, int H, int Hkv,
                                                               int T, int hd, int causal, float scale)
{
    constexpr int KS = AD / 16, NTD = AD / 8, PITCH = (AD + 8) * 2;    // bytes per row of an fp16 tile
    constexpr int TILE = PM_BK * PITCH, STAGE = 4 * TILE;              // K hi, K lo, V hi, V lo
    constexpr int KPW = PM_BK / KH, NKT = KPW / 8;                     // keys of a tile per warp, in 8-key MMA columns
    extern __shared__ __align__(16) uint8_t pm_smem[];                 // two stages
    const uint32_t s_base = smem_u32(pm_smem);
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, g = lane >> 2, t = lane & 3, nthreads = blockDim.x;
    const int G = H / Hkv, kvh = blockIdx.x, part = warp / G, h = kvh * G + (warp - part * G), koff = part * KPW;
    // CTAs start in the order of their linear index, x fastest: every kv head's block with the most keys first, then the next
    // block of every head, so the short blocks fill the gaps at the end (with the heads outermost the last heads' long blocks
    // started when most SMs were already idle: 40 % of the SM time was idle)
    const int qb = gridDim.y - 1 - blockIdx.y, q0 = qb * PM_BQ;
    const int key_end = causal ? min(T, q0 + PM_BQ) : T;                // keys [0, key_end) matter to this block
    const int ntiles = (key_end + PM_BK - 1) / PM_BK;
    const size_t arr = (size_t)Hkv * T * AD;
    pdl_trigger();
    pdl_wait();

    auto issue = [&](int kt) {
        const int key0 = kt * PM_BK;
        const uint32_t st = s_base + (uint32_t)(kt & 1) * STAGE;
        for (int c = tid; c < 4 * PM_BK * (AD / 8); c += nthreads) {
            const int a = c / (PM_BK * (AD / 8)), rem = c - a * (PM_BK * (AD / 8)), row = rem / (AD / 8), ch = rem - row * (AD / 8);
            const int key = key0 + row;
            const __half *src = kv16 + (size_t)a * arr + ((size_t)kvh * T + min(key, T - 1)) * AD + ch * 8;
            pm_cp16(st + (uint32_t)(a * TILE + row * PITCH + ch * 16), src, key < key_end ? 16u : 0u);
        }
    };
    issue(0);
    pm_commit();

    // query fragments of rows g and g + 8 (queries q0 + g, q0 + g + 8), hi and lo pieces
    uint32_t aqh[KS][4], aql[KS][4];
    {
        const float qs = scale * 1.44269504088896340736f * PM_QSCALE;
#pragma unroll
        for (int ks = 0; ks < KS; ++ks)
#pragma unroll
            for (int half = 0; half < 2; ++half) {                     // k = 16ks + 2t (+ 8)
                const int d = 16 * ks + 2 * t + 8 * half;
                float2 u0 = make_float2(0.f, 0.f), u1 = u0;
                if (q0 + g < T) u0 = __ldcg(reinterpret_cast<const float2 *>(q + ((size_t)h * T + q0 + g) * AD + d));
                if (q0 + g + 8 < T) u1 = __ldcg(reinterpret_cast<const float2 *>(q + ((size_t)h * T + q0 + g + 8) * AD + d));
                if (d >= hd) { u0.x = 0.f; u1.x = 0.f; }
                if (d + 1 >= hd) { u0.y = 0.f; u1.y = 0.f; }
                pm_split2(u0.x * qs, u0.y * qs, aqh[ks][2 * half], aql[ks][2 * half]);
                pm_split2(u1.x * qs, u1.y * qs, aqh[ks][2 * half + 1], aql[ks][2 * half + 1]);
            }
    }

    float o[NTD][4];
#pragma unroll
    for (int n = 0; n < NTD; ++n)
#pragma unroll
        for (int e = 0; e < 4; ++e) o[n][e] = 0.0f;
    float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.0f, 0.0f};
    const int mi = lane >> 3, rr = lane & 7;

    for (int kt = 0; kt < ntiles; ++kt) {
        const int key0 = kt * PM_BK;
        if (kt + 1 < ntiles) issue(kt + 1);
        pm_commit();                                                   // an empty group after the last tile keeps the count uniform
        pm_wait1();                                                    // this thread's copies of tile kt have landed
        __syncthreads();                                               // ... and everybody else's
        const uint32_t st = s_base + (uint32_t)(kt & 1) * STAGE;

        // 8-key columns of this warp's part that hold a key the block needs
        const int nt_lim = max(0, min(NKT, (key_end - key0 - koff + 7) / 8));
        if (nt_lim > 0) {
            float s[NKT][4];
#pragma unroll
            for (int n = 0; n < NKT; ++n)
#pragma unroll
                for (int e = 0; e < 4; ++e) s[n][e] = 0.0f;
#pragma unroll
            for (int ks = 0; ks < KS; ++ks) {
#pragma unroll
                for (int n2 = 0; n2 < NKT / 2; ++n2) {
                    if (2 * n2 < nt_lim) {
                        // matrices: (keys 8(2 n2) .., d 16ks ..), (same keys, d 16ks + 8 ..), (keys 8(2 n2 + 1) .., d 16ks ..), (.., d 16ks + 8 ..)
                        const uint32_t addr = st + (uint32_t)((koff + 8 * (2 * n2 + (mi >> 1)) + rr) * PITCH + (16 * ks + 8 * (mi & 1)) * 2);
                        uint32_t kh4[4], kl4[4];
                        pm_ldmatrix(kh4, addr);
                        pm_ldmatrix(kl4, addr + TILE);
                        pm_mma(s[2 * n2], aqh[ks], kh4[0], kh4[1]);
                        pm_mma(s[2 * n2], aql[ks], kh4[0], kh4[1]);
                        pm_mma(s[2 * n2], aqh[ks], kl4[0], kl4[1]);
                        pm_mma(s[2 * n2 + 1], aqh[ks], kh4[2], kh4[3]);
                        pm_mma(s[2 * n2 + 1], aql[ks], kh4[2], kh4[3]);
                        pm_mma(s[2 * n2 + 1], aqh[ks], kl4[2], kl4[3]);
                    }
                }
            }
            // mask, running maximum and sum of rows g (e = 0, 1) and g + 8 (e = 2, 3)
            float mt[2] = {-INFINITY, -INFINITY};
#pragma unroll
            for (int n = 0; n < NKT; ++n)
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const int key = key0 + koff + 8 * n + 2 * t + (e & 1), qrow = q0 + g + ((e & 2) ? 8 : 0);
                    const bool valid = n < nt_lim && key < T && (!causal || key <= qrow);
                    s[n][e] = valid ? s[n][e] * (1.0f / PM_QSCALE) : -INFINITY;
                    mt[e >> 1] = fmaxf(mt[e >> 1], s[n][e]);
                }
            float alpha[2], m_ref[2];
#pragma unroll
            for (int r = 0; r < 2; ++r) {
                mt[r] = fmaxf(mt[r], __shfl_xor_sync(0xffffffffu, mt[r], 1));
                mt[r] = fmaxf(mt[r], __shfl_xor_sync(0xffffffffu, mt[r], 2));
                const float m_new = fmaxf(m_run[r], mt[r]);
                m_ref[r] = m_new == -INFINITY ? 0.0f : m_new;
                alpha[r] = m_run[r] == -INFINITY ? 0.0f : exp2f(m_run[r] - m_ref[r]);
                m_run[r] = m_new;
            }
            float lsum[2] = {0.0f, 0.0f};
#pragma unroll
            for (int n = 0; n < NKT; ++n)
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const float p = s[n][e] == -INFINITY ? 0.0f : exp2f(s[n][e] - m_ref[e >> 1]);
                    lsum[e >> 1] += p;
                    s[n][e] = p * PM_PSCALE;
                }
            l_run[0] = l_run[0] * alpha[0] + lsum[0];
            l_run[1] = l_run[1] * alpha[1] + lsum[1];
#pragma unroll
            for (int n = 0; n < NTD; ++n) {
                o[n][0] *= alpha[0]; o[n][1] *= alpha[0];
                o[n][2] *= alpha[1]; o[n][3] *= alpha[1];
            }
            // probabilities x values, 16 keys per step
#pragma unroll
            for (int kk = 0; kk < NKT / 2; ++kk) {
                if (2 * kk < nt_lim) {
                    uint32_t aph[4], apl[4];
                    pm_split2(s[2 * kk][0], s[2 * kk][1], aph[0], apl[0]);             // row g, keys 2t, 2t + 1
                    pm_split2(s[2 * kk][2], s[2 * kk][3], aph[1], apl[1]);             // row g + 8
                    pm_split2(s[2 * kk + 1][0], s[2 * kk + 1][1], aph[2], apl[2]);     // row g, keys 2t + 8, 2t + 9
                    pm_split2(s[2 * kk + 1][2], s[2 * kk + 1][3], aph[3], apl[3]);
#pragma unroll
                    for (int n2 = 0; n2 < NTD / 2; ++n2) {
                        // transposed matrices: (keys 16kk .., d 8(2 n2) ..), (keys 16kk + 8 .., same d), (keys 16kk .., d 8(2 n2 + 1) ..), (keys 16kk + 8 .., ..)
                        const uint32_t addr = st + 2 * TILE + (uint32_t)((koff + 16 * kk + 8 * (mi & 1) + rr) * PITCH + (8 * (2 * n2 + (mi >> 1))) * 2);
                        uint32_t vh4[4], vl4[4];
                        pm_ldmatrix_t(vh4, addr);
                        pm_ldmatrix_t(vl4, addr + TILE);
                        pm_mma(o[2 * n2], aph, vh4[0], vh4[1]);
                        pm_mma(o[2 * n2], apl, vh4[0], vh4[1]);
                        pm_mma(o[2 * n2], aph, vl4[0], vl4[1]);
                        pm_mma(o[2 * n2 + 1], aph, vh4[2], vh4[3]);
                        pm_mma(o[2 * n2 + 1], apl, vh4[2], vh4[3]);
                        pm_mma(o[2 * n2 + 1], aph, vl4[2], vl4[3]);
                    }
                }
            }
        }
        __syncthreads();                                               // the stage may be refilled (and, after the last tile, reused below)
    }

#pragma unroll
    for (int r = 0; r < 2; ++r) {
        l_run[r] += __shfl_xor_sync(0xffffffffu, l_run[r], 1);
        l_run[r] += __shfl_xor_sync(0xffffffffu, l_run[r], 2);
    }
    if (KH == 2) {
        // the second key part hands (m, l, o) to the first through shared memory: [head][value][lane]
        constexpr int VALS = NTD * 4 + 4;
        float *mb = reinterpret_cast<float *>(pm_smem) + (size_t)(warp - part * G) * VALS * 32 + lane;
        if (part == 1) {
#pragma unroll
            for (int n = 0; n < NTD; ++n)
#pragma unroll
                for (int e = 0; e < 4; ++e) mb[(n * 4 + e) * 32] = o[n][e];
            mb[(NTD * 4 + 0) * 32] = m_run[0]; mb[(NTD * 4 + 1) * 32] = m_run[1];
            mb[(NTD * 4 + 2) * 32] = l_run[0]; mb[(NTD * 4 + 3) * 32] = l_run[1];
        }
        __syncthreads();
        if (part == 1) return;
        float w0[2], w1[2];
#pragma unroll
        for (int r = 0; r < 2; ++r) {
            const float m1 = mb[(NTD * 4 + r) * 32], l1 = mb[(NTD * 4 + 2 + r) * 32];
            const float m = fmaxf(m_run[r], m1);
            w0[r] = m_run[r] == -INFINITY ? 0.0f : exp2f(m_run[r] - m);
            w1[r] = m1 == -INFINITY ? 0.0f : exp2f(m1 - m);
            l_run[r] = l_run[r] * w0[r] + l1 * w1[r];
        }
#pragma unroll
        for (int n = 0; n < NTD; ++n)
#pragma unroll
            for (int e = 0; e < 4; ++e) o[n][e] = o[n][e] * w0[e >> 1] + mb[(n * 4 + e) * 32] * w1[e >> 1];
    }
    const float inv0 = l_run[0] > 0.0f ? 1.0f / (l_run[0] * PM_PSCALE) : 0.0f, inv1 = l_run[1] > 0.0f ? 1.0f / (l_run[1] * PM_PSCALE) : 0.0f;
#pragma unroll
    for (int n = 0; n < NTD; ++n) {
        const int d = 8 * n + 2 * t;
        if (q0 + g < T) *reinterpret_cast<float2 *>(out + ((size_t)h * T + q0 + g) * AD + d) = make_float2(o[n][0] * inv0, o[n][1] * inv0);
        if (q0 + g + 8 < T) *reinterpret_cast<float2 *>(out + ((size_t)h * T + q0 + g + 8) * AD + d) = make_float2(o[n][2] * inv1, o[n][3] * inv1);
    }
}

template <int AD, int KH>
static int pm_launch(const float *q, const float *k, const float *v, float *out, int H, int Hkv, int T, int hd, int kv_stride, int causal, float scale, cudaStream_t st)
{
    constexpr int smem = 2 * 4 * PM_BK * (AD + 8) * 2;
    static_assert(8 * (AD / 8 * 4 + 4) * 32 * 4 <= smem, "the merge buffer of up to 8 heads fits into the stages");
    static bool attr_set = false;
    if (!attr_set) {
        if (ckb_check_cuda((int)cudaFuncSetAttribute(attn_prefill_mma_kernel<AD, KH>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem), "attn_prefill_mma smem")) return CKB_ERR_CUDA;
        attr_set = true;
    }
    const size_t arr = (size_t)Hkv * T * AD;
    __half *kv16 = (__half *)ckb_scratch(CKB_SLOT_S, 4 * arr * sizeof(__half));
    if (!kv16) return CKB_ERR_CUDA;
    const size_t n4 = arr / 4;
    const unsigned blocks = (unsigned)((n4 + 255) / 256 < 8 * 148 ? (n4 + 255) / 256 : 8 * 148);
    if (int rc = launch_pdl("attn_prefill_split_kv", pm_split_kv_kernel<AD>, dim3(blocks), dim3(256), 0, st, k, v, kv16, Hkv, T, hd, kv_stride)) return rc;
    return launch_pdl("attn_prefill_mma", attn_prefill_mma_kernel<AD, KH>, dim3(Hkv, (T + PM_BQ - 1) / PM_BQ), dim3(32 * KH * (H / Hkv)), (size_t)smem, st, q,
                      (const __half *)kv16, out, H, Hkv, T, hd, causal, scale);
}

}  // namespace ckb

using namespace ckb;

// Arguments as ckb200_dev_attention_prefill (no sliding window).  Returns -1 when this kernel does not take the call.
extern "C" int ckb_launch_attn_prefill_mma(const float *q, const float *k, const float *v, float *out, int num_heads, int num_kv_heads, int num_tokens, int head_dim,
                                           int aligned_head_dim, int kv_stride_tokens, int causal, void *stream)
{
    if (!ckb_tune_get("attn_prefill_mma", 1) || num_heads % num_kv_heads || num_heads / num_kv_heads > 8) return -1;
    if ((aligned_head_dim != 64 && aligned_head_dim != 128) || (((uintptr_t)q | (uintptr_t)k | (uintptr_t)v | (uintptr_t)out) & 15)) return -1;
    const float scale = 1.0f / sqrtf((float)head_dim);
    cudaStream_t st = ckb_stream(stream);
    if (num_heads / num_kv_heads <= 4)                     // two warps per query head, 32 keys of a tile each
        return aligned_head_dim == 64 ? pm_launch<64, 2>(q, k, v, out, num_heads, num_kv_heads, num_tokens, head_dim, kv_stride_tokens, causal, scale, st)
                                      : pm_launch<128, 2>(q, k, v, out, num_heads, num_kv_heads, num_tokens, head_dim, kv_stride_tokens, causal, scale, st);
    return aligned_head_dim == 64 ? pm_launch<64, 1>(q, k, v, out, num_heads, num_kv_heads, num_tokens, head_dim, kv_stride_tokens, causal, scale, st)
                                  : pm_launch<128, 1>(q, k, v, out, num_heads, num_kv_heads, num_tokens, head_dim, kv_stride_tokens, causal, scale, st);
}
