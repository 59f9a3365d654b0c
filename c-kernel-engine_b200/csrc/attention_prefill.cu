// Causal (and full) prefill attention over head-major fp32 tensors: the reference's
// attention_forward_causal_head_major_gqa_flash[_strided] / attention_forward_full_head_major_gqa_flash
// (src/kernels/attention_kernels.c:2847-2985): q and out [H][T][ad], K and V [Hkv][kv_stride_tokens][ad], query token i
// of head h attends keys 0 .. i (causal) or 0 .. T-1 of kv head h * Hkv / H with online softmax, scale 1/sqrt(head_dim),
// dot products over head_dim, output pad [head_dim, ad) written as zero (:1546-1602).
//
// One CTA owns one kv head and a block of BT query tokens for all G = H / Hkv query heads of that kv head, so a K/V tile
// staged in shared memory is used by BT * G query rows.  Four lanes share a pair of query rows (the same head, two
// consecutive tokens): each lane keeps a quarter of both query vectors and of both output accumulators in registers,
// reads its quarter of a key (value) once for both rows (a 64-byte broadcast per row pair), and the four partial dot
// products meet in two shuffles.  Keys are taken four at a time (eight independent dot products, one branch-free softmax
// update per block), because a row's keys are a serial chain and the longest CTA sets the kernel's time.  fp32
// arithmetic on the CUDA cores: the reference's tolerance (1e-3 relative on fp32 outputs) leaves no room for fp16/tf32
// score rounding under the exponential.
#include <math.h>

#include "device_common.cuh"
#include "launch.h"
#include "runtime.h"

namespace ckb {

constexpr int AP_BK = 32;            // keys per shared tile
constexpr int AP_MAX_GROUP = 8;      // query heads per kv head on this path

template <int AD>
__global__ void __launch_bounds__(256) attn_prefill_kernel(const float *__restrict__ q, const float *__restrict__ k, const float *__restrict__ v,
                                                           float *__restrict__ out, int H, int Hkv, int T, int head_dim, int kv_stride, int BT, float scale,
                                                           int causal, int window, int nsets)
{
    extern __shared__ __align__(16) float4 ap_smem[];
    constexpr int P = AD / 4;        // float4 pieces per row
    constexpr int NV = AD / 16;      // pieces per lane
    float4 *Ks = ap_smem, *Vs = ap_smem + AP_BK * P;
    // token blocks are dealt from the last (most keys under the causal mask) to the first: the long CTAs start first
    const int G = H / Hkv, kvh = blockIdx.y, t0 = ((int)gridDim.x - 1 - (int)blockIdx.x) * BT;
    // two key sets: the second half of the CTA's threads holds the same rows and takes every other block of four keys, which
    // halves the serial chain of the longest (last) token block; the sets' partial results meet in shared memory at the end
    // (nsets == 2; group sizes whose two sets would not fit 256 threads run one set)
    const int rows_threads = (int)blockDim.x / nsets, ks = (int)threadIdx.x >= rows_threads ? 1 : 0, ltid = (int)threadIdx.x - ks * rows_threads;
    const int l4 = ltid & 3, grp = ltid >> 2, npairs = BT >> 1;
    const int g = grp / npairs, a = grp - g * npairs;
    const int tokA = t0 + 2 * a, tokB = tokA + 1, h = kvh * G + g;
    const bool rowA = g < G && tokA < T, rowB = g < G && tokB < T;

    float4 qA[NV], qB[NV], oA[NV], oB[NV];
#pragma unroll
    for (int i = 0; i < NV; ++i) {
        const int piece = l4 + 4 * i, d = 4 * piece;
        float4 x = make_float4(0.f, 0.f, 0.f, 0.f), y = x;
        if (rowA) x = __ldg(reinterpret_cast<const float4 *>(q + ((size_t)h * T + tokA) * AD) + piece);
        if (rowB) y = __ldg(reinterpret_cast<const float4 *>(q + ((size_t)h * T + tokB) * AD) + piece);
        if (d + 0 >= head_dim) { x.x = 0.f; y.x = 0.f; }
        if (d + 1 >= head_dim) { x.y = 0.f; y.y = 0.f; }
        if (d + 2 >= head_dim) { x.z = 0.f; y.z = 0.f; }
        if (d + 3 >= head_dim) { x.w = 0.f; y.w = 0.f; }
        qA[i] = x; qB[i] = y;
        oA[i] = make_float4(0.f, 0.f, 0.f, 0.f);
        oB[i] = oA[i];
    }
    float mA = -INFINITY, mB = -INFINITY, sA = 0.f, sB = 0.f;

    const int last_tok = min(T, t0 + BT) - 1;
    const int kend = causal ? last_tok + 1 : T;                       // keys 0 .. kend-1 are needed by some row of this CTA
    const int limA = causal ? tokA : T - 1, limB = causal ? tokB : T - 1;
    // sliding window (attention_kernels_sliding.c:391-402): token i sees keys max(0, i - window + 1) .. i
    const int loA = window > 0 ? max(0, tokA - window + 1) : 0, loB = window > 0 ? max(0, tokB - window + 1) : 0;
    const int kbegin = window > 0 ? (max(0, t0 - window + 1) / AP_BK) * AP_BK : 0;      // first tile any row of this CTA needs
    const float *kbase = k + (size_t)kvh * kv_stride * AD, *vbase = v + (size_t)kvh * kv_stride * AD;

    for (int k0 = kbegin; k0 < kend; k0 += AP_BK) {
        const int nk = min(AP_BK, kend - k0), nk4 = (nk + 3) & ~3;
        __syncthreads();                                              // the previous tile has been consumed
        for (int e = threadIdx.x; e < nk4 * P; e += blockDim.x) {     // keys past the end of the block's range read as zero
            const bool in = e < nk * P;
            Ks[e] = in ? __ldg(reinterpret_cast<const float4 *>(kbase + (size_t)k0 * AD) + e) : make_float4(0.f, 0.f, 0.f, 0.f);
            Vs[e] = in ? __ldg(reinterpret_cast<const float4 *>(vbase + (size_t)k0 * AD) + e) : make_float4(0.f, 0.f, 0.f, 0.f);
        }
        __syncthreads();
        // four keys at a time: eight independent dot products, one block-wise softmax update without branches
        for (int jj = 4 * ks; jj < nk4; jj += 4 * nsets) {
            float dA[4] = {0.f, 0.f, 0.f, 0.f}, dB[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
            for (int i = 0; i < NV; ++i) {
#pragma unroll
                for (int c = 0; c < 4; ++c) {
                    const float4 kk = Ks[(jj + c) * P + l4 + 4 * i];
                    dA[c] = fmaf(qA[i].x, kk.x, dA[c]); dA[c] = fmaf(qA[i].y, kk.y, dA[c]); dA[c] = fmaf(qA[i].z, kk.z, dA[c]); dA[c] = fmaf(qA[i].w, kk.w, dA[c]);
                    dB[c] = fmaf(qB[i].x, kk.x, dB[c]); dB[c] = fmaf(qB[i].y, kk.y, dB[c]); dB[c] = fmaf(qB[i].z, kk.z, dB[c]); dB[c] = fmaf(qB[i].w, kk.w, dB[c]);
                }
            }
            float nmA = mA, nmB = mB;
#pragma unroll
            for (int c = 0; c < 4; ++c) {
                dA[c] += __shfl_xor_sync(0xffffffffu, dA[c], 1); dB[c] += __shfl_xor_sync(0xffffffffu, dB[c], 1);
                dA[c] += __shfl_xor_sync(0xffffffffu, dA[c], 2); dB[c] += __shfl_xor_sync(0xffffffffu, dB[c], 2);
                const int j = k0 + jj + c;
                dA[c] = (j <= limA && j >= loA) ? dA[c] * scale : -INFINITY;
                dB[c] = (j <= limB && j >= loB) ? dB[c] * scale : -INFINITY;
                nmA = fmaxf(nmA, dA[c]);
                nmB = fmaxf(nmB, dB[c]);
            }
            // a row may have seen no key yet (its window starts later, or it lies past T): its maximum is still -inf
            const float cA = mA == -INFINITY ? 0.f : __expf(mA - nmA), cB = mB == -INFINITY ? 0.f : __expf(mB - nmB);
            mA = nmA; mB = nmB;
            float pA[4], pB[4];
#pragma unroll
            for (int c = 0; c < 4; ++c) {
                pA[c] = dA[c] == -INFINITY ? 0.f : __expf(dA[c] - nmA);
                pB[c] = dB[c] == -INFINITY ? 0.f : __expf(dB[c] - nmB);
            }
            sA = sA * cA + ((pA[0] + pA[1]) + (pA[2] + pA[3]));
            sB = sB * cB + ((pB[0] + pB[1]) + (pB[2] + pB[3]));
#pragma unroll
            for (int i = 0; i < NV; ++i) {
                float4 x = oA[i], y = oB[i];
                x.x *= cA; x.y *= cA; x.z *= cA; x.w *= cA;
                y.x *= cB; y.y *= cB; y.z *= cB; y.w *= cB;
#pragma unroll
                for (int c = 0; c < 4; ++c) {
                    const float4 vv = Vs[(jj + c) * P + l4 + 4 * i];
                    x.x = fmaf(pA[c], vv.x, x.x); x.y = fmaf(pA[c], vv.y, x.y); x.z = fmaf(pA[c], vv.z, x.z); x.w = fmaf(pA[c], vv.w, x.w);
                    y.x = fmaf(pB[c], vv.x, y.x); y.y = fmaf(pB[c], vv.y, y.y); y.z = fmaf(pB[c], vv.z, y.z); y.w = fmaf(pB[c], vv.w, y.w);
                }
                oA[i] = x; oB[i] = y;
            }
        }
    }

    // merge the two key sets: set 1 parks (max, sum, accumulators) in shared memory, set 0 combines them with its own
    if (nsets == 2) {
    __syncthreads();
    float4 *ms = ap_smem;                                              // [2 * NV + 1][rows_threads] float4
    if (ks == 1) {
#pragma unroll
        for (int i = 0; i < NV; ++i) { ms[i * rows_threads + ltid] = oA[i]; ms[(NV + i) * rows_threads + ltid] = oB[i]; }
        ms[2 * NV * rows_threads + ltid] = make_float4(mA, sA, mB, sB);
    }
    __syncthreads();
    if (ks == 1) return;
    {
        const float4 o = ms[2 * NV * rows_threads + ltid];
        const float nA = fmaxf(mA, o.x), nB = fmaxf(mB, o.z);
        const float fA0 = mA == -INFINITY ? 0.f : __expf(mA - nA), fA1 = o.x == -INFINITY ? 0.f : __expf(o.x - nA);
        const float fB0 = mB == -INFINITY ? 0.f : __expf(mB - nB), fB1 = o.z == -INFINITY ? 0.f : __expf(o.z - nB);
        sA = sA * fA0 + o.y * fA1;
        sB = sB * fB0 + o.w * fB1;
#pragma unroll
        for (int i = 0; i < NV; ++i) {
            const float4 a = ms[i * rows_threads + ltid], b = ms[(NV + i) * rows_threads + ltid];
            oA[i] = make_float4(oA[i].x * fA0 + a.x * fA1, oA[i].y * fA0 + a.y * fA1, oA[i].z * fA0 + a.z * fA1, oA[i].w * fA0 + a.w * fA1);
            oB[i] = make_float4(oB[i].x * fB0 + b.x * fB1, oB[i].y * fB0 + b.y * fB1, oB[i].z * fB0 + b.z * fB1, oB[i].w * fB0 + b.w * fB1);
        }
    }
    }
    const float iA = sA > 0.f ? 1.0f / sA : 0.f, iB = sB > 0.f ? 1.0f / sB : 0.f;
#pragma unroll
    for (int i = 0; i < NV; ++i) {
        const int piece = l4 + 4 * i, d = 4 * piece;
        float4 x = make_float4(oA[i].x * iA, oA[i].y * iA, oA[i].z * iA, oA[i].w * iA);
        float4 y = make_float4(oB[i].x * iB, oB[i].y * iB, oB[i].z * iB, oB[i].w * iB);
        if (d + 0 >= head_dim) { x.x = 0.f; y.x = 0.f; }
        if (d + 1 >= head_dim) { x.y = 0.f; y.y = 0.f; }
        if (d + 2 >= head_dim) { x.z = 0.f; y.z = 0.f; }
        if (d + 3 >= head_dim) { x.w = 0.f; y.w = 0.f; }
        if (rowA) reinterpret_cast<float4 *>(out + ((size_t)h * T + tokA) * AD)[piece] = x;
        if (rowB) reinterpret_cast<float4 *>(out + ((size_t)h * T + tokB) * AD)[piece] = y;
    }
}

}  // namespace ckb

using namespace ckb;

// q, out [H][T][ad]; k, v [Hkv][kv_stride_tokens][ad]; causal != 0: token i sees keys 0 .. i, else all T keys.
extern "C" int ckb_launch_attn_prefill_mma(const float *q, const float *k, const float *v, float *out, int num_heads, int num_kv_heads, int num_tokens, int head_dim,
                                           int aligned_head_dim, int kv_stride_tokens, int causal, void *stream);
extern "C" int ckb200_dev_attention_prefill_window(const float *q, const float *k, const float *v, float *out, int num_heads, int num_kv_heads,
                                                   int num_tokens, int head_dim, int aligned_head_dim, int kv_stride_tokens, int causal,
                                                   int sliding_window, void *stream)
{
    const int window = causal && sliding_window > 0 ? sliding_window : 0;
    if (!q || !k || !v || !out) return 0;
    if (num_heads <= 0 || num_kv_heads <= 0 || num_tokens <= 0 || kv_stride_tokens < num_tokens) return 0;      // the reference returns silently
    if (head_dim <= 0 || aligned_head_dim < head_dim) return 0;
    if (ckb_ensure_init()) return CKB_ERR_NO_DEVICE;
    const int G = num_heads / num_kv_heads;
    if (num_heads % num_kv_heads || G > AP_MAX_GROUP || (aligned_head_dim != 64 && aligned_head_dim != 128))
        return ckb_fail(CKB_ERR_SHAPE, "attention prefill: %d heads / %d kv heads / head size %d is outside this kernel (groups <= %d, aligned head size 64 or 128)",
                        num_heads, num_kv_heads, aligned_head_dim, AP_MAX_GROUP);
    if (((uintptr_t)q | (uintptr_t)k | (uintptr_t)v | (uintptr_t)out) & 15) return ckb_fail(CKB_ERR_ALIGN, "attention prefill: pointers must be 16-byte aligned");
    if (window == 0) {
        // without a sliding window: the tensor-core kernel of attention_prefill_mma.cu (-1: not for this call)
        const int rc = ckb_launch_attn_prefill_mma(q, k, v, out, num_heads, num_kv_heads, num_tokens, head_dim, aligned_head_dim, kv_stride_tokens, causal, stream);
        if (rc >= 0) return rc;
    }
    // 2 * BT * G threads per key set (a multiple of 32); two key sets when both fit 256 threads
    const int BT = G == 1 ? 64 : (G == 2 ? 32 : ((G == 6 || G == 8) ? 8 : 16));
    const int nsets = 2 * (2 * BT * G) <= 256 ? 2 : 1;
    const int threads = nsets * 2 * BT * G;
    const dim3 grid((num_tokens + BT - 1) / BT, num_kv_heads);
    const size_t tile_b = 2 * (size_t)AP_BK * aligned_head_dim * sizeof(float), merge_b = (size_t)(2 * (aligned_head_dim / 16) + 1) * (2 * BT * G) * 16;
    const size_t smem = tile_b > merge_b ? tile_b : merge_b;
    const float scale = 1.0f / sqrtf((float)head_dim);
    cudaStream_t st = ckb_stream(stream);
    if (aligned_head_dim == 64)
        attn_prefill_kernel<64><<<grid, threads, smem, st>>>(q, k, v, out, num_heads, num_kv_heads, num_tokens, head_dim, kv_stride_tokens, BT, scale, causal,
                                                             window, nsets);
    else
        attn_prefill_kernel<128><<<grid, threads, smem, st>>>(q, k, v, out, num_heads, num_kv_heads, num_tokens, head_dim, kv_stride_tokens, BT, scale, causal,
                                                              window, nsets);
    return ckb_check_launch("attn_prefill");
}

extern "C" int ckb200_dev_attention_prefill(const float *q, const float *k, const float *v, float *out, int num_heads, int num_kv_heads, int num_tokens,
                                            int head_dim, int aligned_head_dim, int kv_stride_tokens, int causal, void *stream)
{
    return ckb200_dev_attention_prefill_window(q, k, v, out, num_heads, num_kv_heads, num_tokens, head_dim, aligned_head_dim, kv_stride_tokens, causal, 0,
                                               stream);
}
