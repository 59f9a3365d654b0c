// Decode attention over IEEE fp16 KV caches on the tensor cores (attention_forward_decode_head_major_gqa_flash_f16cache,
// src/kernels/attention_kernels.c:3450-3557), at fp32 accuracy.
//
// The tile kernel of attention_tile.cu widens an fp16 cache to fp32 and then does the fp32 kernel's work, so halving the cache bytes
// does not show up as time (it is bound by its multiply-add, shuffle and shared-memory issue).  With fp16 keys and values the products
// can go to the tensor cores without giving up accuracy, because a product of two fp16 numbers is exact in the fp32 accumulator:
//   * scores: the query row (pre-multiplied by scale * log2 e) is split into two fp16 pieces, q = q_hi + q_lo (22 significant bits);
//     the M = 16 rows of mma.sync.m16n8k16 are the hi pieces of the up to 8 query heads of a kv head and, below them, their lo
//     pieces; a lane holds both results of a head for its keys and adds them;
//   * values: the probabilities of a tile, times 2^14 so that their lo pieces stay out of fp16's subnormal range, are split the same
//     way straight out of the score registers (the accumulator layout of one MMA is the A layout of the next); the 16 output rows are
//     again hi and lo of the 8 heads and are added at the end.
// Keys and values of a 64-key tile come as 128-byte-swizzled tiled bulk copies (the rows of a kv head are contiguous in the cache:
// a 3-d tensor ad x rows x sequences), fragments by ldmatrix (transposed for the values); each of the four warps takes 16 keys of the
// tile with its own running maximum and sum, the warps and then the splits are merged exactly (log-sum-exp) as in the fp32 path.
// CTA per (split, kv head, sequence), three stages of 32 KB, two CTAs per SM.  Waits on the copies are bounded.
//
// The same kernel serves fp32 caches (F32 = true): a key or value element is split into two fp16 pieces like the query, k = k_hi + k_lo,
// when a lane builds its B fragment from the fp32 tile, and every product takes two instructions (A x hi, A x lo) - twice the
// tensor-core work and some conversions, which still fit under the time HBM needs for twice the bytes.  fp16's range applies to
// the pieces: cache values of magnitude 65504 or more are not supported by this form (the tile kernel of attention_tile.cu is).
#include <cuda.h>
#include <cuda_fp16.h>

#include "attention_params.cuh"
#include "launch.h"
#include "pdl.cuh"
#include "runtime.h"

namespace ckb {

constexpr int FM_WARPS = 4, FM_THREADS = 32 * FM_WARPS, FM_TILE = 64, FM_STAGES = 3;
constexpr float FM_PSCALE = 16384.0f;

__device__ __forceinline__ void fm_tma_3d(uint32_t dst, const CUtensorMap *map, int x, int y, int z, uint32_t bar)
{
    asm volatile("cp.async.bulk.tensor.3d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4}], [%5];"
                 ::"r"(dst), "l"(map), "r"(x), "r"(y), "r"(z), "r"(bar) : "memory");
}
__device__ __forceinline__ void fm_ldmatrix(uint32_t (&r)[4], uint32_t addr)
{
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void fm_ldmatrix_t(uint32_t (&r)[4], uint32_t addr)
{
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void fm_mma(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1)
{
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3]) : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
// x = hi + lo with hi = fp16(x), lo = fp16(x - hi); packs (hi(a), hi(b)) and (lo(a), lo(b))
__device__ __forceinline__ void fm_split2(float a, float b, uint32_t &hi, uint32_t &lo)
{
    const __half2 h = __floats2half2_rn(a, b);
    const float2 hf = __half22float2(h);
    const __half2 l = __floats2half2_rn(a - hf.x, b - hf.y);
    hi = *reinterpret_cast<const uint32_t *>(&h);
    lo = *reinterpret_cast<const uint32_t *>(&l);
}

// byte offset of the 16-byte chunk (row r, chunk c) in a 128-byte-swizzled box of 128-byte rows
__device__ __forceinline__ uint32_t fm_swz(int r, int c) { return (uint32_t)(r * 128 + ((c ^ (r & 7)) << 4)); }

template <int AD, bool F32>
__global__ void __launch_bounds__(FM_THREADS, F32 ? 1 : 2) attn_f16mma_kernel(const __grid_constant__ CUtensorMap tm_k, const __grid_constant__ CUtensorMap tm_v, AttnParams p,
                                                                    int *__restrict__ dev_err, int early_trigger)
{
    constexpr int BOXES = F32 ? AD / 32 : AD / 64;             // 128 bytes of a row per box: 64 halves or 32 floats
    constexpr int BOX_BYTES = FM_TILE * 128;                   // 8 KB
    constexpr int STAGE = 2 * BOXES * BOX_BYTES;               // K boxes, then V boxes
    constexpr int KS = AD / 16, NTD = AD / 8;
    extern __shared__ __align__(16) uint8_t fm_smem_raw[];
    __shared__ __align__(8) uint64_t full[FM_STAGES];
    // the swizzle pattern is a function of the shared-memory address: boxes must start on 1024-byte boundaries (the launch asks for 1 KB more)
    uint8_t *fm_smem = fm_smem_raw + ((1024u - (smem_u32(fm_smem_raw) & 1023u)) & 1023u);
    const uint32_t s_base = smem_u32(fm_smem);
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, g = lane >> 2, t = lane & 3;
    const int split = blockIdx.x, kvh = blockIdx.y, b = blockIdx.z;
    const int G = p.H / p.Hkv, h0 = kvh * G;

    if (tid == 0) {
        for (int i = 0; i < FM_STAGES; ++i) mbar_init(smem_u32(&full[i]), 1);
        mbar_fence_init();
    }
    __syncthreads();
    if (early_trigger) pdl_trigger();
    pdl_wait();                                                // q and the newest cache row come from the kernels before this one

    const int T = attn_kv_tokens(p);
    const int tiles_total = (T + FM_TILE - 1) / FM_TILE, tps = (tiles_total + p.splits - 1) / p.splits;
    const int tile0 = split * tps, tile1 = min(tiles_total, tile0 + tps), ntiles = max(0, tile1 - tile0);

    auto issue = [&](int i) {                                  // thread 0: tile tile0 + i into stage i % FM_STAGES
        const uint32_t bar = smem_u32(&full[i % FM_STAGES]), st = s_base + (uint32_t)(i % FM_STAGES) * STAGE;
        const int row = kvh * p.cap + (tile0 + i) * FM_TILE;
        mbar_arrive_expect_tx(bar, STAGE);
#pragma unroll
        for (int x = 0; x < BOXES; ++x) {
            fm_tma_3d(st + x * BOX_BYTES, &tm_k, (F32 ? 32 : 64) * x, row, b, bar);
            fm_tma_3d(st + (BOXES + x) * BOX_BYTES, &tm_v, (F32 ? 32 : 64) * x, row, b, bar);
        }
    };
    if (tid == 0)
        for (int i = 0; i < FM_STAGES - 1 && i < ntiles; ++i) issue(i);

    // query fragments: rows 0..7 the hi pieces of heads h0 .. h0 + 7, rows 8..15 their lo pieces; lane (g, t) holds head g
    uint32_t aq[KS][4];
    {
        const float qs = p.scale * 1.44269504088896340736f;
        const float *qr = p.q + ((size_t)b * p.H + h0 + min(g, G - 1)) * AD;
#pragma unroll
        for (int ks = 0; ks < KS; ++ks) {
            float2 u = make_float2(0.f, 0.f), w = u;
            if (g < G) {
                u = __ldcg(reinterpret_cast<const float2 *>(qr + 16 * ks + 2 * t));
                w = __ldcg(reinterpret_cast<const float2 *>(qr + 16 * ks + 2 * t + 8));
            }
            fm_split2(u.x * qs, u.y * qs, aq[ks][0], aq[ks][1]);
            fm_split2(w.x * qs, w.y * qs, aq[ks][2], aq[ks][3]);
        }
    }

    float o[NTD][4];
#pragma unroll
    for (int n = 0; n < NTD; ++n)
#pragma unroll
        for (int e = 0; e < 4; ++e) o[n][e] = 0.0f;
    float m_run = -INFINITY, l_run = 0.0f;                     // running maximum (log2 units) of head g over this warp's keys; this lane's share of the sum
    bool ok = true;

    // which rows and chunks this lane addresses for ldmatrix: matrix (lane >> 3), row (lane & 7) of it
    const int mi = lane >> 3, rr = lane & 7;
    for (int i = 0; i < ntiles; ++i) {
        __syncthreads();                                       // tile i - 1 is finished everywhere: its stage may be refilled
        if (tid == 0 && i + FM_STAGES - 1 < ntiles) issue(i + FM_STAGES - 1);
        if (ok && !mbar_wait_spin(smem_u32(&full[i % FM_STAGES]), (uint32_t)(i / FM_STAGES) & 1u)) {
            ok = false;
            if (lane == 0) atomicExch(dev_err, DEV_ERR_FULL_WAIT);
        }
        const uint32_t st = s_base + (uint32_t)(i % FM_STAGES) * STAGE;
        const int key0 = (tile0 + i) * FM_TILE + 16 * warp;   // first key of this warp's slice
        if (key0 + 16 > T) {
            // the last tile: rows past the context hold whatever the cache holds; their probabilities are zero, but 0 x inf would not be
            uint8_t *vb = fm_smem + (size_t)(i % FM_STAGES) * STAGE + BOXES * BOX_BYTES;
            for (int x = lane; x < 16 * 8 * BOXES; x += 32) {
                const int r = 16 * warp + (x >> 3) % 16, box = (x >> 3) / 16, c = x & 7;
                if (key0 - 16 * warp + r >= T) *reinterpret_cast<uint4 *>(vb + box * BOX_BYTES + fm_swz(r, c)) = make_uint4(0u, 0u, 0u, 0u);
            }
            __syncwarp();
        }

        // scores of 16 keys x 8 heads (hi and lo rows)
        float s[2][4];
#pragma unroll
        for (int n = 0; n < 2; ++n)
#pragma unroll
            for (int e = 0; e < 4; ++e) s[n][e] = 0.0f;
#pragma unroll
        for (int ks = 0; ks < KS; ++ks) {
            if constexpr (F32) {
                // lane (g, t) of key tile n: key 8n + g, elements 16ks + 2t, + 1 (b0) and + 8, + 9 (b1): two 8-byte loads, split into pieces
                const uint8_t *tile = fm_smem + (size_t)(i % FM_STAGES) * STAGE;
#pragma unroll
                for (int n = 0; n < 2; ++n) {
                    const int r = 16 * warp + 8 * n + g, f0 = 16 * ks + 2 * t, f1 = f0 + 8;
                    const float2 k0 = *reinterpret_cast<const float2 *>(tile + (f0 >> 5) * BOX_BYTES + fm_swz(r, (f0 & 31) >> 2) + (f0 & 3) * 4);
                    const float2 k1 = *reinterpret_cast<const float2 *>(tile + (f1 >> 5) * BOX_BYTES + fm_swz(r, (f1 & 31) >> 2) + (f1 & 3) * 4);
                    uint32_t h0, l0, h1, l1;
                    fm_split2(k0.x, k0.y, h0, l0);
                    fm_split2(k1.x, k1.y, h1, l1);
                    fm_mma(s[n], aq[ks], h0, h1);
                    fm_mma(s[n], aq[ks], l0, l1);
                }
            } else {
                // matrices: (keys 0-7, d chunk 2ks), (keys 0-7, chunk 2ks + 1), (keys 8-15, chunk 2ks), (keys 8-15, chunk 2ks + 1)
                const int r = 16 * warp + (mi >> 1) * 8 + rr, chunk = 2 * ks + (mi & 1);
                uint32_t kb[4];
                fm_ldmatrix(kb, st + (chunk >> 3) * BOX_BYTES + fm_swz(r, chunk & 7));
                fm_mma(s[0], aq[ks], kb[0], kb[1]);
                fm_mma(s[1], aq[ks], kb[2], kb[3]);
            }
        }
        float sc[2][2];
        float mt = -INFINITY;
#pragma unroll
        for (int n = 0; n < 2; ++n)
#pragma unroll
            for (int e = 0; e < 2; ++e) {
                const int key = key0 + 8 * n + 2 * t + e;
                const float v = s[n][e] + s[n][e + 2];
                sc[n][e] = key < T ? v : -INFINITY;            // a select: NaN scores of rows past the context are dropped too
                mt = fmaxf(mt, sc[n][e]);
            }
        mt = fmaxf(mt, __shfl_xor_sync(0xffffffffu, mt, 1));
        mt = fmaxf(mt, __shfl_xor_sync(0xffffffffu, mt, 2));
        const float m_new = fmaxf(m_run, mt);
        const float m_ref = m_new == -INFINITY ? 0.0f : m_new;
        const float alpha = m_run == -INFINITY ? 0.0f : exp2f(m_run - m_ref);
        float pr[2][2];
        float lsum = 0.0f;
#pragma unroll
        for (int n = 0; n < 2; ++n)
#pragma unroll
            for (int e = 0; e < 2; ++e) {
                pr[n][e] = sc[n][e] == -INFINITY ? 0.0f : exp2f(sc[n][e] - m_ref);
                lsum += pr[n][e];
            }
        l_run = l_run * alpha + lsum;
        m_run = m_new;
#pragma unroll
        for (int n = 0; n < NTD; ++n)
#pragma unroll
            for (int e = 0; e < 4; ++e) o[n][e] *= alpha;
        // probabilities as the A operand: rows = heads (hi) / heads (lo), k = the 16 keys
        uint32_t ap[4];
        fm_split2(pr[0][0] * FM_PSCALE, pr[0][1] * FM_PSCALE, ap[0], ap[1]);
        fm_split2(pr[1][0] * FM_PSCALE, pr[1][1] * FM_PSCALE, ap[2], ap[3]);
        if constexpr (F32) {
            // lane (g, t) of output tile n: element 8n + g of keys 2t, 2t + 1 (b0) and 2t + 8, 2t + 9 (b1): four 4-byte loads, no bank conflicts
            const uint8_t *tile = fm_smem + (size_t)(i % FM_STAGES) * STAGE + BOXES * BOX_BYTES;
#pragma unroll
            for (int n = 0; n < NTD; ++n) {
                const int f = 8 * n + g, r = 16 * warp + 2 * t;
                const uint8_t *col = tile + (f >> 5) * BOX_BYTES + (f & 3) * 4;
                const int c = (f & 31) >> 2;
                const float v0 = *reinterpret_cast<const float *>(col + fm_swz(r, c)), v1 = *reinterpret_cast<const float *>(col + fm_swz(r + 1, c));
                const float v2 = *reinterpret_cast<const float *>(col + fm_swz(r + 8, c)), v3 = *reinterpret_cast<const float *>(col + fm_swz(r + 9, c));
                uint32_t h0, l0, h1, l1;
                fm_split2(v0, v1, h0, l0);
                fm_split2(v2, v3, h1, l1);
                fm_mma(o[n], ap, h0, h1);
                fm_mma(o[n], ap, l0, l1);
            }
        } else {
#pragma unroll
            for (int n2 = 0; n2 < NTD / 2; ++n2) {
                // transposed matrices: (keys 0-7, d chunk 2 n2), (keys 8-15, same chunk), (keys 0-7, chunk 2 n2 + 1), (keys 8-15, chunk 2 n2 + 1)
                const int r = 16 * warp + (mi & 1) * 8 + rr, chunk = 2 * n2 + (mi >> 1);
                uint32_t vb[4];
                fm_ldmatrix_t(vb, st + (BOXES + (chunk >> 3)) * BOX_BYTES + fm_swz(r, chunk & 7));
                fm_mma(o[2 * n2], ap, vb[0], vb[1]);
                fm_mma(o[2 * n2 + 1], ap, vb[2], vb[3]);
            }
        }
    }
    __syncthreads();                                           // all copies have landed and been used: the stages become the merge buffer
    // The kernels behind this one start now, not earlier: this kernel fills the shared memory of every SM it runs on, so dependents
    // that were launched early could not become resident beside it and would only queue in front of its own remaining CTAs.
    if (!early_trigger) pdl_trigger();

    // merge the four warps: [warp][head][AD + 2] floats (output, maximum, sum)
    float *mg = reinterpret_cast<float *>(fm_smem);
    l_run += __shfl_xor_sync(0xffffffffu, l_run, 1);
    l_run += __shfl_xor_sync(0xffffffffu, l_run, 2);
    {
        float *dst = mg + ((size_t)warp * 8 + g) * (AD + 2);
#pragma unroll
        for (int n = 0; n < NTD; ++n) {
            dst[8 * n + 2 * t] = o[n][0] + o[n][2];
            dst[8 * n + 2 * t + 1] = o[n][1] + o[n][3];
        }
        if (t == 0) { dst[AD] = m_run; dst[AD + 1] = l_run; }
    }
    __syncthreads();
    for (int idx = tid; idx < G * AD; idx += FM_THREADS) {
        const int hg = idx / AD, c = idx - hg * AD;
        float mm = -INFINITY;
#pragma unroll
        for (int w = 0; w < FM_WARPS; ++w) mm = fmaxf(mm, mg[((size_t)w * 8 + hg) * (AD + 2) + AD]);
        float acc = 0.0f, ll = 0.0f;
#pragma unroll
        for (int w = 0; w < FM_WARPS; ++w) {
            const float *src = mg + ((size_t)w * 8 + hg) * (AD + 2);
            const float f = src[AD] == -INFINITY ? 0.0f : exp2f(src[AD] - mm);
            acc = fmaf(src[c], f, acc);
            ll = fmaf(src[AD + 1], f, ll);
        }
        acc *= 1.0f / FM_PSCALE;
        const size_t head = (size_t)b * p.H + h0 + hg;
        if (p.splits == 1) {
            p.out[head * AD + c] = ll > 0.0f ? acc / ll : 0.0f;
        } else {
            float *dst = p.part + (head * p.splits + split) * (AD + 2);
            dst[c] = acc;
            if (c == 0) {
                dst[AD] = mm == -INFINITY ? -INFINITY : mm * 0.69314718055994530942f;      // the merge kernel works in natural-log units
                dst[AD + 1] = ll;
            }
        }
    }
}

typedef CUresult (*fm_encode_fn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *, const cuuint64_t *, const cuuint32_t *,
                                 const cuuint32_t *, CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
static fm_encode_fn fm_encoder()
{
    static fm_encode_fn fn = nullptr;
    static bool tried = false;
    if (!tried) {
        tried = true;
        void *ptr = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &q) == cudaSuccess && q == cudaDriverEntryPointSuccess) fn = (fm_encode_fn)ptr;
        else cudaGetLastError();
    }
    return fn;
}
// a cache [batch][Hkv * cap rows][ad] of `eb`-byte elements with `batch_stride` elements between sequences: boxes of 128 bytes x 64 rows, 128-byte swizzle
static bool fm_make_map(CUtensorMap *map, const void *base, int ad, long long rows, int batch, long long batch_stride, int eb)
{
    fm_encode_fn enc = fm_encoder();
    if (!enc) return false;
    const cuuint64_t dims[3] = {(cuuint64_t)ad, (cuuint64_t)rows, (cuuint64_t)batch};
    const cuuint64_t strides[2] = {(cuuint64_t)ad * eb, (cuuint64_t)batch_stride * eb};
    const cuuint32_t box[3] = {(cuuint32_t)(128 / eb), FM_TILE, 1}, estr[3] = {1, 1, 1};
    return enc(map, eb == 4 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32 : CU_TENSOR_MAP_DATA_TYPE_UINT16, 3, const_cast<void *>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
               CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

template <int AD, bool F32>
static int fm_launch(const AttnParams *p, int batch, const CUtensorMap &tk, const CUtensorMap &tv, cudaStream_t st)
{
    constexpr int stages = FM_STAGES * 2 * (F32 ? AD / 32 : AD / 64) * FM_TILE * 128, smem = stages + 1024;
    static_assert(smem <= 227 * 1024, "shared memory");
    static_assert(FM_WARPS * 8 * (AD + 2) * 4 <= stages, "the merge buffer fits into the stages");
    static bool attr_set = false;
    if (!attr_set) {
        if (ckb_check_cuda((int)cudaFuncSetAttribute(attn_f16mma_kernel<AD, F32>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem), "attn_f16mma smem")) return CKB_ERR_CUDA;
        attr_set = true;
    }
    const int mode = ckb_tune_get("attn_f16_mma_pdl", 1);      // 1: programmatic dependent launch, trigger after the key loop; 2: trigger at the start; 0: plain launch
    if (mode == 0) {
        attn_f16mma_kernel<AD, F32><<<dim3(p->splits, p->Hkv, batch), dim3(FM_THREADS), (size_t)smem, st>>>(tk, tv, *p, ckb_device_error_word(), 0);
        return ckb_check_launch("attn_f16mma");
    }
    return launch_pdl("attn_f16mma", attn_f16mma_kernel<AD, F32>, dim3(p->splits, p->Hkv, batch), dim3(FM_THREADS), (size_t)smem, st, tk, tv, *p, ckb_device_error_word(),
                      mode == 2 ? 1 : 0);
}

}  // namespace ckb

using namespace ckb;

// p as for the tile kernel (with kv_f16 = 1: k and v point at fp16 data; kv_batch_stride in elements; part sized for p->splits).
// Returns -1 when this kernel does not take the call: the caller runs the tile kernel.
extern "C" int ckb_launch_attn_f16mma(const AttnParams *p, int batch, void *stream)
{
    // One sequence stays with the tile kernel: inside a decode step it is the faster of the two there (11.5 against 11.9 ms per token on
    // the 70B shape: it fetches the older cache rows before its predecessor has finished), from a few sequences up this one wins clearly.
    const int eb = p->kv_f16 ? 2 : 4;
    if (!ckb_tune_get(p->kv_f16 ? "attn_f16_mma" : "attn_f32_mma", 1) || batch < ckb_tune_get("attn_f16_mma_min_batch", 2)) return -1;
    if ((p->ad != 64 && p->ad != 128) || p->H % p->Hkv || p->H / p->Hkv > 8) return -1;
    if ((((uintptr_t)p->k | (uintptr_t)p->v) & 15) || (p->kv_batch_stride * eb) % 16 || ((uintptr_t)p->q & 7) || p->counters || p->q8_out) return -1;
    const long long rows = (long long)p->Hkv * p->cap;
    if (batch > 1 && rows * p->ad > p->kv_batch_stride) return -1;
    const long long stride = batch > 1 ? p->kv_batch_stride : rows * p->ad;
    CUtensorMap tk, tv;
    if (!fm_make_map(&tk, p->k, p->ad, rows, batch, stride, eb) || !fm_make_map(&tv, p->v, p->ad, rows, batch, stride, eb)) return -1;
    cudaStream_t st = ckb_stream(stream);
    if (p->kv_f16) return p->ad == 64 ? fm_launch<64, false>(p, batch, tk, tv, st) : fm_launch<128, false>(p, batch, tk, tv, st);
    return p->ad == 64 ? fm_launch<64, true>(p, batch, tk, tv, st) : fm_launch<128, true>(p, batch, tk, tv, st);
}
