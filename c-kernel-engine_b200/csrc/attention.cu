// Decode attention over the head-major fp32 KV cache with GQA and split-K over the context.
//
// Replaces attention_forward_decode_head_major_gqa_flash (src/kernels/attention_kernels.c:3365-3406),
// which calls attention_flash_decode per Q head (src/kernels/attention_flash_true.c:142-230, :696-722):
// one query token, kv_head = h * Hkv / H, scores (q.k) / sqrt(head_dim), online softmax, out = P.V.
//
// Layout (the reference's memory plan): q [H][ad], K and V cache [Hkv][capacity][ad] fp32,
// out [H][ad]; ad = aligned_head_dim.  Batched form: `batch` independent sequences with their own
// q/out rows and cache slabs (strides given in floats).
//
// Fast path (ad = 64 or 128, group = H/Hkv <= 8): one CTA per (context split, kv head, sequence).
// A warp takes 2 keys per step, 16 lanes per key; each lane owns ad/16 dimensions as float4 pieces so
// that 16 lanes read 256 contiguous bytes, and the rows of the next step are loaded before the current
// step is computed.  K and V rows are read ONCE for all `group` Q heads that share the kv head.  The
// group partial dots are reduced with a transposing butterfly (8 shuffles for 8 heads); each lane keeps
// running (max, sum) for every head and `group` output accumulators for its dimensions.  Splits write (max, sum, unnormalised out) to a scratch buffer
// and a merge kernel combines them with the exact log-sum-exp rule.
#include "device_common.cuh"
#include "pdl.cuh"
#include "attention_params.cuh"

#include <math.h>

namespace ckb {

constexpr int ATTN_G = 8;        // max Q heads per kv head in the fast path
constexpr int ATTN_NW = 4;       // warps per CTA

template <int AD>
__global__ void __launch_bounds__(ATTN_NW * 32) attn_decode_kernel(AttnParams p)
{
    constexpr int LPK = 16;                    // lanes per key
    constexpr int C = AD / (4 * LPK);          // float4 pieces per lane (1 for 64, 2 for 128)
    constexpr int KPI = 32 / LPK;              // keys per warp step
    const int split = blockIdx.x, kvh = blockIdx.y, seq = blockIdx.z;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int sub = lane / LPK, li = lane % LPK;
    const int group = p.H / p.Hkv, h0 = kvh * group;   // heads h0 .. h0+group-1 map to kvh (H % Hkv == 0)

    __shared__ __align__(16) float q_s[ATTN_G][AD];
    __shared__ __align__(16) float merge_s[ATTN_NW][ATTN_G][AD + 4];   // row stride stays a multiple of 16 bytes

    // Launched programmatically: q and the newest cache row come from kernels that may still have been
    // running when this one started, so everything is read through L2 (__ldcg) after the wait.
    pdl_trigger();
    pdl_wait();
    for (int i = threadIdx.x; i < ATTN_G * AD; i += blockDim.x) {
        const int h = i / AD, c = i - h * AD;
        q_s[h][c] = h < group ? __ldcg(p.q + ((size_t)seq * p.H + h0 + h) * AD + c) * p.scale : 0.0f;
    }
    __syncthreads();

    const float *kbase = p.k + (size_t)seq * p.kv_batch_stride + (size_t)kvh * p.cap * AD;
    const float *vbase = p.v + (size_t)seq * p.kv_batch_stride + (size_t)kvh * p.cap * AD;
    const int kv_tokens = attn_kv_tokens(p);
    const int tokens_per_split = (((kv_tokens + p.splits - 1) / p.splits) + 3) & ~3;
    const int t_begin = split * tokens_per_split;
    const int t_end = min(kv_tokens, t_begin + tokens_per_split);

    float m[ATTN_G], l[ATTN_G];
    float4 acc[ATTN_G][C];
#pragma unroll
    for (int h = 0; h < ATTN_G; ++h) {
        m[h] = -INFINITY;
        l[h] = 0.0f;
#pragma unroll
        for (int c = 0; c < C; ++c) acc[h][c] = make_float4(0.f, 0.f, 0.f, 0.f);
    }

    auto load_kv = [&](float4 (&kr)[C], float4 (&vr)[C], int t) {
        const int tc = min(t, t_end - 1);
#pragma unroll
        for (int c = 0; c < C; ++c) {
            kr[c] = __ldcg(reinterpret_cast<const float4 *>(kbase + (size_t)tc * AD) + c * LPK + li);
            vr[c] = __ldcg(reinterpret_cast<const float4 *>(vbase + (size_t)tc * AD) + c * LPK + li);
        }
    };

    float4 kr[C], vr[C], kn[C], vn[C];
    int t0 = t_begin + warp * KPI;
    if (t0 < t_end) load_kv(kr, vr, t0 + sub);
    for (; t0 < t_end; t0 += ATTN_NW * KPI) {
        const int t = t0 + sub;
        const bool valid = t < t_end;
        if (t0 + ATTN_NW * KPI < t_end) load_kv(kn, vn, t + ATTN_NW * KPI);     // next step's rows are in flight during this one
        // partial dots of this lane's dimensions with every head's (pre-scaled) query
        float s[ATTN_G];
#pragma unroll
        for (int h = 0; h < ATTN_G; ++h) {
            float a = 0.0f;
#pragma unroll
            for (int c = 0; c < C; ++c) {
                const float4 qv = *reinterpret_cast<const float4 *>(&q_s[h][(c * LPK + li) * 4]);
                a = fmaf(qv.x, kr[c].x, a);
                a = fmaf(qv.y, kr[c].y, a);
                a = fmaf(qv.z, kr[c].z, a);
                a = fmaf(qv.w, kr[c].w, a);
            }
            s[h] = a;
        }
        // transposing butterfly over lane bits 2,1,0, then a plain add over bit 3: lane li ends with head li & 7
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const float mine = (li & 4) ? s[j + 4] : s[j], theirs = (li & 4) ? s[j] : s[j + 4];
            s[j] = mine + __shfl_xor_sync(0xffffffffu, theirs, 4);
        }
#pragma unroll
        for (int j = 0; j < 2; ++j) {
            const float mine = (li & 2) ? s[j + 2] : s[j], theirs = (li & 2) ? s[j] : s[j + 2];
            s[j] = mine + __shfl_xor_sync(0xffffffffu, theirs, 2);
        }
        {
            const float mine = (li & 1) ? s[1] : s[0], theirs = (li & 1) ? s[0] : s[1];
            s[0] = mine + __shfl_xor_sync(0xffffffffu, theirs, 1);
        }
        s[0] += __shfl_xor_sync(0xffffffffu, s[0], 8);
        const float score = valid ? s[0] : -INFINITY;     // head li & 7, key t
        // broadcast each head's score inside the key's lanes, update the running softmax
#pragma unroll
        for (int h = 0; h < ATTN_G; ++h) {
            const float sh = __shfl_sync(0xffffffffu, score, sub * LPK + h);
            if (h < group && sh > -INFINITY) {
                float pw;
                if (sh > m[h]) {
                    const float corr = expf(m[h] - sh);   // exp(-inf) = 0 on the first key
                    l[h] *= corr;
#pragma unroll
                    for (int c = 0; c < C; ++c) {
                        acc[h][c].x *= corr; acc[h][c].y *= corr; acc[h][c].z *= corr; acc[h][c].w *= corr;
                    }
                    m[h] = sh;
                    pw = 1.0f;
                } else {
                    pw = expf(sh - m[h]);
                }
                l[h] += pw;
#pragma unroll
                for (int c = 0; c < C; ++c) {
                    acc[h][c].x = fmaf(pw, vr[c].x, acc[h][c].x);
                    acc[h][c].y = fmaf(pw, vr[c].y, acc[h][c].y);
                    acc[h][c].z = fmaf(pw, vr[c].z, acc[h][c].z);
                    acc[h][c].w = fmaf(pw, vr[c].w, acc[h][c].w);
                }
            }
        }
#pragma unroll
        for (int c = 0; c < C; ++c) { kr[c] = kn[c]; vr[c] = vn[c]; }
    }

    // merge the key streams of the warp (lanes with the same li)
#pragma unroll
    for (int h = 0; h < ATTN_G; ++h) {
#pragma unroll
        for (int o = LPK; o < 32; o <<= 1) {
            const float mo = __shfl_xor_sync(0xffffffffu, m[h], o), lo = __shfl_xor_sync(0xffffffffu, l[h], o);
            const float mn = fmaxf(m[h], mo);
            const float ca = m[h] == -INFINITY ? 0.0f : expf(m[h] - mn), cb = mo == -INFINITY ? 0.0f : expf(mo - mn);
            l[h] = l[h] * ca + lo * cb;
#pragma unroll
            for (int c = 0; c < C; ++c) {
                acc[h][c].x = acc[h][c].x * ca + __shfl_xor_sync(0xffffffffu, acc[h][c].x, o) * cb;
                acc[h][c].y = acc[h][c].y * ca + __shfl_xor_sync(0xffffffffu, acc[h][c].y, o) * cb;
                acc[h][c].z = acc[h][c].z * ca + __shfl_xor_sync(0xffffffffu, acc[h][c].z, o) * cb;
                acc[h][c].w = acc[h][c].w * ca + __shfl_xor_sync(0xffffffffu, acc[h][c].w, o) * cb;
            }
            m[h] = mn;
        }
    }
    if (sub == 0) {
#pragma unroll
        for (int h = 0; h < ATTN_G; ++h) {
#pragma unroll
            for (int c = 0; c < C; ++c) *reinterpret_cast<float4 *>(&merge_s[warp][h][(c * LPK + li) * 4]) = acc[h][c];
            if (li == 0) { merge_s[warp][h][AD] = m[h]; merge_s[warp][h][AD + 1] = l[h]; }
        }
    }
    __syncthreads();

    // merge the warps; thread -> (head, dimension)
    for (int i = threadIdx.x; i < group * AD; i += blockDim.x) {
        const int h = i / AD, c = i - h * AD;
        float mm = -INFINITY;
#pragma unroll
        for (int w = 0; w < ATTN_NW; ++w) mm = fmaxf(mm, merge_s[w][h][AD]);
        float ll = 0.0f, a = 0.0f;
#pragma unroll
        for (int w = 0; w < ATTN_NW; ++w) {
            const float mw = merge_s[w][h][AD];
            const float f = mw == -INFINITY ? 0.0f : expf(mw - mm);
            ll += merge_s[w][h][AD + 1] * f;
            a += merge_s[w][h][c] * f;
        }
        const size_t head = (size_t)seq * p.H + h0 + h;
        if (p.splits == 1) {
            p.out[head * AD + c] = ll > 0.0f ? a / ll : 0.0f;
        } else {
            float *dst = p.part + (head * p.splits + split) * (AD + 2);
            dst[c] = a;
            if (c == 0) { dst[AD] = mm; dst[AD + 1] = ll; }
        }
    }
}

// out[head][c] = sum_s part[s][c] * exp(m_s - M) / sum_s l_s * exp(m_s - M); one CTA per head.
// The per-split factors are computed once into shared memory; the column sums then run over independent loads.
constexpr int ATTN_MAX_SPLITS = 256;
__global__ void __launch_bounds__(128) attn_merge_kernel(const float *__restrict__ part, float *__restrict__ out, int splits, int ad)
{
    __shared__ float f_s[ATTN_MAX_SPLITS];
    __shared__ float red_m[4], red_l[4];
    const size_t head = blockIdx.x;
    const float *src = part + head * splits * (ad + 2);
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = blockDim.x >> 5;
    pdl_trigger();
    pdl_wait();
    float mloc = -INFINITY;
    for (int s = threadIdx.x; s < splits; s += blockDim.x) {
        const float ms = __ldcg(src + s * (ad + 2) + ad);
        f_s[s] = ms;
        mloc = fmaxf(mloc, ms);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) mloc = fmaxf(mloc, __shfl_xor_sync(0xffffffffu, mloc, o));
    if (lane == 0) red_m[warp] = mloc;
    __syncthreads();
    float mm = red_m[0];
    for (int w = 1; w < nw; ++w) mm = fmaxf(mm, red_m[w]);
    float lloc = 0.0f;
    for (int s = threadIdx.x; s < splits; s += blockDim.x) {
        const float ms = f_s[s];
        const float f = ms == -INFINITY ? 0.0f : expf(ms - mm);
        f_s[s] = f;
        lloc += __ldcg(src + s * (ad + 2) + ad + 1) * f;
    }
    lloc = group_sum<32>(lloc);
    if (lane == 0) red_l[warp] = lloc;
    __syncthreads();
    float ll = 0.0f;
    for (int w = 0; w < nw; ++w) ll += red_l[w];
    const float inv = ll > 0.0f ? 1.0f / ll : 0.0f;
    for (int c = threadIdx.x; c < ad; c += blockDim.x) {
        float a0 = 0.0f, a1 = 0.0f, a2 = 0.0f, a3 = 0.0f;
        int s = 0;
        for (; s + 4 <= splits; s += 4) {
            const float v0 = __ldcg(src + (s + 0) * (ad + 2) + c), v1 = __ldcg(src + (s + 1) * (ad + 2) + c);
            const float v2 = __ldcg(src + (s + 2) * (ad + 2) + c), v3 = __ldcg(src + (s + 3) * (ad + 2) + c);
            a0 = fmaf(v0, f_s[s], a0); a1 = fmaf(v1, f_s[s + 1], a1); a2 = fmaf(v2, f_s[s + 2], a2); a3 = fmaf(v3, f_s[s + 3], a3);
        }
        for (; s < splits; ++s) a0 = fmaf(__ldcg(src + s * (ad + 2) + c), f_s[s], a0);
        out[head * ad + c] = ((a0 + a1) + (a2 + a3)) * inv;
    }
}

// Any head size / group size: one CTA per Q head, warps stride the keys, lanes stride the dimensions.
constexpr int ATTN_GEN_MAXD = 512;
__global__ void __launch_bounds__(128) attn_decode_generic_kernel(AttnParams p)
{
    const int h = blockIdx.x, seq = blockIdx.y;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = blockDim.x >> 5;
    const int ad = p.ad, kvh = (int)((long long)h * p.Hkv / p.H);
    const float *q = p.q + ((size_t)seq * p.H + h) * ad;
    const float *kbase = p.k + (size_t)seq * p.kv_batch_stride + (size_t)kvh * p.cap * ad;
    const float *vbase = p.v + (size_t)seq * p.kv_batch_stride + (size_t)kvh * p.cap * ad;
    constexpr int PER = ATTN_GEN_MAXD / 32;
    float qr[PER], acc[PER];
#pragma unroll
    for (int j = 0; j < PER; ++j) {
        const int c = lane + 32 * j;
        qr[j] = c < ad ? q[c] * p.scale : 0.0f;
        acc[j] = 0.0f;
    }
    float m = -INFINITY, l = 0.0f;
    const int kv_tokens = attn_kv_tokens(p);
    for (int t = warp; t < kv_tokens; t += nw) {
        float s = 0.0f;
#pragma unroll
        for (int j = 0; j < PER; ++j) {
            const int c = lane + 32 * j;
            if (c < ad) s = fmaf(qr[j], kbase[(size_t)t * ad + c], s);
        }
        s = group_sum<32>(s);
        const float mn = fmaxf(m, s);
        const float corr = m == -INFINITY ? 0.0f : expf(m - mn), pw = expf(s - mn);
        l = l * corr + pw;
#pragma unroll
        for (int j = 0; j < PER; ++j) {
            const int c = lane + 32 * j;
            if (c < ad) acc[j] = acc[j] * corr + pw * vbase[(size_t)t * ad + c];
        }
        m = mn;
    }
    __shared__ float ms[4], ls[4];
    __shared__ float acc_s[4][ATTN_GEN_MAXD];
    if (lane == 0) { ms[warp] = m; ls[warp] = l; }
#pragma unroll
    for (int j = 0; j < PER; ++j) {
        const int c = lane + 32 * j;
        if (c < ad) acc_s[warp][c] = acc[j];
    }
    __syncthreads();
    float mm = -INFINITY;
    for (int w = 0; w < nw; ++w) mm = fmaxf(mm, ms[w]);
    for (int c = threadIdx.x; c < ad; c += blockDim.x) {
        float ll = 0.0f, a = 0.0f;
        for (int w = 0; w < nw; ++w) {
            const float f = ms[w] == -INFINITY ? 0.0f : expf(ms[w] - mm);
            ll += ls[w] * f;
            a += acc_s[w][c] * f;
        }
        p.out[((size_t)seq * p.H + h) * ad + c] = ll > 0.0f ? a / ll : 0.0f;
    }
}

}  // namespace ckb

using namespace ckb;

// Set by the step executor around its attention call: within a decode step only the newest cache row is written and the device
// position is stable, so the tile kernel may read both before its dependency wait (see attention_tile.cu).
static int g_attn_early_rows = 0;
extern "C" void ckb_attn_hint_early_rows(int on) { g_attn_early_rows = on; }

extern "C" int ckb_launch_attn_tile(const AttnParams *p, int batch, void *stream);
extern "C" int ckb_launch_attn_f16mma(const AttnParams *p, int batch, void *stream);
extern "C" int ckb_launch_attn_cluster(const AttnParams *p, int batch, int ranks, void *stream);     // attention_tile.cu

extern "C" size_t ckb200_attention_decode_scratch_bytes(int batch, int num_heads, int aligned_head_dim, int splits)
{
    if (splits <= 1) return 0;
    return (size_t)batch * num_heads * splits * (aligned_head_dim + 2) * sizeof(float);
}

// Number of context splits the launcher would use (1 = no scratch needed), given the size of a cache element
// (4 = fp32, 2 = fp16).  From two sequences up the tensor-core kernel serves the call and holds one CTA per SM
// over an fp32 cache, two over an fp16 cache; a CTA beyond those slots starts a second wave that costs as much
// as the first (4 sequences of the 70B shape at 4096 keys over fp32: 41.8 us at 5 splits = 160 CTAs, 28.2 us
// at 4 = 128), so the count there is rounded DOWN to what one wave holds.
extern "C" int ckb200_attention_decode_splits_kv(int batch, int num_kv_heads, int kv_tokens, int kv_element_bytes)
{
    const int forced = ckb_tune_get("attn_splits", 0);
    if (forced > 0) return forced;
    const int sms = ckb_sm_count();
    const long long base = (long long)batch * num_kv_heads;
    const bool f16 = kv_element_bytes == 2;
    const bool mma = batch >= ckb_tune_get("attn_f16_mma_min_batch", 2) && ckb_tune_get(f16 ? "attn_f16_mma" : "attn_f32_mma", 1);
    int splits;
    if (mma) {
        splits = (int)(((f16 ? 2LL : 1LL) * sms) / base);
    } else {
        const long long ctas_wanted = ckb_tune_get("attn_tile", 1) ? sms : 2LL * sms;   // the tile kernel fills an SM with one CTA
        splits = (int)((ctas_wanted + base - 1) / base);
    }
    const int tiles = (kv_tokens + 63) / 64;                 // at least one 64-key tile per split
    if (splits > tiles) splits = tiles;
    if (splits > 256) splits = 256;
    if (splits < 1) splits = 1;
    const int tiles_per_split = (tiles + splits - 1) / splits;
    splits = (tiles + tiles_per_split - 1) / tiles_per_split;   // no split without work
    return splits;
}

extern "C" int ckb200_attention_decode_splits(int batch, int num_kv_heads, int kv_tokens)
{
    return ckb200_attention_decode_splits_kv(batch, num_kv_heads, kv_tokens, 4);
}

// Core launcher: scratch may be NULL when splits == 1.  With pos_dev the context length is read on the
// device as *pos_dev + 1 (kv_tokens then only has to be positive), so a captured graph can be replayed.
extern "C" int ckb200_dev_attention_decode_ws(const float *q, const float *k_cache, const float *v_cache, float *out,
                                              int batch, long long kv_batch_stride, int num_heads, int num_kv_heads,
                                              int kv_tokens, int cache_capacity, int head_dim, int aligned_head_dim,
                                              int splits, float *scratch, const int *pos_dev, void *stream)
{
    if (!q || !k_cache || !v_cache || !out) return 0;
    if (batch <= 0 || num_heads <= 0 || num_kv_heads <= 0 || kv_tokens <= 0 || cache_capacity <= 0) return 0;
    if (kv_tokens > cache_capacity || head_dim <= 0 || aligned_head_dim <= 0) return 0;
    if (ckb_ensure_init()) return CKB_ERR_NO_DEVICE;
    AttnParams p;
    p.q = q; p.k = k_cache; p.v = v_cache; p.out = out; p.part = scratch; p.pos_ptr = pos_dev;
    p.kv_batch_stride = kv_batch_stride;
    p.H = num_heads; p.Hkv = num_kv_heads; p.kv_tokens = kv_tokens; p.cap = cache_capacity; p.ad = aligned_head_dim;
    p.scale = 1.0f / sqrtf((float)head_dim);
    p.counters = NULL; p.q8_out = NULL; p.out_stride = num_heads * aligned_head_dim; p.q8_cols = 0; p.kv_f16 = 0; p.early_rows = pos_dev != NULL && g_attn_early_rows;
    cudaStream_t st = ckb_stream(stream);
    const int group = num_heads / num_kv_heads;
    const bool fast = (aligned_head_dim == 64 || aligned_head_dim == 128) && num_heads % num_kv_heads == 0 &&
                      group <= ATTN_G && (((uintptr_t)q | (uintptr_t)k_cache | (uintptr_t)v_cache) & 15) == 0 &&
                      (kv_batch_stride % 4) == 0 && ckb_tune_get("attn_generic", 0) == 0;
    if (!fast) {
        if (aligned_head_dim > ATTN_GEN_MAXD) return ckb_fail(CKB_ERR_LIMIT, "attention decode: aligned_head_dim %d > %d", aligned_head_dim, ATTN_GEN_MAXD);
        p.splits = 1;
        attn_decode_generic_kernel<<<dim3(num_heads, batch), 128, 0, st>>>(p);
        return ckb_check_launch("attn_decode_generic");
    }
    if (splits < 1) splits = 1;
    if (splits > ATTN_MAX_SPLITS) splits = ATTN_MAX_SPLITS;
    if (splits > 1 && !scratch) return ckb_fail(CKB_ERR_STATE, "attention decode: %d splits need a scratch buffer", splits);
    p.splits = splits;
    const dim3 grid(splits, num_kv_heads, batch);
    int rc = ckb_launch_attn_f16mma(&p, batch, st);           // batches of sequences: the tensor-core form (attention_f16mma.cu); -1: not for this call
    if (rc >= 0) {
    } else if (ckb_tune_get("attn_tile", 1))
        rc = ckb_launch_attn_tile(&p, batch, st);
    else
        rc = aligned_head_dim == 64 ? launch_pdl("attn_decode", attn_decode_kernel<64>, grid, dim3(ATTN_NW * 32), 0, st, p)
                                    : launch_pdl("attn_decode", attn_decode_kernel<128>, grid, dim3(ATTN_NW * 32), 0, st, p);
    if (rc) return rc;
    if (splits > 1)
        return launch_pdl("attn_merge", attn_merge_kernel, dim3(batch * num_heads), dim3(128), 0, st, (const float *)scratch, out, splits,
                          aligned_head_dim);
    return 0;
}

extern "C" int ckb200_dev_quantize_q8_k(const float *, void *, int, int, void *);

extern "C" size_t ckb200_attention_decode_counter_bytes(int batch, int num_kv_heads) { return (size_t)batch * (num_kv_heads + 1) * sizeof(int); }

// One launch for attention + split merge + Q8_K quantisation of the finished rows (what the o-projection GEMV
// consumes).  out rows are out_stride floats apart and the q8_cols - H*ad floats after each row must be zero;
// `counters` is ckb200_attention_decode_counter_bytes() of device memory that was zero before the first call
// (every call leaves it zero).  Shapes outside the tile kernel's fast path run as separate launches.
extern "C" int ckb200_dev_attention_decode_fused(const float *q, const float *k_cache, const float *v_cache, float *out, int out_stride,
                                                 int batch, long long kv_batch_stride, int num_heads, int num_kv_heads, int kv_tokens,
                                                 int cache_capacity, int head_dim, int aligned_head_dim, int splits, float *scratch,
                                                 int *counters, const int *pos_dev, void *q8_out, int q8_cols, void *stream)
{
    if (!q || !k_cache || !v_cache || !out || !counters) return 0;
    if (batch <= 0 || num_heads <= 0 || num_kv_heads <= 0 || kv_tokens <= 0 || cache_capacity <= 0) return 0;
    if (kv_tokens > cache_capacity || head_dim <= 0 || aligned_head_dim <= 0) return 0;
    if (ckb_ensure_init()) return CKB_ERR_NO_DEVICE;
    const int group = num_heads / num_kv_heads;
    const bool fast = (aligned_head_dim == 64 || aligned_head_dim == 128) && num_heads % num_kv_heads == 0 && group <= ATTN_G &&
                      (((uintptr_t)q | (uintptr_t)k_cache | (uintptr_t)v_cache | (uintptr_t)out) & 15) == 0 && (kv_batch_stride % 4) == 0 &&
                      out_stride % 4 == 0 && ckb_tune_get("attn_generic", 0) == 0 && ckb_tune_get("attn_tile", 1) && ckb_tune_get("attn_fused", 1) &&
                      (!q8_out || (q8_cols % 256 == 0 && q8_cols <= out_stride && q8_cols >= num_heads * aligned_head_dim));
    if (!fast) {
        if (out_stride != num_heads * aligned_head_dim && batch > 1)
            return ckb_fail(CKB_ERR_SHAPE, "attention decode (fused): this shape needs densely packed output rows");
        int rc = ckb200_dev_attention_decode_ws(q, k_cache, v_cache, out, batch, kv_batch_stride, num_heads, num_kv_heads, kv_tokens, cache_capacity,
                                                head_dim, aligned_head_dim, splits, scratch, pos_dev, stream);
        if (!rc && q8_out) {
            for (int b = 0; b < batch && !rc; ++b)
                rc = ckb200_dev_quantize_q8_k(out + (size_t)b * out_stride, (uint8_t *)q8_out + (size_t)b * (q8_cols / 256) * Q8K_BYTES, 1, q8_cols, stream);
        }
        return rc;
    }
    if (splits < 1) splits = 1;
    if (splits > ATTN_MAX_SPLITS) splits = ATTN_MAX_SPLITS;
    if (splits > 1 && !scratch) return ckb_fail(CKB_ERR_STATE, "attention decode: %d splits need a scratch buffer", splits);
    AttnParams p;
    p.q = q; p.k = k_cache; p.v = v_cache; p.out = out; p.part = scratch; p.pos_ptr = pos_dev;
    p.kv_batch_stride = kv_batch_stride;
    p.H = num_heads; p.Hkv = num_kv_heads; p.kv_tokens = kv_tokens; p.cap = cache_capacity; p.ad = aligned_head_dim;
    p.scale = 1.0f / sqrtf((float)head_dim);
    p.splits = splits;
    p.counters = counters; p.q8_out = (uint8_t *)q8_out; p.out_stride = out_stride; p.q8_cols = q8_cols; p.kv_f16 = 0; p.early_rows = pos_dev != NULL && g_attn_early_rows;
    if (!q8_out && ckb_tune_get("attn_cluster", 1)) {
        // the CTAs of a kv head as one thread-block cluster: the split merge happens in distributed shared memory
        static int unavailable = 0;
        if (!unavailable) {
            const int rc = ckb_launch_attn_cluster(&p, batch, ckb_tune_get("attn_cluster_ranks", 8), ckb_stream(stream));
            if (rc >= 0) return rc;
            unavailable = 1;
        }
    }
    return ckb_launch_attn_tile(&p, batch, ckb_stream(stream));
}

// attention_forward_decode_head_major_gqa_flash_sliding (src/kernels/attention_kernels_sliding.c:528-600): the query attends
// the last min(kv_tokens, sliding_window) cache rows, which in the head-major cache is the same attention on row pointers
// moved forward by kv_tokens - that many rows (the head stride stays cache_capacity rows).
extern "C" int ckb200_dev_attention_decode(const float *, const float *, const float *, float *, int, long long, int, int, int, int, int, int, void *);
extern "C" int ckb200_dev_attention_decode_sliding(const float *q, const float *k_cache, const float *v_cache, float *out, int batch,
                                                   long long kv_batch_stride, int num_heads, int num_kv_heads, int kv_tokens, int cache_capacity,
                                                   int head_dim, int aligned_head_dim, int sliding_window, void *stream)
{
    if (!q || !k_cache || !v_cache || !out) return 0;
    if (kv_tokens <= 0 || kv_tokens > cache_capacity || aligned_head_dim <= 0) return 0;
    const int eff = sliding_window > 0 && sliding_window < kv_tokens ? sliding_window : kv_tokens;
    const size_t skip = (size_t)(kv_tokens - eff) * aligned_head_dim;
    return ckb200_dev_attention_decode(q, k_cache + skip, v_cache + skip, out, batch, kv_batch_stride, num_heads, num_kv_heads, eff, cache_capacity,
                                       head_dim, aligned_head_dim, stream);
}

// Decode attention over IEEE fp16 caches (attention_forward_decode_head_major_gqa_flash_f16cache,
// src/kernels/attention_kernels.c:3450-3557): the same layout with 2-byte elements, widened to fp32 in the tile kernel;
// the arithmetic after that is the fp32 path's.  Tile kernel shapes only (aligned head size 64 or 128, groups <= 8).
extern "C" int ckb200_dev_attention_decode_f16cache_ws(const float *q, const uint16_t *k_cache, const uint16_t *v_cache, float *out, int batch,
                                                       long long kv_batch_stride, int num_heads, int num_kv_heads, int kv_tokens, int cache_capacity,
                                                       int head_dim, int aligned_head_dim, int splits, float *scratch, const int *pos_dev, void *stream)
{
    if (!q || !k_cache || !v_cache || !out) return 0;
    if (batch <= 0 || num_heads <= 0 || num_kv_heads <= 0 || kv_tokens <= 0 || cache_capacity <= 0) return 0;
    if (kv_tokens > cache_capacity || head_dim <= 0 || aligned_head_dim <= 0) return 0;
    if (ckb_ensure_init()) return CKB_ERR_NO_DEVICE;
    const int group = num_heads / num_kv_heads;
    if ((aligned_head_dim != 64 && aligned_head_dim != 128) || num_heads % num_kv_heads || group > ATTN_G)
        return ckb_fail(CKB_ERR_SHAPE, "attention decode (fp16 cache): %d heads / %d kv heads / head size %d is outside the tile kernel", num_heads,
                        num_kv_heads, aligned_head_dim);
    if ((((uintptr_t)q | (uintptr_t)k_cache | (uintptr_t)v_cache) & 15) || (kv_batch_stride % 8))
        return ckb_fail(CKB_ERR_ALIGN, "attention decode (fp16 cache): pointers and the sequence stride must be 16-byte aligned");
    if (splits < 1) splits = 1;
    if (splits > ATTN_MAX_SPLITS) splits = ATTN_MAX_SPLITS;
    if (splits > 1 && !scratch) return ckb_fail(CKB_ERR_STATE, "attention decode: %d splits need a scratch buffer", splits);
    AttnParams p;
    p.q = q; p.k = reinterpret_cast<const float *>(k_cache); p.v = reinterpret_cast<const float *>(v_cache); p.out = out; p.part = scratch;
    p.pos_ptr = pos_dev;
    p.kv_batch_stride = kv_batch_stride;
    p.H = num_heads; p.Hkv = num_kv_heads; p.kv_tokens = kv_tokens; p.cap = cache_capacity; p.ad = aligned_head_dim;
    p.scale = 1.0f / sqrtf((float)head_dim);
    p.splits = splits;
    p.counters = NULL; p.q8_out = NULL; p.out_stride = num_heads * aligned_head_dim; p.q8_cols = 0; p.kv_f16 = 1; p.early_rows = 0;
    cudaStream_t st = ckb_stream(stream);
    int rc = ckb_launch_attn_f16mma(&p, batch, st);           // tensor-core form (attention_f16mma.cu); -1: not for this call
    if (rc < 0) rc = ckb_launch_attn_tile(&p, batch, st);
    if (rc) return rc;
    if (splits > 1)
        return launch_pdl("attn_merge", attn_merge_kernel, dim3(batch * num_heads), dim3(128), 0, st, (const float *)scratch, out, splits, aligned_head_dim);
    return 0;
}

extern "C" int ckb200_dev_attention_decode_f16cache(const float *q, const uint16_t *k_cache, const uint16_t *v_cache, float *out, int batch,
                                                    long long kv_batch_stride, int num_heads, int num_kv_heads, int kv_tokens, int cache_capacity,
                                                    int head_dim, int aligned_head_dim, void *stream)
{
    if (ckb_ensure_init()) return CKB_ERR_NO_DEVICE;
    const int splits = ckb200_attention_decode_splits_kv(batch, num_kv_heads, kv_tokens, 2);
    float *scratch = NULL;
    if (splits > 1) {
        scratch = (float *)ckb_scratch(CKB_SLOT_T, ckb200_attention_decode_scratch_bytes(batch, num_heads, aligned_head_dim, splits));
        if (!scratch) return CKB_ERR_CUDA;
    }
    return ckb200_dev_attention_decode_f16cache_ws(q, k_cache, v_cache, out, batch, kv_batch_stride, num_heads, num_kv_heads, kv_tokens, cache_capacity,
                                                   head_dim, aligned_head_dim, splits, scratch, NULL, stream);
}

// Convenience form: picks the split count and takes the scratch from the library's own pool.
extern "C" int ckb200_dev_attention_decode(const float *q, const float *k_cache, const float *v_cache, float *out,
                                           int batch, long long kv_batch_stride, int num_heads, int num_kv_heads,
                                           int kv_tokens, int cache_capacity, int head_dim, int aligned_head_dim, void *stream)
{
    if (ckb_ensure_init()) return CKB_ERR_NO_DEVICE;
    const int splits = ckb200_attention_decode_splits(batch, num_kv_heads, kv_tokens);
    float *scratch = NULL;
    if (splits > 1) {
        scratch = (float *)ckb_scratch(CKB_SLOT_T, ckb200_attention_decode_scratch_bytes(batch, num_heads, aligned_head_dim, splits));
        if (!scratch) return CKB_ERR_CUDA;
    }
    return ckb200_dev_attention_decode_ws(q, k_cache, v_cache, out, batch, kv_batch_stride, num_heads, num_kv_heads, kv_tokens,
                                          cache_capacity, head_dim, aligned_head_dim, splits, scratch, NULL, stream);
}

// ------------------------------------------------------------------------------------------------
// Decode attention for callers that must not allocate.
//
// Some hosts of this library cannot call cudaMalloc on the decode path: a model runtime that
// planned every byte of device memory at load time (the reference's own rule is "no malloc in
// kernels, memory comes from the planned arena"), a real-time loop that may not take the
// allocator's locks, or a process that has handed all free memory to another pool.  The split-K
// kernel above needs a scratch buffer for its per-split partial results; here that buffer is a
// fixed array inside the library image, so the call needs nothing but its inputs and outputs.
//
// Limits and rules:
//   * the scratch is CKB_ATTN_STATIC_SCRATCH_BYTES (4 MiB) per GPU that loads the library, held
//     until the process exits; a call whose partials need more is rejected with CKB_ERR_LIMIT
//     (fewer splits, or splits = 1, always fit);
//   * the array's device address is looked up once per device, on the first call made with that
//     device current; make that first call before any stream capture;
//   * every call shares the one array and it keeps the previous call's contents; nothing has to be
//     cleared (each split slot is fully written before the merge reads it), but two calls that
//     overlap on the GPU (different streams without ordering) race on it;
//   * stream = NULL means the legacy default stream here (the library's own stream is not created).
// This entry point calls no cudaMalloc / cudaFree and no allocating library routine.
#define CKB_ATTN_STATIC_SCRATCH_BYTES (4u << 20)
#define CKB_MAX_DEVICES 64

static __device__ __align__(256) float g_attn_static_scratch[CKB_ATTN_STATIC_SCRATCH_BYTES / sizeof(float)];
static float *g_attn_static_ptr[CKB_MAX_DEVICES];     // per device: address of the array on that device
static int g_attn_static_sms[CKB_MAX_DEVICES];

extern "C" size_t ckb200_attention_decode_static_scratch_limit(void) { return CKB_ATTN_STATIC_SCRATCH_BYTES; }

extern "C" int ckb200_dev_attention_decode_static(const float *q, const float *k_cache, const float *v_cache, float *out,
                                                  int batch, long long kv_batch_stride, int num_heads, int num_kv_heads,
                                                  int kv_tokens, int cache_capacity, int head_dim, int aligned_head_dim,
                                                  int splits, void *stream)
{
    if (!q || !k_cache || !v_cache || !out) return 0;
    if (batch <= 0 || num_heads <= 0 || num_kv_heads <= 0 || kv_tokens <= 0 || cache_capacity <= 0) return 0;
    if (kv_tokens > cache_capacity || head_dim <= 0 || aligned_head_dim <= 0) return 0;

    int dev = -1;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= CKB_MAX_DEVICES) {
        cudaGetLastError();
        return ckb_fail(CKB_ERR_NO_DEVICE, "attention decode (static scratch): no current CUDA device");
    }
    float *scratch = __atomic_load_n(&g_attn_static_ptr[dev], __ATOMIC_ACQUIRE);
    if (!scratch) {
        // set-up, once per device, with that device current: the array's name is only a host-side
        // stand-in in host code; the kernel needs the device address.  Two host threads may both get here:
        // they compute the same two values, and the address is published last (release), so a thread
        // that sees it also sees the SM count.  The cached address belongs to this process's CUDA
        // context: after cudaDeviceReset the library must be reloaded.
        float *p = NULL;
        const cudaError_t e = cudaGetSymbolAddress((void **)&p, g_attn_static_scratch);
        if (e != cudaSuccess || !p) {
            ckb_check_cuda((int)e, "cudaGetSymbolAddress(static attention scratch)");
            return CKB_ERR_CUDA;
        }
        int sms = 0;
        if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sms <= 0) { cudaGetLastError(); sms = 148; }
        __atomic_store_n(&g_attn_static_sms[dev], sms, __ATOMIC_RELAXED);
        __atomic_store_n(&g_attn_static_ptr[dev], p, __ATOMIC_RELEASE);
        scratch = p;
    }

    const int group = num_heads / num_kv_heads;
    const bool fast = (aligned_head_dim == 64 || aligned_head_dim == 128) && num_heads % num_kv_heads == 0 && group <= ATTN_G &&
                      (((uintptr_t)q | (uintptr_t)k_cache | (uintptr_t)v_cache) & 15) == 0 && (kv_batch_stride % 4) == 0;
    if (splits <= 0) {                                  // two CTAs per SM, at least 64 keys per split; the attn_splits tune key is not consulted here
        const long long base = (long long)batch * num_kv_heads;
        splits = (int)((2LL * g_attn_static_sms[dev] + base - 1) / base);
        const int max_by_tokens = (kv_tokens + 63) / 64;
        if (splits > max_by_tokens) splits = max_by_tokens;
        if (splits > 256) splits = 256;
        if (splits < 1) splits = 1;
    }
    AttnParams p;
    p.q = q; p.k = k_cache; p.v = v_cache; p.out = out; p.part = scratch; p.pos_ptr = NULL;
    p.kv_batch_stride = kv_batch_stride;
    p.H = num_heads; p.Hkv = num_kv_heads; p.kv_tokens = kv_tokens; p.cap = cache_capacity; p.ad = aligned_head_dim;
    p.scale = 1.0f / sqrtf((float)head_dim);
    p.counters = NULL; p.q8_out = NULL; p.out_stride = num_heads * aligned_head_dim; p.q8_cols = 0; p.kv_f16 = 0; p.early_rows = 0;
    cudaStream_t st = (cudaStream_t)stream;
    if (!fast) {
        if (aligned_head_dim > ATTN_GEN_MAXD) return ckb_fail(CKB_ERR_LIMIT, "attention decode: aligned_head_dim %d > %d", aligned_head_dim, ATTN_GEN_MAXD);
        p.splits = 1;
        attn_decode_generic_kernel<<<dim3(num_heads, batch), 128, 0, st>>>(p);
        return ckb_check_launch("attn_decode_generic");
    }
    if (splits > ATTN_MAX_SPLITS) splits = ATTN_MAX_SPLITS;
    const size_t need = splits > 1 ? (size_t)batch * num_heads * splits * (aligned_head_dim + 2) * sizeof(float) : 0;
    if (need > CKB_ATTN_STATIC_SCRATCH_BYTES)
        return ckb_fail(CKB_ERR_LIMIT, "attention decode (static scratch): %zu bytes of partials for batch %d x %d heads x %d splits "
                        "exceed the built-in %u-byte scratch; use fewer splits or the allocating entry point",
                        need, batch, num_heads, splits, (unsigned)CKB_ATTN_STATIC_SCRATCH_BYTES);
    p.splits = splits;
    const dim3 grid(splits, num_kv_heads, batch);
    if (aligned_head_dim == 64) attn_decode_kernel<64><<<grid, ATTN_NW * 32, 0, st>>>(p);
    else attn_decode_kernel<128><<<grid, ATTN_NW * 32, 0, st>>>(p);
    if (ckb_check_launch("attn_decode")) return CKB_ERR_CUDA;
    if (splits > 1) {
        attn_merge_kernel<<<batch * num_heads, aligned_head_dim < 128 ? 64 : 128, 0, st>>>(scratch, out, splits, aligned_head_dim);
        return ckb_check_launch("attn_merge");
    }
    return 0;
}
