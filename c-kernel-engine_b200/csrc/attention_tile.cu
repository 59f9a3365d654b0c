// Decode attention, bandwidth form: K/V tiles of 64 keys are brought into shared memory with 1-D bulk copies
// (three stages per CTA, so two tiles are always in flight) and every warp works on 8 keys of the tile.
//
// Same mathematics as attention_forward_decode_head_major_gqa_flash (src/kernels/attention_kernels.c:3365-3406;
// per head attention_flash_decode, src/kernels/attention_flash_true.c:142-230): scores (q.k)/sqrt(head_dim),
// softmax, out = P.V, kv_head = h * Hkv / H.  In the head-major cache the rows t .. t+63 of one kv head are one
// contiguous range of 64 * ad * 4 bytes, so a tile is two bulk copies (K and V), each completing on the
// stage's mbarrier.
//
// A warp takes 2 keys per step with 16 lanes per key (each lane owns ad/16 dimensions, read as float4 so that
// 16 lanes read 256 contiguous bytes of shared memory); the query of all <= 8 Q heads of the group lives in
// registers.  The 8 partial dots of a step are reduced with a transposing butterfly, which leaves lane li with
// the score of head li & 7.  The softmax is updated once per 8 keys (tile maximum, one rescale of the
// accumulators) instead of once per key.  Splits write (max, sum, unnormalised out) partials that
// attn_merge_kernel combines with the exact log-sum-exp rule.
//
// All mbarrier waits are bounded; on a timeout the CTA records the device error word and leaves.
#include "attention_params.cuh"
#include "launch.h"
#include "pdl.cuh"
#include "q8k_block.cuh"
#include "runtime.h"

#include <math.h>

namespace ckb {

#ifdef CKB_STEP_TRACE
// Tuning aid (build with -DCKB_STEP_TRACE): global-timer stamps of the first CTA and of the CTA that merges the first kv head.
static __device__ unsigned long long at_trace[8 * 4096];
static __device__ unsigned at_trace_n;
__device__ __forceinline__ unsigned long long at_now() { unsigned long long t; asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t)); return t; }
#define AT_TRACE(slot, k) do { if ((slot) < 4096u) at_trace[8 * (slot) + (k)] = at_now(); } while (0)
#else
#define AT_TRACE(slot, k) do { } while (0)
#endif

constexpr int AT_NW = 8;            // warps per CTA
constexpr int AT_KT = 64;           // keys per tile
constexpr int AT_STAGES = 3;
constexpr int AT_LPK = 16;          // lanes per key

// EB: bytes per cache element, 4 (fp32 cache) or 2 (IEEE fp16 cache, attention_forward_decode_head_major_gqa_flash_f16cache,
// src/kernels/attention_kernels.c:3450-3557: the halves are widened to fp32 and the arithmetic is the same).  The merge
// scratch of the epilogue needs the fp32-sized stages either way.
template <int AD> constexpr int at_stage_bytes() { return 2 * AT_KT * AD * 4; }
template <int AD> constexpr int at_smem_bytes() { return AT_STAGES * at_stage_bytes<AD>() + 2 * AT_STAGES * 8 + 16; }

// this lane's four dimensions of piece `idx` of a cache row in shared memory
template <int EB>
__device__ __forceinline__ float4 at_row_piece(uint32_t row_addr, int idx)
{
    if constexpr (EB == 4) {
        return lds_f4(row_addr + (uint32_t)idx * 16u);
    } else {
        uint32_t lo, hi;
        asm volatile("ld.shared.v2.u32 {%0,%1}, [%2];" : "=r"(lo), "=r"(hi) : "r"(row_addr + (uint32_t)idx * 8u));
        const float2 a = __half22float2(*reinterpret_cast<const __half2 *>(&lo)), b = __half22float2(*reinterpret_cast<const __half2 *>(&hi));
        return make_float4(a.x, a.y, b.x, b.y);
    }
}

// CLUSTER: the CTAs that share a kv head form one thread-block cluster.  Tiles are dealt round-robin to the ranks, and the
// partial results (running max, sum, unnormalised output per head) never leave the chip: each CTA leaves them in its shared
// memory, the cluster synchronises, and every rank combines one slice of the output by reading its peers' shared memory
// (distributed shared memory).  No scratch buffer, no arrival counter, no second pass through L2.
__device__ __forceinline__ uint32_t at_cluster_rank() { uint32_t r; asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r)); return r; }
__device__ __forceinline__ uint32_t at_cluster_size() { uint32_t r; asm volatile("mov.u32 %0, %%cluster_nctarank;" : "=r"(r)); return r; }
__device__ __forceinline__ void at_cluster_sync()
{
    asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
    asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// a float at byte offset `off` of the shared window of cluster rank `rank`
__device__ __forceinline__ float at_ld_peer(uint32_t local_addr, uint32_t rank)
{
    uint32_t remote;
    float v;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(local_addr), "r"(rank));
    asm volatile("ld.shared::cluster.f32 %0, [%1];" : "=f"(v) : "r"(remote) : "memory");
    return v;
}

template <int AD, int EB, bool CLUSTER>
__global__ void __launch_bounds__(AT_NW * 32, 1) attn_tile_kernel(AttnParams p, int *__restrict__ dev_err)
{
    constexpr int C = AD / (4 * AT_LPK);           // float4 pieces per lane (1 for 64, 2 for 128)
    constexpr int G = ATTN_MAX_GROUP;
    constexpr int KPW = AT_KT / AT_NW;             // keys per warp per tile
    constexpr int STEPS = KPW / 2;
    constexpr int ROW = AD * EB;                   // bytes per cache row
    extern __shared__ __align__(128) uint8_t smem[];
    const uint32_t s_base = smem_u32(smem);
    const uint32_t s_bar = s_base + AT_STAGES * at_stage_bytes<AD>();
#define AT_FULL(i) (s_bar + 8u * (uint32_t)(i))
#define AT_EMPTY(i) (s_bar + 8u * (uint32_t)(AT_STAGES + (i)))

    const int split = blockIdx.x, kvh = blockIdx.y, seq = blockIdx.z;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int sub = lane / AT_LPK, li = lane % AT_LPK;
    const int group = p.H / p.Hkv, h0 = kvh * group;

    unsigned tr = 0xffffffffu;
#ifdef CKB_STEP_TRACE
    if (blockIdx.x == 0 && blockIdx.y == 0 && blockIdx.z == 0 && threadIdx.x == 0) tr = atomicAdd(&at_trace_n, 1u);
    AT_TRACE(tr, 0);
#endif
    if (threadIdx.x == 0) {
        for (int i = 0; i < AT_STAGES; ++i) { mbar_init(AT_FULL(i), 1); mbar_init(AT_EMPTY(i), AT_NW); }
        mbar_fence_init();
    }
    pdl_trigger();
    __syncthreads();
    // early_rows (set by the step executor): within a decode step only the newest cache row is written, and the position changes
    // only at the end of a step, after which the next step starts with a fully ordered launch.  The position is then read and the
    // tiles that end before the newest row are requested BEFORE the dependency wait: their HBM latency overlaps the predecessor.
    if (!p.early_rows) {
        pdl_wait();       // q, the newest cache row and the position come from kernels that may still have been running
        AT_TRACE(tr, 1);
    }
    const int kv_tokens = attn_kv_tokens(p);
    const int ntiles_all = (kv_tokens + AT_KT - 1) / AT_KT;
    // plain: split s owns a contiguous run of tiles; cluster: rank r owns tiles r, r + size, r + 2 size, ...
    const int tiles_per_split = CLUSTER ? 0 : (ntiles_all + p.splits - 1) / p.splits;
    const int tile_stride = CLUSTER ? (int)gridDim.x : 1;
    const int tile0 = CLUSTER ? split : split * tiles_per_split;
    const int ntiles = CLUSTER ? (ntiles_all > split ? (ntiles_all - split + tile_stride - 1) / tile_stride : 0)
                               : max(0, min(ntiles_all, tile0 + tiles_per_split) - tile0);
    const uint8_t *kbase = reinterpret_cast<const uint8_t *>(p.k) + ((size_t)seq * p.kv_batch_stride + (size_t)kvh * p.cap * AD) * EB;
    const uint8_t *vbase = reinterpret_cast<const uint8_t *>(p.v) + ((size_t)seq * p.kv_batch_stride + (size_t)kvh * p.cap * AD) * EB;

    auto issue_tile = [&](int i) {                 // one thread: both copies of tile i of this split
        const int st = i % AT_STAGES, t_begin = (tile0 + i * tile_stride) * AT_KT;
        const uint32_t bytes = (uint32_t)min(AT_KT, kv_tokens - t_begin) * ROW;
        const uint32_t dst = s_base + st * at_stage_bytes<AD>();
        mbar_arrive_expect_tx(AT_FULL(st), 2 * bytes);
        bulk_g2s(dst, kbase + (size_t)t_begin * ROW, bytes, AT_FULL(st));
        bulk_g2s(dst + AT_KT * ROW, vbase + (size_t)t_begin * ROW, bytes, AT_FULL(st));
    };
    {
        const int first = min(ntiles, AT_STAGES - 1);
        int early = 0;                             // leading tiles that do not reach the newest row
        if (p.early_rows) {
            while (early < first && (tile0 + early * tile_stride) * AT_KT + AT_KT <= kv_tokens - 1) ++early;
            if (threadIdx.x == 0)
                for (int i = 0; i < early; ++i) issue_tile(i);
            pdl_wait();
            AT_TRACE(tr, 1);
        }
        if (threadIdx.x == 0)
            for (int i = early; i < first; ++i) issue_tile(i);
    }

    // query of the group's heads, pre-scaled, this lane's dimensions
    float4 q[G][C];
#pragma unroll
    for (int h = 0; h < G; ++h)
#pragma unroll
        for (int c = 0; c < C; ++c) {
            float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
            if (h < group) v = __ldcg(reinterpret_cast<const float4 *>(p.q + ((size_t)seq * p.H + h0 + h) * AD) + c * AT_LPK + li);
            q[h][c] = make_float4(v.x * p.scale, v.y * p.scale, v.z * p.scale, v.w * p.scale);
        }

    float m_run = -INFINITY, l_run = 0.0f;         // of head li & 7 (the same value on the lanes that share it)
    float4 acc[G][C];
#pragma unroll
    for (int h = 0; h < G; ++h)
#pragma unroll
        for (int c = 0; c < C; ++c) acc[h][c] = make_float4(0.f, 0.f, 0.f, 0.f);

    bool ok = true;
    for (int i = 0; i < ntiles; ++i) {
        const int st = i % AT_STAGES;
        if (threadIdx.x == 0 && i + AT_STAGES - 1 < ntiles) {
            // the stage of tile i + STAGES - 1 was last used by tile i - 1: wait until all warps have released it
            const int j = i + AT_STAGES - 1;
            if (i >= 1 && !mbar_wait_spin(AT_EMPTY(j % AT_STAGES), (uint32_t)(((j / AT_STAGES) - 1) & 1))) ok = false;
            if (ok) issue_tile(j);
        }
        ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0 && ok;      // warp 0 follows its lane 0
        if (!ok || !mbar_wait_spin(AT_FULL(st), (uint32_t)((i / AT_STAGES) & 1))) { ok = false; break; }

        const int t_tile = (tile0 + i * tile_stride) * AT_KT;
        const int nvalid = min(AT_KT, kv_tokens - t_tile);
        const uint32_t ks = s_base + st * at_stage_bytes<AD>() + (uint32_t)(warp * KPW) * ROW, vs = ks + AT_KT * ROW;

        // ---- scores of this warp's 8 keys: sc[step] = score(head li & 7, key 2 * step + sub)
        float sc[STEPS];
#pragma unroll
        for (int step = 0; step < STEPS; ++step) {
            const int key = 2 * step + sub;
            float4 kr[C];
#pragma unroll
            for (int c = 0; c < C; ++c) kr[c] = at_row_piece<EB>(ks + (uint32_t)key * ROW, c * AT_LPK + li);
            float s[G];
#pragma unroll
            for (int h = 0; h < G; ++h) {
                float a = 0.0f;
#pragma unroll
                for (int c = 0; c < C; ++c) {
                    a = fmaf(q[h][c].x, kr[c].x, a);
                    a = fmaf(q[h][c].y, kr[c].y, a);
                    a = fmaf(q[h][c].z, kr[c].z, a);
                    a = fmaf(q[h][c].w, kr[c].w, a);
                }
                s[h] = a;
            }
            // transposing butterfly over lane bits 2, 1, 0, then a plain add over bit 3
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
            sc[step] = (warp * KPW + key < nvalid) ? s[0] : -INFINITY;
        }

        // ---- softmax update for these 8 keys (per head; identical on the lanes that share the head)
        float tmax = sc[0];
#pragma unroll
        for (int step = 1; step < STEPS; ++step) tmax = fmaxf(tmax, sc[step]);
        tmax = fmaxf(tmax, __shfl_xor_sync(0xffffffffu, tmax, 16));
        const float m_new = fmaxf(m_run, tmax);
        const float corr = m_run == -INFINITY ? 0.0f : expf(m_run - m_new);
        float pw[STEPS], psum = 0.0f;
#pragma unroll
        for (int step = 0; step < STEPS; ++step) {
            pw[step] = sc[step] == -INFINITY ? 0.0f : expf(sc[step] - m_new);
            psum += pw[step];
        }
        psum += __shfl_xor_sync(0xffffffffu, psum, 16);
        l_run = l_run * corr + psum;
        m_run = m_new;

        // ---- rescale once, then accumulate P.V
#pragma unroll
        for (int h = 0; h < G; ++h) {
            const float ch = __shfl_sync(0xffffffffu, corr, h);
#pragma unroll
            for (int c = 0; c < C; ++c) { acc[h][c].x *= ch; acc[h][c].y *= ch; acc[h][c].z *= ch; acc[h][c].w *= ch; }
        }
#pragma unroll
        for (int step = 0; step < STEPS; ++step) {
            const int key = 2 * step + sub;
            const bool valid = warp * KPW + key < nvalid;      // rows past the end of the context were never copied
            float4 vr[C];
#pragma unroll
            for (int c = 0; c < C; ++c) {
                vr[c] = at_row_piece<EB>(vs + (uint32_t)key * ROW, c * AT_LPK + li);
                if (!valid) vr[c] = make_float4(0.f, 0.f, 0.f, 0.f);
            }
#pragma unroll
            for (int h = 0; h < G; ++h) {
                const float ph = __shfl_sync(0xffffffffu, pw[step], sub * AT_LPK + h);
#pragma unroll
                for (int c = 0; c < C; ++c) {
                    acc[h][c].x = fmaf(ph, vr[c].x, acc[h][c].x);
                    acc[h][c].y = fmaf(ph, vr[c].y, acc[h][c].y);
                    acc[h][c].z = fmaf(ph, vr[c].z, acc[h][c].z);
                    acc[h][c].w = fmaf(ph, vr[c].w, acc[h][c].w);
                }
            }
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(AT_EMPTY(st));
    }
    AT_TRACE(tr, 2);
    if (!ok && lane == 0) atomicExch(dev_err, DEV_ERR_FULL_WAIT);
    ok = __syncthreads_and(ok ? 1 : 0) != 0;       // every issued copy has landed and been consumed when all warps got here
    if constexpr (!CLUSTER) {
        if (!ok) return;
    } else if (!ok) {                              // a cluster member may not leave before the cluster barriers: contribute nothing
        m_run = -INFINITY;
        l_run = 0.0f;
#pragma unroll
        for (int h = 0; h < G; ++h)
#pragma unroll
            for (int c = 0; c < C; ++c) acc[h][c] = make_float4(0.f, 0.f, 0.f, 0.f);
    }

    // ---- the two key streams of the warp share (m, l): add their accumulators; then merge the warps through shared memory
    float *merge_s = reinterpret_cast<float *>(smem);              // [AT_NW][G][AD + 4], over the (now idle) stages
#pragma unroll
    for (int h = 0; h < G; ++h)
#pragma unroll
        for (int c = 0; c < C; ++c) {
            acc[h][c].x += __shfl_xor_sync(0xffffffffu, acc[h][c].x, 16);
            acc[h][c].y += __shfl_xor_sync(0xffffffffu, acc[h][c].y, 16);
            acc[h][c].z += __shfl_xor_sync(0xffffffffu, acc[h][c].z, 16);
            acc[h][c].w += __shfl_xor_sync(0xffffffffu, acc[h][c].w, 16);
        }
    if (sub == 0) {
#pragma unroll
        for (int h = 0; h < G; ++h)
#pragma unroll
            for (int c = 0; c < C; ++c) *reinterpret_cast<float4 *>(&merge_s[((warp * G + h) * (AD + 4)) + (c * AT_LPK + li) * 4]) = acc[h][c];
        if (li < G) {
            merge_s[(warp * G + li) * (AD + 4) + AD] = m_run;
            merge_s[(warp * G + li) * (AD + 4) + AD + 1] = l_run;
        }
    }
    __syncthreads();
    if constexpr (CLUSTER) {
        // this CTA's result per head -> cta_s[h][0 .. AD) unnormalised output, [AD] max, [AD + 1] sum (behind the warps' area)
        float *cta_s = merge_s + AT_NW * G * (AD + 4);
        for (int i = threadIdx.x; i < group * (AD + 2); i += blockDim.x) {
            const int h = i / (AD + 2), c = i - h * (AD + 2);       // c < AD: an output column, AD: the max, AD + 1: the sum
            float mm = -INFINITY;
#pragma unroll
            for (int w = 0; w < AT_NW; ++w) mm = fmaxf(mm, merge_s[(w * G + h) * (AD + 4) + AD]);
            float val = mm;
            if (c != AD) {
                val = 0.0f;
#pragma unroll
                for (int w = 0; w < AT_NW; ++w) {
                    const float mw = merge_s[(w * G + h) * (AD + 4) + AD];
                    val += merge_s[(w * G + h) * (AD + 4) + c] * (mw == -INFINITY ? 0.0f : expf(mw - mm));
                }
            }
            cta_s[h * (AD + 4) + c] = val;
        }
        at_cluster_sync();                          // every rank's cta_s is complete and visible
        const uint32_t nrank = at_cluster_size(), me = at_cluster_rank();
        const uint32_t cta_a = smem_u32(cta_s);
        for (int i = (int)me * blockDim.x + threadIdx.x; i < group * AD; i += (int)nrank * blockDim.x) {
            const int h = i / AD, c = i - h * AD;
            float mm = -INFINITY;
            for (uint32_t r = 0; r < nrank; ++r) mm = fmaxf(mm, at_ld_peer(cta_a + 4u * (uint32_t)(h * (AD + 4) + AD), r));
            float ll = 0.0f, a = 0.0f;
            for (uint32_t r = 0; r < nrank; ++r) {
                const float mr = at_ld_peer(cta_a + 4u * (uint32_t)(h * (AD + 4) + AD), r);
                const float f = mr == -INFINITY ? 0.0f : expf(mr - mm);
                ll += at_ld_peer(cta_a + 4u * (uint32_t)(h * (AD + 4) + AD + 1), r) * f;
                a += at_ld_peer(cta_a + 4u * (uint32_t)(h * (AD + 4) + c), r) * f;
            }
            p.out[(size_t)seq * p.out_stride + (size_t)(h0 + h) * AD + c] = ll > 0.0f ? a / ll : 0.0f;
        }
        at_cluster_sync();                          // nobody's shared memory goes away while a peer may still read it
        return;
    }
    const bool fused = p.counters != nullptr;
    for (int i = threadIdx.x; i < group * AD; i += blockDim.x) {
        const int h = i / AD, c = i - h * AD;
        float mm = -INFINITY;
#pragma unroll
        for (int w = 0; w < AT_NW; ++w) mm = fmaxf(mm, merge_s[(w * G + h) * (AD + 4) + AD]);
        float ll = 0.0f, a = 0.0f;
#pragma unroll
        for (int w = 0; w < AT_NW; ++w) {
            const float mw = merge_s[(w * G + h) * (AD + 4) + AD];
            const float f = mw == -INFINITY ? 0.0f : expf(mw - mm);
            ll += merge_s[(w * G + h) * (AD + 4) + AD + 1] * f;
            a += merge_s[(w * G + h) * (AD + 4) + c] * f;
        }
        const size_t head = (size_t)seq * p.H + h0 + h;
        if (p.splits == 1) {
            p.out[(size_t)seq * p.out_stride + (size_t)(h0 + h) * AD + c] = ll > 0.0f ? a / ll : 0.0f;
        } else {
            float *dst = p.part + (head * p.splits + split) * (AD + 2);
            dst[c] = a;
            if (c == 0) { dst[AD] = mm; dst[AD + 1] = ll; }
        }
    }
    AT_TRACE(tr, 3);
    if (!fused) return;

    // ---- fused tail 1: the last split CTA of this (sequence, kv head) merges the partials of its heads
    __shared__ int s_last;
    float *f_s = merge_s + AT_NW * G * (AD + 4);       // [G][splits] factors, then [G] inverse sums
    if (p.splits > 1) {
        __threadfence();
        __syncthreads();
        if (threadIdx.x == 0) {
            int *cnt = p.counters + seq * p.Hkv + kvh;
            const int prev = atomicAdd(cnt, 1);
            s_last = prev == p.splits - 1;
            if (s_last) *cnt = 0;                      // ready for the next launch
        }
        __syncthreads();
        if (!s_last) return;
#ifdef CKB_STEP_TRACE
        if (kvh == 0 && seq == 0 && threadIdx.x == 0 && at_trace_n > 0) { tr = at_trace_n - 1; AT_TRACE(tr, 4); }
#endif
        __threadfence();
        const int S = p.splits;
        const float *part0 = p.part + ((size_t)seq * p.H + h0) * S * (AD + 2);
        for (int i = threadIdx.x; i < group * S; i += blockDim.x) f_s[i] = __ldcg(part0 + (size_t)i * (AD + 2) + AD);
        __syncthreads();
        if (warp < group) {
            float mm = -INFINITY;
            for (int s2 = lane; s2 < S; s2 += 32) mm = fmaxf(mm, f_s[warp * S + s2]);
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) mm = fmaxf(mm, __shfl_xor_sync(0xffffffffu, mm, o));
            float ll = 0.0f;
            for (int s2 = lane; s2 < S; s2 += 32) {
                const float ms = f_s[warp * S + s2];
                const float f = ms == -INFINITY ? 0.0f : expf(ms - mm);
                f_s[warp * S + s2] = f;
                ll += __ldcg(part0 + (size_t)(warp * S + s2) * (AD + 2) + AD + 1) * f;
            }
            ll = group_sum<32>(ll);
            if (lane == 0) f_s[G * S + warp] = ll > 0.0f ? 1.0f / ll : 0.0f;
        }
        __syncthreads();
        for (int i = threadIdx.x; i < group * AD; i += blockDim.x) {
            const int h = i / AD, c = i - h * AD;
            const float *src = part0 + (size_t)h * S * (AD + 2) + c;
            float a0 = 0.0f, a1 = 0.0f, a2 = 0.0f, a3 = 0.0f;
            int s2 = 0;
            for (; s2 + 4 <= S; s2 += 4) {
                const float v0 = __ldcg(src + (size_t)(s2 + 0) * (AD + 2)), v1 = __ldcg(src + (size_t)(s2 + 1) * (AD + 2));
                const float v2 = __ldcg(src + (size_t)(s2 + 2) * (AD + 2)), v3 = __ldcg(src + (size_t)(s2 + 3) * (AD + 2));
                a0 = fmaf(v0, f_s[h * S + s2], a0); a1 = fmaf(v1, f_s[h * S + s2 + 1], a1);
                a2 = fmaf(v2, f_s[h * S + s2 + 2], a2); a3 = fmaf(v3, f_s[h * S + s2 + 3], a3);
            }
            for (; s2 < S; ++s2) a0 = fmaf(__ldcg(src + (size_t)s2 * (AD + 2)), f_s[h * S + s2], a0);
            p.out[(size_t)seq * p.out_stride + (size_t)(h0 + h) * AD + c] = ((a0 + a1) + (a2 + a3)) * f_s[G * S + h];
        }
    }
#ifdef CKB_STEP_TRACE
    if (kvh == 0 && seq == 0 && threadIdx.x == 0) AT_TRACE(tr, 5);
#endif
    if (!p.q8_out) return;

    // ---- fused tail 2: the last kv head of this sequence quantises the finished row for the consumer GEMV
    __threadfence();
    __syncthreads();
    if (threadIdx.x == 0) {
        int *cnt = p.counters + gridDim.z * p.Hkv + seq;
        const int prev = atomicAdd(cnt, 1);
        s_last = prev == p.Hkv - 1;
        if (s_last) *cnt = 0;
    }
    __syncthreads();
    if (!s_last) return;
    __threadfence();
    const float *row = p.out + (size_t)seq * p.out_stride;
    uint8_t *qrow = p.q8_out + (size_t)seq * (p.q8_cols / 256) * Q8K_BYTES;
    for (int blk = warp; blk < p.q8_cols / 256; blk += AT_NW) {
        const float4 lo = __ldcg(reinterpret_cast<const float4 *>(row + blk * 256) + 2 * lane);
        const float4 hi = __ldcg(reinterpret_cast<const float4 *>(row + blk * 256) + 2 * lane + 1);
        const float v[8] = {lo.x, lo.y, lo.z, lo.w, hi.x, hi.y, hi.z, hi.w};
        quantize_block_q8k(v, qrow + (size_t)blk * Q8K_BYTES, lane);
    }
#undef AT_FULL
#undef AT_EMPTY
}

}  // namespace ckb

using namespace ckb;

// Launches the tile kernel for aligned_head_dim 64 or 128; the caller has checked group size and alignment.
template <int AD, int EB>
static int launch_attn_tile(const AttnParams *p, int batch, void *stream)
{
    const int smem = at_smem_bytes<AD>();
    static int attr_set = 0;
    if (!attr_set) {
        if (ckb_check_cuda((int)cudaFuncSetAttribute(attn_tile_kernel<AD, EB, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem), "attention smem attr")) return CKB_ERR_CUDA;
        attr_set = 1;
    }
    const dim3 grid(p->splits, p->Hkv, batch);
    return launch_pdl("attn_tile", attn_tile_kernel<AD, EB, false>, grid, dim3(AT_NW * 32), (size_t)smem, (cudaStream_t)stream, *p, ckb_device_error_word());
}

extern "C" int ckb_launch_attn_tile(const AttnParams *p, int batch, void *stream)
{
    if (p->kv_f16) return p->ad == 64 ? launch_attn_tile<64, 2>(p, batch, stream) : launch_attn_tile<128, 2>(p, batch, stream);
    return p->ad == 64 ? launch_attn_tile<64, 4>(p, batch, stream) : launch_attn_tile<128, 4>(p, batch, stream);
}

// The cluster form: grid (ranks, Hkv, batch) with the `ranks` CTAs of a kv head in one cluster (8: the portable maximum; 16 needs the
// opt-in attribute and is used when the device can place such a cluster).  Returns -1 when the launch is not possible here.
template <int AD, int EB>
static int launch_attn_cluster(const AttnParams *p, int batch, int ranks, void *stream)
{
    const int smem = at_smem_bytes<AD>();
    auto kernel = attn_tile_kernel<AD, EB, true>;
    static int attr_set = 0, max16 = -1;
    if (!attr_set) {
        if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem) != cudaSuccess) { cudaGetLastError(); return -1; }
        if (cudaFuncSetAttribute(kernel, cudaFuncAttributeNonPortableClusterSizeAllowed, 1) != cudaSuccess) { cudaGetLastError(); max16 = 0; }
        attr_set = 1;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(ranks, p->Hkv, batch);
    cfg.blockDim = dim3(AT_NW * 32);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = (cudaStream_t)stream;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = ranks;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[1].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = ckb_tune_get("pdl", 1) ? 2 : 1;
    if (ranks > 8) {
        if (max16 < 0) {
            int n = 0;
            if (cudaOccupancyMaxActiveClusters(&n, kernel, &cfg) != cudaSuccess) { cudaGetLastError(); n = 0; }
            max16 = n;
        }
        if (max16 <= 0) return -1;
    }
    if (cudaLaunchKernelEx(&cfg, kernel, *p, ckb_device_error_word()) != cudaSuccess) { cudaGetLastError(); return -1; }
    return ckb_check_launch("attn_cluster");
}

// ranks: CTAs per kv head (8 or 16).  -1: not available (the caller uses the split form).
extern "C" int ckb_launch_attn_cluster(const AttnParams *p, int batch, int ranks, void *stream)
{
    if (p->kv_f16) return p->ad == 64 ? launch_attn_cluster<64, 2>(p, batch, ranks, stream) : launch_attn_cluster<128, 2>(p, batch, ranks, stream);
    return p->ad == 64 ? launch_attn_cluster<64, 4>(p, batch, ranks, stream) : launch_attn_cluster<128, 4>(p, batch, ranks, stream);
}
