// Fused GEMV of the device-resident decode step: one launch produces the quantised activation vector, multiplies it with up
// to three weight matrices and finishes each output where its consumer wants it.
//
// The reference's generated decode function issues, per layer, residual add, RMSNorm, Q8_K quantisation, the q / k / v
// projections, RoPE, the KV-cache store, ... one call after another (version/v7/scripts/codegen_v7.py:569-931).  On a GPU each
// of those is a kernel launch, and for small models the step is nothing but the chain of launch latencies (a Qwen2-0.5B-shaped
// token streams 400 MB, 62 us at HBM speed, yet spent 820 us in 340 dependent launches).  This kernel removes the links:
//
//   prologue  (every CTA, redundantly: the vector is a few KB and comes from L2; NORM is limited to rows of 8 superblocks -
//             for wider rows the redundant reads of all CTAs cost more than a launch, and the caller runs the stand-alone
//             kernel and hands the quantised vector in)
//       NORM   x_new = x + delta, h = rmsnorm(x_new) * gamma, Q8_K(h) into shared memory    (ck_residual_add_token_major +
//              rmsnorm_forward + quantize_row_q8_k; the first CTA also stores x_new for the next consumer)
//       QUANT  Q8_K of an fp32 row into shared memory                                       (quantize_row_q8_k)
//   product   the Q4_K pair unit (q4p_unit.cuh) or the planar Q6_K unit (q6p_unit.cuh), two rows per lane group; a CTA works
//             on one segment (one weight matrix), segments get CTAs in proportion to their bytes
//   epilogue  STORE | ROPE_Q | ROPE_K (rope_forward_qk + kv_cache_store) | STORE_V (kv_cache_store) | SWIGLU (swiglu_forward)
//             - the two rows of a lane group are chosen so that the pair an epilogue needs (elements j and j + d/2 of a head;
//             gate and up of one output) ends up in one lane.
//
// The arithmetic of every piece is the one of the stand-alone kernels (same unit functions, same rounding calls), so a step
// built from these launches differs from the unfused step only where fp32 sums are taken in another order (the RMSNorm sum of
// squares when the thread count differs).  Launched with programmatic dependent launch: weights of the first work item are
// requested before the kernel waits for its predecessor.
#include "add_rmsnorm_q8k.cuh"
#include "launch.h"
#include "pdl.cuh"
#include "q4p_unit.cuh"
#include "q6p_unit.cuh"
#include "runtime.h"
#include "step_fused.h"

namespace ckb {

#ifdef CKB_STEP_TRACE
// Tuning aid (build with -DCKB_STEP_TRACE): the first thread of the first CTA of every launch records the global timer at
// kernel entry, after the dependency wait, after the activations are staged and at its end; ckb200_step_trace copies them out.
static __device__ unsigned long long sg_trace[8 * 8192];
static __device__ unsigned sg_trace_n;
static __device__ unsigned long long sg_trace_c0[8192];
__device__ __forceinline__ unsigned long long sg_now() { unsigned long long t; asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t)); return t; }
// stamp 0 is the global timer (comparable across kernels), the others are SM cycle counts (cheap to read); stamp 8 + k pairs the
// two clocks at entry
#define SG_TRACE(slot, k) do { if ((slot) < 8192u) sg_trace[8 * (slot) + (k)] = (k) == 0 ? sg_now() : (unsigned long long)clock64(); } while (0)
#else
#define SG_TRACE(slot, k) do { } while (0)
#endif

constexpr int SG_NW = 8;                 // warps per CTA
constexpr int SG_R = 2;                  // rows per lane group: the pair of an epilogue
constexpr int SG_MAX_HALF = 128;         // head_dim / 2 of the rope epilogues (cos / sin row staged in shared memory)

__host__ __device__ inline int sg_raw_bytes(int nb) { return (nb * Q8K_BYTES + 127) & ~127; }
__host__ __device__ inline int sg_work_bytes(int nb, int pro)
{
    const int a = q4p_smem_bytes(nb), b = ringx_smem_bytes(FMT_Q6K, nb), row = pro == SG_PRO_NORM ? nb * QK_K * 4 : 0;
    const int m = a > b ? a : b;
    return m > row ? m : row;
}
__host__ __device__ inline int sg_smem_bytes(int nb, int pro) { return sg_raw_bytes(nb) + sg_work_bytes(nb, pro); }

// logical row n of a segment -> row of the weight matrix; consecutive logical rows (2i, 2i + 1) are the pair of the epilogue
__device__ __forceinline__ int sg_row(int epi, int n, int M, int d)
{
    if (epi == SG_EPI_ROPE_Q || epi == SG_EPI_ROPE_K) {
        const int h = n / d, e = n - h * d;
        return h * d + (e >> 1) + (e & 1) * (d >> 1);
    }
    if (epi == SG_EPI_SWIGLU) return (n >> 1) + (n & 1) * (M >> 1);
    return n;
}

// the two finished dot products of logical rows n0, n0 + 1 (one lane)
__device__ __forceinline__ void sg_epilogue(const StepGemvParams &p, const StepSeg &sg, int n0, float s0, float s1, int pos, const float (*cs)[SG_MAX_HALF],
                                            bool live)
{
    const int d = p.head_dim;
    switch (sg.epi) {
        case SG_EPI_ROPE_Q:
        case SG_EPI_ROPE_K: {
            if (pos < 0 || pos >= p.max_seq) return;
            const int half = d >> 1, h = n0 / d, j = (n0 - h * d) >> 1;
            const float c = cs[0][j], sn = cs[1][j];                              // row `pos` of the tables, staged by sg_prefetch
            float *dst = sg.epi == SG_EPI_ROPE_Q ? sg.out + (size_t)h * d : sg.out + ((size_t)h * p.max_seq + pos) * d;
            const float o0 = __fsub_rn(__fmul_rn(s0, c), __fmul_rn(s1, sn)), o1 = __fadd_rn(__fmul_rn(s0, sn), __fmul_rn(s1, c));
            if (live) {
                dst[j] = o0;
                dst[j + half] = o1;
            }
            return;
        }
        case SG_EPI_STORE_V: {
            if (pos < 0 || pos >= p.max_seq || !live) return;
            const int h0 = n0 / d, e0 = n0 - h0 * d;
            sg.out[((size_t)h0 * p.max_seq + pos) * d + e0] = s0;
            if (n0 + 1 < sg.M) {
                const int h1 = (n0 + 1) / d, e1 = n0 + 1 - h1 * d;
                sg.out[((size_t)h1 * p.max_seq + pos) * d + e1] = s1;
            }
            return;
        }
        case SG_EPI_SWIGLU: {
            const float sgm = __fdiv_rn(1.0f, __fadd_rn(1.0f, expf(-s0)));
            const float o = __fmul_rn(__fmul_rn(s0, sgm), s1);
            if (live) sg.out[n0 >> 1] = o;
            return;
        }
        default:
            if (!live) return;
            sg.out[n0] = s0;
            if (n0 + 1 < sg.M) sg.out[n0 + 1] = s1;
    }
}

// What the prologue may fetch before the dependency wait: nothing of it is written by a kernel of the running step (the norm
// weights and the cos/sin table are constants; the position changes only at the very end of a step, and the first kernel of the
// next step is launched as a full dependency).
struct SgPre {
    float4 g0, g1;      // gamma of this lane's eight elements of block `warp` (NORM, rows of at most SG_NW superblocks)
    int pos;
};

__device__ __forceinline__ SgPre sg_prefetch(const StepGemvParams &p, const StepSeg &sg, float (*cs)[SG_MAX_HALF])
{
    SgPre pre;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    pre.g0 = pre.g1 = make_float4(0.f, 0.f, 0.f, 0.f);
    if (p.pro == SG_PRO_NORM && warp < p.nb) {
        const float4 *g = reinterpret_cast<const float4 *>(p.gamma + (size_t)warp * QK_K) + 2 * lane;
        pre.g0 = __ldg(g);
        pre.g1 = __ldg(g + 1);
    }
    pre.pos = p.pos ? __ldcg(p.pos) : 0;
    if ((sg.epi == SG_EPI_ROPE_Q || sg.epi == SG_EPI_ROPE_K) && pre.pos >= 0 && pre.pos < p.max_seq) {
        const int half = p.head_dim >> 1;
        for (int i = threadIdx.x; i < half; i += blockDim.x) {
            cs[0][i] = __ldg(p.cos_cache + (size_t)pre.pos * half + i);
            cs[1][i] = __ldg(p.sin_cache + (size_t)pre.pos * half + i);
        }
    }
    return pre;
}

// Builds the Q8_K vector of this launch in `raw` (shared memory) unless it already exists in global memory.
// Returns true when `raw` holds it.  Ends with the data written but not yet synchronised.
__device__ __forceinline__ bool sg_prologue(const StepGemvParams &p, const SgPre &pre, uint8_t *raw, float *rowbuf, float *red, unsigned tr, bool live)
{
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nb = p.nb;
    if (p.pro == SG_PRO_GLOBAL) return false;
    if (p.pro == SG_PRO_QUANT) {
        // up to four blocks per warp per round: all their loads are issued before the first block is quantised
        for (int bb = warp; bb < nb; bb += 4 * SG_NW) {
            float4 lo[4], hi[4];
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                const int b = bb + k * SG_NW;
                if (b < nb) {
                    const float4 *s = reinterpret_cast<const float4 *>(p.src + (size_t)b * QK_K) + 2 * lane;
                    lo[k] = __ldcg(s);
                    hi[k] = __ldcg(s + 1);
                }
            }
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                const int b = bb + k * SG_NW;
                if (b < nb) {
                    const float v[8] = {lo[k].x, lo[k].y, lo[k].z, lo[k].w, hi[k].x, hi[k].y, hi[k].z, hi[k].w};
                    quantize_block_q8k(v, raw + (size_t)b * Q8K_BYTES, lane);
                }
            }
        }
        return true;
    }
    // SG_PRO_NORM (rows of at most SG_NW superblocks: one block per warp)
    const int aligned = nb * QK_K, nv = aligned >> 2;
    const bool writer = blockIdx.x == 0 && p.x_out != nullptr && live;
    const float4 *xin = reinterpret_cast<const float4 *>(p.x_in), *din = reinterpret_cast<const float4 *>(p.delta);
    float ss = 0.0f;
    {
        float4 xv[2], dv[2];
#pragma unroll
        for (int k = 0; k < 2; ++k) {
            const int i = k * SG_NW * 32 + threadIdx.x;
            xv[k] = make_float4(0.f, 0.f, 0.f, 0.f);
            dv[k] = xv[k];
            if (i < nv) {
                xv[k] = __ldcg(xin + i);
                if (din) dv[k] = __ldcg(din + i);
            }
        }
#pragma unroll
        for (int k = 0; k < 2; ++k) {
            const int i = k * SG_NW * 32 + threadIdx.x;
            if (i < nv) {
                float4 v = xv[k];
                v.x += dv[k].x; v.y += dv[k].y; v.z += dv[k].z; v.w += dv[k].w;
                if (writer) reinterpret_cast<float4 *>(p.x_out)[i] = v;       // pad columns of x and delta are zero by construction
                arq_keep_piece(v, i, p.d_model, rowbuf, ss);
            }
        }
    }
    SG_TRACE(tr, 4);
    ss = group_sum<32>(ss);
    if (lane == 0) red[warp] = ss;
    __syncthreads();
    SG_TRACE(tr, 5);
    float tot = 0.0f;
#pragma unroll
    for (int w = 0; w < SG_NW; ++w) tot += red[w];
    const float mean = __fmul_rn(tot, __fdiv_rn(1.0f, (float)p.d_model));
    const float rstd = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(mean, p.eps)));
#ifdef CKB_STEP_TRACE_TWICE
#pragma unroll 1
    for (int rep = 0; rep < 2; ++rep) {
    if (rep == 1) SG_TRACE(tr, 6);
#endif
    if (warp < nb) {
        const float4 r0 = *reinterpret_cast<const float4 *>(rowbuf + warp * QK_K + 8 * lane), r1 = *reinterpret_cast<const float4 *>(rowbuf + warp * QK_K + 8 * lane + 4);
        const float rv[8] = {r0.x, r0.y, r0.z, r0.w, r1.x, r1.y, r1.z, r1.w};
        const float gv[8] = {pre.g0.x, pre.g0.y, pre.g0.z, pre.g0.w, pre.g1.x, pre.g1.y, pre.g1.z, pre.g1.w};
        float v[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) v[j] = (warp * QK_K + 8 * lane + j) < p.d_model ? __fmul_rn(__fmul_rn(rv[j], rstd), gv[j]) : 0.0f;
        quantize_block_q8k(v, raw + (size_t)warp * Q8K_BYTES, lane);
    }
#ifdef CKB_STEP_TRACE_TWICE
    }
    SG_TRACE(tr, 7);
#else
    SG_TRACE(tr, 6);
#endif
    return true;
}

// ---------------------------------------------------------------- the two weight formats behind one interface

struct SgQ4 {                                // the reference's 144-byte Q4_K superblocks, two lanes per superblock
    using W = Q4pW;
    using X = Q4pX;
    static constexpr int LPS = 2;
    static __device__ __forceinline__ size_t row_bytes(int nb) { return (size_t)nb * Q4K_BYTES; }
    static __device__ __forceinline__ void load(W &w, const uint8_t *row, int nb, int b, int u)
    {
        const uint8_t *pb = row + (size_t)b * Q4K_BYTES;
        w.hdr = __ldg(reinterpret_cast<const uint4 *>(pb));
        w.a0 = __ldg(reinterpret_cast<const uint4 *>(pb + 16 + 32 * u));
        w.a1 = __ldg(reinterpret_cast<const uint4 *>(pb + 32 + 32 * u));
        w.b0 = __ldg(reinterpret_cast<const uint4 *>(pb + 80 + 32 * u));
        w.b1 = __ldg(reinterpret_cast<const uint4 *>(pb + 96 + 32 * u));
    }
    static __device__ __forceinline__ float unit(const W &w, const X &x, int b, int u) { return q4p_unit(w, x, b, u); }
    template <bool LOCAL>
    static __device__ __forceinline__ X stage(const uint8_t *src, int nb, uint8_t *work) { return q4p_stage_x<LOCAL>(src, nb, work); }
};

struct SgQ6 {                                // Q6_K rows in the row-planar layout, four lanes per superblock
    using W = Q6pW;
    using X = RingX;
    static constexpr int LPS = 4;
    static __device__ __forceinline__ size_t row_bytes(int nb) { return q6p_row_bytes(nb); }
    static __device__ __forceinline__ void load(W &w, const uint8_t *row, int nb, int b, int u) { q6p_load(w, row, nb, b, u >> 1, u & 1); }
    static __device__ __forceinline__ float unit(const W &w, const X &x, int b, int u) { return q6p_unit(w, b, u, x); }
    template <bool LOCAL>
    static __device__ __forceinline__ X stage(const uint8_t *src, int nb, uint8_t *work) { return ring_stage_x<FMT_Q6K, LOCAL>(src, nb, work); }
};

// G lanes per row, T::LPS of them per superblock, so one pass covers G / LPS superblocks of a row.
//   SPLIT = false  a warp owns its rows and walks the passes itself, the loads of the next pass in flight while the current
//                  one is multiplied: the streaming form, for matrices of many megabytes
//   SPLIT = true   the passes of a row pair go to different warps of the CTA and meet in shared memory (fixed order): every
//                  warp has a single load round, issued before the dependency wait: the latency form, for small matrices
//                  with long rows
template <class T, int G, bool SPLIT, bool DRY>
__device__ __forceinline__ void sg_run(const StepGemvParams &p, const StepSeg &sg, uint8_t *smem, float *red, float (*part)[32], float (*cs)[SG_MAX_HALF],
                                       unsigned tr)
{
    constexpr int SPP = G / T::LPS;            // superblocks per pass of one row
    constexpr int RPW = (32 / G) * SG_R;       // rows per warp item
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int li = lane % G, sub = lane / G, u = li % T::LPS, b0 = li / T::LPS;
    const int nb = p.nb, M = sg.M, d = p.head_dim, epi = sg.epi;
    const int nitems = (M + RPW - 1) / RPW;
    const int cta = blockIdx.x - sg.cta0;
    const int npass = (nb + SPP - 1) / SPP;
    const size_t rb = T::row_bytes(nb);
    const uint8_t *Wm = sg.W;

    auto load_item = [&](typename T::W (&w)[SG_R], int item, int pass) {
        const int row0 = item * RPW + sub * SG_R;
        const int b = min(b0 + pass * SPP, nb - 1);
#pragma unroll
        for (int r = 0; r < SG_R; ++r) T::load(w[r], Wm + (size_t)sg_row(epi, min(row0 + r, M - 1), M, d) * rb, nb, b, u);
    };

    typename T::W cur[SG_R], nxt[SG_R];
    // the first work item of this warp: weights are never written by a kernel, so they are requested before the wait
    int item, pass, stride;
    if constexpr (SPLIT) {
        const int ipc = SG_NW / npass;                       // row pairs groups per CTA round (npass <= SG_NW)
        const int slot = warp / npass;
        pass = warp - slot * npass;
        item = slot < ipc ? cta * ipc + slot : nitems;       // warps beyond ipc * npass stay idle
        stride = sg.ncta * ipc;
    } else {
        item = cta + sg.ncta * warp;
        pass = 0;
        stride = sg.ncta * SG_NW;
    }
    if (item < nitems) load_item(cur, item, pass);
    const SgPre pre = sg_prefetch(p, sg, cs);

    // Everything from here on runs twice in the DRY instantiation (picked for small matrices, where the step is a chain of latencies): once BEFORE the dependency wait on whatever the input buffers
    // hold at that moment, with every global store switched off, and then for real.  The first pass costs nothing on the
    // critical path (the kernel would only be waiting for its predecessor) and leaves the instructions of the prologue, the
    // product and the epilogue in the instruction caches: a kernel that runs each of its instructions once per launch
    // otherwise spends about as long fetching them as executing them.
    uint8_t *raw = smem, *work = smem + sg_raw_bytes(nb);
#pragma unroll 1
    for (int live = DRY ? 0 : 1; live < 2; ++live) {
    if (live) {
        pdl_wait();
        SG_TRACE(tr, 1);
    }
    const bool local = sg_prologue(p, pre, raw, reinterpret_cast<float *>(work), red, tr, live != 0);
    __syncthreads();
#ifndef CKB_STEP_TRACE_TWICE
    SG_TRACE(tr, 7);
#endif
    const typename T::X x = local ? T::template stage<true>(raw, nb, work) : T::template stage<false>(p.xq, nb, work);
    __syncthreads();
    SG_TRACE(tr, 2);

    if constexpr (SPLIT) {
        // every warp of the CTA goes round together (the partial sums meet between two barriers)
        const int rounds = live ? (nitems + stride - 1) / stride : 1;
        const int ipc = SG_NW / npass, slot = warp / npass;
        for (int r = 0; r < rounds; ++r) {
            const int it = slot < ipc ? (cta + r * sg.ncta) * ipc + slot : nitems;
            const int nx = slot < ipc && live ? (cta + (r + 1) * sg.ncta) * ipc + slot : nitems;
            if (nx < nitems) load_item(nxt, nx, pass);
            float a0 = 0.0f, a1 = 0.0f;
            const int b = b0 + pass * SPP;
            if (it < nitems && b < nb) {
                a0 = T::unit(cur[0], x, b, u);
                a1 = T::unit(cur[1], x, b, u);
            }
            a0 = group_sum<G>(a0);
            a1 = group_sum<G>(a1);
            if (li == 0) { part[warp][2 * sub] = a0; part[warp][2 * sub + 1] = a1; }
            __syncthreads();
            if (it < nitems && pass == 0 && li == 0) {
                float s0 = 0.0f, s1 = 0.0f;
                for (int q = 0; q < npass; ++q) { s0 += part[warp + q][2 * sub]; s1 += part[warp + q][2 * sub + 1]; }
                const int row0 = it * RPW + sub * SG_R;
                if (row0 < M) sg_epilogue(p, sg, row0, s0, s1, pre.pos, cs, live != 0);
            }
            __syncthreads();
            if (live) {
#pragma unroll
                for (int q = 0; q < SG_R; ++q) cur[q] = nxt[q];
            }
        }
    } else {
        float acc[SG_R];
#pragma unroll
        for (int r = 0; r < SG_R; ++r) acc[r] = 0.0f;
        while (item < nitems) {
            int nitem = item, npass_i = pass + 1;
            if (npass_i == npass) { npass_i = 0; nitem = item + stride; }
            if (live && nitem < nitems) load_item(nxt, nitem, npass_i);
            const int b = b0 + pass * SPP;
            if (b < nb) {
#pragma unroll
                for (int r = 0; r < SG_R; ++r) acc[r] += T::unit(cur[r], x, b, u);
            }
            if (npass_i == 0 || !live) {                 // rows finished
                const int row0 = item * RPW + sub * SG_R;
                const float s0 = group_sum<G>(acc[0]), s1 = group_sum<G>(acc[1]);
                if (li == 0 && row0 < M) sg_epilogue(p, sg, row0, s0, s1, pre.pos, cs, live != 0);
                acc[0] = acc[1] = 0.0f;
            }
            if (!live) break;                            // the rehearsal stops after one item and keeps its weights
#pragma unroll
            for (int r = 0; r < SG_R; ++r) cur[r] = nxt[r];
            item = nitem;
            pass = npass_i;
        }
    }
    __syncthreads();                                     // the rehearsal's shared-memory reads are done before the real pass writes
    }
}

// G4: lanes per Q4_K row (2 per superblock, a power of two up to 32); Q6_K rows take twice as many (4 per superblock)
template <int G4, bool DRY>
__global__ void __launch_bounds__(SG_NW * 32) step_gemv_kernel(const __grid_constant__ StepGemvParams p)
{
    extern __shared__ __align__(128) uint8_t smem[];
    __shared__ float red[SG_NW];
    __shared__ float part[SG_NW][32];
    __shared__ float cs[2][SG_MAX_HALF];
    constexpr int G6 = G4 * 2 > 32 ? 32 : G4 * 2;
    int s = 0;
    if (p.nseg > 1 && (int)blockIdx.x >= p.seg[1].cta0) s = 1;
    if (p.nseg > 2 && (int)blockIdx.x >= p.seg[2].cta0) s = 2;
    const StepSeg &sg = p.seg[s];
    unsigned tr = 0xffffffffu;
#ifdef CKB_STEP_TRACE
    if (blockIdx.x == 0 && threadIdx.x == 0) tr = atomicAdd(&sg_trace_n, 1u);
    SG_TRACE(tr, 0);
    if (tr < 8192u) sg_trace_c0[tr] = (unsigned long long)clock64();
#endif
    pdl_trigger();
    if (sg.fmt == SG_FMT_Q4K) {
        if (sg.split) sg_run<SgQ4, G4, true, DRY>(p, sg, smem, red, part, cs, tr);
        else sg_run<SgQ4, G4, false, DRY>(p, sg, smem, red, part, cs, tr);
    } else {
        if (sg.split) sg_run<SgQ6, G6, true, DRY>(p, sg, smem, red, part, cs, tr);
        else sg_run<SgQ6, G6, false, DRY>(p, sg, smem, red, part, cs, tr);
    }
    SG_TRACE(tr, 3);
    if (p.pos_advance && blockIdx.x == 0 && threadIdx.x == 0) *p.pos_advance = __ldcg(p.pos_advance) + 1;
}

template <int G4, bool DRY>
static int sg_occupancy(int smem)
{
    static int cached_smem = -1, cached_occ = 1, attr_smem = 0;
    auto kernel = step_gemv_kernel<G4, DRY>;
    if (smem > 48 * 1024 && smem > attr_smem) {
        if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem) != cudaSuccess) { cudaGetLastError(); return 0; }
        attr_smem = smem;
    }
    if (cached_smem != smem) {
        int occ = 0;
        if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&occ, kernel, SG_NW * 32, smem) != cudaSuccess) { cudaGetLastError(); occ = 1; }
        cached_occ = occ < 1 ? 1 : occ;
        cached_smem = smem;
    }
    return cached_occ;
}

template <int G4, bool DRY>
static int sg_launch(const StepGemvParams *p, int grid, cudaStream_t st)
{
    const int smem = sg_smem_bytes(p->nb, p->pro);
    if (sg_occupancy<G4, DRY>(smem) == 0) return ckb_fail(CKB_ERR_CUDA, "step_gemv: shared-memory attribute");
    return launch_pdl("step_gemv", step_gemv_kernel<G4, DRY>, dim3(grid), dim3(SG_NW * 32), (size_t)smem, st, *p);
}

static int sg_lanes(int nb)
{
    int g = 2;
    while (g < 32 && g < 2 * nb) g <<= 1;
    return g;
}

}  // namespace ckb

using namespace ckb;

#ifdef CKB_STEP_TRACE
// copies up to `max_launches` records of four timestamps (ns) and resets the recorder; returns the number of launches recorded
extern "C" int ckb200_step_trace(unsigned long long *out, int max_launches)
{
    unsigned n = 0;
    cudaDeviceSynchronize();
    cudaMemcpyFromSymbol(&n, sg_trace_n, sizeof n);
    if (n > 8192u) n = 8192u;
    if ((int)n > max_launches) n = (unsigned)max_launches;
    if (n) {
        static unsigned long long raw[8 * 8192], c0[8192];
        cudaMemcpyFromSymbol(raw, sg_trace, (size_t)n * 8 * sizeof(unsigned long long));
        cudaMemcpyFromSymbol(c0, sg_trace_c0, (size_t)n * sizeof(unsigned long long));
        int khz = 1965000;
        cudaDeviceGetAttribute(&khz, cudaDevAttrClockRate, 0);
        for (unsigned i = 0; i < n; ++i) {                    // everything in ns on the global timer's axis
            out[8 * i] = raw[8 * i];
            for (int k = 1; k < 8; ++k) out[8 * i + k] = raw[8 * i] + (unsigned long long)((double)(raw[8 * i + k] - c0[i]) * 1.0e6 / khz);
        }
    }
    const unsigned zero = 0;
    cudaMemcpyToSymbol(sg_trace_n, &zero, sizeof zero);
    return (int)n;
}
#endif

#define SG_DISPATCH(FN, ...)                                                                        \
    switch (sg_lanes(nb)) {                                                                         \
        case 2: return dry ? FN<2, true>(__VA_ARGS__) : FN<2, false>(__VA_ARGS__);                  \
        case 4: return dry ? FN<4, true>(__VA_ARGS__) : FN<4, false>(__VA_ARGS__);                  \
        case 8: return dry ? FN<8, true>(__VA_ARGS__) : FN<8, false>(__VA_ARGS__);                  \
        case 16: return dry ? FN<16, true>(__VA_ARGS__) : FN<16, false>(__VA_ARGS__);               \
        default: return dry ? FN<32, true>(__VA_ARGS__) : FN<32, false>(__VA_ARGS__);               \
    }

extern "C" int ckb_step_gemv_ctas_per_sm(int nb, int pro, int dry)
{
    const int smem = sg_smem_bytes(nb, pro);
    if (smem > 200 * 1024) return 0;
    SG_DISPATCH(sg_occupancy, smem)
}

extern "C" int ckb_step_gemv_passes(int nb, int fmt)
{
    const int g4 = sg_lanes(nb), g = fmt == SG_FMT_Q6K_PLANAR ? (g4 * 2 > 32 ? 32 : g4 * 2) : g4;
    const int spp = g / (fmt == SG_FMT_Q6K_PLANAR ? 4 : 2);
    return (nb + spp - 1) / spp;
}

extern "C" int ckb_launch_step_gemv(const StepGemvParams *p, int grid, void *stream)
{
    if (!p || p->nseg < 1 || p->nseg > 3 || p->nb <= 0 || grid <= 0) return -1;
    if (sg_smem_bytes(p->nb, p->pro) > 200 * 1024) return -1;
    if (p->pro == SG_PRO_NORM && p->nb > SG_NORM_MAX_NB) return -1;
    for (int i = 0; i < p->nseg; ++i) {
        const StepSeg *sg = &p->seg[i];
        if ((sg->epi == SG_EPI_ROPE_Q || sg->epi == SG_EPI_ROPE_K) && (p->head_dim / 2 > SG_MAX_HALF || p->head_dim % 2 || sg->M % 2)) return -1;
        if (sg->epi == SG_EPI_SWIGLU && sg->M % 2) return -1;
        if (sg->split && ckb_step_gemv_passes(p->nb, sg->fmt) > SG_NW) return -1;
    }
    cudaStream_t st = ckb_stream(stream);
    const int nb = p->nb, dry = p->dry_run != 0;
    SG_DISPATCH(sg_launch, p, grid, st)
}
