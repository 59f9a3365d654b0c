// Fused GEMV of the device-resident decode step: one launch produces the quantised activation vector, multiplies it with up
// to three weight matrices and finishes each output where its consumer wants it.
//
// The reference's generated decode function issues, per layer, residual add, RMSNorm, Q8_K quantisation, the q / k / v
// projections, RoPE, the KV-cache store, ... one call after another (version/v7/scripts/codegen_v7.py:569-931).  On a GPU each
// of those is a kernel launch, and for small models the step is nothing but the chain of launch latencies (a Qwen2-0.5B-shaped
// token streams 400 MB, 62 us at HBM speed, yet spent 820 us in 340 dependent launches).  This kernel removes the links:
//
//   prologue  (every CTA, redundantly: the vector is a few KB and comes from L2)
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

constexpr int SG_NW = 8;                 // warps per CTA
constexpr int SG_R = 2;                  // rows per lane group: the pair of an epilogue

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
__device__ __forceinline__ void sg_epilogue(const StepGemvParams &p, const StepSeg &sg, int n0, float s0, float s1, int pos)
{
    const int d = p.head_dim;
    switch (sg.epi) {
        case SG_EPI_ROPE_Q:
        case SG_EPI_ROPE_K: {
            if (pos < 0 || pos >= p.max_seq) return;
            const int half = d >> 1, h = n0 / d, j = (n0 - h * d) >> 1;
            const float c = p.cos_cache[(size_t)pos * half + j], sn = p.sin_cache[(size_t)pos * half + j];
            float *dst = sg.epi == SG_EPI_ROPE_Q ? sg.out + (size_t)h * d : sg.out + ((size_t)h * p.max_seq + pos) * d;
            dst[j] = __fsub_rn(__fmul_rn(s0, c), __fmul_rn(s1, sn));
            dst[j + half] = __fadd_rn(__fmul_rn(s0, sn), __fmul_rn(s1, c));
            return;
        }
        case SG_EPI_STORE_V: {
            if (pos < 0 || pos >= p.max_seq) return;
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
            sg.out[n0 >> 1] = __fmul_rn(__fmul_rn(s0, sgm), s1);
            return;
        }
        default:
            sg.out[n0] = s0;
            if (n0 + 1 < sg.M) sg.out[n0 + 1] = s1;
    }
}

// Builds the Q8_K vector of this launch in `raw` (shared memory) unless it already exists in global memory.
// Returns true when `raw` holds it.  Ends with the data written but not yet synchronised.
__device__ __forceinline__ bool sg_prologue(const StepGemvParams &p, uint8_t *raw, float *rowbuf, float *red)
{
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nb = p.nb;
    if (p.pro == SG_PRO_GLOBAL) return false;
    if (p.pro == SG_PRO_QUANT) {
        for (int b = warp; b < nb; b += SG_NW) {
            const float4 *s = reinterpret_cast<const float4 *>(p.src + (size_t)b * QK_K) + 2 * lane;
            const float4 lo = __ldcg(s), hi = __ldcg(s + 1);
            const float v[8] = {lo.x, lo.y, lo.z, lo.w, hi.x, hi.y, hi.z, hi.w};
            quantize_block_q8k(v, raw + (size_t)b * Q8K_BYTES, lane);
        }
        return true;
    }
    // SG_PRO_NORM
    const int aligned = nb * QK_K, nv = aligned >> 2;
    const bool writer = blockIdx.x == 0 && p.x_out != nullptr;
    const float4 *xin = reinterpret_cast<const float4 *>(p.x_in), *din = reinterpret_cast<const float4 *>(p.delta);
    float ss = 0.0f;
    for (int base = 0; base < nv; base += 4 * SG_NW * 32) {
        float4 xv[4], dv[4];
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            const int i = base + k * SG_NW * 32 + threadIdx.x;
            xv[k] = make_float4(0.f, 0.f, 0.f, 0.f);
            dv[k] = xv[k];
            if (i < nv) {
                xv[k] = __ldcg(xin + i);
                if (din) dv[k] = __ldcg(din + i);
            }
        }
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            const int i = base + k * SG_NW * 32 + threadIdx.x;
            if (i < nv) {
                float4 v = xv[k];
                v.x += dv[k].x; v.y += dv[k].y; v.z += dv[k].z; v.w += dv[k].w;
                if (writer) reinterpret_cast<float4 *>(p.x_out)[i] = v;       // pad columns of x and delta are zero by construction
                arq_keep_piece(v, i, p.d_model, rowbuf, ss);
            }
        }
    }
    ss = group_sum<32>(ss);
    if (lane == 0) red[warp] = ss;
    __syncthreads();
    float tot = 0.0f;
#pragma unroll
    for (int w = 0; w < SG_NW; ++w) tot += red[w];
    const float mean = __fmul_rn(tot, __fdiv_rn(1.0f, (float)p.d_model));
    const float rstd = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(mean, p.eps)));
    for (int b = warp; b < nb; b += SG_NW) {
        float v[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            const int i = b * QK_K + 8 * lane + j;
            v[j] = i < p.d_model ? __fmul_rn(__fmul_rn(rowbuf[i], rstd), __ldg(p.gamma + i)) : 0.0f;
        }
        quantize_block_q8k(v, raw + (size_t)b * Q8K_BYTES, lane);
    }
    return true;
}

// ---------------------------------------------------------------- Q4_K rows (the reference's 144-byte superblocks)

template <int G>
__device__ __forceinline__ void sg_run_q4k(const StepGemvParams &p, const StepSeg &sg, uint8_t *smem, float *red)
{
    constexpr int SPP = G / 2;                 // superblocks per pass of one row
    constexpr int RPW = (32 / G) * SG_R;       // rows per warp item
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int li = lane % G, sub = lane / G, pp = li & 1, b0 = li >> 1;
    const int nb = p.nb, M = sg.M, d = p.head_dim, epi = sg.epi;
    const int ntiles = (M + RPW - 1) / RPW;
    const int cta = blockIdx.x - sg.cta0, tile_stride = sg.ncta * SG_NW;
    const int npass = (nb + SPP - 1) / SPP;
    const size_t rb = (size_t)nb * Q4K_BYTES;
    const uint8_t *W = sg.W;

    auto load_item = [&](Q4pW (&w)[SG_R], int tile, int pass) {
        const int row0 = tile * RPW + sub * SG_R;
        const int b = min(b0 + pass * SPP, nb - 1);
#pragma unroll
        for (int r = 0; r < SG_R; ++r) {
            const uint8_t *pb = W + (size_t)sg_row(epi, min(row0 + r, M - 1), M, d) * rb + (size_t)b * Q4K_BYTES;
            w[r].hdr = __ldg(reinterpret_cast<const uint4 *>(pb));
            w[r].a0 = __ldg(reinterpret_cast<const uint4 *>(pb + 16 + 32 * pp));
            w[r].a1 = __ldg(reinterpret_cast<const uint4 *>(pb + 32 + 32 * pp));
            w[r].b0 = __ldg(reinterpret_cast<const uint4 *>(pb + 80 + 32 * pp));
            w[r].b1 = __ldg(reinterpret_cast<const uint4 *>(pb + 96 + 32 * pp));
        }
    };

    Q4pW cur[SG_R], nxt[SG_R];
    int tile = cta + sg.ncta * warp, pass = 0;
    if (tile < ntiles) load_item(cur, tile, 0);     // weights are never written by a kernel: safe before the wait

    pdl_wait();
    const int pos = p.pos ? __ldcg(p.pos) : 0;
    uint8_t *raw = smem, *work = smem + sg_raw_bytes(nb);
    const bool local = sg_prologue(p, raw, reinterpret_cast<float *>(work), red);
    __syncthreads();
    const Q4pX x = local ? q4p_stage_x<true>(raw, nb, work) : q4p_stage_x<false>(p.xq, nb, work);
    __syncthreads();

    float acc[SG_R];
#pragma unroll
    for (int r = 0; r < SG_R; ++r) acc[r] = 0.0f;
    while (tile < ntiles) {
        int ntile = tile, npass_i = pass + 1;
        if (npass_i == npass) { npass_i = 0; ntile = tile + tile_stride; }
        if (ntile < ntiles) load_item(nxt, ntile, npass_i);
        const int b = b0 + pass * SPP;
        if (b < nb) {
#pragma unroll
            for (int r = 0; r < SG_R; ++r) acc[r] += q4p_unit(cur[r], x, b, pp);
        }
        if (npass_i == 0) {                          // rows finished
            const int row0 = tile * RPW + sub * SG_R;
            const float s0 = group_sum<G>(acc[0]), s1 = group_sum<G>(acc[1]);
            if (li == 0 && row0 < M) sg_epilogue(p, sg, row0, s0, s1, pos);
            acc[0] = acc[1] = 0.0f;
        }
#pragma unroll
        for (int r = 0; r < SG_R; ++r) cur[r] = nxt[r];
        tile = ntile;
        pass = npass_i;
    }
}

// ---------------------------------------------------------------- Q6_K rows in the row-planar layout

template <int G>
__device__ __forceinline__ void sg_run_q6k(const StepGemvParams &p, const StepSeg &sg, uint8_t *smem, float *red)
{
    constexpr int SPP = G / 4;
    constexpr int RPW = (32 / G) * SG_R;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int li = lane % G, sub = lane / G, u = li & 3, b0 = li >> 2, n = u >> 1, h = u & 1;
    const int nb = p.nb, M = sg.M, d = p.head_dim, epi = sg.epi;
    const int nitems = (M + RPW - 1) / RPW;
    const int cta = blockIdx.x - sg.cta0, item_stride = sg.ncta * SG_NW;
    const int npass = (nb + SPP - 1) / SPP;
    const size_t rb = q6p_row_bytes(nb);
    const uint8_t *W = sg.W;

    auto load_item = [&](Q6pW (&w)[SG_R], int item, int pass) {
        const int row0 = item * RPW + sub * SG_R;
        const int b = min(b0 + pass * SPP, nb - 1);
#pragma unroll
        for (int r = 0; r < SG_R; ++r) q6p_load(w[r], W + (size_t)sg_row(epi, min(row0 + r, M - 1), M, d) * rb, nb, b, n, h);
    };

    Q6pW cur[SG_R], nxt[SG_R];
    int item = cta + sg.ncta * warp, pass = 0;
    if (item < nitems) load_item(cur, item, 0);

    pdl_wait();
    const int pos = p.pos ? __ldcg(p.pos) : 0;
    uint8_t *raw = smem, *work = smem + sg_raw_bytes(nb);
    const bool local = sg_prologue(p, raw, reinterpret_cast<float *>(work), red);
    __syncthreads();
    const RingX x = local ? ring_stage_x<FMT_Q6K, true>(raw, nb, work) : ring_stage_x<FMT_Q6K, false>(p.xq, nb, work);
    __syncthreads();

    float acc[SG_R];
#pragma unroll
    for (int r = 0; r < SG_R; ++r) acc[r] = 0.0f;
    while (item < nitems) {
        int nitem = item, npass_i = pass + 1;
        if (npass_i == npass) { npass_i = 0; nitem = item + item_stride; }
        if (nitem < nitems) load_item(nxt, nitem, npass_i);
        const int b = b0 + pass * SPP;
        if (b < nb) {
#pragma unroll
            for (int r = 0; r < SG_R; ++r) acc[r] += q6p_unit(cur[r], b, u, x);
        }
        if (npass_i == 0) {
            const int row0 = item * RPW + sub * SG_R;
            const float s0 = group_sum<G>(acc[0]), s1 = group_sum<G>(acc[1]);
            if (li == 0 && row0 < M) sg_epilogue(p, sg, row0, s0, s1, pos);
            acc[0] = acc[1] = 0.0f;
        }
#pragma unroll
        for (int r = 0; r < SG_R; ++r) cur[r] = nxt[r];
        item = nitem;
        pass = npass_i;
    }
}

// G4: lanes per Q4_K row (2 per superblock, a power of two up to 32); Q6_K rows take twice as many (4 per superblock)
template <int G4>
__global__ void __launch_bounds__(SG_NW * 32) step_gemv_kernel(const __grid_constant__ StepGemvParams p)
{
    extern __shared__ __align__(128) uint8_t smem[];
    __shared__ float red[SG_NW];
    constexpr int G6 = G4 * 2 > 32 ? 32 : G4 * 2;
    int s = 0;
    if (p.nseg > 1 && (int)blockIdx.x >= p.seg[1].cta0) s = 1;
    if (p.nseg > 2 && (int)blockIdx.x >= p.seg[2].cta0) s = 2;
    const StepSeg &sg = p.seg[s];
    pdl_trigger();
    if (sg.fmt == SG_FMT_Q4K) sg_run_q4k<G4>(p, sg, smem, red);
    else sg_run_q6k<G6>(p, sg, smem, red);
    if (p.pos_advance && blockIdx.x == 0 && threadIdx.x == 0) *p.pos_advance = __ldcg(p.pos_advance) + 1;
}

template <int G4>
static int sg_occupancy(int smem)
{
    static int cached_smem = -1, cached_occ = 1, attr_smem = 0;
    auto kernel = step_gemv_kernel<G4>;
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

template <int G4>
static int sg_launch(const StepGemvParams *p, int grid, cudaStream_t st)
{
    const int smem = sg_smem_bytes(p->nb, p->pro);
    if (sg_occupancy<G4>(smem) == 0) return ckb_fail(CKB_ERR_CUDA, "step_gemv: shared-memory attribute");
    return launch_pdl("step_gemv", step_gemv_kernel<G4>, dim3(grid), dim3(SG_NW * 32), (size_t)smem, st, *p);
}

static int sg_lanes(int nb)
{
    int g = 2;
    while (g < 32 && g < 2 * nb) g <<= 1;
    return g;
}

}  // namespace ckb

using namespace ckb;

extern "C" int ckb_step_gemv_ctas_per_sm(int nb, int pro)
{
    const int smem = sg_smem_bytes(nb, pro);
    if (smem > 200 * 1024) return 0;
    switch (sg_lanes(nb)) {
        case 2: return sg_occupancy<2>(smem);
        case 4: return sg_occupancy<4>(smem);
        case 8: return sg_occupancy<8>(smem);
        case 16: return sg_occupancy<16>(smem);
        default: return sg_occupancy<32>(smem);
    }
}

extern "C" int ckb_launch_step_gemv(const StepGemvParams *p, int grid, void *stream)
{
    if (!p || p->nseg < 1 || p->nseg > 3 || p->nb <= 0 || grid <= 0) return -1;
    if (sg_smem_bytes(p->nb, p->pro) > 200 * 1024) return -1;
    cudaStream_t st = ckb_stream(stream);
    switch (sg_lanes(p->nb)) {
        case 2: return sg_launch<2>(p, grid, st);
        case 4: return sg_launch<4>(p, grid, st);
        case 8: return sg_launch<8>(p, grid, st);
        case 16: return sg_launch<16>(p, grid, st);
        default: return sg_launch<32>(p, grid, st);
    }
}
