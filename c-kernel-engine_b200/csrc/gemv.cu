// Dequant-dot GEMV y[M] = W[M,K] . x for Q4_K / Q6_K weights with Q8_K activations and Q8_0 weights
// with Q8_0 activations.  Replaces the reference's gemv_q4_k_q8_k / gemv_q6_k_q8_k / gemv_q8_0_q8_0
// (src/kernels/gemm_kernels_q4k_q8k.c:183-263, src/kernels/gemm_kernels_q6k_q8k.c:197-214 and :1060-1088,
// src/kernels/gemm_kernels_q8_0.c:1237-1251) and their *_parallel_simd row-split variants: the row split
// over threads becomes the grid.
//
// The kernels are HBM-bound: every weight byte is read exactly once, the activation vector is
// repacked once per CTA into shared memory, integer dots use dp4a and the per-row sums are
// reduced with warp shuffles.  Two families:
//
//   ring    each warp streams its rows through a private ring of shared-memory stages filled by
//           1-D bulk async copies (cp.async.bulk + mbarrier complete_tx); the 210-byte and 34-byte
//           block formats are only 2-byte aligned, so the copies take the 16-byte aligned superset
//           of a row range and the lanes index bytes from the remainder.  All waits are bounded.
//   direct  lanes read 16-byte pieces of 144-byte Q4_K superblocks straight from global memory
//           (always 16-byte aligned); Q6_K / Q8_0 use 2-byte loads.  Any shape, no shared staging.
#include "quant_units.cuh"
#include "pdl.cuh"
#include "ring_x.cuh"

namespace ckb {


template <int FMT> struct FmtTraits;
template <> struct FmtTraits<FMT_Q4K> { static constexpr int BS = Q4K_BYTES, UPB = 4, HP = 1; };
template <> struct FmtTraits<FMT_Q6K> { static constexpr int BS = Q6K_BYTES, UPB = 4, HP = 2; };
template <> struct FmtTraits<FMT_Q80> { static constexpr int BS = Q80_BYTES, UPB = 1, HP = 0; };
template <> struct FmtTraits<FMT_Q50> { static constexpr int BS = Q50_BYTES, UPB = 1, HP = 0; };

struct XView {           // repacked activations in shared memory (either layout)
    XQ8K k;              // Q8_K view (Q4_K / Q6_K weights)
    uint32_t q80;        // Q8_0 view (Q8_0 weights)
};

template <int FMT>
__device__ __forceinline__ XView load_x(const uint8_t *xg, int nb, uint8_t *smem)
{
    XView v;
    if constexpr (FMT == FMT_Q80 || FMT == FMT_Q50) {
        v.q80 = load_x_q80(xg, nb, smem);
        v.k.q = v.k.d = v.k.bs = 0;
    } else {
        v.k = load_x_q8k<FmtTraits<FMT>::HP>(xg, nb, smem);
        v.q80 = 0;
    }
    return v;
}

__host__ __device__ inline int x_smem_bytes(int fmt, int nb)
{
    const int raw = (fmt == FMT_Q80 || fmt == FMT_Q50) ? xq80_smem_bytes(nb) : xq8k_smem_bytes(nb, fmt == FMT_Q4K ? 1 : 2);
    return (raw + 127) & ~127;
}

// ---- one unit from GLOBAL memory: block pointer p (Q4_K: 16-byte aligned; others 2-byte), unit u of block b
template <int FMT>
__device__ __forceinline__ float unit_from_global(const uint8_t *p, int b, int u, const XView &x)
{
    if constexpr (FMT == FMT_Q4K) {
        const uint4 hdr = ldg_stream_u4(p);
        const uint4 qa = ldg_stream_u4(p + 16 + 32 * u);
        const uint4 qb = ldg_stream_u4(p + 32 + 32 * u);
        const Q4kX xr = q4k_load_x(x.k, b, u);
        return q4k_unit(hdr, qa, qb, xr, u);
    } else if constexpr (FMT == FMT_Q6K) {
        const int n = u >> 1, h = u & 1;
        const uint4 ql_a = ldg_u4_align2(p + 64 * n + 16 * h);
        const uint4 ql_b = ldg_u4_align2(p + 64 * n + 32 + 16 * h);
        const uint4 qh = ldg_u4_align2(p + 128 + 32 * n + 16 * h);
        const int8_t *sc = reinterpret_cast<const int8_t *>(p + 192 + 8 * n + h);
        const int s0 = __ldg(sc), s1 = __ldg(sc + 2), s2 = __ldg(sc + 4), s3 = __ldg(sc + 6);
        const uint32_t d = ldg_nc_u16(p + 208);
        const Q6kX xr = q6k_load_x(x.k, b, n, h);
        return q6k_unit(ql_a, ql_b, qh, s0, s1, s2, s3, d, xr);
    } else if constexpr (FMT == FMT_Q50) {
        const uint32_t d = ldg_nc_u16(p), qh = ldg_nc_u16(p + 2) | (ldg_nc_u16(p + 4) << 16);
        return q50_unit(d, qh, ldg_u4_align2(p + 6), x.q80 + 48u * b);
    } else {
        const uint32_t d = ldg_nc_u16(p);
        const uint4 w0 = ldg_u4_align2(p + 2), w1 = ldg_u4_align2(p + 18);
        const uint32_t xa = x.q80 + 48u * b;
        const uint4 x0 = lds_u4(xa), x1 = lds_u4(xa + 16);
        const float xd = __uint_as_float(lds_u32(xa + 32));
        int s = 0;
        s = dp4a_ss(w0.x, x0.x, s); s = dp4a_ss(w0.y, x0.y, s); s = dp4a_ss(w0.z, x0.z, s); s = dp4a_ss(w0.w, x0.w, s);
        s = dp4a_ss(w1.x, x1.x, s); s = dp4a_ss(w1.y, x1.y, s); s = dp4a_ss(w1.z, x1.z, s); s = dp4a_ss(w1.w, x1.w, s);
        return (float)s * (half_bits_to_float(d) * xd);
    }
}

// ---- one unit from SHARED memory: block at shared address a (same alignment rules), unit u of block b
template <int FMT>
__device__ __forceinline__ float unit_from_shared(uint32_t a, int b, int u, const XView &x)
{
    if constexpr (FMT == FMT_Q4K) {
        const uint4 hdr = lds_u4(a);
        const uint4 qa = lds_u4(a + 16 + 32 * u);
        const uint4 qb = lds_u4(a + 32 + 32 * u);
        const Q4kX xr = q4k_load_x(x.k, b, u);
        return q4k_unit(hdr, qa, qb, xr, u);
    } else if constexpr (FMT == FMT_Q6K) {
        const int n = u >> 1, h = u & 1;
        const uint4 ql_a = lds_u4_align2(a + 64 * n + 16 * h);
        const uint4 ql_b = lds_u4_align2(a + 64 * n + 32 + 16 * h);
        const uint4 qh = lds_u4_align2(a + 128 + 32 * n + 16 * h);
        const uint32_t sa = a + 192 + 8 * n + h;
        const int s0 = lds_s8(sa), s1 = lds_s8(sa + 2), s2 = lds_s8(sa + 4), s3 = lds_s8(sa + 6);
        const uint32_t d = lds_u16(a + 208);
        const Q6kX xr = q6k_load_x(x.k, b, n, h);
        return q6k_unit(ql_a, ql_b, qh, s0, s1, s2, s3, d, xr);
    } else if constexpr (FMT == FMT_Q50) {
        const uint32_t d = lds_u16(a), qh = lds_u16(a + 2) | (lds_u16(a + 4) << 16);
        return q50_unit(d, qh, lds_u4_align2(a + 6), x.q80 + 48u * b);
    } else {
        const uint32_t d = lds_u16(a);
        const uint4 w0 = lds_u4_align2(a + 2), w1 = lds_u4_align2(a + 18);
        const uint32_t xa = x.q80 + 48u * b;
        const uint4 x0 = lds_u4(xa), x1 = lds_u4(xa + 16);
        const float xd = __uint_as_float(lds_u32(xa + 32));
        int s = 0;
        s = dp4a_ss(w0.x, x0.x, s); s = dp4a_ss(w0.y, x0.y, s); s = dp4a_ss(w0.z, x0.z, s); s = dp4a_ss(w0.w, x0.w, s);
        s = dp4a_ss(w1.x, x1.x, s); s = dp4a_ss(w1.y, x1.y, s); s = dp4a_ss(w1.z, x1.z, s); s = dp4a_ss(w1.w, x1.w, s);
        return (float)s * (half_bits_to_float(d) * xd);
    }
}

__device__ __forceinline__ float group_sum_rt(float v, int width)
{
    for (int o = width >> 1; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

// =====================================================================================
// direct family, generic: one warp per row, units strided over the lanes.
// =====================================================================================
template <int FMT, int NW>
__global__ void __launch_bounds__(NW * 32) gemv_direct_kernel(const uint8_t *__restrict__ W, const uint8_t *__restrict__ xg,
                                                              float *__restrict__ y, int M, int nb)
{
    extern __shared__ __align__(128) uint8_t smem[];
    const XView x = load_x<FMT>(xg, nb, smem);
    __syncthreads();
    constexpr int BS = FmtTraits<FMT>::BS, UPB = FmtTraits<FMT>::UPB;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int units = nb * UPB;
    for (int row = blockIdx.x * NW + warp; row < M; row += gridDim.x * NW) {
        const uint8_t *wr = W + (size_t)row * nb * BS;
        float acc = 0.0f;
        for (int u = lane; u < units; u += 32) {
            const int b = u / UPB;
            acc += unit_from_global<FMT>(wr + (size_t)b * BS, b, u - b * UPB, x);
        }
        acc = group_sum<32>(acc);
        if (lane == 0) y[row] = acc;
    }
}

// =====================================================================================
// direct family, Q4_K tuned: G lanes per row, R rows per lane group share the activation registers.
// =====================================================================================
template <int G, int R, int NW>
__global__ void __launch_bounds__(NW * 32) gemv_q4k_direct_kernel(const uint8_t *__restrict__ W, const uint8_t *__restrict__ xg,
                                                                  float *__restrict__ y, int M, int nb)
{
    extern __shared__ __align__(128) uint8_t smem[];
    const XView x = load_x<FMT_Q4K>(xg, nb, smem);
    __syncthreads();
    constexpr int RPW = (32 / G) * R;          // rows per warp pass
    constexpr int SPI = G / 4;                 // superblocks per pass of one row
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int li = lane % G, sub = lane / G, q = li & 3, b0 = li >> 2;
    const int ntiles = (M + NW * RPW - 1) / (NW * RPW);
    const size_t rb = (size_t)nb * Q4K_BYTES;
    for (int tile = blockIdx.x; tile < ntiles; tile += gridDim.x) {
        const int row0 = (tile * NW + warp) * RPW + sub * R;
        const uint8_t *wr[R];
        float acc[R];
#pragma unroll
        for (int j = 0; j < R; ++j) {
            wr[j] = W + (size_t)min(row0 + j, M - 1) * rb + 32 * q;
            acc[j] = 0.0f;
        }
        for (int b = b0; b < nb; b += SPI) {
            uint4 hdr[R], qa[R], qb[R];
#pragma unroll
            for (int j = 0; j < R; ++j) {
                const uint8_t *p = wr[j] + (size_t)b * Q4K_BYTES;
                hdr[j] = ldg_stream_u4(p - 32 * q);
                qa[j] = ldg_stream_u4(p + 16);
                qb[j] = ldg_stream_u4(p + 32);
            }
            const Q4kX xr = q4k_load_x(x.k, b, q);
#pragma unroll
            for (int j = 0; j < R; ++j) acc[j] += q4k_unit(hdr[j], qa[j], qb[j], xr, q);
        }
#pragma unroll
        for (int j = 0; j < R; ++j) {
            const float s = group_sum<G>(acc[j]);
            if (li == 0 && row0 + j < M) y[row0 + j] = s;
        }
    }
}

// =====================================================================================
// ring family helpers: activation staging (coherent, batched) and the Q6_K unit used by the ring kernel
// =====================================================================================

// Q6_K quarter (n, h) from shared memory.  sum (q6 - 32) * x is split so that no 6-bit value is ever
// assembled: the nibble planes and the 2-bit planes are multiplied in place (masked, not shifted) and
// the place values are applied to the int32 sums; the -32 goes through the activation block sums.
__device__ __forceinline__ float q6k_ring_unit(uint32_t a, int b, int u, const RingX &x)
{
    const int n = u >> 1, h = u & 1;
    const uint4 qa = lds_u4_align2(a + 64 * n + 16 * h);
    const uint4 qb = lds_u4_align2(a + 64 * n + 32 + 16 * h);
    const uint4 qh = lds_u4_align2(a + 128 + 32 * n + 16 * h);
    const uint32_t sa = a + 192 + 8 * n + h;
    const int s0 = lds_s8(sa), s1 = lds_s8(sa + 2), s2 = lds_s8(sa + 4), s3 = lds_s8(sa + 6);
    const uint32_t dbits = lds_u16(a + 208);
    const uint32_t xa = x.q + (uint32_t)(b * 80 + (10 * n + h) * 4) * 4u;
    const uint4 x0 = lds_u4(xa), x1 = lds_u4(xa + 32), x2 = lds_u4(xa + 64), x3 = lds_u4(xa + 96);
    int S1, S2, S3, S4;
    q6k_plane_sums(qa, qb, qh, x0, x1, x2, x3, S1, S2, S3, S4);
    const uint32_t sc4 = __byte_perm(__byte_perm((uint32_t)s0, (uint32_t)s1, 0x0040), __byte_perm((uint32_t)s2, (uint32_t)s3, 0x0040), 0x5410);
    const uint32_t lo4 = lds_u32(x.lo + 4u * (b * 4 + u)), hi4 = lds_u32(x.hi + 4u * (b * 4 + u));
    const int center = dp4a_ss(sc4, lo4, 0) + 128 * dp4a_ss(sc4, hi4, 0);          // sum_t sc_t * bsum_t
    const int tot = s0 * S1 + s1 * S2 + s2 * S3 + s3 * S4 - 32 * center;
    const float xd = __uint_as_float(lds_u32(x.d + 4u * b));
    return (half_bits_to_float(dbits) * xd) * (float)tot;
}

// =====================================================================================
// ring family: warp-private rings of bulk-copied stages.
// =====================================================================================
struct RingPlan {
    int stage_bytes;     // bytes per stage (multiple of 128)
    int rows_per_tile;   // whole rows per tile (mode A) or 1 (mode B)
    int blocks_per_chunk;// blocks of a row per tile (== nb in mode A)
    int chunks;          // chunks per row (1 in mode A)
    int lanes_per_row;   // power of two <= 32; 32 in mode B
};

template <int FMT>
__device__ __forceinline__ float ring_unit(uint32_t a, int b, int u, const RingX &x)
{
    if constexpr (FMT == FMT_Q6K) {
        return q6k_ring_unit(a, b, u, x);
    } else {
        XView v;
        v.k.q = x.q; v.k.d = x.d; v.k.bs = x.lo; v.q80 = x.q;
        return unit_from_shared<FMT>(a, b, u, v);
    }
}

// Programmatic dependent launch: the first stages of every warp's ring (weights only) are requested before
// the kernel waits for its predecessor, the activation vector is staged after the wait.
template <int FMT, int NWC, int D>
__global__ void __launch_bounds__(NWC * 32, 1) gemv_ring_kernel(const uint8_t *__restrict__ W, const uint8_t *__restrict__ xg,
                                                                 float *__restrict__ y, int M, int nb, RingPlan plan,
                                                                 int *__restrict__ dev_err)
{
    extern __shared__ __align__(128) uint8_t smem[];
    constexpr int BS = FmtTraits<FMT>::BS, UPB = FmtTraits<FMT>::UPB;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int xbytes = ringx_smem_bytes(FMT, nb);
    uint8_t *ring = smem + xbytes + (size_t)warp * D * plan.stage_bytes;
    uint64_t *bars = reinterpret_cast<uint64_t *>(smem + xbytes + (size_t)NWC * D * plan.stage_bytes) + warp * D;
    const uint32_t ring_a = smem_u32(ring), bar_a = smem_u32(bars);

    asm volatile("griddepcontrol.launch_dependents;");

    const size_t rb = (size_t)nb * BS;
    const int RT = plan.rows_per_tile, CB = plan.blocks_per_chunk, NCH = plan.chunks, G = plan.lanes_per_row;
    const int n_row_tiles = (M + RT - 1) / RT;
    const int gw = blockIdx.x * NWC + warp, TW = gridDim.x * NWC;
    const int my_row_tiles = gw < n_row_tiles ? (n_row_tiles - gw + TW - 1) / TW : 0;
    const int n_mine = my_row_tiles * NCH;

    // tile i of this warp -> (first row, rows, first block, blocks, global byte address)
    auto tile_of = [&](int i, int &row0, int &nrows, int &blk0, int &nblk, const uint8_t *&g0, uint32_t &bytes) {
        const int rt = gw + (i / NCH) * TW, c = i - (i / NCH) * NCH;
        row0 = rt * RT;
        nrows = min(RT, M - row0);
        blk0 = c * CB;
        nblk = min(CB, nb - blk0);
        g0 = W + (size_t)row0 * rb + (size_t)blk0 * BS;
        const size_t need = (size_t)(nrows - 1) * rb + (size_t)nblk * BS;
        const uintptr_t a0 = (uintptr_t)g0 & ~(uintptr_t)15, a1 = ((uintptr_t)g0 + need + 15) & ~(uintptr_t)15;
        bytes = (uint32_t)(a1 - a0);
    };
    auto issue = [&](int i) {
        int row0, nrows, blk0, nblk;
        const uint8_t *g0;
        uint32_t bytes;
        tile_of(i, row0, nrows, blk0, nblk, g0, bytes);
        const int s = i % D;
        mbar_arrive_expect_tx(bar_a + 8 * s, bytes);
        bulk_g2s(ring_a + s * plan.stage_bytes, (const void *)((uintptr_t)g0 & ~(uintptr_t)15), bytes, bar_a + 8 * s);
    };

    if (lane == 0) {
#pragma unroll
        for (int s = 0; s < D; ++s) mbar_init(bar_a + 8 * s, 1);
        mbar_fence_init();
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        for (int i = 0; i < min(D, n_mine); ++i) issue(i);          // weights: nothing ever writes them
    }

    asm volatile("griddepcontrol.wait;" ::: "memory");
    const RingX x = ring_stage_x<FMT>(xg, nb, smem);
    __syncthreads();

    const int li = lane & (G - 1), sub = lane / G, rows_per_pass = 32 / G;
    float acc = 0.0f;
    int i = 0;
    bool ok = true;
    for (; i < n_mine; ++i) {
        const int s = i % D;
        // the verdict is made warp-uniform so that no lane leaves the loop alone
        if (!__all_sync(0xffffffffu, mbar_wait_bounded(bar_a + 8 * s, (i / D) & 1))) { ok = false; break; }
        int row0, nrows, blk0, nblk;
        const uint8_t *g0;
        uint32_t bytes;
        tile_of(i, row0, nrows, blk0, nblk, g0, bytes);
        const uint32_t base = ring_a + s * plan.stage_bytes + (uint32_t)((uintptr_t)g0 & 15);
        const bool first_chunk = blk0 == 0, last_chunk = blk0 + nblk == nb;
        const int units = nblk * UPB;
        for (int r0 = 0; r0 < nrows; r0 += rows_per_pass) {
            const int r = r0 + sub;
            if (first_chunk) acc = 0.0f;
            if (r < nrows) {
                const uint32_t ra = base + (uint32_t)(r * rb);
                for (int u = li; u < units; u += G) {
                    const int b = u / UPB;
                    acc += ring_unit<FMT>(ra + b * BS, blk0 + b, u - b * UPB, x);
                }
            }
            if (last_chunk) {
                const float sum = group_sum_rt(acc, G);
                if (li == 0 && r < nrows) y[row0 + r] = sum;
            }
        }
        __syncwarp();
        if (lane == 0 && i + D < n_mine) {
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            issue(i + D);
        }
    }
    if (!ok) {
        // give up: record it, then wait (bounded) for the copies still in flight before leaving
        if (lane == 0) atomicExch(dev_err, DEV_ERR_FULL_WAIT);
        for (int j = i + 1; j < min(i + D, n_mine); ++j) mbar_wait_bounded(bar_a + 8 * (j % D), (j / D) & 1);
    }
}

}  // namespace ckb

// =====================================================================================
// host launchers
// =====================================================================================
using namespace ckb;

namespace {

constexpr int RING_NWC = 16, RING_D = 3;
constexpr int SMEM_BUDGET = 200 * 1024;   // ring + activations; the SM has 227 KB per CTA

template <typename KernelT>
int set_smem(KernelT kernel, int bytes)
{
    if (bytes <= 48 * 1024) return 0;
    return ckb_check_cuda((int)cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes), "smem attr");
}

template <int FMT>
int launch_direct_generic(float *y, const void *W, const void *xq, int M, int nb, cudaStream_t st)
{
    constexpr int NW = 8;
    const int smem = x_smem_bytes(FMT, nb);
    if (smem > 220 * 1024) return ckb_fail(CKB_ERR_LIMIT, "gemv: K too large for the shared activation buffer");
    if (set_smem(gemv_direct_kernel<FMT, NW>, smem)) return CKB_ERR_CUDA;
    const int grid = min((M + NW - 1) / NW, ckb_sm_count() * 4);
    gemv_direct_kernel<FMT, NW><<<grid, NW * 32, smem, st>>>((const uint8_t *)W, (const uint8_t *)xq, y, M, nb);
    return ckb_check_launch("gemv_direct");
}

template <int G, int R>
int launch_q4k_direct(float *y, const void *W, const void *xq, int M, int nb, cudaStream_t st)
{
    constexpr int NW = 8;
    const int smem = x_smem_bytes(FMT_Q4K, nb);
    if (smem > 220 * 1024) return ckb_fail(CKB_ERR_LIMIT, "gemv_q4_k: K too large for the shared activation buffer");
    if (set_smem(gemv_q4k_direct_kernel<G, R, NW>, smem)) return CKB_ERR_CUDA;
    constexpr int rows_per_cta = NW * (32 / G) * R;
    const int ntiles = (M + rows_per_cta - 1) / rows_per_cta;
    const int grid = min(ntiles, ckb_sm_count() * 4);
    gemv_q4k_direct_kernel<G, R, NW><<<grid, NW * 32, smem, st>>>((const uint8_t *)W, (const uint8_t *)xq, y, M, nb);
    return ckb_check_launch("gemv_q4k_direct");
}

// Picks the ring geometry.  Returns false when a row chunk cannot fit (never for the supported formats).
bool plan_ring(int fmt, int bs, int upb, int M, int nb, int grid, RingPlan &p)
{
    const int xb = ringx_smem_bytes(fmt, nb);
    int stage = (SMEM_BUDGET - xb) / (RING_NWC * RING_D);
    stage &= ~127;
    const int cap = ckb_tune_get("ring_stage_bytes", 0);
    if (cap > 0 && cap < stage) stage = cap & ~127;
    if (stage < 1024) return false;
    p.stage_bytes = stage;
    const long long rb = (long long)nb * bs;
    const int usable = stage - 32;   // aligned superset adds at most 30 bytes
    const int TW = grid * RING_NWC;
    if (rb <= usable) {
        const int units = nb * upb;
        int g = 1;
        while (g < 32 && g < units) g <<= 1;
        p.lanes_per_row = g;
        const int rt_max = (int)min((long long)64, usable / rb);
        // balance: minimise the worst warp's row count; prefer bigger tiles on ties
        int best = 1;
        long long best_cost = -1;
        for (int rt = 1; rt <= rt_max; ++rt) {
            const long long tiles = (M + rt - 1) / rt, waves = (tiles + TW - 1) / TW;
            const long long cost = waves * rt;
            if (best_cost < 0 || cost <= best_cost) { best_cost = cost; best = rt; }
        }
        p.rows_per_tile = best;
        p.blocks_per_chunk = nb;
        p.chunks = 1;
    } else {
        p.lanes_per_row = 32;
        p.rows_per_tile = 1;
        int cb = usable / bs;
        const int chunks = (nb + cb - 1) / cb;
        cb = (nb + chunks - 1) / chunks;   // even chunks
        p.blocks_per_chunk = cb;
        p.chunks = chunks;
    }
    return true;
}

template <int FMT>
int launch_ring(float *y, const void *W, const void *xq, int M, int nb, cudaStream_t st)
{
    constexpr int BS = FmtTraits<FMT>::BS, UPB = FmtTraits<FMT>::UPB;
    if ((uintptr_t)W & 15) return ckb_fail(CKB_ERR_ALIGN, "gemv (ring): W must be 16-byte aligned");
    const int grid = ckb_sm_count();
    RingPlan plan;
    if (!plan_ring(FMT, BS, UPB, M, nb, grid, plan)) return ckb_fail(CKB_ERR_LIMIT, "gemv (ring): K too large");
    const int smem = ringx_smem_bytes(FMT, nb) + RING_NWC * RING_D * plan.stage_bytes + RING_NWC * RING_D * 8;
    static int attr_set = 0;
    if (smem > attr_set) {
        if (set_smem(gemv_ring_kernel<FMT, RING_NWC, RING_D>, smem)) return CKB_ERR_CUDA;
        attr_set = smem;
    }
    return launch_pdl("gemv_ring", gemv_ring_kernel<FMT, RING_NWC, RING_D>, dim3(grid), dim3(RING_NWC * 32), (size_t)smem, st,
                      (const uint8_t *)W, (const uint8_t *)xq, y, M, nb, plan, ckb_device_error_word());
}

int check_common(const char *name, const void *y, const void *W, const void *xq, int M, int K, int blk)
{
    if (!y || !W || !xq || M <= 0 || K <= 0) return 1;   // the reference returns silently here
    if (K % blk) { ckb_fail(CKB_ERR_SHAPE, "%s: K=%d is not a multiple of %d", name, K, blk); return 2; }
    if ((uintptr_t)y & 3) { ckb_fail(CKB_ERR_ALIGN, "%s: y must be 4-byte aligned", name); return 2; }
    return 0;
}

}  // namespace

extern "C" int ckb_launch_gemv_q4k_pair(float *y, const void *W, const void *xq, int M, int nb, int r, int l1alloc, void *stream);   // gemv_q4k.cu
extern "C" int ckb_launch_gemv_q4k_xreg(float *y, const void *W, const void *xq, int M, int nb, int r, int l1alloc, void *stream);   // gemv_q4k_xreg.cu

// variant: 0 auto, 1 ring, 2 direct generic, 10.. direct with G lanes per row / R rows, 20/21 pair kernel (R = 1 / 2)
extern "C" int ckb200_dev_gemv_q4_k_q8_k(float *y, const void *W, const void *xq, int M, int K, void *stream)
{
    const int c = check_common("gemv_q4_k_q8_k", y, W, xq, M, K, QK_K);
    if (c) return c == 1 ? 0 : CKB_ERR_SHAPE;
    if (((uintptr_t)W & 15) || ((uintptr_t)xq & 3))
        return ckb_fail(CKB_ERR_ALIGN, "gemv_q4_k_q8_k: W must be 16-byte and x_q8 4-byte aligned");
    const int nb = K / QK_K;
    if (ckb_ensure_init()) return CKB_ERR_NO_DEVICE;
    cudaStream_t st = ckb_stream(stream);
    int v = ckb_tune_get("gemv_q4_k", 0);
    if (v == 0) {
        // measured on B200 over the benchmark and decode shapes: few rows -> activations in registers
        // (every warp bound to one pass of the row); otherwise the shared-activation pair kernel with
        // L1-allocating loads, two rows per step unless rows are a single pass
        if (M <= 2048 && nb <= 128) v = 32;
        else v = nb <= 4 ? 22 : 23;
    }
    switch (v) {
        case 30: case 31: case 32: case 33: {
            const int rc = ckb_launch_gemv_q4k_xreg(y, W, xq, M, nb, (v & 1) ? 2 : 1, v >= 32, st);
            if (rc >= 0) return rc;
            return launch_q4k_direct<32, 2>(y, W, xq, M, nb, st);      // rows longer than 8 passes
        }
        case 20: case 21: case 22: case 23: return ckb_launch_gemv_q4k_pair(y, W, xq, M, nb, (v & 1) ? 2 : 1, v >= 22, st);
        case 1: return launch_ring<FMT_Q4K>(y, W, xq, M, nb, st);
        case 2: return launch_direct_generic<FMT_Q4K>(y, W, xq, M, nb, st);
        case 10: return launch_q4k_direct<32, 1>(y, W, xq, M, nb, st);
        case 11: return launch_q4k_direct<32, 2>(y, W, xq, M, nb, st);
        case 12: return launch_q4k_direct<32, 4>(y, W, xq, M, nb, st);
        case 13: return launch_q4k_direct<16, 2>(y, W, xq, M, nb, st);
        case 14: return launch_q4k_direct<16, 4>(y, W, xq, M, nb, st);
        case 15: return launch_q4k_direct<8, 4>(y, W, xq, M, nb, st);
        case 16: return launch_q4k_direct<4, 4>(y, W, xq, M, nb, st);
        case 17: return launch_q4k_direct<4, 2>(y, W, xq, M, nb, st);
        default: return ckb_fail(CKB_ERR_STATE, "gemv_q4_k_q8_k: unknown variant %d", v);
    }
}

extern "C" int ckb200_dev_gemv_q6_k_q8_k(float *y, const void *W, const void *xq, int M, int K, void *stream)
{
    const int c = check_common("gemv_q6_k_q8_k", y, W, xq, M, K, QK_K);
    if (c) return c == 1 ? 0 : CKB_ERR_SHAPE;
    if (((uintptr_t)W & 1) || ((uintptr_t)xq & 3))
        return ckb_fail(CKB_ERR_ALIGN, "gemv_q6_k_q8_k: W must be 2-byte and x_q8 4-byte aligned");
    const int nb = K / QK_K;
    if (ckb_ensure_init()) return CKB_ERR_NO_DEVICE;
    cudaStream_t st = ckb_stream(stream);
    int v = ckb_tune_get("gemv_q6_k", 0);
    if (v == 0) v = (((uintptr_t)W & 15) || (nb <= 4 && M > 32768)) ? 2 : 1;     // very many short rows: per-tile ring overhead loses
    if (v == 1) return launch_ring<FMT_Q6K>(y, W, xq, M, nb, st);
    return launch_direct_generic<FMT_Q6K>(y, W, xq, M, nb, st);
}

extern "C" int ckb200_dev_gemv_q8_0_q8_0(float *y, const void *W, const void *xq, int M, int K, void *stream)
{
    const int c = check_common("gemv_q8_0_q8_0", y, W, xq, M, K, QK8_0);
    if (c) return c == 1 ? 0 : CKB_ERR_SHAPE;
    if (((uintptr_t)W & 1) || ((uintptr_t)xq & 1))
        return ckb_fail(CKB_ERR_ALIGN, "gemv_q8_0_q8_0: W and x_q8 must be 2-byte aligned");
    const int nb = K / QK8_0;
    if (ckb_ensure_init()) return CKB_ERR_NO_DEVICE;
    cudaStream_t st = ckb_stream(stream);
    int v = ckb_tune_get("gemv_q8_0", 0);
    if (v == 0) v = (((uintptr_t)W & 15) || (nb <= 32 && M > 32768)) ? 2 : 1;
    if (v == 1) return launch_ring<FMT_Q80>(y, W, xq, M, nb, st);
    return launch_direct_generic<FMT_Q80>(y, W, xq, M, nb, st);
}

// gemv_q5_0_q8_0 (src/kernels/gemm_kernels_q5_0.c:1637-1651): Q5_0 weights (22-byte blocks), Q8_0 activations
extern "C" int ckb200_dev_gemv_q5_0_q8_0(float *y, const void *W, const void *xq, int M, int K, void *stream)
{
    const int c = check_common("gemv_q5_0_q8_0", y, W, xq, M, K, QK8_0);
    if (c) return c == 1 ? 0 : CKB_ERR_SHAPE;
    if (((uintptr_t)W & 1) || ((uintptr_t)xq & 1))
        return ckb_fail(CKB_ERR_ALIGN, "gemv_q5_0_q8_0: W and x_q8 must be 2-byte aligned");
    const int nb = K / QK8_0;
    if (ckb_ensure_init()) return CKB_ERR_NO_DEVICE;
    cudaStream_t st = ckb_stream(stream);
    int v = ckb_tune_get("gemv_q5_0", 0);
    if (v == 0) v = (((uintptr_t)W & 15) || (nb <= 32 && M > 32768)) ? 2 : 1;
    if (v == 1) return launch_ring<FMT_Q50>(y, W, xq, M, nb, st);
    return launch_direct_generic<FMT_Q50>(y, W, xq, M, nb, st);
}
