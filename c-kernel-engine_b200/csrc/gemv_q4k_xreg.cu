// Q4_K x Q8_K GEMV with the activations held in registers.
//
// Same work split as gemv_q4k.cu (two lanes per superblock; lane p takes quarters p and p+2), but
// every warp is bound to ONE pass over the row (a fixed set of 16 superblocks), so the 64 activation
// bytes, the Q8_K scale and the four sub-block sums a lane needs never change: they are loaded once
// (through one shared-memory copy per CTA) into registers and the inner loop touches no shared memory at all.  A row
// longer than one pass is split over `npass` warps of the CTA; their partial sums meet in a small
// shared tile that is summed in a fixed order (deterministic) once per row tile.
//
// Reference semantics: gemv_q4_k_q8_k, src/kernels/gemm_kernels_q4k_q8k.c:121-200.
#include "quant_units.cuh"
#include "launch.h"
#include "runtime.h"

namespace ckb {

struct XrW { uint4 hdr, a0, a1, b0, b1; };

struct XrX {                 // one lane's activations: quarter p and quarter p+2 of superblock b
    uint4 al0, al1, ah0, ah1, bl0, bl1, bh0, bh1;
    float d;
    uint32_t lo4, hi4;       // sub-block sums {2p, 2p+1, 2p+4, 2p+5} split as 128*hi + lo, 4 x s8 each
};

// The activation vector was written by the previous kernel, which may overlap this one under programmatic
// launch, so it must come through L2 (__ldcg), never the non-coherent read-only path.  Letting every lane of
// every CTA fetch its slice from L2 hammers the few L2 lines that hold the vector, so the CTA copies the
// raw blocks into shared memory once (one L2 read per word per CTA) and lanes pick their slice from there.
__device__ __forceinline__ void xr_stage_raw(const uint8_t *xg, int nb, uint32_t *raw)
{
    const uint32_t *src = reinterpret_cast<const uint32_t *>(xg);
    const int total = nb * 73;
    for (int base = 0; base < total; base += 8 * blockDim.x) {
        uint32_t v[8];
#pragma unroll
        for (int u = 0; u < 8; ++u) {
            const int i = base + u * blockDim.x + threadIdx.x;
            v[u] = i < total ? __ldcg(src + i) : 0u;
        }
#pragma unroll
        for (int u = 0; u < 8; ++u) {
            const int i = base + u * blockDim.x + threadIdx.x;
            if (i < total) raw[i] = v[u];
        }
    }
}
__device__ __forceinline__ uint4 ldg4w(const uint32_t *p) { return make_uint4(p[0], p[1], p[2], p[3]); }

__device__ __forceinline__ XrX xr_load_x(const uint32_t *raw, int b, int p)
{
    XrX x;
    const uint32_t *blk = raw + b * 73;                              // block b of the staged vector (73 words each)
    const uint32_t *qa = blk + 1 + 16 * p, *qb = blk + 1 + 16 * (p + 2);
    x.al0 = ldg4w(qa); x.al1 = ldg4w(qa + 4); x.ah0 = ldg4w(qa + 8); x.ah1 = ldg4w(qa + 12);
    x.bl0 = ldg4w(qb); x.bl1 = ldg4w(qb + 4); x.bh0 = ldg4w(qb + 8); x.bh1 = ldg4w(qb + 12);
    x.d = __uint_as_float(blk[0]);
    uint32_t lo = 0, hi = 0;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int j = 2 * p + (i & 1) + 4 * (i >> 1);                // sub-block of byte i
        const uint32_t v = blk[65 + j];
        const int s = (int)(short)(v & 0xffffu) + (int)(short)(v >> 16);
        lo |= (uint32_t)(s & 127) << (8 * i);
        hi |= (uint32_t)((s >> 7) & 255) << (8 * i);
    }
    x.lo4 = lo;
    x.hi4 = hi;
    return x;
}

__device__ __forceinline__ void xr_dots(const uint4 &w0, const uint4 &w1, const uint4 &l0, const uint4 &l1, const uint4 &h0,
                                        const uint4 &h1, int &s_lo, int &s_hi16)
{
    const uint32_t ml = 0x0F0F0F0Fu, mh = 0xF0F0F0F0u;
    int lo = 0, hi = 0;
    lo = dp4a_us(w0.x & ml, l0.x, lo); hi = dp4a_us(w0.x & mh, h0.x, hi);
    lo = dp4a_us(w0.y & ml, l0.y, lo); hi = dp4a_us(w0.y & mh, h0.y, hi);
    lo = dp4a_us(w0.z & ml, l0.z, lo); hi = dp4a_us(w0.z & mh, h0.z, hi);
    lo = dp4a_us(w0.w & ml, l0.w, lo); hi = dp4a_us(w0.w & mh, h0.w, hi);
    lo = dp4a_us(w1.x & ml, l1.x, lo); hi = dp4a_us(w1.x & mh, h1.x, hi);
    lo = dp4a_us(w1.y & ml, l1.y, lo); hi = dp4a_us(w1.y & mh, h1.y, hi);
    lo = dp4a_us(w1.z & ml, l1.z, lo); hi = dp4a_us(w1.z & mh, h1.z, hi);
    lo = dp4a_us(w1.w & ml, l1.w, lo); hi = dp4a_us(w1.w & mh, h1.w, hi);
    s_lo = lo;
    s_hi16 = hi;
}

__device__ __forceinline__ float xr_unit(const XrW &w, const XrX &x, int p)
{
    int a_lo, a_hi16, b_lo, b_hi16;
    xr_dots(w.a0, w.a1, x.al0, x.al1, x.ah0, x.ah1, a_lo, a_hi16);
    xr_dots(w.b0, w.b1, x.bl0, x.bl1, x.bh0, x.bh1, b_lo, b_hi16);
    const int t = 16 * p;
    const uint32_t a = w.hdr.y >> t, bb = w.hdr.z >> t, c = w.hdr.w >> t;
    const uint32_t scA = a & 0x3F3Fu, mA = bb & 0x3F3Fu;
    const uint32_t scB = (c & 0x0F0Fu) | ((a >> 2) & 0x3030u);
    const uint32_t mB = ((c >> 4) & 0x0F0Fu) | ((bb >> 2) & 0x3030u);
    const int isum = (int)(scA & 255u) * a_lo + (int)(scB & 255u) * b_lo +
                     (((int)(scA >> 8) * a_hi16 + (int)(scB >> 8) * b_hi16) >> 4);
    const uint32_t m4 = mA | (mB << 16);
    const int imin = dp4a_us(m4, x.lo4, 0) + 128 * dp4a_us(m4, x.hi4, 0);
    const float2 dd = __half22float2(*reinterpret_cast<const __half2 *>(&w.hdr.x));
    return (dd.x * x.d) * (float)isum - (dd.y * x.d) * (float)imin;
}

// G lanes per row pass (SPP = G/2 superblocks), R rows per lane group, T row groups per warp per tile.
// blockDim = npass * kw warps: warp w -> pass w % npass, row slot w / npass.
template <int G, int R, bool L1ALLOC>
__global__ void __launch_bounds__(256) gemv_q4k_xreg_kernel(const uint8_t *__restrict__ W, const uint8_t *__restrict__ xg,
                                                            float *__restrict__ y, int M, int nb, int npass, int kw, int T)
{
    constexpr int SPP = G / 2, RPW = (32 / G) * R;
    __shared__ float part[8][128];                                   // [pass][row in tile], used only when npass > 1
    extern __shared__ __align__(16) uint32_t xraw[];                 // nb * 73 words: the Q8_K vector as stored
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int li = lane % G, sub = lane / G, p = li & 1;
    const int pw = warp % npass, wr = warp / npass;
    const int b_raw = (li >> 1) + pw * SPP;
    const bool live = b_raw < nb;
    const int b = live ? b_raw : nb - 1;
    const int tile_rows = kw * RPW * T;
    const int ntiles = (M + tile_rows - 1) / tile_rows;
    const size_t rb = (size_t)nb * Q4K_BYTES;
    const uint8_t *Wb = W + (size_t)b * Q4K_BYTES + 32 * p;

    asm volatile("griddepcontrol.launch_dependents;");

    auto ld = [&](const uint8_t *q) -> uint4 {
        if constexpr (L1ALLOC) return __ldg(reinterpret_cast<const uint4 *>(q));
        else return ldg_stream_u4(q);
    };
    // item (tile, it): rows tile*tile_rows + (it*kw + wr)*RPW + sub*R + r
    auto load_item = [&](XrW (&w)[R], int tile, int it) {
        const int row0 = tile * tile_rows + (it * kw + wr) * RPW + sub * R;
#pragma unroll
        for (int r = 0; r < R; ++r) {
            const uint8_t *pb = Wb + (size_t)min(row0 + r, M - 1) * rb;
            w[r].hdr = ld(pb - 32 * p);
            w[r].a0 = ld(pb + 16);
            w[r].a1 = ld(pb + 32);
            w[r].b0 = ld(pb + 80);
            w[r].b1 = ld(pb + 96);
        }
    };

    XrW cur[R], nxt[R];
    int tile = blockIdx.x, it = 0;
    if (tile < ntiles) load_item(cur, tile, 0);          // weights are immutable: prefetch before the dependency wait

    asm volatile("griddepcontrol.wait;" ::: "memory");
    xr_stage_raw(xg, nb, xraw);
    __syncthreads();
    const XrX x = xr_load_x(xraw, b, p);

    while (tile < ntiles) {
        int ntile = tile, nit = it + 1;
        if (nit == T) { nit = 0; ntile = tile + gridDim.x; }
        if (ntile < ntiles) load_item(nxt, ntile, nit);
        const int lrow0 = (it * kw + wr) * RPW + sub * R;            // row inside the tile
#pragma unroll
        for (int r = 0; r < R; ++r) {
            float v = live ? xr_unit(cur[r], x, p) : 0.0f;
            v = group_sum<G>(v);
            if (li == 0) {
                if (npass == 1) {
                    const int row = tile * tile_rows + lrow0 + r;
                    if (row < M) y[row] = v;
                } else {
                    part[pw][lrow0 + r] = v;
                }
            }
        }
        if (npass > 1 && nit == 0) {                                 // tile finished: fixed-order sum over the passes
            __syncthreads();
            for (int i = threadIdx.x; i < tile_rows; i += blockDim.x) {
                const int row = tile * tile_rows + i;
                if (row < M) {
                    float s = part[0][i];
                    for (int q = 1; q < npass; ++q) s += part[q][i];
                    y[row] = s;
                }
            }
            __syncthreads();
        }
#pragma unroll
        for (int r = 0; r < R; ++r) cur[r] = nxt[r];
        tile = ntile;
        it = nit;
    }
}

}  // namespace ckb

using namespace ckb;

namespace {

template <int G, int R, bool L1A>
int launch_xreg(float *y, const void *W, const void *xq, int M, int nb, cudaStream_t st)
{
    constexpr int SPP = G / 2, RPW = (32 / G) * R;
    const int npass = (nb + SPP - 1) / SPP;
    if (npass > 8) return -1;                                        // caller falls back
    const int kw = 8 / npass;                                        // warps per pass
    const int nwarps = kw * npass;
    auto kernel = gemv_q4k_xreg_kernel<G, R, L1A>;
    static int occ = 0;
    if (!occ) {
        if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&occ, kernel, 256, 16 * 1024) != cudaSuccess || occ < 1) { cudaGetLastError(); occ = 1; }
    }
    const int cap = ckb_sm_count() * occ;
    // rows per tile: at most 128 (the shared partial-sum tile), but small enough that every CTA slot gets a tile
    int T = 128 / (kw * RPW);
    const int t_fill = M / (kw * RPW * cap * 4);                     // at least ~4 tiles per resident CTA when M allows
    if (T > t_fill) T = t_fill;
    if (T < 1) T = 1;
    const int tile_rows = kw * RPW * T;
    const int ntiles = (M + tile_rows - 1) / tile_rows;
    const int grid = ntiles < cap ? ntiles : cap;

    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(grid);
    cfg.blockDim = dim3(nwarps * 32);
    cfg.dynamicSmemBytes = (size_t)nb * Q8K_BYTES;                   // <= 128 * 292 B
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = ckb_tune_get("pdl", 1) ? 1 : 0;
    const uint8_t *Wp = (const uint8_t *)W, *xp = (const uint8_t *)xq;
    if (ckb_check_cuda((int)cudaLaunchKernelEx(&cfg, kernel, Wp, xp, y, M, nb, npass, kw, T), "gemv_q4k_xreg launch")) return CKB_ERR_CUDA;
    return ckb_check_launch("gemv_q4k_xreg");
}

template <int R, bool L1A>
int pick_g(float *y, const void *W, const void *xq, int M, int nb, cudaStream_t st)
{
    int g = 2;
    while (g < 32 && g < 2 * nb) g <<= 1;
    switch (g) {
        case 2: return launch_xreg<2, R, L1A>(y, W, xq, M, nb, st);
        case 4: return launch_xreg<4, R, L1A>(y, W, xq, M, nb, st);
        case 8: return launch_xreg<8, R, L1A>(y, W, xq, M, nb, st);
        case 16: return launch_xreg<16, R, L1A>(y, W, xq, M, nb, st);
        default: return launch_xreg<32, R, L1A>(y, W, xq, M, nb, st);
    }
}

}  // namespace

// Returns -1 when the row is too long for this kernel (more than 8 passes of 16 superblocks, K > 32768).
extern "C" int ckb_launch_gemv_q4k_xreg(float *y, const void *W, const void *xq, int M, int nb, int r, int l1alloc, void *stream)
{
    cudaStream_t st = (cudaStream_t)stream;
    if (r == 2) return l1alloc ? pick_g<2, true>(y, W, xq, M, nb, st) : pick_g<2, false>(y, W, xq, M, nb, st);
    return l1alloc ? pick_g<1, true>(y, W, xq, M, nb, st) : pick_g<1, false>(y, W, xq, M, nb, st);
}
