// Q4_K x Q8_K GEMV, tuned kernel: y[M] = W[M, K/256 superblocks of 144 B] . x_q8
// (reference: gemv_q4_k_q8_k and its *_parallel_simd row split, src/kernels/gemm_kernels_q4k_q8k.c:183-263,
// src/kernels/gemm_kernels_q4k_avx.c:136-245).
//
// Work split: two lanes per superblock.  Lane p (0/1) of a superblock takes the nibble bytes of
// quarters p and p+2, i.e. sub-blocks 2p, 2p+1 (6-bit scales stored directly) and 2p+4, 2p+5 (scales
// split over two bytes), so each lane decodes both scale encodings exactly once, without a select.
// All loads are 16-byte read-only loads straight from global memory (superblocks are 16-byte aligned);
// the loop is software pipelined (loads of the next superblock pass are in flight while the current
// one is multiplied), and the first pass is issued before the activation vector is staged, so the
// weight stream never waits for anything but HBM.
//
// The kernel is launched with programmatic dependent launch: it lets the next kernel in the stream
// start immediately (griddepcontrol.launch_dependents), prefetches weights (which no kernel ever
// writes), and only then waits for the previous kernel (griddepcontrol.wait) before it touches the
// activations or writes y.  Back-to-back GEMVs therefore overlap their ramp-up and tail.
#include "quant_units.cuh"
#include "launch.h"
#include "runtime.h"

namespace ckb {

// shared-memory layout of the activations for this kernel:
//   q8 data: 17 slots of 16 B per superblock (16 data + 1 pad: 8 consecutive lanes then hit 8 distinct bank groups)
//   d[nb] fp32
//   per (superblock, p): the four 32-element sums of sub-blocks {2p, 2p+1, 2p+4, 2p+5}, split as
//   sum = 128 * hi + lo with lo in [0, 127] and hi in [-32, 31], packed as 4 x s8 (lo word, hi word),
//   so that sum_j m_j * bsum_j is two dp4a
constexpr int Q4P_SLOTS = 17;
__host__ __device__ inline int q4p_smem_bytes(int nb) { return ((nb * (Q4P_SLOTS * 16 + 4 + 16)) + 127) & ~127; }

struct Q4pX { uint32_t q, d, lo, hi; };

__device__ __forceinline__ Q4pX q4p_stage_x(const uint8_t *xg, int nb, uint8_t *smem)
{
    uint32_t *xq = reinterpret_cast<uint32_t *>(smem);
    float *xd = reinterpret_cast<float *>(smem + nb * Q4P_SLOTS * 16);
    int8_t *lo = reinterpret_cast<int8_t *>(smem + nb * (Q4P_SLOTS * 16 + 4));
    int8_t *hi = lo + nb * 8;
    const uint32_t *src = reinterpret_cast<const uint32_t *>(xg);
    // eight independent loads per thread are issued before the first one is used: the staging costs about
    // one L2 round trip, which matters because it sits between the dependency wait and the first multiply
    const int total = nb * 73;
    for (int base = 0; base < total; base += 8 * blockDim.x) {
        uint32_t v[8];
#pragma unroll
        for (int u = 0; u < 8; ++u) {
            const int i = base + u * blockDim.x + threadIdx.x;
            v[u] = i < total ? __ldcg(src + i) : 0u;       // through L2: the producer may overlap this kernel (programmatic launch)
        }
#pragma unroll
        for (int u = 0; u < 8; ++u) {
            const int i = base + u * blockDim.x + threadIdx.x;
            if (i >= total) break;
            const int b = i / 73, w = i - b * 73;
            if (w == 0) {
                xd[b] = __uint_as_float(v[u]);
            } else if (w <= 64) {
                xq[b * Q4P_SLOTS * 4 + (w - 1)] = v[u];
            } else {
                const int j = w - 65;                                  // 32-element sub-block
                const int sum = (int)(short)(v[u] & 0xffffu) + (int)(short)(v[u] >> 16);
                const int p = (j >> 1) & 1, byte = (j & 1) | ((j >> 2) << 1);
                lo[(b * 2 + p) * 4 + byte] = (int8_t)(sum & 127);
                hi[(b * 2 + p) * 4 + byte] = (int8_t)(sum >> 7);
            }
        }
    }
    Q4pX r;
    r.q = smem_u32(xq);
    r.d = smem_u32(xd);
    r.lo = smem_u32(lo);
    r.hi = smem_u32(hi);
    return r;
}

struct Q4pW { uint4 hdr, a0, a1, b0, b1; };     // header, quarter p (32 B), quarter p+2 (32 B)

__device__ __forceinline__ void q4p_nibble_dots(const uint4 &w0, const uint4 &w1, uint32_t xa, int &s_lo, int &s_hi16)
{
    // xa: shared address of the 64 activations of this quarter (32 for the low nibbles, then 32 for the high ones)
    const uint4 l0 = lds_u4(xa), l1 = lds_u4(xa + 16), h0 = lds_u4(xa + 32), h1 = lds_u4(xa + 48);
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
    s_hi16 = hi;          // 16 x the high-nibble sum (the nibbles were left in place)
}

// contribution of (superblock b, lane half p) of one row
__device__ __forceinline__ float q4p_unit(const Q4pW &w, const Q4pX &x, int b, int p)
{
    const uint32_t xa = x.q + (uint32_t)(b * Q4P_SLOTS + 4 * p) * 16u;
    int a_lo, a_hi16, b_lo, b_hi16;
    q4p_nibble_dots(w.a0, w.a1, xa, a_lo, a_hi16);             // sub-blocks 2p, 2p+1
    q4p_nibble_dots(w.b0, w.b1, xa + 128, b_lo, b_hi16);       // sub-blocks 2p+4, 2p+5
    const int t = 16 * p;
    const uint32_t a = w.hdr.y >> t, bb = w.hdr.z >> t, c = w.hdr.w >> t;
    const uint32_t scA = a & 0x3F3Fu, mA = bb & 0x3F3Fu;                               // include/ckernel_quant.h:230-238
    const uint32_t scB = (c & 0x0F0Fu) | ((a >> 2) & 0x3030u);                         // :242-245
    const uint32_t mB = ((c >> 4) & 0x0F0Fu) | ((bb >> 2) & 0x3030u);                  // :247-250
    const int isum = (int)(scA & 255u) * a_lo + (int)(scB & 255u) * b_lo +
                     (((int)(scA >> 8) * a_hi16 + (int)(scB >> 8) * b_hi16) >> 4);   // exact: both terms are multiples of 16
    const uint32_t m4 = mA | (mB << 16);
    const uint32_t blo = lds_u32(x.lo + 4u * (2 * b + p)), bhi = lds_u32(x.hi + 4u * (2 * b + p));
    const int imin = dp4a_us(m4, blo, 0) + 128 * dp4a_us(m4, bhi, 0);
    const float xd = __uint_as_float(lds_u32(x.d + 4u * b));
    const float2 dd = __half22float2(*reinterpret_cast<const __half2 *>(&w.hdr.x));
    return (dd.x * xd) * (float)isum - (dd.y * xd) * (float)imin;
}

template <int G, int R, int NW, bool L1A>
__global__ void __launch_bounds__(NW * 32) gemv_q4k_pair_kernel(const uint8_t *__restrict__ W, const uint8_t *__restrict__ xg,
                                                                float *__restrict__ y, int M, int nb)
{
    extern __shared__ __align__(128) uint8_t smem[];
    constexpr int SPP = G / 2;                 // superblocks per pass of one row
    constexpr int RPW = (32 / G) * R;          // rows per warp
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int li = lane % G, sub = lane / G, p = li & 1, b0 = li >> 1;
    // Work item = the RPW rows one warp reduces.  Item j belongs to CTA j % grid, warp slot j / grid, so the items are
    // dealt round-robin over the CTAs (and with them over the SMs) instead of in blocks of NW: no SM ends up with a
    // whole CTA more than its neighbour.
    const int ntiles = (M + RPW - 1) / RPW;
    const int tile_stride = gridDim.x * NW;
    const int npass = (nb + SPP - 1) / SPP;
    const size_t rb = (size_t)nb * Q4K_BYTES;

    asm volatile("griddepcontrol.launch_dependents;");

    auto ld = [&](const uint8_t *q) -> uint4 {
        if constexpr (L1A) return __ldg(reinterpret_cast<const uint4 *>(q));
        else return ldg_stream_u4(q);
    };
    auto load_item = [&](Q4pW (&w)[R], int tile, int pass) {
        const int row0 = tile * RPW + sub * R;
        const int b = min(b0 + pass * SPP, nb - 1);
#pragma unroll
        for (int r = 0; r < R; ++r) {
            const uint8_t *pb = W + (size_t)min(row0 + r, M - 1) * rb + (size_t)b * Q4K_BYTES;
            w[r].hdr = ld(pb);
            w[r].a0 = ld(pb + 16 + 32 * p);
            w[r].a1 = ld(pb + 32 + 32 * p);
            w[r].b0 = ld(pb + 80 + 32 * p);
            w[r].b1 = ld(pb + 96 + 32 * p);
        }
    };

    Q4pW cur[R], nxt[R];
    int tile = blockIdx.x + gridDim.x * warp, pass = 0;
    if (tile < ntiles) load_item(cur, tile, 0);     // weights are never written by a kernel: safe before the wait

    asm volatile("griddepcontrol.wait;" ::: "memory");
    const Q4pX x = q4p_stage_x(xg, nb, smem);
    __syncthreads();

    float acc[R];
#pragma unroll
    for (int r = 0; r < R; ++r) acc[r] = 0.0f;

    while (tile < ntiles) {
        int ntile = tile, npass_i = pass + 1;
        if (npass_i == npass) { npass_i = 0; ntile = tile + tile_stride; }
        if (ntile < ntiles) load_item(nxt, ntile, npass_i);
        const int b = b0 + pass * SPP;
        if (b < nb) {
#pragma unroll
            for (int r = 0; r < R; ++r) acc[r] += q4p_unit(cur[r], x, b, p);
        }
        if (npass_i == 0) {                          // row finished
            const int row0 = tile * RPW + sub * R;
#pragma unroll
            for (int r = 0; r < R; ++r) {
                const float s = group_sum<G>(acc[r]);
                if (li == 0 && row0 + r < M) y[row0 + r] = s;
                acc[r] = 0.0f;
            }
        }
#pragma unroll
        for (int r = 0; r < R; ++r) cur[r] = nxt[r];
        tile = ntile;
        pass = npass_i;
    }
}

}  // namespace ckb

using namespace ckb;

namespace {

template <typename K>
int occupancy_of(K kernel, int threads, int smem)
{
    int occ = 0;
    if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&occ, kernel, threads, smem) != cudaSuccess) { cudaGetLastError(); occ = 1; }
    return occ < 1 ? 1 : occ;
}

template <int G, int R, bool L1A>
int launch_pair(float *y, const void *W, const void *xq, int M, int nb, cudaStream_t st)
{
    constexpr int NW = 8;
    auto kernel = gemv_q4k_pair_kernel<G, R, NW, L1A>;
    const int smem = q4p_smem_bytes(nb);
    if (smem > 220 * 1024) return ckb_fail(CKB_ERR_LIMIT, "gemv_q4_k_q8_k: K too large for the shared activation buffer");
    static int attr_smem = 0, occ_cache_smem = -1, occ_cache = 1;
    if (smem > 48 * 1024 && smem > attr_smem) {
        if (ckb_check_cuda((int)cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem), "smem attr")) return CKB_ERR_CUDA;
        attr_smem = smem;
    }
    if (occ_cache_smem != smem) { occ_cache = occupancy_of(kernel, NW * 32, smem); occ_cache_smem = smem; }
    constexpr int rows_per_cta = NW * (32 / G) * R;
    const int ntiles = (M + rows_per_cta - 1) / rows_per_cta;    // CTAs needed if every warp took exactly one item
    const int occ_cap = ckb_tune_get("gemv_occ_cap", 0);          // fewer resident CTAs per SM leave room for concurrent launches
    const int cap = ckb_sm_count() * (occ_cap > 0 && occ_cap < occ_cache ? occ_cap : occ_cache);
    int grid = ntiles < cap ? ntiles : cap;
    if (ntiles > ckb_sm_count() && grid % ckb_sm_count()) {       // a whole number of CTAs per SM, so that the round-robin deal is even
        grid = (grid / ckb_sm_count() + 1) * ckb_sm_count();
        if (grid > cap) grid = cap;
    }

    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(grid);
    cfg.blockDim = dim3(NW * 32);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = ckb_tune_get("pdl", 1) ? 1 : 0;
    const uint8_t *Wp = (const uint8_t *)W, *xp = (const uint8_t *)xq;
    if (ckb_check_cuda((int)cudaLaunchKernelEx(&cfg, kernel, Wp, xp, y, M, nb), "gemv_q4k_pair launch")) return CKB_ERR_CUDA;
    return ckb_check_launch("gemv_q4k_pair");
}

}  // namespace

// r = rows sharing one activation fetch (1 or 2); lanes per row follow from K
extern "C" int ckb_launch_gemv_q4k_pair(float *y, const void *W, const void *xq, int M, int nb, int r, int l1alloc, void *stream)
{
    cudaStream_t st = (cudaStream_t)stream;
    int g = 2;
    while (g < 32 && g < 2 * nb) g <<= 1;
#define CKB_PAIR(GG) (l1alloc ? (r == 2 ? launch_pair<GG, 2, true>(y, W, xq, M, nb, st) : launch_pair<GG, 1, true>(y, W, xq, M, nb, st)) \
                             : (r == 2 ? launch_pair<GG, 2, false>(y, W, xq, M, nb, st) : launch_pair<GG, 1, false>(y, W, xq, M, nb, st)))
    switch (g) {
        case 2: return CKB_PAIR(2);
        case 4: return CKB_PAIR(4);
        case 8: return CKB_PAIR(8);
        case 16: return CKB_PAIR(16);
        default: return CKB_PAIR(32);
    }
#undef CKB_PAIR
}
