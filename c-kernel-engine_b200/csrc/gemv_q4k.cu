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
#include "q4p_unit.cuh"
#include "launch.h"
#include "runtime.h"

namespace ckb {

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
