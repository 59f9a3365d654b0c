// Q6_K x Q8_K GEMV over weights kept in HBM in a row-planar layout.
//
// The reference's block_q6_K stream (include/ckernel_quant.h:135-146: ql[128], qh[64], int8 scales[16], fp16 d =
// 210 bytes) is only 2-byte aligned, so no lane can fetch 16 bytes of it with one load.  Weights that stay resident
// on the device are therefore re-laid once, at upload, row by row and without changing a bit of their content:
//
//     row = ql of all nb superblocks (nb * 128 B) | qh (nb * 64 B) | scales (nb * 16 B) | d (nb * 2 B) | pad to 16 B
//
// Every ql / qh / scale piece a lane needs is then a naturally aligned 16-byte (8-byte for the scales) read-only
// load, and a row still costs 210 bytes per superblock of HBM traffic (plus at most 14 bytes of row padding).
//
// The arithmetic is the reference's gemv_q6_k_q8_k (src/kernels/gemm_kernels_q6k_q8k.c:86-116, :197-214) in the
// exact-integer form of the ring kernel: four lanes per superblock, lane (n, h) takes the 64 weights
// ql[64n + 16h ..], ql[64n + 32 + 16h ..], qh[32n + 16h ..] with the four scale groups 8n + h + {0, 2, 4, 6};
// nibble planes and 2-bit planes are multiplied in place by dp4a and recombined with shifts, the -32 offset goes
// through the activation block sums.  Launch structure as the Q4_K kernel: programmatic dependent launch, weights of
// the first pass requested before the dependency wait, activations staged once per CTA after it, software-pipelined
// passes, work items dealt round-robin over the CTAs.
#include "q6p_unit.cuh"
#include "launch.h"
#include "pdl.cuh"
#include "runtime.h"

namespace ckb {

// G lanes per row (4 per superblock), R rows per lane group, NW warps
template <int G, int R, int NW>
__global__ void __launch_bounds__(NW * 32) gemv_q6p_kernel(const uint8_t *__restrict__ W, const uint8_t *__restrict__ xg, float *__restrict__ y, int M, int nb)
{
    extern __shared__ __align__(128) uint8_t smem[];
    constexpr int SPP = G / 4;                 // superblocks per pass of one row
    constexpr int RPW = (32 / G) * R;          // rows per warp item
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int li = lane % G, sub = lane / G, u = li & 3, b0 = li >> 2, n = u >> 1, h = u & 1;
    const int nitems = (M + RPW - 1) / RPW;
    const int item_stride = gridDim.x * NW;
    const int npass = (nb + SPP - 1) / SPP;
    const size_t rb = q6p_row_bytes(nb);
    const size_t off_qh = (size_t)nb * 128, off_sc = (size_t)nb * 192, off_d = (size_t)nb * 208;

    pdl_trigger();

    auto load_item = [&](Q6pW (&w)[R], int item, int pass) {
        const int row0 = item * RPW + sub * R;
        const int b = min(b0 + pass * SPP, nb - 1);
#pragma unroll
        for (int r = 0; r < R; ++r) {
            const uint8_t *row = W + (size_t)min(row0 + r, M - 1) * rb;
            w[r].qa = __ldg(reinterpret_cast<const uint4 *>(row + (size_t)b * 128 + 64 * n + 16 * h));
            w[r].qb = __ldg(reinterpret_cast<const uint4 *>(row + (size_t)b * 128 + 64 * n + 32 + 16 * h));
            w[r].qh = __ldg(reinterpret_cast<const uint4 *>(row + off_qh + (size_t)b * 64 + 32 * n + 16 * h));
            w[r].sc = __ldg(reinterpret_cast<const uint2 *>(row + off_sc + (size_t)b * 16 + 8 * n));
            w[r].d = ldg_nc_u16(row + off_d + (size_t)b * 2);
        }
    };

    Q6pW cur[R], nxt[R];
    int item = blockIdx.x + gridDim.x * warp, pass = 0;
    if (item < nitems) load_item(cur, item, 0);      // weights are never written by a kernel: safe before the wait

    pdl_wait();
    const RingX x = ring_stage_x<FMT_Q6K>(xg, nb, smem);
    __syncthreads();

    float acc[R];
#pragma unroll
    for (int r = 0; r < R; ++r) acc[r] = 0.0f;

    while (item < nitems) {
        int nitem = item, npass_i = pass + 1;
        if (npass_i == npass) { npass_i = 0; nitem = item + item_stride; }
        if (nitem < nitems) load_item(nxt, nitem, npass_i);
        const int b = b0 + pass * SPP;
        if (b < nb) {
#pragma unroll
            for (int r = 0; r < R; ++r) acc[r] += q6p_unit(cur[r], b, u, x);
        }
        if (npass_i == 0) {                          // row finished
            const int row0 = item * RPW + sub * R;
#pragma unroll
            for (int r = 0; r < R; ++r) {
                const float s = group_sum<G>(acc[r]);
                if (li == 0 && row0 + r < M) y[row0 + r] = s;
                acc[r] = 0.0f;
            }
        }
#pragma unroll
        for (int r = 0; r < R; ++r) cur[r] = nxt[r];
        item = nitem;
        pass = npass_i;
    }
}

// ---------------------------------------------------------------- layout conversion (once, at upload)

// src: the reference's rows of nb 210-byte blocks (2-byte aligned); dst: planar rows.  One CTA per row.
__global__ void __launch_bounds__(256) q6k_to_planar_kernel(const uint8_t *__restrict__ src, uint8_t *__restrict__ dst, int nb)
{
    const size_t row = blockIdx.x;
    const unsigned short *s = reinterpret_cast<const unsigned short *>(src + row * (size_t)nb * Q6K_BYTES);
    unsigned short *d = reinterpret_cast<unsigned short *>(dst + row * q6p_row_bytes(nb));
    const int total = nb * (Q6K_BYTES / 2);
    for (int i = threadIdx.x; i < total; i += blockDim.x) {
        const int b = i / 105, o = i - b * 105;      // 2-byte unit o of block b
        int t;
        if (o < 64) t = b * 64 + o;                                  // ql
        else if (o < 96) t = nb * 64 + b * 32 + (o - 64);            // qh
        else if (o < 104) t = nb * 96 + b * 8 + (o - 96);            // scales
        else t = nb * 104 + b;                                       // d
        d[t] = s[i];
    }
    const int pad0 = nb * 105, pad1 = (int)(q6p_row_bytes(nb) / 2);
    for (int i = pad0 + threadIdx.x; i < pad1; i += blockDim.x) d[i] = 0;
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

template <int G, int R>
int launch_q6p(float *y, const void *W, const void *xq, int M, int nb, cudaStream_t st)
{
    constexpr int NW = 8;
    auto kernel = gemv_q6p_kernel<G, R, NW>;
    const int smem = ringx_smem_bytes(FMT_Q6K, nb);
    if (smem > 220 * 1024) return ckb_fail(CKB_ERR_LIMIT, "gemv_q6_k (planar): K too large for the shared activation buffer");
    static int attr_smem = 0, occ_cache_smem = -1, occ_cache = 1;
    if (smem > 48 * 1024 && smem > attr_smem) {
        if (ckb_check_cuda((int)cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem), "smem attr")) return CKB_ERR_CUDA;
        attr_smem = smem;
    }
    if (occ_cache_smem != smem) { occ_cache = occupancy_of(kernel, NW * 32, smem); occ_cache_smem = smem; }
    constexpr int rows_per_cta = NW * (32 / G) * R;
    const int ctas_full = (M + rows_per_cta - 1) / rows_per_cta;
    const int occ_cap = ckb_tune_get("gemv_occ_cap", 0);          // fewer resident CTAs per SM leave room for concurrent launches
    const int sms = ckb_sm_count(), cap = sms * (occ_cap > 0 && occ_cap < occ_cache ? occ_cap : occ_cache);
    int grid = ctas_full < cap ? ctas_full : cap;
    if (ctas_full > sms && grid % sms) {             // a whole number of CTAs per SM, so that the round-robin deal is even
        grid = (grid / sms + 1) * sms;
        if (grid > cap) grid = cap;
    }
    return launch_pdl("gemv_q6k_planar", kernel, dim3(grid), dim3(NW * 32), (size_t)smem, st, (const uint8_t *)W, (const uint8_t *)xq, y, M, nb);
}

}  // namespace

extern "C" size_t ckb200_q6_k_planar_bytes(int rows, int cols) { return cols % QK_K ? 0 : (size_t)rows * q6p_row_bytes(cols / QK_K); }

// dst (16-byte aligned, ckb200_q6_k_planar_bytes) <- the reference's Q6_K rows at src (device memory, 2-byte aligned)
extern "C" int ckb200_dev_q6_k_to_planar(void *dst, const void *src, int rows, int cols, void *stream)
{
    if (!dst || !src || rows <= 0 || cols <= 0) return 0;
    if (cols % QK_K || ((uintptr_t)dst & 15) || ((uintptr_t)src & 1)) return ckb_fail(CKB_ERR_SHAPE, "q6_k_to_planar: K %% 256 or alignment");
    if (ckb_ensure_init()) return CKB_ERR_NO_DEVICE;
    q6k_to_planar_kernel<<<rows, 256, 0, ckb_stream(stream)>>>((const uint8_t *)src, (uint8_t *)dst, cols / QK_K);
    return ckb_check_launch("q6k_to_planar");
}

// y[M] = W . x with W in the planar layout; same result as ckb200_dev_gemv_q6_k_q8_k on the original rows
extern "C" int ckb200_dev_gemv_q6_k_planar_q8_k(float *y, const void *W_planar, const void *x_q8, int M, int K, void *stream)
{
    if (!y || !W_planar || !x_q8 || M <= 0 || K <= 0) return 0;
    if (K % QK_K || ((uintptr_t)W_planar & 15) || ((uintptr_t)x_q8 & 3)) return ckb_fail(CKB_ERR_SHAPE, "gemv_q6_k (planar): K %% 256 or alignment");
    if (ckb_ensure_init()) return CKB_ERR_NO_DEVICE;
    const int nb = K / QK_K;
    cudaStream_t st = ckb_stream(stream);
    const int r = ckb_tune_get("gemv_q6p_rows", 0);
    int g = 4;
    while (g < 32 && g < 4 * nb) g <<= 1;
#define CKB_Q6P(GG) ((r == 1 || (r == 0 && nb <= 4)) ? launch_q6p<GG, 1>(y, W_planar, x_q8, M, nb, st) : launch_q6p<GG, 2>(y, W_planar, x_q8, M, nb, st))
    switch (g) {
        case 4: return CKB_Q6P(4);
        case 8: return CKB_Q6P(8);
        case 16: return CKB_Q6P(16);
        default: return CKB_Q6P(32);
    }
#undef CKB_Q6P
}
