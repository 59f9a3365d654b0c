// Q5_0 x Q8_0 GEMV over weights kept in HBM in a row-planar layout.
//
// block_q5_0 (include/ckernel_quant.h:70-74: fp16 d, 4 bytes of fifth bits, 16 nibble bytes = 22 bytes) is only 2-byte
// aligned.  Resident weights are re-laid once, at upload, without changing a bit:
//
//     row = the nibble bytes of all nb blocks (nb * 16 B) | their fifth bits (nb * 4 B) | d of all blocks (nb * 2 B) | pad to 16 B
//
// so that a lane reads a block with one aligned 16-byte, one 4-byte and one 2-byte load.  Arithmetic as the reference's
// gemv_q5_0_q8_0 / vec_dot_q5_0_q8_0 (src/kernels/gemm_kernels_q5_0.c:901-939, :1637-1651): int32 dot of the 32 products
// of (q5 - 16) and the activation bytes times d_w * d_x, fp32 sum over the blocks.  One lane per block, G lanes per row;
// launch structure as the planar Q8_0 kernel (programmatic dependent launch, weights of the first pass requested before
// the dependency wait, activations staged once per CTA in 48-byte slots, round-robin deal of the work items).
#include "ring_x.cuh"
#include "launch.h"
#include "pdl.cuh"
#include "runtime.h"

namespace ckb {

__host__ __device__ inline size_t q50p_row_bytes(int nb) { return ((size_t)nb * Q50_BYTES + 15) & ~(size_t)15; }

struct Q50pW { uint4 qs; uint32_t qh, d; };

__device__ __forceinline__ float q50p_unit(const Q50pW &w, int b, const RingX &x)
{
    return q50_unit_presum(w.d, w.qh, w.qs, x.q + 48u * b);
}

template <int G, int R, int NW>
__global__ void __launch_bounds__(NW * 32) gemv_q50p_kernel(const uint8_t *__restrict__ W, const uint8_t *__restrict__ xg, float *__restrict__ y, int M, int nb)
{
    extern __shared__ __align__(128) uint8_t smem[];
    constexpr int RPW = (32 / G) * R;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int li = lane % G, sub = lane / G;
    const int nitems = (M + RPW - 1) / RPW, item_stride = gridDim.x * NW;
    const int npass = (nb + G - 1) / G;
    const size_t rb = q50p_row_bytes(nb), off_qh = (size_t)nb * 16, off_d = (size_t)nb * 20;

    pdl_trigger();

    auto load_item = [&](Q50pW (&w)[R], int item, int pass) {
        const int row0 = item * RPW + sub * R;
        const int b = min(li + pass * G, nb - 1);
#pragma unroll
        for (int r = 0; r < R; ++r) {
            const uint8_t *row = W + (size_t)min(row0 + r, M - 1) * rb;
            w[r].qs = __ldg(reinterpret_cast<const uint4 *>(row + (size_t)b * 16));
            w[r].qh = __ldg(reinterpret_cast<const uint32_t *>(row + off_qh + (size_t)b * 4));
            w[r].d = ldg_nc_u16(row + off_d + (size_t)b * 2);
        }
    };

    Q50pW cur[R], nxt[R];
    int item = blockIdx.x + gridDim.x * warp, pass = 0;
    if (item < nitems) load_item(cur, item, 0);

    pdl_wait();
    const RingX x = ring_stage_x<FMT_Q80>(xg, nb, smem);
    __syncthreads();
    q50_store_xsums(x.q, nb);
    __syncthreads();

    float acc[R];
#pragma unroll
    for (int r = 0; r < R; ++r) acc[r] = 0.0f;

    while (item < nitems) {
        int nitem = item, npass_i = pass + 1;
        if (npass_i == npass) { npass_i = 0; nitem = item + item_stride; }
        if (nitem < nitems) load_item(nxt, nitem, npass_i);
        const int b = li + pass * G;
        if (b < nb) {
#pragma unroll
            for (int r = 0; r < R; ++r) acc[r] += q50p_unit(cur[r], b, x);
        }
        if (npass_i == 0) {
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

// src: the reference's rows of nb 22-byte blocks; dst: planar rows.  One CTA per row, 2-byte units (11 per block:
// d, 2 of fifth bits, 8 of nibbles).
__global__ void __launch_bounds__(256) q50_to_planar_kernel(const uint8_t *__restrict__ src, uint8_t *__restrict__ dst, int nb)
{
    const size_t row = blockIdx.x;
    const unsigned short *s = reinterpret_cast<const unsigned short *>(src + row * (size_t)nb * Q50_BYTES);
    unsigned short *d = reinterpret_cast<unsigned short *>(dst + row * q50p_row_bytes(nb));
    const int total = nb * 11;
    for (int i = threadIdx.x; i < total; i += blockDim.x) {
        const int b = i / 11, o = i - b * 11;
        const int to = o == 0 ? nb * 10 + b : (o < 3 ? nb * 8 + 2 * b + (o - 1) : b * 8 + (o - 3));
        d[to] = s[i];
    }
    const int pad0 = nb * 11, pad1 = (int)(q50p_row_bytes(nb) / 2);
    for (int i = pad0 + threadIdx.x; i < pad1; i += blockDim.x) d[i] = 0;
}

}  // namespace ckb

using namespace ckb;

namespace {

template <int G, int R>
int launch_q50p(float *y, const void *W, const void *xq, int M, int nb, cudaStream_t st)
{
    constexpr int NW = 8;
    auto kernel = gemv_q50p_kernel<G, R, NW>;
    const int smem = ringx_smem_bytes(FMT_Q80, nb);
    if (smem > 220 * 1024) return ckb_fail(CKB_ERR_LIMIT, "gemv_q5_0 (planar): K too large for the shared activation buffer");
    static int attr_smem = 0, occ_cache_smem = -1, occ_cache = 1;
    if (smem > 48 * 1024 && smem > attr_smem) {
        if (ckb_check_cuda((int)cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem), "smem attr")) return CKB_ERR_CUDA;
        attr_smem = smem;
    }
    if (occ_cache_smem != smem) {
        int occ = 0;
        if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&occ, kernel, NW * 32, smem) != cudaSuccess) { cudaGetLastError(); occ = 1; }
        occ_cache = occ < 1 ? 1 : occ;
        occ_cache_smem = smem;
    }
    constexpr int rows_per_cta = NW * (32 / G) * R;
    const int ctas_full = (M + rows_per_cta - 1) / rows_per_cta;
    const int occ_cap = ckb_tune_get("gemv_occ_cap", 0);          // fewer resident CTAs per SM leave room for concurrent launches
    const int sms = ckb_sm_count(), cap = sms * (occ_cap > 0 && occ_cap < occ_cache ? occ_cap : occ_cache);
    int grid = ctas_full < cap ? ctas_full : cap;
    if (ctas_full > sms && grid % sms) {
        grid = (grid / sms + 1) * sms;
        if (grid > cap) grid = cap;
    }
    return launch_pdl("gemv_q50_planar", kernel, dim3(grid), dim3(NW * 32), (size_t)smem, st, (const uint8_t *)W, (const uint8_t *)xq, y, M, nb);
}

}  // namespace

extern "C" size_t ckb200_q5_0_planar_bytes(int rows, int cols) { return cols % 32 ? 0 : (size_t)rows * q50p_row_bytes(cols / 32); }

extern "C" int ckb200_dev_q5_0_to_planar(void *dst, const void *src, int rows, int cols, void *stream)
{
    if (!dst || !src || rows <= 0 || cols <= 0) return 0;
    if (cols % 32 || ((uintptr_t)dst & 15) || ((uintptr_t)src & 1)) return ckb_fail(CKB_ERR_SHAPE, "q5_0_to_planar: K %% 32 or alignment");
    if (ckb_ensure_init()) return CKB_ERR_NO_DEVICE;
    q50_to_planar_kernel<<<rows, 256, 0, ckb_stream(stream)>>>((const uint8_t *)src, (uint8_t *)dst, cols / 32);
    return ckb_check_launch("q50_to_planar");
}

extern "C" int ckb200_dev_gemv_q5_0_planar_q8_0(float *y, const void *W_planar, const void *x_q8, int M, int K, void *stream)
{
    if (!y || !W_planar || !x_q8 || M <= 0 || K <= 0) return 0;
    if (K % 32 || ((uintptr_t)W_planar & 15) || ((uintptr_t)x_q8 & 1)) return ckb_fail(CKB_ERR_SHAPE, "gemv_q5_0 (planar): K %% 32 or alignment");
    if (ckb_ensure_init()) return CKB_ERR_NO_DEVICE;
    const int nb = K / 32;
    cudaStream_t st = ckb_stream(stream);
    int g = 1;
    while (g < 32 && g < nb) g <<= 1;
    switch (g) {
        case 1: return launch_q50p<1, 2>(y, W_planar, x_q8, M, nb, st);
        case 2: return launch_q50p<2, 2>(y, W_planar, x_q8, M, nb, st);
        case 4: return launch_q50p<4, 2>(y, W_planar, x_q8, M, nb, st);
        case 8: return launch_q50p<8, 2>(y, W_planar, x_q8, M, nb, st);
        case 16: return launch_q50p<16, 2>(y, W_planar, x_q8, M, nb, st);
        default: return launch_q50p<32, 2>(y, W_planar, x_q8, M, nb, st);
    }
}
