// Q8_0 x Q8_0 GEMV over weights kept in HBM in a row-planar layout.
//
// block_q8_0 (include/ckernel_quant.h:104-110: fp16 d, 32 int8 = 34 bytes) is only 2-byte aligned, like block_q6_K.
// Resident weights are re-laid once, at upload, without changing a bit:
//
//     row = the 32 quants of all nb blocks (nb * 32 B) | d of all blocks (nb * 2 B) | pad to 16 B
//
// so that a lane reads a block's quants with two aligned 16-byte loads.  Arithmetic as the reference's
// gemv_q8_0_q8_0 / vec_dot_q8_0_q8_0 (src/kernels/gemm_kernels_q8_0.c:1237-1251): int32 dot of the 32 products
// times d_w * d_x, fp32 sum over the blocks.  One lane per block, G lanes per row; launch structure as the planar
// Q6_K kernel (programmatic dependent launch, weights of the first pass requested before the dependency wait,
// activations staged once per CTA in 48-byte slots, round-robin deal of the work items).
#include "ring_x.cuh"
#include "launch.h"
#include "pdl.cuh"
#include "runtime.h"

namespace ckb {

__host__ __device__ inline size_t q80p_row_bytes(int nb) { return ((size_t)nb * Q80_BYTES + 15) & ~(size_t)15; }

struct Q80pW { uint4 w0, w1; uint32_t d; };

__device__ __forceinline__ float q80p_unit(const Q80pW &w, int b, const RingX &x)
{
    const uint32_t xa = x.q + 48u * b;
    const uint4 x0 = lds_u4(xa), x1 = lds_u4(xa + 16);
    const float xd = __uint_as_float(lds_u32(xa + 32));
    int s = 0;
    s = dp4a_ss(w.w0.x, x0.x, s); s = dp4a_ss(w.w0.y, x0.y, s); s = dp4a_ss(w.w0.z, x0.z, s); s = dp4a_ss(w.w0.w, x0.w, s);
    s = dp4a_ss(w.w1.x, x1.x, s); s = dp4a_ss(w.w1.y, x1.y, s); s = dp4a_ss(w.w1.z, x1.z, s); s = dp4a_ss(w.w1.w, x1.w, s);
    return (float)s * (half_bits_to_float(w.d) * xd);
}

template <int G, int R, int NW>
__global__ void __launch_bounds__(NW * 32) gemv_q80p_kernel(const uint8_t *__restrict__ W, const uint8_t *__restrict__ xg, float *__restrict__ y, int M, int nb)
{
    extern __shared__ __align__(128) uint8_t smem[];
    constexpr int RPW = (32 / G) * R;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int li = lane % G, sub = lane / G;
    const int nitems = (M + RPW - 1) / RPW, item_stride = gridDim.x * NW;
    const int npass = (nb + G - 1) / G;
    const size_t rb = q80p_row_bytes(nb), off_d = (size_t)nb * 32;

    pdl_trigger();

    auto load_item = [&](Q80pW (&w)[R], int item, int pass) {
        const int row0 = item * RPW + sub * R;
        const int b = min(li + pass * G, nb - 1);
#pragma unroll
        for (int r = 0; r < R; ++r) {
            const uint8_t *row = W + (size_t)min(row0 + r, M - 1) * rb;
            w[r].w0 = __ldg(reinterpret_cast<const uint4 *>(row + (size_t)b * 32));
            w[r].w1 = __ldg(reinterpret_cast<const uint4 *>(row + (size_t)b * 32 + 16));
            w[r].d = ldg_nc_u16(row + off_d + (size_t)b * 2);
        }
    };

    Q80pW cur[R], nxt[R];
    int item = blockIdx.x + gridDim.x * warp, pass = 0;
    if (item < nitems) load_item(cur, item, 0);

    pdl_wait();
    const RingX x = ring_stage_x<FMT_Q80>(xg, nb, smem);
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
            for (int r = 0; r < R; ++r) acc[r] += q80p_unit(cur[r], b, x);
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

// src: the reference's rows of nb 34-byte blocks; dst: planar rows.  One CTA per row, 2-byte units.
__global__ void __launch_bounds__(256) q80_to_planar_kernel(const uint8_t *__restrict__ src, uint8_t *__restrict__ dst, int nb)
{
    const size_t row = blockIdx.x;
    const unsigned short *s = reinterpret_cast<const unsigned short *>(src + row * (size_t)nb * Q80_BYTES);
    unsigned short *d = reinterpret_cast<unsigned short *>(dst + row * q80p_row_bytes(nb));
    const int total = nb * 17;
    for (int i = threadIdx.x; i < total; i += blockDim.x) {
        const int b = i / 17, o = i - b * 17;
        d[o == 0 ? nb * 16 + b : b * 16 + (o - 1)] = s[i];
    }
    const int pad0 = nb * 17, pad1 = (int)(q80p_row_bytes(nb) / 2);
    for (int i = pad0 + threadIdx.x; i < pad1; i += blockDim.x) d[i] = 0;
}

}  // namespace ckb

using namespace ckb;

namespace {

template <int G, int R>
int launch_q80p(float *y, const void *W, const void *xq, int M, int nb, cudaStream_t st)
{
    constexpr int NW = 8;
    auto kernel = gemv_q80p_kernel<G, R, NW>;
    const int smem = ringx_smem_bytes(FMT_Q80, nb);
    if (smem > 220 * 1024) return ckb_fail(CKB_ERR_LIMIT, "gemv_q8_0 (planar): K too large for the shared activation buffer");
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
    return launch_pdl("gemv_q80_planar", kernel, dim3(grid), dim3(NW * 32), (size_t)smem, st, (const uint8_t *)W, (const uint8_t *)xq, y, M, nb);
}

}  // namespace

extern "C" size_t ckb200_q8_0_planar_bytes(int rows, int cols) { return cols % 32 ? 0 : (size_t)rows * q80p_row_bytes(cols / 32); }

extern "C" int ckb200_dev_q8_0_to_planar(void *dst, const void *src, int rows, int cols, void *stream)
{
    if (!dst || !src || rows <= 0 || cols <= 0) return 0;
    if (cols % 32 || ((uintptr_t)dst & 15) || ((uintptr_t)src & 1)) return ckb_fail(CKB_ERR_SHAPE, "q8_0_to_planar: K %% 32 or alignment");
    if (ckb_ensure_init()) return CKB_ERR_NO_DEVICE;
    q80_to_planar_kernel<<<rows, 256, 0, ckb_stream(stream)>>>((const uint8_t *)src, (uint8_t *)dst, cols / 32);
    return ckb_check_launch("q80_to_planar");
}

extern "C" int ckb200_dev_gemv_q8_0_planar_q8_0(float *y, const void *W_planar, const void *x_q8, int M, int K, void *stream)
{
    if (!y || !W_planar || !x_q8 || M <= 0 || K <= 0) return 0;
    if (K % 32 || ((uintptr_t)W_planar & 15) || ((uintptr_t)x_q8 & 1)) return ckb_fail(CKB_ERR_SHAPE, "gemv_q8_0 (planar): K %% 32 or alignment");
    if (ckb_ensure_init()) return CKB_ERR_NO_DEVICE;
    const int nb = K / 32;
    cudaStream_t st = ckb_stream(stream);
    int g = 1;
    while (g < 32 && g < nb) g <<= 1;
    switch (g) {
        case 1: return launch_q80p<1, 2>(y, W_planar, x_q8, M, nb, st);
        case 2: return launch_q80p<2, 2>(y, W_planar, x_q8, M, nb, st);
        case 4: return launch_q80p<4, 2>(y, W_planar, x_q8, M, nb, st);
        case 8: return launch_q80p<8, 2>(y, W_planar, x_q8, M, nb, st);
        case 16: return launch_q80p<16, 2>(y, W_planar, x_q8, M, nb, st);
        default: return launch_q80p<32, 2>(y, W_planar, x_q8, M, nb, st);
    }
}
