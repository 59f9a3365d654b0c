// Q6_K x Q8_K product for a handful of tokens over row-planar weights (gemv_q6k_planar.cu's layout): C[M, N] = A_q8[M, K] . B[N, K]^T + bias,
// M <= 64 - the reference's gemm_nt_q6_k_q8_k (src/kernels/gemm_kernels_q6k_q8k.c:86-116, :238-258) for batched decode.
//
// The Q4_K kernel of gemm_q4k_mma.cu with Q6_K's arithmetic.  A superblock has 16 groups of 16 weights, each with an int8 scale, so
// the tensor-core instruction is mma.sync.m16n8k16 (u8 x s8 -> s32): one per (group, 8 tokens).  A lane builds its A fragment from one
// word of the ql plane (low or high nibbles) and one word of the qh plane (a 2-bit plane shifted to bits 4-5): q6 in 0 .. 63; the
// format's -32 goes through the activation block sums, which Q8_K keeps per 16 elements - exactly Q6_K's groups:
//     sum_g sc_g sum_i (q6 - 32) x  =  sum_g sc_g isum_g  -  32 sum_g sc_g bsum_g
// with the second sum again from the tensor cores (scales as A; low and high bytes of the block sums as B).  All integer parts are
// exact for every scale value; once per superblock acc += (d_w d_x) float(...).
//
// The planes of a superblock arrive as four tiled bulk copies per step and K slice (ql with the 128-byte swizzle so that the eight
// rows a fragment load touches fall into different banks; qh, scales and the 16-byte window around d as they lie), the Q8_K
// windows of all tokens as a fifth; rows past N and token slots past M are zero-filled by the copies.  The copies are issued by
// the first lane of a ninth warp; the eight computing warps wait for a stage on its `full` mbarrier and release it on its `empty`
// one, so no warp waits for another inside the K loop.  Needs K a multiple of 1024 and 16-byte-aligned activation rows (the
// tcgen05 kernel of gemm_tc.cu serves everything else).
#include <cuda.h>

#include "device_common.cuh"
#include "launch.h"
#include "pdl.cuh"
#include "q6p_unit.cuh"
#include "runtime.h"

namespace ckb {

constexpr int QM6_WARPS = 8, QM6_THREADS = 32 * (QM6_WARPS + 1);   // eight computing warps and the warp that issues the copies
constexpr int QM6_XWIN = 304;                                  // a 292-byte Q8_K block from its 16-byte-aligned start

__device__ __forceinline__ void qm6_tma_2d(uint32_t dst, const CUtensorMap *map, int x, int y, uint32_t bar)
{
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
                 ::"r"(dst), "l"(map), "r"(x), "r"(y), "r"(bar) : "memory");
}
// d = a . b, k = 16: a two registers (rows g, g + 8), b one; the accumulator input is one zero register four times
__device__ __forceinline__ void qm6_mma_us(int (&d)[4], uint32_t a0, uint32_t a1, uint32_t b, int zero)
{
    asm volatile("mma.sync.aligned.m16n8k16.row.col.s32.u8.s8.s32 {%0,%1,%2,%3}, {%4,%5}, {%6}, {%7,%7,%7,%7};"
                 : "=r"(d[0]), "=r"(d[1]), "=r"(d[2]), "=r"(d[3]) : "r"(a0), "r"(a1), "r"(b), "r"(zero));
}
__device__ __forceinline__ void qm6_mma_su(int (&d)[4], uint32_t a0, uint32_t a1, uint32_t b, int zero)
{
    asm volatile("mma.sync.aligned.m16n8k16.row.col.s32.s8.u8.s32 {%0,%1,%2,%3}, {%4,%5}, {%6}, {%7,%7,%7,%7};"
                 : "=r"(d[0]), "=r"(d[1]), "=r"(d[2]), "=r"(d[3]) : "r"(a0), "r"(a1), "r"(b), "r"(zero));
}
__device__ __forceinline__ void qm6_mma_ss(int (&d)[4], uint32_t a0, uint32_t a1, uint32_t b, int zero)
{
    asm volatile("mma.sync.aligned.m16n8k16.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5}, {%6}, {%7,%7,%7,%7};"
                 : "=r"(d[0]), "=r"(d[1]), "=r"(d[2]), "=r"(d[3]) : "r"(a0), "r"(a1), "r"(b), "r"(zero));
}
__device__ __forceinline__ int qm6_sbyte(uint32_t w, int j)      // byte j of w, sign-extended
{
    int r;
    asm("bfe.s32 %0, %1, %2, 8;" : "=r"(r) : "r"(w), "r"(8 * j));
    return r;
}

template <int NT, int RW, int KS, int D> struct Qm6Smem {
    static constexpr int MT = 8 * NT;
    static constexpr int ROWS = 16 * RW * (QM6_WARPS / KS);    // rows of the CTA (every K slice covers all of them)
    static constexpr int QL = 0, QH = ROWS * 128, SC = QH + ROWS * 64, DD = SC + ROWS * 16, X = DD + ROWS * 16;       // offsets inside a slice
    static constexpr int WBYTES = ROWS * 224;
    static constexpr int SLICE = ((X + MT * QM6_XWIN + 1023) / 1024) * 1024;             // the swizzled ql box wants 1024-byte alignment
    static constexpr int STAGE = KS * SLICE;
    static constexpr int BYTES = D * STAGE;
};

template <int NT, int RW, int RT, int KS, int D, int OCC>
__global__ void __launch_bounds__(QM6_THREADS, OCC) gemm_q6k_mma_kernel(const __grid_constant__ CUtensorMap tm_ql, const __grid_constant__ CUtensorMap tm_qh,
                                                                   const __grid_constant__ CUtensorMap tm_sc, const __grid_constant__ CUtensorMap tm_x,
                                                                   const float *__restrict__ bias, float *__restrict__ C, int ldc, int M, int N, int nb,
                                                                   int *__restrict__ dev_err)
{
    static_assert(RT * KS == QM6_WARPS, "8 warps");
    using L = Qm6Smem<NT, RW, KS, D>;
    extern __shared__ __align__(16) uint8_t qm6_raw[];
    __shared__ __align__(8) uint64_t full[D], empty[D];
    uint8_t *smem = qm6_raw + ((1024u - (smem_u32(qm6_raw) & 1023u)) & 1023u);           // the launch asks for 1 KB more
    const uint32_t s_base = smem_u32(smem);
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int g = lane >> 2, t = lane & 3;
    const int rt = warp % RT, ks = warp / RT;
    const int row0 = blockIdx.x * L::ROWS;
    const int per = (nb + KS - 1) / KS;
    const int b_first = ks * per;

    if (tid == 0) {
        for (int i = 0; i < D; ++i) { mbar_init(smem_u32(&full[i]), 1); mbar_init(smem_u32(&empty[i]), QM6_WARPS); }
        mbar_fence_init();
    }
    __syncthreads();
    pdl_trigger();

    // the issuing thread: the copies of step s.  Plane offsets inside a planar row: ql at 0, qh at nb * 128, scales at nb * 192, d at nb * 208.
    auto expect = [&](int s) {
        int slices = 0;
        for (int k = 0; k < KS; ++k) slices += (k * per + s < nb);
        mbar_arrive_expect_tx(smem_u32(&full[s % D]), (uint32_t)slices * (uint32_t)(L::WBYTES + L::MT * QM6_XWIN));
    };
    auto issue_w = [&](int s) {
        const uint32_t bar = smem_u32(&full[s % D]);
        for (int k = 0; k < KS; ++k) {
            const int b = k * per + s;
            if (b >= nb) continue;
            const uint32_t sl = s_base + (uint32_t)(s % D) * L::STAGE + (uint32_t)k * L::SLICE;
            qm6_tma_2d(sl + L::QL, &tm_ql, b * 128, row0, bar);
            qm6_tma_2d(sl + L::QH, &tm_qh, nb * 128 + b * 64, row0, bar);
            qm6_tma_2d(sl + L::SC, &tm_sc, nb * 192 + b * 16, row0, bar);
            qm6_tma_2d(sl + L::DD, &tm_sc, (nb * 208 + 2 * b) & ~15, row0, bar);
        }
    };
    auto issue_x = [&](int s) {
        const uint32_t bar = smem_u32(&full[s % D]);
        for (int k = 0; k < KS; ++k) {
            const int b = k * per + s;
            if (b < nb) qm6_tma_2d(s_base + (uint32_t)(s % D) * L::STAGE + (uint32_t)k * L::SLICE + L::X, &tm_x, ((b * Q8K_BYTES) & ~15) / 4, 0, bar);
        }
    };

    const int zero = 0;
    float acc[RW][NT][4];
#pragma unroll
    for (int rw = 0; rw < RW; ++rw)
#pragma unroll
        for (int nt = 0; nt < NT; ++nt)
#pragma unroll
            for (int e = 0; e < 4; ++e) acc[rw][nt][e] = 0.0f;

    // The ninth warp only issues copies: a stage is refilled as soon as the eight computing warps have released it, and no
    // computing warp waits for another between steps (with one thread of a computing warp issuing the twenty copies of a step
    // behind a CTA-wide barrier, three warps in four sat at that barrier).
    if (warp == QM6_WARPS) {
        if (lane == 0) {
            const int pro = per < D ? per : D;
            for (int s = 0; s < pro; ++s) { expect(s); issue_w(s); }                     // weights are not written by any kernel: before the dependency wait
            pdl_wait();
            for (int s = 0; s < pro; ++s) issue_x(s);
            for (int s = D; s < per; ++s) {
                if (!mbar_wait_spin(smem_u32(&empty[s % D]), (uint32_t)(s / D - 1) & 1u)) { atomicExch(dev_err, DEV_ERR_FULL_WAIT); break; }
                expect(s); issue_w(s); issue_x(s);
            }
        }
    } else {
    pdl_wait();
    bool ok = true;
    for (int s = 0; s < per; ++s) {
        const int b = b_first + s;
        if (s > 0) {                                           // step s - 1 is finished in this warp: one more release of its stage
            __syncwarp();
            if (lane == 0) mbar_arrive(smem_u32(&empty[(s - 1) % D]));
        }
        if (b >= nb) continue;
        if (ok && !mbar_wait_spin(smem_u32(&full[s % D]), (uint32_t)(s / D) & 1u)) {
            ok = false;
            if (lane == 0) atomicExch(dev_err, DEV_ERR_FULL_WAIT);
        }
        const uint8_t *sl = smem + (size_t)(s % D) * L::STAGE + (size_t)ks * L::SLICE;
        const uint8_t *xs = sl + L::X + ((b * Q8K_BYTES) & 15);
        const int dph = (nb * 208 + 2 * b) & 15;
        const int r0 = rt * 16 * RW + g;                       // this lane's first row inside the CTA's rows

        uint32_t scw[RW][2][4];
        float dw[RW][2];
#pragma unroll
        for (int rw = 0; rw < RW; ++rw)
#pragma unroll
            for (int r = 0; r < 2; ++r) {
                const int row = r0 + 16 * rw + 8 * r;
                const uint4 w = *reinterpret_cast<const uint4 *>(sl + L::SC + row * 16);
                scw[rw][r][0] = w.x; scw[rw][r][1] = w.y; scw[rw][r][2] = w.z; scw[rw][r][3] = w.w;
                dw[rw][r] = half_bits_to_float(*reinterpret_cast<const unsigned short *>(sl + L::DD + row * 16 + dph));
            }
        int S[RW][NT][4];
#pragma unroll
        for (int rw = 0; rw < RW; ++rw)
#pragma unroll
            for (int nt = 0; nt < NT; ++nt)
#pragma unroll
                for (int e = 0; e < 4; ++e) S[rw][nt][e] = 0;

#pragma unroll
        for (int n = 0; n < 2; ++n)
#pragma unroll
            for (int hf = 0; hf < 2; ++hf) {
                // the 2-bit planes of qh bytes 32n + 16hf + 4t .., moved to bits 4-5, for the four quarters
                uint32_t pl[RW][2][4];
#pragma unroll
                for (int rw = 0; rw < RW; ++rw)
#pragma unroll
                    for (int r = 0; r < 2; ++r) {
                        const int row = r0 + 16 * rw + 8 * r;
                        const uint32_t qh = *reinterpret_cast<const uint32_t *>(sl + L::QH + row * 64 + 32 * n + 16 * hf + 4 * t);
                        pl[rw][r][0] = (qh << 4) & 0x30303030u;
                        pl[rw][r][1] = (qh << 2) & 0x30303030u;
                        pl[rw][r][2] = qh & 0x30303030u;
                        pl[rw][r][3] = (qh >> 2) & 0x30303030u;
                    }
#pragma unroll
                for (int q1 = 0; q1 < 2; ++q1) {
                    // ql bytes 64n + 32 q1 + 16hf + 4t ..: 16-byte chunk 4n + 2 q1 + hf of the row, swizzled with the row
                    uint32_t ql[RW][2];
#pragma unroll
                    for (int rw = 0; rw < RW; ++rw)
#pragma unroll
                        for (int r = 0; r < 2; ++r) {
                            const int row = r0 + 16 * rw + 8 * r, chunk = 4 * n + 2 * q1 + hf;
                            ql[rw][r] = *reinterpret_cast<const uint32_t *>(sl + L::QL + row * 128 + ((chunk ^ (row & 7)) << 4) + 4 * t);
                        }
#pragma unroll
                    for (int hi = 0; hi < 2; ++hi) {
                        const int qtr = q1 + 2 * hi, grp = 8 * n + 2 * qtr + hf;
                        uint32_t a[RW][2];
                        int sc[RW][2];
#pragma unroll
                        for (int rw = 0; rw < RW; ++rw)
#pragma unroll
                            for (int r = 0; r < 2; ++r) {
                                a[rw][r] = ((ql[rw][r] >> (4 * hi)) & 0x0F0F0F0Fu) | pl[rw][r][qtr];
                                sc[rw][r] = qm6_sbyte(scw[rw][r][grp >> 2], grp & 3);
                            }
#pragma unroll
                        for (int nt = 0; nt < NT; ++nt) {
                            const uint32_t bx = *reinterpret_cast<const uint32_t *>(xs + (size_t)(nt * 8 + g) * QM6_XWIN + 4 + 16 * grp + 4 * t);
#pragma unroll
                            for (int rw = 0; rw < RW; ++rw) {
                                int cc[4];
                                qm6_mma_us(cc, a[rw][0], a[rw][1], bx, zero);
                                S[rw][nt][0] += sc[rw][0] * cc[0];
                                S[rw][nt][1] += sc[rw][0] * cc[1];
                                S[rw][nt][2] += sc[rw][1] * cc[2];
                                S[rw][nt][3] += sc[rw][1] * cc[3];
                            }
                        }
                    }
                }
            }
        // the -32: k index = group; A = the scales of rows g, g + 8 (bytes 4t .. 4t + 3), B = low / high bytes of the 16-element block sums
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) {
            const uint32_t *bsp = reinterpret_cast<const uint32_t *>(xs + (size_t)(nt * 8 + g) * QM6_XWIN + 260 + 8 * t);
            const uint32_t bs0 = bsp[0], bs1 = bsp[1];
            const uint32_t lo = __byte_perm(bs0, bs1, 0x6420u), hi = __byte_perm(bs0, bs1, 0x7531u);
            const float dxa = *reinterpret_cast<const float *>(xs + (size_t)(nt * 8 + 2 * t) * QM6_XWIN);
            const float dxb = *reinterpret_cast<const float *>(xs + (size_t)(nt * 8 + 2 * t + 1) * QM6_XWIN);
#pragma unroll
            for (int rw = 0; rw < RW; ++rw) {
                const uint32_t a0 = t == 0 ? scw[rw][0][0] : (t == 1 ? scw[rw][0][1] : (t == 2 ? scw[rw][0][2] : scw[rw][0][3]));
                const uint32_t a1 = t == 0 ? scw[rw][1][0] : (t == 1 ? scw[rw][1][1] : (t == 2 ? scw[rw][1][2] : scw[rw][1][3]));
                int Lo[4], Hi[4];
                qm6_mma_su(Lo, a0, a1, lo, zero);
                qm6_mma_ss(Hi, a0, a1, hi, zero);
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const int total = S[rw][nt][e] - 32 * (Hi[e] * 256 + Lo[e]);
                    acc[rw][nt][e] += __fmul_rn(dw[rw][e >> 1], (e & 1) ? dxb : dxa) * (float)total;
                }
            }
        }
    }
    }
    __syncthreads();                                           // the staging area becomes the reduction buffer (every issued copy was waited for)

    float *red = reinterpret_cast<float *>(smem);
    constexpr int PER_WARP = RW * NT * 4;
    if (KS > 1 && ks > 0 && warp < QM6_WARPS) {
#pragma unroll
        for (int rw = 0; rw < RW; ++rw)
#pragma unroll
            for (int nt = 0; nt < NT; ++nt)
#pragma unroll
                for (int e = 0; e < 4; ++e) red[(((size_t)(ks - 1) * RT + rt) * PER_WARP + (rw * NT + nt) * 4 + e) * 32 + lane] = acc[rw][nt][e];
    }
    if (KS > 1) __syncthreads();
    if (ks == 0 && warp < QM6_WARPS) {
        const int n0 = row0 + rt * 16 * RW;
#pragma unroll
        for (int rw = 0; rw < RW; ++rw)
#pragma unroll
            for (int nt = 0; nt < NT; ++nt)
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    float v = acc[rw][nt][e];
                    for (int k = 1; k < KS; ++k) v += red[(((size_t)(k - 1) * RT + rt) * PER_WARP + (rw * NT + nt) * 4 + e) * 32 + lane];
                    const int row = n0 + 16 * rw + g + ((e & 2) ? 8 : 0), tok = nt * 8 + 2 * t + (e & 1);
                    if (row < N && tok < M) C[(size_t)tok * ldc + row] = bias ? v + bias[row] : v;
                }
    }
}

typedef CUresult (*qm6_encode_fn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *, const cuuint64_t *, const cuuint32_t *,
                                  const cuuint32_t *, CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
static qm6_encode_fn qm6_encoder()
{
    static qm6_encode_fn fn = nullptr;
    static bool tried = false;
    if (!tried) {
        tried = true;
        void *p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess && q == cudaDriverEntryPointSuccess) fn = (qm6_encode_fn)p;
        else cudaGetLastError();
    }
    return fn;
}
// a matrix of `rows` rows of `row_bytes` bytes, boxes of box_bytes x box_rows in elements of `elem` bytes
static bool qm6_make_map(CUtensorMap *map, const void *base, size_t row_bytes, size_t rows, unsigned box_bytes, unsigned box_rows, unsigned elem, bool swizzle128)
{
    qm6_encode_fn enc = qm6_encoder();
    if (!enc || row_bytes % 16 || box_bytes % 16 || box_bytes / elem > 256 || box_rows > 256) return false;
    const cuuint64_t dims[2] = {(cuuint64_t)(row_bytes / elem), (cuuint64_t)rows}, strides[1] = {(cuuint64_t)row_bytes};
    const cuuint32_t box[2] = {box_bytes / elem, box_rows}, estr[2] = {1, 1};
    return enc(map, elem == 4 ? CU_TENSOR_MAP_DATA_TYPE_UINT32 : CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void *>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
               swizzle128 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

template <int NT, int RW, int RT, int KS, int D, int OCC>
static int qm6_launch(const void *A_q8, const void *B, const float *bias, float *C, int ldc, int M, int N, int nb, cudaStream_t st)
{
    using L = Qm6Smem<NT, RW, KS, D>;
    static_assert((KS - 1) * RT * RW * NT * 4 * 32 * 4 <= L::BYTES, "the reduction buffer fits into the staging area");
    static_assert(OCC * (L::BYTES + 2048) <= 227 * 1024, "shared memory of the resident CTAs");
    static_assert(L::ROWS <= 256 && L::MT <= 256, "box limits");
    const size_t rb = q6p_row_bytes(nb);
    CUtensorMap tm_ql, tm_qh, tm_sc, tm_x;
    if (!qm6_make_map(&tm_ql, B, rb, (size_t)N, 128, L::ROWS, 1, true) || !qm6_make_map(&tm_qh, B, rb, (size_t)N, 64, L::ROWS, 1, false) ||
        !qm6_make_map(&tm_sc, B, rb, (size_t)N, 16, L::ROWS, 1, false) || !qm6_make_map(&tm_x, A_q8, (size_t)nb * Q8K_BYTES, (size_t)M, QM6_XWIN, L::MT, 4, false))
        return -1;
    static bool attr_set = false;
    if (!attr_set) {
        if (ckb_check_cuda((int)cudaFuncSetAttribute(gemm_q6k_mma_kernel<NT, RW, RT, KS, D, OCC>, cudaFuncAttributeMaxDynamicSharedMemorySize, L::BYTES + 1024), "gemm_q6k_mma smem"))
            return CKB_ERR_CUDA;
        attr_set = true;
    }
    const int grid = (N + L::ROWS - 1) / L::ROWS;
    return launch_pdl("gemm_q6k_mma", gemm_q6k_mma_kernel<NT, RW, RT, KS, D, OCC>, dim3(grid), dim3(QM6_THREADS), (size_t)(L::BYTES + 1024), st, tm_ql, tm_qh, tm_sc, tm_x, bias, C, ldc,
                      M, N, nb, ckb_device_error_word());
}

template <int NT, int RW>
static int qm6_shape(int shape, const void *A_q8, const void *B, const float *bias, float *C, int ldc, int M, int N, int nb, cudaStream_t st)
{
    constexpr int s1 = Qm6Smem<NT, RW, 1, 1>::SLICE, s2 = 2 * Qm6Smem<NT, RW, 2, 1>::SLICE, s4 = 4 * Qm6Smem<NT, RW, 4, 1>::SLICE;
    constexpr int lim = 225 * 1024;
    constexpr int D1 = 4 * s1 <= lim ? 4 : (3 * s1 <= lim ? 3 : 2), D2 = 4 * s2 <= lim ? 4 : (3 * s2 <= lim ? 3 : 2), D4 = 4 * s4 <= lim ? 4 : (3 * s4 <= lim ? 3 : 2);
    if (shape == 1) return qm6_launch<NT, RW, 8, 1, D1, 1>(A_q8, B, bias, C, ldc, M, N, nb, st);
    if (shape == 2) return qm6_launch<NT, RW, 4, 2, D2, 1>(A_q8, B, bias, C, ldc, M, N, nb, st);
    return qm6_launch<NT, RW, 2, 4, D4, 1>(A_q8, B, bias, C, ldc, M, N, nb, st);
}

// Up to 16 tokens the work of a step is mostly the unpacking of the weights, a chain of dependent integer instructions that eight
// warps do not always hide: two CTAs per SM (one 16-row tile per warp, two stages each) keep sixteen computing warps resident.
template <int NT>
static int qm6_shape_pair(int shape, const void *A_q8, const void *B, const float *bias, float *C, int ldc, int M, int N, int nb, cudaStream_t st)
{
    if (shape == 1) return qm6_launch<NT, 1, 8, 1, 2, 2>(A_q8, B, bias, C, ldc, M, N, nb, st);
    if (shape == 2) return qm6_launch<NT, 1, 4, 2, 2, 2>(A_q8, B, bias, C, ldc, M, N, nb, st);
    return qm6_launch<NT, 1, 2, 4, 2, 2>(A_q8, B, bias, C, ldc, M, N, nb, st);
}

template <int NT>
static int qm6_pick(const void *A_q8, const void *B, const float *bias, float *C, int ldc, int M, int N, int nb, cudaStream_t st)
{
    // CTAs per SM: 0 auto, 1, 2.  Two pay where there are rows for them: up to 8 tokens from about 28000 rows (an LM head: 188 ->
    // 161 us at 128256 x 8192; the 70B down projection, 8192 rows, 45 us with one against 51), 9 to 16 tokens from 4736 rows.
    int occ = ckb_tune_get("gemm_q6k_mma_occ", 0);
    const int sms = ckb_sm_count();
    if (occ != 1 && occ != 2) occ = (NT == 1 && (N + 127) / 128 >= 3 * sms / 2) || (NT == 2 && (N + 31) / 32 >= sms) ? 2 : 1;
    if (NT > 2) occ = 1;
    const int want = 3 * occ * sms / 4;
    int rw = ckb_tune_get("gemm_q6k_mma_rw", 0);               // 16-row tiles per warp: 0 auto, 1, 2 (64 token slots: always 1, registers)
    if (NT >= 8 || occ == 2) rw = 1;
    else if (rw != 1 && rw != 2) rw = (N + 63) / 64 >= want ? 2 : 1;
    int shape = ckb_tune_get("gemm_q6k_mma_shape", 0);         // 1: 8 row warps, 2: 4 x 2 K slices, 4: 2 x 4 K slices, 0: the widest CTA that fills 3/4 of the slots
    if (shape != 1 && shape != 2 && shape != 4) {
        shape = 4;
        for (int cand = 1; cand < 4; cand *= 2) {
            const int rows = 16 * rw * 8 / cand;
            if ((N + rows - 1) / rows >= want || nb < 2 * cand) { shape = cand; break; }
        }
        if (nb < 4 && shape == 4) shape = nb >= 2 ? 2 : 1;
    }
    if constexpr (NT <= 2) {
        if (occ == 2) return qm6_shape_pair<NT>(shape, A_q8, B, bias, C, ldc, M, N, nb, st);
    }
    if constexpr (NT < 8) {
        if (rw == 2) return qm6_shape<NT, 2>(shape, A_q8, B, bias, C, ldc, M, N, nb, st);
    }
    return qm6_shape<NT, 1>(shape, A_q8, B, bias, C, ldc, M, N, nb, st);
}

}  // namespace ckb

using namespace ckb;

// B_planar: ckb200_q6_k_planar_bytes(N, K) of row-planar Q6_K weights.  Returns -1 when this kernel does not take the call.
// Whether the launcher below takes this product (for a caller that runs several products side by side: no workspace here).
extern "C" int ckb_gemm_q6k_mma_takes(const void *A_q8, const void *B_planar, int M, int N, int K)
{
    if (!A_q8 || !B_planar || N <= 0 || K <= 0 || K % 1024) return 0;
    if (M < ckb_tune_get("gemm_q6k_mma_min", 2) || M > ckb_tune_get("gemm_q6k_mma_max", 64) || M > 64 || !ckb_tune_get("gemm_q6k_mma", 1)) return 0;
    return !(((uintptr_t)B_planar & 15) || ((uintptr_t)A_q8 & 15));
}

extern "C" int ckb_launch_gemm_q6k_mma(const void *A_q8, const void *B_planar, const float *bias, float *C, int ldc, int M, int N, int K, void *stream)
{
    if (!C || !ckb_gemm_q6k_mma_takes(A_q8, B_planar, M, N, K)) return -1;
    if (ckb_ensure_init()) return CKB_ERR_NO_DEVICE;
    cudaStream_t st = ckb_stream(stream);
    const int nb = K / QK_K;
    if (M <= 8) return qm6_pick<1>(A_q8, B_planar, bias, C, ldc, M, N, nb, st);
    if (M <= 16) return qm6_pick<2>(A_q8, B_planar, bias, C, ldc, M, N, nb, st);
    if (M <= 32) return qm6_pick<4>(A_q8, B_planar, bias, C, ldc, M, N, nb, st);
    return qm6_pick<8>(A_q8, B_planar, bias, C, ldc, M, N, nb, st);
}
