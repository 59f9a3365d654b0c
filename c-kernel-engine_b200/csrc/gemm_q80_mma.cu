// Batched Q8_0 x Q8_0 product for prefill: C[M,N] = A_q8[M,K] . B[N,K]^T + bias, the reference's gemm_nt_q8_0_q8_0
// (src/kernels/gemm_batch_int8.c:87-120; the symbol version/v7/src/ck_parallel_prefill.h:44-48 dispatches).
//
// Both operands carry one fp16 scale per 32 elements, so the integer part of the product is a sum of 32 int8 x int8 terms per
// block and every block needs its own scale: C[m][n] = sum_b (sum_32 a q) * (d_a[m][b] * d_w[n][b]).  One integer tensor-core
// instruction (mma.sync m16n8k32, s8 x s8 -> s32) is exactly one block deep, so a warp issues one MMA per (16 x 8 outputs, block),
// converts the int32 block sums and adds them, scaled, to fp32 accumulators - block after block in the reference's order, which
// makes the result bit-identical to the scalar loop (int32 sums are exact, the fp32 operations are the same and in the same order).
//
// Operands come in the row-planar layout of gemv_q80_planar.cu (per row all quants, then all scales; the reference's 34-byte
// blocks are only 2-byte aligned), so tiles move with 16-byte cp.async into shared memory: 128 tokens x 128 weight rows per CTA,
// four blocks (128 bytes of k) per stage, three stages; rows padded to 144 bytes in shared memory so that the eight rows a
// fragment load touches fall into different banks.  Every weight tile is read once per 128 tokens instead of once per token.
#include "device_common.cuh"
#include "launch.h"
#include "runtime.h"

namespace ckb {

constexpr int QM_BM = 128, QM_BN = 128, QM_KB = 4, QM_STAGES = 3, QM_THREADS = 256;
constexpr int QM_ROW = QM_KB * 32 + 16;                       // bytes of one tile row in shared memory (padded)
constexpr int QM_TILE = QM_BM * QM_ROW;                       // quants of one operand, one stage
constexpr int QM_SCALES = QM_BM * QM_KB * 2;                  // fp16 scales of one operand, one stage
constexpr int QM_STAGE = 2 * QM_TILE + 2 * QM_SCALES;
constexpr int QM_SMEM = QM_STAGES * QM_STAGE;

__host__ __device__ inline size_t qm_row_bytes(int nb) { return ((size_t)nb * Q80_BYTES + 15) & ~(size_t)15; }

__device__ __forceinline__ void cp_async16(uint32_t dst, const void *src) { asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src) : "memory"); }
__device__ __forceinline__ void cp_async8(uint32_t dst, const void *src) { asm volatile("cp.async.ca.shared.global [%0], [%1], 8;" ::"r"(dst), "l"(src) : "memory"); }
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

__device__ __forceinline__ void mma_s8(int (&c)[4], const uint32_t (&a)[4], const uint32_t (&b)[2])
{
    asm volatile("mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+r"(c[0]), "+r"(c[1]), "+r"(c[2]), "+r"(c[3]) : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b[0]), "r"(b[1]));
}

// A, B: row-planar Q8_0 (rows of nb blocks, nb a multiple of QM_KB).  grid = (N tiles, M tiles).
__global__ void __launch_bounds__(QM_THREADS) gemm_q80_mma_kernel(const uint8_t *__restrict__ A, const uint8_t *__restrict__ B, const float *__restrict__ bias,
                                                                  float *__restrict__ C, int M, int N, int nb)
{
    extern __shared__ __align__(128) uint8_t smem[];
    const uint32_t s_base = smem_u32(smem);
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int wm = warp >> 2, wn = warp & 3;                  // 2 x 4 warps: 64 tokens x 32 weight rows each
    const int g = lane >> 2, t = lane & 3;
    const int m0 = blockIdx.y * QM_BM, n0 = blockIdx.x * QM_BN;
    const size_t rb = qm_row_bytes(nb), off_d = (size_t)nb * 32;
    const int nchunks = nb / QM_KB;

    auto issue = [&](int chunk) {
        const uint32_t st = s_base + (uint32_t)(chunk % QM_STAGES) * QM_STAGE;
        const int kb = chunk * QM_KB;
        // quants: 128 rows x 8 pieces of 16 bytes per operand
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int idx = tid + i * QM_THREADS, row = idx >> 3, piece = idx & 7;
            cp_async16(st + (uint32_t)(row * QM_ROW + piece * 16), A + (size_t)min(m0 + row, M - 1) * rb + (size_t)kb * 32 + piece * 16);
            cp_async16(st + QM_TILE + (uint32_t)(row * QM_ROW + piece * 16), B + (size_t)min(n0 + row, N - 1) * rb + (size_t)kb * 32 + piece * 16);
        }
        // scales: 4 fp16 per row per operand
        {
            const int row = tid & 127;
            const uint8_t *src = tid < 128 ? A + (size_t)min(m0 + row, M - 1) * rb : B + (size_t)min(n0 + row, N - 1) * rb;
            cp_async8(st + 2 * QM_TILE + (tid < 128 ? 0 : QM_SCALES) + (uint32_t)(row * 8), src + off_d + (size_t)kb * 2);
        }
        cp_async_commit();
    };

    float acc[4][4][4];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j)
#pragma unroll
            for (int e = 0; e < 4; ++e) acc[i][j][e] = 0.0f;

    for (int c = 0; c < QM_STAGES - 1; ++c) {
        if (c < nchunks) issue(c);
        else cp_async_commit();
    }
    for (int c = 0; c < nchunks; ++c) {
        cp_async_wait<QM_STAGES - 2>();
        __syncthreads();                                      // chunk c has landed for everyone, and chunk c - 1's stage is free
        if (c + QM_STAGES - 1 < nchunks) issue(c + QM_STAGES - 1);
        else cp_async_commit();
        const uint32_t st = s_base + (uint32_t)(c % QM_STAGES) * QM_STAGE;
        const uint32_t sA = st + (uint32_t)((wm * 64 + g) * QM_ROW + t * 4), sB = st + QM_TILE + (uint32_t)((wn * 32 + g) * QM_ROW + t * 4);
        const uint32_t sDA = st + 2 * QM_TILE + (uint32_t)((wm * 64 + g) * 8), sDB = st + 2 * QM_TILE + QM_SCALES + (uint32_t)((wn * 32 + 2 * t) * 8);
#pragma unroll
        for (int b = 0; b < QM_KB; ++b) {
            uint32_t af[4][4], bf[4][2];
            float da[4][2], db[4][2];
#pragma unroll
            for (int i = 0; i < 4; ++i) {                     // token rows 16 i + g and + 8
                const uint32_t p = sA + (uint32_t)(i * 16 * QM_ROW + b * 32);
                af[i][0] = lds_u32(p);
                af[i][1] = lds_u32(p + 8 * QM_ROW);
                af[i][2] = lds_u32(p + 16);
                af[i][3] = lds_u32(p + 8 * QM_ROW + 16);
                da[i][0] = half_bits_to_float(lds_u16(sDA + (uint32_t)(i * 16 * 8 + b * 2)));
                da[i][1] = half_bits_to_float(lds_u16(sDA + (uint32_t)((i * 16 + 8) * 8 + b * 2)));
            }
#pragma unroll
            for (int j = 0; j < 4; ++j) {                     // weight rows 8 j + g (fragment), outputs 8 j + 2 t and + 1
                const uint32_t p = sB + (uint32_t)(j * 8 * QM_ROW + b * 32);
                bf[j][0] = lds_u32(p);
                bf[j][1] = lds_u32(p + 16);
                db[j][0] = half_bits_to_float(lds_u16(sDB + (uint32_t)(j * 8 * 8 + b * 2)));
                db[j][1] = half_bits_to_float(lds_u16(sDB + (uint32_t)((j * 8 + 1) * 8 + b * 2)));
            }
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    int s[4] = {0, 0, 0, 0};
                    mma_s8(s, af[i], bf[j]);
                    // sumf += (float)sumi * (d_w * d_x), the reference's operations in the reference's order
                    acc[i][j][0] = __fadd_rn(acc[i][j][0], __fmul_rn((float)s[0], __fmul_rn(db[j][0], da[i][0])));
                    acc[i][j][1] = __fadd_rn(acc[i][j][1], __fmul_rn((float)s[1], __fmul_rn(db[j][1], da[i][0])));
                    acc[i][j][2] = __fadd_rn(acc[i][j][2], __fmul_rn((float)s[2], __fmul_rn(db[j][0], da[i][1])));
                    acc[i][j][3] = __fadd_rn(acc[i][j][3], __fmul_rn((float)s[3], __fmul_rn(db[j][1], da[i][1])));
                }
        }
    }
    cp_async_wait<0>();
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int col = n0 + wn * 32 + j * 8 + 2 * t;
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                const int row = m0 + wm * 64 + i * 16 + g + 8 * h;
                if (row < M) {
                    if (col < N) C[(size_t)row * N + col] = acc[i][j][2 * h] + (bias ? bias[col] : 0.0f);
                    if (col + 1 < N) C[(size_t)row * N + col + 1] = acc[i][j][2 * h + 1] + (bias ? bias[col + 1] : 0.0f);
                }
            }
        }
}

}  // namespace ckb

using namespace ckb;

// A_planar [M rows], B_planar [N rows]: row-planar Q8_0 (ckb200_dev_q8_0_to_planar).  Returns -1 when the shape is not handled
// (K not a multiple of 128).
extern "C" int ckb_launch_gemm_q80_mma(const void *A_planar, const void *B_planar, const float *bias, float *C, int M, int N, int K, void *stream)
{
    if (K % (32 * QM_KB) || M <= 0 || N <= 0 || (((uintptr_t)A_planar | (uintptr_t)B_planar) & 15)) return -1;
    static int attr_set = 0;
    if (!attr_set) {
        if (ckb_check_cuda((int)cudaFuncSetAttribute(gemm_q80_mma_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, QM_SMEM), "gemm_q80_mma smem attr")) return CKB_ERR_CUDA;
        attr_set = 1;
    }
    const dim3 grid((N + QM_BN - 1) / QM_BN, (M + QM_BM - 1) / QM_BM);
    gemm_q80_mma_kernel<<<grid, QM_THREADS, QM_SMEM, ckb_stream(stream)>>>((const uint8_t *)A_planar, (const uint8_t *)B_planar, bias, C, M, N, K / 32);
    return ckb_check_launch("gemm_q80_mma");
}
