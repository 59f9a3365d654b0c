// Prefill / batched-decode GEMM on the 5th-generation tensor cores: C[M,N] = A_q8[M,K] . W[N,K]^T (+ bias), M >= 16,
// for Q4_K weights (the reference's block_q4_K rows) and Q6_K weights (row-planar layout, gemv_q6k_planar.cu).
// Replaces gemm_nt_q4_k_q8_k (src/kernels/gemm_kernels_q4k_q8k.c:301-326) and gemm_nt_q6_k_q8_k
// (src/kernels/gemm_kernels_q6k_q8k.c:1243-1268), which the reference computes as one GEMV per token.
//
// Exact-integer formulation.  For one 256-element Q4_K superblock b the reference adds
//     d_x[m,b] * ( d[n,b] * sum_j sc[n,j] * S[m,n,j]  -  dmin[n,b] * sum_j mn[n,j] * bsum[m,j] )
// where S are int32 sub-block dots (gemm_kernels_q4k_q8k.c:144-173).  Here
//     T [n,m] = sum_k (sc[n,k/32] * q4[n,k]) * q8[m,k]        256-deep f16 MMA, every operand an exact integer
//     T2[n,m] = sum_i  mn[n,i/2]  * bsum16[m,i]               16-deep f16 MMA (one k-step)
// are accumulated in fp32 in tensor memory (integers below 2^24 stay exact), read back with tcgen05.ld once per
// superblock and combined with the fp32 scales in registers: acc += d_x * (d * T - dmin * T2).
// Q6_K: A = (q6 - 32) * sc (src/kernels/gemm_kernels_q6k_q8k.c:86-116), the offset is inside the operand, so there
// is no T2; the product is an exact fp16 integer whenever |q6 - 32| * |sc| <= 2048 (always for |sc| <= 64), above
// that it is rounded to the nearest even integer (relative error <= 2^-12 on that element).
//
// Two kernels:
//  * gemm_x_tiles_kernel expands the Q8_K activations once into fp16 operand tiles in the exact shared-memory
//    layout of the MMA (K-major, no swizzle, 8 x 16-byte core matrices), one contiguous blob per (128-token tile,
//    superblock), so the GEMM fetches them with plain 1-D bulk copies.
//  * gemm_kq_tc_kernel<WF>: one CTA owns 128 weight rows (the M = 128 operand, one TMEM lane each) and one 128-token
//    tile (the N = 128 operand, TMEM columns; fewer tokens are zero-padded).  Warp-specialised, 20 warps:
//        warp 0       loader: bulk copies of activation k-stages (and of the bsum tile / block scales of each superblock)
//        warp 1       issuer: tcgen05.mma from one elected lane; tcgen05.commit frees stages and publishes accumulators
//        warps 4-11   two expander warpgroups: weights -> fp16 operand tiles, alternate k-stages (Q4_K) or halves (Q6_K)
//        warps 12-19  drain: tcgen05.ld of T|T2 (two TMEM buffers, 512 columns), fp32 sums in registers
//    One ring of 6 stages carries both operands of a 64-deep k-stage.  A stage has ONE "full" barrier (4 expander
//    warps + the loader's expect_tx arrival + the copy's bytes) and ONE "empty" barrier (a tcgen05.commit) that the
//    loader and the expanders both wait on: the issuer's timeline is a chain of barrier waits, MMA issues and commits
//    of roughly 100-180 cycles each, so every stage costs it one wait and one commit, not two of each.
// Every wait is bounded; a timeout sets the device error word, the CTA drains, frees TMEM and returns.
#include "quant_units.cuh"
#include "launch.h"
#include "pdl.cuh"
#include "runtime.h"

namespace ckb {

constexpr int TC_ROWS = 128;                          // rows of either operand per MMA
constexpr int TC_CHUNK = TC_ROWS * 16;                // one 8-element k-chunk of 128 rows: 2048 B
constexpr int TC_STAGE = 8 * TC_CHUNK;                // 64-deep k-stage of 128 rows: 16 KB
constexpr int TC_AUX = 2 * TC_CHUNK;                  // 16-deep tile (mins / bsums): 4 KB
constexpr int TC_STAGES = 6;                          // ring depth (a stage = weight tile + activation tile)
// activation blob of one (token tile, superblock): 4 k-stages, the bsum tile, 128 block scales
constexpr int TC_XBLOB_B2 = 4 * TC_STAGE;
constexpr int TC_XBLOB_DX = TC_XBLOB_B2 + TC_AUX;
constexpr int TC_XBLOB = TC_XBLOB_DX + TC_ROWS * 4;   // 70144 B, a multiple of 16

constexpr int TC_OFF_A = 0;                                           // weight tiles   [TC_STAGES][16 KB]
constexpr int TC_OFF_B = TC_OFF_A + TC_STAGES * TC_STAGE;             // activation tiles
constexpr int TC_OFF_A2 = TC_OFF_B + TC_STAGES * TC_STAGE;            // mins tiles     [2][4 KB]
constexpr int TC_OFF_B2 = TC_OFF_A2 + 2 * TC_AUX;                     // bsum tiles     [2][4 KB]
constexpr int TC_OFF_DX = TC_OFF_B2 + 2 * TC_AUX;                     // block scales   [2][128] fp32
constexpr int TC_OFF_BAR = TC_OFF_DX + 2 * TC_ROWS * 4;
enum { BAR_FULL = 0, BAR_EMPTY = TC_STAGES, BAR_A2_EMPTY = 2 * TC_STAGES, BAR_B2_EMPTY = BAR_A2_EMPTY + 2, BAR_DX_FULL = BAR_B2_EMPTY + 2,
       BAR_T_FULL = BAR_DX_FULL + 2, BAR_T_EMPTY = BAR_T_FULL + 2, BAR_COUNT = BAR_T_EMPTY + 2 };
constexpr int TC_SMEM = TC_OFF_BAR + BAR_COUNT * 8 + 16;

// shared-memory matrix descriptor: K-major, no swizzle; LBO = distance between the two 8-element k-chunks of
// one MMA (2048 B), SBO = distance between 8-row groups (128 B); version 1 (Blackwell)
__device__ __forceinline__ uint64_t tc_smem_desc(uint32_t addr)
{
    uint64_t d = 0;
    d |= (uint64_t)((addr & 0x3FFFFu) >> 4);
    d |= (uint64_t)(TC_CHUNK >> 4) << 16;
    d |= (uint64_t)(128 >> 4) << 32;
    d |= (uint64_t)1 << 46;
    return d;
}

// instruction descriptor: f16 x f16 -> f32, both operands K-major, M = 128, N = 128
constexpr uint32_t TC_IDESC = (1u << 4) | ((uint32_t)(TC_ROWS >> 3) << 17) | ((uint32_t)(TC_ROWS >> 4) << 24);

__device__ __forceinline__ void tc_mma(uint32_t tmem_d, uint64_t da, uint64_t db, uint32_t accumulate)
{
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, {%5, %5, %5, %5}, p;\n\t}"
        ::"r"(tmem_d), "l"(da), "l"(db), "r"(TC_IDESC), "r"(accumulate), "r"(0u));
}
__device__ __forceinline__ void tc_commit(uint32_t bar)
{
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
// One lane of a converged warp.
__device__ __forceinline__ bool tc_elect_one()
{
    uint32_t pred;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "elect.sync _|p, 0xffffffff;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(pred));
    return pred != 0;
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

__device__ __forceinline__ void tc_ld16(uint32_t taddr, uint32_t (&r)[16])
{
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]),
          "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
        : "r"(taddr));
}

// four unsigned bytes (each < 64) -> two half2 holding 1024 + byte: 0x6400 | b is the fp16 bit pattern of 1024 + b
__device__ __forceinline__ void bytes_to_half2_biased(uint32_t v, uint32_t &h01, uint32_t &h23)
{
    h01 = __byte_perm(v, 0x64646464u, 0x5140);
    h23 = __byte_perm(v, 0x64646464u, 0x7362);
}

// eight 4-bit values (two words of nibbles already masked to 0x0F0F0F0F) times an integer scale -> 8 fp16, exact:
// (1024 + q) * sc - 1024 * sc in one fused multiply-add per pair (only the result, at most 945, is rounded)
__device__ __forceinline__ uint4 q4_chunk_to_half(uint32_t w0, uint32_t w1, __half2 sc2, __half2 bias2)
{
    uint32_t h[4];
    bytes_to_half2_biased(w0, h[0], h[1]);
    bytes_to_half2_biased(w1, h[2], h[3]);
    uint4 out;
    uint32_t *o = reinterpret_cast<uint32_t *>(&out);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const __half2 r = __hfma2(*reinterpret_cast<__half2 *>(&h[i]), sc2, bias2);
        o[i] = *reinterpret_cast<const uint32_t *>(&r);
    }
    return out;
}

// eight int8 -> 8 fp16, exact: (x ^ 0x80) is x + 128 as an unsigned byte; 0x6400 | that is 1152 + x
__device__ __forceinline__ uint4 s8_chunk_to_half(uint32_t w0, uint32_t w1)
{
    uint32_t h[4];
    bytes_to_half2_biased(w0 ^ 0x80808080u, h[0], h[1]);
    bytes_to_half2_biased(w1 ^ 0x80808080u, h[2], h[3]);
    const __half2 off = __floats2half2_rn(1152.0f, 1152.0f);
    uint4 out;
    uint32_t *o = reinterpret_cast<uint32_t *>(&out);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const __half2 r = __hsub2(*reinterpret_cast<__half2 *>(&h[i]), off);
        o[i] = *reinterpret_cast<const uint32_t *>(&r);
    }
    return out;
}

__device__ __forceinline__ uint32_t tc_tile_offset(int row, int kchunk) { return (uint32_t)(kchunk * TC_CHUNK + (row >> 3) * 128 + (row & 7) * 16); }

// ---------------------------------------------------------------- activation tiles

// grid (superblocks, token tiles); consecutive threads take consecutive tokens of one k-chunk, so every warp
// writes 512 contiguous bytes of the blob
__global__ void __launch_bounds__(256) gemm_x_tiles_kernel(const uint8_t *__restrict__ A_q8, uint8_t *__restrict__ xt, int M, int nb)
{
    const int b = blockIdx.x, mt = blockIdx.y;
    uint8_t *blob = xt + ((size_t)mt * nb + b) * TC_XBLOB;
    for (int it = threadIdx.x; it < TC_ROWS * 32; it += 256) {
        const int t = it & (TC_ROWS - 1), kc = it >> 7, m = mt * TC_ROWS + t;
        uint32_t w0 = 0, w1 = 0;
        if (m < M) {
            const uint32_t *blk = reinterpret_cast<const uint32_t *>(A_q8 + ((size_t)m * nb + b) * Q8K_BYTES);
            w0 = __ldcg(blk + 1 + 2 * kc);
            w1 = __ldcg(blk + 2 + 2 * kc);
        }
        *reinterpret_cast<uint4 *>(blob + (kc >> 3) * TC_STAGE + tc_tile_offset(t, kc & 7)) = s8_chunk_to_half(w0, w1);
    }
    {
        const int t = threadIdx.x & (TC_ROWS - 1), g = threadIdx.x >> 7, m = mt * TC_ROWS + t;    // bsums[8g .. 8g+7], |bsum| <= 2048: exact
        uint32_t o[4] = {0u, 0u, 0u, 0u};
        float d = 0.0f;
        if (m < M) {
            const uint32_t *blk = reinterpret_cast<const uint32_t *>(A_q8 + ((size_t)m * nb + b) * Q8K_BYTES);
#pragma unroll
            for (int c = 0; c < 4; ++c) {
                const uint32_t v = __ldcg(blk + 65 + 4 * g + c);
                const __half2 h = __floats2half2_rn((float)(short)(v & 0xffffu), (float)(short)(v >> 16));
                o[c] = *reinterpret_cast<const uint32_t *>(&h);
            }
            d = __uint_as_float(__ldcg(blk));
        }
        *reinterpret_cast<uint4 *>(blob + TC_XBLOB_B2 + tc_tile_offset(t, g)) = make_uint4(o[0], o[1], o[2], o[3]);
        if (g == 0) reinterpret_cast<float *>(blob + TC_XBLOB_DX)[t] = d;
    }
}

// ---------------------------------------------------------------- GEMM

// Timeline of CTA (0,0), a tuning aid compiled out by default: TC_TRACE(role, slot) stores the SM clock.
#ifdef CKB_TC_TRACE
__device__ long long g_tc_trace[4][1024];
#define TC_TRACE(role, slot) do { if (blockIdx.x == 0 && blockIdx.y == 0 && (slot) < 1024) g_tc_trace[role][slot] = clock64(); } while (0)
#else
#define TC_TRACE(role, slot) do { } while (0)
#endif

enum { TC_W_Q4K = 0, TC_W_Q6K_PLANAR = 1 };       // weight operand formats

// Register counts per role after setmaxnreg.  setmaxnreg.inc blocks until the CTA's own pool (threads x registers at
// launch) can supply the registers, so 128 * (CTL + 2 * EXP + 2 * DRAIN) must not exceed 640 * LAUNCH; the launcher
// checks the compiled register count against LAUNCH before the first launch.
constexpr int TC_THREADS = 640, TC_REGS_LAUNCH = 96, TC_REGS_CTL = 32, TC_REGS_EXP = 72, TC_REGS_DRAIN = 152;
static_assert(128 * (TC_REGS_CTL + 2 * TC_REGS_EXP + 2 * TC_REGS_DRAIN) <= TC_THREADS * TC_REGS_LAUNCH, "setmaxnreg targets exceed the CTA's register pool");
static_assert(TC_THREADS * TC_REGS_LAUNCH <= 65536, "register plan");

template <int WF>
__global__ void __launch_bounds__(TC_THREADS, 1)
gemm_kq_tc_kernel(const uint8_t *__restrict__ xt, const uint8_t *__restrict__ B, const float *__restrict__ bias, float *__restrict__ C, int ldc, int M,
                  int N, int nb, int *__restrict__ dev_err)
{
    extern __shared__ __align__(128) uint8_t smem[];
    const uint32_t s_base = smem_u32(smem);
    const uint32_t sA = s_base + TC_OFF_A, sB = s_base + TC_OFF_B, sA2 = s_base + TC_OFF_A2, sB2 = s_base + TC_OFF_B2, sDX = s_base + TC_OFF_DX;
    const uint32_t sBar = s_base + TC_OFF_BAR;
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(smem + TC_OFF_BAR + BAR_COUNT * 8);
#define BAR(i) (sBar + 8u * (uint32_t)(i))

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int n0 = blockIdx.x * TC_ROWS, mt = blockIdx.y, m0 = mt * TC_ROWS;
    const uint32_t stages = (uint32_t)nb * 4u;

    if (tid == 0) {
        for (int i = 0; i < TC_STAGES; ++i) { mbar_init(BAR(BAR_FULL + i), 5); mbar_init(BAR(BAR_EMPTY + i), 1); }
        for (int i = 0; i < 2; ++i) {
            mbar_init(BAR(BAR_A2_EMPTY + i), 1);
            mbar_init(BAR(BAR_B2_EMPTY + i), 9);          // the T2 MMA (or, for Q6_K, the unit's last commit) and the 8 drain warps
            mbar_init(BAR(BAR_DX_FULL + i), 1);
            mbar_init(BAR(BAR_T_FULL + i), 1);
            mbar_init(BAR(BAR_T_EMPTY + i), 8);
        }
        mbar_fence_init();
    }
    if (warp == 0) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(512u));
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = *tmem_slot;                 // buffer u & 1 at column 256 * (u & 1): T at +0, T2 at +128

#define TC_SETMAXNREG(op, n) asm volatile("setmaxnreg." op ".sync.aligned.u32 %0;" ::"n"(n))
#define TC_WAIT(bar, parity, code)                                        \
    if (!mbar_wait_spin(bar, parity)) { atomicExch(dev_err, code); break; }

    if (warp < 4) {
        TC_SETMAXNREG("dec", TC_REGS_CTL);
        if (warp == 0) {
            // ------------------------------------------------------------ loader
            uint32_t issued = 0;
            for (uint32_t it = 0; it < stages; ++it) {
                const uint32_t b = it >> 2, s = it & 3u, i = it % TC_STAGES, x = b & 1u;
                const uint8_t *blob = xt + ((size_t)mt * nb + b) * TC_XBLOB;
                TC_WAIT(BAR(BAR_EMPTY + i), ((it / TC_STAGES) & 1u) ^ 1u, DEV_ERR_EMPTY_WAIT);
                if (s == 3) { TC_WAIT(BAR(BAR_B2_EMPTY + x), ((b >> 1) & 1u) ^ 1u, DEV_ERR_EMPTY_WAIT); }
                if (tc_elect_one()) {
                    // the bsum tile of the superblock rides on the barrier of its last k-stage (the issuer needs it for the T2 MMA
                    // right after that stage); the block scales have their own barrier, for the drain warps
                    const bool with_bsums = s == 3 && WF == TC_W_Q4K;
                    mbar_arrive_expect_tx(BAR(BAR_FULL + i), TC_STAGE + (with_bsums ? TC_AUX : 0));
                    bulk_g2s(sB + i * TC_STAGE, blob + s * TC_STAGE, TC_STAGE, BAR(BAR_FULL + i));
                    if (with_bsums) bulk_g2s(sB2 + x * TC_AUX, blob + TC_XBLOB_B2, TC_AUX, BAR(BAR_FULL + i));
                    if (s == 3) {
                        mbar_arrive_expect_tx(BAR(BAR_DX_FULL + x), TC_ROWS * 4);
                        bulk_g2s(sDX + x * TC_ROWS * 4, blob + TC_XBLOB_DX, TC_ROWS * 4, BAR(BAR_DX_FULL + x));
                    }
                }
                issued = it + 1;
            }
            if (issued < stages) {                     // gave up: copies still in flight must land before the CTA's shared memory goes away
                for (uint32_t c = issued > TC_STAGES ? issued - TC_STAGES : 0; c < issued; ++c)
                    mbar_wait_spin(BAR(BAR_FULL + c % TC_STAGES), (c / TC_STAGES) & 1u);
            }
        } else if (warp == 1) {
            // ------------------------------------------------------------ issuer: the warp runs the loop and the waits uniformly
            // (descriptors and addresses stay in uniform registers), one elected lane issues
            const uint64_t dA = tc_smem_desc(sA), dB = tc_smem_desc(sB), dA2 = tc_smem_desc(sA2), dB2 = tc_smem_desc(sB2);
            for (uint32_t it = 0; it < stages; ++it) {
                const uint32_t b = it >> 2, s = it & 3u, i = it % TC_STAGES, buf = b & 1u, tacc = tmem + 256u * buf;
                if (s == 0) {
                    TC_WAIT(BAR(BAR_T_EMPTY + buf), ((b >> 1) & 1u) ^ 1u, DEV_ERR_MMA_WAIT);
                    tc_fence_after();                  // orders the drain's tcgen05.ld of this buffer before the MMAs that overwrite it
                }
                if (lane == 0) TC_TRACE(0, 3 * it + 0);
                TC_WAIT(BAR(BAR_FULL + i), (it / TC_STAGES) & 1u, DEV_ERR_FULL_WAIT);
                if (lane == 0) TC_TRACE(0, 3 * it + 1);
                const uint64_t da = dA + (uint64_t)(i * (TC_STAGE >> 4)), db = dB + (uint64_t)(i * (TC_STAGE >> 4));
                if (tc_elect_one()) {
#pragma unroll
                    for (int k = 0; k < 4; ++k)
                        tc_mma(tacc, da + (uint64_t)(k * (2 * TC_CHUNK >> 4)), db + (uint64_t)(k * (2 * TC_CHUNK >> 4)), (s | (uint32_t)k) ? 1u : 0u);
                    tc_commit(BAR(BAR_EMPTY + i));
                    if (s == 3) {
                        if constexpr (WF == TC_W_Q4K) {
                            tc_mma(tacc + 128u, dA2 + (uint64_t)(buf * (TC_AUX >> 4)), dB2 + (uint64_t)(buf * (TC_AUX >> 4)), 0u);
                            tc_commit(BAR(BAR_A2_EMPTY + buf));
                        }
                        tc_commit(BAR(BAR_B2_EMPTY + buf));
                        tc_commit(BAR(BAR_T_FULL + buf));
                    }
                    TC_TRACE(0, 3 * it + 2);
                }
            }
        }
    } else if (warp < 12) {
        // ------------------------------------------------------------ weight expanders: thread = row
        TC_SETMAXNREG("dec", TC_REGS_EXP);
        const int set = (warp - 4) >> 2, row = tid & 127;
        if constexpr (WF == TC_W_Q6K_PLANAR) {
            // set e takes half n = e of every superblock: its 64 ql bytes and 32 qh bytes feed two k-stages
            const size_t rb = ((size_t)nb * Q6K_BYTES + 15) & ~(size_t)15;
            const uint8_t *wrow = B + (size_t)min(n0 + row, N - 1) * rb;
            const size_t off_qh = (size_t)nb * 128, off_sc = (size_t)nb * 192;
            const __half2 c66 = __floats2half2_rn(66.0f, 66.0f);
            bool go = true;
            for (uint32_t b = 0; b < (uint32_t)nb && go; ++b) {
                const uint32_t n = (uint32_t)set;
                uint4 ql[4], qh[2];
#pragma unroll
                for (int j = 0; j < 4; ++j) ql[j] = __ldg(reinterpret_cast<const uint4 *>(wrow + (size_t)b * 128 + 64 * n + 16 * j));
#pragma unroll
                for (int j = 0; j < 2; ++j) qh[j] = __ldg(reinterpret_cast<const uint4 *>(wrow + off_qh + (size_t)b * 64 + 32 * n + 16 * j));
                const uint2 sc8 = __ldg(reinterpret_cast<const uint2 *>(wrow + off_sc + (size_t)b * 16 + 8 * n));
                const uint32_t qlw[16] = {ql[0].x, ql[0].y, ql[0].z, ql[0].w, ql[1].x, ql[1].y, ql[1].z, ql[1].w,
                                          ql[2].x, ql[2].y, ql[2].z, ql[2].w, ql[3].x, ql[3].y, ql[3].z, ql[3].w};
                const uint32_t qhw[8] = {qh[0].x, qh[0].y, qh[0].z, qh[0].w, qh[1].x, qh[1].y, qh[1].z, qh[1].w};
#pragma unroll 1
                for (uint32_t hi = 0; hi < 2; ++hi) {
                    const uint32_t it = 4u * b + 2u * n + hi, i = it % TC_STAGES;
                    const uint32_t scw = hi ? sc8.y : sc8.x;       // scale groups 8n + 4hi + {0, 1, 2, 3}
                    if (!mbar_wait_spin(BAR(BAR_EMPTY + i), ((it / TC_STAGES) & 1u) ^ 1u)) { atomicExch(dev_err, DEV_ERR_EMPTY_WAIT); go = false; break; }
                    uint8_t *dst = smem + TC_OFF_A + i * TC_STAGE;
#pragma unroll
                    for (int c = 0; c < 8; ++c) {                  // chunk c: weights (c < 4 ? ql[l] : ql[32 + l]) with l = 8 (c & 3) .. + 7
                        const int sb = 2 * (c >> 2) + ((c & 3) >> 1);
                        const float scf = 16.0f * (float)(int)(int8_t)((scw >> (8 * sb)) & 255u);
                        const __half2 sc2 = __floats2half2_rn(scf, scf);
                        uint32_t o[4];
#pragma unroll
                        for (int w2 = 0; w2 < 2; ++w2) {
                            const uint32_t lw = qlw[8 * (c >> 2) + 2 * (c & 3) + w2], hw = qhw[2 * (c & 3) + w2];
                            const uint32_t nib = (lw >> (4u * hi)) & 0x0F0F0F0Fu;
                            const uint32_t two = ((hw >> (4u * hi + 2u * (uint32_t)(c >> 2))) << 4) & 0x30303030u;
                            // 0x5400 | q is the fp16 bit pattern of 64 + q / 16
                            uint32_t h01 = __byte_perm(nib | two, 0x54545454u, 0x5140), h23 = __byte_perm(nib | two, 0x54545454u, 0x7362);
                            const __half2 r0 = __hmul2(__hsub2(*reinterpret_cast<__half2 *>(&h01), c66), sc2);   // (q - 32) / 16 * 16 sc
                            const __half2 r1 = __hmul2(__hsub2(*reinterpret_cast<__half2 *>(&h23), c66), sc2);
                            o[2 * w2] = *reinterpret_cast<const uint32_t *>(&r0);
                            o[2 * w2 + 1] = *reinterpret_cast<const uint32_t *>(&r1);
                        }
                        *reinterpret_cast<uint4 *>(dst + tc_tile_offset(row, c)) = make_uint4(o[0], o[1], o[2], o[3]);
                    }
                    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");   // generic-proxy writes -> visible to the tensor core
                    __syncwarp();
                    if (lane == 0) mbar_arrive(BAR(BAR_FULL + i));
                }
            }
        } else {
            // set e takes the k-stages (quarters of a superblock) it = e, e + 2, ...
            const uint8_t *wrow = B + (size_t)min(n0 + row, N - 1) * nb * Q4K_BYTES;
            uint4 cur_a, cur_b, hdr;
            {
                const uint8_t *p0 = wrow + 16 + 32 * set;
                cur_a = __ldg(reinterpret_cast<const uint4 *>(p0));
                cur_b = __ldg(reinterpret_cast<const uint4 *>(p0 + 16));
                hdr = __ldg(reinterpret_cast<const uint4 *>(wrow));
            }
            for (uint32_t it = (uint32_t)set; it < stages; it += 2) {
                const uint32_t b = it >> 2, s = it & 3u, i = it % TC_STAGES, x2 = b & 1u;
                uint4 nxt_a = cur_a, nxt_b = cur_b, hdr_next = hdr;
                if (it + 2 < stages) {                    // this thread's next quarter, possibly of the next superblock
                    const uint8_t *pn = wrow + (size_t)((it + 2) >> 2) * Q4K_BYTES;
                    nxt_a = __ldg(reinterpret_cast<const uint4 *>(pn + 16 + 32 * ((it + 2) & 3u)));
                    nxt_b = __ldg(reinterpret_cast<const uint4 *>(pn + 32 + 32 * ((it + 2) & 3u)));
                    if (((it + 2) >> 2) != b) hdr_next = __ldg(reinterpret_cast<const uint4 *>(pn));
                }
                uint32_t sc2, m2;
                q4k_scales(hdr.y, hdr.z, hdr.w, (int)s, sc2, m2);
                const float sclo = (float)(sc2 & 255u), schi = (float)(sc2 >> 8);
                const __half2 s_lo = __floats2half2_rn(sclo, sclo), s_hi = __floats2half2_rn(schi, schi);
                const __half2 b_lo = __floats2half2_rn(-1024.0f * sclo, -1024.0f * sclo), b_hi = __floats2half2_rn(-1024.0f * schi, -1024.0f * schi);
                const float mlo = (float)(m2 & 255u), mhi = (float)(m2 >> 8);
                const __half2 mm_lo = __floats2half2_rn(mlo, mlo), mm_hi = __floats2half2_rn(mhi, mhi);
                if (tid == 128) TC_TRACE(1, 3 * (it >> 1) + 0);
                TC_WAIT(BAR(BAR_EMPTY + i), ((it / TC_STAGES) & 1u) ^ 1u, DEV_ERR_EMPTY_WAIT);
                if (s < 2) { TC_WAIT(BAR(BAR_A2_EMPTY + x2), ((b >> 1) & 1u) ^ 1u, DEV_ERR_EMPTY_WAIT); }   // this set's first write of the superblock's mins
                if (tid == 128) TC_TRACE(1, 3 * (it >> 1) + 1);
                const uint32_t ml = 0x0F0F0F0Fu;
                const uint32_t w[8] = {cur_a.x, cur_a.y, cur_a.z, cur_a.w, cur_b.x, cur_b.y, cur_b.z, cur_b.w};
                uint8_t *dst = smem + TC_OFF_A + i * TC_STAGE;
#pragma unroll
                for (int c = 0; c < 4; ++c) {     // low nibbles = sub-block 2s: k-chunks 0-3 of the stage; high nibbles = sub-block 2s+1: k-chunks 4-7
                    *reinterpret_cast<uint4 *>(dst + tc_tile_offset(row, c)) = q4_chunk_to_half(w[2 * c] & ml, w[2 * c + 1] & ml, s_lo, b_lo);
                    *reinterpret_cast<uint4 *>(dst + tc_tile_offset(row, 4 + c)) = q4_chunk_to_half((w[2 * c] >> 4) & ml, (w[2 * c + 1] >> 4) & ml, s_hi, b_hi);
                }
                // the two mins of this quarter, each doubled (bsums come per 16 elements): positions 4s .. 4s+3 of the 16-deep tile.  They
                // are written before this stage's arrival, and the T2 MMA is issued after the superblock's last stage: no barrier of their own.
                uint32_t *d2 = reinterpret_cast<uint32_t *>(smem + TC_OFF_A2 + x2 * TC_AUX + tc_tile_offset(row, (int)(s >> 1))) + 2 * (s & 1u);
                d2[0] = *reinterpret_cast<const uint32_t *>(&mm_lo);
                d2[1] = *reinterpret_cast<const uint32_t *>(&mm_hi);
                asm volatile("fence.proxy.async.shared::cta;" ::: "memory");   // generic-proxy writes -> visible to the tensor core
                __syncwarp();
                if (lane == 0) mbar_arrive(BAR(BAR_FULL + i));
                cur_a = nxt_a;
                cur_b = nxt_b;
                hdr = hdr_next;
                if (tid == 128) TC_TRACE(1, 3 * (it >> 1) + 2);
            }
        }
    } else {
        // ------------------------------------------------------------ accumulator drain: thread = TMEM lane (weight row), 64 token columns
        TC_SETMAXNREG("inc", TC_REGS_DRAIN);
        const int dw = warp - 12;
        const int q = dw & 3, ch = dw >> 2;           // warp % 4 is the TMEM lane quarter this warp may read (12 % 4 == 0)
        const int row = 32 * q + lane, n = n0 + row;
        constexpr size_t DSTRIDE = WF == TC_W_Q4K ? Q4K_BYTES : 2;        // bytes between the block scales of consecutive superblocks
        const uint8_t *wrow = WF == TC_W_Q4K ? B + (size_t)min(n, N - 1) * nb * Q4K_BYTES
                                             : B + (size_t)min(n, N - 1) * (((size_t)nb * Q6K_BYTES + 15) & ~(size_t)15) + (size_t)nb * 208;
        float acc[64];
#pragma unroll
        for (int i = 0; i < 64; ++i) acc[i] = 0.0f;
        auto load_dd = [&](int b) -> uint32_t {       // Q4_K: fp16 d | dmin of the superblock; Q6_K: fp16 d
            if constexpr (WF == TC_W_Q4K) return __ldg(reinterpret_cast<const uint32_t *>(wrow + (size_t)b * DSTRIDE));
            else return ldg_nc_u16(wrow + (size_t)b * DSTRIDE);
        };
        uint32_t dd_next = load_dd(0);
        int b = 0;
        for (; b < nb; ++b) {
            const uint32_t dd_bits = dd_next;
            if (b + 1 < nb) dd_next = load_dd(b + 1);
            const float2 dd = __half22float2(*reinterpret_cast<const __half2 *>(&dd_bits));
            const uint32_t buf = (uint32_t)b & 1u;
            const float4 *dxp = reinterpret_cast<const float4 *>(smem + TC_OFF_DX + buf * TC_ROWS * 4) + ch * 16;
            if (lane == 0 && dw == 0) TC_TRACE(2, 3 * b + 0);
            TC_WAIT(BAR(BAR_DX_FULL + buf), ((uint32_t)b >> 1) & 1u, DEV_ERR_FULL_WAIT);
            TC_WAIT(BAR(BAR_T_FULL + buf), ((uint32_t)b >> 1) & 1u, DEV_ERR_MMA_WAIT);
            if (lane == 0 && dw == 0) TC_TRACE(2, 3 * b + 1);
            tc_fence_after();
            const uint32_t taddr = tmem + ((uint32_t)(32 * q) << 16) + 256u * buf + 64u * (uint32_t)ch;
#pragma unroll
            for (int c = 0; c < 2; ++c) {             // two rounds of 32 columns
                uint32_t t1[2][16], t2[2][16];
#pragma unroll
                for (int j = 0; j < 2; ++j) {
                    tc_ld16(taddr + (uint32_t)(32 * c + 16 * j), t1[j]);
                    if constexpr (WF == TC_W_Q4K) tc_ld16(taddr + 128u + (uint32_t)(32 * c + 16 * j), t2[j]);
                }
                asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
                for (int j = 0; j < 2; ++j)
#pragma unroll
                    for (int i4 = 0; i4 < 4; ++i4) {
                        const float4 dx = dxp[(32 * c + 16 * j) / 4 + i4];
                        const float dxf[4] = {dx.x, dx.y, dx.z, dx.w};
#pragma unroll
                        for (int i = 0; i < 4; ++i) {
                            if constexpr (WF == TC_W_Q4K)
                                acc[32 * c + 16 * j + 4 * i4 + i] +=
                                    dxf[i] * (dd.x * __uint_as_float(t1[j][4 * i4 + i]) - dd.y * __uint_as_float(t2[j][4 * i4 + i]));
                            else
                                acc[32 * c + 16 * j + 4 * i4 + i] += (dxf[i] * dd.x) * __uint_as_float(t1[j][4 * i4 + i]);
                        }
                    }
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) {
                mbar_arrive(BAR(BAR_T_EMPTY + buf));
                mbar_arrive(BAR(BAR_B2_EMPTY + buf));
            }
            if (lane == 0 && dw == 0) TC_TRACE(2, 3 * b + 2);
        }
        if (b == nb && n < N) {
            const float bv = bias ? bias[n] : 0.0f;
#pragma unroll
            for (int i = 0; i < 64; ++i) {
                const int m = m0 + 64 * ch + i;
                if (m < M) C[(size_t)m * ldc + n] = acc[i] + bv;
            }
        }
    }
#undef TC_WAIT
#undef TC_SETMAXNREG
#undef BAR
    __syncwarp();
    tc_fence_before();
    __syncthreads();
    if (warp == 0) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(512u));
}

}  // namespace ckb

using namespace ckb;

template <int WF>
static int launch_tc(const uint8_t *xt, const void *B, const float *bias, float *C, int ldc, int M, int N, int nb, int mtiles, cudaStream_t st)
{
    static int attr_set = 0;
    if (!attr_set) {
        cudaFuncAttributes fa;
        if (ckb_check_cuda((int)cudaFuncGetAttributes(&fa, gemm_kq_tc_kernel<WF>), "func attributes")) return CKB_ERR_CUDA;
        if (fa.numRegs != TC_REGS_LAUNCH)     // a different allocation at launch would make setmaxnreg.inc wait for registers that never come
            return ckb_fail(CKB_ERR_LIMIT, "gemm_kq_tc: kernel compiled with an unexpected register count");
        if (ckb_check_cuda((int)cudaFuncSetAttribute(gemm_kq_tc_kernel<WF>, cudaFuncAttributeMaxDynamicSharedMemorySize, TC_SMEM), "smem attr")) return CKB_ERR_CUDA;
        attr_set = 1;
    }
    const dim3 grid((N + TC_ROWS - 1) / TC_ROWS, mtiles);
    gemm_kq_tc_kernel<WF><<<grid, TC_THREADS, TC_SMEM, st>>>(xt, (const uint8_t *)B, bias, C, ldc, M, N, nb, ckb_device_error_word());
    return ckb_check_launch("gemm_kq_tc");
}

#ifdef CKB_TC_TRACE
extern "C" int ckb200_tc_trace(long long *out4096) { return (int)cudaMemcpyFromSymbol(out4096, g_tc_trace, sizeof(long long) * 4096); }
#endif

// C[m * ldc + n] = A_q8[m] . W[n] (+ bias[n]).  wf: TC_W_Q4K (the reference's block_q4_K rows) or TC_W_Q6K_PLANAR.
// Returns -1 when the shape is not handled here (caller falls back to the per-token path).  min_tokens: smallest M
// worth the tensor-core path (the token tile is 128 wide; fewer tokens are padded with zeros).
extern "C" int ckb_launch_gemm_tc(int wf, const void *A_q8, const void *B, const float *bias, float *C, int ldc, int M, int N, int K, int min_tokens,
                                  void *stream)
{
    if (M < min_tokens || K % QK_K || ((uintptr_t)B & 15) || ((uintptr_t)A_q8 & 3) || ckb_tune_get("gemm_tc", 1) == 0) return -1;
    const int nb = K / QK_K, mtiles = (M + TC_ROWS - 1) / TC_ROWS;
    uint8_t *xt = (uint8_t *)ckb_scratch(CKB_SLOT_G, (size_t)mtiles * nb * TC_XBLOB);
    if (!xt) return CKB_ERR_CUDA;
    cudaStream_t st = ckb_stream(stream);
    gemm_x_tiles_kernel<<<dim3(nb, mtiles), 256, 0, st>>>((const uint8_t *)A_q8, xt, M, nb);
    if (int rc = ckb_check_launch("gemm_x_tiles")) return rc;
    return wf == TC_W_Q6K_PLANAR ? launch_tc<TC_W_Q6K_PLANAR>(xt, B, bias, C, ldc, M, N, nb, mtiles, st)
                                 : launch_tc<TC_W_Q4K>(xt, B, bias, C, ldc, M, N, nb, mtiles, st);
}

extern "C" int ckb_launch_gemm_q4k_tc(const void *A_q8, const void *B, const float *bias, float *C, int M, int N, int K, void *stream)
{
    return ckb_launch_gemm_tc(TC_W_Q4K, A_q8, B, bias, C, N, M, N, K, ckb_tune_get("gemm_tc_min_tokens", 16), stream);
}

// gemm_nt_q6_k_q8_k (src/kernels/gemm_kernels_q6k_q8k.c:1243-1268) over weights in the row-planar layout
extern "C" int ckb200_dev_gemv_q6_k_planar_q8_k(float *, const void *, const void *, int, int, void *);
extern "C" int ckb200_dev_add_bias_rows(float *, const float *, int, int, void *);
extern "C" int ckb200_dev_gemm_nt_q6_k_planar_q8_k(const void *A_q8, const void *B_planar, const float *bias, float *C, int M, int N, int K, void *stream)
{
    if (!A_q8 || !B_planar || !C || M <= 0 || N <= 0 || K <= 0) return 0;
    if (ckb_ensure_init()) return CKB_ERR_NO_DEVICE;
    const int rc = ckb_launch_gemm_tc(TC_W_Q6K_PLANAR, A_q8, B_planar, bias, C, N, M, N, K, ckb_tune_get("gemm_tc_min_tokens", 16), stream);
    if (rc >= 0) return rc;
    for (int m = 0; m < M; ++m) {
        const int r2 = ckb200_dev_gemv_q6_k_planar_q8_k(C + (size_t)m * N, B_planar, (const uint8_t *)A_q8 + (size_t)m * (K / QK_K) * Q8K_BYTES, N, K, stream);
        if (r2) return r2;
    }
    return bias ? ckb200_dev_add_bias_rows(C, bias, M, N, stream) : 0;
}
