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
//
// Measured and not kept (each correct, each 3-8 % slower than this form): 128-deep ring stages (eight MMAs per barrier round), weight
// bytes loaded a superblock ahead into two register sets with an L2 prefetch (the expanders no longer wait for loads), two issuer
// warps on alternate superblocks (one accumulator buffer each).  The roles are co-limited: issuer chain, expanders, drain and the
// shared-memory data pipe (63 % busy: operand reads by the tensor core, tile writes, bulk copies) each need about a thousand cycles
// per 128-deep step, and they share four schedulers, so relieving one of them moves the wait to the next.
#include "quant_units.cuh"
#include "launch.h"
#include "pdl.cuh"
#include "runtime.h"

namespace ckb {

constexpr int TC_ROWS = 128;                          // rows of either operand per MMA
constexpr int TC_CHUNK = TC_ROWS * 16;                // one 8-element k-chunk of 128 rows: 2048 B
constexpr int TC_STAGE = 8 * TC_CHUNK;                // 64-deep k-stage of 128 rows: 16 KB
constexpr int TC_AUX = 2 * TC_CHUNK;                  // 16-deep tile (mins / bsums): 4 KB

// Everything that depends on the width NT of the token tile (the N operand of the MMA).  NT = 128 is the prefill
// shape: one CTA of 640 threads per SM.  NT = 32 is the batched-decode shape (up to 64 tokens): the activation tiles,
// the drain and the accumulators shrink so far that two CTAs of 512 threads share an SM, and every latency of the
// per-stage chain (weight loads, barrier waits, MMA issue, commit) is overlapped by the neighbour.
template <int NT>
struct TcCfg {
    static constexpr int STAGES = NT == 128 ? 6 : 5;          // ring depth (a stage = weight tile + activation tile)
    static constexpr int B_CHUNK = NT * 16;                   // one 8-element k-chunk of NT tokens
    static constexpr int B_STAGE = 8 * B_CHUNK;               // 64-deep k-stage of NT tokens
    static constexpr int B_AUX = 2 * B_CHUNK;                 // 16-deep bsum tile
    // activation blob of one (token tile, superblock): 4 k-stages, the bsum tile, NT block scales
    static constexpr int XBLOB_B2 = 4 * B_STAGE, XBLOB_DX = XBLOB_B2 + B_AUX, XBLOB = XBLOB_DX + NT * 4;   // a multiple of 16
    static constexpr int OFF_A = 0;                                      // weight tiles   [STAGES][16 KB]
    static constexpr int OFF_B = OFF_A + STAGES * TC_STAGE;              // activation tiles
    static constexpr int OFF_A2 = OFF_B + STAGES * B_STAGE;              // mins tiles     [2][4 KB]
    static constexpr int OFF_B2 = OFF_A2 + 2 * TC_AUX;                   // bsum tiles     [2]
    static constexpr int OFF_DX = OFF_B2 + 2 * B_AUX;                    // block scales   [2][NT] fp32
    static constexpr int OFF_BAR = OFF_DX + 2 * NT * 4;
    static constexpr int BAR_FULL = 0, BAR_EMPTY = STAGES, BAR_A2_EMPTY = 2 * STAGES, BAR_B2_EMPTY = BAR_A2_EMPTY + 2, BAR_DX_FULL = BAR_B2_EMPTY + 2,
                         BAR_T_FULL = BAR_DX_FULL + 2, BAR_T_EMPTY = BAR_T_FULL + 2, BAR_COUNT = BAR_T_EMPTY + 2;
    static constexpr int SMEM = OFF_BAR + BAR_COUNT * 8 + 16;
    static constexpr int DRAIN_WARPS = NT == 128 ? 8 : 4;     // 4 TMEM lane quarters x column halves
    static constexpr int DRAIN_COLS = NT / (DRAIN_WARPS / 4); // token columns per drain thread
    static constexpr int THREADS = (12 + DRAIN_WARPS) * 32, CTAS_PER_SM = NT == 128 ? 1 : 2;
    // Register counts per role after setmaxnreg.  setmaxnreg.inc blocks until the CTA's own pool (threads x registers
    // at launch) can supply the registers, so 128 * CTL + 256 * EXP + 32 * DRAIN_WARPS * DRAIN must not exceed
    // THREADS * LAUNCH; the launcher checks the compiled register count against LAUNCH before the first launch.
    static constexpr int REGS_LAUNCH = NT == 128 ? 96 : 64, REGS_CTL = 32, REGS_EXP = 72, REGS_DRAIN = NT == 128 ? 152 : 80;
    static_assert(128 * REGS_CTL + 256 * REGS_EXP + 32 * DRAIN_WARPS * REGS_DRAIN <= THREADS * REGS_LAUNCH, "setmaxnreg targets exceed the CTA's register pool");
    static_assert(THREADS * REGS_LAUNCH * CTAS_PER_SM <= 65536, "register plan");
    static constexpr uint32_t TMEM_COLS = NT == 128 ? 512 : 128, T_BUF = TMEM_COLS / 2, T2_OFF = NT;   // buffer u & 1 at column T_BUF * (u & 1): T at +0, T2 at +NT
    // instruction descriptor: f16 x f16 -> f32, both operands K-major, M = 128, N = NT
    static constexpr uint32_t IDESC = (1u << 4) | ((uint32_t)(NT >> 3) << 17) | ((uint32_t)(TC_ROWS >> 4) << 24);
    static_assert(CTAS_PER_SM * (SMEM + 1024) <= 228 * 1024 && SMEM <= 227 * 1024, "shared memory plan");
};

// shared-memory matrix descriptor: K-major, no swizzle; LBO = distance between the two 8-element k-chunks of
// one MMA (rows x 16 B), SBO = distance between 8-row groups (128 B); version 1 (Blackwell)
__device__ __forceinline__ uint64_t tc_smem_desc(uint32_t addr, uint32_t chunk_bytes)
{
    uint64_t d = 0;
    d |= (uint64_t)((addr & 0x3FFFFu) >> 4);
    d |= (uint64_t)(chunk_bytes >> 4) << 16;
    d |= (uint64_t)(128 >> 4) << 32;
    d |= (uint64_t)1 << 46;
    return d;
}

__device__ __forceinline__ void tc_mma(uint32_t tmem_d, uint64_t da, uint64_t db, uint32_t idesc, uint32_t accumulate)
{
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, {%5, %5, %5, %5}, p;\n\t}"
        ::"r"(tmem_d), "l"(da), "l"(db), "r"(idesc), "r"(accumulate), "r"(0u));
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
template <int NT>
__device__ __forceinline__ uint32_t tc_xtile_offset(int tok, int kchunk) { return (uint32_t)(kchunk * TcCfg<NT>::B_CHUNK + (tok >> 3) * 128 + (tok & 7) * 16); }

// ---------------------------------------------------------------- activation tiles

// grid (superblocks, token tiles, parts of the 32 k-chunks).  The quants of a token's block are read as they lie (consecutive
// threads, consecutive words) into shared memory and leave it token-major: consecutive threads take consecutive tokens of one
// k-chunk, so every warp writes 512 contiguous bytes of the blob.  (Reading token-major straight from global memory fetched a
// 32-byte sector per 8 bytes used and took 12 us for 512 tokens of 4096 elements.)
template <int NT>
__global__ void __launch_bounds__(256) gemm_x_tiles_kernel(const uint8_t *__restrict__ A_q8, uint8_t *__restrict__ xt, int M, int nb)
{
    using Cfg = TcCfg<NT>;
    constexpr int PITCH = 66;                                  // words per token in shared memory: 64 + 2, 8-byte reads two-way at worst
    __shared__ __align__(8) uint32_t q[NT * PITCH];
    const int b = blockIdx.x, mt = blockIdx.y;
    const int kcz = 32 / (int)gridDim.z, kc0 = (int)blockIdx.z * kcz;     // this CTA's k-chunks [kc0, kc0 + kcz)
    uint8_t *blob = xt + ((size_t)mt * nb + b) * Cfg::XBLOB;
    for (int it = threadIdx.x; it < NT * kcz * 2; it += 256) {
        const int t = it / (2 * kcz), w = it - t * (2 * kcz), m = mt * NT + t;
        uint32_t v = 0;
        if (m < M) v = __ldcg(reinterpret_cast<const uint32_t *>(A_q8 + ((size_t)m * nb + b) * Q8K_BYTES) + 1 + 2 * kc0 + w);
        q[t * PITCH + w] = v;
    }
    __syncthreads();
    for (int it = threadIdx.x; it < NT * kcz; it += 256) {
        const int t = it % NT, kl = it / NT, kc = kc0 + kl;
        const uint2 w = *reinterpret_cast<const uint2 *>(&q[t * PITCH + 2 * kl]);
        *reinterpret_cast<uint4 *>(blob + (kc >> 3) * Cfg::B_STAGE + tc_xtile_offset<NT>(t, kc & 7)) = s8_chunk_to_half(w.x, w.y);
    }
    if (blockIdx.z != 0) return;
    if (threadIdx.x < 2 * NT) {
        const int t = threadIdx.x % NT, g = threadIdx.x / NT, m = mt * NT + t;    // bsums[8g .. 8g+7], |bsum| <= 2048: exact
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
        *reinterpret_cast<uint4 *>(blob + Cfg::XBLOB_B2 + tc_xtile_offset<NT>(t, g)) = make_uint4(o[0], o[1], o[2], o[3]);
        if (g == 0) reinterpret_cast<float *>(blob + Cfg::XBLOB_DX)[t] = d;
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

// Split K: blockIdx.z takes the superblocks [z * nbz, z * nbz + nbz) and writes its partial sums to C + z * cz
// (the launcher adds the slices up in a fixed order); a single slice writes C itself, bias included.
template <int WF, int NT>
__global__ void __launch_bounds__(TcCfg<NT>::THREADS, TcCfg<NT>::CTAS_PER_SM)
gemm_kq_tc_kernel(const uint8_t *__restrict__ xt, const uint8_t *__restrict__ B, const float *__restrict__ bias, float *__restrict__ C, int ldc, size_t cz,
                  int M, int N, int nb_row, int nbz, int *__restrict__ dev_err)
{
    using Cfg = TcCfg<NT>;
    constexpr int TC_STAGES = Cfg::STAGES, BAR_FULL = Cfg::BAR_FULL, BAR_EMPTY = Cfg::BAR_EMPTY, BAR_A2_EMPTY = Cfg::BAR_A2_EMPTY, BAR_B2_EMPTY = Cfg::BAR_B2_EMPTY,
                  BAR_DX_FULL = Cfg::BAR_DX_FULL, BAR_T_FULL = Cfg::BAR_T_FULL, BAR_T_EMPTY = Cfg::BAR_T_EMPTY;
    constexpr int TC_OFF_A = Cfg::OFF_A, TC_OFF_A2 = Cfg::OFF_A2, TC_OFF_DX = Cfg::OFF_DX;
    const int kb0 = blockIdx.z * nbz, nb = min(nbz, nb_row - kb0);         // this slice: superblocks kb0 .. kb0 + nb of rows that hold nb_row
    extern __shared__ __align__(128) uint8_t smem[];
    const uint32_t s_base = smem_u32(smem);
    const uint32_t sA = s_base + Cfg::OFF_A, sB = s_base + Cfg::OFF_B, sA2 = s_base + Cfg::OFF_A2, sB2 = s_base + Cfg::OFF_B2, sDX = s_base + Cfg::OFF_DX;
    const uint32_t sBar = s_base + Cfg::OFF_BAR;
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(smem + Cfg::OFF_BAR + Cfg::BAR_COUNT * 8);
#define BAR(i) (sBar + 8u * (uint32_t)(i))

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int n0 = blockIdx.x * TC_ROWS, mt = blockIdx.y, m0 = mt * NT;
    const uint32_t stages = (uint32_t)nb * 4u;

    if (tid == 0) {
        for (int i = 0; i < TC_STAGES; ++i) { mbar_init(BAR(BAR_FULL + i), 5); mbar_init(BAR(BAR_EMPTY + i), 1); }
        for (int i = 0; i < 2; ++i) {
            mbar_init(BAR(BAR_A2_EMPTY + i), 1);
            mbar_init(BAR(BAR_B2_EMPTY + i), 1 + Cfg::DRAIN_WARPS);   // the T2 MMA (or, for Q6_K, the unit's last commit) and the drain warps
            mbar_init(BAR(BAR_DX_FULL + i), 1);
            mbar_init(BAR(BAR_T_FULL + i), 1);
            mbar_init(BAR(BAR_T_EMPTY + i), Cfg::DRAIN_WARPS);
        }
        mbar_fence_init();
    }
    if (warp == 0) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(Cfg::TMEM_COLS));
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = *tmem_slot;

#define TC_SETMAXNREG(op, n) asm volatile("setmaxnreg." op ".sync.aligned.u32 %0;" ::"n"(n))
#define TC_WAIT(bar, parity, code)                                        \
    if (!mbar_wait_spin(bar, parity)) { atomicExch(dev_err, code); break; }

    if (warp < 4) {
        TC_SETMAXNREG("dec", Cfg::REGS_CTL);
        if (warp == 0) {
            // ------------------------------------------------------------ loader
            uint32_t issued = 0;
            for (uint32_t it = 0; it < stages; ++it) {
                const uint32_t b = it >> 2, s = it & 3u, i = it % TC_STAGES, x = b & 1u;
                const uint8_t *blob = xt + ((size_t)mt * nb_row + kb0 + b) * Cfg::XBLOB;
                TC_WAIT(BAR(BAR_EMPTY + i), ((it / TC_STAGES) & 1u) ^ 1u, DEV_ERR_EMPTY_WAIT);
                if (s == 3) { TC_WAIT(BAR(BAR_B2_EMPTY + x), ((b >> 1) & 1u) ^ 1u, DEV_ERR_EMPTY_WAIT); }
                if (tc_elect_one()) {
                    // the bsum tile of the superblock rides on the barrier of its last k-stage (the issuer needs it for the T2 MMA
                    // right after that stage); the block scales have their own barrier, for the drain warps
                    const bool with_bsums = s == 3 && WF == TC_W_Q4K;
                    mbar_arrive_expect_tx(BAR(BAR_FULL + i), Cfg::B_STAGE + (with_bsums ? Cfg::B_AUX : 0));
                    bulk_g2s(sB + i * Cfg::B_STAGE, blob + s * Cfg::B_STAGE, Cfg::B_STAGE, BAR(BAR_FULL + i));
                    if (with_bsums) bulk_g2s(sB2 + x * Cfg::B_AUX, blob + Cfg::XBLOB_B2, Cfg::B_AUX, BAR(BAR_FULL + i));
                    if (s == 3) {
                        mbar_arrive_expect_tx(BAR(BAR_DX_FULL + x), NT * 4);
                        bulk_g2s(sDX + x * NT * 4, blob + Cfg::XBLOB_DX, NT * 4, BAR(BAR_DX_FULL + x));
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
            const uint64_t dA = tc_smem_desc(sA, TC_CHUNK), dB = tc_smem_desc(sB, Cfg::B_CHUNK), dA2 = tc_smem_desc(sA2, TC_CHUNK), dB2 = tc_smem_desc(sB2, Cfg::B_CHUNK);
            for (uint32_t it = 0; it < stages; ++it) {
                const uint32_t b = it >> 2, s = it & 3u, i = it % TC_STAGES, buf = b & 1u, tacc = tmem + Cfg::T_BUF * buf;
                if (s == 0) {
                    TC_WAIT(BAR(BAR_T_EMPTY + buf), ((b >> 1) & 1u) ^ 1u, DEV_ERR_MMA_WAIT);
                    tc_fence_after();                  // orders the drain's tcgen05.ld of this buffer before the MMAs that overwrite it
                }
                if (lane == 0) TC_TRACE(0, 3 * it + 0);
                TC_WAIT(BAR(BAR_FULL + i), (it / TC_STAGES) & 1u, DEV_ERR_FULL_WAIT);
                if (lane == 0) TC_TRACE(0, 3 * it + 1);
                const uint64_t da = dA + (uint64_t)(i * (TC_STAGE >> 4)), db = dB + (uint64_t)(i * (Cfg::B_STAGE >> 4));
                if (tc_elect_one()) {
#pragma unroll
                    for (int k = 0; k < 4; ++k)
                        tc_mma(tacc, da + (uint64_t)(k * (2 * TC_CHUNK >> 4)), db + (uint64_t)(k * (2 * Cfg::B_CHUNK >> 4)), Cfg::IDESC, (s | (uint32_t)k) ? 1u : 0u);
                    tc_commit(BAR(BAR_EMPTY + i));
                    if (s == 3) {
                        if constexpr (WF == TC_W_Q4K) {
                            tc_mma(tacc + Cfg::T2_OFF, dA2 + (uint64_t)(buf * (TC_AUX >> 4)), dB2 + (uint64_t)(buf * (Cfg::B_AUX >> 4)), Cfg::IDESC, 0u);
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
        if constexpr (Cfg::REGS_EXP < Cfg::REGS_LAUNCH) TC_SETMAXNREG("dec", Cfg::REGS_EXP);
        else TC_SETMAXNREG("inc", Cfg::REGS_EXP);
        const int set = (warp - 4) >> 2, row = tid & 127;
        if constexpr (WF == TC_W_Q6K_PLANAR) {
            // set e takes half n = e of every superblock: its 64 ql bytes and 32 qh bytes feed two k-stages
            const size_t rb = ((size_t)nb_row * Q6K_BYTES + 15) & ~(size_t)15;
            const uint8_t *wrow = B + (size_t)min(n0 + row, N - 1) * rb;
            const size_t off_qh = (size_t)nb_row * 128, off_sc = (size_t)nb_row * 192;
            const __half2 c66 = __floats2half2_rn(66.0f, 66.0f);
            bool go = true;
            for (uint32_t b = 0; b < (uint32_t)nb && go; ++b) {
                const uint32_t n = (uint32_t)set;
                uint4 ql[4], qh[2];
#pragma unroll
                for (int j = 0; j < 4; ++j) ql[j] = __ldg(reinterpret_cast<const uint4 *>(wrow + (size_t)(kb0 + b) * 128 + 64 * n + 16 * j));
#pragma unroll
                for (int j = 0; j < 2; ++j) qh[j] = __ldg(reinterpret_cast<const uint4 *>(wrow + off_qh + (size_t)(kb0 + b) * 64 + 32 * n + 16 * j));
                const uint2 sc8 = __ldg(reinterpret_cast<const uint2 *>(wrow + off_sc + (size_t)(kb0 + b) * 16 + 8 * n));
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
            const uint8_t *wrow = B + ((size_t)min(n0 + row, N - 1) * nb_row + kb0) * Q4K_BYTES;
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
        TC_SETMAXNREG("inc", Cfg::REGS_DRAIN);
        constexpr int COLS = Cfg::DRAIN_COLS;         // token columns of this thread
        const int dw = warp - 12;
        const int q = dw & 3, ch = dw >> 2;           // warp % 4 is the TMEM lane quarter this warp may read (12 % 4 == 0)
        const int row = 32 * q + lane, n = n0 + row;
        constexpr size_t DSTRIDE = WF == TC_W_Q4K ? Q4K_BYTES : 2;        // bytes between the block scales of consecutive superblocks
        const uint8_t *wrow = WF == TC_W_Q4K ? B + ((size_t)min(n, N - 1) * nb_row + kb0) * Q4K_BYTES
                                             : B + (size_t)min(n, N - 1) * (((size_t)nb_row * Q6K_BYTES + 15) & ~(size_t)15) + (size_t)nb_row * 208 + (size_t)kb0 * 2;
        float acc[COLS];
#pragma unroll
        for (int i = 0; i < COLS; ++i) acc[i] = 0.0f;
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
            const float4 *dxp = reinterpret_cast<const float4 *>(smem + TC_OFF_DX + buf * NT * 4) + ch * (COLS / 4);
            if (lane == 0 && dw == 0) TC_TRACE(2, 3 * b + 0);
            TC_WAIT(BAR(BAR_DX_FULL + buf), ((uint32_t)b >> 1) & 1u, DEV_ERR_FULL_WAIT);
            TC_WAIT(BAR(BAR_T_FULL + buf), ((uint32_t)b >> 1) & 1u, DEV_ERR_MMA_WAIT);
            if (lane == 0 && dw == 0) TC_TRACE(2, 3 * b + 1);
            tc_fence_after();
            const uint32_t taddr = tmem + ((uint32_t)(32 * q) << 16) + Cfg::T_BUF * buf + (uint32_t)(COLS * ch);
            constexpr int RJ = NT == 128 ? 2 : 1;     // 16-column loads in flight per round (registers: 16 or 32 per accumulator)
#pragma unroll
            for (int c = 0; c < COLS / (16 * RJ); ++c) {
                uint32_t t1[RJ][16], t2[RJ][16];
#pragma unroll
                for (int j = 0; j < RJ; ++j) {
                    tc_ld16(taddr + (uint32_t)(16 * (RJ * c + j)), t1[j]);
                    if constexpr (WF == TC_W_Q4K) tc_ld16(taddr + Cfg::T2_OFF + (uint32_t)(16 * (RJ * c + j)), t2[j]);
                }
                asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
                for (int j = 0; j < RJ; ++j)
#pragma unroll
                    for (int i4 = 0; i4 < 4; ++i4) {
                        const float4 dx = dxp[4 * (RJ * c + j) + i4];
                        const float dxf[4] = {dx.x, dx.y, dx.z, dx.w};
#pragma unroll
                        for (int i = 0; i < 4; ++i) {
                            if constexpr (WF == TC_W_Q4K)
                                acc[16 * (RJ * c + j) + 4 * i4 + i] +=
                                    dxf[i] * (dd.x * __uint_as_float(t1[j][4 * i4 + i]) - dd.y * __uint_as_float(t2[j][4 * i4 + i]));
                            else
                                acc[16 * (RJ * c + j) + 4 * i4 + i] += (dxf[i] * dd.x) * __uint_as_float(t1[j][4 * i4 + i]);
                        }
                    }
            }
            // Every lane has read block scales from shared memory with plain loads, and lane 0's arrival below tells the loader that
            // the buffer may be overwritten (by a bulk copy, which neither the compiler nor the warp barrier knows about).  The fence
            // makes each lane's loads complete before the warp barrier, so that none of them can still be in flight when the copy
            // lands.  Without it a pipeline that is not starved elsewhere corrupts a few 4-token groups of a 32-row quarter per call.
            __threadfence_block();
            tc_fence_before();
            __syncwarp();
            if (lane == 0) {
                mbar_arrive(BAR(BAR_T_EMPTY + buf));
                mbar_arrive(BAR(BAR_B2_EMPTY + buf));
            }
            if (lane == 0 && dw == 0) TC_TRACE(2, 3 * b + 2);
        }
        if (b == nb && n < N) {
            const float bv = bias && gridDim.z == 1 ? bias[n] : 0.0f;
            float *Cz = C + (size_t)blockIdx.z * cz;
#pragma unroll
            for (int i = 0; i < COLS; ++i) {
                const int m = m0 + COLS * ch + i;
                if (m < M) Cz[(size_t)m * ldc + n] = acc[i] + bv;
            }
        }
    }
#undef TC_WAIT
#undef TC_SETMAXNREG
#undef BAR
    __syncwarp();
    tc_fence_before();
    __syncthreads();
    if (warp == 0) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(Cfg::TMEM_COLS));
}

// sum of the split-K slices in slice order, plus bias: C[m * ldc + n] = sum_z part[z][m][n] + bias[n]
template <bool VEC>
__global__ void __launch_bounds__(256) gemm_splitk_sum_kernel(const float *__restrict__ part, int Z, const float *__restrict__ bias, float *__restrict__ C, int ldc,
                                                              int M, int N)
{
    const size_t mn = (size_t)M * N;
    if (VEC) {                                                 // N and ldc multiples of 4, C and bias 16-byte aligned: four outputs per thread
        for (size_t i = ((size_t)blockIdx.x * 256 + threadIdx.x) * 4; i < mn; i += (size_t)gridDim.x * 1024) {
            const int m = (int)(i / N), n = (int)(i - (size_t)m * N);
            float4 s = __ldcg(reinterpret_cast<const float4 *>(part + i));
            for (int z = 1; z < Z; ++z) {                      // slices in a fixed order
                const float4 v = __ldcg(reinterpret_cast<const float4 *>(part + (size_t)z * mn + i));
                s.x += v.x; s.y += v.y; s.z += v.z; s.w += v.w;
            }
            if (bias) {
                const float4 b = *reinterpret_cast<const float4 *>(bias + n);
                s.x += b.x; s.y += b.y; s.z += b.z; s.w += b.w;
            } else {
                s.x += 0.0f; s.y += 0.0f; s.z += 0.0f; s.w += 0.0f;
            }
            *reinterpret_cast<float4 *>(C + (size_t)m * ldc + n) = s;
        }
        return;
    }
    for (size_t i = (size_t)blockIdx.x * 256 + threadIdx.x; i < mn; i += (size_t)gridDim.x * 256) {
        const int m = (int)(i / N), n = (int)(i - (size_t)m * N);
        float s = __ldcg(part + i);
        for (int z = 1; z < Z; ++z) s += __ldcg(part + (size_t)z * mn + i);
        C[(size_t)m * ldc + n] = s + (bias ? bias[n] : 0.0f);
    }
}

}  // namespace ckb

using namespace ckb;

// How many K slices: enough CTAs to fill the resident slots (SMs x CTAs per SM) in whole waves.  Few tokens only (the
// partial sums cost Z * M * N * 4 bytes of traffic), slices of at least 4 superblocks, at most 16.
static int tc_pick_slices(int tiles, int nb, int slots)
{
    int best = 1;
    double best_eff = 0.0;
    for (int z = 1; z <= 16 && nb / z >= 4; ++z) {
        const long ctas = (long)tiles * z, waves = (ctas + slots - 1) / slots;
        const double eff = (double)ctas / (double)(waves * slots);
        if (eff > best_eff * 1.08) { best_eff = eff; best = z; }      // a larger Z must pay for its partial sums
    }
    return best;
}

// The operand tiles that the last launch made, and the caller's promise that the activations behind them have not changed.
static struct { const void *a; int M, nb, nt; const uint8_t *xt; cudaStream_t st; } g_tc_tiles = {nullptr, 0, 0, 0, nullptr, nullptr};
static int g_tc_same_activations = 0;
extern "C" void ckb_gemm_tc_hint_same_activations(int on) { g_tc_same_activations = on; }

template <int WF, int NT>
static int launch_tc(const void *A_q8, const void *B, const float *bias, float *C, int ldc, int M, int N, int nb, uint8_t *ws, size_t ws_bytes, cudaStream_t st)
{
    using Cfg = TcCfg<NT>;
    auto kernel = gemm_kq_tc_kernel<WF, NT>;
    static int attr_set = 0;
    if (!attr_set) {
        cudaFuncAttributes fa;
        if (ckb_check_cuda((int)cudaFuncGetAttributes(&fa, kernel), "func attributes")) return CKB_ERR_CUDA;
        if (fa.numRegs != Cfg::REGS_LAUNCH)     // a different allocation at launch would make setmaxnreg.inc wait for registers that never come
            return ckb_fail(CKB_ERR_LIMIT, "gemm_kq_tc: kernel compiled with an unexpected register count");
        if (ckb_check_cuda((int)cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::SMEM), "smem attr")) return CKB_ERR_CUDA;
        attr_set = 1;
    }
    const int mtiles = (M + NT - 1) / NT, ntiles = (N + TC_ROWS - 1) / TC_ROWS;
    // K is split for a handful of tokens, and for any product whose tiles leave more than half of the SMs without a CTA (the k and
    // v projections of a prompt: 8 x 4 tiles)
    const int slots = ckb_sm_count() * Cfg::CTAS_PER_SM;
    const int splitk = ckb_tune_get("gemm_tc_splitk", 1);
    int Z = splitk && (M <= 128 || (splitk != 2 && 2 * ntiles * mtiles <= slots)) ? tc_pick_slices(ntiles * mtiles, nb, slots) : 1;
    const int forced = ckb_tune_get("gemm_tc_slices", 0);
    if (forced > 0 && forced <= nb) Z = forced;
    const int nbz = (nb + Z - 1) / Z;
    Z = (nb + nbz - 1) / nbz;                          // no empty slice
    // A grid of whole waves plus a few CTAs pays a full wave for those few (28672 x 4096 at 512 tokens: 896 tiles = 6 waves of 148
    // and 8 tiles).  The row tiles behind that remainder then go to a second launch with K split, which fills the SMs for a
    // fraction of a wave; its partial sums are added as for any split.  Library workspace only (a caller's workspace is sized
    // for one launch).
    int tail_nt = 0, Zt = 1;
    if (Z == 1 && !ws && ckb_tune_get("gemm_tc_tail", 1)) {
        const int tiles = ntiles * mtiles, rem = tiles % slots;
        if (tiles > slots && rem > 0 && 4 * rem <= slots && rem % mtiles == 0 && rem / mtiles < ntiles && N % TC_ROWS == 0) {
            Zt = tc_pick_slices(rem, nb, slots);
            if (Zt > 1) tail_nt = rem / mtiles;
        }
    }
    const int nbzt = (nb + Zt - 1) / Zt;
    if (tail_nt) Zt = (nb + nbzt - 1) / nbzt;
    const int Nt = tail_nt * TC_ROWS;                  // rows (output columns) of the tail launch
    const size_t xt_bytes = ((size_t)mtiles * nb * Cfg::XBLOB + 255) & ~(size_t)255;
    const size_t part_bytes = Z > 1 ? (size_t)Z * M * N * sizeof(float) : (tail_nt ? (size_t)Zt * M * Nt * sizeof(float) : 0);
    // A caller that records the launch in a CUDA graph brings its own workspace: the library's pool may be freed and
    // regrown by any later call that needs more, which would leave a captured pointer dangling.
    if (ws && xt_bytes + part_bytes > ws_bytes)
        return ckb_fail(CKB_ERR_LIMIT, "gemm_kq_tc: the caller's workspace holds %zu bytes, this call needs %zu", ws_bytes, xt_bytes + part_bytes);
    uint8_t *xt = ws ? ws : (uint8_t *)ckb_scratch(CKB_SLOT_G, xt_bytes + part_bytes);
    if (!xt) return CKB_ERR_CUDA;
    float *part = reinterpret_cast<float *>(xt + xt_bytes);
    // q, k and v of a prompt read the same activation rows: a caller that says so between its calls gets the operand tiles of
    // the previous product again, provided they still lie where this call would put them.
    const bool reuse = g_tc_same_activations && g_tc_tiles.a == A_q8 && g_tc_tiles.M == M && g_tc_tiles.nb == nb && g_tc_tiles.nt == NT &&
                       g_tc_tiles.xt == xt && g_tc_tiles.st == st;
    if (!reuse) {
        const int xz = nb * mtiles >= 2 * ckb_sm_count() ? 1 : (nb * mtiles >= ckb_sm_count() ? 2 : 4);      // enough CTAs for every SM
        gemm_x_tiles_kernel<NT><<<dim3(nb, mtiles, xz), 256, 0, st>>>((const uint8_t *)A_q8, xt, M, nb);
        if (int rc = ckb_check_launch("gemm_x_tiles")) return rc;
        g_tc_tiles.a = A_q8; g_tc_tiles.M = M; g_tc_tiles.nb = nb; g_tc_tiles.nt = NT; g_tc_tiles.xt = xt; g_tc_tiles.st = st;
    }
    const dim3 grid(ntiles - tail_nt, mtiles, Z);
    if (Z == 1) {
        kernel<<<grid, Cfg::THREADS, Cfg::SMEM, st>>>(xt, (const uint8_t *)B, bias, C, ldc, (size_t)0, M, N - Nt, nb, nbz, ckb_device_error_word());
        if (int rc = ckb_check_launch("gemm_kq_tc")) return rc;
        if (!tail_nt) return 0;
        const int n0 = N - Nt;
        const size_t rb = WF == TC_W_Q4K ? (size_t)nb * Q4K_BYTES : (((size_t)nb * Q6K_BYTES + 15) & ~(size_t)15);
        kernel<<<dim3(tail_nt, mtiles, Zt), Cfg::THREADS, Cfg::SMEM, st>>>(xt, (const uint8_t *)B + (size_t)n0 * rb, nullptr, part, Nt, (size_t)M * Nt, M, Nt, nb, nbzt,
                                                                         ckb_device_error_word());
        if (int rc = ckb_check_launch("gemm_kq_tc tail")) return rc;
        const size_t mnt = (size_t)M * Nt;
        const unsigned tb = (unsigned)((mnt + 1023) / 1024 < 1184 ? (mnt + 1023) / 1024 : 1184);
        const float *bt = bias ? bias + n0 : nullptr;
        if (ldc % 4 == 0 && (((uintptr_t)(C + n0) | (uintptr_t)bt) & 15) == 0) gemm_splitk_sum_kernel<true><<<tb, 256, 0, st>>>(part, Zt, bt, C + n0, ldc, M, Nt);
        else gemm_splitk_sum_kernel<false><<<tb, 256, 0, st>>>(part, Zt, bt, C + n0, ldc, M, Nt);
        return ckb_check_launch("gemm_splitk_sum");
    }
    kernel<<<grid, Cfg::THREADS, Cfg::SMEM, st>>>(xt, (const uint8_t *)B, nullptr, part, N, (size_t)M * N, M, N, nb, nbz, ckb_device_error_word());
    if (int rc = ckb_check_launch("gemm_kq_tc")) return rc;
    const size_t mn = (size_t)M * N;
    const unsigned blocks = (unsigned)((mn + 1023) / 1024 < 1184 ? (mn + 1023) / 1024 : 1184);
    if (N % 4 == 0 && ldc % 4 == 0 && (((uintptr_t)C | (uintptr_t)bias) & 15) == 0) gemm_splitk_sum_kernel<true><<<blocks, 256, 0, st>>>(part, Z, bias, C, ldc, M, N);
    else gemm_splitk_sum_kernel<false><<<blocks, 256, 0, st>>>(part, Z, bias, C, ldc, M, N);
    return ckb_check_launch("gemm_splitk_sum");
}

#ifdef CKB_TC_TRACE
extern "C" int ckb200_tc_trace(long long *out4096) { return (int)cudaMemcpyFromSymbol(out4096, g_tc_trace, sizeof(long long) * 4096); }
#endif

// C[m * ldc + n] = A_q8[m] . W[n] (+ bias[n]).  wf: TC_W_Q4K (the reference's block_q4_K rows) or TC_W_Q6K_PLANAR.
// Returns -1 when the shape is not handled here (caller falls back to the per-token path).  min_tokens: smallest M
// worth the tensor-core path (the token tile is 128 wide; fewer tokens are padded with zeros).
extern "C" int ckb_launch_gemm_tc_ws(int wf, const void *A_q8, const void *B, const float *bias, float *C, int ldc, int M, int N, int K, int min_tokens,
                                     void *ws, size_t ws_bytes, void *stream)
{
    if (M < min_tokens || K % QK_K || ((uintptr_t)B & 15) || ((uintptr_t)A_q8 & 3) || ((uintptr_t)ws & 255) || ckb_tune_get("gemm_tc", 1) == 0) return -1;
    const int nb = K / QK_K;
    cudaStream_t st = ckb_stream(stream);
    uint8_t *w8 = (uint8_t *)ws;
    if (M <= ckb_tune_get("gemm_tc_small_max", 64))     // batched decode: 32-token tiles, two CTAs per SM
        return wf == TC_W_Q6K_PLANAR ? launch_tc<TC_W_Q6K_PLANAR, 32>(A_q8, B, bias, C, ldc, M, N, nb, w8, ws_bytes, st)
                                     : launch_tc<TC_W_Q4K, 32>(A_q8, B, bias, C, ldc, M, N, nb, w8, ws_bytes, st);
    return wf == TC_W_Q6K_PLANAR ? launch_tc<TC_W_Q6K_PLANAR, 128>(A_q8, B, bias, C, ldc, M, N, nb, w8, ws_bytes, st)
                                 : launch_tc<TC_W_Q4K, 128>(A_q8, B, bias, C, ldc, M, N, nb, w8, ws_bytes, st);
}

extern "C" int ckb_launch_gemm_tc(int wf, const void *A_q8, const void *B, const float *bias, float *C, int ldc, int M, int N, int K, int min_tokens,
                                  void *stream)
{
    return ckb_launch_gemm_tc_ws(wf, A_q8, B, bias, C, ldc, M, N, K, min_tokens, NULL, 0, stream);
}

// Upper bound of the workspace one call with these sizes can need (activation tiles plus the partial sums of the largest
// K split the launcher picks by itself), for callers that allocate it once.
extern "C" size_t ckb_gemm_tc_workspace_bytes(int M, int N, int K)
{
    if (M <= 0 || N <= 0 || K <= 0 || K % QK_K) return 0;
    const int nb = K / QK_K;
    const size_t blob = TcCfg<32>::XBLOB > TcCfg<128>::XBLOB ? TcCfg<32>::XBLOB : TcCfg<128>::XBLOB;
    const size_t mtiles = (size_t)(M + 31) / 32;
    const size_t xt = (mtiles * nb * blob + 255) & ~(size_t)255;
    int zmax = nb / 4 < 1 ? 1 : (nb / 4 > 16 ? 16 : nb / 4);
    if (M > 128) zmax = 1;
    return xt + (zmax > 1 ? (size_t)zmax * M * N * sizeof(float) : 0) + 256;
}

extern "C" int ckb_launch_gemm_q4k_tc(const void *A_q8, const void *B, const float *bias, float *C, int M, int N, int K, void *stream)
{
    return ckb_launch_gemm_tc(TC_W_Q4K, A_q8, B, bias, C, N, M, N, K, ckb_tune_get("gemm_tc_min_tokens", 16), stream);
}

// gemm_nt_q6_k_q8_k (src/kernels/gemm_kernels_q6k_q8k.c:1243-1268) over weights in the row-planar layout
extern "C" int ckb200_dev_gemv_q6_k_planar_q8_k(float *, const void *, const void *, int, int, void *);
extern "C" int ckb200_dev_add_bias_rows(float *, const float *, int, int, void *);
extern "C" int ckb_launch_gemm_q6k_mma(const void *A_q8, const void *B_planar, const float *bias, float *C, int ldc, int M, int N, int K, void *stream);
extern "C" int ckb200_dev_gemm_nt_q6_k_planar_q8_k(const void *A_q8, const void *B_planar, const float *bias, float *C, int M, int N, int K, void *stream)
{
    if (!A_q8 || !B_planar || !C || M <= 0 || N <= 0 || K <= 0) return 0;
    if (ckb_ensure_init()) return CKB_ERR_NO_DEVICE;
    int rc = ckb_launch_gemm_q6k_mma(A_q8, B_planar, bias, C, N, M, N, K, stream);        // 4 to 64 tokens: integer MMA over the planes (gemm_q6k_mma.cu)
    if (rc >= 0) return rc;
    rc = ckb_launch_gemm_tc(TC_W_Q6K_PLANAR, A_q8, B_planar, bias, C, N, M, N, K, ckb_tune_get("gemm_tc_min_tokens", 16), stream);
    if (rc >= 0) return rc;
    for (int m = 0; m < M; ++m) {
        const int r2 = ckb200_dev_gemv_q6_k_planar_q8_k(C + (size_t)m * N, B_planar, (const uint8_t *)A_q8 + (size_t)m * (K / QK_K) * Q8K_BYTES, N, K, stream);
        if (r2) return r2;
    }
    return bias ? ckb200_dev_add_bias_rows(C, bias, M, N, stream) : 0;
}
