// Prefill GEMM on the 5th-generation tensor cores: C[M,N] = A_q8[M,K] . B_q4k[N,K]^T (+ bias), M >= 64.
// Replaces gemm_nt_q4_k_q8_k (src/kernels/gemm_kernels_q4k_q8k.c:301-326), which the reference computes as
// one GEMV per token with no weight reuse.
//
// Exact-integer formulation.  For one 256-element superblock b the reference adds
//     d_x[m,b] * ( d[n,b] * sum_j sc[n,j] * S[m,n,j]  -  dmin[n,b] * sum_j mn[n,j] * bsum[m,j] )
// where S are int32 sub-block dots (gemm_kernels_q4k_q8k.c:144-173).  Here
//     T [n,m] = sum_k (sc[n,k/32] * q4[n,k]) * q8[m,k]        256-deep f16 MMA, every operand an exact integer
//     T2[n,m] = sum_i  mn[n,i/2]  * bsum16[m,i]               16-deep f16 MMA (one k-step)
// are accumulated in fp32 in tensor memory (integers below 2^24 stay exact), read back with tcgen05.ld once
// per superblock and combined with the fp32 scales in registers: acc += d_x * (d * T - dmin * T2).
//
// Two kernels:
//  * gemm_x_tiles_kernel expands the Q8_K activations once into fp16 operand tiles in the exact shared-memory
//    layout of the MMA (K-major, no swizzle, 8 x 16-byte core matrices), one contiguous blob per
//    (128-token tile, superblock), so the GEMM fetches them with plain 1-D bulk copies.
//  * gemm_q4k_tc_kernel<NH>: one CTA owns 128 weight rows (the M = 128 operand, one TMEM lane each) and NH
//    128-token tiles (the N = 128 operand, TMEM columns).  Warp-specialised, 16 warps:
//        warp 0      bulk-copy loader of activation tiles (4-stage ring of 64-deep k-stages)
//        warp 1      MMA issuer: tcgen05.mma from one thread, tcgen05.commit frees stages and publishes accumulators
//        warps 4-7   expand the 4-bit weights to sc*q fp16 tiles (8-stage ring = two superblocks)
//        warps 8-15  drain the accumulators (two TMEM buffers of T|T2, 512 columns) and keep the fp32 sums
//    With NH = 2 a weight tile is expanded once and used against 256 tokens; the two token tiles alternate
//    between the TMEM buffers, with NH = 1 successive superblocks do.
// Every wait is bounded; a timeout sets the device error word, the CTA drains, frees TMEM and returns.
#include "quant_units.cuh"
#include "pdl.cuh"

namespace ckb {

constexpr int TC_ROWS = 128;                          // rows of either operand per MMA
constexpr int TC_CHUNK = TC_ROWS * 16;                // one 8-element k-chunk of 128 rows: 2048 B
constexpr int TC_STAGE = 8 * TC_CHUNK;                // 64-deep k-stage of 128 rows: 16 KB
constexpr int TC_AUX = 2 * TC_CHUNK;                  // 16-deep tile (mins / bsums): 4 KB
constexpr int TC_A_STAGES = 8, TC_B_STAGES = 4;
// activation blob of one (token tile, superblock): 4 k-stages, the bsum tile, 128 block scales
constexpr int TC_XBLOB_B2 = 4 * TC_STAGE;
constexpr int TC_XBLOB_DX = TC_XBLOB_B2 + TC_AUX;
constexpr int TC_XBLOB = TC_XBLOB_DX + TC_ROWS * 4;   // 70144 B, a multiple of 16

constexpr int TC_OFF_A = 0;
constexpr int TC_OFF_B = TC_OFF_A + TC_A_STAGES * TC_STAGE;
constexpr int TC_OFF_A2 = TC_OFF_B + TC_B_STAGES * TC_STAGE;
constexpr int TC_OFF_B2 = TC_OFF_A2 + 2 * TC_AUX;
constexpr int TC_AUXX = TC_AUX + TC_ROWS * 4;           // bsum tile followed by the 128 activation block scales (contiguous in the blob)
constexpr int TC_OFF_BAR = TC_OFF_B2 + 2 * TC_AUXX;
enum { BAR_A_FULL = 0, BAR_A_EMPTY = 8, BAR_B_FULL = 16, BAR_B_EMPTY = 20, BAR_A2_FULL = 24, BAR_A2_EMPTY = 26, BAR_B2_FULL = 28,
       BAR_B2_EMPTY = 30, BAR_T_FULL = 32, BAR_T_EMPTY = 34, BAR_COUNT = 36 };
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
// One lane of a converged warp.  The loader and issuer warps run their loops and waits warp-uniformly and only
// predicate the issuing instructions on this, so that descriptors and addresses stay in uniform registers.
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

struct Q4Stage {
    uint4 qa, qb;
};

// In-kernel cycle counters of CTA (0,0), written over the first output row: a tuning aid, compiled out by default.
#ifdef CKB_TC_PROFILE
__device__ float g_tc_prof[64];
#define TC_PROF_DECL() long long pf[8] = {0, 0, 0, 0, 0, 0, 0, 0}, pf_t = clock64(), pf_begin = pf_t
#define TC_PROF(k) do { const long long now_ = clock64(); pf[k] += now_ - pf_t; pf_t = now_; } while (0)
#define TC_PROF_OUT(slot) do { if (blockIdx.x == 0 && blockIdx.y == 0) { pf[7] = clock64() - pf_begin; for (int i_ = 0; i_ < 8; ++i_) g_tc_prof[8 * (slot) + i_] = (float)pf[i_]; } } while (0)
#else
#define TC_PROF_DECL() do { } while (0)
#define TC_PROF(k) do { } while (0)
#define TC_PROF_OUT(slot) do { } while (0)
#endif

// Register counts per role after setmaxnreg; 128 * (CTL + EW * EXP + 2 * DRAIN) must not exceed threads x launch registers.
enum { TC_W_Q4K = 0, TC_W_Q6K_PLANAR = 1 };       // weight operand formats

template <int NH, int EW> struct TcRegs;
template <> struct TcRegs<1, 2> { static constexpr int CTL = 32, EXP = 72, DRAIN = 152, LAUNCH = 96; };    // 640 threads x 96
template <> struct TcRegs<2, 1> { static constexpr int CTL = 40, EXP = 72, DRAIN = 200, LAUNCH = 128; };   // 512 threads x 128

// WF weight format, NH 128-token tiles per CTA, EW warpgroups of weight expanders.
//
// Q6_K weights (row-planar layout, see gemv_q6k_planar.cu) use the same pipeline with A = (q6 - 32) * sc as fp16: the
// offset is inside the operand, so there is no second accumulator, and each 64-deep k-stage is one (half n, nibble
// half) of a superblock (include/ckernel_quant.h:135-146, src/kernels/gemm_kernels_q6k_q8k.c:86-116).  The product is
// an exact fp16 integer whenever |q6 - 32| * |sc| <= 2048 (always for |sc| <= 64); above that it is rounded to the
// nearest even integer, a relative error of at most 2^-12 on that element.
template <int WF, int NH, int EW>
__global__ void __launch_bounds__(128 * (3 + EW), 1)
gemm_kq_tc_kernel(const uint8_t *__restrict__ xt, const uint8_t *__restrict__ B, const float *__restrict__ bias, float *__restrict__ C, int ldc, int M,
                  int N, int nb, int *__restrict__ dev_err)
{
    extern __shared__ __align__(128) uint8_t smem[];
    const uint32_t s_base = smem_u32(smem);
    const uint32_t sA = s_base + TC_OFF_A, sB = s_base + TC_OFF_B, sA2 = s_base + TC_OFF_A2, sB2 = s_base + TC_OFF_B2, sBar = s_base + TC_OFF_BAR;
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(smem + TC_OFF_BAR + BAR_COUNT * 8);
#define BAR(i) (sBar + 8u * (uint32_t)(i))

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int n0 = blockIdx.x * TC_ROWS, mt0 = blockIdx.y * NH, m0 = mt0 * TC_ROWS;
    const int halves = min(NH, (M - m0 + TC_ROWS - 1) / TC_ROWS);

    if (tid == 0) {
        for (int i = 0; i < 8; ++i) { mbar_init(BAR(BAR_A_FULL + i), 4); mbar_init(BAR(BAR_A_EMPTY + i), 1); }
        for (int i = 0; i < 4; ++i) { mbar_init(BAR(BAR_B_FULL + i), 1); mbar_init(BAR(BAR_B_EMPTY + i), 1); }
        for (int i = 0; i < 2; ++i) {
            mbar_init(BAR(BAR_A2_FULL + i), 4 * EW); mbar_init(BAR(BAR_A2_EMPTY + i), 1);
            mbar_init(BAR(BAR_B2_FULL + i), 1); mbar_init(BAR(BAR_B2_EMPTY + i), 9);   // the T2 MMA and the 8 drain warps (block scales)
            mbar_init(BAR(BAR_T_FULL + i), 1); mbar_init(BAR(BAR_T_EMPTY + i), 8);
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
    const uint32_t tmem = *tmem_slot;                 // buffer u&1 at column 256*(u&1): T at +0, T2 at +128

    // Registers move from the loader/issuer and expander warpgroups to the drain warps, which hold 64 accumulators
    // per token tile.  setmaxnreg.inc blocks until the CTA's own pool (threads x registers at launch) has the registers,
    // so the three counts must fit in that pool: the launcher checks it against the compiled register count.
    constexpr int REGS_CTL = TcRegs<NH, EW>::CTL, REGS_EXP = TcRegs<NH, EW>::EXP, REGS_DRAIN = TcRegs<NH, EW>::DRAIN;
#define TC_SETMAXNREG(op, n) asm volatile("setmaxnreg." op ".sync.aligned.u32 %0;" ::"n"(n))
#define TC_WAIT(bar, parity, code)                                        \
    if (!mbar_wait_spin(bar, parity)) { atomicExch(dev_err, code); break; }

    if (warp < 4) {
        TC_SETMAXNREG("dec", REGS_CTL);
        if (warp == 0) {
            // ------------------------------------------------------------ activation loader
            TC_PROF_DECL();
            uint32_t cb = 0;
            bool go = true;
            for (int b = 0; b < nb && go; ++b) {
                for (int h = 0; h < halves && go; ++h) {
                    go = false;
                    do {
                        const uint8_t *blob = xt + ((size_t)(mt0 + h) * nb + b) * TC_XBLOB;
                        const uint32_t u = (uint32_t)(b * halves + h), x = u & 1u;
                        int s = 0;
                        for (; s < 4; ++s, ++cb) {
                            const uint32_t i = cb & 3u;
                            TC_PROF(0);
                            TC_WAIT(BAR(BAR_B_EMPTY + i), ((cb >> 2) & 1u) ^ 1u, DEV_ERR_EMPTY_WAIT);
                            TC_PROF(1);
                            if (tc_elect_one()) {
                                mbar_arrive_expect_tx(BAR(BAR_B_FULL + i), TC_STAGE);
                                bulk_g2s(sB + i * TC_STAGE, blob + s * TC_STAGE, TC_STAGE, BAR(BAR_B_FULL + i));
                            }
                            __syncwarp();
                            TC_PROF(2);
                        }
                        if (s < 4) break;
                        TC_WAIT(BAR(BAR_B2_EMPTY + x), ((u >> 1) & 1u) ^ 1u, DEV_ERR_EMPTY_WAIT);
                        if (tc_elect_one()) {
                            mbar_arrive_expect_tx(BAR(BAR_B2_FULL + x), TC_AUXX);
                            bulk_g2s(sB2 + x * TC_AUXX, blob + TC_XBLOB_B2, TC_AUXX, BAR(BAR_B2_FULL + x));
                        }
                        __syncwarp();
                        go = true;
                    } while (0);
                }
            }
            if (!go) {                                 // copies still in flight must land before the CTA's shared memory goes away
                for (uint32_t c = cb > 4 ? cb - 4 : 0; c < cb; ++c) mbar_wait_spin(BAR(BAR_B_FULL + (c & 3u)), (c >> 2) & 1u);
            }
            if (lane == 0) TC_PROF_OUT(0);
        } else if (warp == 1) {
            // ------------------------------------------------------------ MMA issuer
            const uint64_t dA = tc_smem_desc(sA), dB = tc_smem_desc(sB), dA2 = tc_smem_desc(sA2), dB2 = tc_smem_desc(sB2);
            TC_PROF_DECL();
            uint32_t cb = 0;
            bool go = true;
            for (int b = 0; b < nb && go; ++b) {
                for (int h = 0; h < halves && go; ++h) {
                    go = false;
                    do {
                        const uint32_t u = (uint32_t)(b * halves + h), buf = u & 1u, tacc = tmem + 256u * buf;
                        const bool last_use = h == halves - 1;
                        TC_PROF(0);
                        TC_WAIT(BAR(BAR_T_EMPTY + buf), ((u >> 1) & 1u) ^ 1u, DEV_ERR_MMA_WAIT);
                        TC_PROF(1);
                        tc_fence_after();                  // orders the drain's tcgen05.ld of this buffer before the MMAs that overwrite it
                        int s = 0;
                        for (; s < 4; ++s, ++cb) {
                            const uint32_t it = (uint32_t)(b * 4 + s), ia = it & 7u, ib = cb & 3u;
                            TC_PROF(0);
                            TC_WAIT(BAR(BAR_A_FULL + ia), (it >> 3) & 1u, DEV_ERR_FULL_WAIT);
                            TC_PROF(2);
                            TC_WAIT(BAR(BAR_B_FULL + ib), (cb >> 2) & 1u, DEV_ERR_FULL_WAIT);
                            TC_PROF(3);
                            const uint64_t da = dA + (uint64_t)(ia * (TC_STAGE >> 4)), db = dB + (uint64_t)(ib * (TC_STAGE >> 4));
                            if (tc_elect_one()) {
#pragma unroll
                                for (int i = 0; i < 4; ++i)
                                    tc_mma(tacc, da + (uint64_t)(i * (2 * TC_CHUNK >> 4)), db + (uint64_t)(i * (2 * TC_CHUNK >> 4)), (s | i) ? 1u : 0u);
                                TC_PROF(4);
                                tc_commit(BAR(BAR_B_EMPTY + ib));
                                if (last_use) tc_commit(BAR(BAR_A_EMPTY + ia));
                            }
                            __syncwarp();
                            TC_PROF(5);
                        }
                        if (s < 4) break;
                        if constexpr (WF == TC_W_Q4K) {
                            const uint32_t x2 = (uint32_t)b & 1u;
                            TC_WAIT(BAR(BAR_A2_FULL + x2), ((uint32_t)b >> 1) & 1u, DEV_ERR_FULL_WAIT);
                            TC_WAIT(BAR(BAR_B2_FULL + buf), (u >> 1) & 1u, DEV_ERR_FULL_WAIT);
                            if (tc_elect_one()) {
                                tc_mma(tacc + 128u, dA2 + (uint64_t)(x2 * (TC_AUX >> 4)), dB2 + (uint64_t)(buf * (TC_AUXX >> 4)), 0u);
                                tc_commit(BAR(BAR_B2_EMPTY + buf));
                                if (last_use) tc_commit(BAR(BAR_A2_EMPTY + x2));
                                tc_commit(BAR(BAR_T_FULL + buf));
                            }
                        } else {
                            if (tc_elect_one()) {
                                tc_commit(BAR(BAR_B2_EMPTY + buf));      // nothing reads the bsum tile; the drain warps still release the block scales
                                tc_commit(BAR(BAR_T_FULL + buf));
                            }
                        }
                        __syncwarp();
                        TC_PROF(6);
                        go = true;
                    } while (0);
                }
            }
            if (lane == 0) TC_PROF_OUT(1);
        }
    } else if (warp < 4 + 4 * EW) {
        // ------------------------------------------------------------ weight expanders: thread = row, stage = quarter of a superblock
        TC_SETMAXNREG("dec", REGS_EXP);
        const int set = (warp - 4) >> 2, row = tid & 127;
        if constexpr (WF == TC_W_Q6K_PLANAR) {
            // set e takes half n = e (EW = 2) or both halves in turn (EW = 1): the 64 ql bytes and 32 qh bytes of a half feed two stages
            const size_t rb = ((size_t)nb * Q6K_BYTES + 15) & ~(size_t)15;
            const uint8_t *wrow = B + (size_t)min(n0 + row, N - 1) * rb;
            const size_t off_qh = (size_t)nb * 128, off_sc = (size_t)nb * 192;
            const __half2 c66 = __floats2half2_rn(66.0f, 66.0f);
            const uint32_t halves_total = (uint32_t)nb * 2u;
            for (uint32_t hf = (uint32_t)set; hf < halves_total; hf += EW) {
                const uint32_t b = hf >> 1, n = hf & 1u;
                uint4 ql[4], qh[2];
#pragma unroll
                for (int j = 0; j < 4; ++j) ql[j] = __ldg(reinterpret_cast<const uint4 *>(wrow + (size_t)b * 128 + 64 * n + 16 * j));
#pragma unroll
                for (int j = 0; j < 2; ++j) qh[j] = __ldg(reinterpret_cast<const uint4 *>(wrow + off_qh + (size_t)b * 64 + 32 * n + 16 * j));
                const uint2 sc8 = __ldg(reinterpret_cast<const uint2 *>(wrow + off_sc + (size_t)b * 16 + 8 * n));
                const uint32_t qlw[16] = {ql[0].x, ql[0].y, ql[0].z, ql[0].w, ql[1].x, ql[1].y, ql[1].z, ql[1].w,
                                          ql[2].x, ql[2].y, ql[2].z, ql[2].w, ql[3].x, ql[3].y, ql[3].z, ql[3].w};
                const uint32_t qhw[8] = {qh[0].x, qh[0].y, qh[0].z, qh[0].w, qh[1].x, qh[1].y, qh[1].z, qh[1].w};
                bool ok_stage = true;
#pragma unroll 1
                for (uint32_t hi = 0; hi < 2 && ok_stage; ++hi) {
                    const uint32_t it = 4u * b + 2u * n + hi, ia = it & 7u;
                    const uint32_t scw = hi ? sc8.y : sc8.x;       // scale groups 8n + 4hi + {0, 1, 2, 3}
                    if (!mbar_wait_spin(BAR(BAR_A_EMPTY + ia), ((it >> 3) & 1u) ^ 1u)) { atomicExch(dev_err, DEV_ERR_EMPTY_WAIT); ok_stage = false; break; }
                    uint8_t *dst = smem + TC_OFF_A + ia * TC_STAGE;
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
                            uint32_t h01, h23;
                            // 0x5400 | q is the fp16 bit pattern of 64 + q / 16
                            h01 = __byte_perm(nib | two, 0x54545454u, 0x5140);
                            h23 = __byte_perm(nib | two, 0x54545454u, 0x7362);
                            const __half2 r0 = __hmul2(__hsub2(*reinterpret_cast<__half2 *>(&h01), c66), sc2);   // (q - 32) / 16 * 16 sc
                            const __half2 r1 = __hmul2(__hsub2(*reinterpret_cast<__half2 *>(&h23), c66), sc2);
                            o[2 * w2] = *reinterpret_cast<const uint32_t *>(&r0);
                            o[2 * w2 + 1] = *reinterpret_cast<const uint32_t *>(&r1);
                        }
                        *reinterpret_cast<uint4 *>(dst + tc_tile_offset(row, c)) = make_uint4(o[0], o[1], o[2], o[3]);
                    }
                    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                    __syncwarp();
                    if (lane == 0) mbar_arrive(BAR(BAR_A_FULL + ia));
                }
                if (!ok_stage) break;
            }
        } else {
            const uint8_t *wrow = B + (size_t)min(n0 + row, N - 1) * nb * Q4K_BYTES;
            const uint32_t stages = (uint32_t)nb * 4u;
            Q4Stage cur;
            uint4 hdr;
            {
                const uint8_t *p0 = wrow + 16 + 32 * set;
                cur.qa = __ldg(reinterpret_cast<const uint4 *>(p0));
                cur.qb = __ldg(reinterpret_cast<const uint4 *>(p0 + 16));
                hdr = __ldg(reinterpret_cast<const uint4 *>(wrow));
            }
            TC_PROF_DECL();
            for (uint32_t it = (uint32_t)set; it < stages; it += EW) {
                const uint32_t b = it >> 2, s = it & 3u, ia = it & 7u, x2 = b & 1u;
                TC_PROF(0);
                Q4Stage nxt = cur;
                uint4 hdr_next = hdr;
                if (it + EW < stages) {                   // this thread's next quarter, possibly of the next superblock
                    const uint8_t *pn = wrow + (size_t)((it + EW) >> 2) * Q4K_BYTES;
                    nxt.qa = __ldg(reinterpret_cast<const uint4 *>(pn + 16 + 32 * ((it + EW) & 3u)));
                    nxt.qb = __ldg(reinterpret_cast<const uint4 *>(pn + 32 + 32 * ((it + EW) & 3u)));
                    if (((it + EW) >> 2) != b) hdr_next = __ldg(reinterpret_cast<const uint4 *>(pn));
                }
                uint32_t sc2, m2;
                q4k_scales(hdr.y, hdr.z, hdr.w, (int)s, sc2, m2);
                const float sclo = (float)(sc2 & 255u), schi = (float)(sc2 >> 8);
                const __half2 s_lo = __floats2half2_rn(sclo, sclo), s_hi = __floats2half2_rn(schi, schi);
                const __half2 b_lo = __floats2half2_rn(-1024.0f * sclo, -1024.0f * sclo), b_hi = __floats2half2_rn(-1024.0f * schi, -1024.0f * schi);
                const float mlo = (float)(m2 & 255u), mhi = (float)(m2 >> 8);
                const __half2 mm_lo = __floats2half2_rn(mlo, mlo), mm_hi = __floats2half2_rn(mhi, mhi);
                TC_PROF(1);
                TC_WAIT(BAR(BAR_A_EMPTY + ia), ((it >> 3) & 1u) ^ 1u, DEV_ERR_EMPTY_WAIT);
                TC_PROF(2);
                if (s < (uint32_t)EW) { TC_WAIT(BAR(BAR_A2_EMPTY + x2), ((b >> 1) & 1u) ^ 1u, DEV_ERR_EMPTY_WAIT); }   // this set's first write of the superblock
                TC_PROF(3);
                const uint32_t ml = 0x0F0F0F0Fu;
                const uint32_t w[8] = {cur.qa.x, cur.qa.y, cur.qa.z, cur.qa.w, cur.qb.x, cur.qb.y, cur.qb.z, cur.qb.w};
                uint8_t *dst = smem + TC_OFF_A + ia * TC_STAGE;
    #pragma unroll
                for (int c = 0; c < 4; ++c) {     // low nibbles = sub-block 2s: k-chunks 0-3 of the stage; high nibbles = sub-block 2s+1: k-chunks 4-7
                    *reinterpret_cast<uint4 *>(dst + tc_tile_offset(row, c)) = q4_chunk_to_half(w[2 * c] & ml, w[2 * c + 1] & ml, s_lo, b_lo);
                    *reinterpret_cast<uint4 *>(dst + tc_tile_offset(row, 4 + c)) = q4_chunk_to_half((w[2 * c] >> 4) & ml, (w[2 * c + 1] >> 4) & ml, s_hi, b_hi);
                }
                // the two mins of this quarter, each doubled (bsums come per 16 elements): positions 4s .. 4s+3 of the 16-deep tile
                uint32_t *d2 = reinterpret_cast<uint32_t *>(smem + TC_OFF_A2 + x2 * TC_AUX + tc_tile_offset(row, (int)(s >> 1))) + 2 * (s & 1u);
                d2[0] = *reinterpret_cast<const uint32_t *>(&mm_lo);
                d2[1] = *reinterpret_cast<const uint32_t *>(&mm_hi);
                TC_PROF(4);
                asm volatile("fence.proxy.async.shared::cta;" ::: "memory");   // generic-proxy writes -> visible to the tensor core
                TC_PROF(5);
                __syncwarp();
                if (lane == 0) {
                    mbar_arrive(BAR(BAR_A_FULL + ia));
                    if (s >= 4u - (uint32_t)EW) mbar_arrive(BAR(BAR_A2_FULL + x2));   // this set's last quarter of the superblock
                }
                cur = nxt;
                hdr = hdr_next;
                TC_PROF(6);
            }
        }
        if (lane == 0 && (warp & 3) == 0) TC_PROF_OUT(2 + set);
    } else {
        // ------------------------------------------------------------ accumulator drain: thread = TMEM lane (weight row), 64 token columns
        TC_SETMAXNREG("inc", REGS_DRAIN);
        constexpr int RC = NH == 2 ? 16 : 32;         // columns per round of tcgen05.ld
        const int dw = warp - (4 + 4 * EW);
        const int q = dw & 3, ch = dw >> 2;           // (4 + 4 * EW) % 4 == 0: warp % 4 is the TMEM lane quarter this warp may read
        const int row = 32 * q + lane, n = n0 + row;
        constexpr size_t DSTRIDE = WF == TC_W_Q4K ? Q4K_BYTES : 2;        // bytes between the block scales of consecutive superblocks
        const uint8_t *wrow = WF == TC_W_Q4K ? B + (size_t)min(n, N - 1) * nb * Q4K_BYTES
                                             : B + (size_t)min(n, N - 1) * (((size_t)nb * Q6K_BYTES + 15) & ~(size_t)15) + (size_t)nb * 208;
        float acc[NH][64];
#pragma unroll
        for (int h = 0; h < NH; ++h)
#pragma unroll
            for (int i = 0; i < 64; ++i) acc[h][i] = 0.0f;
        bool go = true;
        TC_PROF_DECL();
        auto load_dd = [&](int b) -> uint32_t {       // Q4_K: fp16 d | dmin of the superblock; Q6_K: fp16 d
            if constexpr (WF == TC_W_Q4K) return __ldg(reinterpret_cast<const uint32_t *>(wrow + (size_t)b * DSTRIDE));
            else return ldg_nc_u16(wrow + (size_t)b * DSTRIDE);
        };
        uint32_t dd_next = load_dd(0);
        for (int b = 0; b < nb && go; ++b) {
            const uint32_t dd_bits = dd_next;
            if (b + 1 < nb) dd_next = load_dd(b + 1);
            const float2 dd = __half22float2(*reinterpret_cast<const __half2 *>(&dd_bits));
#pragma unroll
            for (int h = 0; h < NH; ++h) {
                if (h < halves && go) {
                    go = false;
                    do {
                        const uint32_t u = (uint32_t)(b * halves + h), buf = u & 1u;
                        const float4 *dxp = reinterpret_cast<const float4 *>(smem + TC_OFF_B2 + buf * TC_AUXX + TC_AUX) + ch * 16;
                        TC_PROF(0);
                        TC_WAIT(BAR(BAR_B2_FULL + buf), (u >> 1) & 1u, DEV_ERR_FULL_WAIT);    // the block scales arrived with the bsum tile
                        TC_PROF(1);
                        TC_WAIT(BAR(BAR_T_FULL + buf), (u >> 1) & 1u, DEV_ERR_MMA_WAIT);
                        TC_PROF(2);
                        tc_fence_after();
                        const uint32_t taddr = tmem + ((uint32_t)(32 * q) << 16) + 256u * buf + 64u * (uint32_t)ch;
#pragma unroll
                        for (int c = 0; c < 64 / RC; ++c) {
                            uint32_t t1[RC / 16][16], t2[RC / 16][16];
#pragma unroll
                            for (int j = 0; j < RC / 16; ++j) {
                                tc_ld16(taddr + (uint32_t)(RC * c + 16 * j), t1[j]);
                                if constexpr (WF == TC_W_Q4K) tc_ld16(taddr + 128u + (uint32_t)(RC * c + 16 * j), t2[j]);
                            }
                            asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
                            TC_PROF(3);
#pragma unroll
                            for (int j = 0; j < RC / 16; ++j)
#pragma unroll
                                for (int i4 = 0; i4 < 4; ++i4) {
                                    const float4 dx = dxp[(RC * c + 16 * j) / 4 + i4];
                                    const float dxf[4] = {dx.x, dx.y, dx.z, dx.w};
#pragma unroll
                                    for (int i = 0; i < 4; ++i) {
                                        if constexpr (WF == TC_W_Q4K)
                                            acc[h][RC * c + 16 * j + 4 * i4 + i] +=
                                                dxf[i] * (dd.x * __uint_as_float(t1[j][4 * i4 + i]) - dd.y * __uint_as_float(t2[j][4 * i4 + i]));
                                        else
                                            acc[h][RC * c + 16 * j + 4 * i4 + i] += (dxf[i] * dd.x) * __uint_as_float(t1[j][4 * i4 + i]);
                                    }
                                }
                        }
                        TC_PROF(4);
                        tc_fence_before();
                        __syncwarp();
                        if (lane == 0) {
                            mbar_arrive(BAR(BAR_T_EMPTY + buf));
                            mbar_arrive(BAR(BAR_B2_EMPTY + buf));
                        }
                        TC_PROF(5);
                        go = true;
                    } while (0);
                }
            }
        }
        if (lane == 0 && dw == 0) TC_PROF_OUT(4);
        if (go && n < N) {
            const float bv = bias ? bias[n] : 0.0f;
#pragma unroll
            for (int h = 0; h < NH; ++h)
#pragma unroll
                for (int i = 0; i < 64; ++i) {
                    const int m = m0 + h * TC_ROWS + 64 * ch + i;
                    if (h < halves && m < M) C[(size_t)m * ldc + n] = acc[h][i] + bv;
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

template <int WF, int NH, int EW>
static int launch_tc(const uint8_t *xt, const void *B, const float *bias, float *C, int ldc, int M, int N, int nb, int mtiles, cudaStream_t st)
{
    static int attr_set = 0;
    if (!attr_set) {
        using R = TcRegs<NH, EW>;
        static_assert(128 * (R::CTL + EW * R::EXP + 2 * R::DRAIN) <= 128 * (3 + EW) * R::LAUNCH, "setmaxnreg targets exceed the CTA's register pool");
        static_assert(128 * (3 + EW) * R::LAUNCH <= 65536 && R::CTL <= R::LAUNCH && R::EXP <= R::LAUNCH && R::DRAIN >= R::LAUNCH, "register plan");
        cudaFuncAttributes fa;
        if (ckb_check_cuda((int)cudaFuncGetAttributes(&fa, gemm_kq_tc_kernel<WF, NH, EW>), "func attributes")) return CKB_ERR_CUDA;
        if (fa.numRegs != R::LAUNCH)          // a different allocation at launch would make setmaxnreg.inc wait for registers that never come
            return ckb_fail(CKB_ERR_LIMIT, "gemm_kq_tc: kernel compiled with an unexpected register count");
        if (ckb_check_cuda((int)cudaFuncSetAttribute(gemm_kq_tc_kernel<WF, NH, EW>, cudaFuncAttributeMaxDynamicSharedMemorySize, TC_SMEM), "smem attr")) return CKB_ERR_CUDA;
        attr_set = 1;
    }
    const dim3 grid((N + TC_ROWS - 1) / TC_ROWS, (mtiles + NH - 1) / NH);
    gemm_kq_tc_kernel<WF, NH, EW><<<grid, 128 * (3 + EW), TC_SMEM, st>>>(xt, (const uint8_t *)B, bias, C, ldc, M, N, nb, ckb_device_error_word());
    return ckb_check_launch("gemm_kq_tc");
}

#ifdef CKB_TC_PROFILE
extern "C" int ckb200_tc_profile(float *out64) { return (int)cudaMemcpyFromSymbol(out64, g_tc_prof, sizeof(float) * 64); }
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
    // One token tile per CTA with two expander warpgroups measured faster at every prefill size tried (the issuer is
    // bound by shared-memory operand traffic, not by the expansion); the two-tile variant stays selectable for tuning.
    const int nh = ckb_tune_get("gemm_tc_nh", 0) == 2 && mtiles >= 2 ? 2 : 1;
    if (wf == TC_W_Q6K_PLANAR)
        return nh == 2 ? launch_tc<TC_W_Q6K_PLANAR, 2, 1>(xt, B, bias, C, ldc, M, N, nb, mtiles, st)
                       : launch_tc<TC_W_Q6K_PLANAR, 1, 2>(xt, B, bias, C, ldc, M, N, nb, mtiles, st);
    return nh == 2 ? launch_tc<TC_W_Q4K, 2, 1>(xt, B, bias, C, ldc, M, N, nb, mtiles, st) : launch_tc<TC_W_Q4K, 1, 2>(xt, B, bias, C, ldc, M, N, nb, mtiles, st);
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
