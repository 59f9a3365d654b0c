// Q4_K x Q8_K product for a handful of tokens (batched decode, short prompts): C[M, N] = A_q8[M, K] . B[N, K]^T + bias with M <= 64,
// the reference's gemm_nt_q4_k_q8_k (src/kernels/gemm_kernels_q4k_q8k.c:264-281: a loop of gemv_q4_k_q8_k over the tokens).
//
// With so few tokens the product is a weight-streaming problem: every weight byte should cross HBM once and be used for all tokens,
// and the work per byte has to stay below what the stream allows.  The tcgen05 kernel of gemm_tc.cu expands the 4-bit weights into
// fp16 operand tiles in shared memory, which costs the same per weight byte whether 32 or 512 tokens share it (about 1.1 TB/s of
// weights at 32 tokens).  Here the weights are never expanded:
//
//   * a warp owns 16 weight rows and walks its superblocks through a ring of its own in shared memory (plain 16-byte cp.async of
//     the 144-byte blocks, two or three superblocks ahead; no other warp touches it); a lane reads the 8 nibble bytes (rows g and
//     g + 8, bytes 8t .. 8t + 7 of a 32-byte chunk) that ARE its share of the A fragment of mma.sync.m16n8k32 once the nibbles are
//     masked apart: `w & 0x0F0F0F0F` is the fragment of the chunk's low sub-block, `(w >> 4) & 0x0F0F0F0F` of the high one.
//     (The instruction's k index is only a summation index: lane t taking bytes 8t .. 8t + 7 instead of 4t .. 4t + 3 and 16 + 4t ..
//     is a permutation of k that the activation fragment follows.)
//   * the Q8_K activations of all tokens for the current superblock are staged in shared memory once per CTA: a block is 292 bytes,
//     so its 16-byte-aligned window of 19 pieces is copied as it lies (with K a multiple of 1024 the window never leaves the buffer);
//   * one MMA per (sub-block, 8 tokens) gives the exact int32 sums of 32 products; they are scaled by the 6-bit sub-block scale in
//     integer arithmetic and summed over the superblock, the `dmin * m * bsum` term comes from two more MMAs per 8 tokens (the 6-bit
//     minima against the low and the high bytes of the block sums), and once per superblock
//         acc += (d_w * d_x) * float(sum_j sc_j * isum_j) - (dmin_w * d_x) * float(sum_j m_j * bsum_j)
//     - the expression of the GEMV kernels, superblock after superblock.
//
// A CTA is 8 warps: RT row tiles (16 rows each) x KS slices of K; the slices are added in a fixed order through shared memory, so
// the result does not depend on timing.  Integer parts are exact; against the reference's per-sub-block fp32 accumulation the
// result differs by fp32 rounding only (same tolerance as the GEMV).
#include <cuda.h>

#include "device_common.cuh"
#include "launch.h"
#include "pdl.cuh"
#include "runtime.h"

namespace ckb {

constexpr int QM4_THREADS = 256, QM4_WARPS = 8;
constexpr int QM4_TMA_THREADS = QM4_THREADS + 32;             // the bulk-copy kernel: eight computing warps and the warp that issues the copies
constexpr int QM4_XPITCH = 352;                                // bytes between token slots: 304 copied, and 88 words = 24 mod 32 banks
constexpr int QM4_XCOPY = 19;                                  // 16-byte pieces that cover one 292-byte block from its 16-byte-aligned start
constexpr int QM4_WPITCH = 160;                                // bytes between weight rows in a warp's ring (144 copied; 40 words = 8 mod 32)
constexpr int QM4_WTILE = 16 * QM4_WPITCH;                     // one superblock of 16 rows

__device__ __forceinline__ void qm4_cp16(uint32_t dst, const void *src) { asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src) : "memory"); }
__device__ __forceinline__ void qm4_cp4(uint32_t dst, const void *src) { asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(dst), "l"(src) : "memory"); }
__device__ __forceinline__ void qm4_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void qm4_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

// d = a . b (the accumulator input is one zero register four times: no per-instruction clearing of a register quad)
__device__ __forceinline__ void qm4_mma_ss(int (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1, int zero)
{
    asm volatile("mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%10,%10,%10};"
                 : "=r"(d[0]), "=r"(d[1]), "=r"(d[2]), "=r"(d[3]) : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1), "r"(zero));
}
__device__ __forceinline__ void qm4_mma_uu(int (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1, int zero)
{
    asm volatile("mma.sync.aligned.m16n8k32.row.col.s32.u8.u8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%10,%10,%10};"
                 : "=r"(d[0]), "=r"(d[1]), "=r"(d[2]), "=r"(d[3]) : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1), "r"(zero));
}
__device__ __forceinline__ void qm4_mma_us(int (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1, int zero)
{
    asm volatile("mma.sync.aligned.m16n8k32.row.col.s32.u8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%10,%10,%10};"
                 : "=r"(d[0]), "=r"(d[1]), "=r"(d[2]), "=r"(d[3]) : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1), "r"(zero));
}

// One superblock of a warp's 16 RW rows against all token slots.  ws: the warp's row g of its first 16-row tile in shared memory (rows
// WP bytes apart, raw 144-byte Q4_K blocks); xs: token slot 0 (slots XP bytes apart, raw Q8_K block at xs: fp32 d, 256 quants, 16 int16 sums).
template <int NT, int RW, int WP, int XP>
__device__ __forceinline__ void qm4_superblock(const uint8_t *ws, const uint8_t *xs, float (&acc)[RW][NT][4], int g, int t, int zero)
{
    // per 16-row tile: rows g and g + 8; 6-bit scales and minima four to a word (include/ckernel_quant.h:227-251)
    uint32_t scw[RW][2][2], mnw[RW][2][2], dd[RW][2];
#pragma unroll
    for (int rw = 0; rw < RW; ++rw)
#pragma unroll
        for (int r = 0; r < 2; ++r) {
            const uint4 hdr = *reinterpret_cast<const uint4 *>(ws + (size_t)rw * (16 * WP) + r * 8 * WP);
            dd[rw][r] = hdr.x;
            scw[rw][r][0] = hdr.y & 0x3F3F3F3Fu;
            mnw[rw][r][0] = hdr.z & 0x3F3F3F3Fu;
            scw[rw][r][1] = (hdr.w & 0x0F0F0F0Fu) | ((hdr.y >> 2) & 0x30303030u);
            mnw[rw][r][1] = ((hdr.w >> 4) & 0x0F0F0F0Fu) | ((hdr.z >> 2) & 0x30303030u);
        }
    int S[RW][NT][4];
#pragma unroll
    for (int rw = 0; rw < RW; ++rw)
#pragma unroll
        for (int nt = 0; nt < NT; ++nt)
#pragma unroll
            for (int e = 0; e < 4; ++e) S[rw][nt][e] = 0;
#pragma unroll
    for (int c = 0; c < 4; ++c) {
        uint2 q[RW][2];
#pragma unroll
        for (int rw = 0; rw < RW; ++rw) {
            q[rw][0] = *reinterpret_cast<const uint2 *>(ws + (size_t)rw * (16 * WP) + 16 + 32 * c + 8 * t);
            q[rw][1] = *reinterpret_cast<const uint2 *>(ws + (size_t)rw * (16 * WP) + 8 * WP + 16 + 32 * c + 8 * t);
        }
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            const int j = 2 * c + h;
            uint32_t a[RW][4];
            int sc[RW][2];
#pragma unroll
            for (int rw = 0; rw < RW; ++rw) {
                a[rw][0] = (q[rw][0].x >> (4 * h)) & 0x0F0F0F0Fu;
                a[rw][1] = (q[rw][1].x >> (4 * h)) & 0x0F0F0F0Fu;
                a[rw][2] = (q[rw][0].y >> (4 * h)) & 0x0F0F0F0Fu;
                a[rw][3] = (q[rw][1].y >> (4 * h)) & 0x0F0F0F0Fu;
                sc[rw][0] = (int)__byte_perm(scw[rw][0][j >> 2], 0u, 0x4440u + (j & 3));
                sc[rw][1] = (int)__byte_perm(scw[rw][1][j >> 2], 0u, 0x4440u + (j & 3));
            }
#pragma unroll
            for (int nt = 0; nt < NT; ++nt) {
                const uint32_t *bp = reinterpret_cast<const uint32_t *>(xs + (size_t)(nt * 8 + g) * XP + 4 + 32 * j + 8 * t);
                const uint32_t b0 = bp[0], b1 = bp[1];
#pragma unroll
                for (int rw = 0; rw < RW; ++rw) {
                    int cc[4];
                    qm4_mma_ss(cc, a[rw], b0, b1, zero);
                    S[rw][nt][0] += sc[rw][0] * cc[0];
                    S[rw][nt][1] += sc[rw][0] * cc[1];
                    S[rw][nt][2] += sc[rw][1] * cc[2];
                    S[rw][nt][3] += sc[rw][1] * cc[3];
                }
            }
        }
    }
    // minima: k index i = 0 .. 15 is the 16-element block sum i, which belongs to sub-block i / 2
    uint32_t am[RW][4];
    float dw[RW][2], mw[RW][2];
#pragma unroll
    for (int rw = 0; rw < RW; ++rw) {
        const uint32_t sel = (t & 1) ? 0x3322u : 0x1100u;
        am[rw][0] = __byte_perm((t & 2) ? mnw[rw][0][1] : mnw[rw][0][0], 0u, sel);
        am[rw][1] = __byte_perm((t & 2) ? mnw[rw][1][1] : mnw[rw][1][0], 0u, sel);
        am[rw][2] = 0u;
        am[rw][3] = 0u;
#pragma unroll
        for (int r = 0; r < 2; ++r) {
            dw[rw][r] = half_bits_to_float(dd[rw][r] & 0xFFFFu);
            mw[rw][r] = half_bits_to_float(dd[rw][r] >> 16);
        }
    }
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) {
        const uint32_t *bsp = reinterpret_cast<const uint32_t *>(xs + (size_t)(nt * 8 + g) * XP + 260 + 8 * t);
        const uint32_t bs0 = bsp[0], bs1 = bsp[1];
        const uint32_t lo = __byte_perm(bs0, bs1, 0x6420u), hi = __byte_perm(bs0, bs1, 0x7531u);
        const float dxa = *reinterpret_cast<const float *>(xs + (size_t)(nt * 8 + 2 * t) * XP);
        const float dxb = *reinterpret_cast<const float *>(xs + (size_t)(nt * 8 + 2 * t + 1) * XP);
#pragma unroll
        for (int rw = 0; rw < RW; ++rw) {
            int Lo[4], Hi[4];
            qm4_mma_uu(Lo, am[rw], lo, 0u, zero);
            qm4_mma_us(Hi, am[rw], hi, 0u, zero);
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const float d = dw[rw][e >> 1], dm = mw[rw][e >> 1], x = (e & 1) ? dxb : dxa;
                const int ms = Hi[e] * 256 + Lo[e];
                acc[rw][nt][e] += __fmul_rn(d, x) * (float)S[rw][nt][e] - __fmul_rn(dm, x) * (float)ms;
            }
        }
    }
}

template <int NT, int RW, int KS, int D> struct Qm4Smem {
    static constexpr int MT = 8 * NT;
    static constexpr int XSLICE = MT * QM4_XPITCH;             // one superblock of all token slots
    static constexpr int WSTAGE = RW * QM4_WTILE;              // one superblock of a warp's rows
    static constexpr int STAGE = QM4_WARPS * WSTAGE + KS * XSLICE;
    static constexpr int BYTES = D * STAGE;
};

// NT: 8-token tiles (tokens padded to 8 NT); RW: 16-row tiles per warp (an activation fragment is read from shared memory once and used
// for all of them); RT x KS warps; D: stages of both rings.  W: [N][nb] Q4_K blocks, 16-byte aligned; X: [M][nb] Q8_K blocks; C[m * ldc + n].
// x_aligned: X is 16-byte aligned and nb a multiple of 4; then every block's 16-byte-aligned window of 19 pieces stays inside the buffer,
// all tokens share the block's offset within its window, and the blocks are copied 16 bytes at a time (otherwise 4 bytes at a time).
template <int NT, int RW, int RT, int KS, int D>
__global__ void __launch_bounds__(QM4_THREADS) gemm_q4k_mma_kernel(const uint8_t *__restrict__ W, const uint8_t *__restrict__ X, const float *__restrict__ bias,
                                                                   float *__restrict__ C, int ldc, int M, int N, int nb, int x_aligned)
{
    static_assert(RT * KS == QM4_WARPS, "8 warps");
    using L = Qm4Smem<NT, RW, KS, D>;
    constexpr int MT = L::MT;
    extern __shared__ __align__(128) uint8_t qm4_smem[];
    const uint32_t s_base = smem_u32(qm4_smem);
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int g = lane >> 2, t = lane & 3;
    const int rt = warp % RT, ks = warp / RT;
    const int n0 = (blockIdx.x * RT + rt) * 16 * RW;
    const int per = (nb + KS - 1) / KS;                        // superblocks per K slice; every warp takes `per` steps
    const size_t wrow = (size_t)nb * Q4K_BYTES, xrow = (size_t)nb * Q8K_BYTES;
    const int b_first = ks * per;

    // token slots beyond M stay zero in every stage: their fragments are zero and their outputs are never stored
    for (int i = tid; i < L::BYTES / 16; i += QM4_THREADS) reinterpret_cast<uint4 *>(qm4_smem)[i] = make_uint4(0u, 0u, 0u, 0u);
    __syncthreads();
    pdl_trigger();

    // a warp's own 16 RW rows of superblock b_first + s: 9 pieces per row, consecutive lanes on consecutive pieces; where a lane's
    // pieces lie (relative to the warp's first row and to its stage) does not change from step to step
    constexpr int WPIECES = (144 * RW + 31) / 32;
    uint32_t wsrc[WPIECES], wdst[WPIECES];
#pragma unroll
    for (int i = 0; i < WPIECES; ++i) {
        const int p = min(lane + 32 * i, 144 * RW - 1), row = p / 9, part = p - row * 9;
        wsrc[i] = (uint32_t)((size_t)(min(n0 + row, N - 1) - min(n0, N - 1)) * wrow) + 16u * part;
        wdst[i] = (uint32_t)(row * QM4_WPITCH + 16 * part);
    }
    const uint8_t *wbase = W + (size_t)min(n0, N - 1) * wrow;
    auto issue_w = [&](int s) {
        const int b = b_first + s;
        if (s < per && b < nb) {
            const uint32_t dst = s_base + (uint32_t)(s % D) * L::STAGE + (uint32_t)warp * L::WSTAGE;
            const uint8_t *src = wbase + (size_t)b * Q4K_BYTES;
#pragma unroll
            for (int i = 0; i < WPIECES; ++i)
                if (lane + 32 * i < 144 * RW) qm4_cp16(dst + wdst[i], src + wsrc[i]);
        }
    };
    // activations of step s: slice k holds superblock k * per + s, every token's block from its 16-byte-aligned start
    auto issue_x = [&](int s) {
        if (s < per) {
            const uint32_t st = s_base + (uint32_t)(s % D) * L::STAGE + QM4_WARPS * L::WSTAGE;
            for (int k = 0; k < KS; ++k) {
                const int b = k * per + s;
                if (b >= nb) break;
                const uint32_t dst = st + (uint32_t)k * L::XSLICE;
                if (x_aligned) {
                    const uint8_t *src = X + (((size_t)b * Q8K_BYTES) & ~(size_t)15);
                    for (int r = tid; r < M * QM4_XCOPY; r += QM4_THREADS) {
                        const int tok = r / QM4_XCOPY, piece = r - tok * QM4_XCOPY;
                        qm4_cp16(dst + (uint32_t)(tok * QM4_XPITCH + 16 * piece), src + (size_t)tok * xrow + 16 * piece);
                    }
                } else {
                    const uint8_t *src = X + (size_t)b * Q8K_BYTES;
                    for (int r = tid; r < M * (Q8K_BYTES / 4); r += QM4_THREADS) {
                        const int tok = r / (Q8K_BYTES / 4), piece = r - tok * (Q8K_BYTES / 4);
                        qm4_cp4(dst + (uint32_t)(tok * QM4_XPITCH + 4 * piece), src + (size_t)tok * xrow + 4 * piece);
                    }
                }
            }
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

    // weights are not written by any kernel: their first stages start before the dependency wait
    for (int s = 0; s < D - 1; ++s) issue_w(s);
    pdl_wait();
    for (int s = 0; s < D - 1; ++s) { issue_x(s); qm4_commit(); }      // group s = activations of step s (+ all early weight stages in group 0)

    for (int s = 0; s < per; ++s) {
        const int b = b_first + s;
        qm4_wait<D - 2>();                                     // this thread's pieces of step s
        __syncthreads();                                       // everyone's pieces; and step s - 1 is finished everywhere: its stage may be refilled
        issue_w(s + D - 1);
        issue_x(s + D - 1);
        qm4_commit();
        if (b >= nb) continue;
        const uint8_t *stage = qm4_smem + (size_t)(s % D) * L::STAGE;
        const uint8_t *ws = stage + (size_t)warp * L::WSTAGE + g * QM4_WPITCH;
        const uint8_t *xs = stage + QM4_WARPS * L::WSTAGE + (size_t)ks * L::XSLICE + (x_aligned ? (int)(((size_t)b * Q8K_BYTES) & 15) : 0);

        qm4_superblock<NT, RW, QM4_WPITCH, QM4_XPITCH>(ws, xs, acc, g, t, zero);
    }
    qm4_wait<0>();
    __syncthreads();                                           // the staging area becomes the reduction buffer

    // slices in order 0, 1, ..: slice k > 0 parks its sums, the warps of slice 0 add them and store
    float *red = reinterpret_cast<float *>(qm4_smem);
    constexpr int PER_WARP = RW * NT * 4;
    if (KS > 1 && ks > 0) {
#pragma unroll
        for (int rw = 0; rw < RW; ++rw)
#pragma unroll
            for (int nt = 0; nt < NT; ++nt)
#pragma unroll
                for (int e = 0; e < 4; ++e) red[(((size_t)(ks - 1) * RT + rt) * PER_WARP + (rw * NT + nt) * 4 + e) * 32 + lane] = acc[rw][nt][e];
    }
    if (KS > 1) __syncthreads();
    if (ks == 0) {
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

// ---------------------------------------------------------------------------------------------------------------------------------
// The same product with both operands brought in by the tensor-memory accelerator.  In the kernel above a third of every step went
// into issuing the step's 16-byte copies (about 2900 requests per CTA and step through the load/store units: measured with clock64,
// and neither spreading the requests over the step nor a warp of its own for them helped).  Here one thread issues, per step and K
// slice, ONE tiled copy for the 144-byte blocks of all the slice's rows (a box of 144 bytes x rows out of the matrix seen as
// N rows of nb * 144 bytes) and one for the 304-byte windows of all tokens; rows past N and token slots past M are filled with
// zeros by the copy itself.  That thread is the first lane of a ninth warp which does nothing else: completion is counted on a
// `full` mbarrier per stage, each of the eight computing warps releases a stage on its `empty` mbarrier when it is done with it,
// and there is no CTA-wide barrier inside the K loop (with the copies issued by a computing warp behind such a barrier, CTAs with
// four K slices lost up to a third of their time at it).  All waits are bounded.  Needs 16-byte-aligned activation rows (K a
// multiple of 1024), otherwise the kernel above runs.
constexpr int QM4_XWIN = 16 * QM4_XCOPY;                       // 304 bytes: a 292-byte block from its 16-byte-aligned start

__device__ __forceinline__ void qm4_tma_2d(uint32_t dst, const CUtensorMap *map, int x, int y, uint32_t bar)
{
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
                 ::"r"(dst), "l"(map), "r"(x), "r"(y), "r"(bar) : "memory");
}

template <int NT, int RW, int KS, int D> struct Qm4TmaSmem {
    static constexpr int MT = 8 * NT;
    static constexpr int ROWS = 16 * RW * (QM4_WARPS / KS);    // rows of one K slice = rows of the CTA
    static constexpr int WSLICE = ROWS * Q4K_BYTES;            // dense 144-byte rows
    static constexpr int XSLICE = ((MT * QM4_XWIN + 127) / 128) * 128;
    static constexpr int STAGE = KS * (WSLICE + XSLICE);
    static constexpr int BYTES = D * STAGE;
    static_assert(WSLICE % 128 == 0, "copy destinations stay 128-byte aligned");
};

template <int NT, int RW, int RT, int KS, int D>
__global__ void __launch_bounds__(QM4_TMA_THREADS) gemm_q4k_mma_tma_kernel(const __grid_constant__ CUtensorMap tm_w, const __grid_constant__ CUtensorMap tm_x,
                                                                       const float *__restrict__ bias, float *__restrict__ C, int ldc, int M, int N, int nb,
                                                                       int *__restrict__ dev_err)
{
    static_assert(RT * KS == QM4_WARPS, "8 warps");
    using L = Qm4TmaSmem<NT, RW, KS, D>;
    extern __shared__ __align__(128) uint8_t qm4_smem[];
    __shared__ __align__(8) uint64_t full[D], empty[D];
    const uint32_t s_base = smem_u32(qm4_smem);
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int g = lane >> 2, t = lane & 3;
    const int rt = warp % RT, ks = warp / RT;
    const int row0 = blockIdx.x * L::ROWS;                     // first row of the CTA
    const int per = (nb + KS - 1) / KS;
    const int b_first = ks * per;

    if (tid == 0) {
        for (int i = 0; i < D; ++i) { mbar_init(smem_u32(&full[i]), 1); mbar_init(smem_u32(&empty[i]), QM4_WARPS); }
        mbar_fence_init();
    }
    __syncthreads();
    pdl_trigger();

    // the issuing thread: the copies of step s; weights and activations of a stage complete the same barrier
    auto expect = [&](int s) {
        int slices = 0;
        for (int k = 0; k < KS; ++k) slices += (k * per + s < nb);
        mbar_arrive_expect_tx(smem_u32(&full[s % D]), (uint32_t)slices * (uint32_t)(L::WSLICE + L::MT * QM4_XWIN));
    };
    auto issue_w = [&](int s) {
        const uint32_t st = s_base + (uint32_t)(s % D) * L::STAGE;
        for (int k = 0; k < KS; ++k) {
            const int b = k * per + s;
            if (b < nb) qm4_tma_2d(st + (uint32_t)k * (L::WSLICE + L::XSLICE), &tm_w, b * Q4K_BYTES, row0, smem_u32(&full[s % D]));
        }
    };
    auto issue_x = [&](int s) {
        const uint32_t st = s_base + (uint32_t)(s % D) * L::STAGE + L::WSLICE;
        for (int k = 0; k < KS; ++k) {
            const int b = k * per + s;
            // the activation matrix is described in 4-byte elements (a box side is at most 256 elements): window start / 4
            if (b < nb) qm4_tma_2d(st + (uint32_t)k * (L::WSLICE + L::XSLICE), &tm_x, ((b * Q8K_BYTES) & ~15) / 4, 0, smem_u32(&full[s % D]));
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
    // computing warp waits for another between steps.
    if (warp == QM4_WARPS) {
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
            ok = false;                                        // the host sees the error word
            if (lane == 0) atomicExch(dev_err, DEV_ERR_FULL_WAIT);
        }
        const uint8_t *slice = qm4_smem + (size_t)(s % D) * L::STAGE + (size_t)ks * (L::WSLICE + L::XSLICE);
        const uint8_t *ws = slice + (size_t)(rt * 16 * RW + g) * Q4K_BYTES;
        const uint8_t *xs = slice + L::WSLICE + ((b * Q8K_BYTES) & 15);
        qm4_superblock<NT, RW, Q4K_BYTES, QM4_XWIN>(ws, xs, acc, g, t, zero);
    }
    }
    __syncthreads();                                           // the staging area becomes the reduction buffer (every issued copy was waited for)

    float *red = reinterpret_cast<float *>(qm4_smem);
    constexpr int PER_WARP = RW * NT * 4;
    if (KS > 1 && ks > 0 && warp < QM4_WARPS) {
#pragma unroll
        for (int rw = 0; rw < RW; ++rw)
#pragma unroll
            for (int nt = 0; nt < NT; ++nt)
#pragma unroll
                for (int e = 0; e < 4; ++e) red[(((size_t)(ks - 1) * RT + rt) * PER_WARP + (rw * NT + nt) * 4 + e) * 32 + lane] = acc[rw][nt][e];
    }
    if (KS > 1) __syncthreads();
    if (ks == 0 && warp < QM4_WARPS) {
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

// Tiled copy descriptors: a matrix of `rows` rows of `row_bytes` bytes (row pitch = row_bytes, a multiple of 16), boxes of box_bytes x box_rows,
// in elements of `elem` bytes (1 or 4).
typedef CUresult (*qm4_encode_fn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *, const cuuint64_t *, const cuuint32_t *,
                                  const cuuint32_t *, CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
static qm4_encode_fn qm4_encoder()
{
    static qm4_encode_fn fn = nullptr;
    static bool tried = false;
    if (!tried) {
        tried = true;
        void *p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess && q == cudaDriverEntryPointSuccess) fn = (qm4_encode_fn)p;
        else cudaGetLastError();
    }
    return fn;
}
static bool qm4_make_map(CUtensorMap *map, const void *base, size_t row_bytes, size_t rows, unsigned box_bytes, unsigned box_rows, unsigned elem)
{
    qm4_encode_fn enc = qm4_encoder();
    if (!enc || row_bytes % 16 || box_bytes % 16 || box_bytes / elem > 256 || box_rows > 256) return false;
    const cuuint64_t dims[2] = {(cuuint64_t)(row_bytes / elem), (cuuint64_t)rows}, strides[1] = {(cuuint64_t)row_bytes};
    const cuuint32_t box[2] = {box_bytes / elem, box_rows}, estr[2] = {1, 1};
    return enc(map, elem == 4 ? CU_TENSOR_MAP_DATA_TYPE_UINT32 : CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void *>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE,
               CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

// -1: this form does not apply (no driver entry point, activations not 16-byte aligned, shared memory)
template <int NT, int RW, int RT, int KS, int D>
static int qm4_launch_tma(const void *A_q8, const void *B, const float *bias, float *C, int ldc, int M, int N, int nb, cudaStream_t st)
{
    using L = Qm4TmaSmem<NT, RW, KS, D>;
    static_assert((KS - 1) * RT * RW * NT * 4 * 32 * 4 <= L::BYTES, "the reduction buffer fits into the staging area");
    static_assert(L::BYTES <= 226 * 1024, "shared memory");
    static_assert(L::ROWS <= 256 && L::MT <= 256 && QM4_XWIN / 4 <= 256 && Q4K_BYTES <= 256, "box limits");
    if (((uintptr_t)A_q8 & 15) || nb % 4 || ((uintptr_t)B & 15)) return -1;
    CUtensorMap tm_w, tm_x;
    if (!qm4_make_map(&tm_w, B, (size_t)nb * Q4K_BYTES, (size_t)N, Q4K_BYTES, L::ROWS, 1)) return -1;
    if (!qm4_make_map(&tm_x, A_q8, (size_t)nb * Q8K_BYTES, (size_t)M, QM4_XWIN, L::MT, 4)) return -1;
    static bool attr_set = false;
    if (!attr_set) {
        if (ckb_check_cuda((int)cudaFuncSetAttribute(gemm_q4k_mma_tma_kernel<NT, RW, RT, KS, D>, cudaFuncAttributeMaxDynamicSharedMemorySize, L::BYTES), "gemm_q4k_mma smem"))
            return CKB_ERR_CUDA;
        attr_set = true;
    }
    const int grid = (N + L::ROWS - 1) / L::ROWS;
    return launch_pdl("gemm_q4k_mma_tma", gemm_q4k_mma_tma_kernel<NT, RW, RT, KS, D>, dim3(grid), dim3(QM4_TMA_THREADS), (size_t)L::BYTES, st, tm_w, tm_x, bias, C, ldc, M, N,
                      nb, ckb_device_error_word());
}

template <int NT, int RW, int RT, int KS, int D>
static int qm4_launch(const void *A_q8, const void *B, const float *bias, float *C, int ldc, int M, int N, int nb, cudaStream_t st)
{
    constexpr int smem = Qm4Smem<NT, RW, KS, D>::BYTES;
    static_assert((KS - 1) * RT * RW * NT * 4 * 32 * 4 <= smem, "the reduction buffer fits into the staging area");
    static_assert(smem <= 227 * 1024, "shared memory");
    static bool attr_set = false;
    if (!attr_set) {
        if (ckb_check_cuda((int)cudaFuncSetAttribute(gemm_q4k_mma_kernel<NT, RW, RT, KS, D>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem), "gemm_q4k_mma smem"))
            return CKB_ERR_CUDA;
        attr_set = true;
    }
    const int rows = 16 * RW * RT, grid = (N + rows - 1) / rows;
    const int x_aligned = !((uintptr_t)A_q8 & 15) && nb % 4 == 0;
    return launch_pdl("gemm_q4k_mma", gemm_q4k_mma_kernel<NT, RW, RT, KS, D>, dim3(grid), dim3(QM4_THREADS), (size_t)smem, st, (const uint8_t *)B, (const uint8_t *)A_q8,
                      bias, C, ldc, M, N, nb, x_aligned);
}

// shape: rows per CTA / K slices.  1: 8 row warps; 2: 4 row warps x 2 slices; 4: 2 row warps x 4 slices.
template <int NT, int RW>
static int qm4_shape(int shape, const void *A_q8, const void *B, const float *bias, float *C, int ldc, int M, int N, int nb, cudaStream_t st)
{
    constexpr int per_stage1 = QM4_WARPS * RW * QM4_WTILE + 8 * NT * QM4_XPITCH, per_stage2 = per_stage1 + 8 * NT * QM4_XPITCH, per_stage4 = per_stage2 + 2 * 8 * NT * QM4_XPITCH;
    constexpr int D1 = 4 * per_stage1 <= 227 * 1024 ? 4 : (3 * per_stage1 <= 227 * 1024 ? 3 : 2), D2 = 4 * per_stage2 <= 227 * 1024 ? 4 : (3 * per_stage2 <= 227 * 1024 ? 3 : 2);
    constexpr int D4 = 4 * per_stage4 <= 227 * 1024 ? 4 : (3 * per_stage4 <= 227 * 1024 ? 3 : 2);
    if (ckb_tune_get("gemm_q4k_mma_tma", 1)) {
        // stages of the tiled-copy form: dense rows, so more of them fit
        constexpr int w1 = QM4_WARPS * 16 * RW * Q4K_BYTES;
        constexpr int t1 = w1 + Qm4TmaSmem<NT, RW, 1, 1>::XSLICE, t2 = w1 + 2 * Qm4TmaSmem<NT, RW, 2, 1>::XSLICE, t4 = w1 + 4 * Qm4TmaSmem<NT, RW, 4, 1>::XSLICE;
        constexpr int T1 = 4 * t1 <= 226 * 1024 ? 4 : 3, T2 = 4 * t2 <= 226 * 1024 ? 4 : 3, T4 = 4 * t4 <= 226 * 1024 ? 4 : (3 * t4 <= 226 * 1024 ? 3 : 2);
        const int rc = shape == 1 ? qm4_launch_tma<NT, RW, 8, 1, T1>(A_q8, B, bias, C, ldc, M, N, nb, st)
                                  : (shape == 2 ? qm4_launch_tma<NT, RW, 4, 2, T2>(A_q8, B, bias, C, ldc, M, N, nb, st)
                                                : qm4_launch_tma<NT, RW, 2, 4, T4>(A_q8, B, bias, C, ldc, M, N, nb, st));
        if (rc >= 0) return rc;
    }
    if (shape == 1) return qm4_launch<NT, RW, 8, 1, D1>(A_q8, B, bias, C, ldc, M, N, nb, st);
    if (shape == 2) return qm4_launch<NT, RW, 4, 2, D2>(A_q8, B, bias, C, ldc, M, N, nb, st);
    return qm4_launch<NT, RW, 2, 4, D4>(A_q8, B, bias, C, ldc, M, N, nb, st);
}

// Shape by measurement on B200 (Llama-3-70B and 8B projection shapes, 8 to 64 tokens): the widest CTA (most rows per staged activation
// block) that still gives three quarters of the SMs a CTA; K slices make up for rows when there are few.
static int qm4_auto_shape(int rows_per_warp, int N, int nb, int want)
{
    for (int shape = 1; shape < 4; shape *= 2) {
        const int rows = rows_per_warp * 8 / shape;
        if ((N + rows - 1) / rows >= want || nb < 2 * shape) return shape;
    }
    return nb >= 4 ? 4 : (nb >= 2 ? 2 : 1);
}

template <int NT>
static int qm4_pick(const void *A_q8, const void *B, const float *bias, float *C, int ldc, int M, int N, int nb, cudaStream_t st)
{
    int rw = ckb_tune_get("gemm_q4k_mma_rw", 0);               // 16-row tiles per warp: 0 auto, 1, 2 (64 token slots: always 1, registers)
    const int want = 3 * ckb_sm_count() / 4;
    // Up to 8 tokens one tile per warp is as fast or faster everywhere (57344 x 8192: 55 us against 60); 9 to 16 tokens only on very
    // tall matrices.  There two K slices per CTA beat eight row warps when K is long (measured on the 70B and 8B projections).
    const bool tall = (N + 63) / 64 >= 4 * want && nb >= 32;
    const bool narrow = NT == 1 || (NT == 2 && tall);
    if (NT >= 8) rw = 1;
    else if (rw != 1 && rw != 2) rw = !narrow && (N + 63) / 64 >= want ? 2 : 1;
    int shape = ckb_tune_get("gemm_q4k_mma_shape", 0);         // 1: 8 row warps, 2: 4 x 2 K slices, 4: 2 x 4 K slices, 0 auto
    if (shape != 1 && shape != 2 && shape != 4) {
        shape = qm4_auto_shape(16 * rw, N, nb, narrow && rw == 1 ? 2 * want : want);       // small CTAs: two per SM wanted (8192 x 8192, 8 tokens: 9.8 us against 16.1)
        if (shape == 1 && narrow && rw == 1 && nb >= 32) shape = 2;
    }
    // From 17 tokens up a CTA fills its SM, so a grid of whole waves plus a part of one pays a whole wave for the part (57344 rows
    // in CTAs of 256 on 148 SMs: 148 + 76).  The rows behind the whole waves then go to a second launch in smaller CTAs (one tile
    // per warp), which spreads them over all SMs.  (Up to 16 tokens several CTAs share an SM and start as others end: there the
    // same tail launch measured slower, 58 against 55 us at 8 tokens on the same matrix.)
    if constexpr (NT >= 4) {
        const int sms = ckb_sm_count();
        const bool tail_on = ckb_tune_get("gemm_q4k_mma_tail", 1) != 0;
        if (tail_on && ckb_tune_get("gemm_q4k_mma_shape", 0) == 0) {
            // time of a shape ~ rows per CTA x (whole waves + the last, partial one; a small remainder costs little once it is a tail
            // launch), with 8 % per halving of the CTA for the activation traffic and pipeline starts that grow with the CTA count
            // (57344 x 8192, 32 tokens: 224 CTAs of 256 rows 114 us, 448 of 128 with a 4-CTA tail 109 us)
            double best_cost = 0.0;
            int best_shape = shape;
            for (int cand = shape, halvings = 0; cand <= 4 && nb >= 2 * cand; cand *= 2, ++halvings) {
                const int rows_c = 16 * rw * 8 / cand, ctas_c = (N + rows_c - 1) / rows_c, rem_c = ctas_c % sms;
                if (cand == shape && ctas_c <= sms) break;                 // one wave: nothing to gain
                const double last = rem_c == 0 ? 0.0 : (4 * rem_c <= sms && N % rows_c == 0 ? 0.3 : 1.0);
                const double cost = (double)rows_c * ((double)(ctas_c / sms) + last) * (1.0 + 0.08 * halvings);
                if (best_cost == 0.0 || cost < best_cost) { best_cost = cost; best_shape = cand; }
            }
            shape = best_shape;
        }
        const int rows = 16 * rw * 8 / shape, ctas = (N + rows - 1) / rows, rem = ctas % sms;
        if (tail_on && ctas > sms && N % rows == 0 && rem > 0 && 4 * rem <= sms) {
            const int n_main = (ctas - rem) * rows, n_tail = N - n_main;
            int rc;
            if constexpr (NT < 8) {
                rc = rw == 2 ? qm4_shape<NT, 2>(shape, A_q8, B, bias, C, ldc, M, n_main, nb, st) : qm4_shape<NT, 1>(shape, A_q8, B, bias, C, ldc, M, n_main, nb, st);
            } else {
                rc = qm4_shape<NT, 1>(shape, A_q8, B, bias, C, ldc, M, n_main, nb, st);
            }
            if (rc) return rc;
            const int shape_t = qm4_auto_shape(16, n_tail, nb, want);
            return qm4_shape<NT, 1>(shape_t, A_q8, (const uint8_t *)B + (size_t)n_main * nb * Q4K_BYTES, bias ? bias + n_main : nullptr, C + n_main, ldc, M, n_tail, nb, st);
        }
    }
    if constexpr (NT < 8) {
        if (rw == 2) return qm4_shape<NT, 2>(shape, A_q8, B, bias, C, ldc, M, N, nb, st);
    }
    return qm4_shape<NT, 1>(shape, A_q8, B, bias, C, ldc, M, N, nb, st);
}

}  // namespace ckb

using namespace ckb;

// Returns -1 when this kernel does not take the call (token count, alignment, switched off): the caller falls through to its other paths.
// Whether the launcher below takes this product (a caller that wants to run several products side by side asks first: this
// kernel needs no workspace, the tcgen05 kernel shares one).
extern "C" int ckb_gemm_q4k_mma_takes(const void *A_q8, const void *B, int M, int N, int K)
{
    if (!A_q8 || !B || N <= 0 || K <= 0 || K % QK_K) return 0;
    // from 2 tokens up one pass of this kernel beats a GEMV per token (measured: up to 8 tokens cost about 1.2 GEMVs on the 57344 x 8192 shape)
    if (M < ckb_tune_get("gemm_q4k_mma_min", 2) || M > ckb_tune_get("gemm_q4k_mma_max", 64) || M > 64 || !ckb_tune_get("gemm_q4k_mma", 1)) return 0;
    return !(((uintptr_t)B & 15) || ((uintptr_t)A_q8 & 3));
}

extern "C" int ckb_launch_gemm_q4k_mma(const void *A_q8, const void *B, const float *bias, float *C, int ldc, int M, int N, int K, void *stream)
{
    if (!C || !ckb_gemm_q4k_mma_takes(A_q8, B, M, N, K)) return -1;
    if (ckb_ensure_init()) return CKB_ERR_NO_DEVICE;
    cudaStream_t st = ckb_stream(stream);
    const int nb = K / QK_K;
    if (M <= 8) return qm4_pick<1>(A_q8, B, bias, C, ldc, M, N, nb, st);
    if (M <= 16) return qm4_pick<2>(A_q8, B, bias, C, ldc, M, N, nb, st);
    if (M <= 32) return qm4_pick<4>(A_q8, B, bias, C, ldc, M, N, nb, st);
    return qm4_pick<8>(A_q8, B, bias, C, ldc, M, N, nb, st);
}
