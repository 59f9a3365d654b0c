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
// One CTA owns a 128 (weight rows) x 128 (tokens) tile of C.  Weight rows are the M = 128 operand of
// tcgen05.mma (they land on the 128 TMEM lanes), tokens are the N = 128 operand (TMEM columns).  Per
// superblock all 8 warps expand the 4-bit weights and the int8 activations into fp16 operand tiles in shared
// memory in the canonical K-major no-swizzle layout (8 x 16-byte core matrices), one thread issues the 17
// MMAs and commits them to an mbarrier, and warps 0-3 (one thread per TMEM lane) drain the accumulators.
// Every wait is bounded; a timeout sets the device error word, frees TMEM and returns.
#include "quant_units.cuh"
#include "pdl.cuh"

namespace ckb {

constexpr int TC_TILE = 128;                         // rows of each operand per CTA
constexpr int TC_KCHUNK_BYTES = TC_TILE * 16;        // one 8-element k-chunk of all 128 rows: 2048 B
constexpr int TC_A_BYTES = 32 * TC_KCHUNK_BYTES;     // 256-deep operand tile: 64 KB
constexpr int TC_A2_BYTES = 2 * TC_KCHUNK_BYTES;     // 16-deep operand tile: 4 KB
constexpr int TC_SMEM = 2 * (TC_A_BYTES + TC_A2_BYTES) + 4 * TC_TILE * 4 + 64;

// shared-memory matrix descriptor: K-major, no swizzle; LBO = distance between the two 8-element k-chunks of
// one MMA (2048 B), SBO = distance between 8-row groups (128 B); version 1 (Blackwell)
__device__ __forceinline__ uint64_t tc_smem_desc(uint32_t addr)
{
    uint64_t d = 0;
    d |= (uint64_t)((addr & 0x3FFFFu) >> 4);
    d |= (uint64_t)(TC_KCHUNK_BYTES >> 4) << 16;
    d |= (uint64_t)(128 >> 4) << 32;
    d |= (uint64_t)1 << 46;
    return d;
}

// instruction descriptor: f16 x f16 -> f32, both operands K-major, M = 128, N = 128
constexpr uint32_t TC_IDESC = (1u << 4) | ((uint32_t)(TC_TILE >> 3) << 17) | ((uint32_t)(TC_TILE >> 4) << 24);

__device__ __forceinline__ void tc_mma(uint32_t tmem_d, uint64_t da, uint64_t db, uint32_t accumulate)
{
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, {%5, %5, %5, %5}, p;\n\t}"
        ::"r"(tmem_d), "l"(da), "l"(db), "r"(TC_IDESC), "r"(accumulate), "r"(0u));
}

__device__ __forceinline__ void tc_ld32(uint32_t taddr, uint32_t (&r)[32])
{
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]),
          "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]),
          "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]),
          "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
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

__device__ __forceinline__ uint32_t tc_tile_offset(int row, int kchunk) { return (uint32_t)(kchunk * TC_KCHUNK_BYTES + (row >> 3) * 128 + (row & 7) * 16); }

__global__ void __launch_bounds__(256, 1) gemm_q4k_tc_kernel(const uint8_t *__restrict__ A_q8, const uint8_t *__restrict__ B, const float *__restrict__ bias,
                                                             float *__restrict__ C, int M, int N, int nb, int *__restrict__ dev_err)
{
    extern __shared__ __align__(128) uint8_t smem[];
    uint8_t *sW = smem;                               // weights  sc*q  [128 x 256] f16
    uint8_t *sW2 = sW + TC_A_BYTES;                   // weights  mins  [128 x 16]
    uint8_t *sX = sW2 + TC_A2_BYTES;                  // tokens   q8    [128 x 256]
    uint8_t *sX2 = sX + TC_A_BYTES;                   // tokens   bsums [128 x 16]
    float *s_dw = reinterpret_cast<float *>(sX2 + TC_A2_BYTES);   // d[n], dmin[n], d_x[m]
    float *s_dmw = s_dw + TC_TILE;
    float *s_dx = s_dmw + TC_TILE;
    uint64_t *bar = reinterpret_cast<uint64_t *>(s_dx + TC_TILE);
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(bar + 1);

    const int tid = threadIdx.x, warp = tid >> 5;
    const int n0 = blockIdx.x * TC_TILE, m0 = blockIdx.y * TC_TILE;
    const uint32_t bar_a = smem_u32(bar);

    if (tid == 0) { mbar_init(bar_a, 1); mbar_fence_init(); }
    if (warp == 0) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(256u));
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;");
    }
    asm volatile("tcgen05.fence::before_thread_sync;");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;");
    const uint32_t tmem = *tmem_slot;                 // lane 0, column 0 of the allocation; T at +0, T2 at +128

    float acc[TC_TILE];
#pragma unroll
    for (int i = 0; i < TC_TILE; ++i) acc[i] = 0.0f;

    bool ok = true;
    for (int b = 0; b < nb && ok; ++b) {
        // ---- expand weights: item = (row, quarter); lanes run over rows so that 8 lanes fill one 128-byte core matrix
        for (int it = tid; it < TC_TILE * 4; it += 256) {
            const int row = it & (TC_TILE - 1), q = it >> 7;
            const uint8_t *p = B + ((size_t)min(n0 + row, N - 1) * nb + b) * Q4K_BYTES;
            const uint4 hdr = __ldg(reinterpret_cast<const uint4 *>(p));
            const uint4 qa = __ldg(reinterpret_cast<const uint4 *>(p + 16 + 32 * q));
            const uint4 qb = __ldg(reinterpret_cast<const uint4 *>(p + 32 + 32 * q));
            uint32_t sc2, m2;
            q4k_scales(hdr.y, hdr.z, hdr.w, q, sc2, m2);
            const float sclo = (float)(sc2 & 255u), schi = (float)(sc2 >> 8);
            const __half2 s_lo = __floats2half2_rn(sclo, sclo), s_hi = __floats2half2_rn(schi, schi);
            const __half2 b_lo = __floats2half2_rn(-1024.0f * sclo, -1024.0f * sclo), b_hi = __floats2half2_rn(-1024.0f * schi, -1024.0f * schi);
            const uint32_t ml = 0x0F0F0F0Fu;
            const uint32_t w[8] = {qa.x, qa.y, qa.z, qa.w, qb.x, qb.y, qb.z, qb.w};
#pragma unroll
            for (int c = 0; c < 4; ++c) {             // sub-block 2q (low nibbles): k-chunks 8q + c; sub-block 2q+1 (high): 8q + 4 + c
                *reinterpret_cast<uint4 *>(sW + tc_tile_offset(row, 8 * q + c)) = q4_chunk_to_half(w[2 * c] & ml, w[2 * c + 1] & ml, s_lo, b_lo);
                *reinterpret_cast<uint4 *>(sW + tc_tile_offset(row, 8 * q + 4 + c)) =
                    q4_chunk_to_half((w[2 * c] >> 4) & ml, (w[2 * c + 1] >> 4) & ml, s_hi, b_hi);
            }
            // the two mins of this quarter, each doubled (bsums come per 16 elements): positions 4q .. 4q+3 of the 16-deep tile
            const float mlo = (float)(m2 & 255u), mhi = (float)(m2 >> 8);
            const __half2 mm_lo = __floats2half2_rn(mlo, mlo), mm_hi = __floats2half2_rn(mhi, mhi);
            uint32_t *dst = reinterpret_cast<uint32_t *>(sW2 + tc_tile_offset(row, q >> 1)) + 2 * (q & 1);
            dst[0] = *reinterpret_cast<const uint32_t *>(&mm_lo);
            dst[1] = *reinterpret_cast<const uint32_t *>(&mm_hi);
            if (q == 0) {
                const float2 dd = __half22float2(*reinterpret_cast<const __half2 *>(&hdr.x));
                s_dw[row] = dd.x;
                s_dmw[row] = dd.y;
            }
        }
        // ---- expand activations: item = (token, k-chunk group of 8 chunks)
        for (int it = tid; it < TC_TILE * 4; it += 256) {
            const int t = it & (TC_TILE - 1), g = it >> 7;
            const uint32_t *blk = reinterpret_cast<const uint32_t *>(A_q8 + ((size_t)min(m0 + t, M - 1) * nb + b) * Q8K_BYTES);
            const bool live = m0 + t < M;
#pragma unroll
            for (int c = 0; c < 8; ++c) {
                const int kc = 8 * g + c;
                const uint32_t w0 = live ? __ldcg(blk + 1 + 2 * kc) : 0u, w1 = live ? __ldcg(blk + 2 + 2 * kc) : 0u;
                *reinterpret_cast<uint4 *>(sX + tc_tile_offset(t, kc)) = s8_chunk_to_half(w0, w1);
            }
            if (g < 2) {                              // bsums[8g .. 8g+7] -> 8 fp16 (|bsum| <= 2048, exact)
                uint32_t o[4];
#pragma unroll
                for (int c = 0; c < 4; ++c) {
                    const uint32_t v = live ? __ldcg(blk + 65 + 4 * g + c) : 0u;
                    const __half2 h = __floats2half2_rn((float)(short)(v & 0xffffu), (float)(short)(v >> 16));
                    o[c] = *reinterpret_cast<const uint32_t *>(&h);
                }
                *reinterpret_cast<uint4 *>(sX2 + tc_tile_offset(t, g)) = make_uint4(o[0], o[1], o[2], o[3]);
            }
            if (g == 3) s_dx[t] = live ? __uint_as_float(__ldcg(blk)) : 0.0f;
        }
        // operand tiles were written through the generic proxy; the tensor core reads them through the async proxy
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        asm volatile("tcgen05.fence::before_thread_sync;");
        __syncthreads();
        if (tid == 0) {
            asm volatile("tcgen05.fence::after_thread_sync;");
            const uint32_t aW = smem_u32(sW), aX = smem_u32(sX);
#pragma unroll 1
            for (int ks = 0; ks < 16; ++ks)
                tc_mma(tmem, tc_smem_desc(aW + ks * 2 * TC_KCHUNK_BYTES), tc_smem_desc(aX + ks * 2 * TC_KCHUNK_BYTES), ks > 0 ? 1u : 0u);
            tc_mma(tmem + 128, tc_smem_desc(smem_u32(sW2)), tc_smem_desc(smem_u32(sX2)), 0u);
            asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar_a) : "memory");
        }
        // everybody waits for the MMAs: the epilogue needs the accumulators, the producers need the operand tiles back
        if (!mbar_wait_bounded(bar_a, b & 1)) ok = false;
        ok = __syncthreads_and(ok);
        if (!ok) break;
        asm volatile("tcgen05.fence::after_thread_sync;");
        if (warp < 4) {
            const float dn = s_dw[tid], dmn = s_dmw[tid];
            const uint32_t lane_base = tmem + ((uint32_t)(warp * 32) << 16);
#pragma unroll
            for (int c0 = 0; c0 < TC_TILE; c0 += 32) {
                uint32_t t1[32], t2[32];
                tc_ld32(lane_base + c0, t1);
                tc_ld32(lane_base + 128 + c0, t2);
                asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
                for (int i = 0; i < 32; ++i)
                    acc[c0 + i] += s_dx[c0 + i] * (dn * __uint_as_float(t1[i]) - dmn * __uint_as_float(t2[i]));
            }
        }
        asm volatile("tcgen05.fence::before_thread_sync;");
        __syncthreads();                              // accumulators drained and scales consumed before the next superblock overwrites them
    }

    if (ok && warp < 4) {
        const int n = n0 + tid;
        if (n < N) {
            const float bv = bias ? bias[n] : 0.0f;
#pragma unroll
            for (int i = 0; i < TC_TILE; ++i)
                if (m0 + i < M) C[(size_t)(m0 + i) * N + n] = acc[i] + bv;
        }
    }
    if (!ok && tid == 0) atomicExch(dev_err, DEV_ERR_MMA_WAIT);
    asm volatile("tcgen05.fence::before_thread_sync;");
    __syncthreads();
    if (warp == 0) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(256u));
}

}  // namespace ckb

using namespace ckb;

// Returns -1 when the shape is not handled here (caller falls back to the per-token path).
extern "C" int ckb_launch_gemm_q4k_tc(const void *A_q8, const void *B, const float *bias, float *C, int M, int N, int K, void *stream)
{
    if (M < 64 || K % QK_K || ((uintptr_t)B & 15) || ((uintptr_t)A_q8 & 3) || ckb_tune_get("gemm_tc", 1) == 0) return -1;
    static int attr_set = 0;
    if (!attr_set) {
        if (ckb_check_cuda((int)cudaFuncSetAttribute(gemm_q4k_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, TC_SMEM), "smem attr")) return CKB_ERR_CUDA;
        attr_set = 1;
    }
    const dim3 grid((N + TC_TILE - 1) / TC_TILE, (M + TC_TILE - 1) / TC_TILE);
    gemm_q4k_tc_kernel<<<grid, 256, TC_SMEM, ckb_stream(stream)>>>((const uint8_t *)A_q8, (const uint8_t *)B, bias, C, M, N, K / QK_K,
                                                                    ckb_device_error_word());
    return ckb_check_launch("gemm_q4k_tc");
}
