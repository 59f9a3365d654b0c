// Fused glue kernels of a device-resident decode step.  Each merges ops that the reference's
// generated decode function issues one after another (version/v7/scripts/codegen_v7.py:569-931):
//
//   add_rmsnorm_q8k   ck_residual_add_token_major + rmsnorm_forward + quantize_row_q8_k
//   swiglu_q8k        swiglu_forward + quantize_row_q8_k
//   rope_kv_store     rope_forward_qk + kv_cache_store
//   advance_pos       model->pos++
//
// The arithmetic of each op is the one in glue.cu / quantize.cu; fusing only removes launches and
// the fp32 round trip through HBM.  All kernels are PDL-aware (pdl.cuh): they may start while their
// producer is still running, so everything a previous kernel wrote is read with __ldcg (through L2);
// the read-only / L1 paths are not coherent across a programmatic launch.  Weights (gamma, cos/sin)
// are never written by a kernel and may use any path.
#include "add_rmsnorm_q8k.cuh"
#include "pdl.cuh"
#include "q8k_block.cuh"

namespace ckb {

// grid = tokens, block = aligned / 4 threads rounded up to a warp multiple, at most 1024.
// x[t] += delta[t] (when delta != NULL; x is updated in place), then h = rmsnorm(x[t]) * gamma, zero beyond
// d_model, quantised to Q8_K blocks of `aligned` elements.  Optionally also writes the fp32 normalised row.
// Every thread issues all of its 16-byte loads before it uses any of them (one L2 round trip per row).
__global__ void __launch_bounds__(1024) add_rmsnorm_q8k_kernel(float *__restrict__ x, const float *__restrict__ delta,
                                                               const float *__restrict__ gamma, uint8_t *__restrict__ out_q8,
                                                               float *__restrict__ norm_out, int d_model, int aligned, float eps)
{
    extern __shared__ __align__(16) float row[];
    __shared__ float red[32];
    pdl_trigger();
    const ArqGamma pre = arq_prefetch_gamma(gamma, d_model);
    pdl_wait();
    const int t = blockIdx.x;
    float *xr = x + (size_t)t * aligned;
    const float *dr = delta ? delta + (size_t)t * aligned : nullptr;
    const int nv = aligned >> 2;
    float4 xv[ARQ_MAX_V4], dv[ARQ_MAX_V4];
#pragma unroll
    for (int k = 0; k < ARQ_MAX_V4; ++k) {
        const int i = threadIdx.x + k * blockDim.x;
        xv[k] = make_float4(0.f, 0.f, 0.f, 0.f);
        dv[k] = xv[k];
        if (i < nv) {
            xv[k] = __ldcg(reinterpret_cast<const float4 *>(xr) + i);
            if (dr) dv[k] = __ldcg(reinterpret_cast<const float4 *>(dr) + i);
        }
    }
    float ss = 0.0f;
#pragma unroll
    for (int k = 0; k < ARQ_MAX_V4; ++k) {
        const int i = threadIdx.x + k * blockDim.x;
        if (i < nv) {
            float4 v = xv[k];
            if (dr) {
                v.x += dv[k].x; v.y += dv[k].y; v.z += dv[k].z; v.w += dv[k].w;
                reinterpret_cast<float4 *>(xr)[i] = v;                 // pad columns of x and delta are zero by construction
            }
            arq_keep_piece(v, i, d_model, row, ss);
        }
    }
    arq_norm_quant(ss, row, red, gamma, out_q8, norm_out, t, d_model, aligned, eps, &pre);
}

// add_rmsnorm_q8k for a consumer that takes Q8_0 activations (Q8_0 / Q5_0 weights): the same row kernel, Q8_0 blocks of the
// first `cols` elements out
__global__ void __launch_bounds__(1024) add_rmsnorm_q80_kernel(float *__restrict__ x, const float *__restrict__ delta, const float *__restrict__ gamma,
                                                               uint8_t *__restrict__ out_q80, int d_model, int aligned, int cols, float eps)
{
    extern __shared__ __align__(16) float row[];
    __shared__ float red[32];
    pdl_trigger();
    pdl_wait();
    const int t = blockIdx.x;
    float *xr = x + (size_t)t * aligned;
    const float *dr = delta ? delta + (size_t)t * aligned : nullptr;
    const int nv = aligned >> 2;
    float ss = 0.0f;
    for (int i = threadIdx.x; i < nv; i += blockDim.x) {
        float4 v = __ldcg(reinterpret_cast<const float4 *>(xr) + i);
        if (dr) {
            const float4 dv = __ldcg(reinterpret_cast<const float4 *>(dr) + i);
            v.x += dv.x; v.y += dv.y; v.z += dv.z; v.w += dv.w;
            reinterpret_cast<float4 *>(xr)[i] = v;
        }
        arq_keep_piece(v, i, d_model, row, ss);
    }
    arq_norm_quant_q80(ss, row, red, gamma, out_q80, t, d_model, cols, eps);
}

// one warp per 256-element block of the output: out = silu(gate) * up, quantised to Q8_K (VEC: gate_up is 16-byte aligned)
template <bool VEC>
__global__ void __launch_bounds__(128) swiglu_q8k_kernel(const float *__restrict__ gate_up, uint8_t *__restrict__ out_q8, int tokens, int dim)
{
    pdl_trigger();
    pdl_wait();
    const int lane = threadIdx.x & 31;
    const int nb = dim / QK_K;
    const long long blk = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (blk >= (long long)tokens * nb) return;
    const int t = (int)(blk / nb), b = (int)(blk - (long long)t * nb);
    const float *g = gate_up + (size_t)t * 2 * dim + (size_t)b * QK_K + 8 * lane;
    const float *u = g + dim;
    // a lane's 32 bytes as two 16-byte loads through L1 (the second finds the sector the first brought): eight 4-byte loads at a
    // 32-byte stride asked L2 for every sector eight times
    float gs[8], us[8];
    if (VEC) {
        const float4 g0 = *reinterpret_cast<const float4 *>(g), g1 = *reinterpret_cast<const float4 *>(g + 4);
        const float4 u0 = *reinterpret_cast<const float4 *>(u), u1 = *reinterpret_cast<const float4 *>(u + 4);
        gs[0] = g0.x; gs[1] = g0.y; gs[2] = g0.z; gs[3] = g0.w; gs[4] = g1.x; gs[5] = g1.y; gs[6] = g1.z; gs[7] = g1.w;
        us[0] = u0.x; us[1] = u0.y; us[2] = u0.z; us[3] = u0.w; us[4] = u1.x; us[5] = u1.y; us[6] = u1.z; us[7] = u1.w;
    } else {
#pragma unroll
        for (int j = 0; j < 8; ++j) { gs[j] = __ldcg(g + j); us[j] = __ldcg(u + j); }
    }
    float v[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) {
        const float sg = __fdiv_rn(1.0f, __fadd_rn(1.0f, expf(-gs[j])));
        v[j] = __fmul_rn(__fmul_rn(gs[j], sg), us[j]);
    }
    quantize_block_q8k(v, out_q8 + blk * Q8K_BYTES, lane);
}

// One token per sequence.  q [B][H][d] is rotated in place; k [B][Hkv][d] is rotated and written, v copied,
// into the caches [B][Hkv][max_seq][d] at position *pos_dev (the same position for every sequence).  CT is the cache
// element: float, or __half rounded to nearest even as kv_cache_store_f16 does (src/kernels/kv_cache_kernels.c).
__device__ __forceinline__ void cache_put(float *p, float x) { *p = x; }
__device__ __forceinline__ void cache_put(__half *p, float x) { *p = __float2half_rn(x); }

template <typename CT>
__global__ void rope_kv_store_kernel(float *__restrict__ q, const float *__restrict__ k, const float *__restrict__ v,
                                     CT *__restrict__ kc, CT *__restrict__ vc, const float *__restrict__ cos_cache,
                                     const float *__restrict__ sin_cache, const int *__restrict__ pos_dev, int batch, int H, int Hkv,
                                     int d, int max_seq, long long kv_batch_stride)
{
    pdl_trigger();
    // The position changes only at the end of a step (advance_pos, after which the next step begins with a fully ordered launch)
    // and the tables are constants: both are read before the dependency wait, off the critical path.
    const int pos = __ldcg(pos_dev);
    const int half = d / 2;
    const int per_seq = (H + 2 * Hkv) * half;
    const int first = blockIdx.x * blockDim.x + threadIdx.x;
    float c0 = 0.0f, s0 = 0.0f;
    if (pos >= 0 && pos < max_seq && first < batch * per_seq) {
        const int j0 = (first % per_seq) % half;
        c0 = cos_cache[(size_t)pos * half + j0];
        s0 = sin_cache[(size_t)pos * half + j0];
    }
    pdl_wait();
    if (pos < 0 || pos >= max_seq) return;
    for (int i = first; i < batch * per_seq; i += gridDim.x * blockDim.x) {
        const int s = i / per_seq, r = i - s * per_seq;
        const int h = r / half, j = r - h * half;
        const float c = i == first ? c0 : cos_cache[(size_t)pos * half + j], sn = i == first ? s0 : sin_cache[(size_t)pos * half + j];
        if (h < H) {
            float *row = q + ((size_t)s * H + h) * d;
            const float a = __ldcg(row + j), b = __ldcg(row + j + half);
            row[j] = __fsub_rn(__fmul_rn(a, c), __fmul_rn(b, sn));
            row[j + half] = __fadd_rn(__fmul_rn(a, sn), __fmul_rn(b, c));
        } else if (h < H + Hkv) {
            const int hk = h - H;
            const float *row = k + ((size_t)s * Hkv + hk) * d;
            CT *dst = kc + (size_t)s * kv_batch_stride + ((size_t)hk * max_seq + pos) * d;
            const float a = __ldcg(row + j), b = __ldcg(row + j + half);
            cache_put(dst + j, __fsub_rn(__fmul_rn(a, c), __fmul_rn(b, sn)));
            cache_put(dst + j + half, __fadd_rn(__fmul_rn(a, sn), __fmul_rn(b, c)));
        } else {
            const int hk = h - H - Hkv;
            const float *row = v + ((size_t)s * Hkv + hk) * d;
            CT *dst = vc + (size_t)s * kv_batch_stride + ((size_t)hk * max_seq + pos) * d;
            cache_put(dst + j, __ldcg(row + j));
            cache_put(dst + j + half, __ldcg(row + j + half));
        }
    }
}

__global__ void advance_pos_kernel(int *pos)
{
    pdl_trigger();
    pdl_wait();
    if (threadIdx.x == 0 && blockIdx.x == 0) *pos = __ldcg(pos) + 1;
}

__global__ void add_inplace_kernel(float *__restrict__ x, const float *__restrict__ delta, long long n)
{
    pdl_trigger();
    pdl_wait();
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) x[i] = __ldcg(x + i) + __ldcg(delta + i);
}

// synthetic fills used by benchmarks of model shapes too large to generate on the host: the same value
// distributions as the host generators (uniform packed fields, small positive fp16 scales, N(0,1) floats)
__device__ __forceinline__ uint32_t mix32(uint64_t z)
{
    z += 0x9E3779B97F4A7C15ull;
    z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
    z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
    return (uint32_t)((z ^ (z >> 31)) >> 16);
}

// fmt 0: Q4_K, 1: Q6_K, 2: Q8_0
__global__ void fill_blocks_kernel(uint8_t *__restrict__ w, long long nblocks, int fmt, uint64_t seed)
{
    const int bs = fmt == 0 ? Q4K_BYTES : (fmt == 1 ? Q6K_BYTES : (fmt == 3 ? Q50_BYTES : Q80_BYTES));     // 3: block_q5_0
    for (long long b = (long long)blockIdx.x * blockDim.x + threadIdx.x; b < nblocks; b += (long long)gridDim.x * blockDim.x) {
        uint8_t *p = w + b * bs;
        const uint64_t base = seed * 0x100000001B3ull + (uint64_t)b * 64;
        for (int i = 0; i < bs; i += 2) {
            const uint32_t r = mix32(base + i);
            p[i] = (uint8_t)r;
            if (i + 1 < bs) p[i + 1] = (uint8_t)(r >> 8);
        }
        const float u0 = (mix32(base + 1000) & 0xFFFFFF) * (1.0f / 16777216.0f), u1 = (mix32(base + 1001) & 0xFFFFFF) * (1.0f / 16777216.0f);
        if (fmt == 0) {
            *reinterpret_cast<unsigned short *>(p) = __half_as_ushort(__float2half_rn(0.02f * u0));
            *reinterpret_cast<unsigned short *>(p + 2) = __half_as_ushort(__float2half_rn(0.01f * u1));
        } else if (fmt == 1) {
            for (int i = 0; i < 16; ++i) p[192 + i] = (uint8_t)(int8_t)((int)(mix32(base + 2000 + i) & 63) - 32);
            *reinterpret_cast<unsigned short *>(p + 208) = __half_as_ushort(__float2half_rn(0.02f * u0));
        } else if (fmt == 3) {
            *reinterpret_cast<unsigned short *>(p) = __half_as_ushort(__float2half_rn(0.02f * u0));       // the other 20 bytes stay uniform random
        } else {
            *reinterpret_cast<unsigned short *>(p) = __half_as_ushort(__float2half_rn(0.01f * u0));
            for (int i = 0; i < 32; ++i) p[2 + i] = (uint8_t)(int8_t)((int)(mix32(base + 3000 + i) % 255u) - 127);
        }
    }
}

// mode 0: N(0,1) (Box-Muller), mode 1: 1 + 0.1 * N(0,1)
template <typename T>
__global__ void fill_normal_kernel(T *__restrict__ x, long long n, int mode, uint64_t seed)
{
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
        const float u0 = ((mix32(seed * 977 + 2 * i) & 0xFFFFFF) + 1) * (1.0f / 16777217.0f);
        const float u1 = (mix32(seed * 977 + 2 * i + 1) & 0xFFFFFF) * (1.0f / 16777216.0f);
        const float z = sqrtf(-2.0f * logf(u0)) * cospif(2.0f * u1);
        cache_put(x + i, mode == 1 ? 1.0f + 0.1f * z : z);
    }
}

static inline unsigned grid_for(long long n, int block, int cap) { long long g = (n + block - 1) / block; return (unsigned)(g < 1 ? 1 : (g > cap ? cap : g)); }

}  // namespace ckb

using namespace ckb;

extern "C" int ckb200_dev_add_rmsnorm_q8k(float *x, const float *delta, const float *gamma, void *out_q8, float *norm_out, int tokens,
                                          int d_model, int aligned_embed_dim, float eps, void *stream)
{
    if (!x || !gamma || !out_q8 || tokens <= 0 || d_model <= 0) return 0;
    if (aligned_embed_dim % QK_K || aligned_embed_dim < d_model) return ckb_fail(CKB_ERR_SHAPE, "add_rmsnorm_q8k: aligned width %d must be a multiple of 256 and >= d_model", aligned_embed_dim);
    if (ckb_ensure_init()) return CKB_ERR_NO_DEVICE;
    if (aligned_embed_dim > 1024 * 4 * ARQ_MAX_V4) return ckb_fail(CKB_ERR_LIMIT, "add_rmsnorm_q8k: rows wider than %d are not supported", 1024 * 4 * ARQ_MAX_V4);
    if (((uintptr_t)x | (uintptr_t)delta) & 15) return ckb_fail(CKB_ERR_ALIGN, "add_rmsnorm_q8k: x and delta must be 16-byte aligned");
    int threads = (aligned_embed_dim / 4 + 31) & ~31;          // one 16-byte piece per thread while that fits a CTA
    if (threads > 1024) threads = 1024;
    // many rows (a prompt): four pieces per thread, so that several rows share an SM instead of one 1024-thread CTA at a time
    if (tokens >= 64 && ckb_tune_get("add_rmsnorm_rows_narrow", 1)) { threads = ((aligned_embed_dim / 4 + ARQ_MAX_V4 - 1) / ARQ_MAX_V4 + 31) & ~31; if (threads < 128) threads = 128; }
    const size_t smem = (size_t)aligned_embed_dim * sizeof(float);
    if (smem > 48 * 1024) {
        static size_t set = 0;
        if (smem > set) {
            if (ckb_check_cuda((int)cudaFuncSetAttribute(add_rmsnorm_q8k_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem), "smem attr")) return CKB_ERR_CUDA;
            set = smem;
        }
    }
    return launch_pdl("add_rmsnorm_q8k", add_rmsnorm_q8k_kernel, dim3(tokens), dim3(threads), smem, ckb_stream(stream), x, delta, gamma,
                      (uint8_t *)out_q8, norm_out, d_model, aligned_embed_dim, eps);
}

extern "C" int ckb200_dev_add_rmsnorm_q8_0(float *x, const float *delta, const float *gamma, void *out_q80, int tokens, int d_model,
                                           int aligned_embed_dim, int cols, float eps, void *stream)
{
    if (!x || !gamma || !out_q80 || tokens <= 0 || d_model <= 0) return 0;
    if (aligned_embed_dim % 4 || aligned_embed_dim < d_model || cols % 32 || cols > aligned_embed_dim || cols <= 0)
        return ckb_fail(CKB_ERR_SHAPE, "add_rmsnorm_q8_0: widths %d / %d / %d", d_model, aligned_embed_dim, cols);
    if (ckb_ensure_init()) return CKB_ERR_NO_DEVICE;
    if ((((uintptr_t)x | (uintptr_t)delta) & 15) || ((uintptr_t)out_q80 & 1)) return ckb_fail(CKB_ERR_ALIGN, "add_rmsnorm_q8_0: x and delta must be 16-byte aligned");
    int threads = (aligned_embed_dim / 4 + 31) & ~31;
    if (threads > 1024) threads = 1024;
    if (threads < 32) threads = 32;
    const size_t smem = (size_t)aligned_embed_dim * sizeof(float);
    if (smem > 48 * 1024) {
        static size_t set = 0;
        if (smem > set) {
            if (ckb_check_cuda((int)cudaFuncSetAttribute(add_rmsnorm_q80_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem), "smem attr")) return CKB_ERR_CUDA;
            set = smem;
        }
    }
    return launch_pdl("add_rmsnorm_q80", add_rmsnorm_q80_kernel, dim3(tokens), dim3(threads), smem, ckb_stream(stream), x, delta, gamma, (uint8_t *)out_q80,
                      d_model, aligned_embed_dim, cols, eps);
}

extern "C" int ckb200_dev_swiglu_q8k(const float *gate_up, void *out_q8, int tokens, int dim, void *stream)
{
    if (!gate_up || !out_q8 || tokens <= 0 || dim <= 0) return 0;
    if (dim % QK_K) return ckb_fail(CKB_ERR_SHAPE, "swiglu_q8k: dim %d is not a multiple of 256", dim);
    if (ckb_ensure_init()) return CKB_ERR_NO_DEVICE;
    const long long nblocks = (long long)tokens * (dim / QK_K);
    if (((uintptr_t)gate_up & 15) == 0)
        return launch_pdl("swiglu_q8k", swiglu_q8k_kernel<true>, dim3((unsigned)((nblocks + 3) / 4)), dim3(128), 0, ckb_stream(stream), gate_up,
                          (uint8_t *)out_q8, tokens, dim);
    return launch_pdl("swiglu_q8k", swiglu_q8k_kernel<false>, dim3((unsigned)((nblocks + 3) / 4)), dim3(128), 0, ckb_stream(stream), gate_up,
                      (uint8_t *)out_q8, tokens, dim);
}

extern "C" int ckb200_dev_rope_kv_store(float *q, const float *k, const float *v, float *k_cache, float *v_cache, const float *cos_cache,
                                        const float *sin_cache, const int *pos_dev, int batch, int num_heads, int num_kv_heads,
                                        int head_dim, int max_seq_len, long long kv_batch_stride, void *stream)
{
    if (!q || !k || !v || !k_cache || !v_cache || !cos_cache || !sin_cache || !pos_dev || batch <= 0) return 0;
    if (ckb_ensure_init()) return CKB_ERR_NO_DEVICE;
    const long long n = (long long)batch * (num_heads + 2 * num_kv_heads) * (head_dim / 2);
    return launch_pdl("rope_kv_store", rope_kv_store_kernel<float>, dim3(grid_for(n, 128, 1024)), dim3(128), 0, ckb_stream(stream), q, k, v, k_cache,
                      v_cache, cos_cache, sin_cache, pos_dev, batch, num_heads, num_kv_heads, head_dim, max_seq_len, kv_batch_stride);
}

// The same step with IEEE fp16 caches (rope_forward_qk + kv_cache_store_f16): q and k are rotated in fp32, k and v rounded once on the store.
extern "C" int ckb200_dev_rope_kv_store_f16(float *q, const float *k, const float *v, uint16_t *k_cache, uint16_t *v_cache, const float *cos_cache,
                                            const float *sin_cache, const int *pos_dev, int batch, int num_heads, int num_kv_heads,
                                            int head_dim, int max_seq_len, long long kv_batch_stride, void *stream)
{
    if (!q || !k || !v || !k_cache || !v_cache || !cos_cache || !sin_cache || !pos_dev || batch <= 0) return 0;
    if (ckb_ensure_init()) return CKB_ERR_NO_DEVICE;
    const long long n = (long long)batch * (num_heads + 2 * num_kv_heads) * (head_dim / 2);
    return launch_pdl("rope_kv_store_f16", rope_kv_store_kernel<__half>, dim3(grid_for(n, 128, 1024)), dim3(128), 0, ckb_stream(stream), q, k, v,
                      reinterpret_cast<__half *>(k_cache), reinterpret_cast<__half *>(v_cache), cos_cache, sin_cache, pos_dev, batch, num_heads,
                      num_kv_heads, head_dim, max_seq_len, kv_batch_stride);
}

extern "C" int ckb200_dev_advance_pos(int *pos_dev, void *stream)
{
    if (!pos_dev) return 0;
    if (ckb_ensure_init()) return CKB_ERR_NO_DEVICE;
    return launch_pdl("advance_pos", advance_pos_kernel, dim3(1), dim3(32), 0, ckb_stream(stream), pos_dev);
}

extern "C" int ckb200_dev_add_inplace(float *x, const float *delta, long long n, void *stream)
{
    if (!x || !delta || n <= 0) return 0;
    if (ckb_ensure_init()) return CKB_ERR_NO_DEVICE;
    return launch_pdl("add_inplace", add_inplace_kernel, dim3(grid_for(n, 256, 2048)), dim3(256), 0, ckb_stream(stream), x, delta, n);
}

extern "C" int ckb200_dev_fill_blocks(void *w, long long nblocks, int fmt, unsigned long long seed, void *stream)
{
    if (!w || nblocks <= 0) return 0;
    if (ckb_ensure_init()) return CKB_ERR_NO_DEVICE;
    fill_blocks_kernel<<<grid_for(nblocks, 256, 8192), 256, 0, ckb_stream(stream)>>>((uint8_t *)w, nblocks, fmt, seed);
    return ckb_check_launch("fill_blocks");
}

extern "C" int ckb200_dev_fill_normal(float *x, long long n, int mode, unsigned long long seed, void *stream)
{
    if (!x || n <= 0) return 0;
    if (ckb_ensure_init()) return CKB_ERR_NO_DEVICE;
    fill_normal_kernel<float><<<grid_for(n, 256, 8192), 256, 0, ckb_stream(stream)>>>(x, n, mode, seed);
    return ckb_check_launch("fill_normal");
}

extern "C" int ckb200_dev_fill_normal_f16(uint16_t *x, long long n, int mode, unsigned long long seed, void *stream)
{
    if (!x || n <= 0) return 0;
    if (ckb_ensure_init()) return CKB_ERR_NO_DEVICE;
    fill_normal_kernel<__half><<<grid_for(n, 256, 8192), 256, 0, ckb_stream(stream)>>>(reinterpret_cast<__half *>(x), n, mode, seed);
    return ckb_check_launch("fill_normal_f16");
}
