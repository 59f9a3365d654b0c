// The small fp32 ops that sit between the quantised matmuls of a decode / prefill step.
// Each follows the reference function it replaces:
//   rmsnorm_forward               src/kernels/rmsnorm_kernels.c:126-250 (scalar form :38-71; zero pad :245-248)
//   rope_precompute_cache_split   src/kernels/rope_kernels.c:221-243
//   rope_forward_qk (rotate-half) src/kernels/rope_kernels.c:320-417, :806-819
//   swiglu_forward                src/kernels/swiglu_kernels.c:140-216 (exact sigmoid form :358-379)
//   ck_residual_add_token_major   src/ckernel_orchestration.c:139-149
//   kv_cache_store                src/kernels/kv_cache_kernels.c:70-129
//   embedding_forward_q4_k/q6_k/q8_0  src/kernels/embedding_kernels.c:76-239
//
// Functions that depend on the decode position take it either by value or, when `pos_dev` is not
// NULL, read it from device memory so that a captured CUDA graph of a whole step can be replayed
// for every token.
#include "dequant_elem.cuh"
#include "launch.h"
#include "runtime.h"

namespace ckb {

__device__ __forceinline__ float block_sum(float v, float *red)
{
    v = group_sum<32>(v);
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
    if (lane == 0) red[warp] = v;
    __syncthreads();
    float t = 0.0f;
    for (int w = 0; w < nw; ++w) t += red[w];
    __syncthreads();
    return t;
}

// one CTA per token row
__global__ void __launch_bounds__(256) rmsnorm_kernel(const float *__restrict__ in, const float *__restrict__ gamma,
                                                      float *__restrict__ out, float *__restrict__ rstd_cache, int d_model,
                                                      int aligned, float eps)
{
    __shared__ float red[8];
    const float *x = in + (size_t)blockIdx.x * aligned;
    float *y = out + (size_t)blockIdx.x * aligned;
    float ss = 0.0f;
    for (int i = threadIdx.x; i < d_model; i += blockDim.x) ss = fmaf(x[i], x[i], ss);
    ss = block_sum(ss, red);
    const float mean = __fmul_rn(ss, __fdiv_rn(1.0f, (float)d_model));
    const float rstd = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(mean, eps)));
    if (rstd_cache && threadIdx.x == 0) rstd_cache[blockIdx.x] = rstd;
    for (int i = threadIdx.x; i < aligned; i += blockDim.x)
        y[i] = i < d_model ? __fmul_rn(__fmul_rn(x[i], rstd), gamma[i]) : 0.0f;
}

// rows of rot_dim / 2 values; frequencies are spaced over rot_dim (head_dim for the split form); with lin_scale > 0 the
// position is divided by it first (the reference's "linear" scaling, src/kernels/rope_kernels.c:270-316)
__global__ void rope_cache_kernel(float *__restrict__ cos_cache, float *__restrict__ sin_cache, int max_seq, int rot_dim, float base, float lin_scale)
{
    const int half = rot_dim / 2;
    const long long n = (long long)max_seq * half;
    const double lb = log((double)base);
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
        const int pos = (int)(i / half), j = (int)(i - (long long)pos * half);
        const float freq = (float)exp(-((double)(2 * j) / (double)rot_dim) * lb);
        const float epos = lin_scale > 0.0f ? __fdiv_rn((float)pos, lin_scale) : (float)pos;
        const float ang = __fmul_rn(epos, freq);
        cos_cache[i] = (float)cos((double)ang);
        sin_cache[i] = (float)sin((double)ang);
    }
}

// x: [heads][tokens][ahd]; pairs (2i, 2i+1) of the first rot_dim elements are rotated with cos/sin rows of rot_dim / 2 values
// (rope_forward_qk_pairwise_with_rotary_dim, src/kernels/rope_kernels.c:419-451, :839-866); the rest of the row is untouched
__global__ void rope_pairwise_kernel(float *__restrict__ q, float *__restrict__ k, const float *__restrict__ cos_cache,
                                     const float *__restrict__ sin_cache, int num_heads, int num_kv_heads, int tokens, int rot_dim, int ahd,
                                     int pos_offset, const int *__restrict__ pos_dev)
{
    const int half = rot_dim / 2;
    const int pos0 = pos_dev ? *pos_dev : pos_offset;
    const long long n = (long long)(num_heads + num_kv_heads) * tokens * half;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
        const int j = (int)(i % half);
        const long long ht = i / half;
        const int t = (int)(ht % tokens), h = (int)(ht / tokens);
        float *row = h < num_heads ? q + ((size_t)h * tokens + t) * ahd : k + ((size_t)(h - num_heads) * tokens + t) * ahd;
        const float c = cos_cache[(size_t)(pos0 + t) * half + j], s = sin_cache[(size_t)(pos0 + t) * half + j];
        const float2 ab = *reinterpret_cast<const float2 *>(row + 2 * j);
        float2 r;
        r.x = __fsub_rn(__fmul_rn(ab.x, c), __fmul_rn(ab.y, s));
        r.y = __fadd_rn(__fmul_rn(ab.x, s), __fmul_rn(ab.y, c));
        *reinterpret_cast<float2 *>(row + 2 * j) = r;
    }
}

// x: [heads][tokens][ahd]; rotate-half over head_dim with cos/sin rows pos_offset + t
__global__ void rope_kernel(float *__restrict__ q, float *__restrict__ k, const float *__restrict__ cos_cache,
                            const float *__restrict__ sin_cache, int num_heads, int num_kv_heads, int tokens, int head_dim, int ahd,
                            int pos_offset, const int *__restrict__ pos_dev)
{
    const int half = head_dim / 2;
    const int pos0 = pos_dev ? *pos_dev : pos_offset;
    const long long n = (long long)(num_heads + num_kv_heads) * tokens * half;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
        const int j = (int)(i % half);
        const long long ht = i / half;
        const int t = (int)(ht % tokens), h = (int)(ht / tokens);
        float *row = h < num_heads ? q + ((size_t)h * tokens + t) * ahd : k + ((size_t)(h - num_heads) * tokens + t) * ahd;
        const float c = cos_cache[(size_t)(pos0 + t) * half + j], s = sin_cache[(size_t)(pos0 + t) * half + j];
        const float a = row[j], b = row[j + half];
        row[j] = __fsub_rn(__fmul_rn(a, c), __fmul_rn(b, s));
        row[j + half] = __fadd_rn(__fmul_rn(a, s), __fmul_rn(b, c));
    }
}

__global__ void swiglu_kernel(const float *__restrict__ in, float *__restrict__ out, int tokens, int dim)
{
    const long long n = (long long)tokens * dim;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
        const long long t = i / dim;
        const int d = (int)(i - t * dim);
        const float g = in[t * 2 * dim + d], u = in[t * 2 * dim + dim + d];
        const float sg = __fdiv_rn(1.0f, __fadd_rn(1.0f, expf(-g)));
        out[i] = __fmul_rn(__fmul_rn(g, sg), u);
    }
}

__global__ void add_kernel(const float *__restrict__ a, const float *__restrict__ b, float *__restrict__ out, long long n)
{
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x)
        out[i] = a[i] + b[i];
}

// k, v: [Hkv][head_dim] of one token -> cache[Hkv][max_seq][head_dim] at pos
__global__ void kv_store_kernel(float *__restrict__ kc, float *__restrict__ vc, const float *__restrict__ k,
                                const float *__restrict__ v, int pos, const int *__restrict__ pos_dev, int num_kv_heads,
                                int head_dim, int max_seq)
{
    const int p = pos_dev ? *pos_dev : pos;
    if (p < 0 || p >= max_seq) return;
    const int n = num_kv_heads * head_dim;
    for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < n; i += gridDim.x * blockDim.x) {
        const int h = i / head_dim, d = i - h * head_dim;
        const size_t dst = ((size_t)h * max_seq + p) * head_dim + d;
        kc[dst] = k[i];
        vc[dst] = v[i];
    }
}

// the same store into IEEE fp16 caches (kv_cache_store_f16, src/kernels/kv_cache_kernels.c:131-163): round to nearest even
__global__ void kv_store_f16_kernel(unsigned short *__restrict__ kc, unsigned short *__restrict__ vc, const float *__restrict__ k,
                                    const float *__restrict__ v, int pos, const int *__restrict__ pos_dev, int num_kv_heads,
                                    int head_dim, int max_seq)
{
    const int p = pos_dev ? *pos_dev : pos;
    if (p < 0 || p >= max_seq) return;
    const int n = num_kv_heads * head_dim;
    for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < n; i += gridDim.x * blockDim.x) {
        const int h = i / head_dim, d = i - h * head_dim;
        const size_t dst = ((size_t)h * max_seq + p) * head_dim + d;
        kc[dst] = __half_as_ushort(__float2half_rn(k[i]));
        vc[dst] = __half_as_ushort(__float2half_rn(v[i]));
    }
}

// one CTA per token: dequantise the table row of its id (out-of-range ids read row 0), zero the padding
template <int FMT>
__global__ void embedding_kernel(const int32_t *__restrict__ ids, int count, int vocab, const uint8_t *__restrict__ table,
                                 const float *__restrict__ pos_emb, float *__restrict__ out, int embed, int aligned, int table_cols, int add_pos)
{
    constexpr int BS = DqTraits<FMT>::BS, BE = DqTraits<FMT>::BE;
    const int t = blockIdx.x;
    float *o = out + (size_t)t * aligned;
    if (t >= count) {
        for (int i = threadIdx.x; i < aligned; i += blockDim.x) o[i] = 0.0f;
        return;
    }
    int id = ids[t];
    if (id < 0 || id >= vocab) id = 0;
    const size_t row_bytes = (size_t)((table_cols + BE - 1) / BE) * BS;
    const uint8_t *row = table + (size_t)id * row_bytes;
    for (int i = threadIdx.x; i < aligned; i += blockDim.x) {
        float v = 0.0f;
        if (i < embed) {
            v = dequant_elem<FMT>(row + (size_t)(i / BE) * BS, i % BE);
            if (add_pos && pos_emb) v += pos_emb[(size_t)t * aligned + i];
        }
        o[i] = v;
    }
}

static inline unsigned grid_for(long long n, int block, int cap) { long long g = (n + block - 1) / block; return (unsigned)(g < 1 ? 1 : (g > cap ? cap : g)); }

}  // namespace ckb

using namespace ckb;

extern "C" int ckb200_dev_rmsnorm_forward(const float *input, const float *gamma, float *output, float *rstd_cache, int tokens,
                                          int d_model, int aligned_embed_dim, float eps, void *stream)
{
    if (!input || !gamma || !output || tokens <= 0 || d_model <= 0 || aligned_embed_dim < d_model) return 0;
    if (ckb_ensure_init()) return CKB_ERR_NO_DEVICE;
    rmsnorm_kernel<<<tokens, 256, 0, ckb_stream(stream)>>>(input, gamma, output, rstd_cache, d_model, aligned_embed_dim, eps);
    return ckb_check_launch("rmsnorm_forward");
}

extern "C" int ckb200_dev_rope_precompute_cache_split(float *cos_cache, float *sin_cache, int max_seq_len, int head_dim,
                                                      float base, void *stream)
{
    if (!cos_cache || !sin_cache || max_seq_len <= 0 || head_dim <= 1) return 0;
    if (ckb_ensure_init()) return CKB_ERR_NO_DEVICE;
    const long long n = (long long)max_seq_len * (head_dim / 2);
    rope_cache_kernel<<<grid_for(n, 256, 2048), 256, 0, ckb_stream(stream)>>>(cos_cache, sin_cache, max_seq_len, head_dim, base, 0.0f);
    return ckb_check_launch("rope_precompute_cache_split");
}

// rope_precompute_cache (src/kernels/rope_kernels.c:270-316): rows of rotary_dim / 2 values, optional linear position scaling
extern "C" int ckb200_dev_rope_precompute_cache(float *cos_cache, float *sin_cache, int max_seq_len, int head_dim, float base, int rotary_dim,
                                                int linear_scaling, float scaling_factor, void *stream)
{
    if (!cos_cache || !sin_cache || max_seq_len <= 0 || head_dim <= 1) return 0;
    if (ckb_ensure_init()) return CKB_ERR_NO_DEVICE;
    if (rotary_dim <= 0 || rotary_dim > head_dim) rotary_dim = head_dim;
    if (rotary_dim < 2) return 0;
    const float lin = (linear_scaling && scaling_factor > 0.0f && scaling_factor != 1.0f) ? scaling_factor : 0.0f;
    const long long n = (long long)max_seq_len * (rotary_dim / 2);
    rope_cache_kernel<<<grid_for(n, 256, 2048), 256, 0, ckb_stream(stream)>>>(cos_cache, sin_cache, max_seq_len, rotary_dim, base, lin);
    return ckb_check_launch("rope_precompute_cache");
}

// rope_forward_qk_pairwise_with_rotary_dim (src/kernels/rope_kernels.c:839-866): the interleaved (Llama) pairing
extern "C" int ckb200_dev_rope_forward_qk_pairwise(float *q, float *k, const float *cos_cache, const float *sin_cache, int num_heads,
                                                   int num_kv_heads, int num_tokens, int head_dim, int aligned_head_dim, int pos_offset,
                                                   int rotary_dim, const int *pos_dev, void *stream)
{
    if (!q || !k || !cos_cache || !sin_cache || num_heads <= 0 || num_kv_heads < 0 || num_tokens <= 0 || head_dim <= 1) return 0;
    if (ckb_ensure_init()) return CKB_ERR_NO_DEVICE;
    if (rotary_dim <= 0 || rotary_dim > head_dim) rotary_dim = head_dim;
    if (rotary_dim < 2) return 0;
    if ((aligned_head_dim & 1) || (((uintptr_t)q | (uintptr_t)k) & 7)) return ckb_fail(CKB_ERR_ALIGN, "rope_forward_qk_pairwise: rows must be 8-byte aligned");
    const long long n = (long long)(num_heads + num_kv_heads) * num_tokens * (rotary_dim / 2);
    rope_pairwise_kernel<<<grid_for(n, 256, 2048), 256, 0, ckb_stream(stream)>>>(q, k, cos_cache, sin_cache, num_heads, num_kv_heads,
                                                                               num_tokens, rotary_dim, aligned_head_dim, pos_offset, pos_dev);
    return ckb_check_launch("rope_forward_qk_pairwise");
}

extern "C" int ckb200_dev_rope_forward_qk(float *q, float *k, const float *cos_cache, const float *sin_cache, int num_heads,
                                          int num_kv_heads, int num_tokens, int head_dim, int aligned_head_dim, int pos_offset,
                                          const int *pos_dev, void *stream)
{
    if (!q || !k || !cos_cache || !sin_cache || num_heads <= 0 || num_kv_heads < 0 || num_tokens <= 0 || head_dim <= 1) return 0;
    if (ckb_ensure_init()) return CKB_ERR_NO_DEVICE;
    const long long n = (long long)(num_heads + num_kv_heads) * num_tokens * (head_dim / 2);
    rope_kernel<<<grid_for(n, 256, 2048), 256, 0, ckb_stream(stream)>>>(q, k, cos_cache, sin_cache, num_heads, num_kv_heads,
                                                                      num_tokens, head_dim, aligned_head_dim, pos_offset, pos_dev);
    return ckb_check_launch("rope_forward_qk");
}

// rope_forward_qk_with_rotary_dim (src/kernels/rope_kernels.c:320-417, :821-837): the half-split rotation over the first rotary_dim
// channels only (pairs i, i + rotary_dim / 2; table rows of rotary_dim / 2 values); the channels above pass through
extern "C" int ckb200_dev_rope_forward_qk_with_rotary_dim(float *q, float *k, const float *cos_cache, const float *sin_cache, int num_heads,
                                                          int num_kv_heads, int num_tokens, int head_dim, int aligned_head_dim, int pos_offset,
                                                          int rotary_dim, const int *pos_dev, void *stream)
{
    if (rotary_dim <= 0 || rotary_dim > head_dim) rotary_dim = head_dim;
    return ckb200_dev_rope_forward_qk(q, k, cos_cache, sin_cache, num_heads, num_kv_heads, num_tokens, rotary_dim, aligned_head_dim, pos_offset, pos_dev, stream);
}

extern "C" int ckb200_dev_swiglu_forward(const float *input, float *output, int tokens, int dim, void *stream)
{
    if (!input || !output || tokens <= 0 || dim <= 0) return 0;
    if (ckb_ensure_init()) return CKB_ERR_NO_DEVICE;
    swiglu_kernel<<<grid_for((long long)tokens * dim, 256, 4096), 256, 0, ckb_stream(stream)>>>(input, output, tokens, dim);
    return ckb_check_launch("swiglu_forward");
}

extern "C" int ckb200_dev_residual_add(const float *a, const float *b, float *out, int tokens, int aligned_embed_dim, void *stream)
{
    if (!a || !b || !out || tokens <= 0 || aligned_embed_dim <= 0) return 0;
    if (ckb_ensure_init()) return CKB_ERR_NO_DEVICE;
    const long long n = (long long)tokens * aligned_embed_dim;
    add_kernel<<<grid_for(n, 256, 4096), 256, 0, ckb_stream(stream)>>>(a, b, out, n);
    return ckb_check_launch("residual_add");
}

extern "C" int ckb200_dev_kv_cache_store(float *kv_cache_k, float *kv_cache_v, const float *k, const float *v, int pos,
                                         const int *pos_dev, int num_kv_heads, int head_dim, int max_seq_len, void *stream)
{
    if (!kv_cache_k || !kv_cache_v || !k || !v || num_kv_heads <= 0 || head_dim <= 0 || max_seq_len <= 0) return 0;
    if (!pos_dev && (pos < 0 || pos >= max_seq_len)) return 0;
    if (ckb_ensure_init()) return CKB_ERR_NO_DEVICE;
    kv_store_kernel<<<grid_for((long long)num_kv_heads * head_dim, 256, 64), 256, 0, ckb_stream(stream)>>>(
        kv_cache_k, kv_cache_v, k, v, pos, pos_dev, num_kv_heads, head_dim, max_seq_len);
    return ckb_check_launch("kv_cache_store");
}

extern "C" int ckb200_dev_kv_cache_store_f16(uint16_t *kv_cache_k, uint16_t *kv_cache_v, const float *k, const float *v, int pos,
                                             const int *pos_dev, int num_kv_heads, int head_dim, int max_seq_len, void *stream)
{
    if (!kv_cache_k || !kv_cache_v || !k || !v || num_kv_heads <= 0 || head_dim <= 0 || max_seq_len <= 0) return 0;
    if (!pos_dev && (pos < 0 || pos >= max_seq_len)) return 0;
    if (ckb_ensure_init()) return CKB_ERR_NO_DEVICE;
    kv_store_f16_kernel<<<grid_for((long long)num_kv_heads * head_dim, 256, 64), 256, 0, ckb_stream(stream)>>>(
        kv_cache_k, kv_cache_v, k, v, pos, pos_dev, num_kv_heads, head_dim, max_seq_len);
    return ckb_check_launch("kv_cache_store_f16");
}

template <int FMT>
static int launch_embedding(const int32_t *ids, int count, int vocab, const void *table, const float *pos_emb, float *out,
                            int embed, int aligned, int table_cols, int ctx, int add_pos, void *stream)
{
    if (!ids || !table || !out || ctx <= 0 || aligned <= 0) return 0;
    if (ckb_ensure_init()) return CKB_ERR_NO_DEVICE;
    int n = count < 0 ? 0 : (count > ctx ? ctx : count);
    embedding_kernel<FMT><<<ctx, 256, 0, ckb_stream(stream)>>>(ids, n, vocab, (const uint8_t *)table, pos_emb, out, embed, aligned, table_cols, add_pos);
    return ckb_check_launch("embedding_forward");
}

// Rows of a table whose width differs from the output stride: a block-32 table of a hidden size that is not a multiple of 256
// (rows of table_cols elements) feeding activation rows padded to out_stride.  fmt: 0 Q4_K, 1 Q6_K, 2 Q8_0.
extern "C" int ckb200_dev_embedding_rows(const int32_t *ids, int count, int vocab, const void *table, int fmt, int table_cols, float *out, int out_stride,
                                         int embed, void *stream)
{
    if (embed > table_cols || embed > out_stride) return ckb_fail(CKB_ERR_SHAPE, "embedding_rows: embed %d exceeds the table row %d or the output row %d", embed, table_cols, out_stride);
    switch (fmt) {
        case 0: return launch_embedding<DQ_Q4K>(ids, count, vocab, table, NULL, out, embed, out_stride, table_cols, count, 0, stream);
        case 1: return launch_embedding<DQ_Q6K>(ids, count, vocab, table, NULL, out, embed, out_stride, table_cols, count, 0, stream);
        case 2: return launch_embedding<DQ_Q80>(ids, count, vocab, table, NULL, out, embed, out_stride, table_cols, count, 0, stream);
    }
    return ckb_fail(CKB_ERR_SHAPE, "embedding_rows: format %d has no embedding kernel", fmt);
}

extern "C" int ckb200_dev_embedding_forward_q4_k(const int32_t *ids, int count, int vocab, const void *table, const float *pos_emb,
                                                 float *out, int embed, int aligned, int ctx, int add_pos, void *stream)
{ return launch_embedding<DQ_Q4K>(ids, count, vocab, table, pos_emb, out, embed, aligned, aligned, ctx, add_pos, stream); }
extern "C" int ckb200_dev_embedding_forward_q6_k(const int32_t *ids, int count, int vocab, const void *table, const float *pos_emb,
                                                 float *out, int embed, int aligned, int ctx, int add_pos, void *stream)
{ return launch_embedding<DQ_Q6K>(ids, count, vocab, table, pos_emb, out, embed, aligned, aligned, ctx, add_pos, stream); }
extern "C" int ckb200_dev_embedding_forward_q8_0(const int32_t *ids, int count, int vocab, const void *table, const float *pos_emb,
                                                 float *out, int embed, int aligned, int ctx, int add_pos, void *stream)
{ return launch_embedding<DQ_Q80>(ids, count, vocab, table, pos_emb, out, embed, aligned, aligned, ctx, add_pos, stream); }
