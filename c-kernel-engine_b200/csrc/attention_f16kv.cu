// The reference's "Llama-parity" attention: attention_forward_decode_head_major_gqa_flash_f16kv and
// attention_forward_causal_head_major_gqa_flash_strided_f16kv (src/kernels/attention_kernels.c:1673-1744, :3006-3046, :3408-3448).
//
// q, k and v pass through fp16 before use and the output accumulator is rounded to fp16 after EVERY key's update, with the online
// max / sum recurrence.  Rounding after each update makes the result depend on the order of the keys, so split-K over the context
// (what the other decode kernels do) would give a different answer: the accumulator has to walk the keys in order.  What can
// still run in parallel is everything that does not touch the accumulator:
//   1. all scores  s_j = scale * sum_d r16(q_d) r16(k_jd)            - warps over keys, lanes over d
//   2. the running max before key j (a prefix maximum) and from it the pair the reference derives per key:
//        new maximum:  max_scale_j = exp(prev - s_j) (0 for the first key), value_scale_j = 1
//        otherwise:    max_scale_j = 1,                                     value_scale_j = exp(s_j - prev)
//      - one warp, 32 keys per step with a shuffle scan
//   3. per output element d (one thread each), key by key:  o = r16(o * max_scale_j) when key j set a new maximum, then
//      o = r16(o + value_scale_j * r16(v_jd));  and  sum = sum * max_scale_j + value_scale_j
//      - the only serial part.  The value rows arrive through a cp.async ring in shared memory, so the walk never waits for DRAM.
//        For heads of at most 128 elements the four warps that own no output element start the copies and turn each staged chunk into
//        the products value_scale_j * r16(v_jd) one chunk ahead of the walk (rounding by arithmetic, so that the conversion unit stays
//        free for the walk), and the walk takes eight keys at a time with their operands loaded a group ahead: when none of the eight
//        sets a new maximum (almost always) the chain per key is one add and the conversion pair.
// One CTA of 256 threads per (query head, query token).  Scores and the per-key pairs live in shared memory (8 bytes per key).
// Against the reference the dot products are summed in another order and expf is the device's, so parity is by tolerance; the
// rounding sequence itself is the reference's.
#include <cuda_fp16.h>

#include "device_common.cuh"
#include "launch.h"
#include "pdl.cuh"
#include "runtime.h"

namespace ckb {

constexpr int FK_THREADS = 256;
constexpr int FK_MAX_SMEM = 220 * 1024;
constexpr int FK_CHUNK = 32;                       // value rows per staged chunk
constexpr int FK_MIN_STAGES = 4, FK_MAX_STAGES = 8; // chunks in the ring: as many as the shared memory left by the per-key arrays holds

__device__ __forceinline__ float r16(float x) { return __half2float(__float2half_rn(x)); }
// fp32 -> nearest fp16 (ties to even) -> fp32 on the fp32 pipe: Veltkamp's split with 2^13 + 1 keeps 11 significant bits.  Exact for
// 2^-14 <= |x| < 65520 (fp16's normal range up to the value that rounds to infinity); compared there with the conversion pair on five
// million random values and every tie of the fp16 grid.  Outside that range (fp16 subnormals, zero, overflow) the caller has to use r16.
// On a dependent chain it is no faster than the conversion pair (17.6 against 16.4 cycles per add-and-round in a loop of its own); it is
// used where many independent values are rounded while another warp's chain needs the conversion unit.
constexpr float FK_FAST_MIN = 6.103515625e-05f, FK_FAST_MAX = 65520.0f;
__device__ __forceinline__ float r16_fast(float x)
{
    const float c = __fmul_rn(x, 8193.0f);
    return __fsub_rn(c, __fsub_rn(c, x));
}
// r16 for any input: the arithmetic form when the value is in fp16's normal range, the conversion pair otherwise (and for NaN, which fails
// both comparisons).  Used where the result feeds more fp32 arithmetic and the branch is rarely taken.
__device__ __forceinline__ float r16x(float x)
{
    const float ax = fabsf(x);
    float r = r16_fast(x);
    if (!(ax >= FK_FAST_MIN && ax < FK_FAST_MAX)) r = r16(x);
    return r;
}
__device__ __forceinline__ void fk_cp16(uint32_t dst, const void *src) { asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src) : "memory"); }
__device__ __forceinline__ void fk_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void fk_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }
// at most `pending` of this thread's copy groups still in flight (the instruction wants an immediate)
__device__ __forceinline__ void fk_wait_n(int pending)
{
    switch (pending) {
        case 0: fk_wait<0>(); break;
        case 1: fk_wait<1>(); break;
        case 2: fk_wait<2>(); break;
        case 3: fk_wait<3>(); break;
        case 4: fk_wait<4>(); break;
        case 5: fk_wait<5>(); break;
        case 6: fk_wait<6>(); break;
        default: fk_wait<7>(); break;
    }
}

// q/out: rows of `ad` floats at (h * q_tokens + i); k/v: [Hkv][kv_stride][ad].  kv_tokens of query i = base_tokens + i, where
// base_tokens comes from *pos_dev + 1 when pos_dev is given.  VEC: ad % 4 == 0 and 16-byte-aligned rows (float4 score loads, value rows
// staged through shared memory by cp.async `stages` - 1 chunks ahead of the walk); otherwise plain loads.
template <bool VEC>
__global__ void __launch_bounds__(FK_THREADS) attn_f16kv_kernel(const float *__restrict__ q, const float *__restrict__ k, const float *__restrict__ v,
                                                                float *__restrict__ out, int num_heads, int num_kv_heads, int q_tokens, int base_tokens,
                                                                const int *__restrict__ pos_dev, int kv_stride, int hd, int ad, int max_keys, int stages)
{
    extern __shared__ __align__(16) float fk_smem[];
    pdl_wait();
    pdl_trigger();
    const int h = blockIdx.x, i = blockIdx.y;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    constexpr int NW = FK_THREADS / 32;
    int T = (pos_dev ? __ldcg(pos_dev) + 1 : base_tokens) + i;
    T = min(T, min(kv_stride, max_keys));
    float *vs = fk_smem, *ms = fk_smem + max_keys;            // scores, then value_scale; max_scale (-1 = no new maximum at this key)
    float *stage = fk_smem + 2 * max_keys;                    // VEC: `stages` chunks of FK_CHUNK value rows
    const int kvh = (int)((long long)h * num_kv_heads / num_heads);
    const float *qr = q + ((size_t)h * q_tokens + i) * ad;
    const float *kh = k + (size_t)kvh * kv_stride * ad, *vh = v + (size_t)kvh * kv_stride * ad;
    float *orow = out + ((size_t)h * q_tokens + i) * ad;
    const float scale = 1.0f / sqrtf((float)hd);

    // value rows are contiguous: chunk c = rows [c * FK_CHUNK, ...) = one block of FK_CHUNK * ad floats; start the first chunks now
    const int nchunks = (T + FK_CHUNK - 1) / FK_CHUNK, chunk_f4 = FK_CHUNK * ad / 4;
    // (threads first, first + step, ... of the issuing set copy it; every thread of the set commits one group per call)
    auto issue_chunk = [&](int c, int first, int step) {
        if (c < nchunks) {
            const int rows = min(FK_CHUNK, T - c * FK_CHUNK), n4 = rows * ad / 4;
            const float4 *src = reinterpret_cast<const float4 *>(vh + (size_t)c * FK_CHUNK * ad);
            const uint32_t dst = smem_u32(stage + (size_t)(c % stages) * FK_CHUNK * ad);
            for (int x = first; x < n4; x += step) fk_cp16(dst + 16u * (uint32_t)x, src + x);
        }
        fk_commit();
    };
    const bool narrow = hd <= FK_THREADS / 2;                 // half of the threads own no output element and prepare the walk's operands
    if constexpr (VEC) {
        (void)chunk_f4;
        for (int c = 0; c < stages - 1; ++c) issue_chunk(c, tid, FK_THREADS);
    }

    // 1. scores
    if constexpr (VEC) {
        // lane holds q elements 4 lane .. 4 lane + 3 (and + 128 for heads wider than 128); eight keys per warp step, one float4 per key in flight
        const int n4 = hd / 4;
        float4 q0 = make_float4(0.f, 0.f, 0.f, 0.f), q1 = q0;
        if (narrow) {
            // One float4 of a key row per lane, eight keys per warp step, and the next step's rows already in flight while this one is
            // rounded and multiplied.  The rounding of k is the packed conversion (two elements per instruction).
            if (lane < n4) { const float4 t = __ldcg(reinterpret_cast<const float4 *>(qr) + lane); q0 = make_float4(r16x(t.x), r16x(t.y), r16x(t.z), r16x(t.w)); }
            const float4 zero4 = make_float4(0.f, 0.f, 0.f, 0.f);
            auto load8 = [&](float4 (&dst)[8], int j0) {
#pragma unroll
                for (int u = 0; u < 8; ++u)
                    dst[u] = lane < n4 && j0 < T ? __ldcg(reinterpret_cast<const float4 *>(kh + (size_t)min(j0 + u, T - 1) * ad) + lane) : zero4;
            };
            auto dot8 = [&](const float4 (&kk)[8], int j0) {
                float d8[8];
#pragma unroll
                for (int u = 0; u < 8; ++u) {
                    const float2 a = __half22float2(__floats2half2_rn(kk[u].x, kk[u].y)), b = __half22float2(__floats2half2_rn(kk[u].z, kk[u].w));
                    d8[u] = fmaf(q0.w, b.y, fmaf(q0.z, b.x, fmaf(q0.y, a.y, q0.x * a.x)));
                }
                // the eight sums over the 32 lanes with 4 + 2 + 1 + 2 exchanges: each step folds the lanes in half and hands half of the values over
#pragma unroll
                for (int u = 0; u < 4; ++u) {
                    const float keep = (lane & 16) ? d8[u + 4] : d8[u], give = (lane & 16) ? d8[u] : d8[u + 4];
                    d8[u] = keep + __shfl_xor_sync(0xffffffffu, give, 16);
                }
#pragma unroll
                for (int u = 0; u < 2; ++u) {
                    const float keep = (lane & 8) ? d8[u + 2] : d8[u], give = (lane & 8) ? d8[u] : d8[u + 2];
                    d8[u] = keep + __shfl_xor_sync(0xffffffffu, give, 8);
                }
                {
                    const float keep = (lane & 4) ? d8[1] : d8[0], give = (lane & 4) ? d8[0] : d8[1];
                    d8[0] = keep + __shfl_xor_sync(0xffffffffu, give, 4);
                }
                d8[0] += __shfl_xor_sync(0xffffffffu, d8[0], 2);
                d8[0] += __shfl_xor_sync(0xffffffffu, d8[0], 1);
                // lanes with bits (16, 8, 4) = (a, b, c) now hold key 4a + 2b + c
                const int key = j0 + ((lane >> 4) & 1) * 4 + ((lane >> 3) & 1) * 2 + ((lane >> 2) & 1);
                if ((lane & 3) == 0 && key < T) vs[key] = d8[0] * scale;
            };
            float4 ka[8], kb[8];
            const int jstep = 8 * NW;
            int j0 = warp * 8;
            load8(ka, j0);
            for (; j0 < T; j0 += 2 * jstep) {
                load8(kb, j0 + jstep);
                dot8(ka, j0);
                load8(ka, j0 + 2 * jstep);
                if (j0 + jstep < T) dot8(kb, j0 + jstep);
            }
        } else {
        if (lane < n4) { const float4 t = __ldcg(reinterpret_cast<const float4 *>(qr) + lane); q0 = make_float4(r16x(t.x), r16x(t.y), r16x(t.z), r16x(t.w)); }
        if (lane + 32 < n4) { const float4 t = __ldcg(reinterpret_cast<const float4 *>(qr) + lane + 32); q1 = make_float4(r16x(t.x), r16x(t.y), r16x(t.z), r16x(t.w)); }
        for (int j0 = warp * 8; j0 < T; j0 += 8 * NW) {
            float4 kv0[8], kv1[8];
#pragma unroll
            for (int u = 0; u < 8; ++u) {
                const float4 *kr = reinterpret_cast<const float4 *>(kh + (size_t)min(j0 + u, T - 1) * ad);
                kv0[u] = lane < n4 ? __ldcg(kr + lane) : make_float4(0.f, 0.f, 0.f, 0.f);
                kv1[u] = lane + 32 < n4 ? __ldcg(kr + lane + 32) : make_float4(0.f, 0.f, 0.f, 0.f);
            }
#pragma unroll
            for (int u = 0; u < 8; ++u) {
                float dot = q0.x * r16x(kv0[u].x);
                dot = fmaf(q0.y, r16x(kv0[u].y), dot);
                dot = fmaf(q0.z, r16x(kv0[u].z), dot);
                dot = fmaf(q0.w, r16x(kv0[u].w), dot);
                dot = fmaf(q1.x, r16x(kv1[u].x), dot);
                dot = fmaf(q1.y, r16x(kv1[u].y), dot);
                dot = fmaf(q1.z, r16x(kv1[u].z), dot);
                dot = fmaf(q1.w, r16x(kv1[u].w), dot);
#pragma unroll
                for (int o = 16; o; o >>= 1) dot += __shfl_xor_sync(0xffffffffu, dot, o);
                if (lane == 0 && j0 + u < T) vs[j0 + u] = dot * scale;
            }
        }
        }
    } else {
        float qv[8];
#pragma unroll
        for (int e = 0; e < 8; ++e) qv[e] = lane + 32 * e < hd ? r16(__ldcg(qr + lane + 32 * e)) : 0.0f;
        for (int j0 = warp * 4; j0 < T; j0 += 4 * NW) {
            float dot[4] = {0.0f, 0.0f, 0.0f, 0.0f};
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                const int j = min(j0 + u, T - 1);
#pragma unroll
                for (int e = 0; e < 8; ++e)
                    if (lane + 32 * e < hd) dot[u] = fmaf(qv[e], r16(__ldcg(kh + (size_t)j * ad + lane + 32 * e)), dot[u]);
            }
#pragma unroll
            for (int u = 0; u < 4; ++u) {
#pragma unroll
                for (int o = 16; o; o >>= 1) dot[u] += __shfl_xor_sync(0xffffffffu, dot[u], o);
                if (lane == 0 && j0 + u < T) vs[j0 + u] = dot[u] * scale;
            }
        }
    }
    __syncthreads();

    // 2. prefix maximum and the per-key pairs: every warp takes one contiguous segment of the keys (a multiple of 32), first its maximum,
    //    then, starting from the maximum of the segments before it, the scan
    {
        __shared__ float seg_max[NW];
        const int seg = ((T + NW - 1) / NW + 31) & ~31, s0 = warp * seg, s1 = min(T, s0 + seg);
        float mx = -INFINITY;
        for (int j = s0 + lane; j < s1; j += 32) mx = fmaxf(mx, vs[j]);
#pragma unroll
        for (int o = 16; o; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
        if (lane == 0) seg_max[warp] = mx;
        __syncthreads();
        float carry = -INFINITY;
        for (int w = 0; w < warp; ++w) carry = fmaxf(carry, seg_max[w]);
        for (int j0 = s0; j0 < s1; j0 += 32) {
            const int j = j0 + lane;
            const float s = j < T ? vs[j] : -INFINITY;
            float incl = s;
#pragma unroll
            for (int o = 1; o < 32; o <<= 1) {
                const float other = __shfl_up_sync(0xffffffffu, incl, o);
                if (lane >= o) incl = fmaxf(incl, other);
            }
            float prev = __shfl_up_sync(0xffffffffu, incl, 1);
            prev = lane == 0 ? carry : fmaxf(prev, carry);
            if (j < T) {
                if (s > prev) {
                    ms[j] = isfinite(prev) ? expf(prev - s) : 0.0f;
                    vs[j] = 1.0f;
                } else {
                    ms[j] = -1.0f;
                    vs[j] = expf(s - prev);
                }
            }
            carry = fmaxf(carry, __shfl_sync(0xffffffffu, incl, 31));
        }
    }
    __syncthreads();

    // 3. the ordered walk: thread d owns output element d
    if constexpr (VEC) {
        float o = 0.0f, sum = 0.0f;
        // one key, the reference's sequence with the conversion instructions; p = value_scale * r16(v)
        auto slow_key = [&](float m, float w, float p) {
            if (m >= 0.0f) { o = r16x(__fmul_rn(o, m)); sum = __fmul_rn(sum, m); }
            o = r16x(__fadd_rn(o, p));
            sum = __fadd_rn(sum, w);
        };
        if (narrow) {
            // Threads [0, hd) walk chunk c; threads [128, 256) meanwhile start the copy of chunk c + stages - 1 and turn chunk c + 1 into
            // products in place.  One barrier per chunk: behind it chunk c + 2 has landed, the products of chunk c + 1 are visible and the
            // stage of chunk c is free.
            constexpr int HALF = FK_THREADS / 2;
            const bool helper = tid >= HALF;
            const int per_row = ad / 4;
            auto round4 = [&](float4 t, float w) {
                const float lo = fminf(fminf(fabsf(t.x), fabsf(t.y)), fminf(fabsf(t.z), fabsf(t.w)));
                const float hi = fmaxf(fmaxf(fabsf(t.x), fabsf(t.y)), fmaxf(fabsf(t.z), fabsf(t.w)));
                float4 r = make_float4(r16_fast(t.x), r16_fast(t.y), r16_fast(t.z), r16_fast(t.w));
                if (!(lo >= FK_FAST_MIN && hi < FK_FAST_MAX)) r = make_float4(r16(t.x), r16(t.y), r16(t.z), r16(t.w));
                return make_float4(__fmul_rn(w, r.x), __fmul_rn(w, r.y), __fmul_rn(w, r.z), __fmul_rn(w, r.w));
            };
            auto convert_chunk = [&](int c, int first, int step) {
                if (c >= nchunks) return;
                const int j0 = c * FK_CHUNK, rows = min(FK_CHUNK, T - j0);
                float4 *base = reinterpret_cast<float4 *>(stage + (size_t)(c % stages) * FK_CHUNK * ad);
                if (step % per_row == 0) {
                    // a thread keeps its column and takes every (step / per_row)-th row, four rows per pass with the loads ahead of the arithmetic
                    const int col = first % per_row, rstep = step / per_row;
                    for (int r = first / per_row; r < rows; r += 4 * rstep) {
                        float4 t[4];
                        float w[4];
#pragma unroll
                        for (int e = 0; e < 4; ++e) {
                            const int rr = min(r + e * rstep, rows - 1);
                            t[e] = base[rr * per_row + col];
                            w[e] = vs[j0 + rr];
                        }
#pragma unroll
                        for (int e = 0; e < 4; ++e) t[e] = round4(t[e], w[e]);
#pragma unroll
                        for (int e = 0; e < 4; ++e)
                            if (r + e * rstep < rows) base[(r + e * rstep) * per_row + col] = t[e];
                    }
                } else {
                    for (int x = first; x < rows * per_row; x += step) base[x] = round4(base[x], vs[j0 + x / per_row]);
                }
            };
            // Chunks 0 .. stages - 2 were started by all threads before the scores.  The walkers copy nothing after that, so they wait for
            // all of theirs here; the helpers keep copying and wait chunk by chunk (here: chunks 0 and 1).
            if (helper) fk_wait_n(stages - 3); else fk_wait<0>();
            __syncthreads();
            convert_chunk(0, tid, FK_THREADS);
            __syncthreads();
            for (int c = 0; c < nchunks; ++c) {
                if (helper) {
                    issue_chunk(c + stages - 1, tid - HALF, HALF);     // into the stage that chunk c - 1 has left
                    convert_chunk(c + 1, tid - HALF, HALF);
                    fk_wait_n(stages - 3);                    // this thread's groups so far: chunks 0 .. c + stages - 1; chunk c + 2 must have landed
                } else if (tid < hd) {
                    const float *prow = stage + (size_t)(c % stages) * FK_CHUNK * ad + tid;
                    const int j0 = c * FK_CHUNK, rows = min(FK_CHUNK, T - j0);
                    if (rows == FK_CHUNK) {
                        // four groups of eight keys; the operands of the next group are loaded before the chain of this one starts
                        float m8[8], w8[8], p8[8], mn[8], wn[8], pn[8];
                        auto load_group = [&](float (&m)[8], float (&w)[8], float (&pp)[8], int u) {
                            *reinterpret_cast<float4 *>(m) = *reinterpret_cast<const float4 *>(ms + j0 + u);
                            *reinterpret_cast<float4 *>(m + 4) = *reinterpret_cast<const float4 *>(ms + j0 + u + 4);
                            *reinterpret_cast<float4 *>(w) = *reinterpret_cast<const float4 *>(vs + j0 + u);
                            *reinterpret_cast<float4 *>(w + 4) = *reinterpret_cast<const float4 *>(vs + j0 + u + 4);
#pragma unroll
                            for (int e = 0; e < 8; ++e) pp[e] = prow[(size_t)(u + e) * ad];
                        };
                        auto walk_group = [&](const float (&m)[8], const float (&w)[8], const float (&pp)[8]) {
                            const float newmax = fmaxf(fmaxf(fmaxf(m[0], m[1]), fmaxf(m[2], m[3])), fmaxf(fmaxf(m[4], m[5]), fmaxf(m[6], m[7])));
                            bool exact = newmax < 0.0f;       // the same for every thread: the factors belong to the keys
                            if (exact) {
#pragma unroll
                                for (int e = 0; e < 8; ++e) {
                                    o = r16(__fadd_rn(o, pp[e]));
                                    sum = __fadd_rn(sum, w[e]);
                                }
                            }
                            if (!exact) {
#pragma unroll
                                for (int e = 0; e < 8; ++e) slow_key(m[e], w[e], pp[e]);
                            }
                        };
                        load_group(m8, w8, p8, 0);
                        load_group(mn, wn, pn, 8);
                        walk_group(m8, w8, p8);
                        load_group(m8, w8, p8, 16);
                        walk_group(mn, wn, pn);
                        load_group(mn, wn, pn, 24);
                        walk_group(m8, w8, p8);
                        walk_group(mn, wn, pn);
                    } else {
                        for (int u = 0; u < rows; ++u) slow_key(ms[j0 + u], vs[j0 + u], prow[(size_t)u * ad]);
                    }
                }
                __syncthreads();
            }
        } else {
            for (int c = 0; c < nchunks; ++c) {
                issue_chunk(c + stages - 1, tid, FK_THREADS); // into the stage that chunk c - 1 has just left (the barrier at the loop's end)
                fk_wait_n(stages - 1);
                __syncthreads();                              // chunk c has landed for every thread
                if (tid < hd) {
                    const float *vrow = stage + (size_t)(c % stages) * FK_CHUNK * ad + tid;
                    const int j0 = c * FK_CHUNK, rows = min(FK_CHUNK, T - j0);
                    for (int u = 0; u < rows; ++u) {
                        const float w = vs[j0 + u];
                        slow_key(ms[j0 + u], w, __fmul_rn(w, r16x(vrow[(size_t)u * ad])));
                    }
                }
                __syncthreads();                              // everyone is done with this stage before it is refilled
            }
        }
        fk_wait<0>();
        for (int d = tid; d < ad; d += FK_THREADS) {
            if (d >= hd) orow[d] = 0.0f;
            else if (d == tid) orow[d] = sum > 0.0f ? __fmul_rn(o, __fdiv_rn(1.0f, sum)) : 0.0f;
        }
    } else {
        for (int d = tid; d < ad; d += FK_THREADS) {
            if (d >= hd) { orow[d] = 0.0f; continue; }
            float o = 0.0f, sum = 0.0f;
            const float *vp = vh + d;
            for (int j = 0; j < T; ++j) {
                const float m = ms[j], w = vs[j], vv = r16(__ldcg(vp + (size_t)j * ad));
                if (m >= 0.0f) { o = r16(__fmul_rn(o, m)); sum = __fmul_rn(sum, m); }
                o = r16(__fadd_rn(o, __fmul_rn(w, vv)));
                sum = __fadd_rn(sum, w);
            }
            orow[d] = sum > 0.0f ? __fmul_rn(o, __fdiv_rn(1.0f, sum)) : 0.0f;
        }
    }
}

static int launch_f16kv(const float *q, const float *k, const float *v, float *out, int num_heads, int num_kv_heads, int q_tokens, int base_tokens,
                        const int *pos_dev, int kv_stride, int hd, int ad, int max_keys, cudaStream_t st, const char *what)
{
    if (hd <= 0 || hd > 256 || ad < hd || num_heads <= 0 || num_kv_heads <= 0 || q_tokens <= 0) return ckb_fail(CKB_ERR_SHAPE, "%s: head size %d / %d not handled", what, hd, ad);
    max_keys = (max_keys + 3) & ~3;                           /* the arrays behind the per-key pairs start on 16-byte boundaries */
    const bool vec = ad % 4 == 0 && hd % 4 == 0 && hd <= FK_THREADS && !((((uintptr_t)q | (uintptr_t)k | (uintptr_t)v) & 15));
    const size_t keys_bytes = (size_t)max_keys * 2 * sizeof(float), stage_bytes = (size_t)FK_CHUNK * ad * sizeof(float);
    int stages = 0;
    if (vec) {
        stages = keys_bytes < FK_MAX_SMEM ? (int)((FK_MAX_SMEM - keys_bytes) / stage_bytes) : 0;
        if (stages > FK_MAX_STAGES) stages = FK_MAX_STAGES;
    }
    const size_t smem = keys_bytes + (size_t)stages * stage_bytes;
    if (smem > FK_MAX_SMEM || (vec && stages < FK_MIN_STAGES))
        return ckb_fail(CKB_ERR_LIMIT, "%s: %d keys need %zu bytes of shared memory for the ordered walk (limit about %d keys)", what, max_keys,
                        keys_bytes + FK_MIN_STAGES * stage_bytes, (int)((FK_MAX_SMEM - FK_MIN_STAGES * stage_bytes) / 8));
    static int attr_set = 0;
    if (!attr_set) {
        if (ckb_check_cuda((int)cudaFuncSetAttribute(attn_f16kv_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, FK_MAX_SMEM), "attn_f16kv smem attr") ||
            ckb_check_cuda((int)cudaFuncSetAttribute(attn_f16kv_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, FK_MAX_SMEM), "attn_f16kv smem attr"))
            return CKB_ERR_CUDA;
        attr_set = 1;
    }
    if (vec)
        return launch_pdl(what, attn_f16kv_kernel<true>, dim3(num_heads, q_tokens), dim3(FK_THREADS), smem, st, q, k, v, out, num_heads, num_kv_heads, q_tokens, base_tokens,
                          pos_dev, kv_stride, hd, ad, max_keys, stages);
    return launch_pdl(what, attn_f16kv_kernel<false>, dim3(num_heads, q_tokens), dim3(FK_THREADS), smem, st, q, k, v, out, num_heads, num_kv_heads, q_tokens, base_tokens,
                      pos_dev, kv_stride, hd, ad, max_keys, stages);
}

}  // namespace ckb

using namespace ckb;

// q/out [H][ad], caches [Hkv][cache_capacity][ad]; with pos_dev the context length is *pos_dev + 1, read on the device (the shared
// memory is then sized for the whole cache).
extern "C" int ckb200_dev_attention_decode_f16kv(const float *q, const float *k_cache, const float *v_cache, float *out, int num_heads, int num_kv_heads,
                                                 int kv_tokens, int cache_capacity, int head_dim, int aligned_head_dim, const int *pos_dev, void *stream)
{
    if (!q || !k_cache || !v_cache || !out) return 0;
    if (!pos_dev && (kv_tokens <= 0 || kv_tokens > cache_capacity)) return 0;
    if (cache_capacity <= 0) return 0;
    return launch_f16kv(q, k_cache, v_cache, out, num_heads, num_kv_heads, 1, kv_tokens, pos_dev, cache_capacity, head_dim, aligned_head_dim,
                        pos_dev ? cache_capacity : kv_tokens, ckb_stream(stream), "attention_decode_f16kv");
}

// q/out [H][T][ad], k/v [Hkv][kv_stride][ad]; query i sees keys 0..i
extern "C" int ckb200_dev_attention_prefill_f16kv(const float *q, const float *k, const float *v, float *out, int num_heads, int num_kv_heads, int num_tokens,
                                                  int head_dim, int aligned_head_dim, int kv_stride_tokens, void *stream)
{
    if (!q || !k || !v || !out) return 0;
    if (num_tokens <= 0 || kv_stride_tokens < num_tokens) return 0;
    return launch_f16kv(q, k, v, out, num_heads, num_kv_heads, num_tokens, 1, NULL, kv_stride_tokens, head_dim, aligned_head_dim, num_tokens,
                        ckb_stream(stream), "attention_prefill_f16kv");
}
