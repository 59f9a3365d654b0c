// Tensor-parallel exchange over peer memory: a one-shot fp32 sum all-reduce for the small [batch, hidden] vectors that
// follow the row-parallel o_proj and down_proj GEMVs of a sharded decode step.  The reference has no collective of any
// kind (one process, one thread pool: include/ck_threadpool.h:1-30); NCCL (tp_nccl.c) is the general path, this kernel is
// the latency path: there are two exchanges per layer and each carries only 32 KB per rank at batch 1.
//
// One process per GPU.  Every rank owns one buffer (cudaMalloc, exported with cudaIpcGetMemHandle, opened by its peers):
//     lines [2 parities][world sources][max_floats / 2] x 16 bytes   { value 2i, call number, value 2i+1, call number }
// Data and flag travel in the same 16-byte store (each 8-byte half is written atomically and carries its own copy of the
// call number), so a receiver that reads both call numbers equal to the current one holds both values: no fence, no
// separate flag, one NVLink crossing of latency.  A call (number e, parity e & 1) on rank r: every thread stores its
// lines into slot (e & 1, r) of every PEER, then polls the same lines of slots (e & 1, s) in its OWN buffer for the
// other sources s, and sums the world values in rank order (deterministic; its own value comes from registers).  Only
// local memory is ever polled or read.  Two parities are enough: a rank cannot finish call e + 1 before every peer has
// stored for e + 1, which a peer does only after it has finished reading call e.  The call number lives in device memory
// and is advanced by the last CTA of a call, so a captured CUDA graph can be replayed.
//
// The poll is bounded (tune key wait_limit_ms, ten seconds by default: ranks reach their first step at different times; the
// limit is read when a call is issued, so a captured graph keeps the value it was captured with); a timeout sets the device
// error word and leaves the vector unreduced, and while that word is set no later call polls at all, so a lost peer costs
// one timeout, not one per call.  The host sees the word at its next synchronising call (CKB_ERR_DEVICE_WAIT).  After a
// timeout the ranks' call numbers may differ: ckb200_tp_p2p_shutdown + create + connect on every rank starts over.
// No multicast, no peer loads: remote stores only.
#include "add_rmsnorm_q8k.cuh"
#include "device_common.cuh"
#include "launch.h"
#include "pdl.cuh"
#include "runtime.h"

#include <string.h>

namespace ckb {

constexpr int P2P_MAX_CTAS = 32, P2P_THREADS = 256, P2P_MAX_WORLD = 8;

struct P2PView {
    uint4 *lines[P2P_MAX_WORLD];         // line area of every rank's buffer (this rank's own included)
    unsigned *epoch;                     // this rank's call number, and behind it the count of CTAs that finished the call
    size_t max_lines;
    int rank, world;
};

__device__ __forceinline__ void st_line(uint4 *p, const uint4 &v)
{
    asm volatile("st.volatile.global.v4.u32 [%0], {%1,%2,%3,%4};" ::"l"(p), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
}
__device__ __forceinline__ uint4 ld_line(const uint4 *p)
{
    uint4 v;
    asm volatile("ld.volatile.global.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p) : "memory");
    return v;
}

__global__ void __launch_bounds__(P2P_THREADS) tp_allreduce_push_kernel(float *__restrict__ buf, size_t count, P2PView v, long long wait_limit, int *__restrict__ dev_err)
{
    pdl_trigger();
    pdl_wait();
    const int W = v.world, me = v.rank;
    const unsigned e = *reinterpret_cast<volatile unsigned *>(v.epoch) + 1u, par = e & 1u;
    const size_t nl = (count + 1) / 2, stride = (size_t)gridDim.x * P2P_THREADS, first = (size_t)blockIdx.x * P2P_THREADS + threadIdx.x;
    const size_t my_slot = ((size_t)par * W + me) * v.max_lines;

    for (size_t i = first; i < nl; i += stride) {
        const float x0 = __ldcg(buf + 2 * i), x1 = 2 * i + 1 < count ? __ldcg(buf + 2 * i + 1) : 0.0f;
        const uint4 line = make_uint4(__float_as_uint(x0), e, __float_as_uint(x1), e);
        for (int r = 0; r < W; ++r)
            if (r != me) st_line(v.lines[r] + my_slot + i, line);
    }
    const long long t0 = clock64();
    bool ok = *reinterpret_cast<volatile int *>(dev_err) == 0;      // after a failure nothing waits again until the host has cleared the error
    for (size_t i = first; i < nl && ok; i += stride) {
        float s0 = 0.0f, s1 = 0.0f;
        for (int src = 0; src < W; ++src) {
            float a, b;
            if (src == me) {
                a = __ldcg(buf + 2 * i);
                b = 2 * i + 1 < count ? __ldcg(buf + 2 * i + 1) : 0.0f;
            } else {
                const uint4 *p = v.lines[me] + ((size_t)par * W + src) * v.max_lines + i;
                uint4 l = ld_line(p);
                while (l.y != e || l.w != e) {
                    if (clock64() - t0 > wait_limit) { ok = false; break; }
                    l = ld_line(p);
                }
                if (!ok) break;
                a = __uint_as_float(l.x);
                b = __uint_as_float(l.z);
            }
            s0 = src ? s0 + a : a;
            s1 = src ? s1 + b : b;
        }
        if (ok) {
            buf[2 * i] = s0;
            if (2 * i + 1 < count) buf[2 * i + 1] = s1;
        }
    }
    if (!ok) atomicExch(dev_err, DEV_ERR_FULL_WAIT);
    __syncthreads();
    if (threadIdx.x == 0) {
        __threadfence();
        if (atomicAdd(v.epoch + 1, 1u) == gridDim.x - 1) {      // last CTA of this call: every CTA has read the call number
            v.epoch[1] = 0;
            *reinterpret_cast<volatile unsigned *>(v.epoch) = e;
        }
    }
}

// The exchange fused into its consumer: x[t] += sum over ranks of delta[t], then RMSNorm and Q8_K quantisation of the row
// (add_rmsnorm_q8k, step_kernels.cu), one CTA per token row.  Every thread stores its pieces of the local delta into the
// peers' slots, polls its own slots for the other ranks' pieces, and adds them up in rank order, the same order and
// arithmetic as tp_allreduce_push_kernel followed by add_rmsnorm_q8k, so both forms give the same bits.  Line index of
// piece i of row t: t * aligned / 2 + 2 i (+1): the whole [tokens][aligned] vector is one call of the exchange.
__global__ void __launch_bounds__(1024) tp_add_rmsnorm_q8k_kernel(float *__restrict__ x, const float *__restrict__ delta, const float *__restrict__ gamma,
                                                                  uint8_t *__restrict__ out_q8, int d_model, int aligned, float eps, P2PView v,
                                                                  long long wait_limit, int *__restrict__ dev_err)
{
    extern __shared__ __align__(16) float row[];
    __shared__ float red[32];
    pdl_trigger();
    pdl_wait();
    const int t = blockIdx.x, W = v.world, me = v.rank;
    const unsigned e = *reinterpret_cast<volatile unsigned *>(v.epoch) + 1u, par = e & 1u;
    float *xr = x + (size_t)t * aligned;
    const float *dr = delta + (size_t)t * aligned;
    const int nv = aligned >> 2;
    const size_t line0 = (size_t)t * (aligned >> 1);
    float4 xv[ARQ_MAX_V4], dv[ARQ_MAX_V4];
#pragma unroll
    for (int k = 0; k < ARQ_MAX_V4; ++k) {
        const int i = threadIdx.x + k * blockDim.x;
        xv[k] = make_float4(0.f, 0.f, 0.f, 0.f);
        dv[k] = xv[k];
        if (i < nv) {
            xv[k] = __ldcg(reinterpret_cast<const float4 *>(xr) + i);
            dv[k] = __ldcg(reinterpret_cast<const float4 *>(dr) + i);
            const uint4 l0 = make_uint4(__float_as_uint(dv[k].x), e, __float_as_uint(dv[k].y), e);
            const uint4 l1 = make_uint4(__float_as_uint(dv[k].z), e, __float_as_uint(dv[k].w), e);
            for (int r = 0; r < W; ++r)
                if (r != me) {
                    uint4 *dst = v.lines[r] + ((size_t)par * W + me) * v.max_lines + line0 + 2 * i;
                    st_line(dst, l0);
                    st_line(dst + 1, l1);
                }
        }
    }
    const long long t0 = clock64();
    bool ok = *reinterpret_cast<volatile int *>(dev_err) == 0;      // after a failure nothing waits again until the host has cleared the error
    float ss = 0.0f;
#pragma unroll
    for (int k = 0; k < ARQ_MAX_V4; ++k) {
        const int i = threadIdx.x + k * blockDim.x;
        if (i < nv) {
            float4 s = make_float4(0.f, 0.f, 0.f, 0.f);
            for (int src = 0; src < W; ++src) {
                float4 a = dv[k];
                if (src != me) {
                    const uint4 *p = v.lines[me] + ((size_t)par * W + src) * v.max_lines + line0 + 2 * i;
                    uint4 l0 = ld_line(p), l1 = ld_line(p + 1);
                    while (ok && (l0.y != e || l0.w != e || l1.y != e || l1.w != e)) {
                        if (clock64() - t0 > wait_limit) ok = false;
                        l0 = ld_line(p);
                        l1 = ld_line(p + 1);
                    }
                    a = make_float4(__uint_as_float(l0.x), __uint_as_float(l0.z), __uint_as_float(l1.x), __uint_as_float(l1.z));
                }
                if (src == 0) s = a;
                else { s.x += a.x; s.y += a.y; s.z += a.z; s.w += a.w; }
            }
            float4 u = xv[k];
            u.x += s.x; u.y += s.y; u.z += s.z; u.w += s.w;
            reinterpret_cast<float4 *>(xr)[i] = u;                 // pad columns of x and delta are zero by construction
            arq_keep_piece(u, i, d_model, row, ss);
        }
    }
    if (!ok) atomicExch(dev_err, DEV_ERR_FULL_WAIT);
    arq_norm_quant(ss, row, red, gamma, out_q8, nullptr, t, d_model, aligned, eps);
    __syncthreads();
    if (threadIdx.x == 0) {
        __threadfence();
        if (atomicAdd(v.epoch + 1, 1u) == gridDim.x - 1) {
            v.epoch[1] = 0;
            *reinterpret_cast<volatile unsigned *>(v.epoch) = e;
        }
    }
}

}  // namespace ckb

using namespace ckb;

static struct {
    uint8_t *local;                      // this rank's buffer
    void *peer_base[P2P_MAX_WORLD];      // opened peer buffers (NULL for self)
    P2PView view;
    size_t bytes;
    int ready;
} g_p2p;

static size_t p2p_line_bytes(int world, size_t max_floats) { return 2 * (size_t)world * (max_floats / 2) * sizeof(uint4); }
static size_t p2p_total_bytes(int world, size_t max_floats) { return p2p_line_bytes(world, max_floats) + 256; }

// Allocates this rank's exchange buffer for vectors of up to max_floats (a multiple of 4) and writes its 64-byte IPC handle.
extern "C" int ckb200_tp_p2p_create(int rank, int world, size_t max_floats, void *handle_out64)
{
    if (!handle_out64 || world < 2 || world > P2P_MAX_WORLD || rank < 0 || rank >= world || max_floats == 0 || max_floats % 4)
        return ckb_fail(CKB_ERR_STATE, "tp_p2p_create: bad rank %d / world %d / size %zu", rank, world, max_floats);
    if (g_p2p.local) return ckb_fail(CKB_ERR_STATE, "tp_p2p_create: already created");
    if (ckb_ensure_init()) return CKB_ERR_NO_DEVICE;
    static_assert(sizeof(cudaIpcMemHandle_t) == 64, "IPC handle size");
    g_p2p.bytes = p2p_total_bytes(world, max_floats);
    if (ckb_check_cuda((int)cudaMalloc((void **)&g_p2p.local, g_p2p.bytes), "cudaMalloc(tp exchange buffer)")) return CKB_ERR_CUDA;
    if (ckb_check_cuda((int)cudaMemset(g_p2p.local, 0, g_p2p.bytes), "cudaMemset(tp exchange buffer)")) return CKB_ERR_CUDA;
    cudaIpcMemHandle_t h;
    if (ckb_check_cuda((int)cudaIpcGetMemHandle(&h, g_p2p.local), "cudaIpcGetMemHandle")) return CKB_ERR_CUDA;
    memcpy(handle_out64, &h, 64);
    memset(&g_p2p.view, 0, sizeof g_p2p.view);
    g_p2p.view.rank = rank;
    g_p2p.view.world = world;
    g_p2p.view.max_lines = max_floats / 2;
    return 0;
}

// all_handles: the 64-byte handles of ranks 0 .. world-1 in rank order (gathered by the host program)
extern "C" int ckb200_tp_p2p_connect(const void *all_handles)
{
    if (!all_handles || !g_p2p.local) return ckb_fail(CKB_ERR_STATE, "tp_p2p_connect: ckb200_tp_p2p_create has not been called");
    const int W = g_p2p.view.world, me = g_p2p.view.rank;
    for (int r = 0; r < W; ++r) {
        uint8_t *base = g_p2p.local;
        if (r != me) {
            cudaIpcMemHandle_t h;
            memcpy(&h, (const uint8_t *)all_handles + 64 * (size_t)r, 64);
            void *p = NULL;
            if (ckb_check_cuda((int)cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess), "cudaIpcOpenMemHandle")) return CKB_ERR_CUDA;
            g_p2p.peer_base[r] = p;
            base = (uint8_t *)p;
        }
        g_p2p.view.lines[r] = (uint4 *)base;
    }
    g_p2p.view.epoch = (unsigned *)(g_p2p.local + p2p_line_bytes(W, 2 * g_p2p.view.max_lines));
    g_p2p.ready = 1;
    return 0;
}

// Every "peer" is this rank's own buffer: the stores land in this rank's own source slot and nothing ever fills the other
// sources' slots, so each exchange runs into its wait limit.  For exercising the timeout path on a single GPU.
extern "C" int ckb200_tp_p2p_connect_self(void)
{
    if (!g_p2p.local) return ckb_fail(CKB_ERR_STATE, "tp_p2p_connect_self: ckb200_tp_p2p_create has not been called");
    const int W = g_p2p.view.world;
    for (int r = 0; r < W; ++r) g_p2p.view.lines[r] = (uint4 *)g_p2p.local;
    g_p2p.view.epoch = (unsigned *)(g_p2p.local + p2p_line_bytes(W, 2 * g_p2p.view.max_lines));
    g_p2p.ready = 1;
    return 0;
}

extern "C" int ckb200_tp_p2p_ready(void) { return g_p2p.ready; }
extern "C" size_t ckb200_tp_p2p_max_floats(void) { return g_p2p.ready ? 2 * g_p2p.view.max_lines : 0; }

// In-place sum over all ranks of buf[0 .. count) (count <= max_floats, buf 16-byte aligned); capturable.
extern "C" int ckb_tp_p2p_allreduce(float *buf, size_t count, void *stream)
{
    if (!g_p2p.ready) return ckb_fail(CKB_ERR_STATE, "tp_p2p_allreduce: not connected");
    if (count > 2 * g_p2p.view.max_lines) return ckb_fail(CKB_ERR_LIMIT, "tp_p2p_allreduce: %zu floats exceed the exchange buffer", count);
    if (count == 0) return 0;
    const size_t nl = (count + 1) / 2;
    size_t ctas = (nl + P2P_THREADS - 1) / P2P_THREADS;
    if (ctas > P2P_MAX_CTAS) ctas = P2P_MAX_CTAS;
    return launch_pdl("tp_allreduce_push", tp_allreduce_push_kernel, dim3((unsigned)ctas), dim3(P2P_THREADS), 0, ckb_stream(stream), buf, count, g_p2p.view,
                      ckb_wait_limit_cycles(), ckb_device_error_word());
}

// ckb200_tp_norm_fn: x[t] += sum over ranks of delta[t]; out_q8[t] = Q8_K(rmsnorm(x[t]) * gamma).  Returns -1 when the
// exchange buffer cannot take the vector (not connected, too large, switched off): the caller then reduces and normalises
// in two steps.
extern "C" int ckb200_tp_add_rmsnorm_q8k(void *ctx, float *x, const float *delta, const float *gamma, void *out_q8, int tokens, int d_model,
                                         int aligned_embed_dim, float eps, void *stream)
{
    (void)ctx;
    if (!g_p2p.ready || !ckb_tune_get("tp_p2p", 1)) return -1;
    // One CTA per token row stores to and then polls every peer in turn: with two ranks that is as fast as the 16-CTA all-reduce
    // kernel plus the norm kernel and saves a launch; from four ranks up the serial peer loop loses (8 ranks, 70B shape, batch 1:
    // 9.1 ms per token against 6.1), so the default there is all-reduce kernel + norm kernel.  tp_fused_norm = 1 / 0 forces either.
    const int fused = ckb_tune_get("tp_fused_norm", -1);
    if (fused == 0 || (fused < 0 && g_p2p.view.world > 2)) return -1;
    if (!x || !delta || !gamma || !out_q8 || tokens <= 0 || d_model <= 0) return -1;
    if (aligned_embed_dim % QK_K || aligned_embed_dim < d_model || aligned_embed_dim > 1024 * 4 * ARQ_MAX_V4) return -1;
    if ((size_t)tokens * aligned_embed_dim > 2 * g_p2p.view.max_lines || (((uintptr_t)x | (uintptr_t)delta) & 15)) return -1;
    int threads = (aligned_embed_dim / 4 + 31) & ~31;
    if (threads > 1024) threads = 1024;
    const size_t smem = (size_t)aligned_embed_dim * sizeof(float);
    if (smem > 48 * 1024) {
        static size_t set = 0;
        if (smem > set) {
            if (ckb_check_cuda((int)cudaFuncSetAttribute(tp_add_rmsnorm_q8k_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem), "smem attr")) return CKB_ERR_CUDA;
            set = smem;
        }
    }
    return launch_pdl("tp_add_rmsnorm_q8k", tp_add_rmsnorm_q8k_kernel, dim3(tokens), dim3(threads), smem, ckb_stream(stream), x, delta, gamma, (uint8_t *)out_q8,
                      d_model, aligned_embed_dim, eps, g_p2p.view, ckb_wait_limit_cycles(), ckb_device_error_word());
}

extern "C" void ckb200_tp_p2p_shutdown(void)
{
    if (!g_p2p.local) return;
    cudaStreamSynchronize(ckb_stream(NULL));
    for (int r = 0; r < P2P_MAX_WORLD; ++r)
        if (g_p2p.peer_base[r]) { cudaIpcCloseMemHandle(g_p2p.peer_base[r]); g_p2p.peer_base[r] = NULL; }
    cudaFree(g_p2p.local);
    memset(&g_p2p, 0, sizeof g_p2p);
}
