// Shared device helpers: block layouts of the quantised formats, streaming loads,
// mbarrier / bulk-copy wrappers with bounded waits, and the error word.
//
// Block layouts follow the reference's include/ckernel_quant.h:104-157 byte for byte.
#pragma once

#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace ckb {

constexpr int QK_K = 256;
constexpr int QK8_0 = 32;
constexpr int Q4K_BYTES = 144;   // fp16 d, fp16 dmin, 12 packed scale bytes, 128 nibble bytes
constexpr int Q6K_BYTES = 210;   // 128 ql, 64 qh, 16 int8 scales, fp16 d
constexpr int Q80_BYTES = 34;    // fp16 d, 32 int8
constexpr int Q50_BYTES = 22;    // fp16 d, 4 bytes of fifth bits, 16 nibble bytes (block_q5_0)
constexpr int Q8K_BYTES = 292;   // fp32 d, 256 int8, 16 int16 bsums

// Device-side error word (one per library).  A kernel that gives up on a bounded wait
// writes a non-zero code here and returns; the host reads it after the next sync.
enum DeviceError : int {
    DEV_OK = 0,
    DEV_ERR_FULL_WAIT = 1,    // consumer gave up waiting for a staged tile
    DEV_ERR_EMPTY_WAIT = 2,   // producer gave up waiting for a free stage
    DEV_ERR_TMEM_ALLOC = 3,
    DEV_ERR_MMA_WAIT = 4,
};

__device__ __forceinline__ uint32_t smem_u32(const void *p) {
    return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

// 16-byte read-only streaming load that does not allocate in L1 (each weight byte is used once).
__device__ __forceinline__ uint4 ldg_stream_u4(const void *p) {
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
    return v;
}
__device__ __forceinline__ uint32_t ldg_stream_u32(const void *p) {
    uint32_t v;
    asm volatile("ld.global.nc.L1::no_allocate.u32 %0, [%1];" : "=r"(v) : "l"(p));
    return v;
}
__device__ __forceinline__ uint32_t ldg_nc_u16(const void *p) {
    unsigned short v;
    asm volatile("ld.global.nc.u16 %0, [%1];" : "=h"(v) : "l"(p));
    return v;
}

__device__ __forceinline__ uint32_t lds_u32(uint32_t addr) {
    uint32_t v;
    asm volatile("ld.shared.u32 %0, [%1];" : "=r"(v) : "r"(addr));
    return v;
}
__device__ __forceinline__ uint4 lds_u4(uint32_t addr) {
    uint4 v;
    asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr));
    return v;
}
__device__ __forceinline__ float4 lds_f4(uint32_t addr) {
    float4 v;
    asm volatile("ld.shared.v4.f32 {%0, %1, %2, %3}, [%4];" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "r"(addr));
    return v;
}
__device__ __forceinline__ uint32_t lds_u16(uint32_t addr) {
    unsigned short v;
    asm volatile("ld.shared.u16 %0, [%1];" : "=h"(v) : "r"(addr));
    return v;
}
__device__ __forceinline__ int lds_s8(uint32_t addr) {
    int v;
    asm volatile("ld.shared.s8 %0, [%1];" : "=r"(v) : "r"(addr));
    return v;
}

__device__ __forceinline__ float half_bits_to_float(uint32_t h16) {
    return __half2float(__ushort_as_half(static_cast<unsigned short>(h16)));
}

__device__ __forceinline__ int dp4a_ss(uint32_t a, uint32_t b, int c) {   // signed x signed bytes
    return __dp4a(static_cast<int>(a), static_cast<int>(b), c);
}
__device__ __forceinline__ int dp4a_us(uint32_t a_unsigned, uint32_t b_signed, int c) {
    int d;
    asm("dp4a.u32.s32 %0, %1, %2, %3;" : "=r"(d) : "r"(a_unsigned), "r"(b_signed), "r"(c));
    return d;
}

template <int WIDTH>
__device__ __forceinline__ float group_sum(float v) {   // sum over WIDTH adjacent lanes (power of two)
#pragma unroll
    for (int o = WIDTH / 2; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

// ---- mbarrier + 1-D bulk async copy (global -> shared), all waits bounded ----

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void mbar_fence_init() {
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
    return ok != 0;
}
// Returns false if the barrier did not flip within the iteration limit (about a second).
__device__ __forceinline__ bool mbar_wait_bounded(uint32_t bar, uint32_t parity) {
    for (uint32_t i = 0; i < (1u << 22); ++i) {
        if (mbar_try_wait(bar, parity)) return true;
        if (i > 64) __nanosleep(64);
    }
    return false;
}
// Same contract, for pipelines whose barriers are usually complete already: polls without sleeping and gives up
// after about a second of SM clock cycles.
__device__ __forceinline__ bool mbar_wait_spin(uint32_t bar, uint32_t parity) {
    if (mbar_try_wait(bar, parity)) return true;
    const long long t0 = clock64();
    for (;;) {
#pragma unroll 1
        for (int i = 0; i < 256; ++i)
            if (mbar_try_wait(bar, parity)) return true;
        if (clock64() - t0 > (1ll << 31)) return false;
    }
}
// src and dst 16-byte aligned, bytes a multiple of 16.  No multicast: one CTA, its own shared memory.
__device__ __forceinline__ void bulk_g2s(uint32_t dst_smem, const void *src, uint32_t bytes, uint32_t bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(dst_smem), "l"(src), "r"(bytes), "r"(bar) : "memory");
}

}  // namespace ckb
