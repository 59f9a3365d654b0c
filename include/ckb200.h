/*
 * ckb200.h - C ABI of libckb200.so, the B200 (sm_100a) implementation of C-Kernel-Engine's
 * quantised decode/prefill hot path.
 *
 * Two layers, both plain C (pointers and sizes only):
 *
 *  1. Device-pointer entry points, `ckb200_dev_*`: every pointer is DEVICE memory, the call
 *     enqueues kernels on `stream` (a cudaStream_t passed as void*, NULL = the library's own
 *     stream) and returns without synchronising.  This is the path the whole-step executor
 *     uses and the one whose throughput is measured against the HBM / tensor roofline.
 *
 *  2. Reference-named entry points (include/ckb200_kernels.h): the reference's own symbols
 *     with the reference's own signatures and HOST pointers, for generated libmodel.so code,
 *     the reference's ctypes unit tests and the *_parallel_dispatch seam.  They copy
 *     activations in and results out around the same kernels.  Weights registered with
 *     ckb200_register_weights() stay resident in HBM and are found by host address range.
 *
 * Every int-returning function returns 0 on success or a CKB_ERR_* code (also kept for
 * ckb200_last_error()).  Nothing aborts; there is no CPU fallback: without a CUDA device
 * every compute call fails with CKB_ERR_NO_DEVICE.
 *
 * Citations are file:line inside the reference project (C-Kernel-Engine).
 */
#ifndef CKB200_H
#define CKB200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* ------------------------------------------------------------------ runtime + error channel
 * The reference's kernels are void and return silently on bad arguments
 * (src/kernels/gemm_kernels_q4k_q8k.c:188-190); GPU-only failures are reported here instead. */
int ckb200_init(int device);                 /* select device, create the stream; idempotent */
void ckb200_shutdown(void);                  /* free scratch, registry and stream */
int ckb200_last_error(void);
const char *ckb200_last_error_message(void);
void ckb200_clear_error(void);
int ckb200_synchronize(void);                /* sync the library stream; folds in the device error word */
void *ckb200_stream(void);                   /* cudaStream_t of the library */
long long ckb200_launch_count(void);         /* kernels launched by this library since load */
int ckb200_tune_set(const char *key, int value);   /* kernel-variant switches for tuning runs */
int ckb200_tune_get(const char *key, int dflt);

/* Weights are immutable after load (generated code reads them from one bump arena at fixed
 * offsets, version/v7/scripts/codegen_v7.py:1211-1232).  Registering the arena (or any
 * weight buffer) uploads it once; later calls that pass a host pointer inside
 * [host_ptr, host_ptr+bytes) use the device copy. */
int ckb200_register_weights(const void *host_ptr, size_t bytes);
int ckb200_unregister_weights(const void *host_ptr);
void ckb200_unregister_all(void);
const void *ckb200_device_ptr(const void *host_ptr);   /* NULL if not inside a registered range */

/* Synchronous copies between host memory and device pointers handed out by this library. */
int ckb200_copy_to_device(void *dev, const void *host, size_t bytes);
int ckb200_copy_to_host(void *host, const void *dev, size_t bytes);

/* Pinned host memory for callers that want the host<->device copies to run at full PCIe rate. */
void *ckb200_host_alloc(size_t bytes);
void ckb200_host_free(void *p);

/* ------------------------------------------------------------------ device-pointer kernels */

/* quantize_row_q8_k / quantize_batch_q8_k (src/kernels/gemm_kernels_q4k_q8k.c:53-119,
 * src/kernels/gemm_kernels_q8_0.c:221-239): x fp32 [rows, k] -> block_q8_K [rows, k/256]; bit-exact. */
int ckb200_dev_quantize_q8_k(const float *x, void *y, int rows, int k, void *stream);
/* quantize_row_q8_0 / quantize_batch_q8_0 (src/kernels/gemm_kernels_q8_0.c:70-209); bit-exact. */
int ckb200_dev_quantize_q8_0(const float *x, void *y, int rows, int k, void *stream);

/* gemv_q4_k_q8_k (src/kernels/gemm_kernels_q4k_q8k.c:183-263): y[M] = W[M, K/256 x 144 B] . x_q8. */
int ckb200_dev_gemv_q4_k_q8_k(float *y, const void *W, const void *x_q8, int M, int K, void *stream);
/* gemv_q6_k_q8_k (src/kernels/gemm_kernels_q6k_q8k.c:1060-1088): 210-byte superblocks. */
int ckb200_dev_gemv_q6_k_q8_k(float *y, const void *W, const void *x_q8, int M, int K, void *stream);
/* gemv_q8_0_q8_0 (src/kernels/gemm_kernels_q8_0.c:1237-1251): 34-byte blocks, Q8_0 activations. */
int ckb200_dev_gemv_q8_0_q8_0(float *y, const void *W, const void *x_q8, int M, int K, void *stream);

/* gemv_q4_k / gemv_q6_k / gemv_q8_0 with fp32 activations (src/kernels/gemm_kernels_q4k.c:285-297,
 * src/kernels/gemm_kernels_q6k.c:169-193, src/kernels/gemm_kernels_q8_0.c:632-649): the reference's debug path. */
int ckb200_dev_gemv_q4_k(float *y, const void *W, const float *x, int M, int K, void *stream);
int ckb200_dev_gemv_q6_k(float *y, const void *W, const float *x, int M, int K, void *stream);
int ckb200_dev_gemv_q8_0(float *y, const void *W, const float *x, int M, int K, void *stream);

/* dequant_q4_k_row / dequant_q6_k_row / dequant_q8_0_row (src/kernels/dequant_kernels.c:372-380, :422-430, :288-296). */
int ckb200_dev_dequant_q4_k_row(const void *src, float *dst, size_t n_elements, void *stream);
int ckb200_dev_dequant_q6_k_row(const void *src, float *dst, size_t n_elements, void *stream);
int ckb200_dev_dequant_q8_0_row(const void *src, float *dst, size_t n_elements, void *stream);

/* gemm_nt_q4_k_q8_k (src/kernels/gemm_kernels_q4k_q8k.c:301-326), gemm_nt_q6_k_q8_k
 * (src/kernels/gemm_kernels_q6k_q8k.c:1243-1268), gemm_nt_q8_0_q8_0 (src/kernels/gemm_batch_int8.c:87-120):
 * C[M,N] = A_q8[M,K] . B[N,K]^T + bias[N] (bias may be NULL). */
/* Q5_0 weights (block_q5_0, include/ckernel_quant.h:70-74: fp16 d, 4 bytes of fifth bits, 16 nibble bytes = 22 B per 32) with
 * Q8_0 activations: gemv_q5_0_q8_0 / gemm_nt_q5_0_q8_0 (src/kernels/gemm_kernels_q5_0.c:1637-1651, :1725-1752); the int32 block
 * sums are exact, fp32 accumulation in block order. */
int ckb200_dev_gemv_q5_0_q8_0(float *y, const void *W, const void *x_q8, int M, int K, void *stream);
/* dequant_q5_0_row (src/kernels/dequant_kernels.c:198-206) and the fp32-activation gemv_q5_0 (src/kernels/gemm_kernels_q5_0.c:67-111) */
int ckb200_dev_dequant_q5_0_row(const void *src, float *dst, size_t n_elements, void *stream);
int ckb200_dev_gemv_q5_0(float *y, const void *W, const float *x, int M, int K, void *stream);
/* Further weight formats (parity path, not tuned).  Q5_K x Q8_K (src/kernels/gemm_kernels_q5_k.c:128-208, :305-367) and Q5_1 x Q8_1 with its
 * activation quantiser (src/kernels/gemm_kernels_q5_1_q8_1.c:27-122): integer block sums combined in the reference's fp32 order, bit-identical
 * to the scalar loops; M tokens per call (M = 1: the GEMV).  Row dequantisers of Q4_0 / Q4_1 / Q5_1 (src/kernels/dequant_kernels.c:40-260) and
 * fp32-activation GEMVs in the element order of the reference's own GEMVs (src/kernels/gemm_kernels_q4_0.c:49-78, gemm_kernels_q4_1.c:50-84,
 * gemm_kernels_q5_1.c:52-100); gemv_q5_k_f32 is the fp32 fall-back of gemv_q5_k (src/kernels/gemm_kernels_q5_k.c:211-245). */
int ckb200_dev_gemm_nt_q5_k_q8_k(const void *A_q8, const void *B, const float *bias, float *C, int M, int N, int K, void *stream);
int ckb200_dev_gemv_q5_k_q8_k(float *y, const void *W, const void *x_q8, int M, int K, void *stream);
int ckb200_dev_quantize_q8_1(const float *x, void *y, int rows, int k, void *stream);
int ckb200_dev_gemm_nt_q5_1_q8_1(const void *A_q8, const void *B, const float *bias, float *C, int M, int N, int K, void *stream);
int ckb200_dev_dequant_q4_0_row(const void *src, float *dst, size_t n_elements, void *stream);
int ckb200_dev_dequant_q4_1_row(const void *src, float *dst, size_t n_elements, void *stream);
int ckb200_dev_dequant_q5_1_row(const void *src, float *dst, size_t n_elements, void *stream);
int ckb200_dev_gemv_q4_0(float *y, const void *W, const float *x, int M, int K, void *stream);
int ckb200_dev_gemv_q4_1(float *y, const void *W, const float *x, int M, int K, void *stream);
int ckb200_dev_gemv_q5_1(float *y, const void *W, const float *x, int M, int K, void *stream);
int ckb200_dev_gemv_q5_k_f32(float *y, const void *W, const float *x, int M, int K, void *stream);

/* Resident Q5_0 weights in a row-planar layout (all nibble bytes | all fifth-bit words | all d, rows padded to 16 B; the same
 * bits, aligned loads): size, conversion from the reference's rows, and the GEMV over it. */
size_t ckb200_q5_0_planar_bytes(int rows, int cols);
int ckb200_dev_q5_0_to_planar(void *dst, const void *src, int rows, int cols, void *stream);
int ckb200_dev_gemv_q5_0_planar_q8_0(float *y, const void *W_planar, const void *x_q8, int M, int K, void *stream);
int ckb200_dev_gemm_nt_q5_0_q8_0(const void *A_q8, const void *B, const float *bias, float *C, int M, int N, int K, void *stream);
int ckb200_dev_gemm_nt_q4_k_q8_k(const void *A_q8, const void *B, const float *bias, float *C, int M, int N, int K, void *stream);
int ckb200_dev_gemm_nt_q6_k_q8_k(const void *A_q8, const void *B, const float *bias, float *C, int M, int N, int K, void *stream);
int ckb200_dev_gemm_nt_q8_0_q8_0(const void *A_q8, const void *B, const float *bias, float *C, int M, int N, int K, void *stream);
/* the bias loop of those functions on its own: c[r][j] += bias[j] */
int ckb200_dev_add_bias_rows(float *c, const float *bias, int rows, int n, void *stream);

/* Q6_K weights that stay resident on the device can be kept in a row-planar layout (per row: all ql, all qh, all
 * scales, all d; same bits, 210 bytes per superblock plus at most 14 bytes of row padding) in which every piece is
 * naturally aligned for 16-byte loads; the block_q6_K stream itself (include/ckernel_quant.h:135-146) is only
 * 2-byte aligned.  ckb200_dev_gemv_q6_k_planar_q8_k gives the same result as ckb200_dev_gemv_q6_k_q8_k
 * (gemv_q6_k_q8_k, src/kernels/gemm_kernels_q6k_q8k.c:197-214) on the original rows. */
size_t ckb200_q6_k_planar_bytes(int rows, int cols);
int ckb200_dev_q6_k_to_planar(void *dst_planar, const void *src_q6k_rows, int rows, int cols, void *stream);
int ckb200_dev_gemv_q6_k_planar_q8_k(float *y, const void *W_planar, const void *x_q8, int M, int K, void *stream);
/* The same for Q8_0 weights (block_q8_0, include/ckernel_quant.h:104-110, 34 bytes, 2-byte aligned): per row all
 * quants, then all d.  Same result as ckb200_dev_gemv_q8_0_q8_0 (gemv_q8_0_q8_0, src/kernels/gemm_kernels_q8_0.c:1237-1251). */
size_t ckb200_q8_0_planar_bytes(int rows, int cols);
int ckb200_dev_q8_0_to_planar(void *dst_planar, const void *src_q8_0_rows, int rows, int cols, void *stream);
int ckb200_dev_gemv_q8_0_planar_q8_0(float *y, const void *W_planar, const void *x_q8_0, int M, int K, void *stream);
/* gemm_nt_q6_k_q8_k (src/kernels/gemm_kernels_q6k_q8k.c:1243-1268) over planar weights: tensor-core kernel from 16 tokens up */
int ckb200_dev_gemm_nt_q6_k_planar_q8_k(const void *A_q8, const void *B_planar, const float *bias, float *C, int M, int N, int K, void *stream);

/* The integer stage of the K-quant dot products, dumped for bit-exact checks.  The reference accumulates int32 sums of
 * (weight code x activation byte) per sub-block before any floating point: for Q4_K the eight 32-element sums
 * sum_q4q8_lo / sum_q4q8_hi of a superblock (dot_q4_k_q8_k_ref, src/kernels/gemm_kernels_q4k_q8k.c:144-167), for Q6_K
 * the sixteen 16-element sums of (q6 - 32) x q8 (dot_q6_k_q8_k_ref, src/kernels/gemm_kernels_q6k_q8k.c:92-111).
 * W: M rows in the reference's layout, x_q8: one Q8_K vector, out: int32 [M][K/256][8] (Q4_K) or [M][K/256][16] (Q6_K).
 * The sums are produced by the device functions the GEMV kernels themselves call; `variant` picks the family:
 * 0 = the tuned kernels' unit (Q4_K pair / register-activation kernels; Q6_K planar and ring kernels, bit-plane form),
 * 1 = the generic direct kernels' unit. */
int ckb200_dev_subblock_sums_q4_k_q8_k(const void *W, const void *x_q8, int M, int K, int32_t *out, int variant, void *stream);
int ckb200_dev_subblock_sums_q6_k_q8_k(const void *W, const void *x_q8, int M, int K, int32_t *out, int variant, void *stream);

/* attention_forward_decode_head_major_gqa_flash (src/kernels/attention_kernels.c:3365-3406) for `batch`
 * independent sequences: q/out [batch][H][ad], caches [batch][Hkv][capacity][ad] with kv_batch_stride floats
 * between sequences.  Split-K over the context; partial results go through a scratch buffer.
 *   ckb200_dev_attention_decode     picks the split count, scratch comes from the library's pool
 *   ckb200_dev_attention_decode_ws  caller gives split count and scratch (ckb200_attention_decode_scratch_bytes);
 *                                   with pos_dev != NULL the context length is *pos_dev + 1, read on the device */
int ckb200_dev_attention_decode(const float *q, const float *k_cache, const float *v_cache, float *out, int batch,
                                long long kv_batch_stride, int num_heads, int num_kv_heads, int kv_tokens,
                                int cache_capacity, int head_dim, int aligned_head_dim, void *stream);
int ckb200_dev_attention_decode_ws(const float *q, const float *k_cache, const float *v_cache, float *out, int batch,
                                   long long kv_batch_stride, int num_heads, int num_kv_heads, int kv_tokens,
                                   int cache_capacity, int head_dim, int aligned_head_dim, int splits, float *scratch,
                                   const int *pos_dev, void *stream);
/* No counterpart in the reference.  The same decode attention for callers that must not allocate device
 * memory on the decode path (a runtime whose device arena was planned at load time, a real-time loop, a
 * process that gave all free memory to another pool): the split-K partials go to a fixed 4 MiB array inside
 * the library instead of a scratch buffer.  splits <= 0 picks the split count; a call that would need more
 * than ckb200_attention_decode_static_scratch_limit() bytes is rejected with CKB_ERR_LIMIT.  Calls share the
 * array: do not overlap two of them on the GPU.  The first call on each device looks the array up; make it
 * before any stream capture.  stream NULL = the legacy default stream.  Calls no cudaMalloc / cudaFree. */
int ckb200_dev_attention_decode_static(const float *q, const float *k_cache, const float *v_cache, float *out, int batch,
                                       long long kv_batch_stride, int num_heads, int num_kv_heads, int kv_tokens,
                                       int cache_capacity, int head_dim, int aligned_head_dim, int splits, void *stream);
size_t ckb200_attention_decode_static_scratch_limit(void);
/* The step executor's form: the same attention, the merge of the context splits and quantize_row_q8_k of the
 * finished rows (src/kernels/gemm_kernels_q4k_q8k.c:53-103; what the o-projection consumes) in ONE launch.
 * out rows are out_stride floats apart; the q8_cols - H*ad floats after each row must be zero; q8_out may be NULL.
 * `counters`: ckb200_attention_decode_counter_bytes() of device memory, zero before the first call (each call
 * leaves it zero).  Shapes outside the tile kernel's fast path run as separate launches with the same result. */
int ckb200_dev_attention_decode_fused(const float *q, const float *k_cache, const float *v_cache, float *out, int out_stride,
                                      int batch, long long kv_batch_stride, int num_heads, int num_kv_heads, int kv_tokens,
                                      int cache_capacity, int head_dim, int aligned_head_dim, int splits, float *scratch,
                                      int *counters, const int *pos_dev, void *q8_out, int q8_cols, void *stream);
size_t ckb200_attention_decode_counter_bytes(int batch, int num_kv_heads);
int ckb200_attention_decode_splits(int batch, int num_kv_heads, int kv_tokens);          /* fp32 cache */
int ckb200_attention_decode_splits_kv(int batch, int num_kv_heads, int kv_tokens, int kv_element_bytes);   /* 4 = fp32, 2 = fp16 */
size_t ckb200_attention_decode_scratch_bytes(int batch, int num_heads, int aligned_head_dim, int splits);

/* fp16 KV cache: kv_cache_store_f16 (src/kernels/kv_cache_kernels.c:131-163; round to nearest even, bit-exact) and
 * attention_forward_decode_head_major_gqa_flash_f16cache (src/kernels/attention_kernels.c:3450-3557): the layouts of the
 * fp32 entry points with 2-byte elements (kv_batch_stride counted in elements, a multiple of 8).  Half the KV bytes per
 * token; the halves are widened to fp32 in shared memory, the arithmetic is the fp32 path's.  Aligned head size 64 or
 * 128 and at most 8 query heads per kv head; other shapes are refused with CKB_ERR_SHAPE. */
int ckb200_dev_kv_cache_store_f16(uint16_t *kv_cache_k, uint16_t *kv_cache_v, const float *k, const float *v, int pos,
                                  const int *pos_dev, int num_kv_heads, int head_dim, int max_seq_len, void *stream);
int ckb200_dev_attention_decode_f16cache(const float *q, const uint16_t *k_cache, const uint16_t *v_cache, float *out, int batch,
                                         long long kv_batch_stride, int num_heads, int num_kv_heads, int kv_tokens, int cache_capacity,
                                         int head_dim, int aligned_head_dim, void *stream);
int ckb200_dev_attention_decode_f16cache_ws(const float *q, const uint16_t *k_cache, const uint16_t *v_cache, float *out, int batch,
                                            long long kv_batch_stride, int num_heads, int num_kv_heads, int kv_tokens, int cache_capacity,
                                            int head_dim, int aligned_head_dim, int splits, float *scratch, const int *pos_dev, void *stream);

/* Prefill attention over head-major fp32 tensors: attention_forward_causal_head_major_gqa_flash[_strided] and
 * attention_forward_full_head_major_gqa_flash[_strided] (src/kernels/attention_kernels.c:2847-3005).
 * q, out [H][T][aligned_head_dim]; k, v [Hkv][kv_stride_tokens][aligned_head_dim]; causal != 0: query token i sees keys
 * 0 .. i, else all T.  Shapes: H a multiple of Hkv with at most 8 query heads per kv head, aligned head size 64 or 128;
 * others are refused with CKB_ERR_SHAPE. */
int ckb200_dev_attention_prefill(const float *q, const float *k, const float *v, float *out, int num_heads, int num_kv_heads,
                                 int num_tokens, int head_dim, int aligned_head_dim, int kv_stride_tokens, int causal, void *stream);
/* The same with a sliding window (src/kernels/attention_kernels_sliding.c:450-600): with causal != 0 and sliding_window > 0
 * token i sees keys max(0, i - sliding_window + 1) .. i; decode: the query sees the last min(kv_tokens, sliding_window) rows. */
int ckb200_dev_attention_prefill_window(const float *q, const float *k, const float *v, float *out, int num_heads, int num_kv_heads,
                                        int num_tokens, int head_dim, int aligned_head_dim, int kv_stride_tokens, int causal,
                                        int sliding_window, void *stream);
int ckb200_dev_attention_decode_sliding(const float *q, const float *k_cache, const float *v_cache, float *out, int batch,
                                        long long kv_batch_stride, int num_heads, int num_kv_heads, int kv_tokens, int cache_capacity,
                                        int head_dim, int aligned_head_dim, int sliding_window, void *stream);
/* attention_forward_decode_head_major_gqa_flash_f16kv (src/kernels/attention_kernels.c:3408-3448) and
 * attention_forward_causal_head_major_gqa_flash_strided_f16kv (:3006-3046), the form the llama template binds: q, k, v go
 * through fp16 and the output accumulator is rounded to fp16 after every key, in key order.  One sequence; with pos_dev the
 * context length is *pos_dev + 1.  At most 25 600 keys (the per-key factors of the ordered walk live in shared memory). */
int ckb200_dev_attention_decode_f16kv(const float *q, const float *k_cache, const float *v_cache, float *out, int num_heads, int num_kv_heads,
                                      int kv_tokens, int cache_capacity, int head_dim, int aligned_head_dim, const int *pos_dev, void *stream);
int ckb200_dev_attention_prefill_f16kv(const float *q, const float *k, const float *v, float *out, int num_heads, int num_kv_heads, int num_tokens,
                                       int head_dim, int aligned_head_dim, int kv_stride_tokens, void *stream);

/* kv_cache_store (src/kernels/kv_cache_kernels.c:111-129): k, v [Hkv][head_dim] -> cache[Hkv][max_seq][head_dim] at pos
 * (or at *pos_dev when given). */
int ckb200_dev_kv_cache_store(float *kv_cache_k, float *kv_cache_v, const float *k, const float *v, int pos,
                              const int *pos_dev, int num_kv_heads, int head_dim, int max_seq_len, void *stream);
/* rmsnorm_forward (src/kernels/rmsnorm_kernels.c:126-250). */
int ckb200_dev_rmsnorm_forward(const float *input, const float *gamma, float *output, float *rstd_cache, int tokens,
                               int d_model, int aligned_embed_dim, float eps, void *stream);
/* rope_precompute_cache_split (src/kernels/rope_kernels.c:221-243) and rope_forward_qk (:806-819), rotate-half. */
int ckb200_dev_rope_precompute_cache_split(float *cos_cache, float *sin_cache, int max_seq_len, int head_dim, float base, void *stream);
int ckb200_dev_rope_forward_qk(float *q, float *k, const float *cos_cache, const float *sin_cache, int num_heads,
                               int num_kv_heads, int num_tokens, int head_dim, int aligned_head_dim, int pos_offset,
                               const int *pos_dev, void *stream);
/* rope_forward_qk_with_rotary_dim (src/kernels/rope_kernels.c:821-837): half-split pairs (i, i + rotary_dim / 2) of the first
 * rotary_dim channels, tables with rows of rotary_dim / 2 values (rope_precompute_cache). */
int ckb200_dev_rope_forward_qk_with_rotary_dim(float *q, float *k, const float *cos_cache, const float *sin_cache, int num_heads,
                                               int num_kv_heads, int num_tokens, int head_dim, int aligned_head_dim, int pos_offset,
                                               int rotary_dim, const int *pos_dev, void *stream);
/* rope_precompute_cache (src/kernels/rope_kernels.c:270-316): rows of rotary_dim / 2 values (rotary_dim <= 0 or > head_dim means
 * head_dim), positions divided by scaling_factor when linear_scaling != 0; and rope_forward_qk_pairwise_with_rotary_dim
 * (:839-866): pairs (2i, 2i+1) of the first rotary_dim elements of every head row are rotated. */
int ckb200_dev_rope_precompute_cache(float *cos_cache, float *sin_cache, int max_seq_len, int head_dim, float base, int rotary_dim,
                                     int linear_scaling, float scaling_factor, void *stream);
int ckb200_dev_rope_forward_qk_pairwise(float *q, float *k, const float *cos_cache, const float *sin_cache, int num_heads,
                                        int num_kv_heads, int num_tokens, int head_dim, int aligned_head_dim, int pos_offset,
                                        int rotary_dim, const int *pos_dev, void *stream);
/* Glue of the batched prefill pass (the generated ck_prefill, version/v7/scripts/codegen_prefill_v7.py:194-208, does these per token):
 * rotate-half RoPE of token-major q [T][H*d] and k [T][Hkv*d] at positions pos0 + t, q scattered to head-major [H][T][d], k and v
 * rows written into the caches [Hkv][max_seq_len][d]; and the way back: head-major attention output [H][T][d] gathered to token
 * rows and quantised to Q8_K rows of `cols` elements (zero-padded). */
int ckb200_dev_prefill_rope_scatter(const float *q_tm, const float *k_tm, const float *v_tm, float *q_hm, float *k_cache, float *v_cache, const float *cos_cache,
                                    const float *sin_cache, int tokens, int num_heads, int num_kv_heads, int head_dim, int max_seq_len, int pos0, void *stream);
int ckb200_dev_prefill_gather_q8k(const float *out_hm, void *out_q8, int tokens, int num_heads, int head_dim, int cols, void *stream);
/* swiglu_forward (src/kernels/swiglu_kernels.c:140-216): input [T][2D] gate then up, output [T][D]. */
int ckb200_dev_swiglu_forward(const float *input, float *output, int tokens, int dim, void *stream);
/* ck_residual_add_token_major (src/ckernel_orchestration.c:139-149). */
int ckb200_dev_residual_add(const float *a, const float *b, float *out, int tokens, int aligned_embed_dim, void *stream);
/* embedding_forward_q4_k / _q6_k / _q8_0 (src/kernels/embedding_kernels.c:76-239); ids are device int32. */
int ckb200_dev_embedding_forward_q4_k(const int32_t *ids, int count, int vocab, const void *table, const float *pos_emb,
                                      float *out, int embed, int aligned, int ctx, int add_pos, void *stream);
int ckb200_dev_embedding_forward_q6_k(const int32_t *ids, int count, int vocab, const void *table, const float *pos_emb,
                                      float *out, int embed, int aligned, int ctx, int add_pos, void *stream);
int ckb200_dev_embedding_forward_q8_0(const int32_t *ids, int count, int vocab, const void *table, const float *pos_emb,
                                      float *out, int embed, int aligned, int ctx, int add_pos, void *stream);
/* The same lookup for a table whose rows are table_cols elements wide while the output rows are out_stride floats apart (a
 * block-32 table of a hidden size that is not a multiple of 256 feeding padded activation rows); fmt 0 Q4_K, 1 Q6_K, 2 Q8_0. */
int ckb200_dev_embedding_rows(const int32_t *ids, int count, int vocab, const void *table, int fmt, int table_cols, float *out, int out_stride,
                              int embed, void *stream);

/* ------------------------------------------------------------------ fused glue of a device-resident step
 * Each merges ops that the reference's generated decode function issues back to back
 * (version/v7/scripts/codegen_v7.py:569-931). */
/* The same fusion for consumers with 32-element blocks (Q8_0 / Q5_0 weights): x[t] += delta[t]; Q8_0 blocks (quantize_row_q8_0,
 * src/kernels/gemm_kernels_q8_0.c:70-175) of the first `cols` elements of rmsnorm(x[t]) * gamma, `cols` a multiple of 32. */
int ckb200_dev_add_rmsnorm_q8_0(float *x, const float *delta, const float *gamma, void *out_q80, int tokens, int d_model,
                                int aligned_embed_dim, int cols, float eps, void *stream);
/* x += delta (delta may be NULL); out_q8 = quantize_row_q8_k(rmsnorm_forward(x)); norm_out (optional) = fp32 rows */
int ckb200_dev_add_rmsnorm_q8k(float *x, const float *delta, const float *gamma, void *out_q8, float *norm_out, int tokens,
                               int d_model, int aligned_embed_dim, float eps, void *stream);
/* out_q8 = quantize_row_q8_k(swiglu_forward(gate_up)) */
int ckb200_dev_swiglu_q8k(const float *gate_up, void *out_q8, int tokens, int dim, void *stream);
/* rope_forward_qk on q and k of one token per sequence, then kv_cache_store at *pos_dev */
int ckb200_dev_rope_kv_store(float *q, const float *k, const float *v, float *k_cache, float *v_cache, const float *cos_cache,
                             const float *sin_cache, const int *pos_dev, int batch, int num_heads, int num_kv_heads,
                             int head_dim, int max_seq_len, long long kv_batch_stride, void *stream);
/* the same with IEEE fp16 caches (kv_cache_store_f16): rotation in fp32, one rounding on the store */
int ckb200_dev_rope_kv_store_f16(float *q, const float *k, const float *v, uint16_t *k_cache, uint16_t *v_cache, const float *cos_cache,
                                 const float *sin_cache, const int *pos_dev, int batch, int num_heads, int num_kv_heads,
                                 int head_dim, int max_seq_len, long long kv_batch_stride, void *stream);
int ckb200_dev_advance_pos(int *pos_dev, void *stream);                       /* model->pos++ on the device */
int ckb200_dev_add_inplace(float *x, const float *delta, long long n, void *stream);
/* synthetic data generated on the device (benchmarks of shapes too large to build on the host) */
int ckb200_dev_fill_blocks(void *w, long long nblocks, int fmt, unsigned long long seed, void *stream);
int ckb200_dev_fill_normal(float *x, long long n, int mode, unsigned long long seed, void *stream);
int ckb200_dev_fill_normal_f16(uint16_t *x, long long n, int mode, unsigned long long seed, void *stream);

#ifdef __cplusplus
}
#endif
#endif /* CKB200_H */
