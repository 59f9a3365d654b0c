/*
 * ckb200_kernels.h - the reference's own kernel symbols, exported by libckb200.so with the
 * reference's signatures and HOST pointers.  A generated libmodel.so, the *_parallel_dispatch
 * seam or a ctypes test that links this library instead of libckernel_engine.so needs no source
 * change.  Each declaration cites the reference prototype or definition it replaces
 * (file:line inside C-Kernel-Engine).
 *
 * Behaviour kept from the reference: functions are void and return silently on NULL pointers or
 * non-positive sizes; nothing is retained between calls; the caller owns every buffer.
 * Added by the GPU: errors that cannot be expressed that way are readable through
 * ckb200_last_error() (ckb200.h).
 */
#ifndef CKB200_KERNELS_H
#define CKB200_KERNELS_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* ---- activation quantisers: include/ckernel_engine.h:269-293 (quantize_row_q8_0, quantize_batch_q8_0,
 *      quantize_row_q8_k, quantize_batch_q8_k); definitions src/kernels/gemm_kernels_q4k_q8k.c:53-119,
 *      src/kernels/gemm_kernels_q8_0.c:70-239 */
void quantize_row_q8_k(const float *x, void *y, int k);
void quantize_row_q8_k_ref(const float *x, void *y, int k);
void quantize_batch_q8_k(const float *x, void *y, int num_rows, int k);
void quantize_row_q8_0(const float *x, void *y, int k);
void quantize_batch_q8_0(const float *x, void *y, int num_rows, int k);

/* ---- Q4_K x Q8_K: include/ckernel_engine.h:295-337; src/kernels/gemm_kernels_q4k_q8k.c:183-326,
 *      ISA variants src/kernels/gemm_kernels_q4k_avx.c:38-245, gemm_kernels_q4k_sse.c:33,
 *      gemm_kernels_q4k_q8k_avx2.c:89-99, gemm_kernels_q4k_q8k_vnni.c:95-105 */
void gemv_q4_k_q8_k(float *y, const void *W, const void *x_q8, int M, int K);
void gemv_q4_k_q8_k_ref(float *y, const void *W, const void *x_q8, int M, int K);
void gemv_q4_k_q8_k_avx(float *y, const void *W, const void *x_q8, int M, int K);
void gemv_q4_k_q8_k_avx2(float *y, const void *W, const void *x_q8, int M, int K);
void gemv_q4_k_q8_k_vnni(float *y, const void *W, const void *x_q8, int M, int K);
void gemv_q4_k_q8_k_sse(float *y, const void *W, const void *x_q8, int M, int K);
void gemv_q4_k_q8_k_parallel(float *y, const void *W, const void *x_q8, int M, int K, int ith, int nth);
void gemv_q4_k_q8_k_parallel_simd(float *y, const void *W, const void *x_q8, int M, int K, int ith, int nth);
void gemm_q4_k_q8_k(float *Y, const void *W, const void *X_q8, int M, int N, int K);
void gemm_q4_k_q8_k_ref(float *Y, const void *W, const void *X_q8, int M, int N, int K);
void gemm_nt_q4_k_q8_k(const void *A_q8, const void *B, const float *bias, float *C, int M, int N, int K);

/* ---- Q6_K x Q8_K: include/ckernel_engine.h:335-358; src/kernels/gemm_kernels_q6k_q8k.c:197-214, :1032-1268 */
void vec_dot_q6_k_q8_k(int n, float *s, const void *vx, const void *vy);
void gemv_q6_k_q8_k(float *y, const void *W, const void *x_q8, int M, int K);
void gemv_q6_k_q8_k_ref(float *y, const void *W, const void *x_q8, int M, int K);
void gemv_q6_k_q8_k_parallel(float *y, const void *W, const void *x_q8, int M, int K, int ith, int nth);
void gemv_q6_k_q8_k_parallel_simd(float *y, const void *W, const void *x_q8, int M, int K, int ith, int nth);
void gemm_q6_k_q8_k(float *Y, const void *W, const void *X_q8, int M, int N, int K);
void gemm_nt_q6_k_q8_k(const void *A_q8, const void *B, const float *bias, float *C, int M, int N, int K);

/* ---- Q8_0: include/ckernel_engine.h:246-284, include/ckernel_quant.h:409; src/kernels/gemm_kernels_q8_0.c:254-277,
 *      :632-649, :1204-1343; src/kernels/gemm_batch_int8.c:87-120 */
void vec_dot_q8_0_q8_0(int n, float *s, const void *vx, const void *vy);
void gemv_q8_0_q8_0(float *y, const void *W, const void *x_q8, int M, int K);
void gemv_q8_0_q8_0_parallel(float *y, const void *W, const void *x_q8, int M, int K, int ith, int nth);
void gemv_q8_0_q8_0_parallel_simd(float *y, const void *W, const void *x_q8, int M, int K, int ith, int nth);
void gemm_nt_q8_0_q8_0(const void *A_q8, const void *B, const float *bias, float *C, int M, int N, int K);
void gemv_q8_0(float *y, const void *W, const float *x, int M, int K);
void gemv_q8_0_ref(float *y, const void *W, const float *x, int M, int K);

/* ---- fp32-activation debug path: include/ckernel_engine.h:192-225 */
void gemv_q4_k(float *y, const void *W, const float *x, int M, int K);
void gemv_q6_k(float *y, const void *W, const float *x, int M, int K);

/* ---- row dequantisers: include/ckernel_engine.h:208, :255, :262; src/kernels/dequant_kernels.c:288-430 */
void dequant_q4_k_row(const void *src, float *dst, size_t n_elements);
void dequant_q6_k_row(const void *src, float *dst, size_t n_elements);
void dequant_q8_0_row(const void *src, float *dst, size_t n_elements);

/* ---- thread-pool dispatch seam: version/v7/src/ck_parallel_decode.h:33-73, version/v7/src/ck_parallel_prefill.h:36-58.
 *      Generated code reaches these through the `#define gemv_q4_k_q8_k(...) gemv_q4_k_q8_k_parallel_dispatch(...)`
 *      overrides (ck_parallel_decode.h:112-123). */
void ck_parallel_decode_init(void);
void ck_parallel_decode_shutdown(void);
void ck_parallel_prefill_init(void);
void ck_parallel_prefill_shutdown(void);
void gemv_q4_k_q8_k_parallel_dispatch(float *y, const void *W, const void *x_q8, int M, int K);
void gemv_q6_k_q8_k_parallel_dispatch(float *y, const void *W, const void *x_q8, int M, int K);
void gemv_q8_0_q8_0_parallel_dispatch(float *y, const void *W, const void *x_q8, int M, int K);
void gemm_nt_q6_k_q8_k_parallel_dispatch(const void *A_q8, const void *B, const float *bias, float *C, int M, int N, int K);
void gemm_nt_q8_0_q8_0_parallel_dispatch(const void *A_q8, const void *B, const float *bias, float *C, int M, int N, int K);

/* ---- decode attention + KV cache: include/ckernel_engine.h:1635-1697; src/kernels/attention_kernels.c:3365-3406,
 *      src/kernels/attention_flash_true.c:696-722, src/kernels/kv_cache_kernels.c:70-129 */
void attention_forward_decode_head_major_gqa_flash(const float *q_token, const float *k_cache, const float *v_cache,
                                                   float *out_token, int num_heads, int num_kv_heads, int kv_tokens,
                                                   int cache_capacity, int head_dim, int aligned_head_dim);
/* Q5_0 x Q8_0: src/kernels/gemm_kernels_q5_0.c:901-939 (vec_dot), :1637-1720 (gemv), :1725-1752 (gemm_nt);
 *      version/v7/src/ck_parallel_decode.h (the _parallel_dispatch seam) */
void gemv_q5_0_q8_0(float *y, const void *W, const void *x_q8, int M, int K);
void gemv_q5_0_q8_0_parallel_simd(float *y, const void *W, const void *x_q8, int M, int K, int ith, int nth);
void gemv_q5_0_q8_0_parallel_dispatch(float *y, const void *W, const void *x_q8, int M, int K);
void vec_dot_q5_0_q8_0(int n, float *s, const void *vx, const void *vy);
void vec_dot_q5_0_q8_0_ref(int n, float *s, const void *vx, const void *vy);
void gemm_nt_q5_0_q8_0(const void *A_q8, const void *B, const float *bias, float *C, int M, int N, int K);
void gemv_q5_0(float *y, const void *W, const float *x, int M, int K);          /* fp32 activations: src/kernels/gemm_kernels_q5_0.c:550-567 */
void gemv_q5_0_ref(float *y, const void *W, const float *x, int M, int K);
void dequant_q5_0_row(const void *src, float *dst, size_t n_elements);          /* src/kernels/dequant_kernels.c:198-206 */
/* sliding-window attention: include/ckernel_engine.h:1259-1273, :1611-1623; src/kernels/attention_kernels_sliding.c:450-600 */
void attention_forward_causal_head_major_gqa_flash_strided_sliding(const float *q, const float *k, const float *v, float *output, int num_heads,
                                                                   int num_kv_heads, int num_tokens, int head_dim, int aligned_head_dim,
                                                                   int kv_stride_tokens, int sliding_window);
void attention_forward_decode_head_major_gqa_flash_sliding(const float *q_token, const float *k_cache, const float *v_cache, float *out_token,
                                                           int num_heads, int num_kv_heads, int kv_tokens, int cache_capacity, int head_dim,
                                                           int aligned_head_dim, int sliding_window);
/* fp16-rounded K/V with an fp16-rounded accumulator, key order kept (src/kernels/attention_kernels.c:3006-3046, :3408-3448) */
void attention_forward_decode_head_major_gqa_flash_f16kv(const float *q_token, const float *k_cache, const float *v_cache, float *out_token,
                                                         int num_heads, int num_kv_heads, int kv_tokens, int cache_capacity, int head_dim,
                                                         int aligned_head_dim);
void attention_forward_causal_head_major_gqa_flash_strided_f16kv(const float *q, const float *k, const float *v, float *output, int num_heads,
                                                                 int num_kv_heads, int num_tokens, int head_dim, int aligned_head_dim,
                                                                 int kv_stride_tokens);
/* fp16 KV cache: include/ckernel_engine.h:1232-1241, :1682-1690 */
void attention_forward_decode_head_major_gqa_flash_f16cache(const float *q_token, const uint16_t *k_cache, const uint16_t *v_cache,
                                                            float *out_token, int num_heads, int num_kv_heads, int kv_tokens,
                                                            int cache_capacity, int head_dim, int aligned_head_dim);
void kv_cache_store_f16(uint16_t *kv_cache_k, uint16_t *kv_cache_v, const float *k, const float *v, int layer, int pos,
                        int num_kv_heads, int head_dim, int max_seq_len);
/* prefill attention: include/ckernel_engine.h:1122-1165; src/kernels/attention_kernels.c:2924-3005 */
void attention_forward_causal_head_major_gqa_flash(const float *q, const float *k, const float *v, float *output, int num_heads,
                                                   int num_kv_heads, int num_tokens, int head_dim, int aligned_head_dim);
void attention_forward_causal_head_major_gqa_flash_strided(const float *q, const float *k, const float *v, float *output, int num_heads,
                                                           int num_kv_heads, int num_tokens, int head_dim, int aligned_head_dim,
                                                           int kv_stride_tokens);
void attention_forward_full_head_major_gqa_flash(const float *q, const float *k, const float *v, float *output, int num_heads,
                                                 int num_kv_heads, int num_tokens, int head_dim, int aligned_head_dim);
void attention_forward_full_head_major_gqa_flash_strided(const float *q, const float *k, const float *v, float *output, int num_heads,
                                                         int num_kv_heads, int num_tokens, int head_dim, int aligned_head_dim,
                                                         int kv_stride_tokens);
void attention_flash_decode(float *out, const float *q, const float *k, const float *v, int T_q, int T_k, int H, int D_h,
                            float scale);
void kv_cache_write_head_major(const float *k_token, const float *v_token, float *k_cache, float *v_cache, int num_kv_heads,
                               int token_index, int cache_capacity, int head_dim, int aligned_head_dim);
void kv_cache_store(float *kv_cache_k, float *kv_cache_v, const float *k, const float *v, int layer, int pos,
                    int num_kv_heads, int head_dim, int max_seq_len);

/* ---- the fp32 ops between the matmuls: src/kernels/rmsnorm_kernels.c:126-250, src/kernels/rope_kernels.c:221-243 and
 *      :806-819, src/kernels/swiglu_kernels.c:140-216, src/ckernel_orchestration.c:139-149,
 *      src/kernels/embedding_kernels.c:76-239 */
void rmsnorm_forward(const float *input, const float *gamma, float *output, float *rstd_cache, int tokens, int d_model,
                     int aligned_embed_dim, float eps);
void rope_precompute_cache_split(float *cos_cache, float *sin_cache, int max_seq_len, int head_dim, float base);
void rope_forward_qk(float *q, float *k, const float *cos_cache, const float *sin_cache, int num_heads, int num_kv_heads,
                     int num_tokens, int head_dim, int aligned_head_dim, int pos_offset);
void swiglu_forward(const float *input, float *output, int tokens, int dim);
void ck_residual_add_token_major(const float *a, const float *b, float *out, int tokens, int aligned_embed_dim);
void embedding_forward_q4_k(const int32_t *token_ids, int token_count, int vocab_size, const void *token_embeddings,
                            const float *pos_embeddings, float *output, int embed_dim, int aligned_embed_dim,
                            int context_window, int add_pos);
void embedding_forward_q6_k(const int32_t *token_ids, int token_count, int vocab_size, const void *token_embeddings,
                            const float *pos_embeddings, float *output, int embed_dim, int aligned_embed_dim,
                            int context_window, int add_pos);
void embedding_forward_q8_0(const int32_t *token_ids, int token_count, int vocab_size, const void *token_embeddings,
                            const float *pos_embeddings, float *output, int embed_dim, int aligned_embed_dim,
                            int context_window, int add_pos);

/* ---- fp32-activation GEMMs (the reference's debug path): one fp32-activation GEMV per token.
 *      gemm_nt_q4_k src/kernels/gemm_kernels_q4k.c:683-711, gemm_q4_k[_ref] :316-326, :461-469;
 *      gemm_nt_q6_k[_ref] src/kernels/gemm_kernels_q6k.c:212-250, gemm_q6_k :195-210; gemm_nt_q6_k_sse
 *      src/kernels/gemm_kernels_q6k_sse.c:66-97 (quantises A to Q8_K itself); gemm_nt_q8_0
 *      src/kernels/gemm_kernels_q8_0.c:683-696, gemm_q8_0 :658-666.  gemm_nt: A [M][K], B [N][K] blocks, C [M][N];
 *      gemm: Y [N][M], W [M][K] blocks, X [N][K]. */
void gemm_nt_q4_k(const float *A, const void *B, const float *bias, float *C, int M, int N, int K);
void gemm_q4_k(float *Y, const void *W, const float *X, int M, int N, int K);
void gemm_q4_k_ref(float *Y, const void *W, const float *X, int M, int N, int K);
void gemm_nt_q6_k(const float *A, const void *B, const float *bias, float *C, int M, int N, int K);
void gemm_nt_q6_k_ref(const float *A, const void *B, const float *bias, float *C, int M, int N, int K);
void gemm_nt_q6_k_sse(const float *A, const void *B, const float *bias, float *C, int M, int N, int K);
void gemm_q6_k(float *Y, const void *W, const float *X, int M, int N, int K);
void gemm_nt_q8_0(const float *A, const void *B, const float *bias, float *C, int M, int N, int K);
void gemm_q8_0(float *Y, const void *W, const float *X, int M, int N, int K);

/* ---- fp32 in, Q8_0 quantisation inside: src/kernels/gemm_kernels_q8_0_q8_0_contract.c:377-406, :408-486
 *      (rows of more than 1024 blocks take the fp32-activation GEMV, as there) */
void gemv_q8_0_q8_0_contract(float *y, const void *W, const float *x, int M, int K);
void gemm_nt_q8_0_q8_0_contract(const float *A, const void *B, const float *bias, float *C, int M, int N, int K);

/* ---- RoPE, general table and pairwise rotation: rope_precompute_cache src/kernels/rope_kernels.c:270-316 (rows of
 *      rotary_dim / 2 values; scaling_type "linear" divides the position by scaling_factor, anything else is ignored as in
 *      the reference), rope_forward_qk_pairwise_with_rotary_dim :839-866 (pairs (2i, 2i+1), the Llama form) */
void rope_precompute_cache(float *cos_cache, float *sin_cache, int max_seq_len, int head_dim, float base, int rotary_dim,
                           const char *scaling_type, float scaling_factor);
void rope_forward_qk_pairwise_with_rotary_dim(float *q, float *k, const float *cos_cache, const float *sin_cache, int num_heads,
                                              int num_kv_heads, int num_tokens, int head_dim, int aligned_head_dim, int pos_offset,
                                              int rotary_dim);
void rope_forward_qk_with_rotary_dim(float *q, float *k, const float *cos_cache, const float *sin_cache, int num_heads, int num_kv_heads,
                                     int num_tokens, int head_dim, int aligned_head_dim, int pos_offset, int rotary_dim);    /* rope_kernels.c:821-837 */

/* ---- small copies: add_inplace_f32 include/ckernel_engine.h:1894 (src/kernels/add_kernels_bf16.c:304-330),
 *      logits_copy_to_position src/kernels/kv_cache_kernels.c:178-191 */
void add_inplace_f32(float *a, const float *b, size_t n);
void logits_copy_to_position(const float *src, float *dst, int position, int vocab_size);

/* ---- the reference's flat parity API (include/ck_parity_api.h, src/ck_parity_api.c:189-694): what its kernel-parity
 *      scripts bind.  Each quantises the fp32 input as the reference wrapper does and runs the quantised kernel. */
void ck_test_dequant_q4_k(const void *src, float *dst, int n);
void ck_test_dequant_q6_k(const void *src, float *dst, int n);
void ck_test_quantize_q8_k(const float *src, void *dst, int n);
void ck_test_gemv_q4_k(const void *weight_q4k, const float *input_f32, float *output, int cols);
void ck_test_gemv_q6_k(const void *weight_q6k, const float *input_f32, float *output, int cols);
void ck_test_gemv_q5_0(const void *weight_q5_0, const float *input_f32, float *output, int rows, int cols);
void ck_test_gemv_q8_0(const void *weight_q8_0, const float *input_f32, float *output, int rows, int cols);
void ck_test_gemv_q5_0_q8_0(const void *weight_q5_0, const float *input_f32, float *output, int rows, int cols);
void ck_test_gemv_q8_0_q8_0(const void *weight_q8_0, const float *input_f32, float *output, int rows, int cols);
void ck_test_vec_dot_q5_0_q8_0(const void *weight_q5_0, const void *input_q8_0, float *output, int cols);
void ck_test_vec_dot_q8_0_q8_0(const void *weight_q8_0, const void *input_q8_0, float *output, int cols);
void ck_test_gemm_q4_k(const void *weight_q4k, const float *input_f32, float *output, int rows, int cols, int n_tokens);
void ck_test_gemm_q6_k(const void *weight_q6k, const float *input_f32, float *output, int rows, int cols, int n_tokens);
void ck_test_gemm_q8_0(const void *weight_q8_0, const float *input_f32, float *output, int rows, int cols, int n_tokens);
void ck_test_gemm_q5_0(const void *weight_q5_0, const float *input_f32, float *output, int rows, int cols, int n_tokens);
void ck_test_rmsnorm(const float *input, const float *weight, float *output, int n_tokens, int dim, float eps);
void ck_test_rope(float *q, float *k, int n_tokens, int n_heads, int n_heads_kv, int head_dim, int pos_offset, float theta);
void ck_test_rope_interleaved(float *q, float *k, int n_tokens, int n_heads, int n_heads_kv, int head_dim, int pos_offset, float theta);   /* :630-687 */
void ck_test_dequant_q4_0(const void *src, float *dst, int n);                                                                                /* :199-202 */
void ck_test_attention_causal(const float *q, const float *k, const float *v, float *out, int num_heads, int num_kv_heads, int tokens,
                              int seq_len, int head_dim);                                                                                    /* :861-881 */
void ck_test_swiglu(const float *gate_up, float *output, int n_tokens, int intermediate_dim);

/* ---- further weight formats: Q5_K (src/kernels/gemm_kernels_q5_k.c:305-520), Q5_1 x Q8_1 (src/kernels/gemm_kernels_q5_1_q8_1.c:75-175),
 *      Q4_0 / Q4_1 / Q5_1 with fp32 activations (src/kernels/gemm_kernels_q4_0.c, gemm_kernels_q4_1.c, gemm_kernels_q5_1.c, dequant_kernels.c) ---- */
void gemv_q5_k_q8_k(float *y, const void *W, const void *x_q8, int M, int K);
void gemv_q5_k_q8_k_ref(float *y, const void *W, const void *x_q8, int M, int K);
void gemm_nt_q5_k_q8_k(const void *A_q8, const void *B, const float *bias, float *C, int M, int N, int K);
void gemm_nt_q5_k_q8_k_ref(const void *A_q8, const void *B, const float *bias, float *C, int M, int N, int K);
void gemv_q5_k(float *y, const void *W, const float *x, int M, int K);
void gemv_q5_k_ref(float *y, const void *W, const float *x, int M, int K);
void gemm_nt_q5_k(const float *A, const void *B, const float *bias, float *C, int M, int N, int K);
void gemm_nt_q5_k_ref(const float *A, const void *B, const float *bias, float *C, int M, int N, int K);
void gemv_q5_1_q8_1(float *y, const void *W, const float *x, int M, int K);
void gemv_q5_1_q8_1_ref(float *y, const void *W, const void *x_q8, int M, int K);
void gemm_nt_q5_1_q8_1(const float *A, const void *B, const float *bias, float *C, int M, int N, int K);
void gemm_nt_q5_1_q8_1_ref(const void *A_q8, const void *B, const float *bias, float *C, int M, int N, int K);
void gemv_q4_0(float *y, const void *W, const float *x, int M, int K);
void gemv_q4_0_ref(float *y, const void *W, const float *x, int M, int K);
void gemm_q4_0(float *Y, const void *W, const float *X, int M, int N, int K);
void gemm_nt_q4_0(const float *A, const void *B, const float *bias, float *C, int M, int N, int K);
float dot_q4_0(const void *w, const float *x, int K);
void dequant_q4_0_row(const void *src, float *dst, size_t n_elements);
void gemv_q4_1(float *y, const void *W, const float *x, int M, int K);
void gemv_q4_1_ref(float *y, const void *W, const float *x, int M, int K);
void gemm_q4_1(float *Y, const void *W, const float *X, int M, int N, int K);
void gemm_nt_q4_1(const float *A, const void *B, const float *bias, float *C, int M, int N, int K);
float dot_q4_1(const void *w, const float *x, int K);
void dequant_q4_1_row(const void *src, float *dst, size_t n_elements);
void gemv_q5_1(float *y, const void *W, const float *x, int M, int K);
void gemv_q5_1_ref(float *y, const void *W, const float *x, int M, int K);
void gemm_q5_1(float *Y, const void *W, const float *X, int M, int N, int K);
void gemm_nt_q5_1(const float *A, const void *B, const float *bias, float *C, int M, int N, int K);
float dot_q5_1(const void *w, const float *x, int K);
void dequant_q5_1_row(const void *src, float *dst, size_t n_elements);

#ifdef __cplusplus
}
#endif
#endif /* CKB200_KERNELS_H */
