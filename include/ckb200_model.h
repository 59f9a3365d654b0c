/*
 * ckb200_model.h - device-resident decode step executor.
 *
 * Runs the op list that the reference's generated ck_decode() issues (version/v7/scripts/codegen_v7.py:886-931;
 * layer template version/v7/templates/qwen2.json:95-110) for a Llama/Qwen-style decoder, with weights, KV
 * cache, activations and the position counter resident in HBM and the whole step captured in one CUDA
 * graph.  It is the device-side counterpart of the reference's ck_model_decode(token, logits)
 * (codegen_v7.py:1384-1390): one call = one token per sequence.
 *
 * Shapes come from a config struct instead of generated macros; tensors are uploaded one by one (or
 * filled with synthetic data on the device for benchmarks) in the reference's own block formats.
 */
#ifndef CKB200_MODEL_H
#define CKB200_MODEL_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* weight block formats (values of the fmt_* fields) */
enum { CKB_FMT_Q4_K = 0, CKB_FMT_Q6_K = 1, CKB_FMT_Q8_0 = 2, CKB_FMT_Q5_0 = 3 };   /* Q5_0: projections only (Q8_0 activations), not the down projection or the token embedding */

/* per-layer tensors; the same order as the reference's layer weight list (ln1, wq, wk, wv, wo, ln2, w1, w2) */
enum {
    CKB_T_LN1 = 0, CKB_T_WQ, CKB_T_WK, CKB_T_WV, CKB_T_WO, CKB_T_LN2, CKB_T_W1, CKB_T_W2, CKB_T_PER_LAYER,
    /* model-level tensors, addressed with layer = -1 */
    CKB_T_FINAL_GAMMA = 100, CKB_T_LM_HEAD = 101, CKB_T_EMBEDDING = 102
};

/* Mirrors CKModelConfig (include/ck_model_api.h:26-40) plus what the generated code has as macros. */
typedef struct {
    int embed_dim, num_heads, num_kv_heads, head_dim, intermediate_size, num_layers, vocab_size, max_seq_len;
    float rms_eps, rope_theta;
    int fmt_q, fmt_k, fmt_v, fmt_o, fmt_gate_up, fmt_down, fmt_lm_head, fmt_embedding;
    int tie_embeddings;      /* token embedding table = LM head matrix */
    int batch;               /* independent sequences advanced per step (all at the same position) */
    int tp_rank, tp_size;    /* tensor-parallel shard held by this process (tp_size <= 1: whole model) */
} CKB200ModelConfig;

typedef struct CKB200Model CKB200Model;

/* sum `count` floats in place over all tensor-parallel ranks, enqueued on `stream`; returns 0 on success */
typedef int (*ckb200_allreduce_fn)(void *ctx, float *buf, size_t count, void *stream);
/* Optional fused form of "all-reduce the residual delta, add it, RMSNorm, quantise to Q8_K" (one kernel per token row that
 * exchanges over peer memory).  Returns -1 when it does not handle the call; the step then uses the all-reduce hook. */
typedef int (*ckb200_tp_norm_fn)(void *ctx, float *x, const float *delta, const float *gamma, void *out_q8, int tokens, int d_model,
                                 int aligned_embed_dim, float eps, void *stream);

/* "synthetic:<qwen2-0.5b|llama3-8b|llama3-70b|mini>[:seed]" or the path of a BUMPWGT5 or CKB2MDL1 model file; batch <= 0 keeps the default */
CKB200Model *ckb200_model_open(const char *spec, int batch);
/* A BUMPWGT5 file of the reference's converter (include/ckernel_bump_v5.h) with its sidecar map (name|dtype|file_offset|size|
 * runtime_offset per line, version/v7/src/ckernel_model_load_v7.c:127-310); manifest_path NULL = weights_manifest.map beside the
 * file.  Both SHA-256 digests of the file are verified; what the step executor cannot run is refused with a message. */
CKB200Model *ckb200_model_open_bump(const char *bump_path, const char *manifest_path, int batch);
void ckb200_sha256(const void *data, size_t bytes, uint8_t out32[32]);
const CKB200ModelConfig *ckb200_model_config(CKB200Model *m);
int ckb200_model_reset(CKB200Model *m);                                  /* zero the KV cache, pos = 0 (ck_model_kv_cache_reset) */
CKB200Model *ckb200_model_create(const CKB200ModelConfig *cfg);          /* NULL on failure (see ckb200_last_error) */
void ckb200_model_free(CKB200Model *m);
size_t ckb200_model_tensor_bytes(CKB200Model *m, int layer, int which);
void *ckb200_model_tensor_ptr(CKB200Model *m, int layer, int which);     /* device pointer */
int ckb200_model_tensor_shape(CKB200Model *m, int layer, int which, int *rows, int *cols, int *fmt);
int ckb200_model_upload_tensor(CKB200Model *m, int layer, int which, const void *host, size_t bytes);
int ckb200_model_fill_synthetic(CKB200Model *m, unsigned long long seed);            /* random blocks, gamma = 1 + 0.1 N(0,1) */
int ckb200_model_fill_kv_synthetic(CKB200Model *m, int tokens, unsigned long long seed);   /* N(0,1) cache, pos = tokens */
int ckb200_model_set_pos(CKB200Model *m, int pos);
int ckb200_model_get_pos(CKB200Model *m);
void ckb200_model_set_allreduce(CKB200Model *m, ckb200_allreduce_fn fn, void *ctx);
void ckb200_model_set_tp_norm(CKB200Model *m, ckb200_tp_norm_fn fn, void *ctx);
/* one decode step: tokens[batch] in, logits[batch][vocab] out (logits_host may be NULL: no copy, no sync) */
int ckb200_model_decode(CKB200Model *m, const int32_t *tokens, float *logits_host);
/* A prompt of `count` tokens appended at the current position; logits_host (may be NULL) receives the last token's logits.
 * From an empty cache (position 0), with 16 tokens or more, one sequence on one GPU and K-quant projections this is ONE batched
 * pass - per layer: rows normalised and quantised together, every projection a tensor-core GEMM, RoPE + KV fill over all tokens,
 * causal prefill attention (the reference's generated ck_prefill, version/v7/scripts/codegen_prefill_v7.py:194-208) - otherwise
 * `count` decode steps.  Either way the cache and the position end as after `count` decode calls. */
int ckb200_model_prefill(CKB200Model *m, const int32_t *tokens, int count, float *logits_host);
int ckb200_model_decode_repeat(CKB200Model *m, int steps);              /* re-launch the captured step `steps` times */
float *ckb200_model_logits_device(CKB200Model *m);
void *ckb200_model_kv_device(CKB200Model *m, int layer, int is_v);       /* [batch][Hkv][max_seq][head_dim], fp32 unless ... */
int ckb200_model_kv_element_bytes(CKB200Model *m);                       /* ... 2: the model was created with tune model_kv_f16 = 1 (IEEE fp16
                                                                          * cache: kv_cache_store_f16 + the _f16cache decode attention,
                                                                          * src/kernels/kv_cache_kernels.c, attention_kernels.c:3450-3557) */
size_t ckb200_model_weight_bytes(CKB200Model *m);                        /* quantised bytes one step streams */


/* ---- tensor-parallel exchange (no counterpart in the reference, which has no collective): fp32 sum all-reduce over
 * NCCL, one process per GPU.  Rank 0 makes the 128-byte id, the caller distributes it, every rank calls tp_init. */
int ckb200_tp_unique_id(void *out128);
int ckb200_tp_init(int rank, int world, const void *id128);
int ckb200_tp_allreduce(void *ctx, float *buf, size_t count, void *stream);   /* a ckb200_allreduce_fn */
int ckb200_tp_rank(void);
int ckb200_tp_world(void);
void ckb200_tp_shutdown(void);
/* Optional latency path for small vectors: a one-shot push all-reduce over peer memory (CUDA IPC, NVLink stores).
 * Every rank calls create (max_floats a multiple of 4; writes its 64-byte handle), the caller gathers the handles
 * of ranks 0 .. world-1 in rank order, every rank calls connect.  ckb200_tp_allreduce then uses it for counts
 * <= max_floats (tune "tp_p2p" 0 switches it off); waits are bounded and report through the device error word. */
int ckb200_tp_p2p_create(int rank, int world, size_t max_floats, void *handle_out64);
int ckb200_tp_p2p_connect(const void *all_handles);
/* Single-GPU loopback for exercising the bounded wait: every peer pointer is this rank's own buffer, so the other ranks'
 * slots are never filled and each exchange runs into its limit (tune key "wait_limit_ms", default 10000), after which the
 * kernel returns, the device error word is set and the next synchronising call reports CKB_ERR_DEVICE_WAIT. */
int ckb200_tp_p2p_connect_self(void);
int ckb200_tp_p2p_ready(void);
size_t ckb200_tp_p2p_max_floats(void);
void ckb200_tp_p2p_shutdown(void);
int ckb200_tp_add_rmsnorm_q8k(void *ctx, float *x, const float *delta, const float *gamma, void *out_q8, int tokens, int d_model,
                              int aligned_embed_dim, float eps, void *stream);                  /* a ckb200_tp_norm_fn */
void ckb200_model_use_tp(CKB200Model *m);       /* set_allreduce(m, ckb200_tp_allreduce, NULL) and set_tp_norm(m, ckb200_tp_add_rmsnorm_q8k, NULL) */

#ifdef __cplusplus
}
#endif
#endif
