/* Decode-step executor driven by the reference's lowered call IR.
 *
 * The v7 pipeline lowers a model to "lowered-ir-v3" (version/v7/scripts/build_ir_v7.py:6414-6876, generate_ir_lower_3): a list of
 * operations, each a C function symbol plus arguments that say where every value comes from (`source`: weight:, weight_f:,
 * activation:, output:, scratch:, dim:, const:, runtime:, null) and which buffer or weight it names (`buffer_ref`, `weight_ref`),
 * together with the memory plan (`memory.weights.entries`, `memory.activations.buffers`).  The reference turns that list into C
 * (version/v7/scripts/codegen_v7.py:569-931) and compiles a libmodel.so per model.  Here the same list is replayed on the device:
 * every op is bound once to the ckb200_dev_* kernel behind its symbol, the whole step is captured in one CUDA graph, and a token
 * is one graph launch.  A model the pipeline lowers differently (pair-rotated or half-rotated RoPE, the fp16-rounded attention of
 * the llama template, Q5_0 / Q8_0 projections with Q8_0 activations, a sliding window) runs without new code here as long as its
 * symbols are in the table below; an op whose symbol is not refuses the file with a message naming it.
 *
 * Memory: the plan's runtime offsets describe the generated CPU model's arena, where activation buffers are only 4-byte aligned.
 * The kernels here want 16-byte alignment, so every weight and every activation buffer of the plan gets its own 256-byte-aligned
 * place in one device arena (by name, with the plan's sizes); the offsets are not used.  Weights come from the BUMPWGT5 file
 * through the sidecar map (bump_loader.c).  Q6_K / Q8_0 / Q5_0 matrices that a GEMV op reads get a row-planar copy.
 * Values the generated code reads from the model struct become device state: model->pos is an int in device memory (kernels take
 * it as pos_dev, so the captured graph is position-independent), model->kv_cache is the plan's kv_cache buffer
 * ([layer][k|v][Hkv][max_seq][head_dim]), model->rope_cos / rope_sin are the two halves of the plan's rope_cache buffer, filled
 * at open by rope_precompute_cache with the config's theta / rotary_dim / scaling. */
#include <math.h>
#include <stdint.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#include <cuda_runtime.h>

#include "../../include/ckb200.h"
#include "../../include/ckb200_ir.h"
#include "bump_file.h"
#include "json_mini.h"
#include "launch.h"
#include "runtime.h"

enum {
    OP_EMBED_Q4K, OP_EMBED_Q6K, OP_EMBED_Q80, OP_MEMCPY, OP_RMSNORM, OP_QUANT_Q8K, OP_QUANT_Q80,
    OP_GEMV_Q4K_Q8K, OP_GEMV_Q6K_Q8K, OP_GEMV_Q80_Q80, OP_GEMV_Q50_Q80, OP_GEMV_Q5K_Q8K, OP_GEMV_Q4K_F32, OP_GEMV_Q6K_F32, OP_GEMV_Q80_F32, OP_GEMV_Q50_F32,
    OP_ROPE_HALF, OP_ROPE_PAIR, OP_KV_STORE, OP_ATTN, OP_ATTN_F16KV, OP_ATTN_SLIDING, OP_RESIDUAL_ADD, OP_SWIGLU, OP_ADD_INPLACE
};

static const struct { const char *symbol; int op; } g_symbols[] = {
    { "embedding_forward_q4_k", OP_EMBED_Q4K }, { "embedding_forward_q6_k", OP_EMBED_Q6K }, { "embedding_forward_q8_0", OP_EMBED_Q80 },
    { "memcpy", OP_MEMCPY }, { "rmsnorm_forward", OP_RMSNORM }, { "quantize_row_q8_k", OP_QUANT_Q8K }, { "quantize_row_q8_0", OP_QUANT_Q80 },
    { "gemv_q4_k_q8_k", OP_GEMV_Q4K_Q8K }, { "gemv_q6_k_q8_k", OP_GEMV_Q6K_Q8K }, { "gemv_q8_0_q8_0", OP_GEMV_Q80_Q80 }, { "gemv_q5_0_q8_0", OP_GEMV_Q50_Q80 },
    { "gemv_q5_k_q8_k", OP_GEMV_Q5K_Q8K },
    { "gemv_q4_k", OP_GEMV_Q4K_F32 }, { "gemv_q6_k", OP_GEMV_Q6K_F32 }, { "gemv_q8_0", OP_GEMV_Q80_F32 }, { "gemv_q5_0", OP_GEMV_Q50_F32 },
    { "rope_forward_qk_with_rotary_dim", OP_ROPE_HALF }, { "rope_forward_qk", OP_ROPE_HALF }, { "rope_forward_qk_pairwise_with_rotary_dim", OP_ROPE_PAIR },
    { "kv_cache_store", OP_KV_STORE }, { "attention_forward_decode_head_major_gqa_flash", OP_ATTN },
    { "attention_forward_decode_head_major_gqa_flash_f16kv", OP_ATTN_F16KV }, { "attention_forward_decode_head_major_gqa_flash_sliding", OP_ATTN_SLIDING },
    { "ck_residual_add_token_major", OP_RESIDUAL_ADD }, { "swiglu_forward", OP_SWIGLU }, { "add_inplace_f32", OP_ADD_INPLACE },
};

#define IR_MAX_ARGS 12

typedef struct {
    int op;
    char symbol[64];
    char opname[40];            /* the IR's op label (q_proj, mlp_gate_up, ...) and layer, for the per-op timing report */
    int layer;
    void *p[IR_MAX_ARGS];       /* pointer arguments in the order of the reference's signature; NULL for null / runtime scalars */
    long long i[IR_MAX_ARGS];   /* integer arguments */
    float f[IR_MAX_ARGS];
} IrOp;

typedef struct { char name[64]; uint8_t *ptr; size_t bytes; } IrBuffer;
typedef struct { char name[96]; char dtype[16]; uint8_t *ptr, *planar; size_t bytes; } IrWeight;

struct CKB200IrModel {
    IrOp *ops;
    int nops;
    IrBuffer *buf;
    int nbuf;
    IrWeight *w;
    int nw;
    uint8_t *arena;
    size_t arena_bytes;
    int *pos_dev;
    int32_t *token_pinned;
    float *rope_cos, *rope_sin, *kv_cache, *logits;
    int32_t *token_ids;
    int vocab, max_seq, layers, kv_heads, head_dim, heads;
    int host_pos;
    float *attn_scratch;
    int attn_splits;
    cudaGraphExec_t graph;
    cudaEvent_t ev_token;
    int token_in_flight;
    int launches;
    cudaEvent_t *prof_ev;        /* nops + 1 events, created on the first profiled step */
    int prof_token;
};

static size_t align_up(size_t v, size_t a) { return (v + a - 1) / a * a; }

static IrBuffer *find_buffer(CKB200IrModel *m, const char *name)
{
    for (int i = 0; i < m->nbuf; ++i) if (!strcmp(m->buf[i].name, name)) return &m->buf[i];
    return NULL;
}

static IrWeight *find_weight(CKB200IrModel *m, const char *name)
{
    for (int i = 0; i < m->nw; ++i) if (!strcmp(m->w[i].name, name)) return &m->w[i];
    return NULL;
}

/* ---------------------------------------------------------------- argument binding */

typedef struct { CKB200IrModel *m; const JsonValue *op; const char *symbol; int layer; int failed; } Binder;

static const JsonValue *arg_named(Binder *b, const char *name)
{
    const JsonValue *args = json_get(b->op, "args");
    for (int i = 0; i < json_len(args); ++i) {
        const JsonValue *a = json_at(args, i);
        if (!strcmp(json_str(json_get(a, "name"), ""), name)) return a;
    }
    if (!b->failed) ckb_fail(CKB_ERR_STATE, "ir: op %s (idx %d) has no argument '%s'", b->symbol, (int)json_num(json_get(b->op, "idx"), -1), name);
    b->failed = 1;
    return NULL;
}

/* a pointer argument: buffer, weight, rope table, a layer's K or V cache, or null */
static void *arg_ptr(Binder *b, const char *name, IrWeight **weight_out)
{
    const JsonValue *a = arg_named(b, name);
    if (!a) return NULL;
    const char *src = json_str(json_get(a, "source"), "");
    CKB200IrModel *m = b->m;
    if (weight_out) *weight_out = NULL;
    if (!strcmp(src, "null")) return NULL;
    const char *wref = json_str(json_get(a, "weight_ref"), NULL), *bref = json_str(json_get(a, "buffer_ref"), NULL);
    if (wref) {
        IrWeight *w = find_weight(m, wref);
        if (w) { if (weight_out) *weight_out = w; return w->ptr; }
        if (!b->failed) ckb_fail(CKB_ERR_STATE, "ir: op %s reads weight '%s', which is not in the memory plan", b->symbol, wref);
        b->failed = 1;
        return NULL;
    }
    if (bref) {
        IrBuffer *bf = find_buffer(m, bref);
        if (bf) return bf->ptr;
        if (!b->failed) ckb_fail(CKB_ERR_STATE, "ir: op %s uses buffer '%s', which is not in the memory plan", b->symbol, bref);
        b->failed = 1;
        return NULL;
    }
    if (!strcmp(src, "runtime:rope_cos")) return m->rope_cos;
    if (!strcmp(src, "runtime:rope_sin")) return m->rope_sin;
    if (!strcmp(src, "runtime:kv_cache_k_layer") || !strcmp(src, "runtime:kv_cache_v_layer")) {
        if (b->layer < 0 || b->layer >= m->layers || !m->kv_cache) {
            if (!b->failed) ckb_fail(CKB_ERR_STATE, "ir: op %s asks for the cache of layer %d (model has %d)", b->symbol, b->layer, m->layers);
            b->failed = 1;
            return NULL;
        }
        const size_t per = (size_t)m->kv_heads * m->max_seq * m->head_dim;
        return m->kv_cache + ((size_t)b->layer * 2 + (src[17] == 'v')) * per;
    }
    if (!b->failed) ckb_fail(CKB_ERR_STATE, "ir: op %s, argument '%s': source '%s' is not a pointer this executor knows", b->symbol, name, src);
    b->failed = 1;
    return NULL;
}

/* a scalar: dim: / const: carry a literal in expr; runtime:pos / runtime:kv_tokens / runtime:layer are bound on the device */
static double arg_num(Binder *b, const char *name)
{
    const JsonValue *a = arg_named(b, name);
    if (!a) return 0;
    const char *src = json_str(json_get(a, "source"), ""), *expr = json_str(json_get(a, "expr"), "");
    if (!strncmp(src, "runtime:", 8)) return !strcmp(src, "runtime:layer") ? b->layer : 0;     /* pos and kv_tokens come from pos_dev */
    char *end = NULL;
    const double v = strtod(expr, &end);
    if (end == expr) {
        if (!b->failed) ckb_fail(CKB_ERR_STATE, "ir: op %s, argument '%s': '%s' is not a literal", b->symbol, name, expr);
        b->failed = 1;
    }
    return v;
}

static int bind_op(CKB200IrModel *m, const JsonValue *jop, IrOp *o)
{
    const char *symbol = json_str(json_get(jop, "function"), "");
    Binder b = { m, jop, symbol, (int)json_num(json_get(jop, "layer"), -1), 0 };
    memset(o, 0, sizeof *o);
    snprintf(o->symbol, sizeof o->symbol, "%s", symbol);
    snprintf(o->opname, sizeof o->opname, "%s", json_str(json_get(jop, "op"), ""));
    o->layer = b.layer;
    o->op = -1;
    for (size_t i = 0; i < sizeof g_symbols / sizeof g_symbols[0]; ++i) if (!strcmp(g_symbols[i].symbol, symbol)) o->op = g_symbols[i].op;
    if (o->op < 0) return ckb_fail(CKB_ERR_STATE, "ir: op %d calls '%s', which this executor has no kernel for", (int)json_num(json_get(jop, "idx"), -1), symbol);
    IrWeight *w = NULL;
    switch (o->op) {
    case OP_EMBED_Q4K: case OP_EMBED_Q6K: case OP_EMBED_Q80:
        o->p[0] = arg_ptr(&b, "token_ids", NULL); o->i[0] = (long long)arg_num(&b, "token_count"); o->i[1] = (long long)arg_num(&b, "vocab_size");
        o->p[1] = arg_ptr(&b, "token_embeddings", NULL); o->p[2] = arg_ptr(&b, "pos_embeddings", NULL); o->p[3] = arg_ptr(&b, "output", NULL);
        o->i[2] = (long long)arg_num(&b, "embed_dim"); o->i[3] = (long long)arg_num(&b, "aligned_embed_dim"); o->i[4] = (long long)arg_num(&b, "context_window");
        o->i[5] = (long long)arg_num(&b, "add_pos");
        break;
    case OP_MEMCPY:
        o->p[0] = arg_ptr(&b, "dst", NULL); o->p[1] = arg_ptr(&b, "src", NULL); o->i[0] = (long long)arg_num(&b, "size");
        break;
    case OP_RMSNORM:
        o->p[0] = arg_ptr(&b, "input", NULL); o->p[1] = arg_ptr(&b, "gamma", NULL); o->p[2] = arg_ptr(&b, "output", NULL); o->p[3] = arg_ptr(&b, "rstd_cache", NULL);
        o->i[0] = (long long)arg_num(&b, "tokens"); o->i[1] = (long long)arg_num(&b, "d_model"); o->i[2] = (long long)arg_num(&b, "aligned_embed_dim");
        o->f[0] = (float)arg_num(&b, "eps");
        break;
    case OP_QUANT_Q8K: case OP_QUANT_Q80:
        o->p[0] = arg_ptr(&b, "x", NULL); o->p[1] = arg_ptr(&b, "y", NULL); o->i[0] = (long long)arg_num(&b, "k");
        break;
    case OP_GEMV_Q4K_Q8K: case OP_GEMV_Q6K_Q8K: case OP_GEMV_Q80_Q80: case OP_GEMV_Q50_Q80: case OP_GEMV_Q5K_Q8K:
        o->p[0] = arg_ptr(&b, "y", NULL); o->p[1] = arg_ptr(&b, "W", &w); o->p[2] = arg_ptr(&b, "x_q8", NULL);
        o->i[0] = (long long)arg_num(&b, "M"); o->i[1] = (long long)arg_num(&b, "K");
        o->p[3] = w;                                         /* resolved to the planar copy after all ops are bound */
        break;
    case OP_GEMV_Q4K_F32: case OP_GEMV_Q6K_F32: case OP_GEMV_Q80_F32: case OP_GEMV_Q50_F32:
        o->p[0] = arg_ptr(&b, "y", NULL); o->p[1] = arg_ptr(&b, "W", NULL); o->p[2] = arg_ptr(&b, "x", NULL);
        o->i[0] = (long long)arg_num(&b, "M"); o->i[1] = (long long)arg_num(&b, "K");
        break;
    case OP_ROPE_HALF: case OP_ROPE_PAIR:
        o->p[0] = arg_ptr(&b, "q", NULL); o->p[1] = arg_ptr(&b, "k", NULL); o->p[2] = arg_ptr(&b, "cos_cache", NULL); o->p[3] = arg_ptr(&b, "sin_cache", NULL);
        o->i[0] = (long long)arg_num(&b, "num_heads"); o->i[1] = (long long)arg_num(&b, "num_kv_heads"); o->i[2] = (long long)arg_num(&b, "num_tokens");
        o->i[3] = (long long)arg_num(&b, "head_dim"); o->i[4] = (long long)arg_num(&b, "aligned_head_dim");
        o->i[5] = strcmp(symbol, "rope_forward_qk") ? (long long)arg_num(&b, "rotary_dim") : o->i[3];
        break;
    case OP_KV_STORE:
        o->p[0] = arg_ptr(&b, "kv_cache_k", NULL); o->p[1] = arg_ptr(&b, "kv_cache_v", NULL); o->p[2] = arg_ptr(&b, "k", NULL); o->p[3] = arg_ptr(&b, "v", NULL);
        o->i[0] = (long long)arg_num(&b, "num_kv_heads"); o->i[1] = (long long)arg_num(&b, "head_dim"); o->i[2] = (long long)arg_num(&b, "max_seq_len");
        break;
    case OP_ATTN: case OP_ATTN_F16KV: case OP_ATTN_SLIDING:
        o->p[0] = arg_ptr(&b, "q_token", NULL); o->p[1] = arg_ptr(&b, "k_cache", NULL); o->p[2] = arg_ptr(&b, "v_cache", NULL); o->p[3] = arg_ptr(&b, "out_token", NULL);
        o->i[0] = (long long)arg_num(&b, "num_heads"); o->i[1] = (long long)arg_num(&b, "num_kv_heads"); o->i[2] = (long long)arg_num(&b, "cache_capacity");
        o->i[3] = (long long)arg_num(&b, "head_dim"); o->i[4] = (long long)arg_num(&b, "aligned_head_dim");
        if (o->op == OP_ATTN_SLIDING && !b.failed)
            return ckb_fail(CKB_ERR_STATE, "ir: %s needs the context length on the host; the captured step has it only on the device", symbol);
        break;
    case OP_RESIDUAL_ADD:
        o->p[0] = arg_ptr(&b, "a", NULL); o->p[1] = arg_ptr(&b, "b", NULL); o->p[2] = arg_ptr(&b, "out", NULL);
        o->i[0] = (long long)arg_num(&b, "tokens"); o->i[1] = (long long)arg_num(&b, "aligned_embed_dim");
        break;
    case OP_SWIGLU:
        o->p[0] = arg_ptr(&b, "input", NULL); o->p[1] = arg_ptr(&b, "output", NULL); o->i[0] = (long long)arg_num(&b, "tokens"); o->i[1] = (long long)arg_num(&b, "dim");
        break;
    case OP_ADD_INPLACE:
        o->p[0] = arg_ptr(&b, "a", NULL); o->p[1] = arg_ptr(&b, "b", NULL); o->i[0] = (long long)arg_num(&b, "n");
        break;
    }
    return b.failed ? CKB_ERR_STATE : 0;
}

/* ---------------------------------------------------------------- one op -> one (or a few) launches */

static int run_op(CKB200IrModel *m, const IrOp *o, void *st)
{
    switch (o->op) {
    case OP_EMBED_Q4K: return ckb200_dev_embedding_forward_q4_k((const int32_t *)o->p[0], (int)o->i[0], (int)o->i[1], o->p[1], (const float *)o->p[2], (float *)o->p[3], (int)o->i[2], (int)o->i[3], (int)o->i[4], (int)o->i[5], st);
    case OP_EMBED_Q6K: return ckb200_dev_embedding_forward_q6_k((const int32_t *)o->p[0], (int)o->i[0], (int)o->i[1], o->p[1], (const float *)o->p[2], (float *)o->p[3], (int)o->i[2], (int)o->i[3], (int)o->i[4], (int)o->i[5], st);
    case OP_EMBED_Q80: return ckb200_dev_embedding_forward_q8_0((const int32_t *)o->p[0], (int)o->i[0], (int)o->i[1], o->p[1], (const float *)o->p[2], (float *)o->p[3], (int)o->i[2], (int)o->i[3], (int)o->i[4], (int)o->i[5], st);
    case OP_MEMCPY: return ckb_check_cuda((int)cudaMemcpyAsync(o->p[0], o->p[1], (size_t)o->i[0], cudaMemcpyDeviceToDevice, (cudaStream_t)st), "ir memcpy") ? CKB_ERR_CUDA : 0;
    case OP_RMSNORM: return ckb200_dev_rmsnorm_forward((const float *)o->p[0], (const float *)o->p[1], (float *)o->p[2], (float *)o->p[3], (int)o->i[0], (int)o->i[1], (int)o->i[2], o->f[0], st);
    case OP_QUANT_Q8K: return ckb200_dev_quantize_q8_k((const float *)o->p[0], o->p[1], 1, (int)o->i[0], st);
    case OP_QUANT_Q80: return ckb200_dev_quantize_q8_0((const float *)o->p[0], o->p[1], 1, (int)o->i[0], st);
    case OP_GEMV_Q4K_Q8K: return ckb200_dev_gemv_q4_k_q8_k((float *)o->p[0], o->p[1], o->p[2], (int)o->i[0], (int)o->i[1], st);
    case OP_GEMV_Q6K_Q8K:
        return o->p[3] ? ckb200_dev_gemv_q6_k_planar_q8_k((float *)o->p[0], o->p[3], o->p[2], (int)o->i[0], (int)o->i[1], st)
                       : ckb200_dev_gemv_q6_k_q8_k((float *)o->p[0], o->p[1], o->p[2], (int)o->i[0], (int)o->i[1], st);
    case OP_GEMV_Q80_Q80:
        return o->p[3] ? ckb200_dev_gemv_q8_0_planar_q8_0((float *)o->p[0], o->p[3], o->p[2], (int)o->i[0], (int)o->i[1], st)
                       : ckb200_dev_gemv_q8_0_q8_0((float *)o->p[0], o->p[1], o->p[2], (int)o->i[0], (int)o->i[1], st);
    case OP_GEMV_Q50_Q80:
        return o->p[3] ? ckb200_dev_gemv_q5_0_planar_q8_0((float *)o->p[0], o->p[3], o->p[2], (int)o->i[0], (int)o->i[1], st)
                       : ckb200_dev_gemv_q5_0_q8_0((float *)o->p[0], o->p[1], o->p[2], (int)o->i[0], (int)o->i[1], st);
    case OP_GEMV_Q5K_Q8K: return ckb200_dev_gemv_q5_k_q8_k((float *)o->p[0], o->p[1], o->p[2], (int)o->i[0], (int)o->i[1], st);
    case OP_GEMV_Q4K_F32: return ckb200_dev_gemv_q4_k((float *)o->p[0], o->p[1], (const float *)o->p[2], (int)o->i[0], (int)o->i[1], st);
    case OP_GEMV_Q6K_F32: return ckb200_dev_gemv_q6_k((float *)o->p[0], o->p[1], (const float *)o->p[2], (int)o->i[0], (int)o->i[1], st);
    case OP_GEMV_Q80_F32: return ckb200_dev_gemv_q8_0((float *)o->p[0], o->p[1], (const float *)o->p[2], (int)o->i[0], (int)o->i[1], st);
    case OP_GEMV_Q50_F32: return ckb200_dev_gemv_q5_0((float *)o->p[0], o->p[1], (const float *)o->p[2], (int)o->i[0], (int)o->i[1], st);
    case OP_ROPE_HALF:
        return ckb200_dev_rope_forward_qk_with_rotary_dim((float *)o->p[0], (float *)o->p[1], (const float *)o->p[2], (const float *)o->p[3], (int)o->i[0], (int)o->i[1],
                                                          (int)o->i[2], (int)o->i[3], (int)o->i[4], 0, (int)o->i[5], m->pos_dev, st);
    case OP_ROPE_PAIR:
        return ckb200_dev_rope_forward_qk_pairwise((float *)o->p[0], (float *)o->p[1], (const float *)o->p[2], (const float *)o->p[3], (int)o->i[0], (int)o->i[1], (int)o->i[2],
                                                   (int)o->i[3], (int)o->i[4], 0, (int)o->i[5], m->pos_dev, st);
    case OP_KV_STORE:
        return ckb200_dev_kv_cache_store((float *)o->p[0], (float *)o->p[1], (const float *)o->p[2], (const float *)o->p[3], 0, m->pos_dev, (int)o->i[0], (int)o->i[1], (int)o->i[2], st);
    case OP_ATTN:
        return ckb200_dev_attention_decode_ws((const float *)o->p[0], (const float *)o->p[1], (const float *)o->p[2], (float *)o->p[3], 1, 0, (int)o->i[0], (int)o->i[1], 1, (int)o->i[2],
                                              (int)o->i[3], (int)o->i[4], m->attn_splits, m->attn_scratch, m->pos_dev, st);
    case OP_ATTN_F16KV:
        return ckb200_dev_attention_decode_f16kv((const float *)o->p[0], (const float *)o->p[1], (const float *)o->p[2], (float *)o->p[3], (int)o->i[0], (int)o->i[1], 1, (int)o->i[2],
                                                 (int)o->i[3], (int)o->i[4], m->pos_dev, st);
    case OP_ATTN_SLIDING: break;                             /* refused at open */
    case OP_RESIDUAL_ADD: return ckb200_dev_residual_add((const float *)o->p[0], (const float *)o->p[1], (float *)o->p[2], (int)o->i[0], (int)o->i[1], st);
    case OP_SWIGLU: return ckb200_dev_swiglu_forward((const float *)o->p[0], (float *)o->p[1], (int)o->i[0], (int)o->i[1], st);
    case OP_ADD_INPLACE: return ckb200_dev_add_inplace((float *)o->p[0], (const float *)o->p[1], o->i[0], st);
    }
    return CKB_ERR_STATE;
}

static int issue_all(CKB200IrModel *m, void *st)
{
    for (int i = 0; i < m->nops; ++i) {
        const int rc = run_op(m, &m->ops[i], st);
        if (rc) return rc;
    }
    return ckb200_dev_advance_pos(m->pos_dev, st);
}

/* ---------------------------------------------------------------- open */

void ckb200_ir_free(CKB200IrModel *m)
{
    if (!m) return;
    if (m->graph) cudaGraphExecDestroy(m->graph);
    if (m->ev_token) cudaEventDestroy(m->ev_token);
    if (m->prof_ev) { for (int i = 0; i <= m->nops; ++i) cudaEventDestroy(m->prof_ev[i]); free(m->prof_ev); }
    if (m->arena) cudaFree(m->arena);
    if (m->token_pinned) cudaFreeHost(m->token_pinned);
    free(m->ops);
    free(m->buf);
    free(m->w);
    free(m);
}

static int planar_format(int op) { return op == OP_GEMV_Q6K_Q8K ? 1 : op == OP_GEMV_Q80_Q80 ? 2 : op == OP_GEMV_Q50_Q80 ? 3 : 0; }

static size_t planar_bytes(int fmt, int rows, int cols)
{
    return fmt == 1 ? ckb200_q6_k_planar_bytes(rows, cols) : fmt == 2 ? ckb200_q8_0_planar_bytes(rows, cols) : ckb200_q5_0_planar_bytes(rows, cols);
}

CKB200IrModel *ckb200_ir_open(const char *call_json_path, const char *bump_path, const char *manifest_map_path)
{
    char err[256];
    JsonValue *doc = json_parse_file(call_json_path, err, sizeof err);
    if (!doc) { ckb_fail(CKB_ERR_STATE, "ir: %s", err); return NULL; }
    CKB200IrModel *m = NULL;
    CkbBump *bump = NULL;
    void *host = NULL;
    size_t host_cap = 0;
    const char *format = json_str(json_get(doc, "format"), ""), *mode = json_str(json_get(doc, "mode"), "");
    if (strcmp(format, "lowered-ir-v3") || strcmp(mode, "decode")) {
        ckb_fail(CKB_ERR_STATE, "ir: %s is '%s' / mode '%s'; this executor replays lowered-ir-v3 decode files", call_json_path, format, mode);
        goto fail;
    }
    if (json_len(json_get(doc, "errors")) > 0) { ckb_fail(CKB_ERR_STATE, "ir: the file lists %d lowering errors", json_len(json_get(doc, "errors"))); goto fail; }
    const JsonValue *cfg = json_get(doc, "config"), *mem = json_get(doc, "memory"), *ops = json_get(doc, "operations");
    const JsonValue *jw = json_get(json_get(mem, "weights"), "entries"), *jb = json_get(json_get(mem, "activations"), "buffers");
    if (!cfg || !jw || !jb || json_len(ops) <= 0) { ckb_fail(CKB_ERR_STATE, "ir: config, memory plan or operations missing"); goto fail; }
    m = (CKB200IrModel *)calloc(1, sizeof *m);
    if (!m) goto fail;
    m->vocab = (int)json_num(json_get(cfg, "vocab_size"), 0);
    m->max_seq = (int)json_num(json_get(cfg, "max_seq_len"), json_num(json_get(cfg, "context_length"), 0));
    m->layers = (int)json_num(json_get(cfg, "num_layers"), 0);
    m->kv_heads = (int)json_num(json_get(cfg, "num_kv_heads"), 0);
    m->heads = (int)json_num(json_get(cfg, "num_heads"), 0);
    m->head_dim = (int)json_num(json_get(cfg, "head_dim"), 0);
    if (m->vocab <= 0 || m->max_seq <= 0 || m->layers <= 0 || m->kv_heads <= 0 || m->head_dim <= 0 || m->heads <= 0) { ckb_fail(CKB_ERR_STATE, "ir: config lacks the model dimensions"); goto fail; }
    if ((int)json_num(json_get(cfg, "num_seqs"), 1) != 1) { ckb_fail(CKB_ERR_SHAPE, "ir: num_seqs != 1 is not handled"); goto fail; }

    bump = ckb_bump_open(bump_path, manifest_map_path);
    if (!bump) goto fail;

    /* the arena: weights, their planar copies (sized after binding), buffers, position, attention scratch */
    m->nw = json_len(jw);
    m->nbuf = json_len(jb);
    m->w = (IrWeight *)calloc((size_t)m->nw + 1, sizeof *m->w);
    m->buf = (IrBuffer *)calloc((size_t)m->nbuf + 1, sizeof *m->buf);
    m->nops = json_len(ops);
    m->ops = (IrOp *)calloc((size_t)m->nops, sizeof *m->ops);
    if (!m->w || !m->buf || !m->ops) goto fail;
    size_t cur = 256;                                        /* offset 0 stays unused so that a NULL offset means "none" */
    for (int i = 0; i < m->nw; ++i) {
        const JsonValue *e = json_at(jw, i);
        IrWeight *w = &m->w[i];
        snprintf(w->name, sizeof w->name, "%s", json_str(json_get(e, "name"), ""));
        snprintf(w->dtype, sizeof w->dtype, "%s", json_str(json_get(e, "dtype"), ""));
        w->bytes = (size_t)json_num(json_get(e, "size"), 0);
        w->ptr = (uint8_t *)cur;
        cur = align_up(cur + w->bytes + 256, 256);           /* 256 spare bytes: the bulk-copy kernels read the 16-byte-aligned superset of a row range */
    }
    for (int i = 0; i < m->nbuf; ++i) {
        const JsonValue *e = json_at(jb, i);
        IrBuffer *bf = &m->buf[i];
        snprintf(bf->name, sizeof bf->name, "%s", json_str(json_get(e, "name"), ""));
        bf->bytes = (size_t)json_num(json_get(e, "size"), 0);
        bf->ptr = (uint8_t *)cur;
        cur = align_up(cur + bf->bytes + 256, 256);
    }
    const size_t pos_off = cur;
    cur += 256;
    m->attn_splits = ckb200_attention_decode_splits(1, m->kv_heads, m->max_seq);
    const size_t scratch_off = cur;
    cur = align_up(cur + ckb200_attention_decode_scratch_bytes(1, m->heads, m->head_dim, m->attn_splits), 256);

    /* bind against offsets first (pointers are arena-relative until the arena exists), find which weights want planar copies */
    {
        IrBuffer *kv = find_buffer(m, "kv_cache"), *rope = find_buffer(m, "rope_cache"), *tok = find_buffer(m, "token_ids"), *lg = find_buffer(m, "logits");
        if (!kv || !rope || !tok || !lg) { ckb_fail(CKB_ERR_STATE, "ir: the memory plan lacks one of kv_cache, rope_cache, token_ids, logits"); goto fail; }
        const size_t need_kv = (size_t)m->layers * 2 * m->kv_heads * m->max_seq * m->head_dim * sizeof(float);
        if (kv->bytes < need_kv) { ckb_fail(CKB_ERR_SHAPE, "ir: kv_cache buffer has %zu bytes, the dimensions need %zu", kv->bytes, need_kv); goto fail; }
        if (lg->bytes < (size_t)m->vocab * sizeof(float)) { ckb_fail(CKB_ERR_SHAPE, "ir: logits buffer smaller than the vocabulary"); goto fail; }
    }
    size_t planar_total = 0;
    /* pass 1 only needs names and dtypes; run the real binding after the arena is allocated */
    for (int i = 0; i < m->nops; ++i) {
        const JsonValue *jop = json_at(ops, i);
        const char *symbol = json_str(json_get(jop, "function"), "");
        int op = -1;
        for (size_t s = 0; s < sizeof g_symbols / sizeof g_symbols[0]; ++s) if (!strcmp(g_symbols[s].symbol, symbol)) op = g_symbols[s].op;
        if (op < 0) { ckb_fail(CKB_ERR_STATE, "ir: op %d calls '%s', which this executor has no kernel for", i, symbol); goto fail; }
        const int pf = planar_format(op);
        if (!pf) continue;
        const JsonValue *args = json_get(jop, "args");
        const char *wref = NULL;
        int M = 0, K = 0;
        for (int a = 0; a < json_len(args); ++a) {
            const JsonValue *arg = json_at(args, a);
            const char *nm = json_str(json_get(arg, "name"), "");
            if (!strcmp(nm, "W")) wref = json_str(json_get(arg, "weight_ref"), NULL);
            if (!strcmp(nm, "M")) M = atoi(json_str(json_get(arg, "expr"), "0"));
            if (!strcmp(nm, "K")) K = atoi(json_str(json_get(arg, "expr"), "0"));
        }
        IrWeight *w = wref ? find_weight(m, wref) : NULL;
        if (!w || w->planar || M <= 0 || K <= 0 || (pf == 1 && K % 256) || (pf != 1 && K % 32)) continue;
        w->planar = (uint8_t *)cur;
        const size_t pb = planar_bytes(pf, M, K);
        cur = align_up(cur + pb + 256, 256);
        planar_total += pb;
    }
    m->arena_bytes = cur;
    for (int i = 0; i < m->nw; ++i) {                        /* every weight of the plan must be in the file, with the plan's size */
        uint64_t size = 0;
        if (ckb_bump_find(bump, m->w[i].name, NULL, NULL, &size)) { ckb_fail(CKB_ERR_STATE, "ir: weight %s of the memory plan is not in the manifest map", m->w[i].name); goto fail; }
        if (size != m->w[i].bytes) { ckb_fail(CKB_ERR_SHAPE, "ir: weight %s has %llu bytes in the file and %zu in the plan", m->w[i].name, (unsigned long long)size, m->w[i].bytes); goto fail; }
    }
    if (ckb_ensure_init()) goto fail;                        /* everything above is host work: malformed files are refused without a device */
    if (ckb_check_cuda((int)cudaMalloc((void **)&m->arena, m->arena_bytes), "ir arena")) goto fail;
    if (ckb_check_cuda((int)cudaMemset(m->arena, 0, m->arena_bytes), "ir arena clear")) goto fail;
    for (int i = 0; i < m->nw; ++i) {
        m->w[i].ptr = m->arena + (uintptr_t)m->w[i].ptr;
        if (m->w[i].planar) m->w[i].planar = m->arena + (uintptr_t)m->w[i].planar;
    }
    for (int i = 0; i < m->nbuf; ++i) m->buf[i].ptr = m->arena + (uintptr_t)m->buf[i].ptr;
    m->pos_dev = (int *)(m->arena + pos_off);
    m->attn_scratch = (float *)(m->arena + scratch_off);
    m->kv_cache = (float *)find_buffer(m, "kv_cache")->ptr;
    m->token_ids = (int32_t *)find_buffer(m, "token_ids")->ptr;
    m->logits = (float *)find_buffer(m, "logits")->ptr;

    /* weights from the file, by name through the sidecar map; sizes must agree with the plan */
    cudaStream_t st = ckb_stream(NULL);
    for (int i = 0; i < m->nw; ++i) {
        IrWeight *w = &m->w[i];
        uint64_t off = 0, size = 0;
        if (ckb_bump_find(bump, w->name, NULL, &off, &size)) goto fail;
        if (w->bytes > host_cap) { free(host); host = malloc(w->bytes); host_cap = host ? w->bytes : 0; }
        if (!host || ckb_bump_read(bump, off, host, w->bytes)) { ckb_fail(CKB_ERR_STATE, "ir: short read of %s", w->name); goto fail; }
        if (ckb_check_cuda((int)cudaMemcpy(w->ptr, host, w->bytes, cudaMemcpyHostToDevice), "ir weight upload")) goto fail;
    }
    /* the ops */
    for (int i = 0; i < m->nops; ++i) {
        if (bind_op(m, json_at(ops, i), &m->ops[i])) goto fail;
        IrOp *o = &m->ops[i];
        const int pf = planar_format(o->op);
        if (pf) {
            IrWeight *w = (IrWeight *)o->p[3];
            o->p[3] = w ? w->planar : NULL;
        }
    }
    /* planar copies (once per weight) */
    for (int i = 0; i < m->nops; ++i) {
        IrOp *o = &m->ops[i];
        const int pf = planar_format(o->op);
        if (!pf || !o->p[3]) continue;
        int done = 0;
        for (int j = 0; j < i; ++j) if (m->ops[j].p[3] == o->p[3] && planar_format(m->ops[j].op) == pf) done = 1;
        if (done) continue;
        const int rc = pf == 1 ? ckb200_dev_q6_k_to_planar(o->p[3], o->p[1], (int)o->i[0], (int)o->i[1], st)
                     : pf == 2 ? ckb200_dev_q8_0_to_planar(o->p[3], o->p[1], (int)o->i[0], (int)o->i[1], st)
                               : ckb200_dev_q5_0_to_planar(o->p[3], o->p[1], (int)o->i[0], (int)o->i[1], st);
        if (rc) goto fail;
    }
    /* model->rope_cos / rope_sin (the init IR's one op, rope_precompute_cache, with the config's values) */
    {
        IrBuffer *rope = find_buffer(m, "rope_cache");
        int rotary = (int)json_num(json_get(cfg, "rotary_dim"), m->head_dim);
        if (rotary <= 0 || rotary > m->head_dim) rotary = m->head_dim;
        const size_t half = (size_t)m->max_seq * (rotary / 2);
        if (rope->bytes < 2 * half * sizeof(float)) { ckb_fail(CKB_ERR_SHAPE, "ir: rope_cache buffer too small for %d positions x %d", m->max_seq, rotary / 2); goto fail; }
        m->rope_cos = (float *)rope->ptr;
        m->rope_sin = m->rope_cos + half;
        const char *scaling = json_str(json_get(cfg, "rope_scaling_type"), "none");
        const int linear = !strcmp(scaling, "linear");
        if (strcmp(scaling, "none") && !linear && strcmp(scaling, "")) { ckb_fail(CKB_ERR_SHAPE, "ir: rope scaling '%s' is not handled", scaling); goto fail; }
        if (ckb200_dev_rope_precompute_cache(m->rope_cos, m->rope_sin, m->max_seq, m->head_dim, (float)json_num(json_get(cfg, "rope_theta"), 10000.0), rotary, linear,
                                             (float)json_num(json_get(cfg, "rope_scaling_factor"), 1.0), st))
            goto fail;
        /* the rope ops were bound before the tables had their place */
        for (int i = 0; i < m->nops; ++i)
            if (m->ops[i].op == OP_ROPE_HALF || m->ops[i].op == OP_ROPE_PAIR) { m->ops[i].p[2] = m->rope_cos; m->ops[i].p[3] = m->rope_sin; }
    }
    if (ckb_check_cuda((int)cudaHostAlloc((void **)&m->token_pinned, 64, cudaHostAllocDefault), "ir token staging")) goto fail;
    if (ckb_check_cuda((int)cudaEventCreateWithFlags(&m->ev_token, cudaEventDisableTiming), "ir event")) goto fail;
    if (ckb_check_cuda((int)cudaStreamSynchronize(st), "ir open")) goto fail;
    (void)planar_total;
    free(host);
    ckb_bump_close(bump);
    json_free(doc);
    return m;
fail:
    free(host);
    if (bump) ckb_bump_close(bump);
    json_free(doc);
    ckb200_ir_free(m);
    return NULL;
}

/* ---------------------------------------------------------------- per-op timing
 *
 * The reference's generated code, built with --profile, brackets every kernel call with clock_gettime and writes
 * mode,kernel,op,layer,time_us,token_id rows to CK_PROFILE_CSV / CK_PROFILE_JSON or stderr, one batch per token
 * (version/v7/scripts/codegen_v7.py:1595-1685).  With CK_PROFILE set in the environment a step is issued op by op with a CUDA event
 * between ops (no graph) and the same rows are written, the times being device times. */

static int profile_on(void)
{
    const char *e = getenv("CK_PROFILE");
    return e && *e && strcmp(e, "0");
}

static int profiled_step(CKB200IrModel *m, cudaStream_t st)
{
    if (!m->prof_ev) {
        m->prof_ev = (cudaEvent_t *)calloc((size_t)m->nops + 1, sizeof *m->prof_ev);
        if (!m->prof_ev) return CKB_ERR_STATE;
        for (int i = 0; i <= m->nops; ++i)
            if (ckb_check_cuda((int)cudaEventCreate(&m->prof_ev[i]), "ir profile event")) return CKB_ERR_CUDA;
    }
    cudaEventRecord(m->prof_ev[0], st);
    for (int i = 0; i < m->nops; ++i) {
        const int rc = run_op(m, &m->ops[i], st);
        if (rc) return rc;
        cudaEventRecord(m->prof_ev[i + 1], st);
    }
    int rc = ckb200_dev_advance_pos(m->pos_dev, st);
    if (rc) return rc;
    if (ckb_check_cuda((int)cudaStreamSynchronize(st), "ir profiled step")) return CKB_ERR_CUDA;
    const char *csv = getenv("CK_PROFILE_CSV"), *json = getenv("CK_PROFILE_JSON");
    FILE *fc = csv ? fopen(csv, m->prof_token == 0 ? "w" : "a") : (json ? NULL : stderr);
    FILE *fj = json ? fopen(json, "w") : NULL;
    if (fc && (m->prof_token == 0 || fc == stderr)) fprintf(fc, "mode,kernel,op,layer,time_us,token_id\n");
    if (fj) fprintf(fj, "{\n  \"entries\": [\n");
    for (int i = 0; i < m->nops; ++i) {
        float ms = 0.0f;
        cudaEventElapsedTime(&ms, m->prof_ev[i], m->prof_ev[i + 1]);
        const IrOp *o = &m->ops[i];
        if (fc) fprintf(fc, "decode,%s,%s,%d,%.1f,%d\n", o->symbol, o->opname, o->layer, ms * 1000.0, m->prof_token);
        if (fj) fprintf(fj, "    {\"mode\":\"decode\",\"kernel\":\"%s\",\"op\":\"%s\",\"layer\":%d,\"time_us\":%.1f,\"token_id\":%d}%s\n", o->symbol, o->opname,
                        o->layer, ms * 1000.0, m->prof_token, i < m->nops - 1 ? "," : "");
    }
    if (fj) { fprintf(fj, "  ],\n  \"total_entries\": %d,\n  \"token_id\": %d\n}\n", m->nops, m->prof_token); fclose(fj); }
    if (fc && fc != stderr) fclose(fc);
    ++m->prof_token;
    return 0;
}

/* ---------------------------------------------------------------- run */

int ckb200_ir_decode(CKB200IrModel *m, int32_t token, float *logits_host)
{
    if (!m) return CKB_ERR_STATE;
    if (m->host_pos >= m->max_seq) return ckb_fail(CKB_ERR_LIMIT, "ir: position %d is past the context length %d", m->host_pos, m->max_seq);
    cudaStream_t st = ckb_stream(NULL);
    if (m->token_in_flight) { cudaEventSynchronize(m->ev_token); m->token_in_flight = 0; }
    m->token_pinned[0] = token;
    if (ckb_check_cuda((int)cudaMemcpyAsync(m->token_ids, m->token_pinned, sizeof(int32_t), cudaMemcpyHostToDevice, st), "ir token")) return CKB_ERR_CUDA;
    cudaEventRecord(m->ev_token, st);
    m->token_in_flight = 1;
    int rc = 0;
    if (profile_on()) {
        if ((rc = profiled_step(m, st))) return rc;
    } else if (ckb_tune_get("model_graph", 1)) {
        if (!m->graph) {
            /* the first token runs eagerly (kernels set their attributes and pools grow outside a capture), then the step is captured */
            cudaGraph_t g = NULL;
            if ((rc = issue_all(m, st))) return rc;
            if (ckb_check_cuda((int)cudaStreamSynchronize(st), "ir first step")) return CKB_ERR_CUDA;
            if (ckb_check_cuda((int)cudaStreamBeginCapture(st, cudaStreamCaptureModeThreadLocal), "ir capture")) return CKB_ERR_CUDA;
            rc = issue_all(m, st);
            const int end = (int)cudaStreamEndCapture(st, &g);
            if (rc || ckb_check_cuda(end, "ir capture end")) { if (g) cudaGraphDestroy(g); return rc ? rc : CKB_ERR_CUDA; }
            size_t nodes = 0;
            cudaGraphGetNodes(g, NULL, &nodes);
            m->launches = (int)nodes;
            const int inst = (int)cudaGraphInstantiate(&m->graph, g, 0);
            cudaGraphDestroy(g);
            if (ckb_check_cuda(inst, "ir graph instantiate")) return CKB_ERR_CUDA;
        } else if (ckb_check_cuda((int)cudaGraphLaunch(m->graph, st), "ir graph launch")) {
            return CKB_ERR_CUDA;
        }
    } else if ((rc = issue_all(m, st))) {
        return rc;
    }
    ++m->host_pos;
    if (logits_host) {
        if (ckb_check_cuda((int)cudaMemcpyAsync(logits_host, m->logits, (size_t)m->vocab * sizeof(float), cudaMemcpyDeviceToHost, st), "ir logits")) return CKB_ERR_CUDA;
        return ckb_sync_check(st, "ir decode");
    }
    return 0;
}

int ckb200_ir_set_pos(CKB200IrModel *m, int pos)
{
    if (!m || pos < 0 || pos > m->max_seq) return CKB_ERR_STATE;
    cudaStream_t st = ckb_stream(NULL);
    if (ckb_check_cuda((int)cudaStreamSynchronize(st), "ir set_pos")) return CKB_ERR_CUDA;
    if (ckb_check_cuda((int)cudaMemcpy(m->pos_dev, &pos, sizeof pos, cudaMemcpyHostToDevice), "ir set_pos")) return CKB_ERR_CUDA;
    m->host_pos = pos;
    return 0;
}

int ckb200_ir_reset(CKB200IrModel *m)
{
    if (!m) return CKB_ERR_STATE;
    const size_t kv = (size_t)m->layers * 2 * m->kv_heads * m->max_seq * m->head_dim * sizeof(float);
    if (ckb_check_cuda((int)cudaMemsetAsync(m->kv_cache, 0, kv, ckb_stream(NULL)), "ir reset")) return CKB_ERR_CUDA;
    return ckb200_ir_set_pos(m, 0);
}

int ckb200_ir_get_pos(const CKB200IrModel *m) { return m ? m->host_pos : -1; }
int ckb200_ir_vocab_size(const CKB200IrModel *m) { return m ? m->vocab : 0; }
int ckb200_ir_context_length(const CKB200IrModel *m) { return m ? m->max_seq : 0; }
int ckb200_ir_num_ops(const CKB200IrModel *m) { return m ? m->nops : 0; }
const char *ckb200_ir_op_symbol(const CKB200IrModel *m, int i) { return m && i >= 0 && i < m->nops ? m->ops[i].symbol : NULL; }
int ckb200_ir_graph_nodes(const CKB200IrModel *m) { return m ? m->launches : 0; }

void *ckb200_ir_buffer(CKB200IrModel *m, const char *name, size_t *bytes)
{
    IrBuffer *b = m ? find_buffer(m, name) : NULL;
    if (bytes) *bytes = b ? b->bytes : 0;
    return b ? b->ptr : NULL;
}
