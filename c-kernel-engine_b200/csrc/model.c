/* Device-resident decode step: the op sequence the reference's generated ck_decode() issues for a
 * Llama/Qwen-style decoder (version/v7/scripts/codegen_v7.py:886-931; per-layer template
 * version/v7/templates/qwen2.json:95-110), run as one CUDA graph on one stream with every activation,
 * the KV cache and the position counter in HBM.  Weights keep the reference's block formats and
 * row-major [out][in] layout; gate and up rows are one [2I][D] matrix, gate first
 * (codegen_v7.py:686-714).
 *
 * Per layer:  x += prev; h = Q8_K(rmsnorm(x))            (add_rmsnorm_q8k)
 *             q,k,v = Wq.h, Wk.h, Wv.h                   (dequant-dot GEMVs)
 *             rope(q,k) ; cache[pos] = k,v               (rope_kv_store)
 *             a = attention(q, cache[0..pos])            (split-K decode attention)
 *             o = Wo.Q8_K(a)
 *             x += o; h = Q8_K(rmsnorm(x))
 *             m = Q8_K(swiglu(W1.h))                     (swiglu_q8k)
 *             prev = W2.m
 * Finally     x += prev; logits = Wlm.Q8_K(rmsnorm(x)); pos += 1
 *
 * K-quant GEMVs need K % 256 == 0: rows that feed them are kept `aligned` = roundup(K, 256) wide with
 * a zero tail, exactly what rmsnorm_forward(..., d_model, aligned_embed_dim, ...) produces in the
 * reference (src/kernels/rmsnorm_kernels.c:245-248).
 *
 * Tensor parallelism: with tp_size > 1 every rank holds tp_size-th of the heads and of the FFN rows
 * (column-parallel Wq/Wk/Wv/W1) and a 256-aligned slice of the input columns of Wo/W2 (row-parallel);
 * the two partial outputs per layer are summed over ranks by the all-reduce hook.
 */
#include <cuda_runtime_api.h>
#include <stdint.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#include "../../include/ckb200.h"
#include "../../include/ckb200_model.h"
#include "launch.h"
#include "runtime.h"
#include "step_fused.h"

/* tensor-core GEMM of gemm_tc.cu: wf 0 = Q4_K rows, 1 = Q6_K row-planar; -1 when the shape is not handled.  The workspace
 * (activation tiles + split-K partial sums) is the model's own: a pointer recorded in the step's graph must not come from
 * the library's grow-on-demand pool, which any later call may free and regrow. */
void ckb_attn_hint_early_rows(int on);      /* attention.cu */
int ckb_launch_gemm_tc_ws(int wf, const void *A_q8, const void *B, const float *bias, float *C, int ldc, int M, int N, int K, int min_tokens, void *ws,
                          size_t ws_bytes, void *stream);
size_t ckb_gemm_tc_workspace_bytes(int M, int N, int K);
/* integer-MMA kernel of gemm_q4k_mma.cu for up to 64 tokens (Q4_K rows, no workspace); -1 when it does not take the call */
int ckb_launch_gemm_q4k_mma(const void *A_q8, const void *B, const float *bias, float *C, int ldc, int M, int N, int K, void *stream);
int ckb_launch_gemm_q6k_mma(const void *A_q8, const void *B_planar, const float *bias, float *C, int ldc, int M, int N, int K, void *stream);   /* gemm_q6k_mma.cu */
int ckb_gemm_q4k_mma_takes(const void *A_q8, const void *B, int M, int N, int K);
int ckb_gemm_q6k_mma_takes(const void *A_q8, const void *B_planar, int M, int N, int K);

/* From this many sequences a projection runs as one batched product instead of a GEMV per sequence.  The tcgen05 kernel's time
 * hardly depends on the token count below 32 (it is bound by expanding the weights), so for the Q6_K matrices it wins from about
 * three sequences: 86 us for the 8192 x 28672 down projection against 36 us per GEMV. */
#define MODEL_GEMM_MIN_BATCH 4

enum { FMT_Q4K = 0, FMT_Q6K = 1, FMT_Q80 = 2, FMT_Q50 = 3 };
/* formats with 32-element blocks take Q8_0 activations, the K-quants take Q8_K */
static int fmt_block32(int fmt) { return fmt == FMT_Q80 || fmt == FMT_Q50; }

typedef struct {
    void *w;            /* device pointer */
    size_t bytes;
    int fmt;            /* block format, or -1 for fp32 */
    int rows, cols;     /* [rows][cols] elements (cols already aligned) */
    void *planar;       /* Q6_K / Q5_0 matrices that feed a GEMV: second copy in the row-planar layout (aligned 16-byte loads), or NULL */
} Tensor;

typedef struct {
    Tensor t[CKB_T_PER_LAYER];
} Layer;

struct CKB200Model {
    CKB200ModelConfig c;
    int D, Da;              /* embed dim and its 256-aligned width */
    int Hl, Hkvl, d;        /* local heads */
    int Al, Ala;            /* local attention width Hl*d and aligned */
    int Il;                 /* local intermediate size */
    int Vl;                 /* local vocab rows */
    Layer *layers;
    Tensor emb, final_gamma, lm_head;
    uint8_t *arena;         /* all weights */
    size_t arena_bytes;
    uint8_t *planar_arena;  /* row-planar copies of the Q6_K projection matrices, rebuilt from `arena` when weights change */
    size_t planar_bytes;
    int planar_ready;
    uint8_t *kv;            /* [L][2][B][Hkvl][S][d], elements of kv_eb bytes */
    int kv_eb;              /* 4: fp32 cache; 2: IEEE fp16 cache (tune model_kv_f16 at creation: kv_cache_store_f16 and the
                             * _f16cache attention of the reference, half the cache bytes per key) */
    long long kv_layer_stride, kv_batch_stride;     /* in elements */
    float *rope_cos, *rope_sin;
    /* activations */
    float *x, *prev, *q, *k, *v, *att, *o, *gu, *logits, *attn_scratch;
    float *x2;              /* second residual row of the fused step (each fused launch reads one and writes the other) */
    float *mf;              /* fp32 SwiGLU output of the fused step, round256(Il) wide, tail zero */
    int *attn_counters;     /* arrival counters of the attention kernel's in-launch split merge */
    /* batched prefill (grown on demand to the longest prompt seen): token-major rows and head-major attention tensors */
    int pf_tokens;
    float *pf_x, *pf_delta, *pf_o, *pf_q, *pf_k, *pf_v, *pf_qh, *pf_oh, *pf_gu;
    uint8_t *pf_hq, *pf_aq, *pf_mq;
    uint8_t *hq, *aq, *mq;
    int32_t *tokens_dev, *pos_dev;
    int32_t *tokens_pinned;
    int host_pos;           /* mirror of *pos_dev as of the last enqueued step (decode refuses to run past the context) */
    uint8_t *gemm_ws;       /* workspace of the tensor-core GEMM of batched decode: the step's graph keeps this pointer */
    size_t gemm_ws_bytes;
    int attn_splits;
    cudaGraphExec_t graph;
    int graph_ready;
    /* q, k and v projections read the same quantised row and are independent: they run on three streams (forked and
     * joined with events, which a stream capture turns into parallel branches of the step's graph) */
    cudaStream_t side[2];
    cudaEvent_t ev_fork, ev_join[2];
    cudaEvent_t ev_tokens;  /* the last copy out of tokens_pinned: the next call waits for it before it overwrites the buffer */
    int tokens_in_flight;
    int have_prev;
    ckb200_allreduce_fn allreduce;
    void *allreduce_ctx;
    ckb200_tp_norm_fn tp_norm;
    void *tp_norm_ctx;
};

static size_t align_up(size_t v, size_t a) { return (v + a - 1) / a * a; }
static size_t kv_bytes(const struct CKB200Model *m) { return (size_t)m->c.num_layers * (size_t)m->kv_layer_stride * (size_t)m->kv_eb; }
/* key (is_v = 0) or value cache of one layer: [B][Hkvl][S][d] */
static void *kv_at(const struct CKB200Model *m, int layer, int is_v)
{
    return m->kv + ((size_t)layer * (size_t)m->kv_layer_stride + (is_v ? (size_t)m->c.batch * (size_t)m->kv_batch_stride : 0)) * (size_t)m->kv_eb;
}
static int round256(int v) { return (v + 255) / 256 * 256; }

static size_t fmt_row_bytes(int fmt, int cols)
{
    switch (fmt) {
        case FMT_Q4K: return (size_t)(cols / 256) * 144;
        case FMT_Q6K: return (size_t)(cols / 256) * 210;
        case FMT_Q80: return (size_t)(cols / 32) * 34;
        case FMT_Q50: return (size_t)(cols / 32) * 22;
        default: return (size_t)cols * 4;
    }
}

static void tensor_plan(Tensor *t, int fmt, int rows, int cols, size_t *cursor)
{
    t->fmt = fmt;
    t->rows = rows;
    t->cols = cols;
    t->bytes = (size_t)rows * fmt_row_bytes(fmt, cols);
    t->w = (void *)(uintptr_t)*cursor;              /* offset for now */
    *cursor = align_up(*cursor + t->bytes + 32, 256);
}

static int cols_for(int fmt, int k) { return fmt_block32(fmt) ? (k + 31) / 32 * 32 : round256(k); }

CKB200Model *ckb200_model_create(const CKB200ModelConfig *cfg)
{
    if (!cfg) return NULL;
    if (ckb_ensure_init()) return NULL;
    const int tp = cfg->tp_size > 0 ? cfg->tp_size : 1;
    if (cfg->num_heads % cfg->num_kv_heads || cfg->num_heads % tp || cfg->intermediate_size % tp ||
        (cfg->num_kv_heads % tp && tp % cfg->num_kv_heads) || cfg->batch <= 0 || cfg->head_dim % 2) {
        ckb_fail(CKB_ERR_SHAPE, "model_create: heads %d / kv heads %d / ffn %d do not split over tp=%d", cfg->num_heads,
                 cfg->num_kv_heads, cfg->intermediate_size, tp);
        return NULL;
    }
    CKB200Model *m = (CKB200Model *)calloc(1, sizeof *m);
    if (!m) return NULL;
    m->c = *cfg;
    m->c.tp_size = tp;
    m->D = cfg->embed_dim;
    m->Da = round256(m->D);
    m->d = cfg->head_dim;
    m->Hl = cfg->num_heads / tp;
    m->Hkvl = cfg->num_kv_heads >= tp ? cfg->num_kv_heads / tp : 1;
    m->Al = m->Hl * m->d;
    m->Ala = round256(m->Al);
    m->Il = cfg->intermediate_size / tp;
    m->Vl = cfg->vocab_size;                           /* the LM head is kept whole on every rank */
    if (cfg->batch > 1 && m->Al != m->Ala) {
        ckb_fail(CKB_ERR_SHAPE, "model_create: batch > 1 needs the attention width %d to be a multiple of 256", m->Al);
        free(m);
        return NULL;
    }
    if (tp > 1 && (m->Al % 256 || m->Il % 256)) {
        ckb_fail(CKB_ERR_SHAPE, "model_create: tp=%d needs the per-rank attention width %d and FFN width %d to be multiples of 256", tp, m->Al, m->Il);
        free(m);
        return NULL;
    }
    m->kv_eb = ckb_tune_get("model_kv_f16", 0) ? 2 : 4;
    if (m->kv_eb == 2 && ((m->d != 64 && m->d != 128) || m->Hl / m->Hkvl > 8 || ((long long)m->Hkvl * cfg->max_seq_len * m->d) % 8)) {
        ckb_fail(CKB_ERR_SHAPE, "model_create: the fp16 cache needs a head size of 64 or 128 and at most 8 query heads per kv head (have %d, %d)", m->d,
                 m->Hl / m->Hkvl);
        free(m);
        return NULL;
    }
    const int L = cfg->num_layers, B = cfg->batch, S = cfg->max_seq_len;
    m->layers = (Layer *)calloc((size_t)L, sizeof(Layer));
    size_t cur = 0;
    for (int l = 0; l < L; ++l) {
        Tensor *t = m->layers[l].t;
        tensor_plan(&t[CKB_T_LN1], -1, 1, m->Da, &cur);
        tensor_plan(&t[CKB_T_WQ], cfg->fmt_q, m->Hl * m->d, cols_for(cfg->fmt_q, m->D), &cur);
        tensor_plan(&t[CKB_T_WK], cfg->fmt_k, m->Hkvl * m->d, cols_for(cfg->fmt_k, m->D), &cur);
        tensor_plan(&t[CKB_T_WV], cfg->fmt_v, m->Hkvl * m->d, cols_for(cfg->fmt_v, m->D), &cur);
        tensor_plan(&t[CKB_T_WO], cfg->fmt_o, m->D, cols_for(cfg->fmt_o, m->Al), &cur);
        tensor_plan(&t[CKB_T_LN2], -1, 1, m->Da, &cur);
        tensor_plan(&t[CKB_T_W1], cfg->fmt_gate_up, 2 * m->Il, cols_for(cfg->fmt_gate_up, m->D), &cur);
        tensor_plan(&t[CKB_T_W2], cfg->fmt_down, m->D, cols_for(cfg->fmt_down, m->Il), &cur);
    }
    tensor_plan(&m->final_gamma, -1, 1, m->Da, &cur);
    tensor_plan(&m->lm_head, cfg->fmt_lm_head, m->Vl, cols_for(cfg->fmt_lm_head, m->D), &cur);
    if (cfg->tie_embeddings) m->emb = m->lm_head;
    else tensor_plan(&m->emb, cfg->fmt_embedding, cfg->vocab_size, cols_for(cfg->fmt_embedding, m->D), &cur);
    {
        /* every fmt_* field names a known block format; token embeddings have no Q5_0 row kernel */
        const int fmts[] = { cfg->fmt_q, cfg->fmt_k, cfg->fmt_v, cfg->fmt_o, cfg->fmt_gate_up, cfg->fmt_down, cfg->fmt_lm_head, m->emb.fmt };
        int bad = m->emb.fmt == FMT_Q50;
        for (unsigned i = 0; i < sizeof fmts / sizeof fmts[0]; ++i) bad |= fmts[i] < FMT_Q4K || fmts[i] > FMT_Q50;
        if (bad) {
            ckb_fail(CKB_ERR_SHAPE, "model_create: unknown weight format, or Q5_0 for the token embedding");
            free(m->layers);
            free(m);
            return NULL;
        }
    }
    m->arena_bytes = cur + 256;
    {
        size_t pc = 0;
        for (int l = 0; l <= L; ++l) {
            Tensor *list[7];
            int n = 0;
            if (l < L) {
                static const int which[6] = { CKB_T_WQ, CKB_T_WK, CKB_T_WV, CKB_T_WO, CKB_T_W1, CKB_T_W2 };
                for (int i = 0; i < 6; ++i) list[n++] = &m->layers[l].t[which[i]];
            } else {
                list[n++] = &m->lm_head;
            }
            for (int i = 0; i < n; ++i) {
                if (list[i]->fmt != FMT_Q6K && list[i]->fmt != FMT_Q50) continue;
                list[i]->planar = (void *)(uintptr_t)(pc + 1);      /* offset + 1 for now (0 = none) */
                pc = align_up(pc + (list[i]->fmt == FMT_Q6K ? ckb200_q6_k_planar_bytes(list[i]->rows, list[i]->cols)
                                                            : ckb200_q5_0_planar_bytes(list[i]->rows, list[i]->cols)), 256);
            }
        }
        m->planar_bytes = pc;
    }

    int ok = 1;
#define DEV_ALLOC(ptr, bytes) do { if (ok && ckb_check_cuda((int)cudaMalloc((void **)&(ptr), (bytes)), "cudaMalloc(model)")) ok = 0; } while (0)
    DEV_ALLOC(m->arena, m->arena_bytes);
    if (m->planar_bytes) DEV_ALLOC(m->planar_arena, m->planar_bytes);
    m->kv_batch_stride = (long long)m->Hkvl * S * m->d;
    m->kv_layer_stride = 2LL * B * m->kv_batch_stride;
    DEV_ALLOC(m->kv, kv_bytes(m));
    DEV_ALLOC(m->rope_cos, (size_t)S * (m->d / 2) * sizeof(float));
    DEV_ALLOC(m->rope_sin, (size_t)S * (m->d / 2) * sizeof(float));
    DEV_ALLOC(m->x, (size_t)B * m->Da * sizeof(float));
    DEV_ALLOC(m->prev, (size_t)B * m->Da * sizeof(float));
    DEV_ALLOC(m->o, (size_t)B * m->Da * sizeof(float));
    DEV_ALLOC(m->q, (size_t)B * m->Al * sizeof(float));
    DEV_ALLOC(m->k, (size_t)B * m->Hkvl * m->d * sizeof(float));
    DEV_ALLOC(m->v, (size_t)B * m->Hkvl * m->d * sizeof(float));
    DEV_ALLOC(m->att, (size_t)B * m->Ala * sizeof(float));
    DEV_ALLOC(m->gu, (size_t)B * 2 * m->Il * sizeof(float));
    DEV_ALLOC(m->logits, (size_t)B * m->Vl * sizeof(float));
    DEV_ALLOC(m->hq, (size_t)B * (m->Da / 32) * 34 + (size_t)B * (m->Da / 256) * 292 + 256);
    DEV_ALLOC(m->aq, (size_t)B * (m->Ala / 32) * 34 + (size_t)B * (m->Ala / 256) * 292 + 256);
    DEV_ALLOC(m->mq, (size_t)B * ((m->Il + 255) / 256) * 292 * 2 + 256);
    DEV_ALLOC(m->x2, (size_t)B * m->Da * sizeof(float));
    DEV_ALLOC(m->mf, (size_t)B * round256(m->Il) * sizeof(float));
    DEV_ALLOC(m->attn_counters, ckb200_attention_decode_counter_bytes(B, m->Hkvl) + 256);
    DEV_ALLOC(m->tokens_dev, (size_t)B * sizeof(int32_t));
    DEV_ALLOC(m->pos_dev, 256);
    if (B >= MODEL_GEMM_MIN_BATCH) {
        /* largest projection of the step (row counts and input widths as planned above) */
        size_t need = 0;
        const int shapes[][2] = { { m->Hl * m->d, m->Da }, { m->D, m->Ala }, { 2 * m->Il, m->Da }, { m->D, round256(m->Il) }, { m->Vl, m->Da } };
        for (unsigned i = 0; i < sizeof shapes / sizeof shapes[0]; ++i) {
            const size_t b = ckb_gemm_tc_workspace_bytes(B, shapes[i][0], shapes[i][1]);
            if (b > need) need = b;
        }
        m->gemm_ws_bytes = need;
        DEV_ALLOC(m->gemm_ws, need);
    }
    m->attn_splits = ckb200_attention_decode_splits_kv(B, m->Hkvl, S, m->kv_eb);
    {
        size_t sb = ckb200_attention_decode_scratch_bytes(B, m->Hl, m->d, m->attn_splits);
        DEV_ALLOC(m->attn_scratch, sb ? sb : 256);
    }
    if (ok && ckb_check_cuda((int)cudaHostAlloc((void **)&m->tokens_pinned, (size_t)B * sizeof(int32_t), cudaHostAllocDefault), "cudaHostAlloc")) ok = 0;
    for (int i = 0; ok && i < 2; ++i) {
        if (ckb_check_cuda((int)cudaStreamCreateWithFlags(&m->side[i], cudaStreamNonBlocking), "side stream")) ok = 0;
        if (ok && ckb_check_cuda((int)cudaEventCreateWithFlags(&m->ev_join[i], cudaEventDisableTiming), "join event")) ok = 0;
    }
    if (ok && ckb_check_cuda((int)cudaEventCreateWithFlags(&m->ev_fork, cudaEventDisableTiming), "fork event")) ok = 0;
    if (ok && ckb_check_cuda((int)cudaEventCreateWithFlags(&m->ev_tokens, cudaEventDisableTiming), "tokens event")) ok = 0;
    if (!ok) { ckb200_model_free(m); return NULL; }
#undef DEV_ALLOC
    /* offsets -> pointers */
    for (int l = 0; l < L; ++l)
        for (int i = 0; i < CKB_T_PER_LAYER; ++i) m->layers[l].t[i].w = m->arena + (uintptr_t)m->layers[l].t[i].w;
    m->final_gamma.w = m->arena + (uintptr_t)m->final_gamma.w;
    m->lm_head.w = m->arena + (uintptr_t)m->lm_head.w;
    m->emb.w = cfg->tie_embeddings ? m->lm_head.w : (void *)(m->arena + (uintptr_t)m->emb.w);
    for (int l = 0; l < L; ++l)
        for (int i = 0; i < CKB_T_PER_LAYER; ++i)
            if (m->layers[l].t[i].planar) m->layers[l].t[i].planar = m->planar_arena + ((uintptr_t)m->layers[l].t[i].planar - 1);
    if (m->lm_head.planar) m->lm_head.planar = m->planar_arena + ((uintptr_t)m->lm_head.planar - 1);
    if (cfg->tie_embeddings) m->emb.planar = NULL;             /* the embedding lookup reads the original rows */

    cudaStream_t st = ckb_stream(NULL);
    cudaMemsetAsync(m->arena, 0, m->arena_bytes, st);
    cudaMemsetAsync(m->kv, 0, kv_bytes(m), st);
    cudaMemsetAsync(m->att, 0, (size_t)B * m->Ala * sizeof(float), st);       /* zero tail of the attention rows stays zero */
    cudaMemsetAsync(m->x, 0, (size_t)B * m->Da * sizeof(float), st);
    cudaMemsetAsync(m->prev, 0, (size_t)B * m->Da * sizeof(float), st);
    cudaMemsetAsync(m->o, 0, (size_t)B * m->Da * sizeof(float), st);
    cudaMemsetAsync(m->pos_dev, 0, 256, st);
    cudaMemsetAsync(m->x2, 0, (size_t)B * m->Da * sizeof(float), st);
    cudaMemsetAsync(m->mf, 0, (size_t)B * round256(m->Il) * sizeof(float), st);
    cudaMemsetAsync(m->attn_counters, 0, ckb200_attention_decode_counter_bytes(B, m->Hkvl) + 256, st);
    ckb200_dev_rope_precompute_cache_split(m->rope_cos, m->rope_sin, S, m->d, cfg->rope_theta, NULL);
    if (ckb_check_cuda((int)cudaStreamSynchronize(st), "model init")) { ckb200_model_free(m); return NULL; }
    return m;
}

void ckb200_model_free(CKB200Model *m)
{
    if (!m) return;
    cudaStreamSynchronize(ckb_stream(NULL));
    if (m->graph_ready) cudaGraphExecDestroy(m->graph);
    void *ptrs[] = { m->arena, m->planar_arena, m->kv, m->rope_cos, m->rope_sin, m->x, m->prev, m->o, m->q, m->k, m->v, m->att, m->gu, m->logits,
                     m->hq, m->aq, m->mq, m->tokens_dev, m->pos_dev, m->attn_scratch, m->gemm_ws, m->x2, m->mf, m->attn_counters,
                     m->pf_x, m->pf_delta, m->pf_o, m->pf_q, m->pf_k, m->pf_v, m->pf_qh, m->pf_oh, m->pf_gu, m->pf_hq, m->pf_aq, m->pf_mq };
    for (size_t i = 0; i < sizeof ptrs / sizeof ptrs[0]; ++i) if (ptrs[i]) cudaFree(ptrs[i]);
    if (m->tokens_pinned) cudaFreeHost(m->tokens_pinned);
    for (int i = 0; i < 2; ++i) {
        if (m->side[i]) cudaStreamDestroy(m->side[i]);
        if (m->ev_join[i]) cudaEventDestroy(m->ev_join[i]);
    }
    if (m->ev_fork) cudaEventDestroy(m->ev_fork);
    if (m->ev_tokens) cudaEventDestroy(m->ev_tokens);
    free(m->layers);
    free(m);
}

static Tensor *find_tensor(CKB200Model *m, int layer, int which)
{
    if (layer >= 0 && layer < m->c.num_layers && which >= 0 && which < CKB_T_PER_LAYER) return &m->layers[layer].t[which];
    if (layer == -1) {
        if (which == CKB_T_FINAL_GAMMA) return &m->final_gamma;
        if (which == CKB_T_LM_HEAD) return &m->lm_head;
        if (which == CKB_T_EMBEDDING) return &m->emb;
    }
    return NULL;
}

size_t ckb200_model_tensor_bytes(CKB200Model *m, int layer, int which)
{
    Tensor *t = m ? find_tensor(m, layer, which) : NULL;
    return t ? t->bytes : 0;
}
void *ckb200_model_tensor_ptr(CKB200Model *m, int layer, int which)
{
    Tensor *t = m ? find_tensor(m, layer, which) : NULL;
    return t ? t->w : NULL;
}
int ckb200_model_tensor_shape(CKB200Model *m, int layer, int which, int *rows, int *cols, int *fmt)
{
    Tensor *t = m ? find_tensor(m, layer, which) : NULL;
    if (!t) return CKB_ERR_STATE;
    if (rows) *rows = t->rows;
    if (cols) *cols = t->cols;
    if (fmt) *fmt = t->fmt;
    return 0;
}

int ckb200_model_upload_tensor(CKB200Model *m, int layer, int which, const void *host, size_t bytes)
{
    Tensor *t = m ? find_tensor(m, layer, which) : NULL;
    if (!t || !host) return ckb_fail(CKB_ERR_STATE, "model_upload_tensor: no such tensor (%d, %d)", layer, which);
    if (bytes != t->bytes) return ckb_fail(CKB_ERR_SHAPE, "model_upload_tensor(%d, %d): got %zu bytes, tensor has %zu", layer, which, bytes, t->bytes);
    m->planar_ready = 0;               /* weights are read through fixed pointers: the captured graph stays valid */
    /* Weights may only change while the stream is idle: queued steps still read them (the GEMVs even prefetch weights ahead
     * of their dependency wait), and this copy runs outside the library's non-blocking stream. */
    if (ckb_check_cuda((int)cudaStreamSynchronize(ckb_stream(NULL)), "upload tensor (drain)")) return CKB_ERR_CUDA;
    return ckb_check_cuda((int)cudaMemcpy(t->w, host, bytes, cudaMemcpyHostToDevice), "upload tensor");
}

static int fill_tensor(Tensor *t, unsigned long long seed)
{
    if (t->fmt < 0) return ckb200_dev_fill_normal((float *)t->w, (long long)t->rows * t->cols, 1, seed, NULL);
    const long long nblocks = (long long)t->rows * (t->cols / (fmt_block32(t->fmt) ? 32 : 256));
    return ckb200_dev_fill_blocks(t->w, nblocks, t->fmt, seed, NULL);
}

int ckb200_model_fill_synthetic(CKB200Model *m, unsigned long long seed)
{
    if (!m) return CKB_ERR_STATE;
    m->planar_ready = 0;
    unsigned long long s = seed * 1000003ull + 17;
    for (int l = 0; l < m->c.num_layers; ++l)
        for (int i = 0; i < CKB_T_PER_LAYER; ++i)
            if (fill_tensor(&m->layers[l].t[i], s++)) return CKB_ERR_CUDA;
    if (fill_tensor(&m->final_gamma, s++) || fill_tensor(&m->lm_head, s++)) return CKB_ERR_CUDA;
    if (!m->c.tie_embeddings && fill_tensor(&m->emb, s++)) return CKB_ERR_CUDA;
    return ckb200_synchronize();
}

int ckb200_model_fill_kv_synthetic(CKB200Model *m, int tokens, unsigned long long seed)
{
    if (!m || tokens < 0 || tokens > m->c.max_seq_len) return ckb_fail(CKB_ERR_STATE, "model_fill_kv_synthetic: bad token count %d", tokens);
    const int L = m->c.num_layers, B = m->c.batch, S = m->c.max_seq_len;
    cudaStream_t st = ckb_stream(NULL);
    cudaMemsetAsync(m->kv, 0, kv_bytes(m), st);
    if (tokens > 0) {
        /* N(0,1) in the first `tokens` positions of every head: fill a compact buffer, then strided copy */
        const size_t heads = (size_t)L * 2 * B * m->Hkvl, eb = (size_t)m->kv_eb;
        uint8_t *tmp = NULL;
        const size_t row = (size_t)tokens * m->d;
        const size_t chunk_heads = heads < 4096 ? heads : 4096;
        if (ckb_check_cuda((int)cudaMalloc((void **)&tmp, chunk_heads * row * eb), "cudaMalloc(kv fill)")) return CKB_ERR_CUDA;
        for (size_t h0 = 0; h0 < heads; h0 += chunk_heads) {
            const size_t n = heads - h0 < chunk_heads ? heads - h0 : chunk_heads;
            if (m->kv_eb == 2) ckb200_dev_fill_normal_f16((uint16_t *)tmp, (long long)(n * row), 0, seed + h0, NULL);
            else ckb200_dev_fill_normal((float *)tmp, (long long)(n * row), 0, seed + h0, NULL);
            cudaMemcpy2DAsync(m->kv + h0 * (size_t)S * m->d * eb, (size_t)S * m->d * eb, tmp, row * eb, row * eb, n, cudaMemcpyDeviceToDevice, st);
        }
        cudaStreamSynchronize(st);
        cudaFree(tmp);
    }
    return ckb200_model_set_pos(m, tokens);
}

int ckb200_model_set_pos(CKB200Model *m, int pos)
{
    if (!m || pos < 0 || pos >= m->c.max_seq_len) return ckb_fail(CKB_ERR_STATE, "model_set_pos: %d outside [0, %d)", pos, m ? m->c.max_seq_len : 0);
    int32_t p = pos;
    cudaStream_t st = ckb_stream(NULL);
    if (ckb_check_cuda((int)cudaMemcpyAsync(m->pos_dev, &p, sizeof p, cudaMemcpyHostToDevice, st), "set pos")) return CKB_ERR_CUDA;
    if (ckb_check_cuda((int)cudaStreamSynchronize(st), "set pos")) return CKB_ERR_CUDA;
    m->host_pos = pos;
    return 0;
}

int ckb200_model_get_pos(CKB200Model *m)
{
    int32_t p = -1;
    if (!m) return -1;
    cudaStreamSynchronize(ckb_stream(NULL));
    cudaMemcpy(&p, m->pos_dev, sizeof p, cudaMemcpyDeviceToHost);
    return p;
}

void ckb200_model_set_tp_norm(CKB200Model *m, ckb200_tp_norm_fn fn, void *ctx)
{
    if (!m) return;
    m->tp_norm = fn;
    m->tp_norm_ctx = ctx;
    m->graph_ready = 0;
}

void ckb200_model_set_allreduce(CKB200Model *m, ckb200_allreduce_fn fn, void *ctx)
{
    if (!m) return;
    m->allreduce = fn;
    m->allreduce_ctx = ctx;
    m->graph_ready = 0;
}

float *ckb200_model_logits_device(CKB200Model *m) { return m ? m->logits : NULL; }
void *ckb200_model_kv_device(CKB200Model *m, int layer, int is_v)
{
    if (!m || layer < 0 || layer >= m->c.num_layers) return NULL;
    return kv_at(m, layer, is_v);
}
int ckb200_model_kv_element_bytes(CKB200Model *m) { return m ? m->kv_eb : 0; }

/* ------------------------------------------------------------------ the step */

static int gemv_q(int fmt, float *y, const Tensor *w, const void *xq, void *st)
{
    switch (fmt) {
        case FMT_Q4K: return ckb200_dev_gemv_q4_k_q8_k(y, w->w, xq, w->rows, w->cols, st);
        case FMT_Q6K:
            /* few long rows: the ring kernel, which splits a row over warps, measured faster than the planar one */
            if (w->planar && !(w->rows <= 2048 && w->cols >= 4096)) return ckb200_dev_gemv_q6_k_planar_q8_k(y, w->planar, xq, w->rows, w->cols, st);
            return ckb200_dev_gemv_q6_k_q8_k(y, w->w, xq, w->rows, w->cols, st);
        case FMT_Q50:
            if (w->planar) return ckb200_dev_gemv_q5_0_planar_q8_0(y, w->planar, xq, w->rows, w->cols, st);
            return ckb200_dev_gemv_q5_0_q8_0(y, w->w, xq, w->rows, w->cols, st);
        default: return ckb200_dev_gemv_q8_0_q8_0(y, w->w, xq, w->rows, w->cols, st);
    }
}


/* A product of matvec() that uses no shared workspace: a per-sequence GEMV, or a batch on the integer-MMA kernels.  Such products
 * may run side by side on the side streams. */
static int matvec_standalone(const CKB200Model *m, const Tensor *w, const uint8_t *xq)
{
    const int B = m->c.batch;
    if (B < MODEL_GEMM_MIN_BATCH) return 1;
    if (w->fmt == FMT_Q4K) return ckb_gemm_q4k_mma_takes(xq, w->w, B, w->rows, w->cols);
    if (w->fmt == FMT_Q6K && w->planar) return ckb_gemm_q6k_mma_takes(xq, w->planar, B, w->rows, w->cols);
    return 0;
}

/* y[b] = W . xq[b] for every sequence b; xq rows are `cols`-wide quantised vectors */
static int matvec(CKB200Model *m, const Tensor *w, const uint8_t *xq, float *y, int y_stride, void *st)
{
    /* batched decode: the weights are streamed once for all sequences.  Q4_K from 4 sequences up on the integer-MMA kernel (no workspace),
     * otherwise from 16 up on the tcgen05 kernel */
    if (w->fmt == FMT_Q4K && m->c.batch > 1) {
        const int rc = ckb_launch_gemm_q4k_mma(xq, w->w, NULL, y, y_stride, m->c.batch, w->rows, w->cols, st);
        if (rc >= 0) return rc;
    }
    if (w->fmt == FMT_Q6K && w->planar && m->c.batch > 1) {
        const int rc = ckb_launch_gemm_q6k_mma(xq, w->planar, NULL, y, y_stride, m->c.batch, w->rows, w->cols, st);
        if (rc >= 0) return rc;
    }
    if (m->c.batch >= MODEL_GEMM_MIN_BATCH && (w->fmt == FMT_Q4K || (w->fmt == FMT_Q6K && w->planar))) {
        const int rc = ckb_launch_gemm_tc_ws(w->fmt == FMT_Q6K, xq, w->fmt == FMT_Q6K ? w->planar : w->w, NULL, y, y_stride, m->c.batch, w->rows, w->cols,
                                             MODEL_GEMM_MIN_BATCH, m->gemm_ws, m->gemm_ws_bytes, st);
        if (rc >= 0) return rc;
    }
    const size_t xrow = fmt_block32(w->fmt) ? (size_t)(w->cols / 32) * 34 : (size_t)(w->cols / 256) * 292;
    for (int b = 0; b < m->c.batch; ++b) {
        const int rc = gemv_q(w->fmt, y + (size_t)b * y_stride, w, xq + b * xrow, st);
        if (rc) return rc;
    }
    return 0;
}

/* h = quantised rmsnorm(x += delta) in the format the consumer `w` wants */
static int norm_quant(CKB200Model *m, const float *delta, const Tensor *gamma, const Tensor *consumer, void *st)
{
    const int B = m->c.batch;
    if (!fmt_block32(consumer->fmt))
        return ckb200_dev_add_rmsnorm_q8k(m->x, delta, (const float *)gamma->w, m->hq, NULL, B, m->D, m->Da, m->c.rms_eps, st);
    if (ckb_tune_get("model_fused_norm_q80", 1))
        return ckb200_dev_add_rmsnorm_q8_0(m->x, delta, (const float *)gamma->w, m->hq, B, m->D, m->Da, consumer->cols, m->c.rms_eps, st);
    /* unfused path through an fp32 row (tune model_fused_norm_q80 = 0) */
    int rc = 0;
    if (delta) rc = ckb200_dev_add_inplace(m->x, delta, (long long)B * m->Da, st);
    if (!rc) rc = ckb200_dev_rmsnorm_forward(m->x, (const float *)gamma->w, m->o, NULL, B, m->D, m->Da, m->c.rms_eps, st);
    if (!rc) {
        /* quantise each row's first `cols` elements */
        for (int b = 0; b < B && !rc; ++b)
            rc = ckb200_dev_quantize_q8_0(m->o + (size_t)b * m->Da, m->hq + (size_t)b * (consumer->cols / 32) * 34, 1, consumer->cols, st);
    }
    return rc;
}

static int quant_rows(const Tensor *consumer, const float *x, int x_stride, uint8_t *out, int rows, void *st)
{
    int rc = 0;
    if (fmt_block32(consumer->fmt)) {
        for (int b = 0; b < rows && !rc; ++b)
            rc = ckb200_dev_quantize_q8_0(x + (size_t)b * x_stride, out + (size_t)b * (consumer->cols / 32) * 34, 1, consumer->cols, st);
    } else if (x_stride == consumer->cols) {
        rc = ckb200_dev_quantize_q8_k(x, out, rows, consumer->cols, st);
    } else {
        for (int b = 0; b < rows && !rc; ++b)
            rc = ckb200_dev_quantize_q8_k(x + (size_t)b * x_stride, out + (size_t)b * (consumer->cols / 256) * 292, 1, consumer->cols, st);
    }
    return rc;
}

static int reduce_partial(CKB200Model *m, float *buf, size_t count, void *st)
{
    if (m->c.tp_size <= 1) return 0;
    if (!m->allreduce) return ckb_fail(CKB_ERR_STATE, "model step: tp_size %d but no all-reduce hook set", m->c.tp_size);
    return m->allreduce(m->allreduce_ctx, buf, count, st);
}

/* norm_quant of a delta that is still a per-rank partial sum (row-parallel o_proj / down_proj): the fused exchange when
 * the hook takes it, else all-reduce in place and the plain kernel */
static int reduce_norm_quant(CKB200Model *m, float *delta, const Tensor *gamma, const Tensor *consumer, void *st)
{
    if (delta && m->c.tp_size > 1) {
        if (m->tp_norm && !fmt_block32(consumer->fmt)) {
            const int rc = m->tp_norm(m->tp_norm_ctx, m->x, delta, (const float *)gamma->w, m->hq, m->c.batch, m->D, m->Da, m->c.rms_eps, st);
            if (rc != -1) return rc;
        }
        const int rc = reduce_partial(m, delta, (size_t)m->c.batch * m->Da, st);
        if (rc) return rc;
    }
    return norm_quant(m, delta, gamma, consumer, st);
}

/* (Re)builds the row-planar copies of the Q6_K and Q5_0 projection matrices from the uploaded rows; outside any capture. */
static int tensor_to_planar(const Tensor *t, void *st)
{
    if (!t->planar) return 0;
    return t->fmt == FMT_Q6K ? ckb200_dev_q6_k_to_planar(t->planar, t->w, t->rows, t->cols, st)
                             : ckb200_dev_q5_0_to_planar(t->planar, t->w, t->rows, t->cols, st);
}

static int ensure_planar(CKB200Model *m, void *st)
{
    if (m->planar_ready || !m->planar_bytes) return 0;
    int rc = 0;
    for (int l = 0; l < m->c.num_layers && !rc; ++l)
        for (int i = 0; i < CKB_T_PER_LAYER && !rc; ++i) rc = tensor_to_planar(&m->layers[l].t[i], st);
    if (!rc) rc = tensor_to_planar(&m->lm_head, st);
    if (rc) return rc;
    if (ckb_check_cuda((int)cudaStreamSynchronize((cudaStream_t)st), "planar weights")) return CKB_ERR_CUDA;
    m->planar_ready = 1;
    return 0;
}

/* ------------------------------------------------------------------ the fused step (one sequence, one GPU)
 *
 * Five launches per layer instead of thirteen (step_fused.cu):
 *   1. q | k | v projections  <- prologue: x += delta, RMSNorm, Q8_K;  epilogue: RoPE, KV-cache store
 *   2. attention over the cache, the split merge done by the last CTA of each kv head
 *   3. o projection            <- prologue: Q8_K of the attention row
 *   4. gate | up projection    <- prologue: x += o, RMSNorm, Q8_K;     epilogue: SwiGLU
 *   5. down projection         <- prologue: Q8_K of the SwiGLU row
 * and the LM head with the final norm in its prologue and the position increment at its end.  The residual row ping-pongs
 * between two buffers: every CTA of a launch reads the old row while the first CTA writes the new one. */

static int fused_fmt(const Tensor *t) { return t->fmt == FMT_Q4K ? SG_FMT_Q4K : (t->fmt == FMT_Q6K && t->planar ? SG_FMT_Q6K_PLANAR : -1); }

static int fused_step_ok(const CKB200Model *m)
{
    if (m->c.batch != 1 || m->c.tp_size != 1 || m->kv_eb != 4 || !ckb_tune_get("model_fused_step", 0)) return 0;
    for (int l = 0; l < m->c.num_layers; ++l) {
        static const int which[6] = { CKB_T_WQ, CKB_T_WK, CKB_T_WV, CKB_T_WO, CKB_T_W1, CKB_T_W2 };
        for (int i = 0; i < 6; ++i)
            if (fused_fmt(&m->layers[l].t[which[i]]) < 0) return 0;
    }
    if (fused_fmt(&m->lm_head) < 0) return 0;
    return m->d % 2 == 0 && m->d / 2 <= 128 && m->Al % 2 == 0 && ckb_step_gemv_ctas_per_sm(m->Da / 256, SG_PRO_GLOBAL, 0) > 0 &&
           ckb_step_gemv_ctas_per_sm(round256(m->Il) / 256, SG_PRO_GLOBAL, 0) > 0 && ckb_step_gemv_ctas_per_sm(m->Ala / 256, SG_PRO_GLOBAL, 0) > 0;
}

static void seg_set(StepSeg *sg, const Tensor *t, float *out, int epi)
{
    sg->fmt = fused_fmt(t);
    sg->W = (const uint8_t *)(sg->fmt == SG_FMT_Q6K_PLANAR ? t->planar : t->w);
    sg->out = out;
    sg->M = t->rows;
    sg->epi = epi;
}

/* Deals the CTAs of the grid to the segments and launches.  In the latency regime (few work items) a segment gets about one
 * CTA per SM of its share of the machine, each with as few busy warps as that allows, and long rows are split over the warps
 * of a CTA so that every warp has one load round; in the streaming regime the resident slots are shared out by bytes. */
static int plan_and_launch(StepGemvParams *p, void *st)
{
    /* matrices of a few megabytes: the launch is a chain of latencies, and the rehearsing instantiation pays */
    double launch_bytes = 0;
    for (int i = 0; i < p->nseg; ++i) launch_bytes += (double)p->seg[i].M * p->nb * (p->seg[i].fmt == SG_FMT_Q6K_PLANAR ? 210 : 144);
    p->dry_run = ckb_tune_get("step_dry_run", 1) && launch_bytes <= (double)ckb_tune_get("step_dry_run_max_mb", 24) * 1048576.0;
    int occ = ckb_step_gemv_ctas_per_sm(p->nb, p->pro, p->dry_run);
    if (occ <= 0) return ckb_fail(CKB_ERR_LIMIT, "fused step: rows of %d superblocks do not fit the kernel's shared memory", p->nb);
    const int occ_cap = ckb_tune_get("step_occ_cap", 0);
    if (occ_cap > 0 && occ_cap < occ) occ = occ_cap;
    const int sms = ckb_sm_count(), cap = sms * occ;
    int g4 = 2;
    while (g4 < 32 && g4 < 2 * p->nb) g4 <<= 1;
    const int g6 = g4 * 2 > 32 ? 32 : g4 * 2;
    long want[3], total_want = 0;
    double bytes[3], total_bytes = 0;
    for (int i = 0; i < p->nseg; ++i) {
        bytes[i] = (double)p->seg[i].M * p->nb * (p->seg[i].fmt == SG_FMT_Q6K_PLANAR ? 210 : 144);
        total_bytes += bytes[i];
    }
    for (int i = 0; i < p->nseg; ++i) {
        StepSeg *sg = &p->seg[i];
        const int q6 = sg->fmt == SG_FMT_Q6K_PLANAR;
        const int rpw = (32 / (q6 ? g6 : g4)) * 2;
        const long items = (sg->M + rpw - 1) / rpw;
        const int passes = ckb_step_gemv_passes(p->nb, sg->fmt);
        long share = (long)((double)sms * bytes[i] / total_bytes + 0.5);       /* SMs of this segment at one CTA per SM */
        if (share < 1) share = 1;
        sg->split = passes > 1 && passes <= 8 && items * passes <= (long)cap * 8 && ckb_tune_get("step_split", 1);
        if (sg->split) {
            const int ipc = 8 / passes;
            want[i] = (items + ipc - 1) / ipc;                                   /* one round per CTA */
        } else {
            long wpc = (items + share - 1) / share;                              /* busy warps per CTA */
            if (wpc > 8) wpc = 8;
            want[i] = (items + wpc - 1) / wpc;
        }
        total_want += want[i];
    }
    int grid = 0;
    for (int i = 0; i < p->nseg; ++i) {
        long n = want[i];
        if (total_want > cap) {
            n = (long)((double)cap * bytes[i] / total_bytes);
            if (n < 1) n = 1;
            if (n > want[i]) n = want[i];
        }
        p->seg[i].cta0 = grid;
        p->seg[i].ncta = (int)n;
        grid += (int)n;
    }
    const int rc = ckb_launch_step_gemv(p, grid, st);
    return rc == -1 ? ckb_fail(CKB_ERR_SHAPE, "fused step: shape not handled") : rc;
}

/* The quantised input of a fused launch: built inside the launch when the row is short (every CTA repeats the work, which is
 * cheaper than a launch), else by the stand-alone kernel into `xq_buf`.  kind: SG_PRO_NORM (x row `cur` += delta, in place
 * when stand-alone, else into `nxt`) or SG_PRO_QUANT (fp32 row `src`).  Returns 1 when the residual row moved to `nxt`. */
static int fused_input(CKB200Model *m, StepGemvParams *p, int kind, float *cur, float *nxt, const float *delta, const float *gamma, const float *src,
                       uint8_t *xq_buf, void *st, int *rc)
{
    *rc = 0;
    if (kind == SG_PRO_NORM) {
        if (p->nb <= SG_NORM_MAX_NB && p->nb <= ckb_tune_get("step_norm_max_nb", SG_NORM_MAX_NB)) {
            p->pro = SG_PRO_NORM;
            p->x_in = cur;
            p->delta = delta;
            p->gamma = gamma;
            p->x_out = delta ? nxt : NULL;
            return delta != NULL;
        }
        *rc = ckb200_dev_add_rmsnorm_q8k(cur, delta, gamma, xq_buf, NULL, 1, m->D, m->Da, m->c.rms_eps, st);
    } else {
        if (p->nb <= ckb_tune_get("step_quant_max_nb", 8)) {       /* one block per warp: beyond that the blocks of a warp queue up */
            p->pro = SG_PRO_QUANT;
            p->src = src;
            return 0;
        }
        *rc = ckb200_dev_quantize_q8_k(src, xq_buf, 1, p->nb * 256, st);
    }
    p->pro = SG_PRO_GLOBAL;
    p->xq = xq_buf;
    return 0;
}

static int issue_step_fused(CKB200Model *m, void *st)
{
    const CKB200ModelConfig *c = &m->c;
    const int L = c->num_layers;
    int rc;
    rc = ckb200_dev_embedding_rows(m->tokens_dev, 1, c->vocab_size, m->emb.w, m->emb.fmt, m->emb.cols, m->x, m->Da, m->D, st);
    if (rc) return rc;
    float *cur = m->x, *nxt = m->x2;
    const float *delta = NULL;
    StepGemvParams base;
    memset(&base, 0, sizeof base);
    base.cos_cache = m->rope_cos;
    base.sin_cache = m->rope_sin;
    base.pos = m->pos_dev;
    base.head_dim = m->d;
    base.max_seq = c->max_seq_len;
    base.d_model = m->D;
    base.eps = c->rms_eps;
    for (int l = 0; l < L; ++l) {
        Tensor *t = m->layers[l].t;
        float *kc = (float *)kv_at(m, l, 0), *vc = (float *)kv_at(m, l, 1);
        StepGemvParams p = base;
        /* 1: q | k | v */
        p.nseg = 3;
        p.nb = m->Da / 256;
        int moved = fused_input(m, &p, SG_PRO_NORM, cur, nxt, delta, (const float *)t[CKB_T_LN1].w, NULL, m->hq, st, &rc);
        if (rc) return rc;
        seg_set(&p.seg[0], &t[CKB_T_WQ], m->q, SG_EPI_ROPE_Q);
        seg_set(&p.seg[1], &t[CKB_T_WK], kc, SG_EPI_ROPE_K);
        seg_set(&p.seg[2], &t[CKB_T_WV], vc, SG_EPI_STORE_V);
        if ((rc = plan_and_launch(&p, st))) return rc;
        if (moved) { float *tmp = cur; cur = nxt; nxt = tmp; }
        /* 2: attention, merge inside */
        ckb_attn_hint_early_rows(ckb_tune_get("model_attn_early_rows", 1));
        if ((rc = ckb200_dev_attention_decode_fused(m->q, kc, vc, m->att, m->Ala, 1, m->kv_batch_stride, m->Hl, m->Hkvl, 1, c->max_seq_len, m->d, m->d,
                                                    m->attn_splits, m->attn_scratch, m->attn_counters, m->pos_dev, NULL, 0, st))) return rc;
        ckb_attn_hint_early_rows(0);
        /* 3: o projection */
        p = base;
        p.nseg = 1;
        p.nb = m->Ala / 256;
        fused_input(m, &p, SG_PRO_QUANT, NULL, NULL, NULL, NULL, m->att, m->aq, st, &rc);
        if (rc) return rc;
        seg_set(&p.seg[0], &t[CKB_T_WO], m->o, SG_EPI_STORE);
        if ((rc = plan_and_launch(&p, st))) return rc;
        /* 4: gate | up with SwiGLU */
        p = base;
        p.nseg = 1;
        p.nb = m->Da / 256;
        moved = fused_input(m, &p, SG_PRO_NORM, cur, nxt, m->o, (const float *)t[CKB_T_LN2].w, NULL, m->hq, st, &rc);
        if (rc) return rc;
        seg_set(&p.seg[0], &t[CKB_T_W1], m->mf, SG_EPI_SWIGLU);
        if ((rc = plan_and_launch(&p, st))) return rc;
        if (moved) { float *tmp = cur; cur = nxt; nxt = tmp; }
        /* 5: down projection */
        p = base;
        p.nseg = 1;
        p.nb = round256(m->Il) / 256;
        fused_input(m, &p, SG_PRO_QUANT, NULL, NULL, NULL, NULL, m->mf, m->mq, st, &rc);
        if (rc) return rc;
        seg_set(&p.seg[0], &t[CKB_T_W2], m->prev, SG_EPI_STORE);
        if ((rc = plan_and_launch(&p, st))) return rc;
        delta = m->prev;
    }
    StepGemvParams p = base;
    p.nseg = 1;
    p.nb = m->Da / 256;
    fused_input(m, &p, SG_PRO_NORM, cur, nxt, delta, (const float *)m->final_gamma.w, NULL, m->hq, st, &rc);
    if (rc) return rc;
    p.x_out = NULL;
    p.pos_advance = m->pos_dev;
    seg_set(&p.seg[0], &m->lm_head, m->logits, SG_EPI_STORE);
    return plan_and_launch(&p, st);
}

static int issue_step(CKB200Model *m, void *st)
{
    if (fused_step_ok(m)) return issue_step_fused(m, st);
    const CKB200ModelConfig *c = &m->c;
    const int B = c->batch, L = c->num_layers;
    int rc;
    /* embedding of the B current tokens -> x */
    rc = ckb200_dev_embedding_rows(m->tokens_dev, B, c->vocab_size, m->emb.w, m->emb.fmt, m->emb.cols, m->x, m->Da, m->D, st);
    if (rc) return rc;
    float *delta = NULL;
    for (int l = 0; l < L; ++l) {
        Tensor *t = m->layers[l].t;
        void *kc = kv_at(m, l, 0), *vc = kv_at(m, l, 1);
        if ((rc = reduce_norm_quant(m, delta, &t[CKB_T_LN1], &t[CKB_T_WQ], st))) return rc;
        if (fmt_block32(t[CKB_T_WK].fmt) != fmt_block32(t[CKB_T_WQ].fmt) || fmt_block32(t[CKB_T_WV].fmt) != fmt_block32(t[CKB_T_WQ].fmt))
            return ckb_fail(CKB_ERR_STATE, "model step: q/k/v must share the activation format (all K-quant or all Q8_0)");
        /* q, k and v side by side, unless one of them is a batched product on the tcgen05 kernel: those share one workspace */
        if (ckb_tune_get("model_qkv_streams", 1) && matvec_standalone(m, &t[CKB_T_WQ], m->hq) && matvec_standalone(m, &t[CKB_T_WK], m->hq) &&
            matvec_standalone(m, &t[CKB_T_WV], m->hq)) {
            cudaStream_t main_st = (cudaStream_t)st;
            if (ckb_check_cuda((int)cudaEventRecord(m->ev_fork, main_st), "fork")) return CKB_ERR_CUDA;
            if ((rc = matvec(m, &t[CKB_T_WQ], m->hq, m->q, m->Al, st))) return rc;
            for (int i = 0; i < 2; ++i) {
                if (ckb_check_cuda((int)cudaStreamWaitEvent(m->side[i], m->ev_fork, 0), "fork wait")) return CKB_ERR_CUDA;
                if ((rc = matvec(m, &t[i ? CKB_T_WV : CKB_T_WK], m->hq, i ? m->v : m->k, m->Hkvl * m->d, m->side[i]))) return rc;
                if (ckb_check_cuda((int)cudaEventRecord(m->ev_join[i], m->side[i]), "join")) return CKB_ERR_CUDA;
                if (ckb_check_cuda((int)cudaStreamWaitEvent(main_st, m->ev_join[i], 0), "join wait")) return CKB_ERR_CUDA;
            }
        } else {
            if ((rc = matvec(m, &t[CKB_T_WQ], m->hq, m->q, m->Al, st))) return rc;
            if ((rc = matvec(m, &t[CKB_T_WK], m->hq, m->k, m->Hkvl * m->d, st))) return rc;
            if ((rc = matvec(m, &t[CKB_T_WV], m->hq, m->v, m->Hkvl * m->d, st))) return rc;
        }
        if (m->kv_eb == 2) {
            /* fp16 caches: the rotation stays fp32, k and v are rounded once on the store, attention widens them again */
            if ((rc = ckb200_dev_rope_kv_store_f16(m->q, m->k, m->v, (uint16_t *)kc, (uint16_t *)vc, m->rope_cos, m->rope_sin, m->pos_dev, B, m->Hl,
                                                   m->Hkvl, m->d, c->max_seq_len, m->kv_batch_stride, st))) return rc;
            if ((rc = ckb200_dev_attention_decode_f16cache_ws(m->q, (const uint16_t *)kc, (const uint16_t *)vc, m->att, B, m->kv_batch_stride, m->Hl,
                                                              m->Hkvl, 1, c->max_seq_len, m->d, m->d, m->attn_splits, m->attn_scratch, m->pos_dev, st)))
                return rc;
            goto attention_done;
        }
        if ((rc = ckb200_dev_rope_kv_store(m->q, m->k, m->v, (float *)kc, (float *)vc, m->rope_cos, m->rope_sin, m->pos_dev, B, m->Hl, m->Hkvl, m->d,
                                           c->max_seq_len, m->kv_batch_stride, st))) return rc;
        /* attention rows are contiguous [B][Al]; with B == 1 the row sits in an Ala-wide buffer whose tail stays zero.
         * Attention, split merge and quantisation stay three launches: chained with programmatic dependent launch inside
         * the step's graph they measured faster than the single-launch form (ckb200_dev_attention_decode_fused), whose
         * merge and quantise tails run serially in the last CTAs. */
        ckb_attn_hint_early_rows(ckb_tune_get("model_attn_early_rows", 1));
        if (ckb_tune_get("model_attn_cluster", 0)) {
            /* one launch: the CTAs of a kv head form a thread-block cluster and merge their partial results in distributed shared memory */
            if ((rc = ckb200_dev_attention_decode_fused(m->q, (const float *)kc, (const float *)vc, m->att, B == 1 ? m->Ala : m->Al, B, m->kv_batch_stride,
                                                        m->Hl, m->Hkvl, 1, c->max_seq_len, m->d, m->d, m->attn_splits, m->attn_scratch, m->attn_counters,
                                                        m->pos_dev, NULL, 0, st))) return rc;
        } else if ((rc = ckb200_dev_attention_decode_ws(m->q, (const float *)kc, (const float *)vc, m->att, B, m->kv_batch_stride, m->Hl, m->Hkvl, 1,
                                                        c->max_seq_len, m->d, m->d, m->attn_splits, m->attn_scratch, m->pos_dev, st))) return rc;
    attention_done:
        ckb_attn_hint_early_rows(0);
        if ((rc = quant_rows(&t[CKB_T_WO], m->att, m->Ala, m->aq, B, st))) return rc;
        if ((rc = matvec(m, &t[CKB_T_WO], m->aq, m->o, m->Da, st))) return rc;
        if ((rc = reduce_norm_quant(m, m->o, &t[CKB_T_LN2], &t[CKB_T_W1], st))) return rc;
        if ((rc = matvec(m, &t[CKB_T_W1], m->hq, m->gu, 2 * m->Il, st))) return rc;
        if (!fmt_block32(t[CKB_T_W2].fmt) && m->Il % 256 == 0) {
            if ((rc = ckb200_dev_swiglu_q8k(m->gu, m->mq, B, m->Il, st))) return rc;
        } else {
            /* swiglu to fp32 (reusing the front of gu is not safe: separate rows), then quantise */
            return ckb_fail(CKB_ERR_STATE, "model step: FFN width %d with this down-projection format is not supported", m->Il);
        }
        if ((rc = matvec(m, &t[CKB_T_W2], m->mq, m->prev, m->Da, st))) return rc;
        delta = m->prev;                         /* a per-rank partial sum when tp_size > 1: reduced where it is consumed */
    }
    if ((rc = reduce_norm_quant(m, delta, &m->final_gamma, &m->lm_head, st))) return rc;
    if ((rc = matvec(m, &m->lm_head, m->hq, m->logits, m->Vl, st))) return rc;
    return ckb200_dev_advance_pos(m->pos_dev, st);
}

int ckb200_model_decode(CKB200Model *m, const int32_t *tokens, float *logits_host)
{
    if (!m || !tokens) return ckb_fail(CKB_ERR_STATE, "model_decode: NULL model or tokens");
    if (m->host_pos >= m->c.max_seq_len)
        return ckb_fail(CKB_ERR_LIMIT, "model_decode: position %d is past the context of %d tokens (reset or set_pos first)", m->host_pos, m->c.max_seq_len);
    cudaStream_t st = ckb_stream(NULL);
    const int B = m->c.batch;
    /* a call without logits_host returns while its step is still queued: the pinned staging buffer may only be reused once the
     * copy out of it has run */
    if (m->tokens_in_flight && ckb_check_cuda((int)cudaEventSynchronize(m->ev_tokens), "tokens staging")) return CKB_ERR_CUDA;
    memcpy(m->tokens_pinned, tokens, (size_t)B * sizeof(int32_t));
    if (ckb_check_cuda((int)cudaMemcpyAsync(m->tokens_dev, m->tokens_pinned, (size_t)B * sizeof(int32_t), cudaMemcpyHostToDevice, st), "tokens H2D")) return CKB_ERR_CUDA;
    if (ckb_check_cuda((int)cudaEventRecord(m->ev_tokens, st), "tokens event")) return CKB_ERR_CUDA;
    m->tokens_in_flight = 1;
    { const int rc = ensure_planar(m, st); if (rc) return rc; }
    const int use_graph = ckb_tune_get("model_graph", 1);
    if (use_graph && !m->graph_ready) {
        /* one eager step first: it sets per-kernel attributes (not allowed while capturing) and is rolled back */
        int32_t pos0 = 0;
        cudaMemcpyAsync(&pos0, m->pos_dev, sizeof pos0, cudaMemcpyDeviceToHost, st);
        cudaStreamSynchronize(st);
        int rc = issue_step(m, st);
        if (rc) return rc;
        cudaMemcpyAsync(m->pos_dev, &pos0, sizeof pos0, cudaMemcpyHostToDevice, st);
        if (ckb_check_cuda((int)cudaStreamSynchronize(st), "warm-up step")) return CKB_ERR_CUDA;
        cudaGraph_t g = NULL;
        if (ckb_check_cuda((int)cudaStreamBeginCapture(st, cudaStreamCaptureModeThreadLocal), "begin capture")) return CKB_ERR_CUDA;
        rc = issue_step(m, st);
        const cudaError_t e = cudaStreamEndCapture(st, &g);
        if (rc || e != cudaSuccess || !g) {
            if (g) cudaGraphDestroy(g);
            return rc ? rc : ckb_check_cuda((int)e, "end capture");
        }
        const cudaError_t ei = cudaGraphInstantiate(&m->graph, g, 0);
        cudaGraphDestroy(g);
        if (ckb_check_cuda((int)ei, "graph instantiate")) return CKB_ERR_CUDA;
        m->graph_ready = 1;
    }
    if (use_graph) {
        if (ckb_check_cuda((int)cudaGraphLaunch(m->graph, st), "graph launch")) return CKB_ERR_CUDA;
    } else {
        const int rc = issue_step(m, st);
        if (rc) return rc;
    }
    m->host_pos += 1;
    if (logits_host) {
        if (ckb_check_cuda((int)cudaMemcpyAsync(logits_host, m->logits, (size_t)B * m->Vl * sizeof(float), cudaMemcpyDeviceToHost, st), "logits D2H")) return CKB_ERR_CUDA;
        return ckb_sync_check(st, "model_decode");        /* a timed-out exchange must not come back as rc 0 with stale logits */
    }
    return 0;
}

/* ------------------------------------------------------------------ batched prefill
 *
 * A prompt of T tokens as ONE pass (the reference's generated ck_prefill, version/v7/scripts/codegen_prefill_v7.py:194-208): per
 * layer the T rows are normalised and quantised together, every projection is one quantised GEMM on the tensor cores (the
 * weights are read once for all tokens), RoPE and the KV-cache fill run over all tokens, attention is the causal prefill
 * kernel.  Only the last token's logits are produced.  Used from an empty cache (position 0) by one sequence on one GPU with
 * K-quant projections; every other case (and prompts shorter than 16 tokens) falls back to T decode steps. */

int ckb_launch_gemm_tc(int wf, const void *A_q8, const void *B, const float *bias, float *C, int ldc, int M, int N, int K, int min_tokens, void *stream);

void ckb_gemm_tc_hint_same_activations(int on);              /* gemm_tc.cu */

static int prefill_ok(const CKB200Model *m, int T)
{
    if (m->c.batch != 1 || m->c.tp_size != 1 || m->kv_eb != 4 || T < 16 || m->host_pos != 0 || T > m->c.max_seq_len || !ckb_tune_get("model_prefill", 1)) return 0;
    for (int l = 0; l < m->c.num_layers; ++l) {
        static const int which[6] = { CKB_T_WQ, CKB_T_WK, CKB_T_WV, CKB_T_WO, CKB_T_W1, CKB_T_W2 };
        for (int i = 0; i < 6; ++i) {
            const Tensor *t = &m->layers[l].t[which[i]];
            if (!(t->fmt == FMT_Q4K || (t->fmt == FMT_Q6K && t->planar))) return 0;
        }
    }
    const int group = m->Hl / m->Hkvl;
    return m->Il % 256 == 0 && m->d % 8 == 0 && (m->d == 64 || m->d == 128) && group <= 8 && m->Hl % m->Hkvl == 0;
}

static int prefill_buffers(CKB200Model *m, int T)
{
    if (T <= m->pf_tokens) return 0;
    cudaStreamSynchronize(ckb_stream(NULL));
    void **ptrs[] = { (void **)&m->pf_x, (void **)&m->pf_delta, (void **)&m->pf_o, (void **)&m->pf_q, (void **)&m->pf_k, (void **)&m->pf_v, (void **)&m->pf_qh,
                      (void **)&m->pf_oh, (void **)&m->pf_gu, (void **)&m->pf_hq, (void **)&m->pf_aq, (void **)&m->pf_mq };
    for (unsigned i = 0; i < sizeof ptrs / sizeof ptrs[0]; ++i) { if (*ptrs[i]) cudaFree(*ptrs[i]); *ptrs[i] = NULL; }
    m->pf_tokens = 0;
    const size_t t = (size_t)T, kvw = (size_t)m->Hkvl * m->d;
    const size_t sizes[] = { t * m->Da * 4, t * m->Da * 4, t * m->Da * 4, t * m->Al * 4, t * kvw * 4, t * kvw * 4, t * m->Al * 4, t * m->Al * 4, t * 2 * m->Il * 4,
                             t * (m->Da / 256) * 292, t * (m->Ala / 256) * 292, t * (m->Il / 256) * 292 };
    for (unsigned i = 0; i < sizeof ptrs / sizeof ptrs[0]; ++i)
        if (ckb_check_cuda((int)cudaMalloc(ptrs[i], sizes[i] + 256), "cudaMalloc(prefill)")) return CKB_ERR_CUDA;
    /* rows wider than the data (Da > D) keep a zero tail: the GEMMs write only the first D columns */
    cudaMemsetAsync(m->pf_delta, 0, sizes[1], ckb_stream(NULL));
    cudaMemsetAsync(m->pf_o, 0, sizes[2], ckb_stream(NULL));
    m->pf_tokens = T;
    return 0;
}

static int prefill_gemm(const Tensor *w, const uint8_t *xq, float *y, int ldc, int T, void *st)
{
    const int rc = ckb_launch_gemm_tc(w->fmt == FMT_Q6K, xq, w->fmt == FMT_Q6K ? w->planar : w->w, NULL, y, ldc, T, w->rows, w->cols, 16, st);
    return rc == -1 ? ckb_fail(CKB_ERR_SHAPE, "prefill: projection %d x %d not handled by the tensor-core GEMM", w->rows, w->cols) : rc;
}

static int issue_prefill(CKB200Model *m, int T, void *st)
{
    const CKB200ModelConfig *c = &m->c;
    const int L = c->num_layers, kvw = m->Hkvl * m->d;
    int rc;
    rc = ckb200_dev_embedding_rows(m->tokens_dev, T, c->vocab_size, m->emb.w, m->emb.fmt, m->emb.cols, m->pf_x, m->Da, m->D, st);
    if (rc) return rc;
    const float *delta = NULL;
    for (int l = 0; l < L; ++l) {
        Tensor *t = m->layers[l].t;
        float *kc = (float *)kv_at(m, l, 0), *vc = (float *)kv_at(m, l, 1);
        if ((rc = ckb200_dev_add_rmsnorm_q8k(m->pf_x, delta, (const float *)t[CKB_T_LN1].w, m->pf_hq, NULL, T, m->D, m->Da, c->rms_eps, st))) return rc;
        if ((rc = prefill_gemm(&t[CKB_T_WQ], m->pf_hq, m->pf_q, m->Al, T, st))) return rc;
        ckb_gemm_tc_hint_same_activations(1);                  /* k and v read the rows q read: one set of operand tiles */
        rc = prefill_gemm(&t[CKB_T_WK], m->pf_hq, m->pf_k, kvw, T, st);
        if (!rc) rc = prefill_gemm(&t[CKB_T_WV], m->pf_hq, m->pf_v, kvw, T, st);
        ckb_gemm_tc_hint_same_activations(0);
        if (rc) return rc;
        if ((rc = ckb200_dev_prefill_rope_scatter(m->pf_q, m->pf_k, m->pf_v, m->pf_qh, kc, vc, m->rope_cos, m->rope_sin, T, m->Hl, m->Hkvl, m->d, c->max_seq_len, 0, st))) return rc;
        if ((rc = ckb200_dev_attention_prefill(m->pf_qh, kc, vc, m->pf_oh, m->Hl, m->Hkvl, T, m->d, m->d, c->max_seq_len, 1, st))) return rc;
        if ((rc = ckb200_dev_prefill_gather_q8k(m->pf_oh, m->pf_aq, T, m->Hl, m->d, m->Ala, st))) return rc;
        if ((rc = prefill_gemm(&t[CKB_T_WO], m->pf_aq, m->pf_o, m->Da, T, st))) return rc;
        if ((rc = ckb200_dev_add_rmsnorm_q8k(m->pf_x, m->pf_o, (const float *)t[CKB_T_LN2].w, m->pf_hq, NULL, T, m->D, m->Da, c->rms_eps, st))) return rc;
        if ((rc = prefill_gemm(&t[CKB_T_W1], m->pf_hq, m->pf_gu, 2 * m->Il, T, st))) return rc;
        if ((rc = ckb200_dev_swiglu_q8k(m->pf_gu, m->pf_mq, T, m->Il, st))) return rc;
        if ((rc = prefill_gemm(&t[CKB_T_W2], m->pf_mq, m->pf_delta, m->Da, T, st))) return rc;
        delta = m->pf_delta;
    }
    /* logits of the last token only: its residual row, final norm, LM head as a GEMV */
    const size_t last = (size_t)(T - 1) * m->Da;
    if ((rc = ckb200_dev_add_rmsnorm_q8k(m->pf_x + last, delta ? delta + last : NULL, (const float *)m->final_gamma.w, m->hq, NULL, 1, m->D, m->Da, c->rms_eps, st))) return rc;
    return matvec(m, &m->lm_head, m->hq, m->logits, m->Vl, st);
}

int ckb200_model_prefill(CKB200Model *m, const int32_t *tokens, int count, float *logits_host)
{
    if (!m || !tokens || count <= 0) return ckb_fail(CKB_ERR_STATE, "model_prefill: NULL model or tokens");
    if (m->host_pos + count > m->c.max_seq_len)
        return ckb_fail(CKB_ERR_LIMIT, "model_prefill: %d tokens from position %d run past the context of %d tokens", count, m->host_pos, m->c.max_seq_len);
    cudaStream_t st = ckb_stream(NULL);
    { const int rc = ensure_planar(m, st); if (rc) return rc; }
    if (!prefill_ok(m, count)) {
        for (int i = 0; i < count; ++i) {
            const int rc = ckb200_model_decode(m, tokens + i, i == count - 1 ? logits_host : NULL);
            if (rc) return rc;
        }
        return 0;
    }
    if (prefill_buffers(m, count)) return CKB_ERR_CUDA;
    int32_t *ids = NULL;
    if (ckb_check_cuda((int)cudaMalloc((void **)&ids, (size_t)count * sizeof(int32_t)), "cudaMalloc(prompt ids)")) return CKB_ERR_CUDA;
    int rc = ckb_check_cuda((int)cudaMemcpyAsync(ids, tokens, (size_t)count * sizeof(int32_t), cudaMemcpyHostToDevice, st), "prompt ids H2D");
    int32_t *saved = m->tokens_dev;
    m->tokens_dev = ids;
    if (!rc) rc = issue_prefill(m, count, st);
    m->tokens_dev = saved;
    if (!rc) {
        const int32_t p = count;
        rc = ckb_check_cuda((int)cudaMemcpyAsync(m->pos_dev, &p, sizeof p, cudaMemcpyHostToDevice, st), "prefill pos");
    }
    if (!rc && logits_host) rc = ckb_check_cuda((int)cudaMemcpyAsync(logits_host, m->logits, (size_t)m->Vl * sizeof(float), cudaMemcpyDeviceToHost, st), "logits D2H");
    if (!rc) rc = ckb_sync_check(st, "model_prefill");
    cudaFree(ids);
    if (!rc) m->host_pos = count;
    return rc;
}

/* Enqueue `steps` decode steps that keep feeding the same token ids (benchmark loop; no host sync). */
int ckb200_model_decode_repeat(CKB200Model *m, int steps)
{
    if (!m || !m->graph_ready) return ckb_fail(CKB_ERR_STATE, "model_decode_repeat: run model_decode once first");
    if (steps > m->c.max_seq_len - m->host_pos)
        return ckb_fail(CKB_ERR_LIMIT, "model_decode_repeat: %d steps from position %d run past the context of %d tokens", steps, m->host_pos, m->c.max_seq_len);
    cudaStream_t st = ckb_stream(NULL);
    for (int i = 0; i < steps; ++i)
        if (ckb_check_cuda((int)cudaGraphLaunch(m->graph, st), "graph launch")) return CKB_ERR_CUDA;
    m->host_pos += steps;
    return 0;
}

size_t ckb200_model_weight_bytes(CKB200Model *m)
{
    if (!m) return 0;
    size_t s = 0;
    for (int l = 0; l < m->c.num_layers; ++l)
        for (int i = 0; i < CKB_T_PER_LAYER; ++i)
            if (m->layers[l].t[i].fmt >= 0) s += m->layers[l].t[i].bytes;
    return s + m->lm_head.bytes;
}

/* ------------------------------------------------------------------ model sources
 *
 * ckb200_model_open(spec, batch):
 *   "synthetic:<shape>[:seed]"  a named model SHAPE with device-generated random weights
 *                               (qwen2-0.5b, llama3-8b, llama3-70b, mini); for benchmarks and smoke runs
 *   "<path>"                    a BUMPWGT5 file of the reference's converter (bump_loader.c; its sidecar map is looked for
 *                               beside it), or a file in the container format below (what tests write)
 *
 * File: magic "CKB2MDL1", u32 version = 1, the config (8 ints, 2 floats, 12 ints as in CKB200ModelConfig),
 * then the tensors in canonical order - per layer ln1, wq, wk, wv, wo, ln2, w1, w2; final gamma; LM head;
 * embedding table unless tied - each as u64 byte count followed by the bytes (block formats as in the
 * reference, fp32 for the norm weights). */

static const struct { const char *name; CKB200ModelConfig cfg; } g_presets[] = {
    { "qwen2-0.5b", { 896, 14, 2, 64, 4864, 24, 151936, 2048, 1e-6f, 1.0e6f, 0, 0, 1, 0, 0, 1, 1, 1, 1, 1, 0, 1 } },
    { "llama3-8b", { 4096, 32, 8, 128, 14336, 32, 128256, 4352, 1e-5f, 5.0e5f, 0, 0, 1, 0, 0, 1, 1, 1, 1, 1, 0, 1 } },
    { "llama3-70b", { 8192, 64, 8, 128, 28672, 80, 128256, 4352, 1e-5f, 5.0e5f, 0, 0, 1, 0, 0, 1, 1, 1, 1, 1, 0, 1 } },
    { "mini", { 384, 6, 2, 64, 768, 3, 1000, 128, 1e-6f, 1.0e6f, 0, 0, 1, 0, 0, 1, 1, 1, 1, 1, 0, 1 } },
};

static int read_exact(FILE *f, void *dst, size_t n) { return fread(dst, 1, n, f) == n ? 0 : -1; }

static CKB200Model *open_file(const char *path, int batch)
{
    FILE *f = fopen(path, "rb");
    if (!f) { ckb_fail(CKB_ERR_STATE, "model_open: cannot open %s", path); return NULL; }
    char magic[8];
    uint32_t version = 0;
    CKB200ModelConfig cfg;
    CKB200Model *m = NULL;
    void *buf = NULL;
    size_t cap = 0;
    if (read_exact(f, magic, 8) || memcmp(magic, "CKB2MDL1", 8) || read_exact(f, &version, 4) || version != 1 || read_exact(f, &cfg, sizeof cfg)) {
        ckb_fail(CKB_ERR_STATE, "model_open: %s is not a CKB2MDL1 file", path);
        goto done;
    }
    if (batch > 0) cfg.batch = batch;
    m = ckb200_model_create(&cfg);
    if (!m) goto done;
    const int L = cfg.num_layers;
    for (int i = 0; i < L * CKB_T_PER_LAYER + 2 + (cfg.tie_embeddings ? 0 : 1); ++i) {
        const int layer = i < L * CKB_T_PER_LAYER ? i / CKB_T_PER_LAYER : -1;
        const int which = layer >= 0 ? i % CKB_T_PER_LAYER : CKB_T_FINAL_GAMMA + (i - L * CKB_T_PER_LAYER);
        uint64_t n = 0;
        if (read_exact(f, &n, 8) || n != ckb200_model_tensor_bytes(m, layer, which)) {
            ckb_fail(CKB_ERR_SHAPE, "model_open: tensor (%d, %d) of %s has %llu bytes, expected %zu", layer, which, path,
                     (unsigned long long)n, ckb200_model_tensor_bytes(m, layer, which));
            ckb200_model_free(m);
            m = NULL;
            goto done;
        }
        if (n > cap) { free(buf); buf = malloc(n); cap = n; }
        if (!buf || read_exact(f, buf, n) || ckb200_model_upload_tensor(m, layer, which, buf, n)) {
            ckb_fail(CKB_ERR_STATE, "model_open: short read in %s", path);
            ckb200_model_free(m);
            m = NULL;
            goto done;
        }
    }
done:
    free(buf);
    fclose(f);
    return m;
}

CKB200Model *ckb200_model_open(const char *spec, int batch)
{
    if (!spec) { ckb_fail(CKB_ERR_STATE, "model_open: NULL spec"); return NULL; }
    if (strncmp(spec, "synthetic:", 10) != 0) {
        /* the reference's own weight file (BUMPWGT5 + sidecar map beside it) or this library's container */
        char magic[8] = { 0 };
        FILE *f = fopen(spec, "rb");
        if (f) { if (fread(magic, 1, 8, f) != 8) magic[0] = 0; fclose(f); }
        if (!memcmp(magic, "BUMPWGT5", 8)) return ckb200_model_open_bump(spec, NULL, batch);
        return open_file(spec, batch);
    }
    char name[64];
    unsigned long long seed = 1;
    const char *p = spec + 10, *colon = strchr(p, ':');
    size_t n = colon ? (size_t)(colon - p) : strlen(p);
    if (n >= sizeof name) n = sizeof name - 1;
    memcpy(name, p, n);
    name[n] = 0;
    if (colon) seed = strtoull(colon + 1, NULL, 10);
    for (size_t i = 0; i < sizeof g_presets / sizeof g_presets[0]; ++i)
        if (!strcmp(g_presets[i].name, name)) {
            CKB200ModelConfig cfg = g_presets[i].cfg;
            if (batch > 0) cfg.batch = batch;
            CKB200Model *m = ckb200_model_create(&cfg);
            if (m && ckb200_model_fill_synthetic(m, seed)) { ckb200_model_free(m); m = NULL; }
            return m;
        }
    ckb_fail(CKB_ERR_STATE, "model_open: unknown synthetic shape '%s'", name);
    return NULL;
}

const CKB200ModelConfig *ckb200_model_config(CKB200Model *m) { return m ? &m->c : NULL; }

int ckb200_model_reset(CKB200Model *m)
{
    if (!m) return CKB_ERR_STATE;
    cudaStream_t st = ckb_stream(NULL);
    cudaMemsetAsync(m->kv, 0, kv_bytes(m), st);
    return ckb200_model_set_pos(m, 0);
}
