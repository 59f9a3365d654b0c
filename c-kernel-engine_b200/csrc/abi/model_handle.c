/* libckb200_model_api.so - the handle-based model ABI of the reference's include/ck_model_api.h:56-113
 * (emitted by the v6.5/v6.6 codegen, used by src/v6.6/test_generic_api.c:247-282): ck_model_get_config,
 * ck_model_create, ck_model_precompute_rope, ck_model_load_weights, ck_model_forward, ck_model_decode,
 * ck_model_get_logits, ck_model_verify_canaries, ck_model_get_base, ck_model_get_total_bytes, ck_model_free.
 *
 * The generated library has its model compiled in; here the model spec comes from the environment
 * variable CKB200_MODEL (default "synthetic:mini") or from the path given to ck_model_load_weights().
 */
#include <stdint.h>
#include <math.h>
#include <stdlib.h>
#include <string.h>

#include "../../../include/ckb200.h"
#include "../../../include/ckb200_model.h"

#define CK_EXPORT __attribute__((visibility("default")))

typedef struct {          /* include/ck_model_api.h:26-40 */
    int embed_dim, num_heads, num_kv_heads, head_dim, intermediate_size, num_layers, vocab_size, max_seq_len;
    size_t total_bytes, weight_bytes, activation_bytes;
    const char *model_name, *model_family;
} CKModelConfig;

typedef struct {
    CKB200Model *m;
    float *logits;
} Handle;

static CKModelConfig g_cfg;
static char g_name[128];

static const char *spec_from_env(void)
{
    const char *s = getenv("CKB200_MODEL");
    return s && *s ? s : "synthetic:mini";
}

static void fill_config(CKB200Model *m)
{
    const CKB200ModelConfig *c = ckb200_model_config(m);
    g_cfg.embed_dim = c->embed_dim; g_cfg.num_heads = c->num_heads; g_cfg.num_kv_heads = c->num_kv_heads; g_cfg.head_dim = c->head_dim;
    g_cfg.intermediate_size = c->intermediate_size; g_cfg.num_layers = c->num_layers; g_cfg.vocab_size = c->vocab_size;
    g_cfg.max_seq_len = c->max_seq_len;
    g_cfg.weight_bytes = ckb200_model_weight_bytes(m);
    g_cfg.activation_bytes = 0;
    g_cfg.total_bytes = g_cfg.weight_bytes;
    strncpy(g_name, spec_from_env(), sizeof g_name - 1);
    g_cfg.model_name = g_name;
    g_cfg.model_family = "llama";
}

CK_EXPORT const CKModelConfig *ck_model_get_config(void) { return &g_cfg; }

CK_EXPORT void *ck_model_create(void)
{
    Handle *h = (Handle *)calloc(1, sizeof *h);
    if (!h) return NULL;
    h->m = ckb200_model_open(spec_from_env(), 1);
    if (!h->m) { free(h); return NULL; }
    fill_config(h->m);
    h->logits = (float *)ckb200_host_alloc((size_t)g_cfg.vocab_size * sizeof(float));
    if (!h->logits) { ckb200_model_free(h->m); free(h); return NULL; }
    return h;
}

CK_EXPORT void ck_model_free(void *model)
{
    Handle *h = (Handle *)model;
    if (!h) return;
    ckb200_model_free(h->m);
    ckb200_host_free(h->logits);
    free(h);
}

CK_EXPORT void ck_model_precompute_rope(void *model) { (void)model; /* done on the device at creation */ }

CK_EXPORT int ck_model_load_weights(void *model, const char *bump_path)
{
    Handle *h = (Handle *)model;
    if (!h || !bump_path) return -1;
    CKB200Model *m = ckb200_model_open(bump_path, 1);
    if (!m) return -1;
    ckb200_model_free(h->m);
    h->m = m;
    fill_config(m);
    return 0;
}

CK_EXPORT void ck_model_decode(void *model, const int *token, int token_index)
{
    Handle *h = (Handle *)model;
    if (!h || !token || token_index < 0) return;
    /* the function is void: a failure (a position past the context, a device error) leaves NaN logits instead of the
     * previous call's, and the reason in ckb200_last_error() */
    const int32_t t = *token;
    if (ckb200_model_set_pos(h->m, token_index) || ckb200_model_decode(h->m, &t, h->logits))
        for (int i = 0; i < g_cfg.vocab_size; ++i) h->logits[i] = NAN;
}

CK_EXPORT void ck_model_forward(void *model, const int *tokens, int num_tokens)
{
    Handle *h = (Handle *)model;
    if (!h || !tokens || num_tokens <= 0) return;
    ckb200_model_reset(h->m);
    int32_t *ids = (int32_t *)malloc((size_t)num_tokens * sizeof(int32_t));
    if (!ids) return;
    for (int i = 0; i < num_tokens; ++i) ids[i] = tokens[i];
    if (ckb200_model_prefill(h->m, ids, num_tokens, h->logits))           /* one batched pass from the empty cache */
        for (int i = 0; i < g_cfg.vocab_size; ++i) h->logits[i] = NAN;
    free(ids);
}

CK_EXPORT float *ck_model_get_logits(void *model) { return model ? ((Handle *)model)->logits : NULL; }
CK_EXPORT int ck_model_verify_canaries(void *model) { (void)model; return ckb200_last_error() ? 1 : 0; }
CK_EXPORT void *ck_model_get_base(void *model) { return model ? (void *)((Handle *)model)->m : NULL; }
CK_EXPORT size_t ck_model_get_total_bytes(void *model) { (void)model; return g_cfg.total_bytes; }
