/* libckb200_model_v7.so - the singleton model ABI that the reference's v7/v8 codegen emits into every
 * libmodel.so and that scripts/ck_chat.py binds with ctypes (version/v7/scripts/codegen_v7.py:1282-1426,
 * scripts/ck_chat.py:533-621): ck_model_init / ck_model_embed_tokens / ck_model_forward /
 * ck_model_decode / ck_model_get_logits and the getters.  0 = success, -1 = failure.
 *
 * `weights_path` is the reference's weights.bump (its map and, when present, the lowered call IR are looked for beside it), a CKB2MDL1
 * file or "synthetic:<shape>" (ckb200_model.h).  With a call IR the model is replayed from that op list (ckb200_ir.h); without one the
 * device-resident step executor runs the weights with its own recipe.  The logits of the last position are kept on the host for
 * ck_model_get_logits().
 */
#include <stdint.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#include "../../../include/ckb200.h"
#include "../../../include/ckb200_ir.h"
#include "../../../include/ckb200_model.h"

#define CK_EXPORT __attribute__((visibility("default")))

CK_EXPORT void ck_model_free(void);

static CKB200Model *g_model;         /* the step executor (hard-wired Llama/Qwen recipe), or ... */
static CKB200IrModel *g_ir;          /* ... the replay of the model's own lowered call IR */
static float *g_logits;
static int g_pos, g_vocab, g_ctx;

static int finish_init(void)
{
    if (!g_model && !g_ir) return -1;
    g_vocab = g_ir ? ckb200_ir_vocab_size(g_ir) : ckb200_model_config(g_model)->vocab_size;
    g_ctx = g_ir ? ckb200_ir_context_length(g_ir) : ckb200_model_config(g_model)->max_seq_len;
    g_logits = (float *)ckb200_host_alloc((size_t)g_vocab * sizeof(float));
    if (!g_logits) { ck_model_free(); return -1; }
    memset(g_logits, 0, (size_t)g_vocab * sizeof(float));
    g_pos = 0;
    return 0;
}

/* The reference's run folder holds weights.bump, weights_manifest.map and lowered_decode_call.json side by side
 * (version/v7/scripts/ck_run_v7.py:2229, :2312).  When the call IR is there (or CKB200_CALL_IR names one) the model runs as that op
 * list says - whatever template the pipeline lowered it with; otherwise the step executor's own recipe runs the weights. */
static int call_ir_path(const char *weights_path, char *out, size_t cap)
{
    const char *env = getenv("CKB200_CALL_IR");
    if (env && *env) { snprintf(out, cap, "%s", env); return 1; }
    if (!weights_path || !strncmp(weights_path, "synthetic:", 10)) return 0;
    const char *slash = strrchr(weights_path, '/');
    snprintf(out, cap, "%.*slowered_decode_call.json", slash ? (int)(slash - weights_path + 1) : 0, weights_path);
    FILE *f = fopen(out, "rb");
    if (!f) return 0;
    fclose(f);
    return 1;
}

static int init_common(const char *weights_path, const char *manifest_path)
{
    if (g_model || g_ir) return 0;
    char ir[4096];
    if (call_ir_path(weights_path, ir, sizeof ir)) g_ir = ckb200_ir_open(ir, weights_path, manifest_path);
    else if (manifest_path) g_model = ckb200_model_open_bump(weights_path, manifest_path, 1);
    else g_model = ckb200_model_open(weights_path, 1);
    return finish_init();
}

CK_EXPORT int ck_model_init(const char *weights_path) { return init_common(weights_path, NULL); }

/* weights.bump + weights_manifest.map as the reference's converter writes them */
CK_EXPORT int ck_model_init_with_manifest(const char *weights_path, const char *manifest_path) { return init_common(weights_path, manifest_path); }

CK_EXPORT void ck_model_free(void)
{
    if (g_model) ckb200_model_free(g_model);
    if (g_ir) ckb200_ir_free(g_ir);
    if (g_logits) ckb200_host_free(g_logits);
    g_model = NULL;
    g_ir = NULL;
    g_logits = NULL;
}

CK_EXPORT void ck_model_kv_cache_reset(void)
{
    if (g_model) ckb200_model_reset(g_model);
    if (g_ir) ckb200_ir_reset(g_ir);
    g_pos = 0;
}

CK_EXPORT int ck_model_kv_cache_enable(int capacity) { (void)capacity; return 0; }

static int step(int32_t token, int want_logits)
{
    if (g_pos >= g_ctx) return -1;
    const int rc = g_ir ? ckb200_ir_decode(g_ir, token, want_logits ? g_logits : NULL) : ckb200_model_decode(g_model, &token, want_logits ? g_logits : NULL);
    if (rc != 0) return -1;
    ++g_pos;
    return 0;
}

CK_EXPORT int ck_model_embed_tokens(const int32_t *tokens, int count)
{
    if ((!g_model && !g_ir) || !tokens || count <= 0) return -1;
    if (g_pos + count > g_ctx) return -1;
    if (g_ir) {                       /* the decode op list, token by token; logits of the last one */
        for (int i = 0; i < count; ++i) if (step(tokens[i], i == count - 1)) return -1;
        return 0;
    }
    /* a prompt from an empty cache runs as one batched pass (tensor-core GEMMs, causal prefill attention), otherwise token by token */
    if (ckb200_model_prefill(g_model, tokens, count, g_logits) != 0) return -1;
    g_pos += count;
    return 0;
}

CK_EXPORT int ck_model_forward(float *output)
{
    if (!g_model && !g_ir) return -1;
    if (output) memcpy(output, g_logits, (size_t)g_vocab * sizeof(float));
    return 0;
}

CK_EXPORT int ck_model_decode(int32_t token, float *output)
{
    if (!g_model && !g_ir) return -1;
    if (step(token, 1)) return -1;
    if (output) memcpy(output, g_logits, (size_t)g_vocab * sizeof(float));
    return 0;
}

CK_EXPORT int ck_model_get_vocab_size(void) { return g_model || g_ir ? g_vocab : 0; }
CK_EXPORT int ck_model_get_context_window(void) { return g_model || g_ir ? g_ctx : 0; }
CK_EXPORT int ck_model_get_active_tokens(void) { return g_model || g_ir ? g_pos : 0; }
CK_EXPORT int ck_model_get_logits_stride(void) { return g_model || g_ir ? g_vocab : 0; }
CK_EXPORT float *ck_model_get_logits(void) { return g_model || g_ir ? g_logits : NULL; }
CK_EXPORT uintptr_t ck_model_get_base_ptr(void) { return g_ir ? (uintptr_t)g_ir : (uintptr_t)g_model; }
/* no tokenizer or stop-token table travels with a model spec */
CK_EXPORT int ck_model_get_vocab_strings_size(void) { return 0; }
CK_EXPORT int ck_model_get_num_merges(void) { return 0; }
CK_EXPORT int ck_model_get_num_stop_tokens(void) { return 0; }
CK_EXPORT int ck_model_is_stop_token(int32_t token_id) { (void)token_id; return 0; }
CK_EXPORT int32_t ck_model_get_eos_token_id(void) { return -1; }
CK_EXPORT int32_t ck_model_get_bos_token_id(void) { return -1; }
