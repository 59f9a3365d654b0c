/* libckb200_model_v7.so - the singleton model ABI that the reference's v7/v8 codegen emits into every
 * libmodel.so and that scripts/ck_chat.py binds with ctypes (version/v7/scripts/codegen_v7.py:1282-1426,
 * scripts/ck_chat.py:533-621): ck_model_init / ck_model_embed_tokens / ck_model_forward /
 * ck_model_decode / ck_model_get_logits and the getters.  0 = success, -1 = failure.
 *
 * The model behind it is the device-resident step executor.  `weights_path` is a model spec
 * ("synthetic:<shape>" or a CKB2MDL1 file, see ckb200_model.h).  Prompt tokens are run one decode step
 * at a time; the logits of the last position are kept on the host for ck_model_get_logits().
 */
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#include "../../../include/ckb200.h"
#include "../../../include/ckb200_model.h"

#define CK_EXPORT __attribute__((visibility("default")))

static CKB200Model *g_model;
static float *g_logits;
static int g_pos;

static int finish_init(void)
{
    if (!g_model) return -1;
    g_logits = (float *)ckb200_host_alloc((size_t)ckb200_model_config(g_model)->vocab_size * sizeof(float));
    if (!g_logits) { ckb200_model_free(g_model); g_model = NULL; return -1; }
    memset(g_logits, 0, (size_t)ckb200_model_config(g_model)->vocab_size * sizeof(float));
    g_pos = 0;
    return 0;
}

CK_EXPORT int ck_model_init(const char *weights_path)
{
    if (g_model) return 0;
    g_model = ckb200_model_open(weights_path, 1);
    return finish_init();
}

/* weights.bump + weights_manifest.map as the reference's converter writes them */
CK_EXPORT int ck_model_init_with_manifest(const char *weights_path, const char *manifest_path)
{
    if (g_model) return 0;
    if (!manifest_path) return ck_model_init(weights_path);
    g_model = ckb200_model_open_bump(weights_path, manifest_path, 1);
    return finish_init();
}

CK_EXPORT void ck_model_free(void)
{
    if (!g_model) return;
    ckb200_model_free(g_model);
    ckb200_host_free(g_logits);
    g_model = NULL;
    g_logits = NULL;
}

CK_EXPORT void ck_model_kv_cache_reset(void)
{
    if (!g_model) return;
    ckb200_model_reset(g_model);
    g_pos = 0;
}

CK_EXPORT int ck_model_kv_cache_enable(int capacity) { (void)capacity; return 0; }

static int step(int32_t token, int want_logits)
{
    if (g_pos >= ckb200_model_config(g_model)->max_seq_len) return -1;
    if (ckb200_model_decode(g_model, &token, want_logits ? g_logits : NULL) != 0) return -1;
    ++g_pos;
    return 0;
}

CK_EXPORT int ck_model_embed_tokens(const int32_t *tokens, int count)
{
    if (!g_model || !tokens || count <= 0) return -1;
    if (g_pos + count > ckb200_model_config(g_model)->max_seq_len) return -1;
    /* a prompt from an empty cache runs as one batched pass (tensor-core GEMMs, causal prefill attention), otherwise token by token */
    if (ckb200_model_prefill(g_model, tokens, count, g_logits) != 0) return -1;
    g_pos += count;
    return 0;
}

CK_EXPORT int ck_model_forward(float *output)
{
    if (!g_model) return -1;
    if (output) memcpy(output, g_logits, (size_t)ckb200_model_config(g_model)->vocab_size * sizeof(float));
    return 0;
}

CK_EXPORT int ck_model_decode(int32_t token, float *output)
{
    if (!g_model) return -1;
    if (step(token, 1)) return -1;
    if (output) memcpy(output, g_logits, (size_t)ckb200_model_config(g_model)->vocab_size * sizeof(float));
    return 0;
}

CK_EXPORT int ck_model_get_vocab_size(void) { return g_model ? ckb200_model_config(g_model)->vocab_size : 0; }
CK_EXPORT int ck_model_get_context_window(void) { return g_model ? ckb200_model_config(g_model)->max_seq_len : 0; }
CK_EXPORT int ck_model_get_active_tokens(void) { return g_model ? g_pos : 0; }
CK_EXPORT int ck_model_get_logits_stride(void) { return g_model ? ckb200_model_config(g_model)->vocab_size : 0; }
CK_EXPORT float *ck_model_get_logits(void) { return g_model ? g_logits : NULL; }
CK_EXPORT uintptr_t ck_model_get_base_ptr(void) { return (uintptr_t)g_model; }
/* no tokenizer or stop-token table travels with a model spec */
CK_EXPORT int ck_model_get_vocab_strings_size(void) { return 0; }
CK_EXPORT int ck_model_get_num_merges(void) { return 0; }
CK_EXPORT int ck_model_get_num_stop_tokens(void) { return 0; }
CK_EXPORT int ck_model_is_stop_token(int32_t token_id) { (void)token_id; return 0; }
CK_EXPORT int32_t ck_model_get_eos_token_id(void) { return -1; }
CK_EXPORT int32_t ck_model_get_bos_token_id(void) { return -1; }
