/*
 * ckb200_model_v7.h - singleton model ABI exported by libckb200_model_v7.so.
 *
 * The functions the reference's v7/v8 code generator emits into every libmodel.so
 * (version/v7/scripts/codegen_v7.py:1282-1426) and scripts/ck_chat.py:533-621 binds with ctypes.
 * 0 = success, -1 = failure.  `weights_path` names the model: "synthetic:<shape>[:seed]" or a CKB2MDL1
 * file (ckb200_model.h); the step itself runs on the device-resident executor.
 */
#ifndef CKB200_MODEL_V7_H
#define CKB200_MODEL_V7_H
#include <stdint.h>
#ifdef __cplusplus
extern "C" {
#endif
int ck_model_init(const char *weights_path);                                   /* codegen_v7.py:1282-1299 */
int ck_model_init_with_manifest(const char *weights_path, const char *manifest_path);
void ck_model_free(void);
void ck_model_kv_cache_reset(void);                                            /* codegen_v7.py:1340-1344 */
int ck_model_kv_cache_enable(int capacity);
int ck_model_embed_tokens(const int32_t *tokens, int count);                   /* codegen_v7.py:1357-1373 */
int ck_model_forward(float *output);                                           /* codegen_v7.py:1376-1381 */
int ck_model_decode(int32_t token, float *output);                             /* codegen_v7.py:1384-1390 */
int ck_model_get_vocab_size(void);
int ck_model_get_context_window(void);
int ck_model_get_active_tokens(void);
int ck_model_get_logits_stride(void);
float *ck_model_get_logits(void);
uintptr_t ck_model_get_base_ptr(void);
int ck_model_get_vocab_strings_size(void);
int ck_model_get_num_merges(void);
int ck_model_get_num_stop_tokens(void);                                        /* codegen_v7.py:1056-1081 */
int ck_model_is_stop_token(int32_t token_id);
int32_t ck_model_get_eos_token_id(void);
int32_t ck_model_get_bos_token_id(void);
#ifdef __cplusplus
}
#endif
#endif
