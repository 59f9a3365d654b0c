/*
 * ckb200_model_handle.h - handle-based model ABI exported by libckb200_model_api.so: the functions of the
 * reference's include/ck_model_api.h:56-113 (used by src/v6.6/test_generic_api.c:247-282), same names and
 * signatures.  The model spec comes from the environment variable CKB200_MODEL or from the path passed to
 * ck_model_load_weights().
 */
#ifndef CKB200_MODEL_HANDLE_H
#define CKB200_MODEL_HANDLE_H
#include <stddef.h>
#ifdef __cplusplus
extern "C" {
#endif
struct CKModelConfigHandleApi;                       /* layout: include/ck_model_api.h:26-40 */
const struct CKModelConfigHandleApi *ck_model_get_config(void);   /* include/ck_model_api.h:56 */
void *ck_model_create(void);                         /* :62 */
void ck_model_free(void *model);                     /* :67 */
void ck_model_precompute_rope(void *model);          /* :73 */
int ck_model_load_weights(void *model, const char *bump_path);    /* :79 */
void ck_model_forward(void *model, const int *tokens, int num_tokens);   /* :85 */
void ck_model_decode(void *model, const int *token, int token_index);    /* :91 */
float *ck_model_get_logits(void *model);             /* :97 */
int ck_model_verify_canaries(void *model);           /* :103 */
void *ck_model_get_base(void *model);                /* :108 */
size_t ck_model_get_total_bytes(void *model);        /* :113 */
#ifdef __cplusplus
}
#endif
#endif
