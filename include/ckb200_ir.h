/* Decode steps replayed from the reference's lowered call IR.
 *
 * Replaces the per-model C that version/v7/scripts/codegen_v7.py:569-931 generates from "lowered-ir-v3" files
 * (version/v7/scripts/build_ir_v7.py:6414-6876, written with --call-output): instead of compiling the op list, this library
 * binds every op to the device kernel behind its symbol and replays the list as one CUDA graph per token.  Weights come from
 * the BUMPWGT5 file and its sidecar map (include/ckernel_bump_v5.h:19-52, version/v7/src/ckernel_model_load_v7.c:127-310).
 * One sequence, one GPU.  Files that call a symbol without a kernel here are refused at open with a message naming it. */
#ifndef CKB200_IR_H
#define CKB200_IR_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef struct CKB200IrModel CKB200IrModel;

/* manifest_map_path NULL = weights_manifest.map beside the bump file; NULL on failure (ckb200_last_error_message) */
CKB200IrModel *ckb200_ir_open(const char *call_json_path, const char *bump_path, const char *manifest_map_path);
void ckb200_ir_free(CKB200IrModel *m);
/* one token at the current position (the generated ck_model_decode); logits_host may be NULL (no read back, no synchronisation) */
int ckb200_ir_decode(CKB200IrModel *m, int32_t token, float *logits_host);
int ckb200_ir_reset(CKB200IrModel *m);                       /* zero the KV cache, position 0 */
int ckb200_ir_set_pos(CKB200IrModel *m, int pos);
int ckb200_ir_get_pos(const CKB200IrModel *m);
int ckb200_ir_vocab_size(const CKB200IrModel *m);
int ckb200_ir_context_length(const CKB200IrModel *m);
int ckb200_ir_num_ops(const CKB200IrModel *m);
const char *ckb200_ir_op_symbol(const CKB200IrModel *m, int i);
int ckb200_ir_graph_nodes(const CKB200IrModel *m);           /* nodes of the captured step (0 before the second token) */
/* device address and size of an activation buffer of the memory plan, by name (tests and tools) */
void *ckb200_ir_buffer(CKB200IrModel *m, const char *name, size_t *bytes);

#ifdef __cplusplus
}
#endif
#endif
