/*
 * ckb200_registry.h - the supported-op registry of the reference, exported by libckb200.so.
 *
 * Same symbols, enum values and struct layouts as the reference's include/ckernel_registry.h:10-12 and
 * include/ckernel_ir.h:38-79 (CKOpType, CKKernelId, CKInputRef, CKIRNode, CKIRGraph), so a caller built
 * against those headers can link this library instead.  Behaviour follows src/ckernel_registry.c:26-60:
 * the seven forward ops are supported (each is backed by CUDA kernels of this library), backward ops
 * are not; ck_ir_validate_supported() returns 0, or -1 after printing the first unsupported node.
 */
#ifndef CKB200_REGISTRY_H
#define CKB200_REGISTRY_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#ifndef CKERNEL_IR_H   /* the reference's own header wins when both are included */
typedef struct {
    int num_layers, hidden_size, intermediate_size, num_heads, num_kv_heads, vocab_size, context_window;
    float rms_norm_eps, rope_theta;
    int rotary_dim;
    float rope_scaling_factor;
    char rope_scaling_type[16];
} CKModelConfig;

typedef enum {
    CK_OP_RMSNORM = 0, CK_OP_LINEAR_QKV, CK_OP_ATTENTION, CK_OP_ADD, CK_OP_LINEAR, CK_OP_SPLIT, CK_OP_SWIGLU,
    CK_OP_RMSNORM_BWD, CK_OP_LINEAR_QKV_BWD, CK_OP_ATTENTION_BWD, CK_OP_ADD_BWD, CK_OP_LINEAR_BWD, CK_OP_SPLIT_BWD, CK_OP_SWIGLU_BWD
} CKOpType;

typedef struct { uint16_t layer, node; } CKKernelId;
typedef struct { CKKernelId producer; uint8_t out_index; } CKInputRef;
typedef struct { CKKernelId id; CKOpType op; CKInputRef inputs[4]; uint8_t n_inputs, n_outputs; } CKIRNode;
typedef struct { CKModelConfig config; int num_nodes; CKIRNode *nodes; } CKIRGraph;
#endif

int ck_op_supported(CKOpType op);
int ck_ir_validate_supported(const CKIRGraph *graph);
/* which kernels of this library carry out a supported op (NULL for unsupported ops); not in the reference */
const char *ckb200_op_kernels(CKOpType op);

#ifdef __cplusplus
}
#endif
#endif
