/* Supported-op registry: ck_op_supported / ck_ir_validate_supported with the reference's contract
 * (src/ckernel_registry.c:26-60), stating which CUDA kernels back each forward op. */
#include <stdio.h>

#include "../../include/ckb200_registry.h"

static const struct { CKOpType op; const char *name; const char *kernels; } g_ops[] = {
    { CK_OP_RMSNORM, "RMSNORM", "rmsnorm_forward, add_rmsnorm_q8k" },
    { CK_OP_LINEAR_QKV, "LINEAR_QKV", "quantize_row_q8_k/q8_0 + gemv_q4_k_q8_k / gemv_q6_k_q8_k / gemv_q8_0_q8_0 (gemm_nt_* for prefill)" },
    { CK_OP_ATTENTION, "ATTENTION", "rope_forward_qk + kv_cache_store + attention_forward_decode_head_major_gqa_flash" },
    { CK_OP_ADD, "ADD", "ck_residual_add_token_major (fused into add_rmsnorm_q8k in the step executor)" },
    { CK_OP_LINEAR, "LINEAR", "quantize_row_q8_k/q8_0 + gemv_* / gemm_nt_*" },
    { CK_OP_SPLIT, "SPLIT", "no kernel: gate and up are the two halves of one [2I] GEMV output" },
    { CK_OP_SWIGLU, "SWIGLU", "swiglu_forward, swiglu_q8k" },
};

static const char *op_name(CKOpType op)
{
    static const char *bwd[] = { "RMSNORM_BWD", "LINEAR_QKV_BWD", "ATTENTION_BWD", "ADD_BWD", "LINEAR_BWD", "SPLIT_BWD", "SWIGLU_BWD" };
    for (unsigned i = 0; i < sizeof g_ops / sizeof g_ops[0]; ++i)
        if (g_ops[i].op == op) return g_ops[i].name;
    if (op >= CK_OP_RMSNORM_BWD && op <= CK_OP_SWIGLU_BWD) return bwd[op - CK_OP_RMSNORM_BWD];
    return "UNKNOWN";
}

const char *ckb200_op_kernels(CKOpType op)
{
    for (unsigned i = 0; i < sizeof g_ops / sizeof g_ops[0]; ++i)
        if (g_ops[i].op == op) return g_ops[i].kernels;
    return NULL;
}

int ck_op_supported(CKOpType op) { return ckb200_op_kernels(op) != NULL; }

int ck_ir_validate_supported(const CKIRGraph *graph)
{
    if (!graph || !graph->nodes || graph->num_nodes <= 0) return -1;
    for (int i = 0; i < graph->num_nodes; ++i) {
        const CKIRNode *n = &graph->nodes[i];
        if (!ck_op_supported(n->op)) {
            fprintf(stderr, "Unsupported op in IR: %s (layer=%u node=%u)\n", op_name(n->op), (unsigned)n->id.layer, (unsigned)n->id.node);
            return -1;
        }
    }
    return 0;
}
