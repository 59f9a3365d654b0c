// Arguments shared by the decode-attention kernels (attention.cu, attention_tile.cu).
#pragma once
#include "device_common.cuh"

namespace ckb {

struct AttnParams {
    const float *q;        // [batch][H][ad]
    const float *k;        // [batch][Hkv][cap][ad] (batch stride kv_batch_stride floats)
    const float *v;
    float *out;            // [batch][H][ad]
    float *part;           // scratch [batch][H][splits][ad + 2] (only when splits > 1)
    const int *pos_ptr;    // when not NULL the context length is *pos_ptr + 1 (read on the device, graph-replayable)
    long long kv_batch_stride;
    int H, Hkv, kv_tokens, cap, ad, splits;
    float scale;
};

__device__ __forceinline__ int attn_kv_tokens(const AttnParams &p) { return p.pos_ptr ? min(__ldcg(p.pos_ptr) + 1, p.cap) : p.kv_tokens; }

constexpr int ATTN_MAX_GROUP = 8;    // most Q heads per kv head handled by the fast paths

}  // namespace ckb
