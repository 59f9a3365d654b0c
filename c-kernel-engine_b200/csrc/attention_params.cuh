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
    // Fused tail of the tile kernel (all optional).  `counters` (zero on entry, left zero on exit) holds one arrival
    // count per (sequence, kv head) followed by one per sequence: the last split CTA of a kv head merges its heads'
    // partials, and the last kv head of a sequence quantises the finished row to Q8_K blocks for the consumer GEMV.
    int *counters;
    uint8_t *q8_out;       // [batch][q8_cols / 256] Q8_K blocks, or NULL
    int out_stride;        // floats between the out rows of consecutive sequences (>= H * ad)
    int q8_cols;           // elements quantised per row (multiple of 256, <= out_stride; the row's tail must be zero)
    int kv_f16;            // the caches hold IEEE fp16 (k and v then point at uint16 data, strides counted in elements)
    int early_rows;        // tile kernel: cache rows before the newest one and *pos_ptr may be read before the dependency wait
};

__device__ __forceinline__ int attn_kv_tokens(const AttnParams &p) { return p.pos_ptr ? min(__ldcg(p.pos_ptr) + 1, p.cap) : p.kv_tokens; }

constexpr int ATTN_MAX_GROUP = 8;    // most Q heads per kv head handled by the fast paths

}  // namespace ckb
