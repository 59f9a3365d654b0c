/* BUMPWGT5 weight files -> the device-resident step executor.
 *
 * The reference's converter writes one flat file (include/ckernel_bump_v5.h:19-52): a 128-byte header with the model
 * dimensions and the SHA-256 of the payload, 24 reserved bytes, a dtype table, the tensors back to back in the
 * reference's block formats, and, appended at the end of the file, a JSON metadata blob located by a 48-byte footer
 * ("BUMPV5MD", blob size, SHA-256 of the blob).  Where each tensor lies is recorded in a sidecar map, one line per tensor,
 * name|dtype|file_offset|size|runtime_offset - the file the reference's own C loader walks
 * (version/v7/src/ckernel_model_load_v7.c:127-310).  Tensor names are the converter's
 * (version/v7/scripts/convert_gguf_to_bump_v7.py:1200-1228, :3218-3395): token_emb, output.weight (when the LM head is
 * not tied), layer.N.{ln1_gamma, wq, wk, wv, wo, ln2_gamma, w1 (gate rows then up rows), w2}, final_ln_weight.
 *
 * This loader checks both digests, reads the header and the config object of the metadata (rope_theta, rms_eps,
 * tie_word_embeddings are not in the header), walks the map and uploads every tensor the decode step uses into a model
 * created for those dimensions.  The runtime offsets of the map belong to the generated CPU model and are ignored: the
 * executor has its own arena.  What it cannot run is refused with a message instead of being approximated: attention
 * biases or q/k norms with non-zero content, fp32 / fp16 weight matrices, layers that disagree on their weight formats.
 */
#define _FILE_OFFSET_BITS 64
#define _POSIX_C_SOURCE 200809L
#include <ctype.h>
#include <stdint.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>
#include <sys/types.h>

#include "../../include/ckb200.h"
#include "../../include/ckb200_model.h"
#include "bump_file.h"
#include "launch.h"

/* ------------------------------------------------------------------ SHA-256 (FIPS 180-4) */

typedef struct { uint32_t h[8]; uint8_t buf[64]; uint64_t bytes; size_t fill; } Sha256;

static const uint32_t SHA_K[64] = {
    0x428a2f98, 0x71374491, 0xb5c0fbcf, 0xe9b5dba5, 0x3956c25b, 0x59f111f1, 0x923f82a4, 0xab1c5ed5, 0xd807aa98, 0x12835b01, 0x243185be, 0x550c7dc3,
    0x72be5d74, 0x80deb1fe, 0x9bdc06a7, 0xc19bf174, 0xe49b69c1, 0xefbe4786, 0x0fc19dc6, 0x240ca1cc, 0x2de92c6f, 0x4a7484aa, 0x5cb0a9dc, 0x76f988da,
    0x983e5152, 0xa831c66d, 0xb00327c8, 0xbf597fc7, 0xc6e00bf3, 0xd5a79147, 0x06ca6351, 0x14292967, 0x27b70a85, 0x2e1b2138, 0x4d2c6dfc, 0x53380d13,
    0x650a7354, 0x766a0abb, 0x81c2c92e, 0x92722c85, 0xa2bfe8a1, 0xa81a664b, 0xc24b8b70, 0xc76c51a3, 0xd192e819, 0xd6990624, 0xf40e3585, 0x106aa070,
    0x19a4c116, 0x1e376c08, 0x2748774c, 0x34b0bcb5, 0x391c0cb3, 0x4ed8aa4a, 0x5b9cca4f, 0x682e6ff3, 0x748f82ee, 0x78a5636f, 0x84c87814, 0x8cc70208,
    0x90befffa, 0xa4506ceb, 0xbef9a3f7, 0xc67178f2 };

static uint32_t rotr(uint32_t x, int n) { return (x >> n) | (x << (32 - n)); }

static void sha_block(Sha256 *s, const uint8_t *p)
{
    uint32_t w[64], a[8];
    for (int i = 0; i < 16; ++i) w[i] = (uint32_t)p[4 * i] << 24 | (uint32_t)p[4 * i + 1] << 16 | (uint32_t)p[4 * i + 2] << 8 | p[4 * i + 3];
    for (int i = 16; i < 64; ++i) {
        const uint32_t s0 = rotr(w[i - 15], 7) ^ rotr(w[i - 15], 18) ^ (w[i - 15] >> 3), s1 = rotr(w[i - 2], 17) ^ rotr(w[i - 2], 19) ^ (w[i - 2] >> 10);
        w[i] = w[i - 16] + s0 + w[i - 7] + s1;
    }
    memcpy(a, s->h, sizeof a);
    for (int i = 0; i < 64; ++i) {
        const uint32_t S1 = rotr(a[4], 6) ^ rotr(a[4], 11) ^ rotr(a[4], 25), ch = (a[4] & a[5]) ^ (~a[4] & a[6]);
        const uint32_t t1 = a[7] + S1 + ch + SHA_K[i] + w[i];
        const uint32_t S0 = rotr(a[0], 2) ^ rotr(a[0], 13) ^ rotr(a[0], 22), maj = (a[0] & a[1]) ^ (a[0] & a[2]) ^ (a[1] & a[2]);
        const uint32_t t2 = S0 + maj;
        a[7] = a[6]; a[6] = a[5]; a[5] = a[4]; a[4] = a[3] + t1; a[3] = a[2]; a[2] = a[1]; a[1] = a[0]; a[0] = t1 + t2;
    }
    for (int i = 0; i < 8; ++i) s->h[i] += a[i];
}

static void sha_init(Sha256 *s)
{
    static const uint32_t h0[8] = { 0x6a09e667, 0xbb67ae85, 0x3c6ef372, 0xa54ff53a, 0x510e527f, 0x9b05688c, 0x1f83d9ab, 0x5be0cd19 };
    memcpy(s->h, h0, sizeof h0);
    s->bytes = 0;
    s->fill = 0;
}

static void sha_update(Sha256 *s, const uint8_t *p, size_t n)
{
    s->bytes += n;
    while (n) {
        if (s->fill == 0 && n >= 64) { sha_block(s, p); p += 64; n -= 64; continue; }
        const size_t take = 64 - s->fill < n ? 64 - s->fill : n;
        memcpy(s->buf + s->fill, p, take);
        s->fill += take; p += take; n -= take;
        if (s->fill == 64) { sha_block(s, s->buf); s->fill = 0; }
    }
}

static void sha_final(Sha256 *s, uint8_t out[32])
{
    const uint64_t bits = s->bytes * 8;
    uint8_t pad[72] = { 0x80 };
    const size_t padlen = (s->fill < 56 ? 56 : 120) - s->fill;
    sha_update(s, pad, padlen);
    uint8_t len[8];
    for (int i = 0; i < 8; ++i) len[i] = (uint8_t)(bits >> (56 - 8 * i));
    sha_update(s, len, 8);
    for (int i = 0; i < 8; ++i) { out[4 * i] = (uint8_t)(s->h[i] >> 24); out[4 * i + 1] = (uint8_t)(s->h[i] >> 16); out[4 * i + 2] = (uint8_t)(s->h[i] >> 8); out[4 * i + 3] = (uint8_t)s->h[i]; }
}

/* exported for the tests of the loader: digest of a buffer */
void ckb200_sha256(const void *data, size_t bytes, uint8_t out32[32])
{
    Sha256 s;
    sha_init(&s);
    sha_update(&s, (const uint8_t *)data, bytes);
    sha_final(&s, out32);
}

/* ------------------------------------------------------------------ file pieces */

#define BUMP_HEADER 128
#define BUMP_DATA_START 152          /* header + 24 reserved bytes (CK_BUMP_DATA_START) */
#define BUMP_FOOTER 48

typedef struct {
    uint32_t version, model_type, num_layers, vocab_size, embed_dim, intermediate_size, context_length, num_heads, num_kv_heads, head_dim;
    uint64_t aligned_embed_dim, aligned_head_dim, aligned_intermediate, aligned_context;
    uint8_t checksum[32];
} BumpHeader;

static uint32_t rd32(const uint8_t *p) { return (uint32_t)p[0] | (uint32_t)p[1] << 8 | (uint32_t)p[2] << 16 | (uint32_t)p[3] << 24; }
static uint64_t rd64(const uint8_t *p) { return (uint64_t)rd32(p) | (uint64_t)rd32(p + 4) << 32; }

static int parse_header(const uint8_t *b, BumpHeader *h)
{
    if (memcmp(b, "BUMPWGT5", 8)) return -1;
    h->version = rd32(b + 8); h->model_type = rd32(b + 12); h->num_layers = rd32(b + 16); h->vocab_size = rd32(b + 20);
    h->embed_dim = rd32(b + 24); h->intermediate_size = rd32(b + 28); h->context_length = rd32(b + 32); h->num_heads = rd32(b + 36);
    h->num_kv_heads = rd32(b + 40); h->head_dim = rd32(b + 44);
    h->aligned_embed_dim = rd64(b + 48); h->aligned_head_dim = rd64(b + 56); h->aligned_intermediate = rd64(b + 64); h->aligned_context = rd64(b + 72);
    memcpy(h->checksum, b + 88, 32);             /* after num_merges and total_vocab_bytes (2 x u32 at 80) */
    return 0;
}

/* value of "key": inside the first {...} that follows "config": in the metadata blob; number or true/false */
static int meta_number(const char *meta, const char *key, double *out)
{
    const char *cfg = strstr(meta, "\"config\"");
    if (!cfg) return -1;
    char pat[96];
    snprintf(pat, sizeof pat, "\"%s\"", key);
    const char *p = strstr(cfg, pat);
    if (!p) return -1;
    p += strlen(pat);
    while (*p && (isspace((unsigned char)*p) || *p == ':')) ++p;
    if (!strncmp(p, "true", 4)) { *out = 1; return 0; }
    if (!strncmp(p, "false", 5)) { *out = 0; return 0; }
    char *end = NULL;
    const double v = strtod(p, &end);
    if (end == p) return -1;
    *out = v;
    return 0;
}

typedef struct { char name[96]; char dtype[16]; uint64_t off, size; } MapEntry;

static int fmt_of(const char *dtype)
{
    if (!strcmp(dtype, "q4_k") || !strcmp(dtype, "q4k")) return 0;
    if (!strcmp(dtype, "q6_k") || !strcmp(dtype, "q6k")) return 1;
    if (!strcmp(dtype, "q8_0")) return 2;
    if (!strcmp(dtype, "q5_0")) return 3;
    return -1;
}

static const MapEntry *find_entry(const MapEntry *e, int n, const char *name)
{
    for (int i = 0; i < n; ++i) if (!strcmp(e[i].name, name)) return &e[i];
    return NULL;
}

static int read_at(FILE *f, uint64_t off, void *dst, size_t n)
{
    if (fseeko(f, (off_t)off, SEEK_SET)) return -1;
    return fread(dst, 1, n, f) == n ? 0 : -1;
}

static int all_zero_at(FILE *f, uint64_t off, uint64_t n)
{
    uint8_t buf[4096];
    if (fseeko(f, (off_t)off, SEEK_SET)) return 0;
    while (n) {
        const size_t take = n < sizeof buf ? (size_t)n : sizeof buf;
        if (fread(buf, 1, take, f) != take) return 0;
        for (size_t i = 0; i < take; ++i) if (buf[i]) return 0;
        n -= take;
    }
    return 1;
}

/* uploads tensor `name` (exact byte count expected by the model) */
static int upload_named(CKB200Model *m, FILE *f, const MapEntry *e, int n, const char *name, int layer, int which, void **buf, size_t *cap)
{
    const MapEntry *t = find_entry(e, n, name);
    if (!t) return ckb_fail(CKB_ERR_STATE, "bump: tensor %s is not in the manifest", name);
    const size_t want = ckb200_model_tensor_bytes(m, layer, which);
    if (t->size != want) return ckb_fail(CKB_ERR_SHAPE, "bump: tensor %s has %llu bytes, the model expects %zu", name, (unsigned long long)t->size, want);
    if (want > *cap) { free(*buf); *buf = malloc(want); *cap = *buf ? want : 0; }
    if (!*buf || read_at(f, t->off, *buf, want)) return ckb_fail(CKB_ERR_STATE, "bump: short read of %s", name);
    return ckb200_model_upload_tensor(m, layer, which, *buf, want);
}

/* norm weights: the file holds aligned_embed_dim floats, the model round256(embed_dim); copy what both have, zero the rest */
static int upload_gamma(CKB200Model *m, FILE *f, const MapEntry *e, int n, const char *name, int layer, int which)
{
    const MapEntry *t = find_entry(e, n, name);
    if (!t) return ckb_fail(CKB_ERR_STATE, "bump: tensor %s is not in the manifest", name);
    const size_t want = ckb200_model_tensor_bytes(m, layer, which);
    float *tmp = (float *)calloc(1, want);
    if (!tmp) return CKB_ERR_STATE;
    const size_t take = t->size < want ? (size_t)t->size : want;
    int rc = read_at(f, t->off, tmp, take) ? ckb_fail(CKB_ERR_STATE, "bump: short read of %s", name) : ckb200_model_upload_tensor(m, layer, which, tmp, want);
    free(tmp);
    return rc;
}

/* ------------------------------------------------------------------ an opened, verified file (shared with the lowered-IR executor) */

struct CkbBump {
    FILE *f;
    BumpHeader h;
    char *meta;              /* the JSON metadata blob (NUL-terminated) or NULL */
    MapEntry *ent;
    int n;
    uint64_t payload_end;
};

void ckb_bump_close(CkbBump *b)
{
    if (!b) return;
    if (b->f) fclose(b->f);
    free(b->meta);
    free(b->ent);
    free(b);
}

CkbBump *ckb_bump_open(const char *bump_path, const char *manifest_path)
{
    if (!bump_path) { ckb_fail(CKB_ERR_STATE, "bump: NULL path"); return NULL; }
    CkbBump *b = (CkbBump *)calloc(1, sizeof *b);
    if (!b) return NULL;
    b->f = fopen(bump_path, "rb");
    if (!b->f) { ckb_fail(CKB_ERR_STATE, "bump: cannot open %s", bump_path); free(b); return NULL; }
    FILE *f = b->f, *mf = NULL;
    uint8_t hb[BUMP_HEADER], fb[BUMP_FOOTER];
    if (fread(hb, 1, BUMP_HEADER, f) != BUMP_HEADER || parse_header(hb, &b->h)) { ckb_fail(CKB_ERR_STATE, "bump: %s is not a BUMPWGT5 file", bump_path); goto fail; }
    if (fseeko(f, 0, SEEK_END)) goto fail;
    const uint64_t file_size = (uint64_t)ftello(f);
    uint64_t payload_end = file_size;
    if (file_size >= BUMP_DATA_START + BUMP_FOOTER && !read_at(f, file_size - BUMP_FOOTER, fb, BUMP_FOOTER) && !memcmp(fb, "BUMPV5MD", 8)) {
        const uint64_t meta_size = rd64(fb + 8);
        if (meta_size > file_size - BUMP_FOOTER - BUMP_DATA_START) { ckb_fail(CKB_ERR_STATE, "bump: metadata size in the footer exceeds the file"); goto fail; }
        payload_end = file_size - BUMP_FOOTER - meta_size;
        b->meta = (char *)malloc(meta_size + 1);
        if (!b->meta || read_at(f, payload_end, b->meta, meta_size)) { ckb_fail(CKB_ERR_STATE, "bump: cannot read the metadata blob"); goto fail; }
        b->meta[meta_size] = 0;
        uint8_t dig[32];
        ckb200_sha256(b->meta, meta_size, dig);
        if (memcmp(dig, fb + 16, 32)) { ckb_fail(CKB_ERR_STATE, "bump: metadata SHA-256 mismatch in %s", bump_path); goto fail; }
    }
    b->payload_end = payload_end;
    {   /* payload digest: dtype table + tensors, [data start, payload end) */
        Sha256 s;
        sha_init(&s);
        uint8_t *chunk = (uint8_t *)malloc(1 << 20);
        if (!chunk || fseeko(f, BUMP_DATA_START, SEEK_SET)) { free(chunk); goto fail; }
        uint64_t left = payload_end - BUMP_DATA_START;
        while (left) {
            const size_t take = left < (1u << 20) ? (size_t)left : (1u << 20);
            if (fread(chunk, 1, take, f) != take) { free(chunk); ckb_fail(CKB_ERR_STATE, "bump: short read of the payload"); goto fail; }
            sha_update(&s, chunk, take);
            left -= take;
        }
        free(chunk);
        uint8_t dig[32];
        sha_final(&s, dig);
        if (memcmp(dig, b->h.checksum, 32)) { ckb_fail(CKB_ERR_STATE, "bump: payload SHA-256 mismatch in %s (file corrupted or truncated)", bump_path); goto fail; }
    }
    /* the sidecar map: given, or weights_manifest.map beside the file */
    char derived[4096];
    if (!manifest_path) {
        const char *slash = strrchr(bump_path, '/');
        snprintf(derived, sizeof derived, "%.*sweights_manifest.map", slash ? (int)(slash - bump_path + 1) : 0, bump_path);
        manifest_path = derived;
    }
    mf = fopen(manifest_path, "r");
    if (!mf) { ckb_fail(CKB_ERR_STATE, "bump: cannot open the manifest map %s", manifest_path); goto fail; }
    int ncap = 0;
    char line[4096];
    while (fgets(line, sizeof line, mf)) {
        if (line[0] == '#' || line[0] == '\n' || line[0] == '\r') continue;
        line[strcspn(line, "\r\n")] = 0;
        char *name = strtok(line, "|"), *dtype = strtok(NULL, "|"), *off = strtok(NULL, "|"), *size = strtok(NULL, "|"), *rt = strtok(NULL, "|");
        if (!name || !dtype || !off || !size || !rt) { ckb_fail(CKB_ERR_STATE, "bump: malformed manifest line (name|dtype|file_offset|size|runtime_offset)"); goto fail; }
        if (b->n == ncap) {
            ncap = ncap ? 2 * ncap : 256;
            MapEntry *g = (MapEntry *)realloc(b->ent, (size_t)ncap * sizeof *b->ent);
            if (!g) goto fail;
            b->ent = g;
        }
        MapEntry *e = &b->ent[b->n];
        snprintf(e->name, sizeof e->name, "%s", name);
        snprintf(e->dtype, sizeof e->dtype, "%s", dtype);
        e->off = strtoull(off, NULL, 0);
        e->size = strtoull(size, NULL, 0);
        if (e->off < BUMP_DATA_START || e->off + e->size > payload_end) { ckb_fail(CKB_ERR_STATE, "bump: tensor %s lies outside the payload", name); goto fail; }
        ++b->n;
    }
    fclose(mf);
    return b;
fail:
    if (mf) fclose(mf);
    ckb_bump_close(b);
    return NULL;
}

int ckb_bump_find(const CkbBump *b, const char *name, const char **dtype, uint64_t *off, uint64_t *size)
{
    const MapEntry *e = find_entry(b->ent, b->n, name);
    if (!e) return -1;
    if (dtype) *dtype = e->dtype;
    if (off) *off = e->off;
    if (size) *size = e->size;
    return 0;
}

int ckb_bump_read(const CkbBump *b, uint64_t off, void *dst, size_t n) { return read_at(b->f, off, dst, n); }
const char *ckb_bump_meta(const CkbBump *b) { return b->meta; }

CKB200Model *ckb200_model_open_bump(const char *bump_path, const char *manifest_path, int batch)
{
    CkbBump *bf = ckb_bump_open(bump_path, manifest_path);
    if (!bf) return NULL;
    FILE *f = bf->f;
    const BumpHeader h = bf->h;
    const char *meta = bf->meta;
    MapEntry *ent = bf->ent;
    const int n = bf->n;
    CKB200Model *m = NULL;
    void *buf = NULL;
    size_t cap = 0;
    /* configuration: header dimensions, metadata for what the header lacks, formats from the map */
    CKB200ModelConfig cfg;
    memset(&cfg, 0, sizeof cfg);
    cfg.embed_dim = (int)h.embed_dim; cfg.num_heads = (int)h.num_heads; cfg.num_kv_heads = (int)h.num_kv_heads; cfg.head_dim = (int)h.head_dim;
    cfg.intermediate_size = (int)h.intermediate_size; cfg.num_layers = (int)h.num_layers; cfg.vocab_size = (int)h.vocab_size; cfg.max_seq_len = (int)h.context_length;
    cfg.rms_eps = 1e-5f; cfg.rope_theta = 10000.0f;
    double v;
    if (meta && !meta_number(meta, "rms_eps", &v)) cfg.rms_eps = (float)v;
    if (meta && !meta_number(meta, "rope_theta", &v)) cfg.rope_theta = (float)v;
    const MapEntry *out_w = find_entry(ent, n, "output.weight"), *tok = find_entry(ent, n, "token_emb");
    if (!tok) { ckb_fail(CKB_ERR_STATE, "bump: no token_emb in the manifest"); goto fail; }
    cfg.tie_embeddings = out_w ? 0 : 1;
    static const char *names[6] = { "wq", "wk", "wv", "wo", "w1", "w2" };
    int fmts[6];
    for (int i = 0; i < 6; ++i) {
        for (uint32_t l = 0; l < h.num_layers; ++l) {
            char nm[96];
            snprintf(nm, sizeof nm, "layer.%u.%s", l, names[i]);
            const MapEntry *t = find_entry(ent, n, nm);
            const int fm = t ? fmt_of(t->dtype) : -1;
            if (fm < 0) { ckb_fail(CKB_ERR_SHAPE, "bump: %s is missing or has a weight format this library does not run (%s)", nm, t ? t->dtype : "absent"); goto fail; }
            if (l == 0) fmts[i] = fm;
            else if (fm != fmts[i]) { ckb_fail(CKB_ERR_SHAPE, "bump: %s is %s but layer 0 uses another format; the step executor takes one format per projection", nm, t->dtype); goto fail; }
        }
    }
    cfg.fmt_q = fmts[0]; cfg.fmt_k = fmts[1]; cfg.fmt_v = fmts[2]; cfg.fmt_o = fmts[3]; cfg.fmt_gate_up = fmts[4]; cfg.fmt_down = fmts[5];
    cfg.fmt_embedding = fmt_of(tok->dtype);
    cfg.fmt_lm_head = out_w ? fmt_of(out_w->dtype) : cfg.fmt_embedding;
    if (cfg.fmt_embedding < 0 || cfg.fmt_lm_head < 0) { ckb_fail(CKB_ERR_SHAPE, "bump: token_emb / output.weight in a format this library does not run (%s)", tok->dtype); goto fail; }
    cfg.batch = batch > 0 ? batch : 1;
    cfg.tp_rank = 0; cfg.tp_size = 1;
    /* what the executor has no op for must be absent or zero */
    for (int i = 0; i < n; ++i) {
        const char *dot = strrchr(ent[i].name, '.');
        const char *leaf = dot ? dot + 1 : ent[i].name;
        if (!strcmp(leaf, "bq") || !strcmp(leaf, "bk") || !strcmp(leaf, "bv") || !strcmp(leaf, "bo") || !strcmp(leaf, "b1") || !strcmp(leaf, "b2") ||
            !strcmp(ent[i].name, "final_ln_bias")) {
            if (!all_zero_at(f, ent[i].off, ent[i].size)) { ckb_fail(CKB_ERR_SHAPE, "bump: %s is a non-zero bias; the step executor has no bias add", ent[i].name); goto fail; }
        } else if (!strcmp(leaf, "q_norm") || !strcmp(leaf, "k_norm") || !strcmp(leaf, "post_attention_norm") || !strcmp(leaf, "post_ffn_norm")) {
            ckb_fail(CKB_ERR_SHAPE, "bump: %s: this model family needs ops the step executor does not have", ent[i].name);
            goto fail;
        }
    }
    m = ckb200_model_create(&cfg);
    if (!m) goto fail;
    int rc = 0;
    for (uint32_t l = 0; l < h.num_layers && !rc; ++l) {
        char nm[96];
        static const int which[6] = { CKB_T_WQ, CKB_T_WK, CKB_T_WV, CKB_T_WO, CKB_T_W1, CKB_T_W2 };
        snprintf(nm, sizeof nm, "layer.%u.ln1_gamma", l);
        rc = upload_gamma(m, f, ent, n, nm, (int)l, CKB_T_LN1);
        snprintf(nm, sizeof nm, "layer.%u.ln2_gamma", l);
        if (!rc) rc = upload_gamma(m, f, ent, n, nm, (int)l, CKB_T_LN2);
        for (int i = 0; i < 6 && !rc; ++i) {
            snprintf(nm, sizeof nm, "layer.%u.%s", l, names[i]);
            rc = upload_named(m, f, ent, n, nm, (int)l, which[i], &buf, &cap);
        }
    }
    if (!rc) rc = upload_gamma(m, f, ent, n, "final_ln_weight", -1, CKB_T_FINAL_GAMMA);
    if (!rc) rc = upload_named(m, f, ent, n, out_w ? "output.weight" : "token_emb", -1, CKB_T_LM_HEAD, &buf, &cap);
    if (!rc && out_w) rc = upload_named(m, f, ent, n, "token_emb", -1, CKB_T_EMBEDDING, &buf, &cap);
    if (rc) goto fail;
    free(buf);
    ckb_bump_close(bf);
    return m;
fail:
    if (m) ckb200_model_free(m);
    free(buf);
    ckb_bump_close(bf);
    return NULL;
}
