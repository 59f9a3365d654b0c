/* A small JSON reader (RFC 8259 values into a tree) for the lowered-IR files the executor consumes.  No writer, no streaming:
 * the files are a few megabytes at most.  Strings are unescaped in place (\uXXXX becomes UTF-8); numbers are doubles. */
#include "json_mini.h"

#include <ctype.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

typedef struct { const char *p, *end; char err[128]; int depth; } Parser;

static void skip_ws(Parser *ps) { while (ps->p < ps->end && (*ps->p == ' ' || *ps->p == '\t' || *ps->p == '\n' || *ps->p == '\r')) ++ps->p; }

static JsonValue *new_value(int type)
{
    JsonValue *v = (JsonValue *)calloc(1, sizeof *v);
    if (v) v->type = type;
    return v;
}

void json_free(JsonValue *v)
{
    if (!v) return;
    for (int i = 0; i < v->count; ++i) {
        if (v->keys) free(v->keys[i]);
        json_free(v->items[i]);
    }
    free(v->keys);
    free(v->items);
    free(v->str);
    free(v);
}

static int fail(Parser *ps, const char *what)
{
    if (!ps->err[0]) snprintf(ps->err, sizeof ps->err, "%s", what);
    return -1;
}

static int put_utf8(char *dst, unsigned cp)
{
    if (cp < 0x80) { dst[0] = (char)cp; return 1; }
    if (cp < 0x800) { dst[0] = (char)(0xC0 | (cp >> 6)); dst[1] = (char)(0x80 | (cp & 0x3F)); return 2; }
    if (cp < 0x10000) { dst[0] = (char)(0xE0 | (cp >> 12)); dst[1] = (char)(0x80 | ((cp >> 6) & 0x3F)); dst[2] = (char)(0x80 | (cp & 0x3F)); return 3; }
    dst[0] = (char)(0xF0 | (cp >> 18)); dst[1] = (char)(0x80 | ((cp >> 12) & 0x3F)); dst[2] = (char)(0x80 | ((cp >> 6) & 0x3F)); dst[3] = (char)(0x80 | (cp & 0x3F));
    return 4;
}

static int hex4(const char *p, unsigned *out)
{
    unsigned v = 0;
    for (int i = 0; i < 4; ++i) {
        const int c = (unsigned char)p[i];
        if (!isxdigit(c)) return -1;
        v = v * 16 + (unsigned)(isdigit(c) ? c - '0' : (tolower(c) - 'a' + 10));
    }
    *out = v;
    return 0;
}

static char *parse_string(Parser *ps)
{
    if (ps->p >= ps->end || *ps->p != '"') { fail(ps, "expected a string"); return NULL; }
    const char *q = ++ps->p;
    while (q < ps->end && *q != '"') q += (*q == '\\' && q + 1 < ps->end) ? 2 : 1;
    if (q >= ps->end) { fail(ps, "unterminated string"); return NULL; }
    char *out = (char *)malloc((size_t)(q - ps->p) + 1), *w = out;
    if (!out) return NULL;
    for (const char *r = ps->p; r < q; ++r) {
        if (*r != '\\') { *w++ = *r; continue; }
        ++r;
        switch (*r) {
        case 'n': *w++ = '\n'; break;
        case 't': *w++ = '\t'; break;
        case 'r': *w++ = '\r'; break;
        case 'b': *w++ = '\b'; break;
        case 'f': *w++ = '\f'; break;
        case 'u': {
            unsigned cp = 0, lo = 0;
            if (r + 4 >= q + 1 || hex4(r + 1, &cp)) { free(out); fail(ps, "bad \\u escape"); return NULL; }
            r += 4;
            if (cp >= 0xD800 && cp < 0xDC00 && r + 6 < q + 1 && r[1] == '\\' && r[2] == 'u' && !hex4(r + 3, &lo) && lo >= 0xDC00 && lo < 0xE000) {
                cp = 0x10000 + ((cp - 0xD800) << 10) + (lo - 0xDC00);
                r += 6;
            }
            w += put_utf8(w, cp);
            break;
        }
        default: *w++ = *r;            /* \" \\ \/ */
        }
    }
    *w = 0;
    ps->p = q + 1;
    return out;
}

static JsonValue *parse_value(Parser *ps);

static int push(JsonValue *v, char *key, JsonValue *item)
{
    if (v->count == v->cap) {
        const int cap = v->cap ? 2 * v->cap : 8;
        JsonValue **it = (JsonValue **)realloc(v->items, (size_t)cap * sizeof *it);
        if (!it) return -1;
        v->items = it;
        if (v->type == JSON_OBJECT) {
            char **k = (char **)realloc(v->keys, (size_t)cap * sizeof *k);
            if (!k) return -1;
            v->keys = k;
        }
        v->cap = cap;
    }
    if (v->type == JSON_OBJECT) v->keys[v->count] = key;
    v->items[v->count++] = item;
    return 0;
}

static JsonValue *parse_container(Parser *ps, int type)
{
    const char close = type == JSON_OBJECT ? '}' : ']';
    JsonValue *v = new_value(type);
    if (!v) return NULL;
    ++ps->p;
    if (++ps->depth > 256) { fail(ps, "nesting too deep"); goto bad; }
    skip_ws(ps);
    if (ps->p < ps->end && *ps->p == close) { ++ps->p; --ps->depth; return v; }
    for (;;) {
        char *key = NULL;
        skip_ws(ps);
        if (type == JSON_OBJECT) {
            key = parse_string(ps);
            if (!key) goto bad;
            skip_ws(ps);
            if (ps->p >= ps->end || *ps->p != ':') { free(key); fail(ps, "expected ':'"); goto bad; }
            ++ps->p;
        }
        JsonValue *item = parse_value(ps);
        if (!item) { free(key); goto bad; }
        if (push(v, key, item)) { free(key); json_free(item); goto bad; }
        skip_ws(ps);
        if (ps->p < ps->end && *ps->p == ',') { ++ps->p; continue; }
        if (ps->p < ps->end && *ps->p == close) { ++ps->p; break; }
        fail(ps, "expected ',' or the end of the container");
        goto bad;
    }
    --ps->depth;
    return v;
bad:
    json_free(v);
    return NULL;
}

static JsonValue *parse_value(Parser *ps)
{
    skip_ws(ps);
    if (ps->p >= ps->end) { fail(ps, "unexpected end of input"); return NULL; }
    const char c = *ps->p;
    if (c == '{') return parse_container(ps, JSON_OBJECT);
    if (c == '[') return parse_container(ps, JSON_ARRAY);
    if (c == '"') {
        char *s = parse_string(ps);
        if (!s) return NULL;
        JsonValue *v = new_value(JSON_STRING);
        if (!v) { free(s); return NULL; }
        v->str = s;
        return v;
    }
    const size_t left = (size_t)(ps->end - ps->p);
    if (left >= 4 && !memcmp(ps->p, "true", 4)) { ps->p += 4; JsonValue *v = new_value(JSON_BOOL); if (v) v->num = 1; return v; }
    if (left >= 5 && !memcmp(ps->p, "false", 5)) { ps->p += 5; return new_value(JSON_BOOL); }
    if (left >= 4 && !memcmp(ps->p, "null", 4)) { ps->p += 4; return new_value(JSON_NULL); }
    if (left >= 3 && !memcmp(ps->p, "NaN", 3)) { ps->p += 3; JsonValue *v = new_value(JSON_NUMBER); if (v) v->num = 0.0 / 0.0; return v; }   /* Python's json writes these */
    if (left >= 8 && !memcmp(ps->p, "Infinity", 8)) { ps->p += 8; JsonValue *v = new_value(JSON_NUMBER); if (v) v->num = 1.0 / 0.0; return v; }
    if (left >= 9 && !memcmp(ps->p, "-Infinity", 9)) { ps->p += 9; JsonValue *v = new_value(JSON_NUMBER); if (v) v->num = -1.0 / 0.0; return v; }
    if (c == '-' || isdigit((unsigned char)c)) {
        char tmp[64];
        size_t n = 0;
        while (n < sizeof tmp - 1 && ps->p + n < ps->end && (isdigit((unsigned char)ps->p[n]) || strchr("+-.eE", ps->p[n]))) { tmp[n] = ps->p[n]; ++n; }
        tmp[n] = 0;
        char *endp = NULL;
        const double d = strtod(tmp, &endp);
        if (endp == tmp) { fail(ps, "bad number"); return NULL; }
        ps->p += endp - tmp;
        JsonValue *v = new_value(JSON_NUMBER);
        if (v) v->num = d;
        return v;
    }
    fail(ps, "unexpected character");
    return NULL;
}

JsonValue *json_parse(const char *text, size_t len, char *err, size_t err_len)
{
    Parser ps;
    memset(&ps, 0, sizeof ps);
    ps.p = text;
    ps.end = text + len;
    JsonValue *v = parse_value(&ps);
    if (v) {
        skip_ws(&ps);
        if (ps.p != ps.end) { json_free(v); v = NULL; snprintf(ps.err, sizeof ps.err, "trailing data after the value"); }
    }
    if (!v && err && err_len) snprintf(err, err_len, "%s (byte %ld)", ps.err[0] ? ps.err : "out of memory", (long)(ps.p - text));
    return v;
}

JsonValue *json_parse_file(const char *path, char *err, size_t err_len)
{
    FILE *f = fopen(path, "rb");
    if (!f) { if (err) snprintf(err, err_len, "cannot open %s", path); return NULL; }
    fseek(f, 0, SEEK_END);
    const long n = ftell(f);
    fseek(f, 0, SEEK_SET);
    char *buf = n >= 0 ? (char *)malloc((size_t)n + 1) : NULL;
    if (!buf || fread(buf, 1, (size_t)n, f) != (size_t)n) { fclose(f); free(buf); if (err) snprintf(err, err_len, "cannot read %s", path); return NULL; }
    fclose(f);
    JsonValue *v = json_parse(buf, (size_t)n, err, err_len);
    free(buf);
    return v;
}

const JsonValue *json_get(const JsonValue *obj, const char *key)
{
    if (!obj || obj->type != JSON_OBJECT) return NULL;
    for (int i = 0; i < obj->count; ++i) if (!strcmp(obj->keys[i], key)) return obj->items[i];
    return NULL;
}

const JsonValue *json_at(const JsonValue *arr, int i) { return arr && arr->type == JSON_ARRAY && i >= 0 && i < arr->count ? arr->items[i] : NULL; }
int json_len(const JsonValue *v) { return v && (v->type == JSON_ARRAY || v->type == JSON_OBJECT) ? v->count : 0; }
const char *json_str(const JsonValue *v, const char *dflt) { return v && v->type == JSON_STRING ? v->str : dflt; }
double json_num(const JsonValue *v, double dflt) { return v && (v->type == JSON_NUMBER || v->type == JSON_BOOL) ? v->num : dflt; }
