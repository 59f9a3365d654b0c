/* Tree form of a JSON document (json_mini.c). */
#ifndef CKB200_JSON_MINI_H
#define CKB200_JSON_MINI_H

#include <stddef.h>

enum { JSON_NULL = 0, JSON_BOOL, JSON_NUMBER, JSON_STRING, JSON_ARRAY, JSON_OBJECT };

typedef struct JsonValue {
    int type;
    double num;                 /* JSON_NUMBER, JSON_BOOL (0 / 1) */
    char *str;                  /* JSON_STRING */
    int count, cap;             /* JSON_ARRAY, JSON_OBJECT */
    char **keys;                /* JSON_OBJECT: keys in document order */
    struct JsonValue **items;
} JsonValue;

JsonValue *json_parse(const char *text, size_t len, char *err, size_t err_len);      /* NULL on error, message in err */
JsonValue *json_parse_file(const char *path, char *err, size_t err_len);
void json_free(JsonValue *v);
const JsonValue *json_get(const JsonValue *obj, const char *key);                    /* NULL when absent or not an object */
const JsonValue *json_at(const JsonValue *arr, int i);
int json_len(const JsonValue *v);
const char *json_str(const JsonValue *v, const char *dflt);
double json_num(const JsonValue *v, double dflt);

#endif
