/* An opened BUMPWGT5 file: header and digests checked, the sidecar map parsed (bump_loader.c). */
#ifndef CKB200_BUMP_FILE_H
#define CKB200_BUMP_FILE_H

#include <stddef.h>
#include <stdint.h>

typedef struct CkbBump CkbBump;

/* manifest_path NULL = weights_manifest.map beside the file; NULL on failure (ckb200_last_error_message says why) */
CkbBump *ckb_bump_open(const char *bump_path, const char *manifest_path);
void ckb_bump_close(CkbBump *b);
/* entry of the map by tensor name; 0 when found */
int ckb_bump_find(const CkbBump *b, const char *name, const char **dtype, uint64_t *file_offset, uint64_t *size);
int ckb_bump_read(const CkbBump *b, uint64_t file_offset, void *dst, size_t n);
const char *ckb_bump_meta(const CkbBump *b);       /* the JSON metadata blob or NULL */

#endif
