/* Internal host-side interface between runtime.c, the launchers (.cu) and the host-pointer shims. */
#ifndef CKB200_RUNTIME_H
#define CKB200_RUNTIME_H

#include <cuda_runtime_api.h>
#include <stddef.h>

#ifdef __cplusplus
extern "C" {
#endif

enum { CKB_SLOT_W = 0, CKB_SLOT_X = 1, CKB_SLOT_Y = 2, CKB_SLOT_A = 3, CKB_SLOT_B = 4, CKB_SLOT_C = 5, CKB_SLOT_T = 6, CKB_SLOT_G = 7, CKB_SLOT_P = 8, CKB_SLOT_S = 9, CKB_NSLOTS = 10 };

int ckb_ensure_init(void);                 /* 0 or CKB_ERR_NO_DEVICE; initialises on first use */
int ckb_sm_count(void);
int *ckb_device_error_word(void);
cudaStream_t ckb_stream(void *user);       /* user stream, or the library stream when NULL */
int ckb_tune_get(const char *key, int dflt);
int ckb_is_device_ptr(const void *p);      /* device or managed memory */
int ckb_sync_check(cudaStream_t st, const char *what);   /* sync + device error word -> 0, CKB_ERR_CUDA or CKB_ERR_DEVICE_WAIT */
long long ckb_wait_limit_cycles(void);     /* tune key wait_limit_ms in SM cycles */
/* Row-planar copy (aligned 16-byte loads: gemv_q6k_planar.cu, gemv_q80_planar.cu, gemv_q50_planar.cu) of `rows` rows of a
 * REGISTERED weight range, built on first use and kept until the range is unregistered; NULL when dev_raw is not inside a
 * registered range or the cache is full.  fmt: 1 Q6_K, 2 Q8_0, 3 Q5_0. */
const void *ckb_planar_shadow(int fmt, const void *dev_raw, int rows, int cols);

/* Device scratch that grows on demand (never shrinks); one buffer per slot. */
void *ckb_scratch(int slot, size_t bytes);
/* Input staging: resident copy if registered (try_registry), the pointer itself if it is device
 * memory, else an async H2D copy into the slot.  NULL on failure. */
const void *ckb_stage_in(const void *host, size_t bytes, int slot, int try_registry);
/* Output staging: the pointer itself if device memory, else the slot (copied back by ckb_finish_out). */
void *ckb_stage_out(void *host, size_t bytes, int slot, int *needs_copy_back);
/* D2H copy when needed, then synchronise the library stream. */
int ckb_finish_out(void *host, const void *dev, size_t bytes, int needs_copy_back);
int ckb_finish_out_nowait(void *host, const void *dev, size_t bytes, int needs_copy_back);   /* kernels without bounded waits */

#ifdef __cplusplus
}
#endif
#endif
