/* Host runtime of libckb200.so: device selection, the library stream, the error side channel,
 * the resident-weight registry and the staging buffers behind the host-pointer entry points.
 *
 * Plain C on top of the CUDA runtime API.  One caller thread per process is assumed for the
 * compute calls, as in the reference where exactly one thread issues ops
 * (src/ck_threadpool.c:289-343: workers only run inside a blocking dispatch); the registry
 * and error state are nevertheless guarded by a mutex because tests call from Python.
 */
#include <cuda_runtime_api.h>
#include <pthread.h>
#include <stdarg.h>
#include <stdint.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#include "../../include/ckb200.h"
#include "launch.h"
#include "runtime.h"

static pthread_mutex_t g_lock = PTHREAD_MUTEX_INITIALIZER;

static struct {
    int inited;
    int device;
    int sm_count;
    cudaStream_t stream;
    int *dev_err;               /* device error word */
    int *err_pinned;            /* pinned host word the device error word is copied into before a sync */
    int clock_khz;              /* SM clock, for wait limits given in milliseconds */
    int err_code;
    char err_msg[512];
    long long launches;
} g;

/* ------------------------------------------------------------------ errors */

int ckb_fail(int code, const char *fmt, ...)
{
    char buf[512];
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(buf, sizeof buf, fmt, ap);
    va_end(ap);
    pthread_mutex_lock(&g_lock);
    if (g.err_code == 0) {
        g.err_code = code;
        snprintf(g.err_msg, sizeof g.err_msg, "%s", buf);
    }
    pthread_mutex_unlock(&g_lock);
    fprintf(stderr, "[ckb200] error %d: %s\n", code, buf);
    return code;
}

int ckb_check_cuda(int e, const char *what)
{
    if (e == (int)cudaSuccess) return 0;
    return ckb_fail(CKB_ERR_CUDA, "%s: %s", what, cudaGetErrorString((cudaError_t)e));
}

int ckb_check_launch(const char *what)
{
    ++g.launches;
    return ckb_check_cuda((int)cudaGetLastError(), what);
}

int ckb200_last_error(void) { return g.err_code; }
const char *ckb200_last_error_message(void) { return g.err_msg; }
void ckb200_clear_error(void)
{
    pthread_mutex_lock(&g_lock);
    g.err_code = 0;
    g.err_msg[0] = 0;
    pthread_mutex_unlock(&g_lock);
}
long long ckb200_launch_count(void) { return g.launches; }

/* ------------------------------------------------------------------ tuning switches */

#define CKB_MAX_TUNE 32
static struct { char key[32]; int value; } g_tune[CKB_MAX_TUNE];
static int g_ntune;

int ckb200_tune_set(const char *key, int value)
{
    if (!key) return CKB_ERR_STATE;
    for (int i = 0; i < g_ntune; ++i)
        if (!strcmp(g_tune[i].key, key)) { g_tune[i].value = value; return 0; }
    if (g_ntune == CKB_MAX_TUNE || strlen(key) >= sizeof g_tune[0].key) return CKB_ERR_LIMIT;
    strcpy(g_tune[g_ntune].key, key);
    g_tune[g_ntune++].value = value;
    return 0;
}

int ckb200_tune_get(const char *key, int dflt)
{
    for (int i = 0; i < g_ntune; ++i)
        if (!strcmp(g_tune[i].key, key)) return g_tune[i].value;
    return dflt;
}
int ckb_tune_get(const char *key, int dflt) { return ckb200_tune_get(key, dflt); }

/* ------------------------------------------------------------------ init */

int ckb200_init(int device)
{
    if (g.inited) return 0;
    int n = 0;
    if (cudaGetDeviceCount(&n) != cudaSuccess || n <= 0) {
        cudaGetLastError();
        return ckb_fail(CKB_ERR_NO_DEVICE, "no CUDA device visible; this library has no CPU fallback");
    }
    if (device < 0) {
        const char *lr = getenv("LOCAL_RANK");
        device = lr ? atoi(lr) % n : 0;
    }
    if (ckb_check_cuda((int)cudaSetDevice(device), "cudaSetDevice")) return CKB_ERR_CUDA;
    struct cudaDeviceProp prop;
    if (ckb_check_cuda((int)cudaGetDeviceProperties(&prop, device), "cudaGetDeviceProperties")) return CKB_ERR_CUDA;
    if (prop.major != 10) return ckb_fail(CKB_ERR_NO_DEVICE, "device %d is sm_%d%d; this library is built for sm_100a only",
                                          device, prop.major, prop.minor);
    g.device = device;
    g.sm_count = prop.multiProcessorCount;
    if (ckb_check_cuda((int)cudaStreamCreateWithFlags(&g.stream, cudaStreamNonBlocking), "cudaStreamCreate")) return CKB_ERR_CUDA;
    if (ckb_check_cuda((int)cudaMalloc((void **)&g.dev_err, 256), "cudaMalloc(error word)")) return CKB_ERR_CUDA;
    if (ckb_check_cuda((int)cudaMemset(g.dev_err, 0, 256), "cudaMemset(error word)")) return CKB_ERR_CUDA;
    if (ckb_check_cuda((int)cudaHostAlloc((void **)&g.err_pinned, 64, cudaHostAllocDefault), "cudaHostAlloc(error word)")) return CKB_ERR_CUDA;
    *g.err_pinned = 0;
    g.clock_khz = 0;
    cudaDeviceGetAttribute(&g.clock_khz, cudaDevAttrClockRate, device);
    if (g.clock_khz <= 0) g.clock_khz = 1965000;
    g.inited = 1;
    return 0;
}

int ckb_ensure_init(void) { return g.inited ? 0 : ckb200_init(-1); }
int ckb_sm_count(void) { return g.sm_count > 0 ? g.sm_count : 148; }
int *ckb_device_error_word(void) { return g.dev_err; }
void *ckb200_stream(void) { return ckb_ensure_init() ? NULL : (void *)g.stream; }
cudaStream_t ckb_stream(void *user) { return user ? (cudaStream_t)user : g.stream; }

/* Synchronises `st` and folds in the device error word: kernels that gave up on a bounded wait (a peer that never wrote,
 * a copy that never landed) leave a code there and return, so without this check the caller would get rc 0 and a result
 * built from stale data.  The word travels in the same stream, just before the sync (4 bytes, pinned). */
int ckb_sync_check(cudaStream_t st, const char *what)
{
    if (ckb_check_cuda((int)cudaMemcpyAsync(g.err_pinned, g.dev_err, sizeof(int), cudaMemcpyDeviceToHost, st), "read error word")) return CKB_ERR_CUDA;
    if (ckb_check_cuda((int)cudaStreamSynchronize(st), what)) return CKB_ERR_CUDA;
    const int word = *g.err_pinned;
    if (word != 0) {
        cudaMemsetAsync(g.dev_err, 0, sizeof(int), st);
        cudaStreamSynchronize(st);
        *g.err_pinned = 0;
        return ckb_fail(CKB_ERR_DEVICE_WAIT, "%s: a kernel gave up on a bounded wait (device code %d)", what, word);
    }
    return 0;
}

int ckb200_synchronize(void)
{
    if (ckb_ensure_init()) return CKB_ERR_NO_DEVICE;
    return ckb_sync_check(g.stream, "ckb200_synchronize");
}

/* Limit of the waits on another GPU, in SM clock cycles: tune key wait_limit_ms (default 10 s: ranks reach their first
 * step at different times). */
long long ckb_wait_limit_cycles(void)
{
    int ms = ckb200_tune_get("wait_limit_ms", 10000);
    if (ms < 1) ms = 1;
    return (long long)ms * (long long)(g.clock_khz > 0 ? g.clock_khz : 1965000);
}

/* ------------------------------------------------------------------ resident weights */

#define CKB_MAX_REG 256
static struct { const uint8_t *host; size_t bytes; uint8_t *dev; } g_reg[CKB_MAX_REG];
static int g_nreg;

int ckb200_register_weights(const void *host_ptr, size_t bytes)
{
    if (!host_ptr || bytes == 0) return ckb_fail(CKB_ERR_STATE, "register_weights: empty range");
    if (ckb_ensure_init()) return CKB_ERR_NO_DEVICE;
    ckb200_unregister_weights(host_ptr);
    if (g_nreg == CKB_MAX_REG) return ckb_fail(CKB_ERR_LIMIT, "register_weights: more than %d ranges", CKB_MAX_REG);
    uint8_t *dev = NULL;
    /* 256 spare bytes: the bulk-copy GEMVs read the 16-byte aligned superset of a row range */
    if (ckb_check_cuda((int)cudaMalloc((void **)&dev, bytes + 256), "cudaMalloc(weights)")) return CKB_ERR_CUDA;
    if (ckb_check_cuda((int)cudaMemcpy(dev, host_ptr, bytes, cudaMemcpyHostToDevice), "upload weights")) {
        cudaFree(dev);
        return CKB_ERR_CUDA;
    }
    cudaMemset(dev + bytes, 0, 256);
    pthread_mutex_lock(&g_lock);
    g_reg[g_nreg].host = (const uint8_t *)host_ptr;
    g_reg[g_nreg].bytes = bytes;
    g_reg[g_nreg].dev = dev;
    ++g_nreg;
    pthread_mutex_unlock(&g_lock);
    return 0;
}

/* ---- row-planar shadows of registered weights (the reference's 210- / 34- / 22-byte blocks are only 2-byte aligned) */
size_t ckb200_q6_k_planar_bytes(int rows, int cols);
size_t ckb200_q8_0_planar_bytes(int rows, int cols);
size_t ckb200_q5_0_planar_bytes(int rows, int cols);
int ckb200_dev_q6_k_to_planar(void *dst, const void *src, int rows, int cols, void *stream);
int ckb200_dev_q8_0_to_planar(void *dst, const void *src, int rows, int cols, void *stream);
int ckb200_dev_q5_0_to_planar(void *dst, const void *src, int rows, int cols, void *stream);

#define CKB_MAX_SHADOW 256
static struct { const uint8_t *raw; void *planar; int fmt, rows, cols; } g_shadow[CKB_MAX_SHADOW];
static int g_nshadow;

static void drop_shadows_in(const uint8_t *dev, size_t bytes)
{
    for (int i = 0; i < g_nshadow;) {
        if (g_shadow[i].raw >= dev && g_shadow[i].raw < dev + bytes) {
            cudaFree(g_shadow[i].planar);
            g_shadow[i] = g_shadow[--g_nshadow];
        } else {
            ++i;
        }
    }
}

const void *ckb_planar_shadow(int fmt, const void *dev_raw, int rows, int cols)
{
    const uint8_t *p = (const uint8_t *)dev_raw;
    if (!ckb200_tune_get("planar_shadow", 1)) return NULL;
    for (int i = 0; i < g_nshadow; ++i)
        if (g_shadow[i].raw == p && g_shadow[i].fmt == fmt && g_shadow[i].rows == rows && g_shadow[i].cols == cols) return g_shadow[i].planar;
    int inside = 0;
    pthread_mutex_lock(&g_lock);
    for (int i = 0; i < g_nreg; ++i)
        if (p >= g_reg[i].dev && p < g_reg[i].dev + g_reg[i].bytes) { inside = 1; break; }
    pthread_mutex_unlock(&g_lock);
    if (!inside || g_nshadow == CKB_MAX_SHADOW || ((uintptr_t)p & 15)) return NULL;
    const size_t bytes = fmt == 1 ? ckb200_q6_k_planar_bytes(rows, cols) : (fmt == 2 ? ckb200_q8_0_planar_bytes(rows, cols) : ckb200_q5_0_planar_bytes(rows, cols));
    if (!bytes) return NULL;
    void *dst = NULL;
    if (cudaMalloc(&dst, bytes + 256) != cudaSuccess) { cudaGetLastError(); return NULL; }
    const int rc = fmt == 1 ? ckb200_dev_q6_k_to_planar(dst, p, rows, cols, NULL) : (fmt == 2 ? ckb200_dev_q8_0_to_planar(dst, p, rows, cols, NULL)
                                                                                             : ckb200_dev_q5_0_to_planar(dst, p, rows, cols, NULL));
    if (rc) { cudaFree(dst); return NULL; }
    g_shadow[g_nshadow].raw = p;
    g_shadow[g_nshadow].planar = dst;
    g_shadow[g_nshadow].fmt = fmt;
    g_shadow[g_nshadow].rows = rows;
    g_shadow[g_nshadow].cols = cols;
    ++g_nshadow;
    return dst;
}

int ckb200_unregister_weights(const void *host_ptr)
{
    pthread_mutex_lock(&g_lock);
    for (int i = 0; i < g_nreg; ++i)
        if (g_reg[i].host == (const uint8_t *)host_ptr) {
            uint8_t *dev = g_reg[i].dev;
            const size_t bytes = g_reg[i].bytes;
            g_reg[i] = g_reg[--g_nreg];
            pthread_mutex_unlock(&g_lock);
            cudaStreamSynchronize(g.stream);
            drop_shadows_in(dev, bytes);
            cudaFree(dev);
            return 0;
        }
    pthread_mutex_unlock(&g_lock);
    return 1;
}

void ckb200_unregister_all(void)
{
    while (g_nreg > 0) ckb200_unregister_weights(g_reg[0].host);
}

const void *ckb200_device_ptr(const void *host_ptr)
{
    const uint8_t *p = (const uint8_t *)host_ptr;
    const void *out = NULL;
    pthread_mutex_lock(&g_lock);
    for (int i = 0; i < g_nreg; ++i)
        if (p >= g_reg[i].host && p < g_reg[i].host + g_reg[i].bytes) { out = g_reg[i].dev + (p - g_reg[i].host); break; }
    pthread_mutex_unlock(&g_lock);
    return out;
}

int ckb200_copy_to_device(void *dev, const void *host, size_t bytes)
{
    if (ckb_ensure_init()) return CKB_ERR_NO_DEVICE;
    cudaStreamSynchronize(g.stream);
    return ckb_check_cuda((int)cudaMemcpy(dev, host, bytes, cudaMemcpyHostToDevice), "copy_to_device");
}

int ckb200_copy_to_host(void *host, const void *dev, size_t bytes)
{
    if (ckb_ensure_init()) return CKB_ERR_NO_DEVICE;
    cudaStreamSynchronize(g.stream);
    return ckb_check_cuda((int)cudaMemcpy(host, dev, bytes, cudaMemcpyDeviceToHost), "copy_to_host");
}

/* Pinned ranges handed out by ckb200_host_alloc: a pointer inside one is host memory by construction, so the staging code
 * need not ask the driver what it is (a pointer-attribute query per argument is a measurable part of a small host call). */
#define CKB_MAX_PINNED 64
#define CKB_STAGING_KERNEL_MAX ((size_t)4 << 20)       /* above this the copy engine's bandwidth matters more than its start-up */
int ckb_staging_copy(void *dst, const void *src, size_t bytes, cudaStream_t st);       /* staging.cu */
static struct { const uint8_t *p; size_t bytes; } g_pinned[CKB_MAX_PINNED];
static int g_npinned;

static int known_pinned(const void *p)
{
    for (int i = 0; i < g_npinned; ++i)
        if ((const uint8_t *)p >= g_pinned[i].p && (const uint8_t *)p < g_pinned[i].p + g_pinned[i].bytes) return 1;
    return 0;
}

void *ckb200_host_alloc(size_t bytes)
{
    void *p = NULL;
    if (ckb_ensure_init()) return NULL;
    if (ckb_check_cuda((int)cudaHostAlloc(&p, bytes, cudaHostAllocMapped | cudaHostAllocPortable), "cudaHostAlloc")) return NULL;
    pthread_mutex_lock(&g_lock);
    if (g_npinned < CKB_MAX_PINNED) { g_pinned[g_npinned].p = (const uint8_t *)p; g_pinned[g_npinned].bytes = bytes; ++g_npinned; }
    pthread_mutex_unlock(&g_lock);
    return p;
}
void ckb200_host_free(void *p)
{
    if (!p) return;
    pthread_mutex_lock(&g_lock);
    for (int i = 0; i < g_npinned; ++i)
        if (g_pinned[i].p == (const uint8_t *)p) { g_pinned[i] = g_pinned[--g_npinned]; break; }
    pthread_mutex_unlock(&g_lock);
    cudaFreeHost(p);
}

/* ------------------------------------------------------------------ staging for host pointers */

static struct { uint8_t *p; size_t cap; } g_slot[CKB_NSLOTS];

void *ckb_scratch(int slot, size_t bytes)
{
    if (bytes <= g_slot[slot].cap) return g_slot[slot].p;
    if (g_slot[slot].p) {
        cudaStreamSynchronize(g.stream);
        cudaFree(g_slot[slot].p);
        g_slot[slot].p = NULL;
        g_slot[slot].cap = 0;
    }
    size_t cap = (bytes + 256 + ((size_t)1 << 20) - 1) & ~(((size_t)1 << 20) - 1);
    if (ckb_check_cuda((int)cudaMalloc((void **)&g_slot[slot].p, cap), "cudaMalloc(staging)")) return NULL;
    g_slot[slot].cap = cap;
    return g_slot[slot].p;
}

int ckb_is_device_ptr(const void *p)
{
    struct cudaPointerAttributes a;
    if (known_pinned(p)) return 0;
    if (cudaPointerGetAttributes(&a, p) != cudaSuccess) { cudaGetLastError(); return 0; }
    return a.type == cudaMemoryTypeDevice || a.type == cudaMemoryTypeManaged;
}

const void *ckb_stage_in(const void *host, size_t bytes, int slot, int try_registry)
{
    if (try_registry) {
        const void *d = ckb200_device_ptr(host);
        if (d) return d;
    }
    if (ckb_is_device_ptr(host)) return host;
    void *d = ckb_scratch(slot, bytes);
    if (!d) return NULL;
    /* inputs stay with the copy engine: fetching a 4.6 KB activation row by a kernel (reads across the bus from the SMs) measured
     * about 4 us SLOWER than the engine's copy; only the way back gains from the kernel (copy_back below) */
    if (ckb_check_cuda((int)cudaMemcpyAsync(d, host, bytes, cudaMemcpyHostToDevice, g.stream), "H2D")) return NULL;
    return d;
}

static int copy_back(void *host, const void *dev, size_t bytes)
{
    if (bytes <= CKB_STAGING_KERNEL_MAX && known_pinned(host) && ckb200_tune_get("staging_kernel", 1)) return ckb_staging_copy(host, dev, bytes, g.stream);
    return ckb_check_cuda((int)cudaMemcpyAsync(host, dev, bytes, cudaMemcpyDeviceToHost, g.stream), "D2H") ? CKB_ERR_CUDA : 0;
}

void *ckb_stage_out(void *host, size_t bytes, int slot, int *needs_copy_back)
{
    if (ckb_is_device_ptr(host)) { *needs_copy_back = 0; return host; }
    *needs_copy_back = 1;
    return ckb_scratch(slot, bytes);
}

int ckb_finish_out(void *host, const void *dev, size_t bytes, int needs_copy_back)
{
    if (needs_copy_back && copy_back(host, dev, bytes)) return CKB_ERR_CUDA;
    return ckb_sync_check(g.stream, "sync");
}

/* The same for calls whose kernels contain no bounded wait (nothing in them can set the device error word): the 4-byte read of the
 * word is left to the next call that needs it. */
int ckb_finish_out_nowait(void *host, const void *dev, size_t bytes, int needs_copy_back)
{
    if (needs_copy_back && copy_back(host, dev, bytes)) return CKB_ERR_CUDA;
    return ckb_check_cuda((int)cudaStreamSynchronize(g.stream), "sync") ? CKB_ERR_CUDA : 0;
}

void ckb200_shutdown(void)
{
    if (!g.inited) return;
    cudaStreamSynchronize(g.stream);
    ckb200_unregister_all();
    for (int i = 0; i < CKB_NSLOTS; ++i) {
        if (g_slot[i].p) cudaFree(g_slot[i].p);
        g_slot[i].p = NULL;
        g_slot[i].cap = 0;
    }
    cudaFree(g.dev_err);
    cudaFreeHost(g.err_pinned);
    cudaStreamDestroy(g.stream);
    g.inited = 0;
}
