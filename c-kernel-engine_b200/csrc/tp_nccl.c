/* Tensor-parallel exchange step: fp32 sum all-reduce of the row-parallel partial outputs (after o_proj and
 * down_proj) over NCCL / NVLink.  The reference has no collective of any kind (one process, one thread pool:
 * include/ck_threadpool.h:1-30); this is the one exchange the sharded decode step needs.
 *
 * NCCL is loaded at run time (dlopen of libnccl.so.2 - the copy a host process such as PyTorch already
 * mapped is reused), so the library itself has no link-time dependency on it.  One communicator per
 * process (one process per GPU).  The 128-byte unique id is created on rank 0 and must reach the other
 * ranks out of band (the benchmark and tests broadcast it with torch.distributed).
 */
#include <cuda_runtime_api.h>
#include <dlfcn.h>
#include <stddef.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#include "../../include/ckb200.h"
#include "../../include/ckb200_model.h"
#include "launch.h"
#include "runtime.h"

typedef struct { char internal[128]; } nccl_uid;
typedef void *nccl_comm;
enum { NCCL_FLOAT = 7, NCCL_SUM = 0 };

static struct {
    void *dl;
    int (*GetUniqueId)(nccl_uid *);
    int (*CommInitRank)(nccl_comm *, int, nccl_uid, int);
    int (*AllReduce)(const void *, void *, size_t, int, int, nccl_comm, cudaStream_t);
    int (*CommDestroy)(nccl_comm);
    const char *(*GetErrorString)(int);
    nccl_comm comm;
    int rank, world;
} g_tp;

static int tp_load(void)
{
    if (g_tp.dl) return 0;
    const char *cands[] = { getenv("CKB200_NCCL_LIB"), "libnccl.so.2", "libnccl.so" };
    for (unsigned i = 0; i < sizeof cands / sizeof cands[0] && !g_tp.dl; ++i)
        if (cands[i] && *cands[i]) g_tp.dl = dlopen(cands[i], RTLD_NOW | RTLD_GLOBAL);
    if (!g_tp.dl) return ckb_fail(CKB_ERR_STATE, "tensor parallel: cannot load libnccl.so.2 (%s)", dlerror());
    *(void **)&g_tp.GetUniqueId = dlsym(g_tp.dl, "ncclGetUniqueId");
    *(void **)&g_tp.CommInitRank = dlsym(g_tp.dl, "ncclCommInitRank");
    *(void **)&g_tp.AllReduce = dlsym(g_tp.dl, "ncclAllReduce");
    *(void **)&g_tp.CommDestroy = dlsym(g_tp.dl, "ncclCommDestroy");
    *(void **)&g_tp.GetErrorString = dlsym(g_tp.dl, "ncclGetErrorString");
    if (!g_tp.GetUniqueId || !g_tp.CommInitRank || !g_tp.AllReduce || !g_tp.CommDestroy || !g_tp.GetErrorString) {
        dlclose(g_tp.dl);
        g_tp.dl = NULL;
        return ckb_fail(CKB_ERR_STATE, "tensor parallel: libnccl is missing expected symbols");
    }
    return 0;
}

static int tp_check(int rc, const char *what)
{
    if (rc == 0) return 0;
    return ckb_fail(CKB_ERR_CUDA, "%s: NCCL error %d (%s)", what, rc, g_tp.GetErrorString ? g_tp.GetErrorString(rc) : "?");
}

int ckb200_tp_unique_id(void *out128)
{
    if (!out128) return CKB_ERR_STATE;
    if (tp_load()) return CKB_ERR_STATE;
    nccl_uid id;
    if (tp_check(g_tp.GetUniqueId(&id), "ncclGetUniqueId")) return CKB_ERR_CUDA;
    memcpy(out128, &id, sizeof id);
    return 0;
}

int ckb200_tp_init(int rank, int world, const void *id128)
{
    if (!id128 || world < 1 || rank < 0 || rank >= world) return ckb_fail(CKB_ERR_STATE, "tp_init: bad rank %d / world %d", rank, world);
    if (g_tp.comm) return 0;
    if (ckb_ensure_init()) return CKB_ERR_NO_DEVICE;
    if (tp_load()) return CKB_ERR_STATE;
    nccl_uid id;
    memcpy(&id, id128, sizeof id);
    if (tp_check(g_tp.CommInitRank(&g_tp.comm, world, id, rank), "ncclCommInitRank")) { g_tp.comm = NULL; return CKB_ERR_CUDA; }
    g_tp.rank = rank;
    g_tp.world = world;
    return 0;
}

int ckb_tp_p2p_allreduce(float *buf, size_t count, void *stream);   /* tp_p2p.cu */

/* ckb200_allreduce_fn: in-place fp32 sum over all ranks, enqueued on `stream` (capturable in a CUDA graph).
 * Vectors that fit the peer-memory exchange buffer (when the ranks have connected one) take the one-shot push
 * kernel; everything else goes through NCCL.  Every rank takes the same branch: the choice depends only on the
 * count and on state that all ranks set up together. */
int ckb200_tp_allreduce(void *ctx, float *buf, size_t count, void *stream)
{
    (void)ctx;
    if (ckb200_tp_p2p_ready() && count <= ckb200_tp_p2p_max_floats() && !((uintptr_t)buf & 15) && ckb_tune_get("tp_p2p", 1))
        return ckb_tp_p2p_allreduce(buf, count, stream);
    if (!g_tp.comm) return ckb_fail(CKB_ERR_STATE, "tp_allreduce: ckb200_tp_init has not been called");
    return tp_check(g_tp.AllReduce(buf, buf, count, NCCL_FLOAT, NCCL_SUM, g_tp.comm, ckb_stream(stream)), "ncclAllReduce");
}

int ckb200_tp_rank(void) { return g_tp.comm ? g_tp.rank : 0; }
int ckb200_tp_world(void) { return g_tp.comm ? g_tp.world : 1; }

void ckb200_tp_shutdown(void)
{
    ckb200_tp_p2p_shutdown();
    if (g_tp.comm) {
        cudaStreamSynchronize(ckb_stream(NULL));
        g_tp.CommDestroy(g_tp.comm);
        g_tp.comm = NULL;
    }
}

/* convenience: bind the all-reduce and the fused exchange + norm to a tensor-parallel model */
void ckb200_model_use_tp(CKB200Model *m)
{
    ckb200_model_set_allreduce(m, ckb200_tp_allreduce, NULL);
    ckb200_model_set_tp_norm(m, ckb200_tp_add_rmsnorm_q8k, NULL);
}
