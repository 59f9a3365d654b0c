/* Host-side plumbing shared by every launcher: the error side channel and the launch counter.
 *
 * The reference's kernels are `void` and return silently on bad arguments
 * (e.g. src/kernels/gemm_kernels_q4k_q8k.c:188-190), so errors that only exist on a GPU
 * (no device, bad alignment, a failed launch) are recorded here and read back through
 * ckb200_last_error(); nothing aborts the process.
 */
#ifndef CKB200_LAUNCH_H
#define CKB200_LAUNCH_H

#ifdef __cplusplus
extern "C" {
#endif

enum {
    CKB_OK = 0,
    CKB_ERR_CUDA = 1,       /* a CUDA runtime call or a launch failed */
    CKB_ERR_SHAPE = 2,      /* dimension not supported by the format (K % 256, K % 32, ...) */
    CKB_ERR_ALIGN = 3,      /* pointer alignment the kernel needs is not met */
    CKB_ERR_NO_DEVICE = 4,  /* no CUDA device: there is no CPU fallback */
    CKB_ERR_DEVICE_WAIT = 5,/* a kernel gave up on a bounded wait (device error word set) */
    CKB_ERR_LIMIT = 6,      /* a documented size limit was exceeded */
    CKB_ERR_STATE = 7       /* call made in the wrong state (model not loaded, ...) */
};

/* Records the error (first one wins until cleared), prints it to stderr, returns `code`. */
int ckb_fail(int code, const char *fmt, ...);
/* cudaGetLastError() after a launch; counts the launch; returns 0 or CKB_ERR_CUDA. */
int ckb_check_launch(const char *what);
/* Returns 0 or records CKB_ERR_CUDA for a cudaError_t passed as int. */
int ckb_check_cuda(int cuda_error, const char *what);

#ifdef __cplusplus
}
#endif
#endif
