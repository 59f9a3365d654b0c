/* Arguments of the fused step GEMV (step_fused.cu): one launch = an activation-producing prologue, up to three row segments of
 * dequant-dot products over the same quantised input vector, and a per-segment epilogue.  Plain C: model.c fills it. */
#ifndef CKB200_STEP_FUSED_H
#define CKB200_STEP_FUSED_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

enum {                      /* how the Q8_K input vector comes to be */
    SG_PRO_GLOBAL = 0,      /* already quantised, in global memory (xq) */
    SG_PRO_NORM = 1,        /* x_new = x_in + delta; out = Q8_K(rmsnorm(x_new) * gamma); the first CTA also writes x_new to x_out */
    SG_PRO_QUANT = 2        /* out = Q8_K(src), src an fp32 row of nb * 256 values whose tail beyond the data is zero */
};

enum {                      /* what happens to the finished dot products of a segment */
    SG_EPI_STORE = 0,       /* out[row] = s */
    SG_EPI_ROPE_Q = 1,      /* rows (j, j + d/2) of a head are rotated with cos/sin[pos][j] and written to out (the query) */
    SG_EPI_ROPE_K = 2,      /* the same, written into the key cache row of position pos */
    SG_EPI_STORE_V = 3,     /* written into the value cache row of position pos */
    SG_EPI_SWIGLU = 4       /* rows (j, j + M/2) are gate and up of output j: out[j] = silu(gate) * up */
};

enum { SG_FMT_Q4K = 0, SG_FMT_Q6K_PLANAR = 1 };

typedef struct {
    const uint8_t *W;       /* Q4_K rows as in the reference, or Q6_K rows in the row-planar layout */
    float *out;             /* y / q / activation row; the cache base for SG_EPI_ROPE_K and SG_EPI_STORE_V */
    int M;                  /* rows */
    int fmt;
    int epi;
    int cta0, ncta;         /* the CTAs [cta0, cta0 + ncta) of the grid work on this segment */
    int split;              /* the passes of a row go to different warps of a CTA (small matrices with long rows); needs
                               ckb_step_gemv_passes() <= 8 for the segment's format */
} StepSeg;

typedef struct {
    StepSeg seg[3];
    int nseg;
    int nb;                 /* superblocks per row (K / 256), the same for all segments */
    int pro;
    const uint8_t *xq;      /* SG_PRO_GLOBAL */
    const float *x_in, *delta, *gamma;     /* SG_PRO_NORM (delta may be NULL) */
    float *x_out;           /* SG_PRO_NORM: where the first CTA stores x_in + delta (NULL: nowhere) */
    int d_model;
    float eps;
    const float *src;       /* SG_PRO_QUANT */
    const float *cos_cache, *sin_cache;    /* [max_seq][head_dim / 2] */
    const int *pos;         /* device position (rope and cache epilogues) */
    int *pos_advance;       /* when not NULL the first CTA stores *pos_advance + 1 there after its rows (end of a step) */
    int head_dim, max_seq;
    int dry_run;            /* rehearse prologue, product and epilogue before the dependency wait (stores off): warms the instruction
                               caches; an instantiation of its own with more registers, for small matrices */
} StepGemvParams;

/* grid = total CTAs (sum of ncta).  Returns 0 or a CKB_ERR_* code; -1 when the shape is outside what the kernel handles. */
int ckb_launch_step_gemv(const StepGemvParams *p, int grid, void *stream);
/* passes a warp needs for one row of nb superblocks in the given format */
int ckb_step_gemv_passes(int nb, int fmt);
/* the largest row (in superblocks) whose SG_PRO_NORM prologue the kernel handles */
#define SG_NORM_MAX_NB 8
/* resident CTAs per SM of the instantiation that handles rows of nb superblocks with this prologue (for sizing the grid) */
int ckb_step_gemv_ctas_per_sm(int nb, int pro, int dry_run);

#ifdef __cplusplus
}
#endif
#endif
