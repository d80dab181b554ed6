// Kernel-side description of one fused dequant-GEMV product (built by the host from GemvArgs).
#pragma once
#include <stdint.h>

#include "stage.cuh"

namespace juno {

struct GemvParams {
    const uint8_t *w[3];
    float *out[3];
    int rows[3];
    int seg_type[3];  // block format per segment (used by mixed launches)
    int rt_begin[4];  // cumulative row-tile starts, rt_begin[nseg] = total
    int nseg, total_rt;
    int K, nb;
    int kin, tpt, groups, n_ctasks;  // warps per row tile, tiles per warp per task, row tiles per CTA task
    int ld_out, epi;
    const uint8_t *ximg;
    unsigned img_bytes;
    unsigned *counters;  // {next task, CTAs done}
    // RMSNorm scale of the input, applied to the outputs: 1/sqrt(sum(ss_parts[b][0..n_parts))/scale_n + eps)
    const float *ss_parts;
    int n_parts, ss_ld, scale_n;
    float eps;
    // EPI_RESID_NORM: x_out = resid + y; image of normw_next*x_out; per-task sums of squares
    const float *resid;
    float *x_out;
    int ldx;
    const float *normw_next;
    float *ss_out;
    int ss_out_ld;
    StageImage img_next;  // also used by EPI_SILU_PAIR / EPI_STORE to emit the output as a staged activation
    // L2 prefetch hints issued by every CTA, at kernel entry before it waits for the producer of x: row tiles
    // [0, pf_rt) of this product (the CTA tasks that are handed out first), and up to three byte ranges of the
    // products that follow in the stream (each CTA takes a 1/grid slice).
    int pf_rt;
    int pf_late;  // the ranges of the following products are requested when the CTA runs out of tasks, not at entry
    const uint8_t *pfx[3];
    unsigned pfx_bytes[3];
};

__device__ __forceinline__ int seg_of(const GemvParams &p, int R) {
    int s = 0;
    if (p.nseg > 1 && R >= p.rt_begin[1]) s = 1;
    if (p.nseg > 2 && R >= p.rt_begin[2]) s = 2;
    return s;
}
}  // namespace juno
