// Host-side interface of the work-list decode kernel (zq_gemv_wl.cu): a list of independent projections, each
// y[m, rows] = x[m, cols] W^T (+ residual), or silu(x gate^T) * (x up^T) when `w_up` is given, run in as few launches as
// their (weight type, row count, plain / gated) classes allow.
#pragma once
#include "zq_common.cuh"

namespace zq {

constexpr int kWlMaxJobs = 32;  // jobs per launch (the job table travels as a kernel parameter)

struct WlHostJob {
    const zq_weight *w;
    const zq_weight *w_up;  // gated pair, or null
    const void *x;          // [m, cols]
    size_t m;               // 1..16
    void *y;                // [m, rows]
    const void *residual;   // [m, rows] in the output dtype, or null
    int y_dtype;            // output dtype of this job, or -1 for the call's
};

// True when the job can ride in a work-list launch (Q4_K / Q4_0 / Q8_0, up to 16 activation rows).
bool gemv_wl_supported(const zq_ctx *ctx, const WlHostJob &job);
int launch_gemv_wl(zq_ctx *ctx, const WlHostJob *jobs, size_t n_jobs, int x_dtype, int y_dtype, zq_error *err);

}  // namespace zq
