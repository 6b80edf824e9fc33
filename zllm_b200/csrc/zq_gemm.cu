// Prefill GEMM entry (placeholder body: rows are processed in groups of 8 by the decode kernel until the
// tcgen05 pipeline lands).
#include "zq_common.cuh"

namespace zq {
int launch_gemm(zq_ctx *ctx, const zq_weight *w, const zq_weight *w_up, const void *x, int x_dtype, size_t m, void *y, int y_dtype, const void *residual, zq_error *err) {
    return launch_gemv(ctx, w, w_up, x, x_dtype, m, y, y_dtype, residual, err);
}
}  // namespace zq
