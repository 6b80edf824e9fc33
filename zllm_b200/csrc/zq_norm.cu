// RMSNorm in front of a quantized projection: Backend::rmsnorm_linear / rmsnorm_dual_linear
// (src/backend/mod.rs:455-464) = rmsnorm (src/kernel/cpu/rmsnorm.rs:7-41), then the linear layer(s).
//   out[i] = x[i] * (1 / sqrt(mean(x^2) + eps)) * (w[i] + weight_offset)     (offset 1 = the "Gemma" form)
// One CTA per activation row writes the normalised row as f32 into a context buffer; the projection that follows is
// launched with programmatic dependent launch, so its weight prefetch runs under this kernel and the normalised row
// never leaves L2.  The operation order of the scaling is the reference's (x * inv_rms, then * weight); the sum of
// squares is a tree sum, which differs from the reference's 8-lane running sums in the last bits only.
#include "zq_common.cuh"

namespace zq {

__global__ void __launch_bounds__(256) rmsnorm_kernel(const void *__restrict__ x, int x_dtype, int cols, const float *__restrict__ weight, float eps, float weight_offset, float *__restrict__ out) {
    pdl_launch_dependents();
    pdl_wait_prior_grid();  // the input belongs to the previous kernel until it completes
    __shared__ float partial[8];
    __shared__ float s_inv;
    const size_t base = (size_t)blockIdx.x * cols;
    float acc = 0.f;
    for (int i = threadIdx.x; i < cols; i += blockDim.x) {
        const float v = load_as_f32(x, x_dtype, base + i);
        acc = fmaf(v, v, acc);
    }
#pragma unroll
    for (int s = 16; s > 0; s >>= 1) acc += __shfl_xor_sync(0xFFFFFFFFu, acc, s);
    if ((threadIdx.x & 31) == 0) partial[threadIdx.x >> 5] = acc;
    __syncthreads();
    if (threadIdx.x == 0) {
        float total = 0.f;
        for (int w = 0; w < 8; ++w) total += partial[w];
        const float mean_sq = __fdiv_rn(total, (float)cols);
        s_inv = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(mean_sq, eps)));
    }
    __syncthreads();
    const float inv = s_inv;
    for (int i = threadIdx.x; i < cols; i += blockDim.x) {
        const float v = load_as_f32(x, x_dtype, base + i);
        const float w = weight_offset == 0.0f ? weight[i] : __fadd_rn(weight_offset, weight[i]);
        out[base + i] = __fmul_rn(__fmul_rn(v, inv), w);
    }
}

int launch_rmsnorm(zq_ctx *ctx, const void *x, int x_dtype, size_t m, size_t cols, const float *weight, float eps, float weight_offset, float *out, zq_error *err) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)m);
    cfg.blockDim = dim3(256);
    cfg.stream = ctx->stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = ctx->disable_pdl ? 0 : 1;
    ZQ_CUDA_CHECK(cudaLaunchKernelEx(&cfg, rmsnorm_kernel, x, x_dtype, (int)cols, weight, eps, weight_offset, out), err);
    ctx->launches++;
    return ZQ_OK;
}

}  // namespace zq

// ---------------------------------------------------------------------------------------------------------------
// Arg-max over the columns of every row: the greedy token choice behind an LM-head projection, left on the device so
// that the logits (vocabulary x 4 bytes per row) never travel to the host.  Ties go to the lower index; NaN entries are
// never chosen (a row of nothing but NaN yields index 0).  One CTA per row.
// ---------------------------------------------------------------------------------------------------------------
namespace zq {

__global__ void __launch_bounds__(1024) argmax_rows_kernel(const void *__restrict__ x, int dtype, int cols, uint32_t *__restrict__ out) {
    pdl_launch_dependents();
    pdl_wait_prior_grid();
    const size_t row = blockIdx.x;
    float best = -INFINITY;
    int best_i = 0x7fffffff;
    for (int c = threadIdx.x; c < cols; c += blockDim.x) {
        const float v = load_as_f32(x, dtype, row * cols + c);
        if (v > best || (v == best && c < best_i)) { best = v; best_i = c; }
    }
    __shared__ float s_best[32];
    __shared__ int s_idx[32];
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, best, o);
        const int oi = __shfl_xor_sync(0xffffffffu, best_i, o);
        if (ov > best || (ov == best && oi < best_i)) { best = ov; best_i = oi; }
    }
    if ((threadIdx.x & 31) == 0) {
        s_best[threadIdx.x >> 5] = best;
        s_idx[threadIdx.x >> 5] = best_i;
    }
    __syncthreads();
    if (threadIdx.x < 32) {
        const int warps = (blockDim.x + 31) / 32;
        best = threadIdx.x < warps ? s_best[threadIdx.x] : -INFINITY;
        best_i = threadIdx.x < warps ? s_idx[threadIdx.x] : 0x7fffffff;
        for (int o = 16; o > 0; o >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, best, o);
            const int oi = __shfl_xor_sync(0xffffffffu, best_i, o);
            if (ov > best || (ov == best && oi < best_i)) { best = ov; best_i = oi; }
        }
        if (threadIdx.x == 0) out[row] = best_i == 0x7fffffff ? 0u : (uint32_t)best_i;
    }
}

}  // namespace zq

extern "C" int zq_argmax_rows(zq_ctx *ctx, const void *dev_x, int dtype, size_t rows, size_t cols, uint32_t *dev_ids, zq_error *err) {
    using namespace zq;
    if (!ctx || !dev_x || !dev_ids) return set_error(err, ZQ_ERR_ARG, "zq_argmax_rows: null argument");
    if (dtype != ZQ_F32 && dtype != ZQ_F16 && dtype != ZQ_BF16) return set_error(err, ZQ_ERR_ARG, "zq_argmax_rows: unknown dtype %d", dtype);
    if (rows == 0 || cols == 0 || cols > (size_t)INT32_MAX || rows > (size_t)INT32_MAX) return set_error(err, ZQ_ERR_SHAPE, "zq_argmax_rows: shape [%zu, %zu]", rows, cols);
    int rc = use_device(ctx, err);
    if (rc) return rc;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)rows);
    cfg.blockDim = dim3(1024);
    cfg.stream = ctx->stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = ctx->disable_pdl ? 0 : 1;
    ZQ_CUDA_CHECK(cudaLaunchKernelEx(&cfg, argmax_rows_kernel, dev_x, dtype, (int)cols, dev_ids), err);
    ctx->launches++;
    return ZQ_OK;
}

// LM head: logits = W x into a context buffer (f32), then the arg-max of every row.
extern "C" int zq_lm_head_argmax(zq_ctx *ctx, const zq_weight *head, const void *dev_x, int x_dtype, size_t m, uint32_t *dev_ids, zq_error *err) {
    using namespace zq;
    if (!ctx || !head || !dev_x || !dev_ids) return set_error(err, ZQ_ERR_ARG, "zq_lm_head_argmax: null argument");
    if (m == 0) return set_error(err, ZQ_ERR_SHAPE, "zq_lm_head_argmax: no rows");
    int rc = ensure_scratch_norm(ctx, m * head->rows * sizeof(float) + 256, err);  // the logits share the buffer of the normalised rows
    if (rc) return rc;
    rc = zq_linear(ctx, head, dev_x, x_dtype, m, ctx->norm, ZQ_F32, nullptr, err);
    if (rc) return rc;
    return zq_argmax_rows(ctx, ctx->norm, ZQ_F32, m, head->rows, dev_ids, err);
}
