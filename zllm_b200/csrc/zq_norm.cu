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
