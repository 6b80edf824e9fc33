// Rotary position embedding on projection outputs: the step behind the q and k projections of a decode step.
//
// Reference: Backend::rope / rope_prefix / rope_prefix_qk (src/backend/mod.rs:545-583); arithmetic
// attention::rope::apply_f32 (src/attention/rope.rs:120-165):
//     out[real] = real * cos - imaginary * sin;   out[imaginary] = imaginary * cos + real * sin
// with separately rounded products (the CPU fast path keeps that order too, src/backend/cpu/context.rs:590-625), so f32
// rows come out bit-identical to the CPU path; half-precision rows are computed in f32 and rounded once.  q and k (their
// head counts may differ: grouped-query attention) are rotated by ONE launch, in place.
#include "zq_common.cuh"

namespace zq {

struct RopeArgs {
    void *q, *k;               // [rows, q_heads * head_dim], [rows, k_heads * head_dim]; k may be null
    const float *cos_table, *sin_table;  // [positions, rotary_dim / 2]
    int dtype, rows, q_heads, k_heads, head_dim, rotary_dim, layout, placement, position;
};

__global__ void __launch_bounds__(256) rope_kernel(const RopeArgs a) {
    pdl_launch_dependents();
    pdl_wait_prior_grid();  // q and k come from the projections launched just before
    const int half = a.rotary_dim / 2, heads = a.q_heads + a.k_heads;
    const long long total = (long long)a.rows * heads * half;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
        const int pair = (int)(i % half);
        const long long rest = i / half;
        const int head = (int)(rest % heads), row = (int)(rest / heads);
        const bool is_k = head >= a.q_heads;
        void *base = is_k ? a.k : a.q;
        const int h = is_k ? head - a.q_heads : head, cols = (is_k ? a.k_heads : a.q_heads) * a.head_dim;
        const size_t start = (size_t)row * cols + (size_t)h * a.head_dim + (a.placement == 0 ? 0 : a.head_dim - a.rotary_dim);
        const size_t ri = start + (a.layout == 0 ? pair : 2 * pair), ii = start + (a.layout == 0 ? half + pair : 2 * pair + 1);
        const float c = a.cos_table[(size_t)(a.position + row) * half + pair], s = a.sin_table[(size_t)(a.position + row) * half + pair];
        const float real = load_as_f32(base, a.dtype, ri), imaginary = load_as_f32(base, a.dtype, ii);
        store_from_f32(base, a.dtype, ri, __fsub_rn(__fmul_rn(real, c), __fmul_rn(imaginary, s)));
        store_from_f32(base, a.dtype, ii, __fadd_rn(__fmul_rn(imaginary, c), __fmul_rn(real, s)));
    }
}

}  // namespace zq

using namespace zq;

extern "C" int zq_rope_qk(zq_ctx *ctx, void *dev_q, size_t q_heads, void *dev_k, size_t k_heads, int dtype, size_t rows, size_t head_dim, size_t rotary_dim, int layout, int placement, size_t position,
                          const float *dev_cos, const float *dev_sin, size_t table_len, zq_error *err) {
    if (!ctx || !dev_q || !dev_cos || !dev_sin) return set_error(err, ZQ_ERR_ARG, "zq_rope_qk: null argument");
    if (dtype != ZQ_F32 && dtype != ZQ_F16 && dtype != ZQ_BF16) return set_error(err, ZQ_ERR_ARG, "zq_rope_qk: unknown dtype %d", dtype);
    if ((layout != ZQ_ROPE_SPLIT_HALF && layout != ZQ_ROPE_INTERLEAVED) || (placement != ZQ_ROPE_PREFIX && placement != ZQ_ROPE_SUFFIX)) return set_error(err, ZQ_ERR_ARG, "zq_rope_qk: unknown layout %d or placement %d", layout, placement);
    // the reference's parameter errors (src/attention/rope.rs:124-139)
    if (q_heads == 0 || rotary_dim == 0 || rotary_dim % 2 || head_dim == 0) return set_error(err, ZQ_ERR_SHAPE, "zq_rope_qk: heads=%zu head_dim=%zu rotary=%zu (rotary must be even and positive)", q_heads, head_dim, rotary_dim);
    if (rotary_dim > head_dim) return set_error(err, ZQ_ERR_SHAPE, "zq_rope_qk: rotary=%zu exceeds head_dim=%zu", rotary_dim, head_dim);
    if (dev_k && k_heads == 0) return set_error(err, ZQ_ERR_SHAPE, "zq_rope_qk: key given with zero heads");
    if (rows == 0) return set_error(err, ZQ_ERR_SHAPE, "zq_rope_qk: no rows");
    if ((position + rows) * (rotary_dim / 2) > table_len) return set_error(err, ZQ_ERR_SHAPE, "zq_rope_qk: the tables hold %zu values, %zu are needed", table_len, (position + rows) * (rotary_dim / 2));
    if (rows > (size_t)INT32_MAX / 4 || position > (size_t)INT32_MAX / 4 || (q_heads + k_heads) * head_dim > (size_t)INT32_MAX / 4) return set_error(err, ZQ_ERR_SHAPE, "zq_rope_qk: shape too large");
    int rc = use_device(ctx, err);
    if (rc) return rc;
    RopeArgs a;
    a.q = dev_q;
    a.k = dev_k;
    a.cos_table = dev_cos;
    a.sin_table = dev_sin;
    a.dtype = dtype;
    a.rows = (int)rows;
    a.q_heads = (int)q_heads;
    a.k_heads = dev_k ? (int)k_heads : 0;
    a.head_dim = (int)head_dim;
    a.rotary_dim = (int)rotary_dim;
    a.layout = layout;
    a.placement = placement;
    a.position = (int)position;
    const size_t total = rows * (size_t)(a.q_heads + a.k_heads) * (rotary_dim / 2);
    size_t blocks = (total + 255) / 256;
    if (blocks > (size_t)ctx->sm_count * 8) blocks = (size_t)ctx->sm_count * 8;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)blocks);
    cfg.blockDim = dim3(256);
    cfg.stream = ctx->stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = ctx->disable_pdl ? 0 : 1;
    ZQ_CUDA_CHECK(cudaLaunchKernelEx(&cfg, rope_kernel, a), err);
    ctx->launches++;
    return ZQ_OK;
}
