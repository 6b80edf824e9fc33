// C-ABI entry points, context and resident-weight management of the zq_b200 library.
#include "zq_common.cuh"
#include "zq_dist.cuh"
#include "zq_wl.cuh"

namespace zq {

int set_error(zq_error *err, int code, const char *fmt, ...) {
    if (err) {
        va_list args;
        va_start(args, fmt);
        vsnprintf(err->message, sizeof(err->message), fmt, args);
        va_end(args);
    }
    return code;
}

// cuTensorMapEncodeTiled is fetched through the runtime so that the library does not link libcuda and can be
// loaded (symbols inspected, argument checks exercised) on a machine without a driver.
EncodeTiledFn get_encode_tiled(zq_error *err) {
    static EncodeTiledFn fn = nullptr;
    static std::once_flag once;
    std::call_once(once, [] {
        void *ptr = nullptr;
        cudaDriverEntryPointQueryResult qres;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &qres) == cudaSuccess && qres == cudaDriverEntryPointSuccess) fn = reinterpret_cast<EncodeTiledFn>(ptr);
    });
    if (!fn) set_error(err, ZQ_ERR_CUDA, "cuTensorMapEncodeTiled is not available from the CUDA driver");
    return fn;
}

// Tensor map over the resident bytes of a weight seen as u32 [rows, row_pitch/4]; OOB reads give zeros.
int make_weight_map(const zq_weight *w, int box_words, int box_rows, CUtensorMap *out, zq_error *err) {
    EncodeTiledFn encode = get_encode_tiled(err);
    if (!encode) return ZQ_ERR_CUDA;
    cuuint64_t dims[2] = {(cuuint64_t)(w->row_pitch / 4), (cuuint64_t)w->rows};
    cuuint64_t strides[1] = {(cuuint64_t)w->row_pitch};
    cuuint32_t box[2] = {(cuuint32_t)box_words, (cuuint32_t)box_rows};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = encode(out, CU_TENSOR_MAP_DATA_TYPE_UINT32, 2, w->data, dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                         CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return set_error(err, ZQ_ERR_CUDA, "cuTensorMapEncodeTiled failed with code %d (rows=%zu pitch=%zu box=%dx%d)", (int)r, w->rows, w->row_pitch, box_words, box_rows);
    return ZQ_OK;
}

int ensure_workspace(zq_ctx *ctx, size_t bytes, zq_error *err) {
    if (bytes <= ctx->workspace_bytes) return ZQ_OK;
    // growing is rare (first call at a new size); wait for queued work that may still read the old buffer
    ZQ_CUDA_CHECK(cudaStreamSynchronize(ctx->stream), err);
    if (ctx->workspace) cudaFree(ctx->workspace);
    ctx->workspace = nullptr;
    ctx->workspace_bytes = 0;
    size_t rounded = (bytes + (size_t(1) << 20) - 1) & ~((size_t(1) << 20) - 1);
    ZQ_CUDA_CHECK(cudaMalloc(&ctx->workspace, rounded), err);
    ctx->workspace_bytes = rounded;
    return ZQ_OK;
}

int ensure_xq(zq_ctx *ctx, size_t bytes, zq_error *err) {
    if (bytes <= ctx->xq_bytes) return ZQ_OK;
    ZQ_CUDA_CHECK(cudaStreamSynchronize(ctx->stream), err);
    if (ctx->xq) cudaFree(ctx->xq);
    ctx->xq = nullptr;
    ctx->xq_bytes = 0;
    size_t rounded = (bytes + (size_t(1) << 20) - 1) & ~((size_t(1) << 20) - 1);
    ZQ_CUDA_CHECK(cudaMalloc(&ctx->xq, rounded), err);
    ctx->xq_bytes = rounded;
    return ZQ_OK;
}

int ensure_scratch_mid(zq_ctx *ctx, size_t bytes, zq_error *err) {
    if (bytes <= ctx->mid_bytes) return ZQ_OK;
    ZQ_CUDA_CHECK(cudaStreamSynchronize(ctx->stream), err);
    if (ctx->mid) cudaFree(ctx->mid);
    ctx->mid = nullptr;
    ctx->mid_bytes = 0;
    size_t rounded = (bytes + (size_t(1) << 20) - 1) & ~((size_t(1) << 20) - 1);
    ZQ_CUDA_CHECK(cudaMalloc(&ctx->mid, rounded), err);
    ctx->mid_bytes = rounded;
    return ZQ_OK;
}

int ensure_scratch_norm(zq_ctx *ctx, size_t bytes, zq_error *err) {
    if (bytes <= ctx->norm_bytes) return ZQ_OK;
    ZQ_CUDA_CHECK(cudaStreamSynchronize(ctx->stream), err);
    if (ctx->norm) cudaFree(ctx->norm);
    ctx->norm = nullptr;
    ctx->norm_bytes = 0;
    size_t rounded = (bytes + (size_t(1) << 20) - 1) & ~((size_t(1) << 20) - 1);
    ZQ_CUDA_CHECK(cudaMalloc(&ctx->norm, rounded), err);
    ctx->norm_bytes = rounded;
    return ZQ_OK;
}

// Every entry point that allocates or launches makes the context's device current first: a host that drives several
// GPUs from one thread (one context each) must never get memory or a launch on the wrong device.
int use_device(zq_ctx *ctx, zq_error *err) {
    int current = -1;
    if (cudaGetDevice(&current) == cudaSuccess && current == ctx->device) return ZQ_OK;
    ZQ_CUDA_CHECK(cudaSetDevice(ctx->device), err);
    return ZQ_OK;
}

static int check_dtype(int dtype, const char *what, zq_error *err) {
    if (dtype != ZQ_F32 && dtype != ZQ_F16 && dtype != ZQ_BF16) return set_error(err, ZQ_ERR_ARG, "%s: unknown dtype %d", what, dtype);
    return ZQ_OK;
}

static int prepare_common(zq_ctx *ctx, uint32_t type, size_t nbytes, size_t rows, size_t cols, zq_weight **out, zq_error *err) {
    if (!ctx || !out) return set_error(err, ZQ_ERR_ARG, "weight prepare: null context or output");
    FormatInfo f = format_info(type);
    if (!f.ggml_type) return set_error(err, ZQ_ERR_UNSUPPORTED, "GGUF tensor type %u is not supported (supported: 2, 6, 7, 8, 11, 12, 13, 14, 20, 23)", type);
    if (rows == 0 || cols == 0 || cols % f.block_elems) return set_error(err, ZQ_ERR_SHAPE, "GGUF type %u weight [%zu, %zu]: columns must be a positive multiple of %d", type, rows, cols, f.block_elems);
    size_t expected = rows * (cols / f.block_elems) * f.block_bytes;
    if (nbytes != expected) return set_error(err, ZQ_ERR_SHAPE, "GGUF type %u weight [%zu, %zu]: %zu bytes given, %zu expected", type, rows, cols, nbytes, expected);
    if (rows > (size_t)INT32_MAX || cols > (size_t)INT32_MAX) return set_error(err, ZQ_ERR_SHAPE, "weight [%zu, %zu] is too large", rows, cols);
    zq_weight *w = new zq_weight();
    w->ctx = ctx;
    w->type = type;
    w->rows = rows;
    w->cols = cols;
    w->units_per_row = (cols + kUnitWeights - 1) / kUnitWeights;
    w->row_pitch = w->units_per_row * f.unit_bytes;
    // block-32 types kept in GGUF order: a row is exactly its blocks (a last unit may be short; nothing reads past the columns)
    if (type == ZQ_Q5_0 || type == ZQ_Q5_1) w->row_pitch = (cols / f.block_elems) * f.block_bytes;
    w->gguf_bytes = nbytes;
    *out = w;
    return ZQ_OK;
}

static int finish_prepare(zq_ctx *ctx, zq_weight *w, zq_error *err) {
    if (!has_i8_decode(w->type)) return ZQ_OK;  // no decode kernel reads these through TMA (Q6_K blocks are not even 4-byte multiples)
    FormatInfo f = format_info(w->type);
    int rc = make_weight_map(w, 2 * f.unit_bytes / 4, 128, &w->gemv_map, err);
    if (!rc) rc = make_weight_map(w, 2 * f.unit_bytes / 4, 64, &w->gemv_map_half, err);
    if (!rc) rc = make_weight_map(w, f.unit_bytes / 4, 128, &w->qmv_map, err);
    if (rc) return rc;
    // device copies, in the tail of the weight's own allocation (see resident_alloc_bytes)
    const size_t tail = (w->rows * w->row_pitch + 255) & ~size_t(255);
    CUtensorMap host_maps[3] = {w->gemv_map, w->gemv_map_half, w->qmv_map};
    ZQ_CUDA_CHECK(cudaMemcpyAsync(w->data + tail, host_maps, sizeof(host_maps), cudaMemcpyHostToDevice, ctx->stream), err);
    ZQ_CUDA_CHECK(cudaStreamSynchronize(ctx->stream), err);  // host_maps is a stack array
    w->d_maps = reinterpret_cast<CUtensorMap *>(w->data + tail);
    return ZQ_OK;
}

}  // namespace zq

using namespace zq;

static int ctx_allocate(zq_ctx *ctx, zq_error *err) {
    ZQ_CUDA_CHECK(cudaStreamCreateWithFlags(&ctx->own_stream, cudaStreamNonBlocking), err);
    ctx->stream = ctx->own_stream;
    ctx->gemv_partials_floats = (size_t)ctx->sm_count * 2 * 128 * 16;  // two partial-tile slots (128 rows x 16 activation rows) per CTA
    ZQ_CUDA_CHECK(cudaMalloc(&ctx->gemv_partials, ctx->gemv_partials_floats * sizeof(float)), err);
    ctx->gemv_counters_n = 1 << 16;
    ZQ_CUDA_CHECK(cudaMalloc(&ctx->gemv_counters, ctx->gemv_counters_n * sizeof(uint32_t)), err);
    ZQ_CUDA_CHECK(cudaMemset(ctx->gemv_counters, 0, ctx->gemv_counters_n * sizeof(uint32_t)), err);
    ZQ_CUDA_CHECK(cudaHostAlloc(reinterpret_cast<void **>(&ctx->status_host), sizeof(uint32_t), cudaHostAllocMapped), err);
    *ctx->status_host = 0;
    ZQ_CUDA_CHECK(cudaHostGetDevicePointer(reinterpret_cast<void **>(&ctx->status_dev), ctx->status_host, 0), err);
    ZQ_CUDA_CHECK(cudaDeviceSynchronize(), err);
    return ZQ_OK;
}

extern "C" {

int zq_ctx_create(int device, zq_ctx **out, zq_error *err) {
    if (!out) return set_error(err, ZQ_ERR_ARG, "zq_ctx_create: null output");
    int count = 0;
    cudaError_t e = cudaGetDeviceCount(&count);
    if (e != cudaSuccess || count == 0) return set_error(err, ZQ_ERR_CUDA, "no CUDA device is available (%s); this library has no CPU fallback", cudaGetErrorString(e));
    if (device < 0 || device >= count) return set_error(err, ZQ_ERR_ARG, "device %d out of range (0..%d)", device, count - 1);
    ZQ_CUDA_CHECK(cudaSetDevice(device), err);
    cudaDeviceProp prop;
    ZQ_CUDA_CHECK(cudaGetDeviceProperties(&prop, device), err);
    if (prop.major != 10) return set_error(err, ZQ_ERR_UNSUPPORTED, "device %d is sm_%d%d; this library is built for sm_100a only", device, prop.major, prop.minor);
    zq_ctx *ctx = new zq_ctx();
    ctx->device = device;
    ctx->sm_count = prop.multiProcessorCount;
    int rc = ctx_allocate(ctx, err);
    if (rc) {
        zq_ctx_destroy(ctx);  // frees whatever part of the state exists
        return rc;
    }
    *out = ctx;
    return ZQ_OK;
}

void zq_ctx_destroy(zq_ctx *ctx) {
    if (!ctx) return;
    zq_moe_ep_shutdown(ctx);
    zq_dist_shutdown(ctx);
    cudaSetDevice(ctx->device);
    if (ctx->own_stream || ctx->stream) cudaStreamSynchronize(ctx->stream);
    if (ctx->gemv_partials) cudaFree(ctx->gemv_partials);
    if (ctx->gemv_counters) cudaFree(ctx->gemv_counters);
    if (ctx->workspace) cudaFree(ctx->workspace);
    if (ctx->mid) cudaFree(ctx->mid);
    if (ctx->norm) cudaFree(ctx->norm);
    if (ctx->xq) cudaFree(ctx->xq);
    if (ctx->moe_ws) cudaFree(ctx->moe_ws);
    if (ctx->status_host) cudaFreeHost(ctx->status_host);
    if (ctx->pinned) cudaFreeHost(ctx->pinned);
    if (ctx->host_io_dev) cudaFree(ctx->host_io_dev);
    for (auto &c : ctx->io_chunks) {
        cudaFreeHost(c.pinned);
        cudaFree(c.dev);
    }
    if (ctx->io_in) cudaStreamDestroy(ctx->io_in);
    if (ctx->io_out) cudaStreamDestroy(ctx->io_out);
    if (ctx->ev_in) cudaEventDestroy(ctx->ev_in);
    if (ctx->ev_done) cudaEventDestroy(ctx->ev_done);
    if (ctx->own_stream) cudaStreamDestroy(ctx->own_stream);
    delete ctx;
}

int zq_ctx_set_stream(zq_ctx *ctx, void *cuda_stream, zq_error *err) {
    if (!ctx) return set_error(err, ZQ_ERR_ARG, "zq_ctx_set_stream: null context");
    ctx->stream = reinterpret_cast<cudaStream_t>(cuda_stream);
    return ZQ_OK;
}

int zq_ctx_use_own_stream(zq_ctx *ctx, zq_error *err) {
    if (!ctx) return set_error(err, ZQ_ERR_ARG, "zq_ctx_use_own_stream: null context");
    ctx->stream = ctx->own_stream;
    return ZQ_OK;
}

int zq_ctx_sync(zq_ctx *ctx, zq_error *err) {
    if (!ctx) return set_error(err, ZQ_ERR_ARG, "zq_ctx_sync: null context");
    ZQ_CUDA_CHECK(cudaStreamSynchronize(ctx->stream), err);
    uint32_t status = *reinterpret_cast<volatile uint32_t *>(ctx->status_host);
    if (status != kStatusOk) {
        *ctx->status_host = 0;
        const char *what = status == kStatusTmaTimeout ? "a TMA copy did not complete within its wait limit"
                         : status == kStatusMmaTimeout ? "a tensor-core pipeline wait ran out"
                         : status == kStatusTmemAlloc ? "tensor memory could not be allocated"
                         : status == kStatusBadIndex ? "an index argument was out of range (the access was skipped)"
                         : status == kStatusPeerTimeout ? "a peer rank's partial result did not arrive within the wait limit" : "unknown device status";
        return set_error(err, ZQ_ERR_DEVICE_STATUS, "device status %u: %s", status, what);
    }
    return ZQ_OK;
}

int zq_ctx_set_option(zq_ctx *ctx, const char *key, int value, zq_error *err) {
    if (!ctx || !key) return set_error(err, ZQ_ERR_ARG, "zq_ctx_set_option: null argument");
    if (!strcmp(key, "force_staged_gemv")) {
        ctx->force_staged_gemv = value;
        return ZQ_OK;
    }
    if (!strcmp(key, "narrow_gemv_tiles")) {
        ctx->narrow_gemv_tiles = value;
        return ZQ_OK;
    }
    if (!strcmp(key, "force_fused_gemm")) {
        ctx->force_fused_gemm = value;
        return ZQ_OK;
    }
    if (!strcmp(key, "disable_fused_gemm")) {
        ctx->disable_fused_gemm = value;
        return ZQ_OK;
    }
    if (!strcmp(key, "force_moe_per_expert")) {
        ctx->force_moe_per_expert = value;
        return ZQ_OK;
    }
    if (!strcmp(key, "force_moe_host_grouping")) {
        ctx->force_moe_host_grouping = value;
        return ZQ_OK;
    }
    if (!strcmp(key, "disable_worklist")) {
        ctx->disable_worklist = value;
        return ZQ_OK;
    }
    if (!strcmp(key, "disable_pdl")) {
        ctx->disable_pdl = value;
        return ZQ_OK;
    }
    if (!strcmp(key, "force_f16_gemv")) {
        ctx->force_f16_gemv = value;
        return ZQ_OK;
    }
    if (!strcmp(key, "enable_tcgen05_gemv")) {
        ctx->enable_tcgen05_gemv = value;
        return ZQ_OK;
    }
    return set_error(err, ZQ_ERR_ARG, "zq_ctx_set_option: unknown option '%s'", key);
}

int zq_ctx_sm_count(const zq_ctx *ctx) { return ctx ? ctx->sm_count : 0; }
uint64_t zq_ctx_launch_count(const zq_ctx *ctx) { return ctx ? ctx->launches.load() : 0; }

int zq_weight_prepare_device(zq_ctx *ctx, uint32_t ggml_type, const void *dev_bytes, size_t nbytes, size_t rows, size_t cols, zq_weight **out, zq_error *err) {
    if (!dev_bytes) return set_error(err, ZQ_ERR_ARG, "weight prepare: null bytes");
    zq_weight *w = nullptr;
    int rc = prepare_common(ctx, ggml_type, nbytes, rows, cols, &w, err);
    if (!rc && (rc = use_device(ctx, err))) delete w;
    if (rc) return rc;
    // resident bytes, then (256-byte aligned) room for the device copies of three tensor maps
    size_t resident = ((w->rows * w->row_pitch + 255) & ~size_t(255)) + 3 * sizeof(CUtensorMap);
    cudaError_t e = cudaMalloc(reinterpret_cast<void **>(&w->data), resident);
    if (e != cudaSuccess) {
        delete w;
        return set_error(err, ZQ_ERR_CUDA, "cudaMalloc of %zu resident bytes failed: %s", resident, cudaGetErrorString(e));
    }
    if (resident_is_gguf_layout(ggml_type)) {
        e = cudaMemcpyAsync(w->data, dev_bytes, nbytes, cudaMemcpyDeviceToDevice, ctx->stream);
        if (e != cudaSuccess) rc = set_error(err, ZQ_ERR_CUDA, "copy of packed weight failed: %s", cudaGetErrorString(e));
    } else {
        rc = launch_repack(ctx, ggml_type, reinterpret_cast<const uint8_t *>(dev_bytes), w->data, rows, cols, err);
    }
    if (!rc) rc = finish_prepare(ctx, w, err);
    if (rc) {
        cudaFree(w->data);
        delete w;
        return rc;
    }
    *out = w;
    return ZQ_OK;
}

int zq_weight_prepare(zq_ctx *ctx, uint32_t ggml_type, const void *host_bytes, size_t nbytes, size_t rows, size_t cols, zq_weight **out, zq_error *err) {
    if (!host_bytes) return set_error(err, ZQ_ERR_ARG, "weight prepare: null bytes");
    zq_weight *probe = nullptr;
    int rc = prepare_common(ctx, ggml_type, nbytes, rows, cols, &probe, err);  // validates before any allocation
    if (rc) return rc;
    delete probe;
    void *staging = nullptr;
    ZQ_CUDA_CHECK(cudaSetDevice(ctx->device), err);
    ZQ_CUDA_CHECK(cudaMalloc(&staging, nbytes), err);
    cudaError_t e = cudaMemcpyAsync(staging, host_bytes, nbytes, cudaMemcpyHostToDevice, ctx->stream);
    if (e != cudaSuccess) {
        cudaFree(staging);
        return set_error(err, ZQ_ERR_CUDA, "upload of packed weight failed: %s", cudaGetErrorString(e));
    }
    rc = zq_weight_prepare_device(ctx, ggml_type, staging, nbytes, rows, cols, out, err);
    cudaStreamSynchronize(ctx->stream);  // host bytes are only borrowed for the duration of this call
    cudaFree(staging);
    return rc;
}

void zq_weight_release(zq_weight *w) {
    if (!w) return;
    if (w->ctx) {
        cudaSetDevice(w->ctx->device);
        cudaStreamSynchronize(w->ctx->stream);
    }
    if (w->owns_data && w->data) cudaFree(w->data);
    delete w;
}

size_t zq_weight_rows(const zq_weight *w) { return w ? w->rows : 0; }
size_t zq_weight_cols(const zq_weight *w) { return w ? w->cols : 0; }
uint32_t zq_weight_type(const zq_weight *w) { return w ? w->type : 0; }
size_t zq_weight_gguf_bytes(const zq_weight *w) { return w ? w->gguf_bytes : 0; }

int zq_dequantize_f32(zq_ctx *ctx, const zq_weight *w, float *dev_out, zq_error *err) {
    if (!ctx || !w || !dev_out) return set_error(err, ZQ_ERR_ARG, "zq_dequantize_f32: null argument");
    if (int rc = use_device(ctx, err)) return rc;
    return launch_dequantize(ctx, w, nullptr, w->rows, dev_out, ZQ_F32, err);
}

int zq_gather_rows(zq_ctx *ctx, const zq_weight *w, const uint32_t *dev_row_ids, size_t n_rows, void *dev_out, int out_dtype, zq_error *err) {
    if (!ctx || !w || !dev_out) return set_error(err, ZQ_ERR_ARG, "zq_gather_rows: null argument");
    int rc = check_dtype(out_dtype, "zq_gather_rows", err);
    if (rc) return rc;
    if ((rc = use_device(ctx, err))) return rc;
    if (!dev_row_ids && n_rows > w->rows) return set_error(err, ZQ_ERR_SHAPE, "zq_gather_rows: %zu rows requested from a weight with %zu rows", n_rows, w->rows);
    return launch_dequantize(ctx, w, dev_row_ids, n_rows, dev_out, out_dtype, err);
}

int zq_quantize(zq_ctx *ctx, uint32_t ggml_type, const float *dev_values, size_t rows, size_t cols, void *dev_gguf_bytes, size_t nbytes, zq_error *err) {
    if (!ctx || !dev_values || !dev_gguf_bytes) return set_error(err, ZQ_ERR_ARG, "zq_quantize: null argument");
    FormatInfo f = format_info(ggml_type);
    if (!f.ggml_type || is_operand_pass_only(ggml_type)) return set_error(err, ZQ_ERR_UNSUPPORTED, "zq_quantize: no encoder for GGUF tensor type %u", ggml_type);
    if (cols % f.block_elems) return set_error(err, ZQ_ERR_SHAPE, "zq_quantize: columns %zu not aligned to block %d", cols, f.block_elems);
    size_t expected = rows * (cols / f.block_elems) * f.block_bytes;
    if (nbytes != expected) return set_error(err, ZQ_ERR_SHAPE, "zq_quantize: output holds %zu bytes, %zu expected", nbytes, expected);
    if (int rc = use_device(ctx, err)) return rc;
    return launch_quantize(ctx, ggml_type, dev_values, rows, cols, dev_gguf_bytes, err);
}

static int check_linear(zq_ctx *ctx, const zq_weight *w, const void *x, int x_dtype, size_t m, void *y, int y_dtype, zq_error *err) {
    if (!ctx || !w || !x || !y) return set_error(err, ZQ_ERR_ARG, "linear: null argument");
    if (w->ctx != ctx) return set_error(err, ZQ_ERR_ARG, "linear: weight belongs to another context");
    int rc = check_dtype(x_dtype, "linear input", err);
    if (!rc) rc = check_dtype(y_dtype, "linear output", err);
    if (rc) return rc;
    if (m == 0) return set_error(err, ZQ_ERR_SHAPE, "linear: input has no rows");
    if ((reinterpret_cast<uintptr_t>(x) & 15) || (reinterpret_cast<uintptr_t>(y) & 15)) return set_error(err, ZQ_ERR_ARG, "linear: device buffers must be 16-byte aligned");
    return use_device(ctx, err);
}

int zq_linear(zq_ctx *ctx, const zq_weight *w, const void *dev_x, int x_dtype, size_t m, void *dev_y, int y_dtype, const void *dev_residual, zq_error *err) {
    int rc = check_linear(ctx, w, dev_x, x_dtype, m, dev_y, y_dtype, err);
    if (rc) return rc;
    // Q5_K, Q6_K: the integer-MMA kernel (launch_gemv falls back to the GEMM where that one does not fit)
    if ((w->type == ZQ_Q5_K || w->type == ZQ_Q6_K) && m <= 16 && !ctx->force_f16_gemv && !ctx->force_staged_gemv) return launch_gemv(ctx, w, nullptr, dev_x, x_dtype, m, dev_y, y_dtype, dev_residual, err);
    if (m <= 16 && !is_operand_pass_only(w->type)) return launch_gemv(ctx, w, nullptr, dev_x, x_dtype, m, dev_y, y_dtype, dev_residual, err);
    return launch_gemm(ctx, w, nullptr, dev_x, x_dtype, m, dev_y, y_dtype, dev_residual, err);
}

// One job of a batch through the single-job entry points (the route for whatever the work-list kernel does not take).
static int run_job_alone(zq_ctx *ctx, const zq_linear_job &j, int x_dtype, int y_dtype, zq_error *err) {
    if (j.w_up) return zq_gated_silu(ctx, j.w, j.w_up, j.dev_x, x_dtype, j.m, j.dev_y, y_dtype, err);
    return zq_linear(ctx, j.w, j.dev_x, x_dtype, j.m, j.dev_y, y_dtype, j.dev_residual, err);
}

int zq_linear_batch(zq_ctx *ctx, const zq_linear_job *jobs, size_t n_jobs, int x_dtype, int y_dtype, zq_error *err) {
    if (!ctx || (!jobs && n_jobs)) return set_error(err, ZQ_ERR_ARG, "zq_linear_batch: null argument");
    const bool grouped = ctx->dist && ctx->dist->world > 1;  // row-parallel jobs are summed over the peer group
    // validate everything before anything is enqueued: a bad job must not leave half a batch running
    size_t rp_floats = 0, rp_jobs = 0;
    for (size_t i = 0; i < n_jobs; ++i) {
        const zq_linear_job &j = jobs[i];
        int rc = check_linear(ctx, j.w, j.dev_x, x_dtype, j.m, j.dev_y, y_dtype, err);
        if (rc) return rc;
        if (j.flags & ~(uint32_t)ZQ_JOB_ROW_PARALLEL) return set_error(err, ZQ_ERR_ARG, "zq_linear_batch: job %zu: unknown flag bits 0x%x", i, j.flags);
        if (j.w_up) {
            if (j.w_up->ctx != ctx) return set_error(err, ZQ_ERR_ARG, "zq_linear_batch: job %zu: up weight belongs to another context", i);
            if (j.w->rows != j.w_up->rows || j.w->cols != j.w_up->cols || j.w->type != j.w_up->type) return set_error(err, ZQ_ERR_SHAPE, "zq_linear_batch: job %zu: gate and up differ in shape or type", i);
            if (j.dev_residual) return set_error(err, ZQ_ERR_ARG, "zq_linear_batch: job %zu: a gated job takes no residual", i);
            if (j.flags & ZQ_JOB_ROW_PARALLEL) return set_error(err, ZQ_ERR_ARG, "zq_linear_batch: job %zu: a gated job cannot be row-parallel (the activation is not linear)", i);
        }
        if (reinterpret_cast<uintptr_t>(j.dev_residual) & 15) return set_error(err, ZQ_ERR_ARG, "zq_linear_batch: job %zu: residual must be 16-byte aligned", i);
        if (grouped && (j.flags & ZQ_JOB_ROW_PARALLEL)) {
            rp_floats += (j.m * j.w->rows + 3) & ~size_t(3);
            ++rp_jobs;
        }
    }
    if (rp_jobs > (size_t)kDistMaxJobs) return set_error(err, ZQ_ERR_DIST, "zq_linear_batch: %zu row-parallel jobs in one call, at most %d", rp_jobs, kDistMaxJobs);
    // the exchange slot carries 8 bytes per f32 partial (value + epoch)
    if (rp_jobs && rp_floats * 8 > ctx->dist->slot_bytes) return set_error(err, ZQ_ERR_DIST, "zq_linear_batch: the row-parallel jobs need %zu bytes of exchange slot, it holds %zu (zq_dist_export)", rp_floats * 8, ctx->dist->slot_bytes);
    std::vector<WlHostJob> listed;
    std::vector<zq_linear_job> alone;
    std::vector<int> alone_y_dtype;
    std::vector<DistReduceJob> reduce;
    size_t staged = 0;
    for (size_t i = 0; i < n_jobs; ++i) {
        zq_linear_job j = jobs[i];
        int jy = -1;
        if (grouped && (j.flags & ZQ_JOB_ROW_PARALLEL)) {
            // the partial result goes to the staging vector as f32; the reduce kernel adds the peers' partials and the residual
            reduce.push_back({j.dev_y, j.dev_residual, j.m * j.w->rows});
            j.dev_y = ctx->dist->staging + staged * sizeof(float);
            j.dev_residual = nullptr;
            staged += (j.m * j.w->rows + 3) & ~size_t(3);
            jy = ZQ_F32;
        }
        WlHostJob h = {j.w, j.w_up, j.dev_x, j.m, j.dev_y, j.dev_residual, jy};
        // the diagnostic switches that pick a decode kernel hold for batches too: with one set, every job runs alone on it
        if (!ctx->disable_worklist && !ctx->force_f16_gemv && !ctx->force_staged_gemv && !ctx->enable_tcgen05_gemv && gemv_wl_supported(ctx, h)) {
            listed.push_back(h);
        } else {
            alone.push_back(j);
            alone_y_dtype.push_back(jy >= 0 ? jy : y_dtype);
        }
    }
    int rc = launch_gemv_wl(ctx, listed.data(), listed.size(), x_dtype, y_dtype, err);
    for (size_t k = 0; k < alone.size() && !rc; ++k) rc = run_job_alone(ctx, alone[k], x_dtype, alone_y_dtype[k], err);
    if (!rc && !reduce.empty()) rc = launch_tp_allreduce(ctx, reduce.data(), reduce.size(), y_dtype, err);
    return rc;
}

int zq_linear_row_parallel(zq_ctx *ctx, const zq_weight *w, const void *dev_x, int x_dtype, size_t m, void *dev_y, int y_dtype, const void *dev_residual, zq_error *err) {
    zq_linear_job job = {w, nullptr, dev_x, m, dev_y, dev_residual, ZQ_JOB_ROW_PARALLEL};
    return zq_linear_batch(ctx, &job, 1, x_dtype, y_dtype, err);
}

int zq_linear_multi(zq_ctx *ctx, const zq_weight *const *w, size_t n_weights, const void *dev_x, int x_dtype, size_t m, void *const *dev_y, int y_dtype, zq_error *err) {
    if (!w || !dev_y || n_weights == 0 || n_weights > 3) return set_error(err, ZQ_ERR_ARG, "zq_linear_multi: 1 to 3 weights expected");
    zq_linear_job jobs[3];
    for (size_t i = 0; i < n_weights; ++i) {
        if (!w[i] || w[i]->cols != w[0]->cols) return set_error(err, ZQ_ERR_SHAPE, "zq_linear_multi: weights must share the input width");
        jobs[i] = {w[i], nullptr, dev_x, m, dev_y[i], nullptr, 0};
    }
    return zq_linear_batch(ctx, jobs, n_weights, x_dtype, y_dtype, err);  // one launch: the input is quantised once
}

int zq_rmsnorm_linear(zq_ctx *ctx, const zq_weight *const *w, size_t n_weights, const void *dev_x, int x_dtype, size_t m, const float *dev_norm_weight, float eps, float weight_offset, void *const *dev_y,
                      int y_dtype, zq_error *err) {
    if (!ctx || !w || !dev_y || !dev_x || !dev_norm_weight || n_weights == 0 || n_weights > 3) return set_error(err, ZQ_ERR_ARG, "zq_rmsnorm_linear: null argument, or not 1 to 3 weights");
    for (size_t i = 0; i < n_weights; ++i) {
        if (!w[i] || !dev_y[i] || w[i]->ctx != ctx) return set_error(err, ZQ_ERR_ARG, "zq_rmsnorm_linear: weight %zu is null or belongs to another context", i);
        if (w[i]->cols != w[0]->cols) return set_error(err, ZQ_ERR_SHAPE, "zq_rmsnorm_linear: weights must share the input width");
    }
    int rc = check_dtype(x_dtype, "rmsnorm input", err);
    if (rc) return rc;
    if (m == 0) return set_error(err, ZQ_ERR_SHAPE, "zq_rmsnorm_linear: input has no rows");
    if (!(eps >= 0.0f)) return set_error(err, ZQ_ERR_ARG, "zq_rmsnorm_linear: eps must be non-negative");
    if ((rc = use_device(ctx, err))) return rc;
    const size_t cols = w[0]->cols;
    rc = ensure_scratch_norm(ctx, m * cols * sizeof(float), err);
    if (rc) return rc;
    rc = launch_rmsnorm(ctx, dev_x, x_dtype, m, cols, dev_norm_weight, eps, weight_offset, reinterpret_cast<float *>(ctx->norm), err);
    if (rc) return rc;
    zq_linear_job jobs[3];
    for (size_t i = 0; i < n_weights; ++i) jobs[i] = {w[i], nullptr, ctx->norm, m, dev_y[i], nullptr, 0};
    return zq_linear_batch(ctx, jobs, n_weights, ZQ_F32, y_dtype, err);
}

int zq_gated_silu(zq_ctx *ctx, const zq_weight *gate, const zq_weight *up, const void *dev_x, int x_dtype, size_t m, void *dev_y, int y_dtype, zq_error *err) {
    int rc = check_linear(ctx, gate, dev_x, x_dtype, m, dev_y, y_dtype, err);
    if (rc) return rc;
    if (!up || up->ctx != ctx) return set_error(err, ZQ_ERR_ARG, "gated linear: bad up weight");
    if (gate->rows != up->rows || gate->cols != up->cols || gate->type != up->type) return set_error(err, ZQ_ERR_SHAPE, "gated linear: gate [%zu, %zu] type %u and up [%zu, %zu] type %u differ", gate->rows, gate->cols, gate->type, up->rows, up->cols, up->type);
    if (m <= 16 && (!is_operand_pass_only(gate->type) || ((gate->type == ZQ_Q5_K || gate->type == ZQ_Q6_K) && !ctx->force_f16_gemv && !ctx->force_staged_gemv))) return launch_gemv(ctx, gate, up, dev_x, x_dtype, m, dev_y, y_dtype, nullptr, err);
    return launch_gemm(ctx, gate, up, dev_x, x_dtype, m, dev_y, y_dtype, nullptr, err);
}

int zq_gated_mlp(zq_ctx *ctx, const zq_weight *gate, const zq_weight *up, const zq_weight *down, const void *dev_x, int x_dtype, size_t m, void *dev_y, int y_dtype, const void *dev_residual, zq_error *err) {
    if (!ctx || !down || !gate || !up) return set_error(err, ZQ_ERR_ARG, "gated mlp: null context or weight");
    if (down->cols != gate->rows) return set_error(err, ZQ_ERR_SHAPE, "gated mlp: down expects %zu inputs, gate produces %zu", down->cols, gate->rows);
    // the activated intermediate [m, I] lives in the context workspace: f32 for the decode kernels; f16 for the tensor-core
    // GEMM, whose operands are f16 anyway (a bf16 or f32 intermediate would be rounded to f16 by the next GEMM's operand
    // pass, a bf16 one after losing three more bits first)
    int mid_dtype = m <= 16 ? ZQ_F32 : ZQ_F16;
    size_t mid_bytes = m * gate->rows * dtype_size(mid_dtype);
    int rc = ensure_scratch_mid(ctx, mid_bytes, err);
    if (rc) return rc;
    rc = zq_gated_silu(ctx, gate, up, dev_x, x_dtype, m, ctx->mid, mid_dtype, err);
    if (rc) return rc;
    return zq_linear(ctx, down, ctx->mid, mid_dtype, m, dev_y, y_dtype, dev_residual, err);
}

int zq_linear_noalloc(zq_ctx *ctx, const zq_weight *w, const void *dev_x, int x_dtype, size_t m, void *dev_y, int y_dtype, zq_error *err) {
    int rc = check_linear(ctx, w, dev_x, x_dtype, m, dev_y, y_dtype, err);
    if (rc) return rc;
    if (is_operand_pass_only(w->type)) return set_error(err, ZQ_ERR_UNSUPPORTED, "zq_linear_noalloc: GGUF type %u has no decode kernel (its layers need the operand workspace)", w->type);
    return launch_gemv_noalloc(ctx, w, dev_x, x_dtype, m, dev_y, y_dtype, err);
}

// True when a host pointer is page-locked memory the GPU can copy from / to directly (cudaHostAlloc,
// cudaHostRegister, a pinned tensor of the host framework): such buffers need no staging copy.
static bool is_pinned_host(const void *p) {
    cudaPointerAttributes a;
    if (cudaPointerGetAttributes(&a, p) != cudaSuccess) {
        cudaGetLastError();  // older runtimes report pageable memory as an error: not pinned, and not an error of ours
        return false;
    }
    return a.type == cudaMemoryTypeHost;
}

// Staging memory of a batch bracket: a (pinned, device) pair of `bytes` bytes, 256-byte aligned, valid until the
// bracket's finish.  Chunks are kept for the next bracket; a new one is allocated only when the existing ones are full.
static int batch_io_alloc(zq_ctx *ctx, size_t bytes, uint8_t **pinned, uint8_t **dev, zq_error *err) {
    bytes = (bytes + 255) & ~size_t(255);
    for (auto &c : ctx->io_chunks) {
        if (c.bytes - c.used >= bytes) {
            *pinned = c.pinned + c.used;
            *dev = c.dev + c.used;
            c.used += bytes;
            return ZQ_OK;
        }
    }
    zq_ctx::IoChunk c;
    c.bytes = bytes > (size_t(8) << 20) ? bytes : (size_t(8) << 20);
    c.used = bytes;
    void *p = nullptr, *d = nullptr;
    ZQ_CUDA_CHECK(cudaHostAlloc(&p, c.bytes, cudaHostAllocDefault), err);
    cudaError_t e = cudaMalloc(&d, c.bytes);
    if (e != cudaSuccess) {
        cudaFreeHost(p);
        return set_error(err, ZQ_ERR_CUDA, "batch staging: cudaMalloc of %zu bytes failed: %s", c.bytes, cudaGetErrorString(e));
    }
    c.pinned = reinterpret_cast<uint8_t *>(p);
    c.dev = reinterpret_cast<uint8_t *>(d);
    ctx->io_chunks.push_back(c);
    *pinned = c.pinned;
    *dev = c.dev;
    return ZQ_OK;
}

// Drops whatever an open bracket holds: waits for what was enqueued, fills no output, forgets every caller pointer.
static int batch_streams(zq_ctx *ctx, zq_error *err) {
    if (ctx->io_in) return ZQ_OK;
    ZQ_CUDA_CHECK(cudaStreamCreateWithFlags(&ctx->io_in, cudaStreamNonBlocking), err);
    ZQ_CUDA_CHECK(cudaStreamCreateWithFlags(&ctx->io_out, cudaStreamNonBlocking), err);
    ZQ_CUDA_CHECK(cudaEventCreateWithFlags(&ctx->ev_in, cudaEventDisableTiming), err);
    ZQ_CUDA_CHECK(cudaEventCreateWithFlags(&ctx->ev_done, cudaEventDisableTiming), err);
    return ZQ_OK;
}

static void batch_abandon(zq_ctx *ctx) {
    if (ctx->io_in) cudaStreamSynchronize(ctx->io_in);
    cudaStreamSynchronize(ctx->stream);
    if (ctx->io_out) cudaStreamSynchronize(ctx->io_out);
    ctx->io_out_used = false;
    ctx->pending_out.clear();
    ctx->pending_linear.clear();
    ctx->pending_in.clear();
    for (auto &c : ctx->io_chunks) c.used = 0;
    ctx->batch_active = false;
}

// Runs the bracket's deferred layers: one zq_linear_batch call per run of layers with the same dtypes (in call order),
// then the copies out.
static int batch_flush(zq_ctx *ctx, zq_error *err) {
    size_t i = 0;
    std::vector<zq_linear_job> jobs;
    while (i < ctx->pending_linear.size()) {
        const int xd = ctx->pending_linear[i].x_dtype, yd = ctx->pending_linear[i].y_dtype;
        size_t e = i;
        jobs.clear();
        while (e < ctx->pending_linear.size() && ctx->pending_linear[e].x_dtype == xd && ctx->pending_linear[e].y_dtype == yd) {
            const zq_ctx::PendingLinear &p = ctx->pending_linear[e];
            zq_linear_job j = {p.w, nullptr, p.dev_x, p.m, p.dev_y, nullptr, 0};
            jobs.push_back(j);
            ++e;
        }
        // the layers wait for the inputs copied so far; the copies out wait for the layers and run beside the next batch
        ZQ_CUDA_CHECK(cudaEventRecord(ctx->ev_in, ctx->io_in), err);
        ZQ_CUDA_CHECK(cudaStreamWaitEvent(ctx->stream, ctx->ev_in, 0), err);
        int rc = zq_linear_batch(ctx, jobs.data(), jobs.size(), xd, yd, err);
        if (rc) return rc;
        ZQ_CUDA_CHECK(cudaEventRecord(ctx->ev_done, ctx->stream), err);
        ZQ_CUDA_CHECK(cudaStreamWaitEvent(ctx->io_out, ctx->ev_done, 0), err);
        for (size_t k = i; k < e; ++k) {
            const zq_ctx::PendingLinear &p = ctx->pending_linear[k];
            ZQ_CUDA_CHECK(cudaMemcpyAsync(p.host_y_direct, p.dev_y, p.y_bytes, cudaMemcpyDeviceToHost, ctx->io_out), err);
        }
        ctx->io_out_used = true;
        i = e;
    }
    ctx->pending_linear.clear();
    return ZQ_OK;
}

int zq_batch_begin(zq_ctx *ctx, zq_error *err) {
    if (!ctx) return set_error(err, ZQ_ERR_ARG, "zq_batch_begin: null context");
    if (ctx->batch_active) return set_error(err, ZQ_ERR_ARG, "zq_batch_begin: a batch is already open");
    ctx->batch_active = true;
    return ZQ_OK;
}

int zq_batch_finish(zq_ctx *ctx, zq_error *err) {
    if (!ctx) return set_error(err, ZQ_ERR_ARG, "zq_batch_finish: null context");
    if (!ctx->batch_active) return set_error(err, ZQ_ERR_ARG, "zq_batch_finish: no batch is open");
    int rc = batch_flush(ctx, err);
    if (!rc) rc = zq_ctx_sync(ctx, err);
    if (!rc && ctx->io_out_used) {
        cudaError_t ce = cudaStreamSynchronize(ctx->io_out);
        if (ce != cudaSuccess) rc = set_error(err, ZQ_ERR_CUDA, "zq_batch_finish: copies out failed: %s", cudaGetErrorString(ce));
    }
    if (rc) {
        batch_abandon(ctx);
        return rc;
    }
    ctx->io_out_used = false;
    ctx->batch_active = false;
    for (const auto &o : ctx->pending_out) memcpy(o.host, o.pinned, o.bytes);
    ctx->pending_out.clear();
    ctx->pending_in.clear();
    for (auto &c : ctx->io_chunks) c.used = 0;
    return ZQ_OK;
}

int zq_linear_host(zq_ctx *ctx, const zq_weight *w, const void *host_x, int x_dtype, size_t m, void *host_y, int y_dtype, zq_error *err) {
    if (!ctx || !w || !host_x || !host_y) return set_error(err, ZQ_ERR_ARG, "zq_linear_host: null argument");
    int rc = check_dtype(x_dtype, "linear input", err);
    if (!rc) rc = check_dtype(y_dtype, "linear output", err);
    if (!rc && w->ctx != ctx) rc = set_error(err, ZQ_ERR_ARG, "zq_linear_host: weight belongs to another context");
    if (!rc && m == 0) rc = set_error(err, ZQ_ERR_SHAPE, "zq_linear_host: no activation rows");
    if (rc) {
        if (ctx->batch_active) batch_abandon(ctx);  // a failed call closes the bracket
        return rc;
    }
    size_t xb = m * w->cols * dtype_size(x_dtype), yb = m * w->rows * dtype_size(y_dtype);
    size_t xb_al = (xb + 255) & ~size_t(255);
    const bool x_pinned = is_pinned_host(host_x), y_pinned = is_pinned_host(host_y);
    if (ctx->batch_active) {
        // Inside a bracket the input starts its way to the device now and the layer itself is deferred: the finish runs
        // the bracket's layers as one batch (work-list launches: several matrices per kernel), copies the results out
        // and waits once.  Page-locked caller buffers are copied from / to directly; a page-locked input that an earlier
        // call of the bracket already brought over is not copied again (it must stay unchanged until the finish).
        const uint8_t *dev_in = nullptr;
        if (x_pinned)
            for (const auto &pi : ctx->pending_in)
                if (pi.host == host_x && pi.bytes == xb) dev_in = pi.dev;
        uint8_t *px = nullptr, *dx = nullptr;
        rc = use_device(ctx, err);
        if (!rc) rc = batch_streams(ctx, err);
        if (!rc) rc = batch_io_alloc(ctx, (dev_in ? 0 : xb_al) + yb, &px, &dx, err);
        if (!rc && !dev_in) {
            const void *src = host_x;
            if (!x_pinned) {
                memcpy(px, host_x, xb);
                src = px;
            }
            cudaError_t ce = cudaMemcpyAsync(dx, src, xb, cudaMemcpyHostToDevice, ctx->io_in);
            if (ce != cudaSuccess) rc = set_error(err, ZQ_ERR_CUDA, "zq_linear_host: copy in failed: %s", cudaGetErrorString(ce));
            if (!rc && x_pinned) ctx->pending_in.push_back({host_x, xb, dx});
        }
        if (rc) {
            batch_abandon(ctx);
            return rc;
        }
        // The GPU should not sit idle while the host records a long bracket: what is pending goes out as soon as it is a
        // launch's worth, i.e. when the next layer is of another kernel class (weight type, row-count class, dtypes) or
        // when the pending weights pass ~160 MB (tens of microseconds of streaming).
        auto row_class = [](size_t rows) { return rows <= 4 ? 1 : rows <= 8 ? 2 : rows <= 16 ? 4 : 0; };
        if (!ctx->pending_linear.empty()) {
            const zq_ctx::PendingLinear &last = ctx->pending_linear.back();
            if (last.w->type != w->type || row_class(last.m) != row_class(m) || last.x_dtype != x_dtype || last.y_dtype != y_dtype) {
                rc = batch_flush(ctx, err);
                if (rc) {
                    batch_abandon(ctx);
                    return rc;
                }
            }
        }
        const size_t y_off = dev_in ? 0 : xb_al;
        ctx->pending_linear.push_back({w, dev_in ? dev_in : dx, m, dx + y_off, y_pinned ? host_y : px + y_off, yb, x_dtype, y_dtype});
        if (!y_pinned) ctx->pending_out.push_back({host_y, px + y_off, yb});
        size_t pending_bytes = 0;
        for (const auto &p : ctx->pending_linear) pending_bytes += p.w->gguf_bytes;
        if (pending_bytes >= (size_t(160) << 20)) {
            rc = batch_flush(ctx, err);
            if (rc) {
                batch_abandon(ctx);
                return rc;
            }
        }
        return ZQ_OK;
    }
    if (ctx->host_io_bytes < xb_al + yb) {
        ZQ_CUDA_CHECK(cudaStreamSynchronize(ctx->stream), err);
        if (ctx->host_io_dev) cudaFree(ctx->host_io_dev);
        if (ctx->pinned) cudaFreeHost(ctx->pinned);
        ctx->host_io_dev = nullptr;
        ctx->pinned = nullptr;
        ctx->host_io_bytes = 0;
        ZQ_CUDA_CHECK(cudaMalloc(&ctx->host_io_dev, xb_al + yb), err);
        ZQ_CUDA_CHECK(cudaHostAlloc(&ctx->pinned, xb_al + yb, cudaHostAllocDefault), err);
        ctx->host_io_bytes = xb_al + yb;
    }
    uint8_t *dx = reinterpret_cast<uint8_t *>(ctx->host_io_dev), *dy = dx + xb_al;
    uint8_t *px = reinterpret_cast<uint8_t *>(ctx->pinned), *py = px + xb_al;
    const void *src = host_x;
    if (!x_pinned) {
        memcpy(px, host_x, xb);
        src = px;
    }
    ZQ_CUDA_CHECK(cudaMemcpyAsync(dx, src, xb, cudaMemcpyHostToDevice, ctx->stream), err);
    rc = zq_linear(ctx, w, dx, x_dtype, m, dy, y_dtype, nullptr, err);
    if (rc) return rc;
    ZQ_CUDA_CHECK(cudaMemcpyAsync(y_pinned ? host_y : py, dy, yb, cudaMemcpyDeviceToHost, ctx->stream), err);
    rc = zq_ctx_sync(ctx, err);
    if (rc) return rc;
    if (!y_pinned) memcpy(host_y, py, yb);
    return ZQ_OK;
}

int zq_linear_host_batch(zq_ctx *ctx, const zq_linear_host_job *jobs, size_t n_jobs, int x_dtype, int y_dtype, zq_error *err) {
    if (!ctx || (!jobs && n_jobs)) return set_error(err, ZQ_ERR_ARG, "zq_linear_host_batch: null argument");
    if (ctx->batch_active) {  // like every error inside a bracket, this one closes it
        batch_abandon(ctx);
        return set_error(err, ZQ_ERR_ARG, "zq_linear_host_batch: called inside an open bracket (the bracket is closed, none of its outputs is filled)");
    }
    int rc = zq_batch_begin(ctx, err);
    if (rc) return rc;
    for (size_t i = 0; i < n_jobs; ++i) {
        rc = zq_linear_host(ctx, jobs[i].w, jobs[i].host_x, x_dtype, jobs[i].m, jobs[i].host_y, y_dtype, err);
        if (rc) return rc;  // the failed call closed the bracket
    }
    return zq_batch_finish(ctx, err);
}

}  // extern "C"
