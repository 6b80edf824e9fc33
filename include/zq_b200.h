/*
 * zq_b200 — C ABI of the B200 (sm_100a) GGUF block-quantized linear layer.
 *
 * This is the boundary a zLLM CUDA backend binds instead of its NVRTC kernel layer.  Every entry point names
 * the reference interface it replaces (paths relative to the reference project root).  Conventions:
 *   - weights W[rows = out features, cols = in features], GGUF packed rows (src/kernel/cpu/ggml_quant.rs:193-197);
 *     activations X[m, cols] row-major; outputs Y[m, rows] row-major, Y[token*rows + row]
 *     (src/kernel/cpu/ggml_quant.rs:309-313);
 *   - GGUF type ids: Q4_0 = 2, Q8_0 = 8, Q4_K = 12, IQ4_NL = 20 (src/weight/container/gguf.rs:112-151);
 *   - every call returns 0 on success; on failure it returns a non-zero code and, when `err` is not NULL, fills
 *     err->message.  Shape and byte-count mismatches are errors, never undefined behaviour
 *     (src/kernel/cuda/linear.rs:1441-1444).  The layout of zq_error follows the reference's own native-FFI
 *     convention, NativeError{ message: [c_char; 512] } (src/backend/qnn/mod.rs:64-133);
 *   - all work is enqueued on the context's stream and is asynchronous unless the name says `_host`;
 *   - device pointers are plain `void*`/`float*`; no framework types cross this boundary.
 */
#ifndef ZQ_B200_H
#define ZQ_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef struct zq_ctx zq_ctx;
typedef struct zq_weight zq_weight;
typedef struct zq_moe_experts zq_moe_experts;

typedef struct zq_error { char message[512]; } zq_error;

/* GGUF tensor type ids (src/weight/container/gguf.rs:112-151).  Q4_K, Q4_0, Q8_0, IQ4_NL, Q5_K and Q6_K
 * (src/weight/codec/ggml.rs:102-109, 229-244, 408-469; reference CUDA kernels src/kernel/cuda/linear.rs:139-294, 1167-1234,
 * 1967-2101) decode (up to 16 activation rows, plain, residual and gated) on the integer-MMA kernels; all dequantise
 * bit-exactly.  Q5_K and Q6_K have no encoder (zq_quantize) and no allocation-free entry; Q6_K is re-laid into 224-byte
 * units at prepare time (zq_weight_gguf_bytes still reports the 210-byte packing).  Q5_0 / Q5_1 (types 6, 7, which the
 * reference CUDA backend accepts, src/backend/cuda/mod.rs:62-72), Q3_K (11) and IQ4_XS (23)
 * (src/weight/codec/ggml.rs:111-130, 384-406, 246-261) dequantise bit-exactly too and run every projection through the
 * f16 operand pass and the tensor-core GEMM.  The codebook-grid types (IQ2_*, IQ3_*) are not taken. */
enum { ZQ_Q4_0 = 2, ZQ_Q5_0 = 6, ZQ_Q5_1 = 7, ZQ_Q8_0 = 8, ZQ_Q3_K = 11, ZQ_Q4_K = 12, ZQ_Q5_K = 13, ZQ_Q6_K = 14, ZQ_IQ4_NL = 20, ZQ_IQ4_XS = 23 };
enum { ZQ_F32 = 0, ZQ_F16 = 1, ZQ_BF16 = 2 };
enum { ZQ_OK = 0, ZQ_ERR_SHAPE = 1, ZQ_ERR_UNSUPPORTED = 2, ZQ_ERR_CUDA = 3, ZQ_ERR_ARG = 4, ZQ_ERR_DEVICE_STATUS = 5, ZQ_ERR_DIST = 6 };

/* ---- context: CudaContext::new (src/backend/cuda/context.rs:248-276): one device, one compute stream. ---- */
int zq_ctx_create(int device, zq_ctx **out, zq_error *err);
void zq_ctx_destroy(zq_ctx *ctx);
/* Run on a caller-owned cudaStream_t instead of the context's own stream.  NULL is a valid handle: it is the
 * legacy default stream.  zq_ctx_use_own_stream goes back to the stream the context created. */
int zq_ctx_set_stream(zq_ctx *ctx, void *cuda_stream, zq_error *err);
int zq_ctx_use_own_stream(zq_ctx *ctx, zq_error *err);
/* Waits for the stream and reports any status word a kernel left behind (bounded waits that ran out). */
int zq_ctx_sync(zq_ctx *ctx, zq_error *err);
/* Diagnostic switches (the counterpart of the reference's ZLLM_CUDA_* environment switches, kept per context).
 * Known keys (0/1): "force_staged_gemv", "force_f16_gemv" (decode on the f16 kernels instead of the integer-MMA kernel),
 * "enable_tcgen05_gemv" (Q4_K decode on the tcgen05 kernel), "disable_pdl" (decode kernels without programmatic dependent launch), "disable_worklist" (zq_linear_batch and the multi-weight entries launch one kernel per job), "force_moe_per_expert" (MoE forward always on the host-grouped path), "force_moe_host_grouping" (MoE prefill: routes grouped on the host instead of on the device), "narrow_gemv_tiles" (decode, up to 4 rows: 64-row tiles, two CTAs per SM), "disable_fused_gemm" / "force_fused_gemm" (Q4_K prefill never / always on the kernel that dequantises inside the GEMM; default: up to 1024 tokens and MoE prefill). */
int zq_ctx_set_option(zq_ctx *ctx, const char *key, int value, zq_error *err);
int zq_ctx_sm_count(const zq_ctx *ctx);
/* Number of kernels this library has launched on the context since creation (bench accounting). */
uint64_t zq_ctx_launch_count(const zq_ctx *ctx);

/* ---- weights: Backend::prepare_weight(LinearWeight::gguf) (src/backend/mod.rs:333; src/backend/cuda/mod.rs:61-72)
 * and CudaGgufPacked (src/backend/cuda/resident.rs:82-107).  `nbytes` must equal rows*cols/block*block_bytes
 * (src/kernel/cuda/linear.rs:1441-1444).  The library owns the resident copy. ---- */
int zq_weight_prepare(zq_ctx *ctx, uint32_t ggml_type, const void *host_bytes, size_t nbytes, size_t rows, size_t cols, zq_weight **out, zq_error *err);
/* Same, from GGUF-layout bytes already on the device (expert tensors sliced on device, synthetic inputs). */
int zq_weight_prepare_device(zq_ctx *ctx, uint32_t ggml_type, const void *dev_bytes, size_t nbytes, size_t rows, size_t cols, zq_weight **out, zq_error *err);
/* Release every weight (and expert table) of a context before zq_ctx_destroy: releasing waits on the context's stream. */
void zq_weight_release(zq_weight *w);
size_t zq_weight_rows(const zq_weight *w);
size_t zq_weight_cols(const zq_weight *w);
uint32_t zq_weight_type(const zq_weight *w);
/* Bytes of the original GGUF packing (the figure roofline accounting uses). */
size_t zq_weight_gguf_bytes(const zq_weight *w);

/* ---- codec: codec::ggml::dequantize (src/weight/codec/ggml.rs:146-160), bit-exact f32 [rows, cols]. ---- */
int zq_dequantize_f32(zq_ctx *ctx, const zq_weight *w, float *dev_out, zq_error *err);
/* gguf_rows_f16 (src/kernel/cuda/linear.rs:1420-1437): dequantise the listed rows (embedding gather).
 * dev_row_ids may be NULL for rows 0..n_rows-1.  out dtype ZQ_F32 / ZQ_F16 / ZQ_BF16. */
int zq_gather_rows(zq_ctx *ctx, const zq_weight *w, const uint32_t *dev_row_ids, size_t n_rows, void *dev_out, int out_dtype, zq_error *err);
/* requantize_q4_k / encode_q4_k (src/weight/codec/ggml.rs:163-227) on the device: f32 [rows, cols] -> GGUF bytes.
 * Q4_K follows the reference encoder bit for bit; Q4_0, Q8_0 and IQ4_NL (no encoder in the reference) use
 * round-to-nearest encoders meant for generating synthetic inputs. */
int zq_quantize(zq_ctx *ctx, uint32_t ggml_type, const float *dev_values, size_t rows, size_t cols, void *dev_gguf_bytes, size_t nbytes, zq_error *err);

/* ---- linear: gguf_kq_matmul_f16 (src/kernel/cuda/linear.rs:1440-1584) behind Backend::linear / linear_add
 * (src/backend/mod.rs:389, 417).  m <= 16 runs the decode GEMV, larger m the prefill GEMM.  `dev_residual`
 * (same shape and dtype as y) may be NULL; when given, y = W x + residual (matvec_residual,
 * src/kernel/cpu/ggml_quant.rs:224-233). ---- */
int zq_linear(zq_ctx *ctx, const zq_weight *w, const void *dev_x, int x_dtype, size_t m, void *dev_y, int y_dtype, const void *dev_residual, zq_error *err);
/* Backend::dual_linear / triple_linear (src/backend/mod.rs:444-451): up to 3 weights share one input. */
int zq_linear_multi(zq_ctx *ctx, const zq_weight *const *w, size_t n_weights, const void *dev_x, int x_dtype, size_t m, void *const *dev_y, int y_dtype, zq_error *err);
/* A list of INDEPENDENT decode projections in as few launches as possible (no job may read another job's output).
 * It generalises Backend::dual_linear / triple_linear (src/backend/mod.rs:444-451) and the Metal backend's two-weight
 * decode launch gguf_dual_gemv_q4k_f16 (src/kernel/metal/gguf/mod.rs:1787-1824) to any number of weights and inputs:
 * the projections of a decode step that are ready together (q, k, v; gate and up; the layers of several sequences)
 * stream through one persistent kernel whose TMA ring never drains between matrices.  Per job: y = W x (+ residual),
 * or y = silu(gate x) * (up x) when `w_up` is given (then `w` is the gate; no residual).  Jobs of Q4_K / Q4_0 / Q8_0
 * weights with up to 16 rows share launches (one per weight type, row-count class 1-4 / 5-8 / 9-16 and plain / gated);
 * every other job runs as its own zq_linear / zq_gated_silu call.  All jobs share x_dtype and y_dtype.  Results do not
 * depend on how the jobs are grouped beyond f32 rounding of the split-tile sums, and are the same from run to run. */
enum { ZQ_JOB_ROW_PARALLEL = 1 };  /* zq_linear_job.flags: sum this job's result over the ranks of the peer group (zq_dist_init) */
typedef struct zq_linear_job {
    const zq_weight *w;        /* the weight, or the gate of a gated pair */
    const zq_weight *w_up;     /* NULL, or the up weight of a gated pair */
    const void *dev_x;         /* [m, cols] */
    size_t m;
    void *dev_y;               /* [m, rows] */
    const void *dev_residual;  /* NULL, or [m, rows] in y_dtype */
    uint32_t flags;            /* 0, or ZQ_JOB_ROW_PARALLEL (plain jobs only) */
} zq_linear_job;
int zq_linear_batch(zq_ctx *ctx, const zq_linear_job *jobs, size_t n_jobs, int x_dtype, int y_dtype, zq_error *err);
/* ---- tensor parallelism over the GPUs of one node (one process and one context per GPU).
 * Column split (output rows divided over the ranks) needs nothing from this library: every rank prepares its rows as a
 * weight of its own.  Row split (input columns divided on 256-column boundaries, the rule of the reference's two-GPU
 * operator pair, src/backend/rocm/expert.rs:182-207) leaves every rank with a partial result; the ranks' partials are
 * exchanged and added (src/backend/rocm/expert.rs:1394-1409; the fused join of
 * src/kernel/rocm/hip/peer_copy/source.hip:64-81) by ONE kernel per call that stores them into every peer's exchange
 * buffer over NVLink (plain 8-byte stores of {value, epoch} into memory mapped with CUDA IPC), polls the peers' words with
 * a bounded wait and adds in rank order: no host-launched collective, so a whole decode step stays one CUDA graph.  A wait that runs
 * out sets the device status word (zq_ctx_sync reports it) and the kernel returns; nothing hangs.
 *   zq_dist_export  allocates this rank's exchange buffer (`slot_bytes` = 8 bytes per f32 partial result of the largest
 *                   call, the same on every rank) and writes ZQ_DIST_HANDLE_BYTES bytes to hand to the other ranks;
 *   zq_dist_init    takes the blobs of all ranks in rank order (exchanged by the host: a channel, a file, MPI, NCCL ...).
 * Every rank must issue the same sequence of row-parallel calls with the same shapes. */
#define ZQ_DIST_HANDLE_BYTES 80
int zq_dist_export(zq_ctx *ctx, size_t slot_bytes, void *out_handle, zq_error *err);
int zq_dist_init(zq_ctx *ctx, int rank, int world, const void *all_handles, zq_error *err);
int zq_dist_set_wait_ms(zq_ctx *ctx, unsigned milliseconds, zq_error *err);
int zq_dist_rank(const zq_ctx *ctx);
int zq_dist_world(const zq_ctx *ctx);
void zq_dist_shutdown(zq_ctx *ctx);
/* y = sum over ranks of (W_rank x_rank) (+ residual): this rank's column slice of the weight against its slice of the
 * input, any number of rows (decode kernel up to 16 rows, tensor-core GEMM above).  Same as a one-job zq_linear_batch
 * with ZQ_JOB_ROW_PARALLEL.  Without a peer group (or a group of one) it is zq_linear. */
int zq_linear_row_parallel(zq_ctx *ctx, const zq_weight *w, const void *dev_x, int x_dtype, size_t m, void *dev_y, int y_dtype, const void *dev_residual, zq_error *err);

/* Backend::rmsnorm_linear / rmsnorm_dual_linear (src/backend/mod.rs:455-464): RMSNorm of every input row
 * (src/kernel/cpu/rmsnorm.rs:7-41: x * 1/sqrt(mean(x^2) + eps) * (norm_weight + weight_offset); offset 0 = plain,
 * 1 = the "Gemma" form), then 1 to 3 linear layers on the normalised rows.  `dev_norm_weight`: f32 [cols].  The
 * normalised rows stay in a context buffer (f32); the projections start under the normalisation kernel. */
int zq_rmsnorm_linear(zq_ctx *ctx, const zq_weight *const *w, size_t n_weights, const void *dev_x, int x_dtype, size_t m, const float *dev_norm_weight, float eps, float weight_offset, void *const *dev_y,
                      int y_dtype, zq_error *err);
/* Backend::rope / rope_prefix / rope_prefix_qk (src/backend/mod.rs:545-583): rotary position embedding of the q and k
 * projection outputs, in place, one launch for both (their head counts may differ).  Arithmetic and parameter errors are
 * those of attention::rope::apply_f32 (src/attention/rope.rs:120-165); f32 rows are bit-identical to the CPU path.
 * q: [rows, q_heads * head_dim]; k: [rows, k_heads * head_dim] or NULL; row r uses table row `position + r` of the f32
 * tables cos / sin [table_len / (rotary_dim / 2), rotary_dim / 2] on the device. */
enum { ZQ_ROPE_SPLIT_HALF = 0, ZQ_ROPE_INTERLEAVED = 1 };  /* RotaryLayout */
enum { ZQ_ROPE_PREFIX = 0, ZQ_ROPE_SUFFIX = 1 };           /* RotaryPlacement: rope_prefix / rope */
int zq_rope_qk(zq_ctx *ctx, void *dev_q, size_t q_heads, void *dev_k, size_t k_heads, int dtype, size_t rows, size_t head_dim, size_t rotary_dim, int layout, int placement, size_t position,
               const float *dev_cos, const float *dev_sin, size_t table_len, zq_error *err);
/* gated_linear_q4_k_silu_f16 / gated_linear_q4_0_silu_f16 (src/kernel/cuda/linear.rs:1683, 1916) behind
 * Backend::gated_linear (src/backend/mod.rs:467): y = silu(gate x) * (up x). */
int zq_gated_silu(zq_ctx *ctx, const zq_weight *gate, const zq_weight *up, const void *dev_x, int x_dtype, size_t m, void *dev_y, int y_dtype, zq_error *err);
/* Backend::gated_mlp / gated_mlp_add_residual (src/backend/mod.rs:474, 483): down(silu(gate x) * up x) (+ residual). */
int zq_gated_mlp(zq_ctx *ctx, const zq_weight *gate, const zq_weight *up, const zq_weight *down, const void *dev_x, int x_dtype, size_t m, void *dev_y, int y_dtype, const void *dev_residual, zq_error *err);

/* Decode linear (1..8 activation rows, y = W x) that allocates nothing.  It has no counterpart in the reference:
 * it exists for callers that cannot allocate device memory where they run a layer (a host application that owns
 * the allocator, a fixed-budget real-time loop, a region in which allocator calls are forbidden).  The kernel's
 * scratch (partial tiles and arrival counters of the split-tile fix-up) lives in a fixed device array inside the
 * library, about 2.6 MB per GPU, held from library load until process exit.  Limits: at most 8 activation rows per
 * call, weights of at most 524 288 rows, devices of at most 160 SMs; anything beyond is rejected with an error.
 * The first call on a device looks up the array's device address (no allocation).  Results equal zq_linear's bit
 * for bit for 1..4 rows; 5..8 rows of Q4_K / Q4_0 / Q8_0 / IQ4_NL run on the f16-limb kernel rather than zq_linear's
 * integer-MMA one (whose activation workspace may have to grow) and agree within that kernel's activation rounding
 * (16-bit integers per 256-column slice: a few 1e-5 of the largest output).  All calls on a device
 * share the array: calls that overlap on the GPU (two streams, two contexts)
 * race; calls ordered on one stream do not.  Inputs, outputs and the prepared weight are the caller's, as for
 * zq_linear. */
int zq_linear_noalloc(zq_ctx *ctx, const zq_weight *w, const void *dev_x, int x_dtype, size_t m, void *dev_y, int y_dtype, zq_error *err);

/* Host-buffer form of zq_linear: copies x from host memory, runs, copies y back and waits.  This is what a
 * backend that keeps activations on the host between operators calls (CpuTensor in, CpuTensor out). */
int zq_linear_host(zq_ctx *ctx, const zq_weight *w, const void *host_x, int x_dtype, size_t m, void *host_y, int y_dtype, zq_error *err);

/* Backend::begin_batch / finish_batch (src/backend/mod.rs:307-323; the reference's Vulkan backend defers its command
 * submission the same way, src/backend/vulkan/mod.rs:194-215).  Between the two calls zq_linear_host only starts its
 * copy in and records the layer; recorded layers run as zq_linear_batch calls (several matrices per kernel launch),
 * as soon as a launch's worth of them is pending (inputs and results travel on copy streams of the context's own beside
 * the layers) and the rest at zq_batch_finish, which copies the last results out,
 * waits once and then fills the callers' output buffers; these must stay valid and must not be read until then.  An
 * error of a recorded layer is reported by the call that launches it or by the finish; any error closes the bracket.  Pageable input buffers may be reused
 * as soon as their zq_linear_host call returns (they are copied into the library's staging memory inside the call);
 * page-locked input buffers (cudaHostAlloc, cudaHostRegister, a pinned tensor) are read by the GPU's copy engine
 * directly and must stay untouched until zq_batch_finish returns (the same page-locked input given to several calls
 * of one bracket is copied once). */
int zq_batch_begin(zq_ctx *ctx, zq_error *err);
int zq_batch_finish(zq_ctx *ctx, zq_error *err);
/* A whole bracket in one call: zq_batch_begin, zq_linear_host for every job in order, zq_batch_finish.  For hosts whose
 * per-call cost is not negligible (a scripting-language binding), and for callers that already hold a layer's list of
 * projections.  Must not be called inside an open bracket (an error that, like every error, closes that bracket). */
typedef struct zq_linear_host_job {
    const zq_weight *w;
    const void *host_x;  /* [m, cols] */
    size_t m;
    void *host_y;        /* [m, rows] */
} zq_linear_host_job;
int zq_linear_host_batch(zq_ctx *ctx, const zq_linear_host_job *jobs, size_t n_jobs, int x_dtype, int y_dtype, zq_error *err);

/* ---- MoE: kernel::cuda::routing (src/kernel/cuda/routing.rs:167-210) and the expert entry points
 * (src/kernel/cuda/linear.rs:1735-1819; src/backend/cuda/expert.rs:572-918). ---- */
/* moe_route_softmax_topk_device_f32: logits = x router^T (+ bias), softmax top-k with ties to the lower expert id.
 * router_f32 [num_experts, hidden] on the device; bias may be NULL.  Writes ids [m, top_k] and weights [m, top_k]. */
int zq_moe_route_softmax_topk(zq_ctx *ctx, const void *dev_x, int x_dtype, size_t m, size_t hidden, const float *dev_router_f32, const float *dev_bias_f32, size_t num_experts, size_t top_k, float scaling_factor, int normalize_selected, uint32_t *dev_ids, float *dev_weights, zq_error *err);
/* The same call with the router family of src/moe/routing.rs as a parameter.  ZQ_ROUTE_SOFTMAX is the call above.
 * ZQ_ROUTE_SIGMOID_BIAS (route_sigmoid_bias_logits, :74) and ZQ_ROUTE_SQRT_SOFTPLUS_BIAS (route_sqrt_softplus_bias_logits,
 * :79) follow route_bias_corrected_logits (:45-67): raw score sigmoid(logit) or sqrt(softplus(logit)); the bias only takes
 * part in choosing the top-k (raw + bias, ties to the lower id); the chosen experts' raw scores are normalised to sum 1
 * and multiplied by scaling_factor (`normalize_selected` is ignored; a NULL bias counts as zero). */
enum { ZQ_ROUTE_SOFTMAX = 0, ZQ_ROUTE_SIGMOID_BIAS = 1, ZQ_ROUTE_SQRT_SOFTPLUS_BIAS = 2 };
int zq_moe_route_topk(zq_ctx *ctx, int scoring, const void *dev_x, int x_dtype, size_t m, size_t hidden, const float *dev_router_f32, const float *dev_bias_f32, size_t num_experts, size_t top_k, float scaling_factor,
                      int normalize_selected, uint32_t *dev_ids, float *dev_weights, zq_error *err);
/* The gather / scatter halves of the MoE trait on their own, for callers that orchestrate experts themselves
 * (Backend::moe_gather_rows / moe_scatter_add_rows, src/backend/mod.rs:1657-1662; kernels gather_rows_f16 and
 * scatter_add_rows_f32, src/kernel/cuda/routing.rs:112-125; prefill_expert_batch callers, src/moe/prefill.rs:291-327):
 *   gather       out[i] = x[row_ids[i]]                          (rows in x's dtype; a row must be a multiple of 16 bytes)
 *   scatter-add  out_f32[row_ids[i]] += weights[i] * rows[i]     (weights may be NULL = 1; the accumulator is f32
 *                [out_rows, hidden], zeroed by the caller = moe_zeros; atomic adds as in the reference)
 * Row ids out of range are skipped and reported by zq_ctx_sync. */
int zq_moe_gather_rows(zq_ctx *ctx, const void *dev_x, int dtype, size_t x_rows, size_t hidden, const uint32_t *dev_row_ids, size_t n_rows, void *dev_out, zq_error *err);
int zq_moe_scatter_add_rows(zq_ctx *ctx, const void *dev_rows, int dtype, const uint32_t *dev_row_ids, const float *dev_weights, size_t n_rows, size_t hidden, float *dev_out_f32, size_t out_rows, zq_error *err);
/* The resident expert table that replaces CudaMoeState's LRU/arena cache (src/backend/cuda/expert.rs:284-570)
 * when every expert fits in HBM.  gate/up: [intermediate, hidden]; down: [hidden, intermediate].  The table
 * borrows the weights; release them after zq_moe_experts_destroy. */
int zq_moe_experts_create(zq_ctx *ctx, const zq_weight *const *gate, const zq_weight *const *up, const zq_weight *const *down, size_t num_experts, zq_moe_experts **out, zq_error *err);
void zq_moe_experts_destroy(zq_moe_experts *experts);
/* Routed experts (+ optional shared expert and residual): prefill_resident_routed_experts(_add) /
 * decode_routed_experts (src/backend/mod.rs:1921-1960, 2012-2024).
 * y[m, hidden] = residual + shared(x) + sum_k w_k * expert_k(x), contributions added in ascending expert id per
 * token (src/backend/cpu/moe.rs:107-141).  shared_* may be NULL. */
#define ZQ_MOE_NO_ROUTE 0xFFFFFFFFu /* an expert id that means "no route in this place": no expert runs, nothing is added */
int zq_moe_forward(zq_ctx *ctx, const zq_moe_experts *experts, const zq_weight *shared_gate, const zq_weight *shared_up, const zq_weight *shared_down, const void *dev_x, int x_dtype, size_t m, const uint32_t *dev_ids, const float *dev_weights, size_t top_k, void *dev_y, int y_dtype, const void *dev_residual, zq_error *err);

/* ---- GGUF container: GgufReader (src/weight/container/gguf.rs:332-566).  open / parse_shard (:364-412, :663-725): GGUF
 * v3 header, metadata, tensor directory, data offset from general.alignment, every tensor inside its file, split files
 * "<prefix>-00001-of-0000N.gguf" opened together (:727-750).  Metadata scalars and strings can be read; arrays only
 * report their length.  Errors (not a GGUF file, another version, unknown type, a tensor beyond the file, duplicate
 * names, split counts that do not add up) come back as codes with a message. */
typedef struct zq_gguf zq_gguf;
int zq_gguf_open(const char *path, zq_gguf **out, zq_error *err);
void zq_gguf_close(zq_gguf *file);
size_t zq_gguf_tensor_count(const zq_gguf *file);
int zq_gguf_tensor_name(const zq_gguf *file, size_t index, char *out, size_t capacity, zq_error *err);
/* dims4: the GGUF dimension order (a matrix is [columns, rows]; an expert tensor [columns, rows, count]), padded with 1. */
int zq_gguf_tensor_info(const zq_gguf *file, const char *name, uint32_t *type, uint32_t *n_dims, uint64_t *dims4, uint64_t *nbytes, zq_error *err);
int zq_gguf_metadata_u64(const zq_gguf *file, const char *key, uint64_t *out, zq_error *err);
int zq_gguf_metadata_f64(const zq_gguf *file, const char *key, double *out, zq_error *err);
int zq_gguf_metadata_str(const zq_gguf *file, const char *key, char *out, size_t capacity, zq_error *err);
/* read_matrix (:506-514) / read_matrix_slice (:516-534) + prepare_weight: the tensor's bytes go from the file to a resident
 * weight.  The slice form takes matrix `index` of a [columns, rows, count] tensor: one expert of an expert tensor. */
int zq_gguf_load_matrix(zq_ctx *ctx, const zq_gguf *file, const char *name, zq_weight **out, zq_error *err);
int zq_gguf_load_matrix_slice(zq_ctx *ctx, const zq_gguf *file, const char *name, size_t index, zq_weight **out, zq_error *err);
/* embedding_rows (:618-629) is zq_gather_rows on the loaded embedding matrix.  The LM head of a greedy decode step:
 * logits = head x (any row count) and the arg-max of every row on the device (ties to the lower token id, NaN never
 * chosen), so the logits do not travel to the host; zq_argmax_rows is the second half on its own. */
int zq_argmax_rows(zq_ctx *ctx, const void *dev_x, int dtype, size_t rows, size_t cols, uint32_t *dev_ids, zq_error *err);
int zq_lm_head_argmax(zq_ctx *ctx, const zq_weight *head, const void *dev_x, int x_dtype, size_t m, uint32_t *dev_ids, zq_error *err);

/* ---- expert parallelism over the GPUs of one node.  The reference keeps every expert on (or cached by) one device
 * (src/backend/cuda/expert.rs:284-570) and has no counterpart; the arithmetic of an expert and the ascending-expert order
 * of a token's sum are its own (src/kernel/cpu/moe.rs:122-138, src/backend/cpu/moe.rs:107-141).  Rank r of the peer group
 * owns the contiguous block of experts [r E / W, (r + 1) E / W) (the first E % W ranks hold one more) and passes a table of
 * exactly those; tokens stay with the rank that brings them, with GLOBAL expert ids.  Each token travels once per owner
 * rank it routes to (not once per route), its routes on that rank are weighted and summed there, one f32 row per (token,
 * rank) comes back, and the token's rank adds shared expert, residual and the returned rows in ascending rank order.
 * Transport: plain stores into peer memory mapped with CUDA IPC, {count, epoch} flags, bounded waits that set the
 * status word and go on (zq_ctx_sync reports them).  Needs zq_dist_init first; every rank makes the same calls.
 *   zq_moe_ep_export   allocates the exchange buffers for up to `max_tokens_per_rank` tokens per rank and call, writes
 *                      ZQ_DIST_HANDLE_BYTES bytes for the other ranks;  zq_moe_ep_init maps the peers' buffers. */
int zq_moe_ep_export(zq_ctx *ctx, size_t max_tokens_per_rank, size_t hidden, size_t top_k, size_t num_experts_total, int x_dtype, void *out_handle, zq_error *err);
int zq_moe_ep_init(zq_ctx *ctx, const void *all_handles, zq_error *err);
void zq_moe_ep_shutdown(zq_ctx *ctx);
/* `m` = this rank's tokens; `m_cap` = the largest m of any rank in this call (the same value on every rank, at most the
 * allocated bound; 0 = every rank passes the same m).  Every call advances an exchange epoch that the host passes to the
 * kernels, so the call is issued from the host each time (a replayed CUDA graph would repeat a stale epoch), unlike the
 * row-parallel reduce, whose epoch lives on the device. */
int zq_moe_forward_ep(zq_ctx *ctx, const zq_moe_experts *local_experts, const zq_weight *shared_gate, const zq_weight *shared_up, const zq_weight *shared_down, const void *dev_x, int x_dtype, size_t m, size_t m_cap,
                      const uint32_t *dev_ids, const float *dev_weights, size_t top_k, void *dev_y, int y_dtype, const void *dev_residual, zq_error *err);

#ifdef __cplusplus
}
#endif
#endif /* ZQ_B200_H */
