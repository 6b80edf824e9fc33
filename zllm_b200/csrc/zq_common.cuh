// Shared definitions for the zq_b200 CUDA library: resident weight layouts, PTX wrappers (mbarrier, TMA bulk
// tensor copies, warp MMA), host-side context and error plumbing.  sm_100a only.
#pragma once

#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <atomic>
#include <cstdarg>
#include <cstdio>
#include <cstring>
#include <mutex>
#include <string>
#include <vector>

#include "../../include/zq_b200.h"

namespace zq {

// ---------------------------------------------------------------------------------------------------------------
// Resident layouts.
//
// Q4_K keeps the GGUF layout: 144-byte super-blocks of 256 weights (d:f16, dmin:f16, scales[12], qs[128]).
//
// The 32-weight block formats (Q4_0, IQ4_NL: 18 B; Q8_0: 34 B) are only 2-byte aligned in GGUF.  They are
// re-laid at prepare time, without adding bytes, into "units" of 8 blocks = 256 weights whose pieces are 16-byte
// aligned, so that one unit has the same geometry as a Q4_K super-block:
//   Q4_0 / IQ4_NL unit (144 B): d[8]:f16 | 8 pieces of 16 B.  Piece u = t + 4h (t = u%4, h = u/4) holds, for
//       bb = 0..3, 32-bit word t of the 16 quant bytes of block 4h+bb.
//   Q8_0 unit (272 B): d[8]:f16 | 16 pieces of 16 B.  Piece u = t + 4h (h = 0..3) holds, for j = 0..3, 32-bit
//       word 4*(j%2)+t of the 32 quant bytes of block 2h + j/2.
// Rows whose block count is not a multiple of 8 are padded with zero blocks (d = 0).  The interleave puts, in
// each thread's 16-byte piece, exactly the words its warp-MMA fragment consumes (see zq_gemv.cu).
// ---------------------------------------------------------------------------------------------------------------

constexpr int kUnitWeights = 256;

struct FormatInfo {
    uint32_t ggml_type;
    int block_elems;   // GGUF block size in weights
    int block_bytes;   // GGUF block size in bytes
    int unit_bytes;    // resident bytes per 256 weights
};

__host__ __device__ inline FormatInfo format_info(uint32_t t) {
    switch (t) {
    case ZQ_Q4_0: return {ZQ_Q4_0, 32, 18, 144};
    case ZQ_IQ4_NL: return {ZQ_IQ4_NL, 32, 18, 144};
    case ZQ_Q8_0: return {ZQ_Q8_0, 32, 34, 272};
    case ZQ_Q4_K: return {ZQ_Q4_K, 256, 144, 144};
    case ZQ_Q5_K: return {ZQ_Q5_K, 256, 176, 176};
    case ZQ_Q6_K: return {ZQ_Q6_K, 256, 210, 224};   // re-laid: see kQ6k* below
    case ZQ_Q5_0: return {ZQ_Q5_0, 32, 22, 176};   // unit = 8 consecutive GGUF blocks
    case ZQ_Q5_1: return {ZQ_Q5_1, 32, 24, 192};
    case ZQ_Q3_K: return {ZQ_Q3_K, 256, 110, 110};
    case ZQ_IQ4_XS: return {ZQ_IQ4_XS, 256, 136, 136};
    default: return {0, 0, 0, 0};
    }
}

// Types without an unpacker in the f16 decode kernels and without an encoder.  Of these, Q5_K and Q6_K
// (src/weight/codec/ggml.rs:425-469) decode on the integer-MMA kernels (has_i8_decode); with more than 16 rows, or with a
// diagnostic switch that turns those kernels off, they take the f16 operand pass + tensor-core GEMM like the rest.
__host__ __device__ inline bool is_operand_pass_only(uint32_t type) { return type == ZQ_Q5_K || type == ZQ_Q6_K || type == ZQ_Q5_0 || type == ZQ_Q5_1 || type == ZQ_Q3_K || type == ZQ_IQ4_XS; }
// Q5_0, Q5_1, Q3_K and IQ4_XS (src/weight/codec/ggml.rs:111-130, 246-261, 384-406) are resident in GGUF layout, dequantise
// bit-exactly, and run every projection through the f16 operand pass and the tensor-core GEMM.
// Q5_K is Q4_K plus one high bit per weight in a 32-byte field (176-byte super-blocks, a multiple of 16, so TMA can carry
// its rows as they are): its decode (1..16 rows, plain and gated) also runs on the integer-MMA kernels; the f16 kernels
// have no unpacker for it.
__host__ __device__ inline bool has_i8_decode(uint32_t type) { return type == ZQ_Q4_K || type == ZQ_Q4_0 || type == ZQ_Q8_0 || type == ZQ_IQ4_NL || type == ZQ_Q5_K || type == ZQ_Q6_K; }
// Types whose resident bytes are the GGUF bytes; the others are re-laid at prepare time.
__host__ __device__ inline bool resident_is_gguf_layout(uint32_t type) { return type == ZQ_Q4_K || type == ZQ_Q5_K || type == ZQ_Q5_0 || type == ZQ_Q5_1 || type == ZQ_Q3_K || type == ZQ_IQ4_XS; }

// Q6_K resident unit (224 bytes for the 210 of a GGUF super-block, so that rows are 16-byte multiples and TMA can carry
// them): d (f16) and 14 zero bytes; the 16 i8 scales in file order; then the 6-bit codes as c = (q - 32) mod 64 (two's
// complement), split into a low nibble and a high bit pair and ordered for the integer-MMA fragments.  Column
// 32 G + 16 h + 4 t + i of the unit (G 0..7, h 0..1, t 0..3, i 0..3):
//   low nibble   byte kQ6kLow  + 32 t + 4 G + i, bits [4h+3 : 4h]
//   high bits    byte kQ6kHigh + 16 t + 4 (G / 2) + i, bits [2x+1 : 2x], x = 2 (G & 1) + h
// so that lane-in-quad t reads its 48 bytes of a row's unit with three 16-byte loads, and a word of low nibbles masked by
// 0x0F0F0F0F / 0xF0F0F0F0 is the operand of the first / second 16-column scale group of block G.
constexpr int kQ6kScales = 16, kQ6kLow = 32, kQ6kHigh = 160;
// The two formats whose records carry group sums (for the min term) and the Q4_K column order.
__host__ __device__ constexpr bool is_kclass(uint32_t type) { return type == ZQ_Q4_K || type == ZQ_Q5_K; }

// Byte offset, inside a resident unit, of the quant byte that holds element `i` (0..255) of the unit.
__host__ __device__ inline int unit_quant_offset(uint32_t type, int i) {
    if (type == ZQ_Q4_K) {
        int g = i >> 5, j = i & 31;
        return 16 + (g >> 1) * 32 + j;
    }
    int blk = i >> 5, e = i & 31;
    if (type == ZQ_Q8_0) {
        int wv = e >> 2, eh = wv >> 2, t = wv & 3, s = 2 * blk + eh, h = s >> 2, j = s & 3;
        return 16 + 16 * (t + 4 * h) + 4 * j + (e & 3);
    }
    int idx = e & 15, t = idx >> 2, h = blk >> 2, bb = blk & 3;  // Q4_0 / IQ4_NL: nibble = e >> 4
    return 16 + 16 * (t + 4 * h) + 4 * bb + (idx & 3);
}

__device__ __constant__ const int8_t kIq4nlValues[16] = {-127, -104, -83, -65, -49, -35, -22, -10, 1, 13, 25, 38, 53, 69, 89, 113};

// ---------------------------------------------------------------------------------------------------------------
// Device status word: kernels never trap or spin forever.  A bounded wait that runs out records a code here
// and the kernel returns; zq_ctx_sync reports it.
// ---------------------------------------------------------------------------------------------------------------
enum DeviceStatus : uint32_t { kStatusOk = 0, kStatusTmaTimeout = 1, kStatusMmaTimeout = 2, kStatusTmemAlloc = 3, kStatusBadIndex = 4, kStatusPeerTimeout = 5 };

// ---------------------------------------------------------------------------------------------------------------
// PTX wrappers.
// ---------------------------------------------------------------------------------------------------------------
// Programmatic dependent launch.  A decode kernel launched with the stream-serialization attribute may start while
// the previous kernel of the stream is still draining: it sets up its barriers and starts streaming its (constant)
// weights, and only then waits for the previous kernel to complete before it touches activations or outputs.
// Both instructions do nothing in a kernel launched without the attribute.
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;"); }
__device__ __forceinline__ void pdl_wait_prior_grid() { asm volatile("griddepcontrol.wait;" ::: "memory"); }

__device__ __forceinline__ uint32_t smem_u32(const void *p) { return static_cast<uint32_t>(__cvta_generic_to_shared(p)); }

__device__ __forceinline__ void mbar_init(uint64_t *bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t *bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t *bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
// One poll of an mbarrier phase.  The suspend-time hint lets the hardware park the thread (up to ~10 us) until the
// phase completes instead of spinning, so waiting warps do not eat issue slots of the warps that have work.
__device__ __forceinline__ bool mbar_try_wait(uint64_t *bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(parity), "r"(10000u)
        : "memory");
    return ok != 0;
}
// Bounded wait: returns false when the barrier did not complete within `limit` polls (each poll may itself
// block for a hardware-defined short time).  Callers record a status and leave.
__device__ __forceinline__ bool mbar_wait_bounded(uint64_t *bar, uint32_t parity, uint32_t limit = (1u << 22)) {
    for (uint32_t i = 0; i < limit; ++i)
        if (mbar_try_wait(bar, parity)) return true;
    return false;
}
__device__ __forceinline__ void fence_mbar_init() { asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory"); }
__device__ __forceinline__ void fence_proxy_async() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

__device__ __forceinline__ void tma_prefetch_desc(const CUtensorMap *map) {
    asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(map)) : "memory");
}
// 2-D tiled bulk tensor load, global -> this CTA's shared memory, completion on an mbarrier.  No multicast.
__device__ __forceinline__ void tma_load_2d(void *dst, const CUtensorMap *map, uint64_t *bar, int x, int y) {
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];" ::"r"(smem_u32(dst)),
                 "l"(reinterpret_cast<uint64_t>(map)), "r"(smem_u32(bar)), "r"(x), "r"(y)
                 : "memory");
}
// 1-D bulk copy, global -> this CTA's shared memory, completion on an mbarrier.  Both addresses 16-byte aligned, size a
// multiple of 16 bytes.  No multicast.
__device__ __forceinline__ void bulk_load_1d(void *dst, const void *src, uint32_t bytes, uint64_t *bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(smem_u32(dst)), "l"(reinterpret_cast<uint64_t>(src)), "r"(bytes),
                 "r"(smem_u32(bar))
                 : "memory");
}
__device__ __forceinline__ void tma_load_3d(void *dst, const CUtensorMap *map, uint64_t *bar, int x, int y, int z) {
    asm volatile("cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];" ::"r"(smem_u32(dst)),
                 "l"(reinterpret_cast<uint64_t>(map)), "r"(smem_u32(bar)), "r"(x), "r"(y), "r"(z)
                 : "memory");
}

// Warp-level MMA m16n8k16, f16 inputs, f32 accumulate: D = A*B + C.
__device__ __forceinline__ void mma_16816(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

__device__ __forceinline__ uint32_t h2_as_u32(__half2 v) { return *reinterpret_cast<uint32_t *>(&v); }
__device__ __forceinline__ __half2 u32_as_h2(uint32_t v) { return *reinterpret_cast<__half2 *>(&v); }
__device__ __forceinline__ uint32_t lop3_and_or(uint32_t a, uint32_t mask, uint32_t orv) {
    uint32_t r;
    asm("lop3.b32 %0, %1, %2, %3, 0xEA;" : "=r"(r) : "r"(a), "r"(mask), "r"(orv));  // (a & mask) | orv
    return r;
}
__device__ __forceinline__ uint32_t hfma2_u32(uint32_t a, uint32_t b, uint32_t c) {
    uint32_t r;
    asm("fma.rn.f16x2 %0, %1, %2, %3;" : "=r"(r) : "r"(a), "r"(b), "r"(c));
    return r;
}
__device__ __forceinline__ uint32_t hsub2_u32(uint32_t a, uint32_t b) {
    uint32_t r;
    asm("sub.rn.f16x2 %0, %1, %2;" : "=r"(r) : "r"(a), "r"(b));
    return r;
}
__device__ __forceinline__ uint32_t hmul2_u32(uint32_t a, uint32_t b) {
    uint32_t r;
    asm("mul.rn.f16x2 %0, %1, %2;" : "=r"(r) : "r"(a), "r"(b));
    return r;
}

__device__ __forceinline__ float load_as_f32(const void *base, int dtype, size_t index) {
    if (dtype == ZQ_F32) return reinterpret_cast<const float *>(base)[index];
    if (dtype == ZQ_F16) return __half2float(reinterpret_cast<const __half *>(base)[index]);
    return __bfloat162float(reinterpret_cast<const __nv_bfloat16 *>(base)[index]);
}
__device__ __forceinline__ void store_from_f32(void *base, int dtype, size_t index, float v) {
    if (dtype == ZQ_F32) reinterpret_cast<float *>(base)[index] = v;
    else if (dtype == ZQ_F16) reinterpret_cast<__half *>(base)[index] = __float2half_rn(v);
    else reinterpret_cast<__nv_bfloat16 *>(base)[index] = __float2bfloat16_rn(v);
}
__host__ __device__ inline size_t dtype_size(int dtype) { return dtype == ZQ_F32 ? 4 : 2; }

// ---------------------------------------------------------------------------------------------------------------
// Host side.
// ---------------------------------------------------------------------------------------------------------------
int set_error(zq_error *err, int code, const char *fmt, ...);

#define ZQ_CUDA_CHECK(expr, err)                                                                                            \
    do {                                                                                                                    \
        cudaError_t _e = (expr);                                                                                            \
        if (_e != cudaSuccess) return zq::set_error((err), ZQ_ERR_CUDA, "%s failed: %s (%s:%d)", #expr, cudaGetErrorString(_e), __FILE__, __LINE__); \
    } while (0)

typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *, const cuuint64_t *, const cuuint32_t *, const cuuint32_t *,
                                  CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
EncodeTiledFn get_encode_tiled(zq_error *err);

}  // namespace zq

struct zq_dist_state;
struct zq_ep_state;

struct zq_ctx {
    int device = 0;
    zq_dist_state *dist = nullptr;  // peer group of the node (zq_dist_export / zq_dist_init), or null
    zq_ep_state *ep = nullptr;      // expert-parallel exchange buffers (zq_moe_ep_export / zq_moe_ep_init), or null
    int sm_count = 0;
    cudaStream_t own_stream = nullptr;
    cudaStream_t stream = nullptr;
    // Split-K fix-up scratch of the decode GEMV: partial tiles and per-tile arrival counters (zeroed once;
    // the finishing CTA of every tile resets its counter).
    float *gemv_partials = nullptr;
    uint32_t *gemv_counters = nullptr;
    size_t gemv_partials_floats = 0;
    size_t gemv_counters_n = 0;
    // General workspace (grows on demand, never shrinks): dequantised operands of the prefill GEMM, MoE buffers.
    void *workspace = nullptr;
    size_t workspace_bytes = 0;
    // MoE buffers: routing tables, gathered rows, per-route activations and outputs (grows on demand).
    void *moe_ws = nullptr;
    size_t moe_ws_bytes = 0;
    // Quantised activations of the integer-MMA decode kernel for more than 4 rows (grows on demand).
    void *xq = nullptr;
    size_t xq_bytes = 0;
    // Activated intermediate [m, I] of gated_mlp (grows on demand).
    void *mid = nullptr;
    size_t mid_bytes = 0;
    void *norm = nullptr;  // normalised activations of zq_rmsnorm_linear (f32)
    size_t norm_bytes = 0;
    // Device status word (mapped pinned host memory so the host can read it without a copy).
    uint32_t *status_host = nullptr;
    uint32_t *status_dev = nullptr;
    // Pinned staging for the *_host entry points.
    void *pinned = nullptr;
    size_t pinned_bytes = 0;
    void *host_io_dev = nullptr;
    size_t host_io_bytes = 0;
    // Batch bracket (zq_batch_begin / zq_batch_finish): host-buffer calls inside it stage through these chunks and
    // defer their copy-out to the finish.
    struct IoChunk { uint8_t *pinned; uint8_t *dev; size_t bytes, used; };
    struct PendingOut { void *host; const uint8_t *pinned; size_t bytes; };
    // A host-buffer linear of an open bracket: its input is already on its way to `dev_x`; the layer itself runs at the
    // bracket's finish, together with the bracket's other layers, as one zq_linear_batch call (work-list launches).
    struct PendingLinear { const zq_weight *w; const uint8_t *dev_x; size_t m; uint8_t *dev_y; void *host_y_direct; size_t y_bytes; int x_dtype, y_dtype; };
    struct PendingIn { const void *host; size_t bytes; const uint8_t *dev; };  // page-locked inputs already copied in this bracket
    // Copy streams of a bracket: inputs travel on io_in and results on io_out while the compute stream runs the layers
    // (events order a batch of layers after its inputs and the copies out after the batch); created on first use.
    cudaStream_t io_in = nullptr, io_out = nullptr;
    cudaEvent_t ev_in = nullptr, ev_done = nullptr;
    bool io_out_used = false;
    std::vector<IoChunk> io_chunks;
    std::vector<PendingOut> pending_out;
    std::vector<PendingLinear> pending_linear;
    std::vector<PendingIn> pending_in;
    bool batch_active = false;
    // Diagnostics: 1 = always use the per-item activation staging GEMV (the variant for activations too large to
    // stay resident in shared memory), so that tests can cover it at small sizes.
    int force_staged_gemv = 0;
    // 1 = run Q4_K decode on the tcgen05 kernel (zq_qmv.cu) instead of the warp-MMA kernels.  Off by default: it is
    // parity-clean but, as measured, not yet faster than the warp-MMA path.
    int enable_tcgen05_gemv = 0;
    int force_f16_gemv = 0;  // skip the integer-MMA decode kernel (tests of the f16 kernels)
    int narrow_gemv_tiles = 0;  // integer-MMA decode, up to 4 rows: 64-row tiles, two CTAs per SM (measured slower; off)
    int disable_pdl = 0;     // launch decode kernels without programmatic dependent launch
    int disable_worklist = 0;  // zq_linear_batch and the multi-weight entries: one launch per job instead of the work-list kernel
    int force_fused_gemm = 0;      // Q4_K prefill: the fused kernel for every token count (tests)
    int disable_fused_gemm = 0;    // Q4_K prefill: separate f16 operand pass + plain GEMM instead of the fused kernel
    int force_moe_per_expert = 0;  // MoE forward: always the host-grouped per-expert path (tests)
    const void *moe_row_sink = nullptr;  // zq::PeerRowSink of the expert-parallel forward while it runs its local experts, else null
    int force_moe_host_grouping = 0;  // MoE prefill: group the routes on the host instead of on the device (tests, A/B)
    std::atomic<uint64_t> launches{0};
    std::mutex mutex;
};

struct zq_weight {
    zq_ctx *ctx = nullptr;
    uint32_t type = 0;
    size_t rows = 0, cols = 0;
    size_t units_per_row = 0;    // ceil(cols / 256)
    size_t row_pitch = 0;        // resident bytes per row = units_per_row * unit_bytes
    size_t gguf_bytes = 0;       // bytes of the original packing
    uint8_t *data = nullptr;     // resident layout, device
    bool owns_data = true;
    CUtensorMap gemv_map;        // u32 tensor [rows, row_pitch/4], box = (chunk words, 128 rows): decode GEMV
    CUtensorMap qmv_map;         // same tensor, box of one unit x 128 rows: tcgen05 decode kernel
    CUtensorMap gemv_map_half;   // same tensor, box of 64 rows: gated GEMV (gate and up halves of one stage)
    // Device copies {gemv_map, gemv_map_half, qmv_map} behind the resident bytes (same allocation), for kernels that
    // pick their weight from a table at run time; null for the types no decode kernel reads through TMA.
    CUtensorMap *d_maps = nullptr;
};

namespace zq {
int use_device(zq_ctx *ctx, zq_error *err);
int ensure_workspace(zq_ctx *ctx, size_t bytes, zq_error *err);
int ensure_xq(zq_ctx *ctx, size_t bytes, zq_error *err);
int launch_gemm_fused_grouped(zq_ctx *ctx, const CUtensorMap *w_maps, const CUtensorMap *w2_maps, size_t rows, size_t k, const __half *x, size_t x_rows, const int4 *items, int n_items, const int *n_items_dev, void *y, int y_dtype, zq_error *err);
int launch_gemm_f16(zq_ctx *ctx, const __half *w, size_t rows, size_t k, const __half *x, size_t m, void *y, int y_dtype, zq_error *err);
int launch_to_f16(zq_ctx *ctx, const void *x, int x_dtype, __half *out, size_t n, zq_error *err);
int launch_gemm_grouped(zq_ctx *ctx, const __half *w, const __half *w2, size_t mats, size_t rows, size_t k, const __half *x, size_t x_rows, const int4 *items, int n_items, void *y, int y_dtype, zq_error *err);
int ensure_scratch_mid(zq_ctx *ctx, size_t bytes, zq_error *err);
int ensure_scratch_norm(zq_ctx *ctx, size_t bytes, zq_error *err);
int launch_rmsnorm(zq_ctx *ctx, const void *x, int x_dtype, size_t m, size_t cols, const float *weight, float eps, float weight_offset, float *out, zq_error *err);
int make_weight_map(const zq_weight *w, int box_words, int box_rows, CUtensorMap *out, zq_error *err);

// Launchers implemented in the .cu files.
int launch_repack(zq_ctx *ctx, uint32_t type, const uint8_t *gguf, uint8_t *resident, size_t rows, size_t cols, zq_error *err);
int launch_dequantize(zq_ctx *ctx, const zq_weight *w, const uint32_t *row_ids, size_t n_rows, void *out, int out_dtype, zq_error *err);
int launch_dequantize_f16(zq_ctx *ctx, const zq_weight *w, __half *out, zq_error *err);
int launch_dequantize_f16_batch(zq_ctx *ctx, const zq_weight *const *weights, __half *const *outs, size_t count, zq_error *err);
int launch_quantize(zq_ctx *ctx, uint32_t type, const float *values, size_t rows, size_t cols, void *out, zq_error *err);
int launch_gemv(zq_ctx *ctx, const zq_weight *w, const zq_weight *w_up, const void *x, int x_dtype, size_t m, void *y, int y_dtype, const void *residual, zq_error *err);
int launch_gemv_noalloc(zq_ctx *ctx, const zq_weight *w, const void *x, int x_dtype, size_t m, void *y, int y_dtype, zq_error *err);
int launch_gemm(zq_ctx *ctx, const zq_weight *w, const zq_weight *w_up, const void *x, int x_dtype, size_t m, void *y, int y_dtype, const void *residual, zq_error *err);
}  // namespace zq
