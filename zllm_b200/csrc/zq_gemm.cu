// Prefill GEMM for GGUF block-quantised weights on the 5th-generation tensor cores (tcgen05 + TMEM), sm_100a.
//
// Replaces the reference's prefill kernels gguf_kq_matmul_f16 / gated_linear_q4_k_silu_rows8_f16 and its
// "dequantise, then cuBLAS" Q4_0 path (src/kernel/cuda/linear.rs:94-138, 880-941, 1141-1166, 1345-1390); the
// arithmetic contract is ggml_quant::matmul / gated_silu_matmul (src/kernel/cpu/ggml_quant.rs:280-362):
// Y[token, row] = sum_k X[token, k] * dequant(W)[row, k], f32 accumulation.
//
// Data flow of this version:
//   1. dequantise the resident packed weight once into an f16 [rows, K] operand in the context workspace
//      (f32 value rounded once to f16: 2^-12 relative, which keeps layer outputs inside the 2e-3 bound; bf16
//      operands would not), and convert the activations to f16 (exact for bf16/f16 inputs in f16 range);
//   2. persistent CTAs (one per SM) walk output tiles of 128 weight rows x 256 tokens: a TMA warp streams
//      64-column K blocks of both operands (128-byte swizzle) through a 4-stage mbarrier ring; one thread issues
//      tcgen05.mma (M=128, N=256, K=16, kind::f16, f32 accumulator in 256 TMEM columns); tcgen05.commit releases
//      ring stages and signals the epilogue warps, which read the accumulator with tcgen05.ld and store
//      Y (+ residual) in the requested dtype while the MMAs of the next tile fill the second accumulator.  For the
//      gated form two accumulators (gate and up, all 512 TMEM columns) share the activation tile and the epilogue
//      applies silu(gate) * up.
// Every wait is bounded; a wait that runs out raises the CTA's abort flag, all roles fall through to the end,
// TMEM is released and the context status word reports it.
#include "zq_common.cuh"

namespace zq {

constexpr int kBM = 128;   // weight rows per CTA (UMMA M)
constexpr int kBN = 256;   // tokens per CTA (UMMA N)
constexpr int kBK = 64;    // K elements per ring stage (128 bytes of f16: one swizzle atom row)
constexpr int kGemmThreads = 192;  // warp 0: TMA, warp 1: MMA + TMEM owner, warps 2..5: epilogue

struct GemmParams {
    void *y;
    const void *residual;
    uint32_t *status;
    int y_dtype;
    int m;       // tokens
    int n_out;   // weight rows
    int k;       // input columns
    // Grouped form (MoE prefill): the work list replaces the tile grid.  Item = {weight matrix z of the 3-D weight
    // operand, first row of the tile, first token row, end of the matrix's token rows}; tokens are rows of one
    // activation operand shared by all matrices, outputs are rows of y with n_out columns.
    const int4 *items;
    int n_items;
};

// ---- tcgen05 wrappers -------------------------------------------------------------------------------------------
__device__ __forceinline__ void tmem_alloc(uint32_t *smem_dst, uint32_t cols) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(smem_dst)), "r"(cols) : "memory");
}
__device__ __forceinline__ void tmem_relinquish() { asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t cols) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(cols) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_commit(uint64_t *bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}
// D[tmem] (+)= A[smem] * B[smem], both K-major, f16 inputs, f32 accumulate.
__device__ __forceinline__ void umma_f16_ss(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
        : "memory");
}
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t (&r)[16]) {
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]),
                   "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
                 : "r"(taddr)
                 : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// K-major operand tile in shared memory, rows of 128 bytes, 128-byte swizzle: 8-row groups are 1024 bytes apart.
__device__ __forceinline__ uint64_t make_sw128_desc(uint32_t smem_addr) {
    uint64_t desc = 0;
    desc |= (uint64_t)((smem_addr & 0x3FFFFu) >> 4);   // start address, 16-byte units
    desc |= (uint64_t)1 << 16;                         // leading byte offset: unused for swizzled K-major, 1 by convention
    desc |= (uint64_t)(1024 >> 4) << 32;               // stride byte offset between 8-row groups
    desc |= (uint64_t)1 << 46;                         // descriptor version of this architecture
    desc |= (uint64_t)2 << 61;                         // SWIZZLE_128B
    return desc;
}

__device__ __forceinline__ bool wait_flag(uint64_t *bar, uint32_t parity, volatile int *abort_flag, uint32_t *status, uint32_t code) {
    for (uint32_t i = 0; i < (1u << 22); ++i) {
        if (mbar_try_wait(bar, parity)) return true;
        if (*abort_flag) return false;
    }
    *abort_flag = 1;
    atomicMax(status, code);
    return false;
}

template <bool GATED> struct GemmSmem {
    static constexpr int stages = GATED ? 3 : 4;
    static constexpr int acc_bufs = GATED ? 1 : 2;  // 256-column accumulators that fit the 512 TMEM columns
    static constexpr int a_bytes = kBM * kBK * 2;  // 16 KB
    static constexpr int b_bytes = kBN * kBK * 2;  // 32 KB
    static constexpr int stage_bytes = (GATED ? 2 : 1) * a_bytes + b_bytes;
    static constexpr int off_bar = stages * stage_bytes;
    static constexpr int total = off_bar + 256 + 1024;  // barriers, tmem slot, slack for 1024-byte alignment
};

constexpr int kTokGroup = 8;  // token tiles per raster group: a weight tile is reused by 8 token tiles while it is hot in L2

// Persistent CTA (one per SM) over output tiles of 128 weight rows x 256 tokens.  Tiles are rastered in groups of
// 8 token tiles x all row tiles (token tile fastest), so that the CTAs in flight share weight tiles and the group's
// activation tiles stay in L2.  The plain form double-buffers the accumulator in tensor memory: the epilogue of tile
// i runs while the MMAs of tile i+1 fill the other buffer, and the TMA ring never drains between tiles.
template <bool GATED>
__global__ void __launch_bounds__(kGemmThreads, 1) gemm_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_w2, const __grid_constant__ CUtensorMap map_x, const GemmParams p) {
    using S = GemmSmem<GATED>;
    constexpr int STAGES = S::stages;
    constexpr int ACC = S::acc_bufs;
    constexpr uint32_t ACC_COLS = GATED ? 512 : 256;
    constexpr uint32_t TMEM_COLS = 512;
    extern __shared__ uint8_t smem_raw[];
    uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint64_t *full = reinterpret_cast<uint64_t *>(smem + S::off_bar);
    uint64_t *empty = full + STAGES;
    uint64_t *acc_full = empty + STAGES;
    uint64_t *acc_empty = acc_full + 2;
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(acc_empty + 2);
    __shared__ int s_abort;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int k_blocks = (p.k + kBK - 1) / kBK;
    const int n_row_tiles = (p.n_out + kBM - 1) / kBM, n_tok_tiles = (p.m + kBN - 1) / kBN;
    const bool grouped = p.items != nullptr;
    const int total_tiles = grouped ? p.n_items : n_row_tiles * n_tok_tiles;
    auto tile_coords = [&](int tile, int &row0, int &tok0, int &tok_end, int &z) {
        if (grouped) {
            const int4 it = p.items[tile];
            z = it.x;
            row0 = it.y;
            tok0 = it.z;
            tok_end = it.w;
            return;
        }
        z = 0;
        tok_end = p.m;
        const int per_group = kTokGroup * n_row_tiles;
        const int group = tile / per_group, in_group = tile - group * per_group;
        const int group_toks = (n_tok_tiles - group * kTokGroup) < kTokGroup ? (n_tok_tiles - group * kTokGroup) : kTokGroup;
        row0 = (in_group / group_toks) * kBM;
        tok0 = (group * kTokGroup + in_group % group_toks) * kBN;
    };

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(&full[s], 1);
            mbar_init(&empty[s], 1);
        }
        for (int b = 0; b < 2; ++b) {
            mbar_init(&acc_full[b], 1);
            mbar_init(&acc_empty[b], 4);
        }
        fence_mbar_init();
        s_abort = 0;
        tma_prefetch_desc(&map_w);
        tma_prefetch_desc(&map_x);
        if (GATED) tma_prefetch_desc(&map_w2);
    }
    if (warp == 1) {
        tmem_alloc(tmem_slot, TMEM_COLS);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *reinterpret_cast<volatile uint32_t *>(tmem_slot);

    if (warp == 0) {
        // ------------------------------------------------ TMA producer
        if (lane == 0) {
            long long kg = 0;  // k-block counter over all tiles of this CTA: ring position
            for (int tile = blockIdx.x; tile < total_tiles; tile += gridDim.x) {
                int row0, tok0, tok_end, z;
                tile_coords(tile, row0, tok0, tok_end, z);
                for (int kb = 0; kb < k_blocks; ++kb, ++kg) {
                    const int s = (int)(kg % STAGES);
                    if (kg >= STAGES && !wait_flag(&empty[s], (uint32_t)((kg / STAGES) - 1) & 1, &s_abort, p.status, kStatusMmaTimeout)) break;
                    uint8_t *st = smem + (size_t)s * S::stage_bytes;
                    mbar_expect_tx(&full[s], S::stage_bytes);
                    if (grouped) {
                        tma_load_3d(st, &map_w, &full[s], kb * kBK, row0, z);
                        if (GATED) tma_load_3d(st + S::a_bytes, &map_w2, &full[s], kb * kBK, row0, z);
                    } else {
                        tma_load_2d(st, &map_w, &full[s], kb * kBK, row0);
                        if (GATED) tma_load_2d(st + S::a_bytes, &map_w2, &full[s], kb * kBK, row0);
                    }
                    tma_load_2d(st + (GATED ? 2 : 1) * S::a_bytes, &map_x, &full[s], kb * kBK, tok0);
                }
                if (*(volatile int *)&s_abort) break;
            }
        }
    } else if (warp == 1) {
        // ------------------------------------------------ MMA issuer
        if (lane == 0) {
            long long kg = 0;
            int iter = 0;
            bool ok = true;
            for (int tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x, ++iter) {
                // instruction descriptor: f32 accumulator, f16 A and B, both K-major, M = 128, N = the tile's token
                // count rounded up to 16 (a ragged last tile of a matrix does not pay for 256 columns)
                int row0, tok0, tok_end, z;
                tile_coords(tile, row0, tok0, tok_end, z);
                int n_eff = tok_end - tok0;
                n_eff = n_eff >= kBN ? kBN : ((n_eff + 15) & ~15);
                if (n_eff < 16) n_eff = 16;
                const uint32_t idesc = (1u << 4) | ((uint32_t)(n_eff >> 3) << 17) | ((uint32_t)(kBM >> 4) << 24);
                const int b = iter % ACC;
                if (iter >= ACC) ok = wait_flag(&acc_empty[b], (uint32_t)((iter / ACC) - 1) & 1, &s_abort, p.status, kStatusMmaTimeout);
                if (!ok) break;
                tc_fence_after();
                const uint32_t acc_addr = tmem_base + (uint32_t)b * ACC_COLS;
                for (int kb = 0; kb < k_blocks && ok; ++kb, ++kg) {
                    const int s = (int)(kg % STAGES);
                    ok = wait_flag(&full[s], (uint32_t)(kg / STAGES) & 1, &s_abort, p.status, kStatusTmaTimeout);
                    if (!ok) break;
                    tc_fence_after();
                    const uint32_t st = smem_u32(smem + (size_t)s * S::stage_bytes);
                    const uint64_t da = make_sw128_desc(st);
                    const uint64_t da2 = make_sw128_desc(st + S::a_bytes);
                    const uint64_t db = make_sw128_desc(st + (GATED ? 2 : 1) * S::a_bytes);
#pragma unroll
                    for (int k = 0; k < kBK / 16; ++k) {
                        const uint32_t acc = (kb > 0 || k > 0) ? 1u : 0u;
                        // 16 K elements = 32 bytes = 2 descriptor units along the swizzled row
                        umma_f16_ss(acc_addr, da + 2 * k, db + 2 * k, idesc, acc);
                        if (GATED) umma_f16_ss(acc_addr + kBN, da2 + 2 * k, db + 2 * k, idesc, acc);
                    }
                    tc_commit(&empty[s]);  // arrives once the MMAs above have read the stage
                }
                tc_commit(&acc_full[b]);   // arrives when every MMA of the tile has completed
            }
        }
    } else {
        // ------------------------------------------------ epilogue: warp q of 4 owns TMEM lanes 32q..32q+31
        const int q = warp & 3;
        int iter = 0;
        for (int tile = blockIdx.x; tile < total_tiles; tile += gridDim.x, ++iter) {
            int row0, tok0, tok_end, z;
            tile_coords(tile, row0, tok0, tok_end, z);
            const int b = iter % ACC;
            const int row = row0 + q * 32 + lane;
            const bool ok = wait_flag(&acc_full[b], (uint32_t)(iter / ACC) & 1, &s_abort, p.status, kStatusMmaTimeout);
            tc_fence_after();
            if (ok) {
                const uint32_t lane_base = tmem_base + (uint32_t)b * ACC_COLS + ((uint32_t)(q * 32) << 16);
                for (int c0 = 0; c0 < kBN; c0 += 16) {
                    if (tok0 + c0 >= tok_end) break;  // warp-uniform
                    uint32_t v[16], u[16];
                    tmem_ld16(lane_base + c0, v);
                    if (GATED) tmem_ld16(lane_base + kBN + c0, u);
                    tmem_ld_wait();
                    if (row < p.n_out) {
#pragma unroll
                        for (int j = 0; j < 16; ++j) {
                            const int tok = tok0 + c0 + j;
                            if (tok < tok_end) {
                                float val = __uint_as_float(v[j]);
                                if (GATED) {
                                    const float up = __uint_as_float(u[j]);
                                    val = (val / (1.0f + expf(-val))) * up;  // src/kernel/cpu/ggml_quant.rs:352
                                }
                                const size_t o = (size_t)tok * p.n_out + row;
                                if (p.residual) val += load_as_f32(p.residual, p.y_dtype, o);
                                store_from_f32(p.y, p.y_dtype, o, val);
                            }
                        }
                    }
                }
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(&acc_empty[b]);  // this warp's quarter of the accumulator may be overwritten
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 1) tmem_dealloc(tmem_base, TMEM_COLS);
}

// activations of any supported dtype -> f16 [m, k]
__global__ void to_f16_kernel(const void *__restrict__ x, int x_dtype, __half *__restrict__ out, size_t n) {
    for (size_t i = ((size_t)blockIdx.x * blockDim.x + threadIdx.x) * 4; i < n; i += (size_t)gridDim.x * blockDim.x * 4) {
#pragma unroll
        for (int j = 0; j < 4; ++j)
            if (i + j < n) out[i + j] = __float2half_rn(load_as_f32(x, x_dtype, i + j));
    }
}

static int make_f16_map(const void *base, size_t rows, size_t cols, int box_rows, CUtensorMap *out, zq_error *err) {
    EncodeTiledFn encode = get_encode_tiled(err);
    if (!encode) return ZQ_ERR_CUDA;
    cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
    cuuint64_t strides[1] = {(cuuint64_t)cols * 2};
    cuuint32_t box[2] = {(cuuint32_t)kBK, (cuuint32_t)box_rows};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = encode(out, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, const_cast<void *>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                         CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return set_error(err, ZQ_ERR_CUDA, "cuTensorMapEncodeTiled (f16 operand %zux%zu) failed with code %d", rows, cols, (int)r);
    return ZQ_OK;
}

// y[m, n] = x[m, k] W^T (+ residual), or silu(x gate^T) * (x up^T) when w_up is given.
int launch_gemm(zq_ctx *ctx, const zq_weight *w, const zq_weight *w_up, const void *x, int x_dtype, size_t m, void *y, int y_dtype, const void *residual, zq_error *err) {
    const bool gated = w_up != nullptr;
    const size_t n = w->rows, k = w->cols;
    if (k % 8) return set_error(err, ZQ_ERR_SHAPE, "prefill GEMM needs columns aligned to 8, got %zu", k);
    const size_t w_bytes = (n * k * 2 + 255) & ~size_t(255);
    const size_t x_bytes = (m * k * 2 + 255) & ~size_t(255);
    int rc = ensure_workspace(ctx, (gated ? 2 : 1) * w_bytes + x_bytes, err);
    if (rc) return rc;
    uint8_t *ws = reinterpret_cast<uint8_t *>(ctx->workspace);
    __half *w16 = reinterpret_cast<__half *>(ws);
    __half *w16b = reinterpret_cast<__half *>(ws + w_bytes);
    __half *x16 = reinterpret_cast<__half *>(ws + (gated ? 2 : 1) * w_bytes);
    rc = launch_dequantize_f16(ctx, w, w16, err);
    if (!rc && gated) rc = launch_dequantize_f16(ctx, w_up, w16b, err);
    if (rc) return rc;
    const __half *xin = reinterpret_cast<const __half *>(x);
    if (x_dtype != ZQ_F16) {
        const size_t total = m * k;
        size_t blocks = (total / 4 + 255) / 256;
        if (blocks > (size_t)ctx->sm_count * 32) blocks = (size_t)ctx->sm_count * 32;
        if (blocks == 0) blocks = 1;
        to_f16_kernel<<<(unsigned)blocks, 256, 0, ctx->stream>>>(x, x_dtype, x16, total);
        ctx->launches++;
        ZQ_CUDA_CHECK(cudaGetLastError(), err);
        xin = x16;
    }
    CUtensorMap map_w, map_w2, map_x;
    rc = make_f16_map(w16, n, k, kBM, &map_w, err);
    if (!rc) rc = make_f16_map(gated ? w16b : w16, n, k, kBM, &map_w2, err);
    if (!rc) rc = make_f16_map(xin, m, k, kBN, &map_x, err);
    if (rc) return rc;
    GemmParams p;
    p.y = y;
    p.residual = residual;
    p.status = ctx->status_dev;
    p.y_dtype = y_dtype;
    p.m = (int)m;
    p.n_out = (int)n;
    p.k = (int)k;
    p.items = nullptr;
    p.n_items = 0;
    const size_t total_tiles = ((n + kBM - 1) / kBM) * ((m + kBN - 1) / kBN);
    dim3 grid((unsigned)(total_tiles < (size_t)ctx->sm_count ? total_tiles : (size_t)ctx->sm_count));
    static bool configured[2][64] = {};
    if (gated) {
        if (!configured[1][ctx->device & 63]) {
            ZQ_CUDA_CHECK(cudaFuncSetAttribute(gemm_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, GemmSmem<true>::total), err);
            configured[1][ctx->device & 63] = true;
        }
        gemm_kernel<true><<<grid, kGemmThreads, GemmSmem<true>::total, ctx->stream>>>(map_w, map_w2, map_x, p);
    } else {
        if (!configured[0][ctx->device & 63]) {
            ZQ_CUDA_CHECK(cudaFuncSetAttribute(gemm_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, GemmSmem<false>::total), err);
            configured[0][ctx->device & 63] = true;
        }
        gemm_kernel<false><<<grid, kGemmThreads, GemmSmem<false>::total, ctx->stream>>>(map_w, map_w2, map_x, p);
    }
    ctx->launches++;
    ZQ_CUDA_CHECK(cudaGetLastError(), err);
    return ZQ_OK;
}

static int make_f16_map3(const void *base, size_t mats, size_t rows, size_t cols, CUtensorMap *out, zq_error *err) {
    EncodeTiledFn encode = get_encode_tiled(err);
    if (!encode) return ZQ_ERR_CUDA;
    cuuint64_t dims[3] = {(cuuint64_t)cols, (cuuint64_t)rows, (cuuint64_t)mats};
    cuuint64_t strides[2] = {(cuuint64_t)cols * 2, (cuuint64_t)rows * cols * 2};
    cuuint32_t box[3] = {(cuuint32_t)kBK, (cuuint32_t)kBM, 1};
    cuuint32_t estr[3] = {1, 1, 1};
    CUresult r = encode(out, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 3, const_cast<void *>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                         CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return set_error(err, ZQ_ERR_CUDA, "cuTensorMapEncodeTiled (f16 operand %zux%zux%zu) failed with code %d", mats, rows, cols, (int)r);
    return ZQ_OK;
}

int launch_to_f16(zq_ctx *ctx, const void *x, int x_dtype, __half *out, size_t n, zq_error *err) {
    size_t blocks = (n / 4 + 255) / 256;
    if (blocks > (size_t)ctx->sm_count * 32) blocks = (size_t)ctx->sm_count * 32;
    if (blocks == 0) blocks = 1;
    to_f16_kernel<<<(unsigned)blocks, 256, 0, ctx->stream>>>(x, x_dtype, out, n);
    ctx->launches++;
    ZQ_CUDA_CHECK(cudaGetLastError(), err);
    return ZQ_OK;
}

// Grouped GEMM (MoE prefill): `mats` f16 weight matrices [rows, k] stacked in one buffer (and a second stack for the
// gated form), one f16 activation operand [x_rows, k] whose row ranges belong to the matrices, a device work list of
// {matrix, first row, first token row, end token row}.  y[token row, rows] in y_dtype; gated: silu(w x) * (w2 x).
int launch_gemm_grouped(zq_ctx *ctx, const __half *w, const __half *w2, size_t mats, size_t rows, size_t k, const __half *x, size_t x_rows, const int4 *items, int n_items, void *y, int y_dtype, zq_error *err) {
    if (n_items <= 0) return ZQ_OK;
    if (k % 8) return set_error(err, ZQ_ERR_SHAPE, "grouped GEMM needs columns aligned to 8, got %zu", k);
    const bool gated = w2 != nullptr;
    CUtensorMap map_w, map_w2, map_x;
    int rc = make_f16_map3(w, mats, rows, k, &map_w, err);
    if (!rc) rc = make_f16_map3(gated ? w2 : w, mats, rows, k, &map_w2, err);
    if (!rc) rc = make_f16_map(x, x_rows, k, kBN, &map_x, err);
    if (rc) return rc;
    GemmParams p;
    p.y = y;
    p.residual = nullptr;
    p.status = ctx->status_dev;
    p.y_dtype = y_dtype;
    p.m = (int)x_rows;
    p.n_out = (int)rows;
    p.k = (int)k;
    p.items = items;
    p.n_items = n_items;
    dim3 grid((unsigned)(n_items < ctx->sm_count ? n_items : ctx->sm_count));
    static bool configured[2][64] = {};
    if (gated) {
        if (!configured[1][ctx->device & 63]) {
            ZQ_CUDA_CHECK(cudaFuncSetAttribute(gemm_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, GemmSmem<true>::total), err);
            configured[1][ctx->device & 63] = true;
        }
        gemm_kernel<true><<<grid, kGemmThreads, GemmSmem<true>::total, ctx->stream>>>(map_w, map_w2, map_x, p);
    } else {
        if (!configured[0][ctx->device & 63]) {
            ZQ_CUDA_CHECK(cudaFuncSetAttribute(gemm_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, GemmSmem<false>::total), err);
            configured[0][ctx->device & 63] = true;
        }
        gemm_kernel<false><<<grid, kGemmThreads, GemmSmem<false>::total, ctx->stream>>>(map_w, map_w2, map_x, p);
    }
    ctx->launches++;
    ZQ_CUDA_CHECK(cudaGetLastError(), err);
    return ZQ_OK;
}

// Plain f16 x f16 GEMM on raw operands: y[m, rows] = x[m, k] w[rows, k]^T, f32 accumulation (router logits).
int launch_gemm_f16(zq_ctx *ctx, const __half *w, size_t rows, size_t k, const __half *x, size_t m, void *y, int y_dtype, zq_error *err) {
    if (k % 8) return set_error(err, ZQ_ERR_SHAPE, "f16 GEMM needs columns aligned to 8, got %zu", k);
    CUtensorMap map_w, map_x;
    int rc = make_f16_map(w, rows, k, kBM, &map_w, err);
    if (!rc) rc = make_f16_map(x, m, k, kBN, &map_x, err);
    if (rc) return rc;
    GemmParams p;
    p.y = y;
    p.residual = nullptr;
    p.status = ctx->status_dev;
    p.y_dtype = y_dtype;
    p.m = (int)m;
    p.n_out = (int)rows;
    p.k = (int)k;
    p.items = nullptr;
    p.n_items = 0;
    const size_t total_tiles = ((rows + kBM - 1) / kBM) * ((m + kBN - 1) / kBN);
    dim3 grid((unsigned)(total_tiles < (size_t)ctx->sm_count ? total_tiles : (size_t)ctx->sm_count));
    static bool configured[64] = {};
    if (!configured[ctx->device & 63]) {
        ZQ_CUDA_CHECK(cudaFuncSetAttribute(gemm_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, GemmSmem<false>::total), err);
        configured[ctx->device & 63] = true;
    }
    gemm_kernel<false><<<grid, kGemmThreads, GemmSmem<false>::total, ctx->stream>>>(map_w, map_w, map_x, p);
    ctx->launches++;
    ZQ_CUDA_CHECK(cudaGetLastError(), err);
    return ZQ_OK;
}

}  // namespace zq
