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
    const int *n_items_dev;  // when set, the item count is read from device memory (a plan kernel wrote it); n_items is then its upper bound
    // fused Q4_K kernel, grouped form: per-matrix tensor maps of the packed weights (device table indexed by z)
    const CUtensorMap *w_maps, *w2_maps;
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

// Same, for roles that share a scheduler with working warps: a failed poll is followed by a short sleep, so that
// the waiting warp does not take issue slots from the warps that are dequantising (a bare poll loop re-issues every
// few tens of nanoseconds).
__device__ __forceinline__ bool wait_flag_backoff(uint64_t *bar, uint32_t parity, volatile int *abort_flag, uint32_t *status, uint32_t code, unsigned sleep_ns) {
    for (uint32_t i = 0; i < (1u << 22); ++i) {
        if (mbar_try_wait(bar, parity)) return true;
        if (*abort_flag) return false;
        __nanosleep(sleep_ns);
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
    const int total_tiles = grouped ? (p.n_items_dev ? *p.n_items_dev : p.n_items) : n_row_tiles * n_tok_tiles;
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

// ---------------------------------------------------------------------------------------------------------------
// Fused form for Q4_K: the packed weight tile is dequantised inside the kernel, straight into the swizzled shared-
// memory operand the tensor core reads, so the weight crosses HBM once (0.56 bytes per weight instead of the
// 0.56 + 2 + 2 of a separate f16 operand pass).  Same tile walk, MMA issue and epilogue as gemm_kernel; what differs is
// the A side of the ring:
//   warp 0        TMA: one packed box per 256 K columns (128 rows x 144 bytes) into a 2-deep ring, and the
//                 activation k-blocks (256 tokens x 64 K, 128-byte swizzle) into the main ring
//   warps 6..13   dequantisers: thread = (row, half of the 64-column k-block) = one 32-weight scale group; reads the
//                 group's packed bytes and (once per super-block) the row's scales from the packed box, forms
//                 fma(d*sc, q, -dmin*m) in f32, rounds once to f16 and stores its four
//                 16-byte chunks at their 128-byte-swizzle positions (chunk c of row r sits at c ^ (r & 7)), then
//                 fence.proxy.async and one arrival per warp on the stage's a_full barrier
//   warp 1        waits for a_full and b_full of a stage, issues the four K=16 MMAs, commits the stage's `empty`
// The operand bits are exactly those the separate operand pass writes (same formula), so both paths give identical
// results.  A last warp issues the packed boxes on a ring of its own.
// ---------------------------------------------------------------------------------------------------------------
constexpr int kFusedDqWarps = 8;   // thread = (row, half of the k-block) = one 32-weight scale group
constexpr int kFusedThreads = (7 + kFusedDqWarps) * 32;  // + TMA (activations), MMA, 4 epilogue, TMA (packed boxes)
constexpr int kFusedPackedWarp = 6 + kFusedDqWarps;
constexpr int kQ4kUnitBytes = 144;

template <bool GATED> struct FusedSmem {
    static constexpr int stages = GATED ? 2 : 3;
    static constexpr int pstages = GATED ? 2 : 3;
    static constexpr int acc_bufs = GATED ? 1 : 2;
    static constexpr int a_bytes = kBM * kBK * 2;
    static constexpr int b_bytes = kBN * kBK * 2;
    static constexpr int p_bytes = kBM * kQ4kUnitBytes;  // one packed box
    static constexpr int stage_bytes = (GATED ? 2 : 1) * a_bytes + b_bytes;
    static constexpr int pstage_bytes = (GATED ? 2 : 1) * p_bytes;
    static constexpr int off_p = stages * stage_bytes;
    static constexpr int off_bar = off_p + pstages * pstage_bytes;
    static constexpr int total = off_bar + 512 + 1024;
};

// One scale group (32 weights) of one row of a packed Q4_K box -> 32 f16 in the swizzled A tile.
// Integer -> float without the conversion unit: byte q under the exponent of 2^23 is the float 2^23 + q, and
// subtracting 2^23 is exact, so d*sc*q - dmin*m comes out with the codec's own two roundings.
__device__ __forceinline__ float nib_to_float(uint32_t masked, int byte) {
    uint32_t r;
    switch (byte) {
    case 0: asm("prmt.b32 %0, %1, %2, 0x7540;" : "=r"(r) : "r"(masked), "r"(0x4B000000u)); break;
    case 1: asm("prmt.b32 %0, %1, %2, 0x7541;" : "=r"(r) : "r"(masked), "r"(0x4B000000u)); break;
    case 2: asm("prmt.b32 %0, %1, %2, 0x7542;" : "=r"(r) : "r"(masked), "r"(0x4B000000u)); break;
    default: asm("prmt.b32 %0, %1, %2, 0x7543;" : "=r"(r) : "r"(masked), "r"(0x4B000000u)); break;
    }
    return __fadd_rn(__uint_as_float(r), -8388608.0f);
}

// The f16 operand value of a Q4_K weight, as both GEMM paths form it: fma(d*sc, q, -(dmin*m)) in f32 (one rounding,
// slightly closer to the exact value than the codec's multiply-then-subtract), rounded once to f16.
__device__ __forceinline__ uint32_t q4k_pair_f16(float dsc, float ndm, float qa, float qb) { return h2_as_u32(__floats2half2_rn(fmaf(dsc, qa, ndm), fmaf(dsc, qb, ndm))); }

// The 8 (d*sc, -dmin*m) pairs of one super-block header (src/weight/codec/ggml.rs:471-473).
__device__ __forceinline__ void q4k_group_scales(const uint4 &hdr, int g, float &dsc, float &ndm) {
    const __half2 dd = u32_as_h2(hdr.x);
    const float d = __low2float(dd), dmin = __high2float(dd);
    uint32_t sc, mn;
    if (g < 4) {
        sc = (hdr.y >> (8 * g)) & 63u;
        mn = (hdr.z >> (8 * g)) & 63u;
    } else {
        const int j = 8 * (g - 4);
        sc = ((hdr.w >> j) & 0x0Fu) | (((hdr.y >> (j + 6)) & 3u) << 4);
        mn = ((hdr.w >> (j + 4)) & 0x0Fu) | (((hdr.z >> (j + 6)) & 3u) << 4);
    }
    dsc = __fmul_rn(d, (float)sc);
    ndm = -__fmul_rn(dmin, (float)mn);
}

// One scale group (32 weights: low or high nibbles of the pair's 32 quant bytes) of one row of a packed Q4_K box ->
// 32 f16 in the swizzled A tile (the four 16-byte chunks 4 half .. 4 half + 3 of row `row`).
__device__ __forceinline__ void dequant_group_to_sw128(const uint8_t *unit, int pair, int half, float dsc, float ndm, uint8_t *a_tile, int row) {
    const uint4 q0 = *reinterpret_cast<const uint4 *>(unit + 16 + pair * 32), q1 = *reinterpret_cast<const uint4 *>(unit + 16 + pair * 32 + 16);
    const uint32_t qw[8] = {q0.x, q0.y, q0.z, q0.w, q1.x, q1.y, q1.z, q1.w};
    const int shift = half * 4;
    uint8_t *row_base = a_tile + (row >> 3) * 1024 + (row & 7) * 128;
#pragma unroll
    for (int c = 0; c < 4; ++c) {  // chunk = 8 consecutive K = 2 packed words
        uint32_t h[4];
#pragma unroll
        for (int j = 0; j < 2; ++j) {
            const uint32_t m = (qw[2 * c + j] >> shift) & 0x0F0F0F0Fu;
            h[2 * j] = q4k_pair_f16(dsc, ndm, nib_to_float(m, 0), nib_to_float(m, 1));
            h[2 * j + 1] = q4k_pair_f16(dsc, ndm, nib_to_float(m, 2), nib_to_float(m, 3));
        }
        const int chunk = half * 4 + c;
        *reinterpret_cast<uint4 *>(row_base + ((chunk ^ (row & 7)) << 4)) = make_uint4(h[0], h[1], h[2], h[3]);
    }
}

template <bool GATED>
__global__ void __launch_bounds__(kFusedThreads, 1) gemm_q4k_fused_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_w2, const __grid_constant__ CUtensorMap map_x, const GemmParams p) {
    using S = FusedSmem<GATED>;
    constexpr int STAGES = S::stages;
    constexpr int PST = S::pstages;
    constexpr int ACC = S::acc_bufs;
    constexpr uint32_t ACC_COLS = GATED ? 512 : 256;
    constexpr uint32_t TMEM_COLS = 512;
    extern __shared__ uint8_t smem_raw[];
    uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint64_t *a_full = reinterpret_cast<uint64_t *>(smem + S::off_bar);
    uint64_t *b_full = a_full + STAGES;
    uint64_t *empty = b_full + STAGES;
    uint64_t *p_full = empty + STAGES;
    uint64_t *p_empty = p_full + PST;
    uint64_t *acc_full = p_empty + PST;
    uint64_t *acc_empty = acc_full + 2;
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(acc_empty + 2);
    __shared__ int s_abort;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int n_sb = p.k / kUnitWeights;  // Q4_K: K is a multiple of 256
    const int n_row_tiles = (p.n_out + kBM - 1) / kBM, n_tok_tiles = (p.m + kBN - 1) / kBN;
    const bool grouped = p.items != nullptr;
    const int total_tiles = grouped ? (p.n_items_dev ? *p.n_items_dev : p.n_items) : n_row_tiles * n_tok_tiles;
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
            mbar_init(&a_full[s], kFusedDqWarps);
            mbar_init(&b_full[s], 1);
            mbar_init(&empty[s], 1);
        }
        for (int s = 0; s < PST; ++s) {
            mbar_init(&p_full[s], 1);
            mbar_init(&p_empty[s], kFusedDqWarps);
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
        // ------------------------------------------------ TMA producer: activation k-blocks
        if (lane == 0) {
            long long kg = 0;
            bool ok = true;
            for (int tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x) {
                int row0, tok0, tok_end, z;
                tile_coords(tile, row0, tok0, tok_end, z);
                for (int kb = 0; kb < n_sb * (kUnitWeights / kBK) && ok; ++kb, ++kg) {
                    const int s = (int)(kg % STAGES);
                    if (kg >= STAGES) ok = wait_flag(&empty[s], (uint32_t)((kg / STAGES) - 1) & 1, &s_abort, p.status, kStatusMmaTimeout);
                    if (!ok) break;
                    uint8_t *st = smem + (size_t)s * S::stage_bytes;
                    mbar_expect_tx(&b_full[s], S::b_bytes);
                    tma_load_2d(st + (GATED ? 2 : 1) * S::a_bytes, &map_x, &b_full[s], kb * kBK, tok0);
                }
            }
        }
    } else if (warp == kFusedPackedWarp) {
        // ------------------------------------------------ TMA producer: packed boxes, a ring of their own, so that a box
        // is requested as soon as the dequantisers free its slot, not when the activation ring gets round to it
        if (lane == 0) {
            long long pq = 0;
            bool ok = true;
            for (int tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x) {
                int row0, tok0, tok_end, z;
                tile_coords(tile, row0, tok0, tok_end, z);
                const CUtensorMap *mw = grouped ? &p.w_maps[z] : &map_w;
                const CUtensorMap *mw2 = grouped ? (GATED ? &p.w2_maps[z] : mw) : &map_w2;
                for (int sb = 0; sb < n_sb && ok; ++sb, ++pq) {
                    const int ps = (int)(pq % PST);
                    if (pq >= PST) ok = wait_flag_backoff(&p_empty[ps], (uint32_t)((pq / PST) - 1) & 1, &s_abort, p.status, kStatusMmaTimeout, 100);
                    if (!ok) break;
                    uint8_t *pst = smem + S::off_p + (size_t)ps * S::pstage_bytes;
                    mbar_expect_tx(&p_full[ps], S::pstage_bytes);
                    tma_load_2d(pst, mw, &p_full[ps], sb * (kQ4kUnitBytes / 4), row0);
                    if (GATED) tma_load_2d(pst + S::p_bytes, mw2, &p_full[ps], sb * (kQ4kUnitBytes / 4), row0);
                }
            }
        }
    } else if (warp == 1) {
        // ------------------------------------------------ MMA issuer
        if (lane == 0) {
            long long kg = 0;
            int iter = 0;
            bool ok = true;
            const int k_blocks = n_sb * (kUnitWeights / kBK);
            for (int tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x, ++iter) {
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
                    ok = wait_flag(&b_full[s], (uint32_t)(kg / STAGES) & 1, &s_abort, p.status, kStatusTmaTimeout);
                    if (ok) ok = wait_flag(&a_full[s], (uint32_t)(kg / STAGES) & 1, &s_abort, p.status, kStatusMmaTimeout);
                    if (!ok) break;
                    tc_fence_after();
                    const uint32_t st = smem_u32(smem + (size_t)s * S::stage_bytes);
                    const uint64_t da = make_sw128_desc(st);
                    const uint64_t da2 = make_sw128_desc(st + S::a_bytes);
                    const uint64_t db = make_sw128_desc(st + (GATED ? 2 : 1) * S::a_bytes);
#pragma unroll
                    for (int k = 0; k < kBK / 16; ++k) {
                        const uint32_t acc = (kb > 0 || k > 0) ? 1u : 0u;
                        umma_f16_ss(acc_addr, da + 2 * k, db + 2 * k, idesc, acc);
                        if (GATED) umma_f16_ss(acc_addr + kBN, da2 + 2 * k, db + 2 * k, idesc, acc);
                    }
                    tc_commit(&empty[s]);
                }
                tc_commit(&acc_full[b]);
            }
        }
    } else if (warp < 6) {
        // ------------------------------------------------ epilogue: warp q of 4 owns TMEM lanes 32q..32q+31
        const int q = warp & 3;
        int iter = 0;
        for (int tile = blockIdx.x; tile < total_tiles; tile += gridDim.x, ++iter) {
            int row0, tok0, tok_end, z;
            tile_coords(tile, row0, tok0, tok_end, z);
            const int b = iter % ACC;
            const int row = row0 + q * 32 + lane;
            const bool ok = wait_flag_backoff(&acc_full[b], (uint32_t)(iter / ACC) & 1, &s_abort, p.status, kStatusMmaTimeout, 400);
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
            if (lane == 0) mbar_arrive(&acc_empty[b]);
        }
    } else {
        // ------------------------------------------------ dequantisers: thread = (row, half of the k-block)
        const int t = threadIdx.x - 6 * 32;
        const int row = t & (kBM - 1), half = t >> 7;
        long long kg = 0, pq = 0;
        bool ok = true;
        for (int tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x) {
            for (int sb = 0; sb < n_sb && ok; ++sb, ++pq) {
                const int ps = (int)(pq % PST);
                ok = wait_flag_backoff(&p_full[ps], (uint32_t)(pq / PST) & 1, &s_abort, p.status, kStatusTmaTimeout, 60);
                if (!ok) break;
                const uint8_t *u0 = smem + S::off_p + (size_t)ps * S::pstage_bytes + (size_t)row * kQ4kUnitBytes;
                const uint8_t *u1 = u0 + S::p_bytes;
                // the four groups this thread will meet in this super-block: 2 kb + half
                float dsc0[4], ndm0[4], dsc1[4], ndm1[4];
                {
                    const uint4 hdr = *reinterpret_cast<const uint4 *>(u0);
#pragma unroll
                    for (int kb = 0; kb < 4; ++kb) q4k_group_scales(hdr, 2 * kb + half, dsc0[kb], ndm0[kb]);
                }
                if (GATED) {
                    const uint4 hdr = *reinterpret_cast<const uint4 *>(u1);
#pragma unroll
                    for (int kb = 0; kb < 4; ++kb) q4k_group_scales(hdr, 2 * kb + half, dsc1[kb], ndm1[kb]);
                }
#pragma unroll
                for (int kb = 0; kb < kUnitWeights / kBK; ++kb, ++kg) {
                    if (!ok) break;
                    const int s = (int)(kg % STAGES);
                    if (kg >= STAGES) ok = wait_flag_backoff(&empty[s], (uint32_t)((kg / STAGES) - 1) & 1, &s_abort, p.status, kStatusMmaTimeout, 60);
                    if (!ok) break;
                    uint8_t *st = smem + (size_t)s * S::stage_bytes;
                    dequant_group_to_sw128(u0, kb, half, dsc0[kb], ndm0[kb], st, row);
                    if (GATED) dequant_group_to_sw128(u1, kb, half, dsc1[kb], ndm1[kb], st + S::a_bytes, row);
                    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");  // generic-proxy stores -> visible to the tensor core
                    __syncwarp();
                    if (lane == 0) mbar_arrive(&a_full[s]);
                }
                __syncwarp();
                if (lane == 0 && ok) mbar_arrive(&p_empty[ps]);
            }
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
    // The fused kernel saves the operand pass (one read of the packed weight, one write and one read of its f16 form),
    // which dominates for few tokens; with many tokens the pass is amortised and the plain kernel, whose shared-memory
    // traffic per k-block is lower (no operand stores by threads), runs the tensor core at a higher duty.
    const bool fused = !ctx->disable_fused_gemm && (ctx->force_fused_gemm || m <= 1024) && w->type == ZQ_Q4_K && (!gated || w_up->type == ZQ_Q4_K) && k % kUnitWeights == 0;
    if (fused) {
        // Q4_K: dequantisation fused into the kernel; the workspace only holds the f16 copy of the activations
        const size_t xb = (m * k * 2 + 255) & ~size_t(255);
        const __half *xin = reinterpret_cast<const __half *>(x);
        if (x_dtype != ZQ_F16) {
            int rc = ensure_workspace(ctx, xb, err);
            if (rc) return rc;
            rc = launch_to_f16(ctx, x, x_dtype, reinterpret_cast<__half *>(ctx->workspace), m * k, err);
            if (rc) return rc;
            xin = reinterpret_cast<const __half *>(ctx->workspace);
        }
        CUtensorMap map_x;
        int rc = make_f16_map(xin, m, k, kBN, &map_x, err);
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
        p.n_items_dev = nullptr;
        const size_t total_tiles = ((n + kBM - 1) / kBM) * ((m + kBN - 1) / kBN);
        dim3 grid((unsigned)(total_tiles < (size_t)ctx->sm_count ? total_tiles : (size_t)ctx->sm_count));
        static bool configured[2][64] = {};
        if (gated) {
            if (!configured[1][ctx->device & 63]) {
                ZQ_CUDA_CHECK(cudaFuncSetAttribute(gemm_q4k_fused_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, FusedSmem<true>::total), err);
                configured[1][ctx->device & 63] = true;
            }
            gemm_q4k_fused_kernel<true><<<grid, kFusedThreads, FusedSmem<true>::total, ctx->stream>>>(w->qmv_map, w_up->qmv_map, map_x, p);
        } else {
            if (!configured[0][ctx->device & 63]) {
                ZQ_CUDA_CHECK(cudaFuncSetAttribute(gemm_q4k_fused_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, FusedSmem<false>::total), err);
                configured[0][ctx->device & 63] = true;
            }
            gemm_q4k_fused_kernel<false><<<grid, kFusedThreads, FusedSmem<false>::total, ctx->stream>>>(w->qmv_map, w->qmv_map, map_x, p);
        }
        ctx->launches++;
        ZQ_CUDA_CHECK(cudaGetLastError(), err);
        return ZQ_OK;
    }
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
    p.n_items_dev = nullptr;
    p.w_maps = p.w2_maps = nullptr;
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
    p.n_items_dev = nullptr;
    p.w_maps = p.w2_maps = nullptr;
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
    p.n_items_dev = nullptr;
    p.w_maps = p.w2_maps = nullptr;
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

// Grouped fused form (MoE prefill, Q4_K experts): no f16 copy of the weights at all.  `w_maps` / `w2_maps`: device
// tables of the experts' packed-weight tensor maps (one unit x 128 rows boxes), indexed by the work items' z.
int launch_gemm_fused_grouped(zq_ctx *ctx, const CUtensorMap *w_maps, const CUtensorMap *w2_maps, size_t rows, size_t k, const __half *x, size_t x_rows, const int4 *items, int n_items, const int *n_items_dev, void *y, int y_dtype,
                              zq_error *err) {
    if (n_items <= 0) return ZQ_OK;
    if (k % kUnitWeights) return set_error(err, ZQ_ERR_SHAPE, "fused Q4_K GEMM needs columns aligned to 256, got %zu", k);
    const bool gated = w2_maps != nullptr;
    CUtensorMap map_x;
    int rc = make_f16_map(x, x_rows, k, kBN, &map_x, err);
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
    p.n_items_dev = n_items_dev;
    p.w_maps = w_maps;
    p.w2_maps = w2_maps;
    dim3 grid((unsigned)(n_items < ctx->sm_count ? n_items : ctx->sm_count));
    static bool configured[2][64] = {};
    if (gated) {
        if (!configured[1][ctx->device & 63]) {
            ZQ_CUDA_CHECK(cudaFuncSetAttribute(gemm_q4k_fused_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, FusedSmem<true>::total), err);
            configured[1][ctx->device & 63] = true;
        }
        gemm_q4k_fused_kernel<true><<<grid, kFusedThreads, FusedSmem<true>::total, ctx->stream>>>(map_x, map_x, map_x, p);
    } else {
        if (!configured[0][ctx->device & 63]) {
            ZQ_CUDA_CHECK(cudaFuncSetAttribute(gemm_q4k_fused_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, FusedSmem<false>::total), err);
            configured[0][ctx->device & 63] = true;
        }
        gemm_q4k_fused_kernel<false><<<grid, kFusedThreads, FusedSmem<false>::total, ctx->stream>>>(map_x, map_x, map_x, p);
    }
    ctx->launches++;
    ZQ_CUDA_CHECK(cudaGetLastError(), err);
    return ZQ_OK;
}

}  // namespace zq
