// Decode GEMV for GGUF block-quantised weights (1..8 activation rows per launch), sm_100a.
//
// Replaces, behind the same operator surface, the reference's decode kernels gguf_kq_gemv_f16,
// gguf_block32_gemv_f16, linear_q4_0_gemv_f16 and gated_linear_q4_k_silu_f16
// (src/kernel/cuda/linear.rs:139-204, 267-294, 799-852); the arithmetic contract is the CPU path
// ggml_quant::matvec / matvec_residual / gated_silu_matvec (src/kernel/cpu/ggml_quant.rs:189-277).
//
// Design (HBM-bound: 0.5625 B per weight, so only ~3 issue slots per weight exist at full bandwidth):
//   * Work item = (tile of 128 weight rows) x (chunk of 2 units = 512 input columns).  All items are laid out
//     in one line (tile-major) and cut into gridDim.x equal contiguous ranges, one persistent CTA per SM, so every
//     SM streams the same number of bytes whatever the matrix shape.  A tile whose chunks are split between CTAs
//     is finished by whichever CTA arrives last, which adds the partial tiles in CTA order (deterministic).
//   * Packed rows are staged by TMA (cp.async.bulk.tensor.2d, one box of 128 rows x 288/544 bytes per item)
//     through a ring of shared-memory stages with mbarrier completion; rows past the matrix and units past the
//     row are zero-filled by the TMA unit, so edge tiles need no special code.
//   * The dot products run on the tensor cores as m16n8k16 f16 MMAs with f32 accumulation.  The A operand is
//     built in registers from the packed quants with exact integer-in-f16 tricks: Q4_K feeds scale*quant
//     (<= 63*15, exact in f16) and handles the min term with one extra MMA against per-group activation sums;
//     Q4_0 feeds nibble-8, Q8_0 the int8 value and IQ4_NL the codebook entry, each scaled per block in f32.
//     The B operand is the activation row split into two f16 limbs (hi + lo, ~22 bits) so that the result
//     carries f32-level accuracy; limbs of up to 4 rows fill the 8 MMA columns.
//   * Which four weights a thread feeds into MMA step s is free (a dot product does not care about the order
//     of k), so it is chosen to make every shared-memory read a conflict-free 16-byte load of bytes the thread
//     needs anyway; the activation staging applies the same permutation.
#include "zq_gemv_frag.cuh"

namespace zq {

template <uint32_t TYPE, int NT, bool GATED>
__global__ void __launch_bounds__(kGemvThreads, 1) gemv_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b, const GemvParams p) {
    using S = GemvSmem<TYPE, NT>;
    constexpr int STAGES = S::stages;
    constexpr int UB = Fmt<TYPE>::unit_bytes;
    constexpr int XQ = NT == 1 ? 1 : 4;  // activation quads per thread per item: up to 16 rows x 128 quads over 512 threads
    extern __shared__ uint8_t smem_raw[];
    uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 127) & ~uintptr_t(127));
    uint8_t *ws = smem + S::off_w;
    uint2 *xs = reinterpret_cast<uint2 *>(smem + S::off_x);
    uint2 *sxs = reinterpret_cast<uint2 *>(smem + S::off_sx);
    float *red = reinterpret_cast<float *>(smem + S::off_red);
    uint32_t *lut = reinterpret_cast<uint32_t *>(smem + S::off_lut);
    uint64_t *full = reinterpret_cast<uint64_t *>(smem + S::off_bar);
    __shared__ int s_flag;

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int g = lane >> 2, t = lane & 3;
    const int rs = warp & 7, ul = warp >> 3;
    const int rows_per_tile = GATED ? kTileRows / 2 : kTileRows;

    // ---- this CTA's contiguous range of work items
    const long long T = (long long)p.tiles * p.chunks;
    const long long G = gridDim.x;
    const long long begin = (long long)blockIdx.x * T / G;
    const long long end = (long long)(blockIdx.x + 1) * T / G;
    const int n_items = (int)(end - begin);

    if (tid == 0) {
        for (int s = 0; s < STAGES; ++s) mbar_init(&full[s], 1);
        fence_mbar_init();
        tma_prefetch_desc(&map_a);
        if (GATED) tma_prefetch_desc(&map_b);
    }
    // zero the activation staging once: lanes of unused MMA columns must read zeros
    for (int i = tid; i < (STAGES * (S::stage_x + S::stage_sx)) / 4; i += kGemvThreads) reinterpret_cast<uint32_t *>(smem + S::off_x)[i] = 0;
    if constexpr (Fmt<TYPE>::lut) {
        // codebook pairs, one private copy per lane (entry*32 + lane) so that the random lookups never conflict
        for (int i = tid; i < 256 * 32; i += kGemvThreads) {
            int b = i >> 5;
            __half2 v = __halves2half2(__int2half_rn(kIq4nlValues[b & 15]), __int2half_rn(kIq4nlValues[b >> 4]));
            lut[i] = h2_as_u32(v);
        }
    }
    __syncthreads();

    auto issue_tma = [&](int local, int stage) {
        long long item = begin + local;
        int tile = (int)(item / p.chunks), chunk = (int)(item % p.chunks);
        uint8_t *dst = ws + (size_t)stage * S::stage_w;
        mbar_expect_tx(&full[stage], S::stage_w);
        if (GATED) {
            tma_load_2d(dst, &map_a, &full[stage], chunk * p.chunk_words, tile * rows_per_tile);
            tma_load_2d(dst + S::stage_w / 2, &map_b, &full[stage], chunk * p.chunk_words, tile * rows_per_tile);
        } else {
            tma_load_2d(dst, &map_a, &full[stage], chunk * p.chunk_words, tile * rows_per_tile);
        }
    };

    // activation quads of one item: register staging (load early, convert after the MMAs)
    float4 xr[XQ];
    auto load_x = [&](int local) {
        long long item = begin + local;
        int chunk = (int)(item % p.chunks);
#pragma unroll
        for (int r = 0; r < XQ; ++r) {
            int q = tid + r * kGemvThreads;
            int m = q >> 7, quad = q & 127;
            int k0 = chunk * kChunkCols + quad * 4;
            float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
            if (m < p.m && k0 < p.cols) {
                size_t o = (size_t)m * p.cols + k0;
                if (p.x_dtype == ZQ_F32) v = *reinterpret_cast<const float4 *>(reinterpret_cast<const float *>(p.x) + o);
                else v = make_float4(load_as_f32(p.x, p.x_dtype, o), load_as_f32(p.x, p.x_dtype, o + 1), load_as_f32(p.x, p.x_dtype, o + 2), load_as_f32(p.x, p.x_dtype, o + 3));
            }
            xr[r] = v;
        }
    };
    auto store_x = [&](int stage) {
        uint2 *xst = xs + (size_t)stage * (S::stage_x / 8);
        uint2 *sxst = sxs + (size_t)stage * (S::stage_sx / 8);
#pragma unroll
        for (int r = 0; r < XQ; ++r) {
            int q = tid + r * kGemvThreads;
            int m = q >> 7, quad = q & 127;
            if (m >= p.m) continue;  // whole warps: 128 quads per row
            float v[4] = {xr[r].x, xr[r].y, xr[r].z, xr[r].w};
            __half hi[4], lo[4];
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                hi[j] = __float2half_rn(v[j]);
                lo[j] = __float2half_rn(v[j] - __half2float(hi[j]));
            }
            int unit = quad >> 6, i = (quad & 63) * 4;
            // two limbs: row m owns columns 2(m%4), 2(m%4)+1 of tile m/4; one limb: column m%8 of tile m/8
            const bool two = p.limbs == 2;
            int nt = two ? (m >> 2) : (m >> 3), col = two ? 2 * (m & 3) : (m & 7);
            if constexpr (TYPE == ZQ_IQ4_NL) {
                // element i+by of the quad pairs with the other nibble of the same byte: MMA step 8h+2bb+(by>>1),
                // register by&1, half index = nibble (see the A-fragment construction below)
                int blk = i >> 5, nib = (i >> 4) & 1, tt = (i >> 2) & 3;
                int step0 = 8 * (blk >> 2) + 2 * (blk & 3);
#pragma unroll
                for (int by = 0; by < 4; ++by) {
                    int step = step0 + (by >> 1);
                    __half *dst_hi = reinterpret_cast<__half *>(&xst[((nt * kChunkUnits + unit) * 16 + step) * 32 + (col * 4 + tt)]);
                    __half *dst_lo = reinterpret_cast<__half *>(&xst[((nt * kChunkUnits + unit) * 16 + step) * 32 + ((col + 1) * 4 + tt)]);
                    dst_hi[(by & 1) * 2 + nib] = hi[by];
                    if (two) dst_lo[(by & 1) * 2 + nib] = lo[by];
                }
            } else {
                int step, tt;
                quad_slot<TYPE>(i, step, tt);
                uint2 *base = &xst[((nt * kChunkUnits + unit) * 16 + step) * 32];
                base[col * 4 + tt] = make_uint2(h2_as_u32(__halves2half2(hi[0], hi[2])), h2_as_u32(__halves2half2(hi[1], hi[3])));
                if (two) base[(col + 1) * 4 + tt] = make_uint2(h2_as_u32(__halves2half2(lo[0], lo[2])), h2_as_u32(__halves2half2(lo[1], lo[3])));
            }
            if constexpr (TYPE == ZQ_Q4_K) {
                // per-group activation sums (32 columns = 8 consecutive quads = 8 consecutive lanes)
                // sums of the values the MMAs really see (the staged limbs), so that the scale and min terms cancel
                // exactly as in the reference's per-element form
                float sum = 0.f;
#pragma unroll
                for (int j = 0; j < 4; ++j) sum += __half2float(hi[j]) + (two ? __half2float(lo[j]) : 0.f);
                sum += __shfl_xor_sync(0xffffffffu, sum, 1);
                sum += __shfl_xor_sync(0xffffffffu, sum, 2);
                sum += __shfl_xor_sync(0xffffffffu, sum, 4);
                if ((lane & 7) == 0) {
                    int G8 = (i >> 5);  // group inside the unit
                    __half shi = __float2half_rn(sum);
                    __half slo = __float2half_rn(sum - __half2float(shi));
                    // lane (column, t') of the min-term fragment: .x = hi limbs of sums 2t', 2t'+1, .y = their lo limbs;
                    // the sums ride in the row's first column (its second, lo-limb column keeps zeros)
                    __half *dst = reinterpret_cast<__half *>(&sxst[(nt * kChunkUnits + unit) * 32 + col * 4 + (G8 >> 1)]);
                    dst[G8 & 1] = shi;
                    dst[2 + (G8 & 1)] = slo;
                }
            }
        }
    };

    // ---- prologue: fill the ring
    const int pre = n_items < STAGES - 1 ? n_items : STAGES - 1;
    for (int s = 0; s < pre; ++s) {
        if (tid == 0) issue_tma(s, s);
        load_x(s);
        store_x(s);
    }
    __syncthreads();

    float yacc[NT][2][2];
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) yacc[nt][0][0] = yacc[nt][0][1] = yacc[nt][1][0] = yacc[nt][1][1] = 0.f;

    const int r0 = 16 * rs + frag_row(g);  // tile row of fragment row g; the g+8 row is r0 + 8
    bool failed = false;

    for (int it = 0; it < n_items; ++it) {
        const int stage = it % STAGES;
        const int nxt = it + STAGES - 1;
        const int nstage = nxt % STAGES;
        if (nxt < n_items) {
            if (tid == 0) issue_tma(nxt, nstage);
            load_x(nxt);
        }
        if (!mbar_wait_bounded(&full[stage], (it / STAGES) & 1)) {
            failed = true;
        }
        if (__syncthreads_or(failed ? 1 : 0)) {  // a TMA that never landed: record and leave together
            if (tid == 0) atomicMax(p.status, (uint32_t)kStatusTmaTimeout);
            return;
        }

        // ---------------- MMAs of this item: this warp's 16 rows x one unit
        {
            const uint8_t *w0 = ws + (size_t)stage * S::stage_w + (size_t)r0 * S::pitch + ul * UB;
            const uint8_t *w1 = w0 + 8 * S::pitch;
            const uint2 *xb = xs + (size_t)stage * (S::stage_x / 8) + (size_t)ul * 16 * 32 + lane;
            const uint2 *sxb = sxs + (size_t)stage * (S::stage_sx / 8) + (size_t)ul * 32 + lane;
            auto getb = [&](int nt, int step) -> uint2 { return xb[((size_t)nt * kChunkUnits * 16 + step) * 32]; };
            auto getsx = [&](int nt) -> uint2 { return sxb[(size_t)nt * kChunkUnits * 32]; };
            consume_unit<TYPE, NT>(w0, w1, t, lut + lane, getb, getsx, yacc);
        }

        if (nxt < n_items) store_x(nstage);

        // ---------------- end of a tile (or of this CTA's range): reduce, then store or hand over
        const long long item = begin + it;
        const int tile = (int)(item / p.chunks);
        const bool tile_ends = (it == n_items - 1) || ((int)((item + 1) / p.chunks) != tile);
        if (tile_ends) {
            // the two warps that share a row sub-tile add up through shared memory: red[ul][row][token]
#pragma unroll
            for (int nt = 0; nt < NT; ++nt) {
                float *ra_ = red + (ul * kTileRows + r0) * (NT * 8), *rb_ = red + (ul * kTileRows + r0 + 8) * (NT * 8);
                if (p.limbs == 2) {  // the thread's two columns are the limbs of activation row 4nt + t
                    ra_[nt * 4 + t] = yacc[nt][0][0] + yacc[nt][0][1];
                    rb_[nt * 4 + t] = yacc[nt][1][0] + yacc[nt][1][1];
                } else {             // two activation rows: 8nt + 2t and 8nt + 2t + 1
                    ra_[nt * 8 + 2 * t] = yacc[nt][0][0];
                    ra_[nt * 8 + 2 * t + 1] = yacc[nt][0][1];
                    rb_[nt * 8 + 2 * t] = yacc[nt][1][0];
                    rb_[nt * 8 + 2 * t + 1] = yacc[nt][1][1];
                }
                yacc[nt][0][0] = yacc[nt][0][1] = yacc[nt][1][0] = yacc[nt][1][1] = 0.f;
            }
            __syncthreads();
            const long long tile_first = (long long)tile * p.chunks, tile_last = tile_first + p.chunks - 1;
            const bool whole = begin <= tile_first && tile_last < end;
            const int c_first = (int)(((tile_first + 1) * G - 1) / T), c_last = (int)(((tile_last + 1) * G - 1) / T);
            bool finish = whole;
            if (!whole) {
                const int which = (tile == (int)(begin / p.chunks)) ? 0 : 1;
                float *slot = p.partials + ((size_t)blockIdx.x * 2 + which) * kSlotFloats;
                for (int i = tid; i < kTileRows * p.m; i += kGemvThreads) {
                    int row = i & (kTileRows - 1), tok = i >> 7;
                    slot[tok * kTileRows + row] = red[row * (NT * 8) + tok] + red[(kTileRows + row) * (NT * 8) + tok];
                }
                __syncthreads();
                if (tid == 0) {
                    __threadfence();  // the barrier orders the CTA's stores before this thread; one fence publishes them
                    unsigned old = atomicAdd(&p.counters[tile], 1u);
                    s_flag = (old == (unsigned)(c_last - c_first)) ? 1 : 0;
                }
                __syncthreads();
                finish = s_flag != 0;
                if (finish) __threadfence();
            }
            if (finish) {
                // final value of every (row, token) of the tile, staged in red[0] as fin[token][row]
                float vals[(kTileRows * kMaxGemvRows + kGemvThreads - 1) / kGemvThreads];
                int cnt = 0;
                for (int i = tid; i < kTileRows * p.m; i += kGemvThreads, ++cnt) {
                    int row = i & (kTileRows - 1), tok = i >> 7;
                    float v;
                    if (whole) {
                        v = red[row * (NT * 8) + tok] + red[(kTileRows + row) * (NT * 8) + tok];
                    } else {
                        v = 0.f;
                        for (int c = c_first; c <= c_last; ++c) {  // fixed order: deterministic
                            long long cb = (long long)c * T / G;
                            int which = (tile == (int)(cb / p.chunks)) ? 0 : 1;
                            v += __ldcg(p.partials + ((size_t)c * 2 + which) * kSlotFloats + tok * kTileRows + row);
                        }
                    }
                    vals[cnt] = v;
                }
                __syncthreads();
                cnt = 0;
                for (int i = tid; i < kTileRows * p.m; i += kGemvThreads, ++cnt) red[i] = vals[cnt];  // fin[tok*128 + row]
                __syncthreads();
                const int out_rows = rows_per_tile;
                for (int i = tid; i < out_rows * p.m; i += kGemvThreads) {
                    int row = i % out_rows, tok = i / out_rows;
                    int n = tile * out_rows + row;
                    if (n >= p.n_out) continue;
                    float v;
                    if (GATED) {
                        float gate = red[tok * kTileRows + row], up = red[tok * kTileRows + out_rows + row];
                        v = (gate / (1.0f + expf(-gate))) * up;  // src/kernel/cpu/ggml_quant.rs:274
                    } else {
                        v = red[tok * kTileRows + row];
                    }
                    size_t o = (size_t)tok * p.n_out + n;
                    if (p.residual) v += load_as_f32(p.residual, p.y_dtype, o);
                    store_from_f32(p.y, p.y_dtype, o, v);
                }
                if (!whole && tid == 0) p.counters[tile] = 0;  // leave the counter ready for the next launch
            }
        }
        __syncthreads();
    }
}

// ---------------------------------------------------------------------------------------------------------------
// Host launcher.
// ---------------------------------------------------------------------------------------------------------------

template <uint32_t TYPE, int NT, bool GATED>
static int launch_one(zq_ctx *ctx, const zq_weight *w, const zq_weight *w_up, const GemvParams &p, int grid, zq_error *err) {
    using S = GemvSmem<TYPE, NT>;
    static bool configured[64] = {};
    auto kernel = gemv_kernel<TYPE, NT, GATED>;
    if (!configured[ctx->device & 63]) {
        ZQ_CUDA_CHECK(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, S::total), err);
        configured[ctx->device & 63] = true;
    }
    const CUtensorMap &ma = GATED ? w->gemv_map_half : w->gemv_map;
    const CUtensorMap &mb = GATED ? w_up->gemv_map_half : w->gemv_map;
    kernel<<<grid, kGemvThreads, S::total, ctx->stream>>>(ma, mb, p);
    ctx->launches++;
    ZQ_CUDA_CHECK(cudaGetLastError(), err);
    return ZQ_OK;
}

template <uint32_t TYPE>
static int launch_type(zq_ctx *ctx, const zq_weight *w, const zq_weight *w_up, const GemvParams &p, int grid, zq_error *err) {
    const bool gated = w_up != nullptr;
    if (p.m * p.limbs <= 8) return gated ? launch_one<TYPE, 1, true>(ctx, w, w_up, p, grid, err) : launch_one<TYPE, 1, false>(ctx, w, w_up, p, grid, err);
    return gated ? launch_one<TYPE, 2, true>(ctx, w, w_up, p, grid, err) : launch_one<TYPE, 2, false>(ctx, w, w_up, p, grid, err);
}

// y[m, n] = x[m, k] W^T (+ residual), or silu(x gate^T) * (x up^T) when w_up is given.  m may exceed 8: the rows
// are then processed in groups of 8 (each group streams the weights once).
int launch_gemv(zq_ctx *ctx, const zq_weight *w, const zq_weight *w_up, const void *x, int x_dtype, size_t m, void *y, int y_dtype, const void *residual, zq_error *err) {
    const FormatInfo f = format_info(w->type);
    const bool gated = w_up != nullptr;
    const int rows_per_tile = gated ? kTileRows / 2 : kTileRows;
    GemvParams p;
    p.partials = ctx->gemv_partials;
    p.counters = ctx->gemv_counters;
    p.status = ctx->status_dev;
    p.x_dtype = x_dtype;
    p.y_dtype = y_dtype;
    p.cols = (int)w->cols;
    p.n_out = (int)w->rows;
    p.tiles = (int)((w->rows + rows_per_tile - 1) / rows_per_tile);
    p.chunks = (int)((w->units_per_row + kChunkUnits - 1) / kChunkUnits);
    p.chunk_words = kChunkUnits * f.unit_bytes / 4;
    if ((size_t)p.tiles > ctx->gemv_counters_n) return set_error(err, ZQ_ERR_UNSUPPORTED, "GEMV needs %d tile counters, context has %zu", p.tiles, ctx->gemv_counters_n);
    long long total = (long long)p.tiles * p.chunks;
    int grid = (int)(total < ctx->sm_count ? total : ctx->sm_count);
    // When the tiles alone nearly fill the machine, give every CTA one whole tile: a few SMs idle, but no tile is
    // split, so the partial-tile hand-over (several microseconds of fences and atomics per launch) disappears.
    if (p.tiles <= ctx->sm_count && p.tiles * 100 >= ctx->sm_count * 85) grid = p.tiles;
    if (grid <= 0) return ZQ_OK;
    // up to 8 rows per pass as two f16 limbs each (f32-level accuracy); 9..16 rows go in one pass as single f16
    // limbs (the reference's CUDA path takes f16 activations throughout, src/kernel/cuda/linear.rs:1440)
    const size_t per_pass = m > 8 ? 16 : 8;
    for (size_t m0 = 0; m0 < m; m0 += per_pass) {
        size_t mm = m - m0 < per_pass ? m - m0 : per_pass;
        p.m = (int)mm;
        p.limbs = mm > 8 ? 1 : 2;
        p.x = reinterpret_cast<const uint8_t *>(x) + m0 * w->cols * dtype_size(x_dtype);
        p.y = reinterpret_cast<uint8_t *>(y) + m0 * w->rows * dtype_size(y_dtype);
        p.residual = residual ? reinterpret_cast<const uint8_t *>(residual) + m0 * w->rows * dtype_size(y_dtype) : nullptr;
        int rc;
        if (ctx->enable_tcgen05_gemv && !ctx->force_staged_gemv && !gated && w->type == ZQ_Q4_K) {
            bool taken = false;
            rc = launch_qmv(ctx, w, p, taken, err);
            if (rc) return rc;
            if (taken) continue;
        }
        if (!ctx->force_staged_gemv && !ctx->force_f16_gemv) {
            bool taken = false;
            rc = launch_gemv_i8(ctx, w, w_up, p, taken, err);
            if (rc) return rc;
            if (taken) continue;
        }
        if (!ctx->force_staged_gemv) {
            bool taken = false;
            rc = launch_gemv_resident(ctx, w, w_up, p, grid, taken, err);
            if (rc) return rc;
            if (taken) continue;
        }
        switch (w->type) {
        case ZQ_Q4_K: rc = launch_type<ZQ_Q4_K>(ctx, w, w_up, p, grid, err); break;
        case ZQ_Q4_0: rc = launch_type<ZQ_Q4_0>(ctx, w, w_up, p, grid, err); break;
        case ZQ_IQ4_NL: rc = launch_type<ZQ_IQ4_NL>(ctx, w, w_up, p, grid, err); break;
        case ZQ_Q8_0: rc = launch_type<ZQ_Q8_0>(ctx, w, w_up, p, grid, err); break;
        case ZQ_Q5_K:  // only the integer-MMA kernel unpacks these; where that one did not fit: the operand pass + GEMM
        case ZQ_Q6_K:
            rc = launch_gemm(ctx, w, w_up, p.x, x_dtype, mm, p.y, y_dtype, p.residual, err);
            break;
        default: return set_error(err, ZQ_ERR_UNSUPPORTED, "GEMV: unsupported GGUF type %u", w->type);
        }
        if (rc) return rc;
    }
    return ZQ_OK;
}


// ---------------------------------------------------------------------------------------------------------------
// Allocation-free decode entry (zq_linear_noalloc).
//
// Some hosts may not allocate device memory at the point where they run a layer: code running inside a
// stream-ordered region that forbids allocator calls, a real-time loop with a fixed memory budget, or a plugin
// whose host application owns the allocator.  For them the split-tile fix-up scratch of the decode GEMV (partial
// tiles + per-tile arrival counters) lives in the two file-scope device arrays below instead of in memory the
// context allocated.  Every GPU that loads the library holds these ~2.6 MB until the process exits.
//
// In host code the array names are host-side stand-ins, not device addresses; the device addresses are looked
// up once per device with cudaGetSymbolAddress (with that device current) and passed to the kernel.
// ---------------------------------------------------------------------------------------------------------------
constexpr int kStaticMaxSms = 160;       // partial-tile slots: two per persistent CTA
constexpr int kStaticMaxTiles = 4096;    // arrival counters: one per 128-row tile (weights up to 524 288 rows)
static __device__ __align__(256) float g_static_partials[(size_t)kStaticMaxSms * 2 * kSlotFloats];
static __device__ __align__(256) uint32_t g_static_counters[kStaticMaxTiles];

struct StaticScratch {
    float *partials = nullptr;
    uint32_t *counters = nullptr;
    bool ready = false;
};
static StaticScratch g_static_scratch[64];
static std::mutex g_static_mutex;

// First call on a device resolves the device addresses of the static arrays (no allocation involved).
static int static_scratch_for(zq_ctx *ctx, StaticScratch **out, zq_error *err) {
    if (ctx->device < 0 || ctx->device >= 64) return set_error(err, ZQ_ERR_ARG, "zq_linear_noalloc: device index %d is outside the supported 0..63", ctx->device);
    std::lock_guard<std::mutex> lock(g_static_mutex);
    StaticScratch &s = g_static_scratch[ctx->device];
    if (!s.ready) {
        int current = -1;
        ZQ_CUDA_CHECK(cudaGetDevice(&current), err);
        if (current != ctx->device) ZQ_CUDA_CHECK(cudaSetDevice(ctx->device), err);
        void *pp = nullptr, *pc = nullptr;
        cudaError_t e1 = cudaGetSymbolAddress(&pp, g_static_partials);
        cudaError_t e2 = cudaGetSymbolAddress(&pc, g_static_counters);
        if (current != ctx->device && current >= 0) cudaSetDevice(current);
        if (e1 != cudaSuccess) return set_error(err, ZQ_ERR_CUDA, "cudaGetSymbolAddress(partials) failed: %s", cudaGetErrorString(e1));
        if (e2 != cudaSuccess) return set_error(err, ZQ_ERR_CUDA, "cudaGetSymbolAddress(counters) failed: %s", cudaGetErrorString(e2));
        s.partials = reinterpret_cast<float *>(pp);
        s.counters = reinterpret_cast<uint32_t *>(pc);
        s.ready = true;
    }
    *out = &s;
    return ZQ_OK;
}

// y[m, n] = x[m, k] W^T for 1..8 activation rows, one launch, scratch in the static device arrays.
int launch_gemv_noalloc(zq_ctx *ctx, const zq_weight *w, const void *x, int x_dtype, size_t m, void *y, int y_dtype, zq_error *err) {
    if (m == 0 || m > 8) return set_error(err, ZQ_ERR_SHAPE, "zq_linear_noalloc handles 1..8 activation rows per call, got %zu", m);
    if (ctx->sm_count > kStaticMaxSms) return set_error(err, ZQ_ERR_UNSUPPORTED, "zq_linear_noalloc: device has %d SMs, the static scratch is sized for %d", ctx->sm_count, kStaticMaxSms);
    const FormatInfo f = format_info(w->type);
    GemvParams p;
    p.x = x;
    p.y = y;
    p.residual = nullptr;
    p.status = ctx->status_dev;
    p.x_dtype = x_dtype;
    p.y_dtype = y_dtype;
    p.m = (int)m;
    p.limbs = 2;
    p.cols = (int)w->cols;
    p.n_out = (int)w->rows;
    p.tiles = (int)((w->rows + kTileRows - 1) / kTileRows);
    p.chunks = (int)((w->units_per_row + kChunkUnits - 1) / kChunkUnits);
    p.chunk_words = kChunkUnits * f.unit_bytes / 4;
    if (p.tiles > kStaticMaxTiles) return set_error(err, ZQ_ERR_UNSUPPORTED, "zq_linear_noalloc: weight has %zu rows; the static scratch covers at most %d rows", w->rows, kStaticMaxTiles * kTileRows);
    StaticScratch *scratch = nullptr;
    int rc = static_scratch_for(ctx, &scratch, err);
    if (rc) return rc;
    p.partials = scratch->partials;
    p.counters = scratch->counters;
    // the array keeps whatever the previous call (or an interrupted one) left: arrival counters must start at zero
    ZQ_CUDA_CHECK(cudaMemsetAsync(scratch->counters, 0, (size_t)p.tiles * sizeof(uint32_t), ctx->stream), err);
    long long total = (long long)p.tiles * p.chunks;
    int grid = (int)(total < ctx->sm_count ? total : ctx->sm_count);
    if (p.tiles <= ctx->sm_count && p.tiles * 100 >= ctx->sm_count * 85) grid = p.tiles;  // launch_gemv's whole-tile rule: same grid, same summation order
    if (grid <= 0) return ZQ_OK;
    // Kernel choice and grid follow launch_gemv, so 1..4 rows (and every row count of a type or option that
    // zq_linear also runs on the f16-limb kernels) agree with zq_linear bit for bit.  The one difference: zq_linear
    // runs 5..8 rows on the integer-MMA kernel, which reads activation records from a workspace the context may
    // have to grow; here those rows take the f16-limb kernel, and agree with zq_linear within the integer kernel's
    // activation rounding (16-bit integers per 256-column slice) instead.
    bool taken = false;
    if (ctx->enable_tcgen05_gemv && !ctx->force_staged_gemv) {
        rc = launch_qmv(ctx, w, p, taken, err);
        if (rc || taken) return rc;
    }
    if (!ctx->force_staged_gemv && !ctx->force_f16_gemv && m <= 4) {
        rc = launch_gemv_i8(ctx, w, nullptr, p, taken, err);
        if (rc || taken) return rc;
    }
    if (!ctx->force_staged_gemv) {
        rc = launch_gemv_resident(ctx, w, nullptr, p, grid, taken, err);
        if (rc || taken) return rc;
    }
    switch (w->type) {
    case ZQ_Q4_K: return launch_type<ZQ_Q4_K>(ctx, w, nullptr, p, grid, err);
    case ZQ_Q4_0: return launch_type<ZQ_Q4_0>(ctx, w, nullptr, p, grid, err);
    case ZQ_IQ4_NL: return launch_type<ZQ_IQ4_NL>(ctx, w, nullptr, p, grid, err);
    case ZQ_Q8_0: return launch_type<ZQ_Q8_0>(ctx, w, nullptr, p, grid, err);
    default: return set_error(err, ZQ_ERR_UNSUPPORTED, "zq_linear_noalloc: unsupported GGUF type %u", w->type);
    }
}

}  // namespace zq
