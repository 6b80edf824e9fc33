// Decode GEMV, resident-activation variant: the whole activation block (all K columns of up to 8 rows, split into
// f16 limbs and permuted into MMA B-fragment order) is staged in shared memory once per CTA, so the steady-state
// loop has no CTA-wide barrier at all:
//   * every warp waits for a ring stage's `full` mbarrier, turns its 16 rows x 1 unit into MMAs
//     (zq_gemv_frag.cuh) against the resident activations, and releases the stage (mbarrier `empty`, one
//     arrival per warp);
//   * the refill of a released stage (wait for `empty`, re-arm `full`, issue the TMA box of the item STAGES-1
//     ahead) is done by one lane of a different warp each iteration, so no warp is the permanent straggler.
// Only the end of a 128-row tile (every `chunks` items) synchronises the warps.
// Work partition, split-tile fix-up, arithmetic and operator contract are those of zq_gemv.cu; this variant is
// chosen whenever the staged activations fit beside at least two ring stages.
#include "zq_gemv_frag.cuh"

namespace zq {

constexpr int kConsumerThreads = 512;
constexpr int kResidentThreads = kConsumerThreads;

struct ResidentArgs {
    int stages;       // 2..4 ring stages
    int units_total;  // resident units per row (ceil(K / 256))
    int off_x, off_sx, off_red, off_lut, off_bar;  // byte offsets from the 128-byte aligned base (weights at 0)
};

__device__ __forceinline__ void consumer_bar() { __syncthreads(); }

// Bounded wait that never strands the CTA: when the barrier does not complete (or another warp already gave up)
// the abort flag is raised and every later wait in the CTA falls through, so all warps still walk the same
// control flow, reach every barrier and return; the host sees the status word.
__device__ __forceinline__ void wait_or_abort(uint64_t *bar, uint32_t parity, volatile int *abort_flag, uint32_t *status) {
    for (uint32_t i = 0; i < (1u << 22); ++i) {
        if (mbar_try_wait(bar, parity)) return;
        if (*abort_flag) return;
    }
    *abort_flag = 1;
    atomicMax(status, (uint32_t)kStatusTmaTimeout);
}

template <uint32_t TYPE, int NT, bool GATED>
__global__ void __launch_bounds__(kResidentThreads, 1) gemv_resident_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b, const GemvParams p, const ResidentArgs ra) {
    using S = GemvSmem<TYPE, NT>;
    constexpr int UB = Fmt<TYPE>::unit_bytes;
    extern __shared__ uint8_t smem_raw[];
    uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 127) & ~uintptr_t(127));
    uint8_t *ws = smem;
    uint2 *xs = reinterpret_cast<uint2 *>(smem + ra.off_x);
    __half *sxs = reinterpret_cast<__half *>(smem + ra.off_sx);
    float *red = reinterpret_cast<float *>(smem + ra.off_red);
    uint32_t *lut = reinterpret_cast<uint32_t *>(smem + ra.off_lut);
    uint64_t *full = reinterpret_cast<uint64_t *>(smem + ra.off_bar);
    uint64_t *empty = full + 4;
    __shared__ int s_flag;
    __shared__ int s_abort;

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int STAGES = ra.stages;
    const int rows_per_tile = GATED ? kTileRows / 2 : kTileRows;
    const long long T = (long long)p.tiles * p.chunks;
    const long long G = gridDim.x;
    const long long begin = (long long)blockIdx.x * T / G;
    const long long end = (long long)(blockIdx.x + 1) * T / G;
    const int n_items = (int)(end - begin);

    if (tid == 0) {
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(&full[s], 1);
            mbar_init(&empty[s], kConsumerThreads / 32);
        }
        fence_mbar_init();
        tma_prefetch_desc(&map_a);
        if (GATED) tma_prefetch_desc(&map_b);
        s_abort = 0;
    }
    __syncthreads();

    auto issue_tma = [&](int local, int stage) {
        const long long item = begin + local;
        const int tile = (int)(item / p.chunks), chunk = (int)(item % p.chunks);
        uint8_t *dst = ws + (size_t)stage * S::stage_w;
        mbar_expect_tx(&full[stage], S::stage_w);
        if (GATED) {
            tma_load_2d(dst, &map_a, &full[stage], chunk * p.chunk_words, tile * rows_per_tile);
            tma_load_2d(dst + S::stage_w / 2, &map_b, &full[stage], chunk * p.chunk_words, tile * rows_per_tile);
        } else {
            tma_load_2d(dst, &map_a, &full[stage], chunk * p.chunk_words, tile * rows_per_tile);
        }
    };
    if (tid == 0) {
        const int pre = n_items < STAGES - 1 ? n_items : STAGES - 1;
        for (int s = 0; s < pre; ++s) issue_tma(s, s);
    }

    // ---------------------------------------------------- consumers
    const int g = lane >> 2, t = lane & 3;
    const int rs = warp & 7, ul = warp >> 3;
    const int cols2 = 2 * p.m;  // staged MMA columns: (hi, lo) limb per activation row

    if constexpr (Fmt<TYPE>::lut) {
        for (int i = tid; i < 256 * 32; i += kConsumerThreads) {
            int b = i >> 5;
            lut[i] = h2_as_u32(__halves2half2(__int2half_rn(kIq4nlValues[b & 15]), __int2half_rn(kIq4nlValues[b >> 4])));
        }
    }
    {
        // stage every activation quad: B-fragment slot (unit, step, column, t); Q4_K also gets per-group sums
        const int quads_per_row = ra.units_total * (kUnitWeights / 4);
        const int total_quads = p.m * quads_per_row;
        for (int q = tid; q < total_quads; q += kConsumerThreads) {  // whole warps stay together (multiples of 64)
            const int m = q / quads_per_row, quad = q - m * quads_per_row;
            const int k0 = quad * 4;
            float v[4] = {0.f, 0.f, 0.f, 0.f};
            if (k0 < p.cols) {
                const size_t o = (size_t)m * p.cols + k0;
                if (p.x_dtype == ZQ_F32) {
                    const float4 f = *reinterpret_cast<const float4 *>(reinterpret_cast<const float *>(p.x) + o);
                    v[0] = f.x; v[1] = f.y; v[2] = f.z; v[3] = f.w;
                } else {
#pragma unroll
                    for (int j = 0; j < 4; ++j) v[j] = load_as_f32(p.x, p.x_dtype, o + j);
                }
            }
            __half hi[4], lo[4];
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                hi[j] = __float2half_rn(v[j]);
                lo[j] = __float2half_rn(v[j] - __half2float(hi[j]));
            }
            const int unit = k0 >> 8, i = k0 & 255;
            const int col = 2 * m;
            if constexpr (TYPE == ZQ_IQ4_NL) {
                const int blk = i >> 5, nib = (i >> 4) & 1, tt = (i >> 2) & 3;
                const int step0 = 8 * (blk >> 2) + 2 * (blk & 3);
#pragma unroll
                for (int by = 0; by < 4; ++by) {
                    const int step = step0 + (by >> 1);
                    __half *dh = reinterpret_cast<__half *>(&xs[((size_t)(unit * 16 + step) * cols2 + col) * 4 + tt]);
                    __half *dl = reinterpret_cast<__half *>(&xs[((size_t)(unit * 16 + step) * cols2 + col + 1) * 4 + tt]);
                    dh[(by & 1) * 2 + nib] = hi[by];
                    dl[(by & 1) * 2 + nib] = lo[by];
                }
            } else {
                int step, tt;
                quad_slot<TYPE>(i, step, tt);
                uint2 *base = &xs[(size_t)(unit * 16 + step) * cols2 * 4];
                base[col * 4 + tt] = make_uint2(h2_as_u32(__halves2half2(hi[0], hi[2])), h2_as_u32(__halves2half2(hi[1], hi[3])));
                base[(col + 1) * 4 + tt] = make_uint2(h2_as_u32(__halves2half2(lo[0], lo[2])), h2_as_u32(__halves2half2(lo[1], lo[3])));
            }
            if constexpr (TYPE == ZQ_Q4_K) {
                float sum = (v[0] + v[1]) + (v[2] + v[3]);
                sum += __shfl_xor_sync(0xffffffffu, sum, 1);
                sum += __shfl_xor_sync(0xffffffffu, sum, 2);
                sum += __shfl_xor_sync(0xffffffffu, sum, 4);
                if ((lane & 7) == 0) {
                    const int G8 = i >> 5;
                    const __half shi = __float2half_rn(sum);
                    const __half slo = __float2half_rn(sum - __half2float(shi));
                    // fragment of the min-term MMA: lane (column, t') holds (sum of group 2t', sum of group 2t'+1)
                    sxs[(((size_t)unit * cols2 + col) * 4 + (G8 >> 1)) * 2 + (G8 & 1)] = shi;
                    sxs[(((size_t)unit * cols2 + col + 1) * 4 + (G8 >> 1)) * 2 + (G8 & 1)] = slo;
                }
            }
        }
    }
    consumer_bar();

    float yacc[NT][2];
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) yacc[nt][0] = yacc[nt][1] = 0.f;
    const int r0 = 16 * rs + frag_row(g);

    for (int it = 0; it < n_items; ++it) {
        const int stage = it % STAGES;
        const long long item = begin + it;
        const int tile = (int)(item / p.chunks), chunk = (int)(item % p.chunks);
        {
            // refill: the stage consumed one iteration ago takes the item STAGES-1 ahead
            const int nxt = it + STAGES - 1;
            if (nxt < n_items && warp == (it & 15) && lane == 0) {
                const int nstage = nxt % STAGES;
                if (it >= 1) wait_or_abort(&empty[nstage], ((it - 1) / STAGES) & 1, &s_abort, p.status);
                if (!*(volatile int *)&s_abort) issue_tma(nxt, nstage);  // never start a copy nobody will wait for
            }
            __syncwarp();
        }
        wait_or_abort(&full[stage], (it / STAGES) & 1, &s_abort, p.status);

        const int unit = chunk * kChunkUnits + ul;
        if (unit < ra.units_total) {
            const uint8_t *w0 = ws + (size_t)stage * S::stage_w + (size_t)r0 * S::pitch + ul * UB;
            const uint8_t *w1 = w0 + 8 * S::pitch;
            const uint2 *xu = xs + (size_t)unit * 16 * cols2 * 4 + t;
            const uint32_t *sxu = reinterpret_cast<const uint32_t *>(sxs) + (size_t)unit * cols2 * 4 + t;
            auto getb = [&](int nt, int step) -> uint2 {
                const int col = 8 * nt + g;
                return col < cols2 ? xu[(step * cols2 + col) * 4] : make_uint2(0u, 0u);
            };
            auto getsx = [&](int nt) -> uint32_t {
                const int col = 8 * nt + g;
                return col < cols2 ? sxu[col * 4] : 0u;
            };
            consume_unit<TYPE, NT>(w0, w1, t, lut + lane, getb, getsx, yacc);
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(&empty[stage]);

        const bool tile_ends = (it == n_items - 1) || ((int)((item + 1) / p.chunks) != tile);
        if (tile_ends) {
#pragma unroll
            for (int nt = 0; nt < NT; ++nt) {
                red[(ul * kTileRows + r0) * (NT * 4) + nt * 4 + t] = yacc[nt][0];
                red[(ul * kTileRows + r0 + 8) * (NT * 4) + nt * 4 + t] = yacc[nt][1];
                yacc[nt][0] = yacc[nt][1] = 0.f;
            }
            consumer_bar();
            const long long tile_first = (long long)tile * p.chunks, tile_last = tile_first + p.chunks - 1;
            const bool whole = begin <= tile_first && tile_last < end;
            const int c_first = (int)(((tile_first + 1) * G - 1) / T), c_last = (int)(((tile_last + 1) * G - 1) / T);
            bool finish = whole;
            if (!whole) {
                const int which = (tile == (int)(begin / p.chunks)) ? 0 : 1;
                float *slot = p.partials + ((size_t)blockIdx.x * 2 + which) * kSlotFloats;
                for (int i = tid; i < kTileRows * p.m; i += kConsumerThreads) {
                    int row = i & (kTileRows - 1), tok = i >> 7;
                    slot[tok * kTileRows + row] = red[row * (NT * 4) + tok] + red[(kTileRows + row) * (NT * 4) + tok];
                }
                __threadfence();
                consumer_bar();
                if (tid == 0) {
                    unsigned old = atomicAdd(&p.counters[tile], 1u);
                    s_flag = (old == (unsigned)(c_last - c_first)) ? 1 : 0;
                }
                consumer_bar();
                finish = s_flag != 0;
                if (finish) __threadfence();
            }
            if (finish) {
                float vals[(kTileRows * kMaxGemvRows + kConsumerThreads - 1) / kConsumerThreads];
                int cnt = 0;
                for (int i = tid; i < kTileRows * p.m; i += kConsumerThreads, ++cnt) {
                    int row = i & (kTileRows - 1), tok = i >> 7;
                    float v;
                    if (whole) {
                        v = red[row * (NT * 4) + tok] + red[(kTileRows + row) * (NT * 4) + tok];
                    } else {
                        v = 0.f;
                        for (int c = c_first; c <= c_last; ++c) {
                            long long cb = (long long)c * T / G;
                            int which = (tile == (int)(cb / p.chunks)) ? 0 : 1;
                            v += __ldcg(p.partials + ((size_t)c * 2 + which) * kSlotFloats + tok * kTileRows + row);
                        }
                    }
                    vals[cnt] = v;
                }
                consumer_bar();
                cnt = 0;
                for (int i = tid; i < kTileRows * p.m; i += kConsumerThreads, ++cnt) red[i] = vals[cnt];
                consumer_bar();
                const int out_rows = rows_per_tile;
                for (int i = tid; i < out_rows * p.m; i += kConsumerThreads) {
                    int row = i % out_rows, tok = i / out_rows;
                    int n = tile * out_rows + row;
                    if (n >= p.n_out) continue;
                    float v;
                    if (GATED) {
                        float gate = red[tok * kTileRows + row], up = red[tok * kTileRows + out_rows + row];
                        v = (gate / (1.0f + expf(-gate))) * up;
                    } else {
                        v = red[tok * kTileRows + row];
                    }
                    size_t o = (size_t)tok * p.n_out + n;
                    if (p.residual) v += load_as_f32(p.residual, p.y_dtype, o);
                    store_from_f32(p.y, p.y_dtype, o, v);
                }
                if (!whole && tid == 0) p.counters[tile] = 0;
            }
            consumer_bar();  // red is free again before the next tile's sums land in it
        }
    }
}

// Shared-memory plan of the resident variant; returns false when fewer than two ring stages would fit.
template <uint32_t TYPE, int NT>
static bool plan_resident(int m, int units_total, ResidentArgs &ra, int &total_bytes) {
    using S = GemvSmem<TYPE, NT>;
    const int max_smem = 232448 - 256;  // 227 KB opt-in limit minus static shared and alignment slack
    const int x_bytes = units_total * 16 * (2 * m) * 4 * 8;
    const int sx_bytes = TYPE == ZQ_Q4_K ? units_total * (2 * m) * 4 * 4 : 0;
    const int fixed = x_bytes + sx_bytes + S::red_bytes + S::lut_bytes + 64 + 128;
    int stages = (max_smem - fixed) / S::stage_w;
    if (stages > 4) stages = 4;
    if (stages < 2) return false;
    ra.stages = stages;
    ra.units_total = units_total;
    ra.off_x = stages * S::stage_w;
    ra.off_sx = ra.off_x + x_bytes;
    ra.off_red = ra.off_sx + sx_bytes;
    ra.off_lut = ra.off_red + S::red_bytes;
    ra.off_bar = ra.off_lut + S::lut_bytes;
    total_bytes = ra.off_bar + 64 + 128;
    return true;
}

template <uint32_t TYPE, int NT, bool GATED>
static int launch_resident_one(zq_ctx *ctx, const zq_weight *w, const zq_weight *w_up, const GemvParams &p, int grid, bool &taken, zq_error *err) {
    ResidentArgs ra;
    int total = 0;
    taken = plan_resident<TYPE, NT>(p.m, (int)w->units_per_row, ra, total);
    if (!taken) return ZQ_OK;
    auto kernel = gemv_resident_kernel<TYPE, NT, GATED>;
    static bool configured[64] = {};
    if (!configured[ctx->device & 63]) {
        ZQ_CUDA_CHECK(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 232448 - 256), err);
        configured[ctx->device & 63] = true;
    }
    const CUtensorMap &ma = GATED ? w->gemv_map_half : w->gemv_map;
    const CUtensorMap &mb = GATED ? w_up->gemv_map_half : w->gemv_map;
    kernel<<<grid, kResidentThreads, total, ctx->stream>>>(ma, mb, p, ra);
    ctx->launches++;
    ZQ_CUDA_CHECK(cudaGetLastError(), err);
    return ZQ_OK;
}

template <uint32_t TYPE>
static int launch_resident_type(zq_ctx *ctx, const zq_weight *w, const zq_weight *w_up, const GemvParams &p, int grid, bool &taken, zq_error *err) {
    const bool gated = w_up != nullptr;
    if (p.m <= 4) return gated ? launch_resident_one<TYPE, 1, true>(ctx, w, w_up, p, grid, taken, err) : launch_resident_one<TYPE, 1, false>(ctx, w, w_up, p, grid, taken, err);
    return gated ? launch_resident_one<TYPE, 2, true>(ctx, w, w_up, p, grid, taken, err) : launch_resident_one<TYPE, 2, false>(ctx, w, w_up, p, grid, taken, err);
}

// Tries the resident-activation kernel for one group of up to 8 rows; `taken` tells whether it was launched.
int launch_gemv_resident(zq_ctx *ctx, const zq_weight *w, const zq_weight *w_up, const GemvParams &p, int grid, bool &taken, zq_error *err) {
    taken = false;
    switch (w->type) {
    case ZQ_Q4_K: return launch_resident_type<ZQ_Q4_K>(ctx, w, w_up, p, grid, taken, err);
    case ZQ_Q4_0: return launch_resident_type<ZQ_Q4_0>(ctx, w, w_up, p, grid, taken, err);
    case ZQ_IQ4_NL: return launch_resident_type<ZQ_IQ4_NL>(ctx, w, w_up, p, grid, taken, err);
    case ZQ_Q8_0: return launch_resident_type<ZQ_Q8_0>(ctx, w, w_up, p, grid, taken, err);
    default: return ZQ_OK;
    }
}

}  // namespace zq
