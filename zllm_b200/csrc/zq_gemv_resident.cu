// Decode GEMV, resident-activation variant: the whole activation block (all K columns of up to 8 rows, split into
// f16 limbs and permuted into MMA B-fragment order) is staged in shared memory once per CTA, so the steady-state
// loop has no CTA-wide barrier at all:
//   * every warp waits for a ring stage's `full` mbarrier, turns its 16 rows x 1 unit into MMAs
//     (zq_gemv_frag.cuh) against the resident activations, and releases the stage (mbarrier `empty`, one
//     arrival per warp);
//   * the refill of a released stage (wait for `empty`, re-arm `full`, issue the TMA box of the item STAGES-1
//     ahead) is done by one lane of a different warp each iteration, so no warp is the permanent straggler.
// Work partition: one CTA per (128-row tile, K slice).  When the tiles alone do not fill the machine, each tile is
// split over a thread-block cluster of 2, 4 or 8 CTAs (one K slice each); the slices' partial sums meet in
// distributed shared memory: every CTA leaves its partial tile in its own shared memory, the cluster synchronises,
// and rank 0 adds the partials in rank order (deterministic) and stores the tile.  No global scratch, no atomics.
// Arithmetic and operator contract are those of zq_gemv.cu; this variant is chosen whenever the staged activations
// of a K slice fit beside at least two ring stages.
#include "zq_gemv_frag.cuh"

namespace zq {

constexpr int kConsumerThreads = 512;
constexpr int kResidentThreads = kConsumerThreads;

struct ResidentArgs {
    int stages;       // 2..5 ring stages
    int split;        // CTAs per tile (cluster size): 1, 2, 4 or 8
    int slice_units;  // units of activations staged per CTA (upper bound over the K slices)
    int units_total;  // resident units per row (ceil(K / 256))
    int off_x, off_sx, off_red, off_lut, off_bar;  // byte offsets from the 128-byte aligned base (weights at 0)
};

__device__ __forceinline__ void consumer_bar() { __syncthreads(); }
__device__ __forceinline__ void cluster_sync_all() {
    asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// f32 at the same shared-memory offset in the CTA of rank `rank` of this cluster
__device__ __forceinline__ float ld_cluster_f32(const float *local, uint32_t rank) {
    uint32_t remote;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(smem_u32(local)), "r"(rank));
    float v;
    asm volatile("ld.shared::cluster.f32 %0, [%1];" : "=f"(v) : "r"(remote) : "memory");
    return v;
}

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
    uint2 *sxs = reinterpret_cast<uint2 *>(smem + ra.off_sx);
    float *red = reinterpret_cast<float *>(smem + ra.off_red);
    uint32_t *lut = reinterpret_cast<uint32_t *>(smem + ra.off_lut);
    uint64_t *full = reinterpret_cast<uint64_t *>(smem + ra.off_bar);
    uint64_t *empty = full + 8;
    __shared__ int s_flag;
    __shared__ int s_abort;

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int STAGES = ra.stages;
    const int rows_per_tile = GATED ? kTileRows / 2 : kTileRows;
    // this CTA: tile blockIdx.x / split, K slice (cluster rank) blockIdx.x % split
    const int split = ra.split;
    const int my_tile = blockIdx.x / split, my_rank = blockIdx.x % split;
    const int chunk_begin = (int)((long long)my_rank * p.chunks / split), chunk_end = (int)((long long)(my_rank + 1) * p.chunks / split);
    const long long begin = (long long)my_tile * p.chunks + chunk_begin;
    const int n_items = chunk_end - chunk_begin;
    const int unit0 = chunk_begin * kChunkUnits;  // first unit of the staged activation slice

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
    const int limbs = p.limbs;
    const int cols2 = limbs * p.m;  // staged MMA columns: (hi, lo) limb per activation row, or one column per row

    if constexpr (Fmt<TYPE>::lut) {
        for (int i = tid; i < 256 * 32; i += kConsumerThreads) {
            int b = i >> 5;
            lut[i] = h2_as_u32(__halves2half2(__int2half_rn(kIq4nlValues[b & 15]), __int2half_rn(kIq4nlValues[b >> 4])));
        }
    }
    if constexpr (TYPE == ZQ_Q4_K) {
        for (int i = tid; i < (ra.off_red - ra.off_sx) / 8; i += kConsumerThreads) sxs[i] = make_uint2(0u, 0u);
        __syncthreads();
    }
    pdl_launch_dependents();
    pdl_wait_prior_grid();  // activations (and, later, outputs) belong to the previous kernel until it completes
    {
        // stage every activation quad: B-fragment slot (unit, step, column, t); Q4_K also gets per-group sums
        int slice_units = chunk_end * kChunkUnits;
        if (slice_units > ra.units_total) slice_units = ra.units_total;
        slice_units -= unit0;
        if (slice_units < 0) slice_units = 0;
        const int quads_per_row = slice_units * (kUnitWeights / 4);
        const int total_quads = p.m * quads_per_row;
        for (int q = tid; q < total_quads; q += kConsumerThreads) {  // whole warps stay together (multiples of 64)
            const int m = q / quads_per_row, quad = q - m * quads_per_row;
            const int k0 = quad * 4;  // column inside the slice
            float v[4] = {0.f, 0.f, 0.f, 0.f};
            if (unit0 * kUnitWeights + k0 < p.cols) {
                const size_t o = (size_t)m * p.cols + (size_t)unit0 * kUnitWeights + k0;
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
            const int col = limbs * m;
            const bool two = limbs == 2;
            if constexpr (TYPE == ZQ_IQ4_NL) {
                const int blk = i >> 5, nib = (i >> 4) & 1, tt = (i >> 2) & 3;
                const int step0 = 8 * (blk >> 2) + 2 * (blk & 3);
#pragma unroll
                for (int by = 0; by < 4; ++by) {
                    const int step = step0 + (by >> 1);
                    __half *dh = reinterpret_cast<__half *>(&xs[((size_t)(unit * 16 + step) * cols2 + col) * 4 + tt]);
                    __half *dl = reinterpret_cast<__half *>(&xs[((size_t)(unit * 16 + step) * cols2 + col + (two ? 1 : 0)) * 4 + tt]);
                    dh[(by & 1) * 2 + nib] = hi[by];
                    if (two) dl[(by & 1) * 2 + nib] = lo[by];
                }
            } else {
                int step, tt;
                quad_slot<TYPE>(i, step, tt);
                uint2 *base = &xs[(size_t)(unit * 16 + step) * cols2 * 4];
                base[col * 4 + tt] = make_uint2(h2_as_u32(__halves2half2(hi[0], hi[2])), h2_as_u32(__halves2half2(hi[1], hi[3])));
                if (two) base[(col + 1) * 4 + tt] = make_uint2(h2_as_u32(__halves2half2(lo[0], lo[2])), h2_as_u32(__halves2half2(lo[1], lo[3])));
            }
            if constexpr (TYPE == ZQ_Q4_K) {
                // sums of the values the MMAs really see (the staged limbs), so that the scale and min terms cancel
                // exactly as in the reference's per-element form
                float sum = 0.f;
#pragma unroll
                for (int j = 0; j < 4; ++j) sum += __half2float(hi[j]) + (two ? __half2float(lo[j]) : 0.f);
                sum += __shfl_xor_sync(0xffffffffu, sum, 1);
                sum += __shfl_xor_sync(0xffffffffu, sum, 2);
                sum += __shfl_xor_sync(0xffffffffu, sum, 4);
                if ((lane & 7) == 0) {
                    const int G8 = i >> 5;
                    const __half shi = __float2half_rn(sum);
                    const __half slo = __float2half_rn(sum - __half2float(shi));
                    // fragment of the min-term MMA: lane (column, t') holds .x = hi limbs of sums 2t', 2t'+1 and .y = their
                    // lo limbs; the sums ride in the row's first column (a lo-limb column keeps zeros)
                    __half *dst = reinterpret_cast<__half *>(&sxs[((size_t)unit * cols2 + col) * 4 + (G8 >> 1)]);
                    dst[G8 & 1] = shi;
                    dst[2 + (G8 & 1)] = slo;
                }
            }
        }
    }
    consumer_bar();

    float yacc[NT][2][2];
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) yacc[nt][0][0] = yacc[nt][0][1] = yacc[nt][1][0] = yacc[nt][1][1] = 0.f;
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

        const int unit = chunk * kChunkUnits + ul - unit0;  // unit inside the staged slice
        if (unit + unit0 < ra.units_total) {
            const uint8_t *w0 = ws + (size_t)stage * S::stage_w + (size_t)r0 * S::pitch + ul * UB;
            const uint8_t *w1 = w0 + 8 * S::pitch;
            const uint2 *xu = xs + (size_t)unit * 16 * cols2 * 4 + t;
            const uint2 *sxu = sxs + (size_t)unit * cols2 * 4 + t;
            auto getb = [&](int nt, int step) -> uint2 {
                const int col = 8 * nt + g;
                return col < cols2 ? xu[(step * cols2 + col) * 4] : make_uint2(0u, 0u);
            };
            auto getsx = [&](int nt) -> uint2 {
                const int col = 8 * nt + g;
                return col < cols2 ? sxu[col * 4] : make_uint2(0u, 0u);
            };
            consume_unit<TYPE, NT>(w0, w1, t, lut + lane, getb, getsx, yacc);
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(&empty[stage]);

    }

    // ---------------------------------------------------- end of the K slice: combine and store
    {
        const int tile = my_tile;
        // the two warps that share a row sub-tile add up through shared memory: red[ul][row][token]
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) {
            float *ra_ = red + (ul * kTileRows + r0) * (NT * 8), *rb_ = red + (ul * kTileRows + r0 + 8) * (NT * 8);
            if (limbs == 2) {  // the thread's two columns are the limbs of activation row 4nt + t
                ra_[nt * 4 + t] = yacc[nt][0][0] + yacc[nt][0][1];
                rb_[nt * 4 + t] = yacc[nt][1][0] + yacc[nt][1][1];
            } else {           // two activation rows: 8nt + 2t and 8nt + 2t + 1
                ra_[nt * 8 + 2 * t] = yacc[nt][0][0];
                ra_[nt * 8 + 2 * t + 1] = yacc[nt][0][1];
                rb_[nt * 8 + 2 * t] = yacc[nt][1][0];
                rb_[nt * 8 + 2 * t + 1] = yacc[nt][1][1];
            }
        }
        consumer_bar();
        float vals[(kTileRows * kMaxGemvRows + kConsumerThreads - 1) / kConsumerThreads];
        int cnt = 0;
        for (int i = tid; i < kTileRows * p.m; i += kConsumerThreads, ++cnt) {
            int row = i & (kTileRows - 1), tok = i >> 7;
            vals[cnt] = red[row * (NT * 8) + tok] + red[(kTileRows + row) * (NT * 8) + tok];
        }
        consumer_bar();
        cnt = 0;
        for (int i = tid; i < kTileRows * p.m; i += kConsumerThreads, ++cnt) red[i] = vals[cnt];  // part[tok * 128 + row]
        if (split > 1) {
            cluster_sync_all();  // every slice's partial tile is in its CTA's shared memory
            if (my_rank == 0) {
                cnt = 0;
                for (int i = tid; i < kTileRows * p.m; i += kConsumerThreads, ++cnt) {
                    float v = vals[cnt];
                    for (int r = 1; r < split; ++r) v += ld_cluster_f32(&red[i], (uint32_t)r);  // rank order: deterministic
                    vals[cnt] = v;
                }
                consumer_bar();
                cnt = 0;
                for (int i = tid; i < kTileRows * p.m; i += kConsumerThreads, ++cnt) red[i] = vals[cnt];
            }
        }
        consumer_bar();
        if (my_rank == 0) {
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
        }
        if (split > 1) cluster_sync_all();  // nobody leaves while rank 0 may still read its shared memory
    }
}

// Plan of the resident variant: CTAs per tile (cluster size) and shared-memory layout; returns false when fewer
// than two ring stages would fit beside the staged activation slice.
template <uint32_t TYPE, int NT>
static bool plan_resident(int cols2, int units_total, int tiles, int chunks, int sm_count, ResidentArgs &ra, int &total_bytes) {
    using S = GemvSmem<TYPE, NT>;
    int split = 1;
    while (split < 8 && tiles * split * 2 <= sm_count && split * 2 <= chunks) split *= 2;
    const int slice_chunks = (chunks + split - 1) / split;
    int slice_units = slice_chunks * kChunkUnits;
    if (slice_units > units_total) slice_units = units_total;
    const int max_smem = 232448 - 256;  // 227 KB opt-in limit minus static shared and alignment slack
    const int x_bytes = slice_units * 16 * cols2 * 4 * 8;
    const int sx_bytes = TYPE == ZQ_Q4_K ? slice_units * cols2 * 4 * 8 : 0;
    const int fixed = x_bytes + sx_bytes + S::red_bytes + S::lut_bytes + 128 + 128;
    int stages = (max_smem - fixed) / S::stage_w;
    if (stages > 5) stages = 5;
    if (stages < 2) return false;
    ra.stages = stages;
    ra.split = split;
    ra.slice_units = slice_units;
    ra.units_total = units_total;
    ra.off_x = stages * S::stage_w;
    ra.off_sx = ra.off_x + x_bytes;
    ra.off_red = ra.off_sx + sx_bytes;
    ra.off_lut = ra.off_red + S::red_bytes;
    ra.off_bar = ra.off_lut + S::lut_bytes;
    total_bytes = ra.off_bar + 128 + 128;
    return true;
}

template <uint32_t TYPE, int NT, bool GATED>
static int launch_resident_one(zq_ctx *ctx, const zq_weight *w, const zq_weight *w_up, const GemvParams &p, int grid, bool &taken, zq_error *err) {
    (void)grid;
    ResidentArgs ra;
    int total = 0;
    taken = plan_resident<TYPE, NT>(p.m * p.limbs, (int)w->units_per_row, p.tiles, p.chunks, ctx->sm_count, ra, total);
    if (!taken) return ZQ_OK;
    auto kernel = gemv_resident_kernel<TYPE, NT, GATED>;
    static bool configured[64] = {};
    if (!configured[ctx->device & 63]) {
        ZQ_CUDA_CHECK(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 232448 - 256), err);
        ZQ_CUDA_CHECK(cudaFuncSetAttribute(kernel, cudaFuncAttributeNonPortableClusterSizeAllowed, 0), err);
        configured[ctx->device & 63] = true;
    }
    const CUtensorMap &ma = GATED ? w->gemv_map_half : w->gemv_map;
    const CUtensorMap &mb = GATED ? w_up->gemv_map_half : w->gemv_map;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)(p.tiles * ra.split));
    cfg.blockDim = dim3(kResidentThreads);
    cfg.dynamicSmemBytes = (size_t)total;
    cfg.stream = ctx->stream;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = (unsigned)ra.split;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[1].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = ctx->disable_pdl ? 1 : 2;
    ZQ_CUDA_CHECK(cudaLaunchKernelEx(&cfg, kernel, ma, mb, p, ra), err);
    ctx->launches++;
    return ZQ_OK;
}

template <uint32_t TYPE>
static int launch_resident_type(zq_ctx *ctx, const zq_weight *w, const zq_weight *w_up, const GemvParams &p, int grid, bool &taken, zq_error *err) {
    const bool gated = w_up != nullptr;
    if (p.m * p.limbs <= 8) return gated ? launch_resident_one<TYPE, 1, true>(ctx, w, w_up, p, grid, taken, err) : launch_resident_one<TYPE, 1, false>(ctx, w, w_up, p, grid, taken, err);
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
