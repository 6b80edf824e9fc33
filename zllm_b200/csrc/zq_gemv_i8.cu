// Decode GEMV on the integer tensor-core path (mma.sync m16n8k32, u8/s8 x s8 -> s32).
//
// Why integers: the packed weights ARE small integers.  Turning a 32-bit word of nibbles into an MMA operand costs
// one AND per four weights here (the low nibbles as they are, the high nibbles left in place as 16 q), against an
// AND-OR plus a scaled half-precision FMA per two weights on the f16 path, and one MMA covers a whole 32-weight
// scale group, so the group's scale is applied once to the s32 accumulator instead of to every operand pair.
// That cuts the instruction count per weight to under a half, which is what bounds these kernels.
//
// Activations: each row is cut into 256-column slices; a slice is scaled by its own absolute maximum to a signed
// 16-bit integer x_q in [-32512, 32512] and split into two s8 limbs, x_q = 256 hi + lo with lo in [-128, 127].
// The two limbs ride in neighbouring MMA columns, so one MMA column pair carries one activation row at an
// element-wise relative resolution of 2^-16 of the slice maximum (f16 activations carry 2^-11).
//   Q4_K   y += s_x * ( d/16 * sum_G sc_G * [16 * sum q x_q]  -  dmin * sum_G m_G * S_G ),   S_G = sum of x_q in group G
//          the bracket is what the MMAs return (low-nibble groups are multiplied by 16 in the integer domain);
//          the min term is one f16 MMA per unit on the exact integer sums S_G = 1024 a + r (a and r exact in f16).
//   Q4_0   y += s_x * d_b/16 * [sum 16 (q - 8) x_q]     (operand bytes (16 q) ^ 0x80 read as s8)
//   Q8_0   y += s_x * d_b * [sum q x_q]
//   IQ4_NL y += s_x * d_b * [sum K[q] x_q]               (codebook bytes looked up with PRMT, zq_i8.cuh)
// Everything up to the final scale is exact integer arithmetic; the result differs from the f32 reference only by
// the 2^-16 activation resolution and f32 rounding of the per-unit terms.
//
// Work partition: one CTA per (128-row tile, K slice); the CTAs of a thread-block cluster are `tshare`
// neighbouring tiles times `split` K slices.
//   * The K slices of one tile meet at the end in distributed shared memory: every CTA leaves its partial tile in
//     its own shared memory, the cluster synchronises, and the CTA of slice 0 adds the partials in slice order
//     (deterministic) and stores the tile.  No global scratch, no atomics.
//   * The tiles of a cluster need the same quantised activations.  Quantising them is the expensive part of the
//     prologue (it grows with the number of activation rows), so the CTAs that share a K slice divide it: each
//     quantises every tshare-th 256-column record and stores it into the shared memory of all of them.
// The weights stream through a ring of TMA stages (128 rows x 2 units each); every wait is bounded and a wait that
// runs out raises a CTA-wide abort flag plus the device status word, so the kernel always returns.
#include <map>
#include <mutex>
#include <tuple>

#include "zq_i8.cuh"

namespace zq {

// Quantises all records of an activation block [m, K] into global memory (record index = unit * m + row), for
// the kernel variant that streams the records through its ring instead of keeping them resident.
template <uint32_t TYPE>
__global__ void __launch_bounds__(256) quantize_acts_kernel(const void *x, int x_dtype, int M, int cols, int units_total, uint8_t *out) {
    pdl_launch_dependents();
    pdl_wait_prior_grid();
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int rec = blockIdx.x * 8 + warp;
    if (rec >= M * units_total) return;  // warp-uniform
    const int unit = rec / M, m = rec - unit * M;
    const int k0 = unit * kUnitWeights + 8 * lane;
    float v[8];
    load_act8(x, x_dtype, (size_t)m * cols + k0, k0 < cols, v);
    const RecLane o = quantize_record<TYPE>(v, lane);
    uint8_t *dst = out + (size_t)rec * kRec;
    *reinterpret_cast<uint4 *>(dst + o.slot) = make_uint4(o.ph0, o.ph1, o.pl0, o.pl1);
    if (is_kclass(TYPE) && (lane & 7) == 0) *reinterpret_cast<uint2 *>(dst + kRecSums + (lane >> 3) * 8) = make_uint2(o.sw0, o.sw1);
    if (lane == 0) *reinterpret_cast<float *>(dst + kRecScale) = o.scale;
}

// ROWS = weight rows per CTA: 128 (512 threads, one CTA per SM) or 64 (256 threads, two CTAs per SM).  The small
// form was built for the launch-to-launch hand-over: with two CTAs per SM, a CTA of the NEXT kernel (programmatic
// dependent launch) moves in as soon as ONE of the current kernel's CTAs leaves, and streams its first weights while
// the other is still working.  Measured on the decode sweep it loses 3 % to the large form (every CTA repeats the
// per-CTA work for half the rows), so it is kept behind the context option narrow_gemv_tiles.
template <uint32_t TYPE, int NT, bool GATED, int ROWS>
__global__ void __launch_bounds__(ROWS * 4, ROWS == 128 ? 1 : 2) gemv_i8_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b, const GemvParams p, const I8Args ia) {
    constexpr int THREADS = ROWS * 4, WARPS = THREADS / 32, SUBTILES = ROWS / 16;
    static_assert(ROWS == 128 || (ROWS == 64 && !GATED), "64-row tiles: plain projections only");
    constexpr int UB = Fmt<TYPE>::unit_bytes;
    constexpr int PITCH = kChunkUnits * UB;
    constexpr int STAGE_W = ROWS * PITCH;
    // More than 4 activation rows: the records would crowd the ring out of shared memory, and quantising them in every
    // CTA would cost more than the matrix; a small kernel quantises them once into global memory and every ring stage
    // brings the records of its two units along with the weights.
    constexpr bool XS = NT > 1;
    extern __shared__ uint8_t smem_raw[];
    uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 127) & ~uintptr_t(127));
    uint8_t *ws = smem;
    float *red = reinterpret_cast<float *>(smem + ia.off_red);
    uint64_t *full = reinterpret_cast<uint64_t *>(smem + ia.off_bar);
    uint64_t *empty = full + 8;
    __shared__ int s_abort;

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int STAGES = ia.stages;
    const int rows_per_tile = GATED ? ROWS / 2 : ROWS;
    const int split = ia.split, tshare = ia.tshare;
    const bool clustered = split * tshare > 1;
    const int my_tile = blockIdx.x / split, my_rank = blockIdx.x % split;
    const uint32_t crank = clustered ? i8_cluster_rank() : 0u;
    const int tile_local = (int)crank / split;  // which of the cluster's tiles
    const int chunk_begin = (int)((long long)my_rank * p.chunks / split), chunk_end = (int)((long long)(my_rank + 1) * p.chunks / split);
    const int n_items = chunk_end - chunk_begin;
    const int unit0 = chunk_begin * kChunkUnits;

    if (tshare > 1) i8_cluster_arrive();  // "this CTA runs": peers wait for it before they store into this CTA
    if (tid == 0) {
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(&full[s], 1);
            mbar_init(&empty[s], WARPS);
        }
        fence_mbar_init();
        tma_prefetch_desc(&map_a);
        if (GATED) tma_prefetch_desc(&map_b);
        s_abort = 0;
    }
    __syncthreads();

    const int M = p.m;
    const int stage_stride = ia.stage_stride;
    // weights of ring item `local` (and the byte count the stage's barrier has to see)
    auto issue_w = [&](int local, int stage) {
        const int chunk = chunk_begin + local;
        uint8_t *dst = ws + (size_t)stage * stage_stride;
        uint32_t bytes = STAGE_W;
        if (XS) {
            int nu = ia.units_total - chunk * kChunkUnits;
            if (nu > kChunkUnits) nu = kChunkUnits;
            bytes += (uint32_t)(nu * M * kRec);
        }
        mbar_expect_tx(&full[stage], bytes);
        if (GATED) {
            tma_load_2d(dst, &map_a, &full[stage], chunk * p.chunk_words, my_tile * rows_per_tile);
            tma_load_2d(dst + STAGE_W / 2, &map_b, &full[stage], chunk * p.chunk_words, my_tile * rows_per_tile);
        } else {
            tma_load_2d(dst, &map_a, &full[stage], chunk * p.chunk_words, my_tile * rows_per_tile);
        }
    };
    // streamed variant: the records of the item's units, right behind the weights of the stage
    auto issue_x = [&](int local, int stage) {
        if (!XS) return;
        const int chunk = chunk_begin + local;
        int nu = ia.units_total - chunk * kChunkUnits;
        if (nu > kChunkUnits) nu = kChunkUnits;
        bulk_load_1d(ws + (size_t)stage * stage_stride + STAGE_W, ia.xq + (size_t)chunk * kChunkUnits * M * kRec, (uint32_t)(nu * M * kRec), &full[stage]);
    };
    const int pre = n_items < STAGES - 1 ? n_items : STAGES - 1;
    if (tid == 0) {
        for (int s = 0; s < pre; ++s) issue_w(s, s);
    }
    pdl_launch_dependents();

    const int g = lane >> 2, t = lane & 3;
    const int rs = warp & (SUBTILES - 1), ul = warp / SUBTILES;

    int slice_units = chunk_end * kChunkUnits;
    if (slice_units > ia.units_total) slice_units = ia.units_total;
    slice_units -= unit0;
    if (slice_units < 0) slice_units = 0;
    const uint32_t x_base = smem_u32(smem + ia.off_x);

    pdl_wait_prior_grid();  // activations (and, later, outputs) belong to the previous kernel until it completes
    if (XS) {
        if (tid == 0) {
            for (int s = 0; s < pre; ++s) issue_x(s, s);
        }
    } else {
    if (tshare > 1) i8_cluster_wait();  // every CTA of the cluster is running: its shared memory may be written
    {
        // Quantise this CTA's share of the activation slice (every tshare-th record), one warp per record, 8
        // consecutive columns per lane, four records at a time with all loads first so that their latencies overlap;
        // each record goes to all CTAs of the cluster that work on this K slice.  Records of activation rows past m
        // do not exist: lanes whose MMA column has no row read some existing record instead, and whatever they
        // compute only reaches accumulator columns no one reads.
        constexpr int kBatch = 4, kWarps = WARPS;
        uint32_t peer_x[8];
#pragma unroll
        for (int q = 0; q < 8; ++q) peer_x[q] = (clustered && q < tshare) ? i8_mapa(x_base, (uint32_t)(q * split + my_rank)) : x_base;
        const int total = M * slice_units;
        const int n_mine = total > tile_local ? (total - tile_local + tshare - 1) / tshare : 0;
        for (int base = warp; base < n_mine; base += kBatch * kWarps) {
            float v[kBatch][8];
            int trec[kBatch];
#pragma unroll
            for (int b = 0; b < kBatch; ++b) {
                const int k = base + b * kWarps;
                const int task = tile_local + tshare * k;  // record index inside the slice: unit-major, then activation row
                trec[b] = k < n_mine ? task : -1;
                const int unit = task / M, m = task - unit * M;
                const int k0 = (unit0 + unit) * kUnitWeights + 8 * lane;
                // K is a multiple of 32, so a lane's 8 columns are all inside or all outside
                load_act8(p.x, p.x_dtype, (size_t)m * p.cols + k0, trec[b] >= 0 && k0 < p.cols, v[b]);
            }
#pragma unroll
            for (int b = 0; b < kBatch; ++b) {
                if (trec[b] < 0) continue;  // warp-uniform
                const RecLane o = quantize_record<TYPE>(v[b], lane);
                const uint32_t rec_off = (uint32_t)trec[b] * kRec;
                if (tshare == 1) {  // plain shared-memory stores
                    uint8_t *dst = smem + ia.off_x + rec_off;
                    *reinterpret_cast<uint4 *>(dst + o.slot) = make_uint4(o.ph0, o.ph1, o.pl0, o.pl1);
                    if (is_kclass(TYPE) && (lane & 7) == 0) *reinterpret_cast<uint2 *>(dst + kRecSums + (lane >> 3) * 8) = make_uint2(o.sw0, o.sw1);
                    if (lane == 0) *reinterpret_cast<float *>(dst + kRecScale) = o.scale;
                } else {
#pragma unroll
                    for (int q = 0; q < 8; ++q) {
                        if (q < tshare) {
                            const uint32_t dst = peer_x[q] + rec_off;
                            i8_st_cluster_v4(dst + o.slot, o.ph0, o.ph1, o.pl0, o.pl1);
                            if (is_kclass(TYPE) && (lane & 7) == 0) i8_st_cluster_v2(dst + kRecSums + (lane >> 3) * 8, o.sw0, o.sw1);
                            if (lane == 0) i8_st_cluster_u32(dst + kRecScale, __float_as_uint(o.scale));
                        }
                    }
                }
            }
        }
    }
    if (tshare > 1) {
        i8_cluster_arrive();
        i8_cluster_wait();
    } else {
        __syncthreads();
    }
    }  // !XS

    float yacc[NT][2];
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) yacc[nt][0] = yacc[nt][1] = 0.f;
    const int r0 = 16 * rs + frag_row(g);

    {
        const uint32_t w_first = smem_u32(ws) + (uint32_t)(r0 * PITCH + ul * UB);
        const uint32_t xoff = (uint32_t)(16 * t + 8 * (g & 1));
        // records of the activation rows this lane touches (clamped to an existing row): its B column of tile nt is
        // row 4 nt + g / 2, its accumulator columns are row 4 nt + t
        uint32_t moff[NT], soff[NT];
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) {
            int m = 4 * nt + (g >> 1), ms = 4 * nt + t;
            if (m > M - 1) m = M - 1;
            if (ms > M - 1) ms = M - 1;
            moff[nt] = (uint32_t)(m * kRec);
            soff[nt] = (uint32_t)(ms * kRec);
        }
        const uint32_t unit_stride = (uint32_t)(M * kRec);
        // resident: walks the slice's records; streamed: the stage's own two units
        uint32_t recu = (XS ? smem_u32(ws) + STAGE_W : x_base) + (uint32_t)ul * unit_stride;
        int stage = 0;
        uint32_t phase = 0;
        int unit_abs = unit0 + ul;
        for (int it = 0; it < n_items; ++it) {
            {
                // refill: the stage consumed one iteration ago takes the item STAGES-1 ahead; a different warp each time
                const int nxt = it + STAGES - 1;
                if (nxt < n_items && warp == (it & (WARPS - 1)) && lane == 0) {
                    const int nstage = stage == 0 ? STAGES - 1 : stage - 1;
                    if (it >= 1) i8_wait_or_abort(&empty[nstage], stage == 0 ? phase ^ 1u : phase, &s_abort, p.status);
                    if (!*(volatile int *)&s_abort) {  // never start a copy nobody will wait for
                        issue_w(nxt, nstage);
                        issue_x(nxt, nstage);
                    }
                }
                __syncwarp();
            }
            i8_wait_or_abort(&full[stage], phase, &s_abort, p.status);
            if (unit_abs < ia.units_total) {
                const uint32_t soffs = (uint32_t)(stage * stage_stride);
                const uint32_t wq0 = w_first + soffs, wq1 = wq0 + 8 * PITCH;
                const uint32_t rb = XS ? recu + soffs : recu;
                uint32_t rec[NT], srec[NT];
#pragma unroll
                for (int nt = 0; nt < NT; ++nt) {
                    rec[nt] = rb + moff[nt];
                    srec[nt] = rb + soff[nt];
                }
                if constexpr (TYPE == ZQ_Q6_K) consume_q6k_i8<NT>(wq0, wq1, t, rec, srec, xoff, yacc);
            else if constexpr (is_kclass(TYPE)) consume_q4k_i8<NT, TYPE == ZQ_Q5_K>(wq0, wq1, t, rec, srec, xoff, yacc);
                else consume_b32_i8<TYPE, NT>(wq0, wq1, t, rec, srec, xoff, yacc);
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(&empty[stage]);
            if (++stage == STAGES) {
                stage = 0;
                phase ^= 1u;
            }
            unit_abs += kChunkUnits;
            if (!XS) recu += kChunkUnits * unit_stride;
        }
    }

    // ---------------------------------------------------- end of the K slice: combine and store
    {
        // Every CTA leaves its partial tile (one copy per unit half) in its own shared memory; after one barrier
        // (cluster-wide when the tile is split) the threads of slice 0 add up, for their output element, the halves
        // of every slice in slice order (deterministic), apply the epilogue and store.
        constexpr int RS = NT * 4;  // activation rows a tile row can hold
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) {
            red[(ul * RS + nt * 4 + t) * ROWS + r0] = yacc[nt][0];  // [unit half][activation row][tile row]
            red[(ul * RS + nt * 4 + t) * ROWS + r0 + 8] = yacc[nt][1];
        }
        if (split > 1) {
            i8_cluster_arrive();
            i8_cluster_wait();
        } else {
            __syncthreads();
        }
        if (my_rank == 0) {
            constexpr int out_rows = GATED ? ROWS / 2 : ROWS;
            auto total_of = [&](int rr, int tok) -> float {
                const float *a = &red[tok * ROWS + rr], *b = &red[(RS + tok) * ROWS + rr];
                float v = *a + *b;
                for (int r = 1; r < split; ++r) {
                    const uint32_t peer = (uint32_t)(tile_local * split + r);
                    v += i8_ld_cluster_f32(i8_mapa(smem_u32(a), peer)) + i8_ld_cluster_f32(i8_mapa(smem_u32(b), peer));
                }
                return v;
            };
            for (int i = tid; i < out_rows * M; i += THREADS) {
                const int row = i & (out_rows - 1), tok = i / out_rows;
                const int n = my_tile * out_rows + row;
                if (n >= p.n_out) continue;
                float v;
                if (GATED) {
                    const float gate = total_of(row, tok), up = total_of(out_rows + row, tok);
                    v = (gate / (1.0f + expf(-gate))) * up;
                } else {
                    v = total_of(row, tok);
                }
                const size_t o = (size_t)tok * p.n_out + n;
                if (p.residual) v += load_as_f32(p.residual, p.y_dtype, o);
                store_from_f32(p.y, p.y_dtype, o, v);
            }
        }
        if (split > 1) {  // nobody leaves while slice 0 may still read its shared memory
            i8_cluster_arrive();
            i8_cluster_wait();
        }
    }
}

// How many clusters of a configuration can be resident at once (cached: the query is a host-side driver call).
template <class Kernel>
static int max_active_clusters(Kernel kernel, int device, int cluster, int smem_bytes, int grid, int threads) {
    static std::mutex mu;
    static std::map<std::tuple<const void *, int, int, int>, int> cache;
    const auto key = std::make_tuple((const void *)kernel, device, cluster, smem_bytes);
    std::lock_guard<std::mutex> lock(mu);
    auto it = cache.find(key);
    if (it != cache.end()) return it->second;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)(grid - grid % cluster));
    cfg.blockDim = dim3((unsigned)threads);
    cfg.dynamicSmemBytes = (size_t)smem_bytes;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = (unsigned)cluster;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    int n = 0;
    if (cudaOccupancyMaxActiveClusters(&n, kernel, &cfg) != cudaSuccess) {
        cudaGetLastError();
        n = 0;
    }
    cache[key] = n;
    return n;
}

// Shared-memory plan: K slices per tile, ring depth and offsets; false when fewer than two ring stages fit beside
// the quantised activation slice.
template <uint32_t TYPE, int NT, int ROWS>
static bool plan_i8(int m, int units_total, int tiles, int chunks, int sm_count, I8Args &ia, int &total_bytes) {
    constexpr int STAGE_W = ROWS * kChunkUnits * Fmt<TYPE>::unit_bytes;
    // 227 KB opt-in limit minus static shared and alignment slack; the 64-row form must leave room for a second CTA
    const int max_smem = ROWS == 128 ? 232448 - 256 : 112 * 1024;
    const int red_bytes = 2 * ROWS * NT * 4 * 4;
    const int slots = sm_count * (ROWS == 128 ? 1 : 2);
    // K slices per tile: as many as fill the SMs (any count up to 8, not only powers of two); more than that, i.e.
    // more CTAs than SMs, only when the activation slice would otherwise leave no room for the ring
    int split = slots / (tiles > 0 ? tiles : 1);
    if (split > 8) split = 8;
    if (split > chunks) split = chunks;
    if (split < 1) split = 1;
    int room = 0, slice_chunks = 0, x_bytes = 0;  // room: ring stages that fit
    int stage_stride = STAGE_W;
    if (NT > 1) {  // records stream through the ring: nothing resident, no reason to split beyond the SM count
        stage_stride = STAGE_W + kChunkUnits * m * kRec;
        slice_chunks = (chunks + split - 1) / split;
        room = (max_smem - (red_bytes + 128 + 128)) / stage_stride;
    } else {
        for (;; ++split) {
            slice_chunks = (chunks + split - 1) / split;
            int slice_units = slice_chunks * kChunkUnits;
            if (slice_units > units_total) slice_units = units_total;
            x_bytes = (slice_units * m * kRec + 127) & ~127;
            room = (max_smem - (x_bytes + red_bytes + 128 + 128)) / STAGE_W;
            if (room >= 3 || split >= 8 || split >= chunks) break;
        }
    }
    if (room < 2) return false;
    int stages = room > 5 ? 5 : room;
    if (stages > slice_chunks + 1) stages = slice_chunks + 1;  // no point in more ring than work
    if (stages < 2) stages = 2;
    ia.stage_stride = stage_stride;
    ia.xq = nullptr;
    ia.stages = stages;
    ia.split = split;
    ia.tshare = 1;
    ia.units_total = units_total;
    ia.off_x = stages * stage_stride;
    ia.off_red = ia.off_x + x_bytes;
    ia.off_bar = ia.off_red + red_bytes;
    total_bytes = ia.off_bar + 128 + 128;
    return true;
}

template <uint32_t TYPE, int NT, bool GATED, int ROWS>
static int launch_i8_one(zq_ctx *ctx, const zq_weight *w, const zq_weight *w_up, const GemvParams &p, bool &taken, zq_error *err) {
    I8Args ia;
    int total = 0;
    const int rows_per_tile = GATED ? ROWS / 2 : ROWS;
    const int tiles = (p.n_out + rows_per_tile - 1) / rows_per_tile;
    taken = plan_i8<TYPE, NT, ROWS>(p.m, (int)w->units_per_row, tiles, p.chunks, ctx->sm_count, ia, total);
    if (ROWS == 64 && taken && ia.stages < 3) taken = false;  // too little ring for the small form: the caller tries the large one
    if (!taken) return ZQ_OK;
    auto kernel = gemv_i8_kernel<TYPE, NT, GATED, ROWS>;
    static bool configured[64] = {};
    if (!configured[ctx->device & 63]) {
        ZQ_CUDA_CHECK(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, ROWS == 128 ? 232448 - 256 : 112 * 1024 + 512), err);
        configured[ctx->device & 63] = true;
    }
    if (NT > 1) {
        // quantise the activation block once; the main kernel's ring picks the records up
        const int records = p.m * (int)w->units_per_row;
        int rc = ensure_xq(ctx, (size_t)records * kRec, err);
        if (rc) return rc;
        ia.xq = reinterpret_cast<const uint8_t *>(ctx->xq);
        cudaLaunchConfig_t qcfg = {};
        qcfg.gridDim = dim3((unsigned)((records + 7) / 8));
        qcfg.blockDim = dim3(256);
        qcfg.stream = ctx->stream;
        cudaLaunchAttribute qattr[1];
        qattr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        qattr[0].val.programmaticStreamSerializationAllowed = 1;
        qcfg.attrs = qattr;
        qcfg.numAttrs = ctx->disable_pdl ? 0 : 1;
        ZQ_CUDA_CHECK(cudaLaunchKernelEx(&qcfg, quantize_acts_kernel<TYPE>, p.x, p.x_dtype, p.m, p.cols, (int)w->units_per_row, reinterpret_cast<uint8_t *>(ctx->xq)), err);
        ctx->launches++;
    }
    // Tiles per cluster that share the activation staging: the largest divisor of the tile count that keeps the
    // cluster within 8 CTAs and still lets as many CTAs run at once as unshared clusters would.
    const int grid = tiles * ia.split;
    if (NT == 1 && p.m * (int)w->units_per_row >= 32) {  // a handful of records is quicker done by every CTA for itself
        const int base_active = max_active_clusters(kernel, ctx->device, ia.split, total, grid, ROWS * 4) * ia.split;
        const int want = grid < base_active ? grid : base_active;
        for (int ts = 8 / ia.split; ts > 1; --ts) {
            if (tiles % ts) continue;
            const int c = ia.split * ts;
            if (max_active_clusters(kernel, ctx->device, c, total, grid, ROWS * 4) * c >= want) {
                ia.tshare = ts;
                break;
            }
        }
    }
    const CUtensorMap &ma = (GATED || ROWS == 64) ? w->gemv_map_half : w->gemv_map;  // 64-row boxes
    const CUtensorMap &mb = GATED ? w_up->gemv_map_half : ma;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)grid);
    cfg.blockDim = dim3((unsigned)(ROWS * 4));
    cfg.dynamicSmemBytes = (size_t)total;
    cfg.stream = ctx->stream;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = (unsigned)(ia.split * ia.tshare);
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[1].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = ctx->disable_pdl ? 1 : 2;
    ZQ_CUDA_CHECK(cudaLaunchKernelEx(&cfg, kernel, ma, mb, p, ia), err);
    ctx->launches++;
    return ZQ_OK;
}

template <uint32_t TYPE>
static int launch_i8_type(zq_ctx *ctx, const zq_weight *w, const zq_weight *w_up, const GemvParams &p, bool &taken, zq_error *err) {
    const bool gated = w_up != nullptr;
    if (p.m <= 4) {
        if (gated) return launch_i8_one<TYPE, 1, true, 128>(ctx, w, w_up, p, taken, err);
        if (ctx->narrow_gemv_tiles) {  // opt-in: two 64-row CTAs per SM, so that the next kernel overlaps this one's tail
            int rc = launch_i8_one<TYPE, 1, false, 64>(ctx, w, w_up, p, taken, err);
            if (rc || taken) return rc;
        }
        return launch_i8_one<TYPE, 1, false, 128>(ctx, w, w_up, p, taken, err);
    }
    if (p.m <= 8) return gated ? launch_i8_one<TYPE, 2, true, 128>(ctx, w, w_up, p, taken, err) : launch_i8_one<TYPE, 2, false, 128>(ctx, w, w_up, p, taken, err);
    return gated ? launch_i8_one<TYPE, 4, true, 128>(ctx, w, w_up, p, taken, err) : launch_i8_one<TYPE, 4, false, 128>(ctx, w, w_up, p, taken, err);
}

// Tries the integer-MMA kernel for one pass of up to 16 activation rows; `taken` tells whether it was launched
// (slices that do not fit stay on the f16 kernels).
int launch_gemv_i8(zq_ctx *ctx, const zq_weight *w, const zq_weight *w_up, const GemvParams &p, bool &taken, zq_error *err) {
    taken = false;
    if (p.m < 1 || p.m > kMaxGemvRows) return ZQ_OK;
    switch (w->type) {
    case ZQ_Q4_K: return launch_i8_type<ZQ_Q4_K>(ctx, w, w_up, p, taken, err);
    case ZQ_Q5_K: return launch_i8_type<ZQ_Q5_K>(ctx, w, w_up, p, taken, err);
    case ZQ_Q6_K: return launch_i8_type<ZQ_Q6_K>(ctx, w, w_up, p, taken, err);
    case ZQ_Q4_0: return launch_i8_type<ZQ_Q4_0>(ctx, w, w_up, p, taken, err);
    case ZQ_IQ4_NL: return launch_i8_type<ZQ_IQ4_NL>(ctx, w, w_up, p, taken, err);
    case ZQ_Q8_0: return launch_i8_type<ZQ_Q8_0>(ctx, w, w_up, p, taken, err);
    default: return ZQ_OK;
    }
}

}  // namespace zq
