// Decode GEMV over a work list: several independent projections (jobs) in ONE persistent launch.
//
// A decode step is a handful of matrices of 1..50 MB each.  At B200 bandwidth such a matrix streams in 1..8 us, about
// the cost of starting a kernel, filling its TMA ring and draining it again, so a launch per matrix leaves HBM idle
// between matrices.  Here the (job, 128-row tile, 2-unit chunk) items of all jobs form one sequence that is cut into
// equal contiguous ranges, one per SM ("stream-K"): every CTA streams its range through one TMA ring that never
// drains between tiles or matrices, all SMs stay busy whatever the tile counts of the single matrices are, and the
// launch cost is paid once.
//
//   wl_quantize_kernel   activation records (zq_i8.cuh) of every distinct input block of the list, once, into global
//                        memory; each ring stage then brings the records of its two units along with the weights
//   gemv_wl_kernel       integer-MMA decode (arithmetic of zq_gemv_i8.cu) over the CTA's range
//
// Tiles that a range boundary cuts are finished without any CTA waiting for another: each contributor leaves its
// partial tile in its own slot of the context's scratch and bumps the tile's arrival counter; whoever arrives last
// adds the partials in CTA order (a fixed order: results are deterministic), applies the epilogue and stores.
// A CTA has at most two such tiles (the first and the last of its range).
//
// Reference behaviour covered: ggml_quant::matvec / matvec_residual / gated_silu_matvec
// (src/kernel/cpu/ggml_quant.rs:189-277) for a list of weights, as Backend::dual_linear / triple_linear
// (src/backend/mod.rs:444-451) and the Metal backend's gguf_dual_gemv_q4k_f16 (src/kernel/metal/gguf/mod.rs:1787-1824)
// do for two or three.
#include "zq_i8.cuh"
#include "zq_wl.cuh"

namespace zq {

constexpr int kWlMaxSegs = 128;  // (tile, chunk range) pieces of one CTA's range kept in shared memory

struct WlJob {
    const CUtensorMap *map_a;  // device copy of the weight's tensor map: 128-row boxes, or (gated) gate, 64-row boxes
    const CUtensorMap *map_b;  // gated: up, 64-row boxes
    const uint8_t *xq;         // records of the job's activation block, [unit][row]
    void *y;                   // [m, n_out]
    const void *residual;      // [m, n_out] or null
    int m;                     // activation rows (1 .. 4 NT)
    int n_out;                 // output features
    int units;                 // 256-column units per weight row
    int chunks;                // ring items per tile = ceil(units / 2)
    int tiles;                 // row tiles
    int q_begin;               // first ring item of the job in the launch's (job, tile, chunk) order
    int y_dtype;               // output (and residual) dtype of this job
    int pad;
};

struct WlArgs {
    WlJob jobs[kWlMaxJobs];
    int n_jobs;
    int q_total;       // ring items of the whole launch
    int chunk_words;   // 32-bit words per chunk of a weight row
    int y_dtype;
    float *partials;   // [2 * grid][kSlotFloats]: slot 2c + 1 = the tile CTA c begins, slot 2c = the tile it continues
    uint32_t *counters;  // [grid], zero between launches: arrivals at the cut tile that CTA c begins
    uint32_t *status;
};

struct WlQuantSrc {
    const void *x;
    int m, cols, units;
    int rec_begin;  // first record of the block in the record buffer
};
struct WlQuantArgs {
    WlQuantSrc src[kWlMaxJobs];
    int n_src, total, x_dtype;
    uint8_t *out;
};

// Records of every distinct activation block of the list: one warp per (block, unit, row).
template <uint32_t TYPE>
__global__ void __launch_bounds__(256) wl_quantize_kernel(const __grid_constant__ WlQuantArgs qa) {
    pdl_launch_dependents();
    pdl_wait_prior_grid();  // the record buffer may still be read by the previous launch
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int rec = blockIdx.x * 8 + warp;
    if (rec >= qa.total) return;  // warp-uniform
    int s = 0;
    while (s + 1 < qa.n_src && qa.src[s + 1].rec_begin <= rec) ++s;
    const WlQuantSrc &q = qa.src[s];
    const int local = rec - q.rec_begin;
    const int unit = local / q.m, row = local - unit * q.m;
    const int k0 = unit * kUnitWeights + 8 * lane;
    float v[8];
    load_act8(q.x, qa.x_dtype, (size_t)row * q.cols + k0, k0 < q.cols, v);
    const RecLane o = quantize_record<TYPE>(v, lane);
    uint8_t *dst = qa.out + (size_t)rec * kRec;
    *reinterpret_cast<uint4 *>(dst + o.slot) = make_uint4(o.ph0, o.ph1, o.pl0, o.pl1);
    if (is_kclass(TYPE) && (lane & 7) == 0) *reinterpret_cast<uint2 *>(dst + kRecSums + (lane >> 3) * 8) = make_uint2(o.sw0, o.sw1);
    if (lane == 0) *reinterpret_cast<float *>(dst + kRecScale) = o.scale;
}

// Shared-memory plan of one instantiation: as many ring stages (up to 5) as fit beside the exchange buffers.
template <uint32_t TYPE, int NT> struct WlSmem {
    static constexpr int UB = Fmt<TYPE>::unit_bytes;
    static constexpr int PITCH = kChunkUnits * UB;
    static constexpr int STAGE_W = kTileRows * PITCH;
    static constexpr int MROWS = 4 * NT;                                  // activation rows a launch class holds
    static constexpr int STRIDE = STAGE_W + kChunkUnits * MROWS * kRec;   // weights, then the chunk's records
    static constexpr int XCH_FLOATS = 16 * 32 * NT * 2;                   // one buffer: [consumer warp][lane][accumulator]
    static constexpr int LIMIT = 232448 - 1024;                           // opt-in maximum minus static shared memory
    static constexpr int MISC = 2 * XCH_FLOATS * 4 + kWlMaxSegs * 16 + 128 + 128;  // exchange (2 buffers), segment list, barriers, slack
    static constexpr int STAGES = (LIMIT - MISC) / STRIDE > 5 ? 5 : (LIMIT - MISC) / STRIDE;
    static constexpr int OFF_XCH = STAGES * STRIDE;
    static constexpr int OFF_SEG = OFF_XCH + 2 * XCH_FLOATS * 4;
    static constexpr int OFF_BAR = OFF_SEG + kWlMaxSegs * 16;
    static constexpr int TOTAL = OFF_BAR + 128 + 128;
    static_assert(STAGES >= 2, "work-list decode kernel: fewer than two ring stages fit");
    static_assert(STRIDE % 128 == 0 && STAGE_W % 256 == 0, "ring stages must keep TMA destinations 128-byte aligned");
};

constexpr int kWlConsumers = kI8Threads;        // 16 consumer warps: 8 row sub-tiles x 2 units
constexpr int kWlThreads = kWlConsumers + 64;   // + the producer warp and the finisher warp
// Named barriers (0 is left to __syncthreads, which this kernel never uses: the producer warp runs its own loop).
constexpr int kBarQuad = 1;    // 1..4: the four warps that hold gate and up sums of the same 16 output rows (gated tiles)
constexpr int kBarPair = 5;    // 5..12: the two warps (unit halves) of one row sub-tile
constexpr int kBarFix = 13;    // 13, 14: the 16 consumer warps hand a cut tile's partial sums to the finisher warp (first / second cut piece)
constexpr int kBarAll = 15;    // the 16 consumer warps among themselves (9..16 activation rows: they finish cut tiles on their own)

__device__ __forceinline__ void named_bar_sync(int id, int threads) { asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(threads) : "memory"); }
// Release / acquire fence at GPU scope: orders this thread's (and, after a CTA barrier, its CTA's) earlier accesses before
// its later ones; lighter than the sequentially consistent fence __threadfence() stands for.
__device__ __forceinline__ void fence_acq_rel_gpu() { asm volatile("fence.acq_rel.gpu;" ::: "memory"); }
__device__ __forceinline__ void named_bar_arrive(int id, int threads) { asm volatile("bar.arrive %0, %1;" ::"r"(id), "r"(threads) : "memory"); }

// CTA that owns ring item q when Q items are cut into G ranges [floor(c Q / G), floor((c + 1) Q / G)).
__device__ __forceinline__ int wl_owner(long long q, long long G, long long Q) { return (int)(((q + 1) * G - 1) / Q); }

// Bounded mbarrier wait that reads the abort flag through its shared address.
__device__ __forceinline__ void wl_wait(uint64_t *bar, uint32_t parity, uint32_t abort_addr, uint32_t *status) {
    for (uint32_t i = 0; i < (1u << 22); ++i) {
        if (mbar_try_wait(bar, parity)) return;
        uint32_t f;
        asm volatile("ld.volatile.shared.u32 %0, [%1];" : "=r"(f) : "r"(abort_addr));
        if (f) return;
    }
    asm volatile("st.volatile.shared.u32 [%0], %1;" ::"r"(abort_addr), "r"(1u));
    atomicMax(status, (uint32_t)kStatusTmaTimeout);
}

// Warp-specialised: warp 16 is the producer (it alone waits for free ring stages and issues the TMA copies, so no
// consumer ever stalls on another consumer's progress); warps 0..15 consume.  At the end of a tile only the warps
// that hold sums of the same output rows meet (named barriers of 64 or 128 threads): the two unit halves of a row
// sub-tile, plus the gate / up partners of a gated tile.  The accumulators of partner warps sit in the same lanes, so
// the exchange buffer is indexed by lane and the owning warp stores its 16 rows straight from its fragments.
template <uint32_t TYPE, int NT, bool GATED>
__global__ void __launch_bounds__(kWlThreads, 1) gemv_wl_kernel(const __grid_constant__ WlArgs a) {
    using S = WlSmem<TYPE, NT>;
    constexpr int STAGES = S::STAGES, STRIDE = S::STRIDE, STAGE_W = S::STAGE_W, PITCH = S::PITCH, UB = S::UB;
    constexpr int XCH_FLOATS = S::XCH_FLOATS, NACC = NT * 2;
    constexpr int out_rows = GATED ? kTileRows / 2 : kTileRows;
    extern __shared__ uint8_t smem_raw[];
    uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 127) & ~uintptr_t(127));
    uint8_t *ws = smem;
    float *xch = reinterpret_cast<float *>(smem + S::OFF_XCH);
    int4 *segs = reinterpret_cast<int4 *>(smem + S::OFF_SEG);  // {job, tile, first chunk | end chunk << 16, first item (CTA-relative)}
    uint64_t *full = reinterpret_cast<uint64_t *>(smem + S::OFF_BAR);
    uint64_t *empty = full + 8;
    __shared__ uint32_t s_abort;
    __shared__ int s_nseg, s_last, s_c0, s_cl;
    // Up to 8 activation rows a cut tile's partial sums are a few KB and one warp adds them up beside the consumers; with
    // 9..16 rows that warp would need longer than the consumers themselves, so they do it together (and wait for it).
    constexpr bool kAsyncFix = NT < 4;

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const long long G = gridDim.x, Q = a.q_total;
    const int bid = blockIdx.x;
    const int q0 = (int)(bid * Q / G), q1 = (int)((bid + 1) * Q / G);
    const int n_items = q1 - q0;

    // the tensor maps live in global memory: fetch them into the descriptor cache while thread 0 lays out the range
    if (tid >= 32 && tid < 32 + a.n_jobs) {
        tma_prefetch_desc(a.jobs[tid - 32].map_a);
        if (GATED) tma_prefetch_desc(a.jobs[tid - 32].map_b);
    }
    if (tid == 0) {
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(&full[s], 1);
            mbar_init(&empty[s], kWlConsumers / 32);
        }
        fence_mbar_init();
        s_abort = 0;
        // this CTA's range as (job, tile, chunk range) pieces
        int j = 0;
        while (j + 1 < a.n_jobs && a.jobs[j + 1].q_begin <= q0) ++j;
        const int rel = q0 - a.jobs[j].q_begin;
        int tile = rel / a.jobs[j].chunks, cb = rel - tile * a.jobs[j].chunks;
        int q = q0, n = 0;
        while (q < q1 && n < kWlMaxSegs && j < a.n_jobs) {
            const int chunks = a.jobs[j].chunks;
            int ce = chunks;
            if (q + (ce - cb) > q1) ce = cb + (q1 - q);
            segs[n++] = make_int4(j, tile, cb | (ce << 16), q - q0);
            q += ce - cb;
            cb = 0;
            if (ce == chunks && ++tile == a.jobs[j].tiles) {
                tile = 0;
                ++j;
            }
        }
        if (q < q1) atomicMax(a.status, (uint32_t)kStatusBadIndex);  // the host sizes launches so that this never happens
        // Cut tiles first: a piece of a tile that a range boundary cuts (only the first and the last piece of a range can
        // be one) is finished by whichever contributor arrives last, so every CTA does its cut pieces at the start and
        // the hand-over completes under the streaming of the whole tiles instead of at the very end of the kernel.
        if (n >= 2) {
            const int4 last = segs[n - 1];
            const bool last_cut = !((last.z & 0xFFFF) == 0 && (last.z >> 16) == a.jobs[last.x].chunks);
            const int4 first = segs[0];
            const bool first_cut = !((first.z & 0xFFFF) == 0 && (first.z >> 16) == a.jobs[first.x].chunks);
            if (last_cut) {
                const int pos = first_cut ? 1 : 0;
                for (int k = n - 1; k > pos; --k) segs[k] = segs[k - 1];
                segs[pos] = last;
                int item = 0;
                for (int k = 0; k < n; ++k) {
                    segs[k].w = item;
                    item += (segs[k].z >> 16) - (segs[k].z & 0xFFFF);
                }
            }
        }
        s_nseg = n;
    }
    __syncthreads();  // the only CTA-wide barrier: before the roles part
    const int nseg = s_nseg;
    const int last_item = nseg ? segs[nseg - 1].w + ((segs[nseg - 1].z >> 16) - (segs[nseg - 1].z & 0xFFFF)) : 0;
    const int total_items = last_item < n_items ? last_item : n_items;
    const uint32_t abort_addr = smem_u32(&s_abort);

    if (warp == kWlConsumers / 32 + 1) {
        // ------------------------------------------------------------------------------------------ finisher warp
        // Completes the tiles this CTA shares with its neighbours, off the consumers' path: waits until the consumers
        // have stored a cut piece's partial sums, publishes them (fence + arrival count) and, if this CTA was the last
        // contributor, adds all partials in CTA order and stores the tile.
        pdl_launch_dependents();
        if (!kAsyncFix) return;
        pdl_wait_prior_grid();  // outputs and the fix-up scratch belong to earlier kernels until they complete
        constexpr int G4 = 4 * NT;  // float4 groups per lane: 128 rows x (4 NT) activation rows / 4 / 32 lanes
        for (int k = 0; k < 2 && k < nseg; ++k) {
            const int4 sg = segs[k];
            const WlJob &jb = a.jobs[sg.x];
            const int tile = sg.y, cb = sg.z & 0xFFFF, ce = sg.z >> 16, M = jb.m;
            if (cb == 0 && ce == jb.chunks) break;  // cut pieces come first
            named_bar_sync(kBarFix + k, kWlConsumers + 32);  // the consumers have stored this piece's partial sums
            int last = 0, c0 = 0, cl = 0;
            if (lane == 0) {
                fence_acq_rel_gpu();
                const long long ts = (long long)jb.q_begin + (long long)tile * jb.chunks;
                c0 = wl_owner(ts, G, Q);
                cl = wl_owner(ts + jb.chunks - 1, G, Q);
                last = atomicAdd(&a.counters[c0], 1u) == (uint32_t)(cl - c0);
            }
            last = __shfl_sync(0xffffffffu, last, 0);
            c0 = __shfl_sync(0xffffffffu, c0, 0);
            cl = __shfl_sync(0xffffffffu, cl, 0);
            if (!last) continue;
            fence_acq_rel_gpu();
            // A slot is [activation row][128 tile rows] f32.  Lane L owns tile rows 4L..4L+3 (one float4) of every
            // activation row; up to 8 activation rows are summed at a time so that a contributor costs one round trip.
            constexpr int GB = G4 < 8 ? G4 : 8;
            for (int qb = 0; qb < G4 && qb < M; qb += GB) {
                float4 acc[GB];
#pragma unroll
                for (int i = 0; i < GB; ++i) acc[i] = make_float4(0.f, 0.f, 0.f, 0.f);
                for (int c = c0; c <= cl; ++c) {
                    const float4 *ps = reinterpret_cast<const float4 *>(a.partials + (size_t)(2 * c + (c == c0 ? 1 : 0)) * kSlotFloats);
                    float4 got[GB];
#pragma unroll
                    for (int i = 0; i < GB; ++i) got[i] = qb + i < M ? __ldcg(ps + lane + 32 * (qb + i)) : make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
                    for (int i = 0; i < GB; ++i) {
                        acc[i].x += got[i].x; acc[i].y += got[i].y; acc[i].z += got[i].z; acc[i].w += got[i].w;
                    }
                }
#pragma unroll
                for (int i = 0; i < GB; ++i) {
                    const int tok = qb + i;
                    if (tok >= M) break;  // warp-uniform
                    const float vv[4] = {acc[i].x, acc[i].y, acc[i].z, acc[i].w};
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        const int row = 4 * lane + e;  // row inside the 128-row slot
                        float v = vv[e];
                        if (GATED) {
                            const float up = __shfl_down_sync(0xffffffffu, v, 16);  // lanes 16..31 hold rows 64..127: the up sums
                            if (row >= out_rows) continue;
                            v = (v / (1.0f + expf(-v))) * up;
                        }
                        const int n = tile * out_rows + row;
                        if (n >= jb.n_out) continue;
                        const size_t o = (size_t)tok * jb.n_out + n;
                        if (jb.residual) v += load_as_f32(jb.residual, jb.y_dtype, o);
                        store_from_f32(jb.y, jb.y_dtype, o, v);
                    }
                }
            }
            if (lane == 0) a.counters[c0] = 0;  // ready for the next launch
        }
        return;
    }
    if (warp == kWlConsumers / 32) {
        // ------------------------------------------------------------------------------------------ producer warp
        if (lane == 0) {
            int psi = 0;
            auto locate = [&](int i) {
                while (psi + 1 < nseg && segs[psi + 1].w <= i) ++psi;
            };
            auto issue_w = [&](int i, int stage) {
                const int4 sg = segs[psi];
                const WlJob &jb = a.jobs[sg.x];
                const int chunk = (sg.z & 0xFFFF) + (i - sg.w);
                int nu = jb.units - chunk * kChunkUnits;
                if (nu > kChunkUnits) nu = kChunkUnits;
                uint8_t *dst = ws + (size_t)stage * STRIDE;
                mbar_expect_tx(&full[stage], (uint32_t)(STAGE_W + nu * jb.m * kRec));
                tma_load_2d(dst, jb.map_a, &full[stage], chunk * a.chunk_words, sg.y * out_rows);
                if (GATED) tma_load_2d(dst + STAGE_W / 2, jb.map_b, &full[stage], chunk * a.chunk_words, sg.y * out_rows);
            };
            auto issue_x = [&](int i, int stage) {
                const int4 sg = segs[psi];
                const WlJob &jb = a.jobs[sg.x];
                const int chunk = (sg.z & 0xFFFF) + (i - sg.w);
                int nu = jb.units - chunk * kChunkUnits;
                if (nu > kChunkUnits) nu = kChunkUnits;
                bulk_load_1d(ws + (size_t)stage * STRIDE + STAGE_W, jb.xq + (size_t)chunk * kChunkUnits * jb.m * kRec, (uint32_t)(nu * jb.m * kRec), &full[stage]);
            };
            const int pre = total_items < STAGES ? total_items : STAGES;
            for (int s = 0; s < pre; ++s) {
                locate(s);
                issue_w(s, s);  // weights are constants: they may stream while the previous kernel still runs
            }
            pdl_launch_dependents();
            pdl_wait_prior_grid();  // the records belong to the record pass, which waits for everything before it
            psi = 0;
            for (int s = 0; s < pre; ++s) {
                locate(s);
                issue_x(s, s);
            }
            int stage = 0;
            uint32_t phase = 0;
            for (int i = pre; i < total_items; ++i) {
                wl_wait(&empty[stage], phase, abort_addr, a.status);  // every consumer warp is done with the stage's previous item
                uint32_t f;
                asm volatile("ld.volatile.shared.u32 %0, [%1];" : "=r"(f) : "r"(abort_addr));
                if (f) break;  // never start a copy nobody will wait for
                locate(i);
                issue_w(i, stage);
                issue_x(i, stage);
                if (++stage == STAGES) {
                    stage = 0;
                    phase ^= 1u;
                }
            }
        } else {
            pdl_launch_dependents();
        }
        return;
    }

    // ---------------------------------------------------------------------------------------------- consumer warps
    pdl_launch_dependents();
    pdl_wait_prior_grid();  // outputs and the fix-up scratch belong to earlier kernels until they complete
    const int g = lane >> 2, t = lane & 3;
    const int rs = warp & 7, ul = warp >> 3;
    const int r0 = 16 * rs + frag_row(g);
    const uint32_t w_first = smem_u32(ws) + (uint32_t)(r0 * PITCH + ul * UB);
    const uint32_t rec_base = smem_u32(ws) + STAGE_W;
    const uint32_t xoff = (uint32_t)(16 * t + 8 * (g & 1));

    float yacc[NT][2];
    uint32_t moff[NT], soff[NT];
    int si = -1, seg_end = 0, chunk = 0, units = 0, M = 1, buf = 0, cut_k = 0;
    uint32_t rec_unit = 0;  // byte offset of this warp's unit inside a stage's records
    int stage = 0;
    uint32_t phase = 0;
    for (int it = 0; it < total_items; ++it) {
        if (it == seg_end) {  // a new piece: its job's row count, fresh accumulators
            ++si;
            const int4 sg = segs[si];
            const WlJob &jb = a.jobs[sg.x];
            M = jb.m;
            units = jb.units;
            chunk = sg.z & 0xFFFF;
            seg_end = sg.w + ((sg.z >> 16) - chunk);
#pragma unroll
            for (int nt = 0; nt < NT; ++nt) {
                int mb = 4 * nt + (g >> 1), ms = 4 * nt + t;  // B column / accumulator column rows, clamped to an existing row
                if (mb > M - 1) mb = M - 1;
                if (ms > M - 1) ms = M - 1;
                moff[nt] = (uint32_t)(mb * kRec);
                soff[nt] = (uint32_t)(ms * kRec);
                yacc[nt][0] = yacc[nt][1] = 0.f;
            }
            rec_unit = (uint32_t)(ul * M * kRec);
        }
        wl_wait(&full[stage], phase, abort_addr, a.status);
        if (chunk * kChunkUnits + ul < units) {
            const uint32_t soffs = (uint32_t)(stage * STRIDE);
            const uint32_t wq0 = w_first + soffs, wq1 = wq0 + 8 * PITCH;
            const uint32_t rb = rec_base + soffs + rec_unit;
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
        ++chunk;
        if (it + 1 == seg_end) {
            // ------------------------------------------------ end of a piece
            const int4 sg = segs[si];
            const WlJob &jb = a.jobs[sg.x];
            const int tile = sg.y, cb = sg.z & 0xFFFF, ce = sg.z >> 16;
            const bool whole = cb == 0 && ce == jb.chunks;  // the whole tile was this CTA's
            float *xb = xch + buf * XCH_FLOATS;
            buf ^= 1;  // a buffer is written again only two pieces later, behind the barrier of the piece in between
            const bool quad = GATED && whole;
            const bool owner = ul == 0 && (!quad || rs < 4);  // the warp that adds up and stores
            if (!owner) {
#pragma unroll
                for (int nt = 0; nt < NT; ++nt) {
                    xb[(warp * 32 + lane) * NACC + 2 * nt] = yacc[nt][0];
                    xb[(warp * 32 + lane) * NACC + 2 * nt + 1] = yacc[nt][1];
                }
            }
            if (quad) named_bar_sync(kBarQuad + (rs & 3), 128);
            else named_bar_sync(kBarPair + rs, 64);
            auto finish = [&](int row, int tok, float v, float vup) {
                const int n = tile * out_rows + row;
                if (n >= jb.n_out || tok >= M) return;
                if (GATED) v = (v / (1.0f + expf(-v))) * vup;
                const size_t o = (size_t)tok * jb.n_out + n;
                if (jb.residual) v += load_as_f32(jb.residual, jb.y_dtype, o);
                store_from_f32(jb.y, jb.y_dtype, o, v);
            };
            if (whole) {
                if (owner) {
#pragma unroll
                    for (int nt = 0; nt < NT; ++nt) {
#pragma unroll
                        for (int h = 0; h < 2; ++h) {  // fragment rows g and g + 8
                            float v = yacc[nt][h] + xb[((warp + 8) * 32 + lane) * NACC + 2 * nt + h], vup = 0.f;
                            if (GATED) vup = xb[((warp + 4) * 32 + lane) * NACC + 2 * nt + h] + xb[((warp + 12) * 32 + lane) * NACC + 2 * nt + h];
                            finish(r0 + 8 * h, 4 * nt + t, v, vup);
                        }
                    }
                }
            } else {
                // a tile cut by a range boundary: leave the partial sums (all 128 rows) in this CTA's slot, count the arrival
                float *slot = a.partials + (size_t)(2 * bid + (cb == 0 ? 1 : 0)) * kSlotFloats;
                if (owner) {
#pragma unroll
                    for (int nt = 0; nt < NT; ++nt) {
                        const int tok = 4 * nt + t;
                        if (tok < M) {
                            slot[tok * kTileRows + r0] = yacc[nt][0] + xb[((warp + 8) * 32 + lane) * NACC + 2 * nt];
                            slot[tok * kTileRows + r0 + 8] = yacc[nt][1] + xb[((warp + 8) * 32 + lane) * NACC + 2 * nt + 1];
                        }
                    }
                }
                if constexpr (kAsyncFix) {
                    named_bar_arrive(kBarFix + cut_k, kWlConsumers + 32);  // over to the finisher warp; this warp goes on
                    ++cut_k;
                } else {
                    __threadfence();
                    named_bar_sync(kBarAll, kWlConsumers);
                    if (tid == 0) {
                        const long long ts = (long long)jb.q_begin + (long long)tile * jb.chunks;
                        const int c0 = wl_owner(ts, G, Q), cl = wl_owner(ts + jb.chunks - 1, G, Q);
                        const uint32_t old = atomicAdd(&a.counters[c0], 1u);
                        s_last = old == (uint32_t)(cl - c0);
                        s_c0 = c0;
                        s_cl = cl;
                    }
                    named_bar_sync(kBarAll, kWlConsumers);
                    if (s_last) {  // every contributor has arrived: add the partials in CTA order
                        __threadfence();
                        const int c0 = s_c0, cl = s_cl;
                        for (int i = tid; i < out_rows * M; i += kWlConsumers) {
                            const int row = i & (out_rows - 1), tok = i / out_rows;
                            float v = 0.f, vup = 0.f;
                            for (int c = c0; c <= cl; ++c) {
                                const float *ps = a.partials + (size_t)(2 * c + (c == c0 ? 1 : 0)) * kSlotFloats + tok * kTileRows;
                                v += __ldcg(ps + row);
                                if (GATED) vup += __ldcg(ps + out_rows + row);
                            }
                            finish(row, tok, v, vup);
                        }
                        if (tid == 0) a.counters[c0] = 0;  // ready for the next launch
                    }
                    named_bar_sync(kBarAll, kWlConsumers);  // s_last may be rewritten by the next cut tile only after everyone read it
                }
            }
        }
    }
}

template <uint32_t TYPE>
static int launch_wl_quantize(zq_ctx *ctx, const WlQuantArgs &qa, zq_error *err) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)((qa.total + 7) / 8));
    cfg.blockDim = dim3(256);
    cfg.stream = ctx->stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = ctx->disable_pdl ? 0 : 1;
    ZQ_CUDA_CHECK(cudaLaunchKernelEx(&cfg, wl_quantize_kernel<TYPE>, qa), err);
    ctx->launches++;
    return ZQ_OK;
}

template <uint32_t TYPE, int NT, bool GATED>
static int launch_wl_one(zq_ctx *ctx, const WlArgs &wa, zq_error *err) {
    using S = WlSmem<TYPE, NT>;
    auto kernel = gemv_wl_kernel<TYPE, NT, GATED>;
    static bool configured[64] = {};
    if (!configured[ctx->device & 63]) {
        ZQ_CUDA_CHECK(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, S::TOTAL), err);
        configured[ctx->device & 63] = true;
    }
    int grid = ctx->sm_count < wa.q_total ? ctx->sm_count : wa.q_total;  // every CTA gets at least one item
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)grid);
    cfg.blockDim = dim3(kWlThreads);
    cfg.dynamicSmemBytes = S::TOTAL;
    cfg.stream = ctx->stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = ctx->disable_pdl ? 0 : 1;
    ZQ_CUDA_CHECK(cudaLaunchKernelEx(&cfg, kernel, wa), err);
    ctx->launches++;
    return ZQ_OK;
}

template <uint32_t TYPE>
static int launch_wl_type(zq_ctx *ctx, const WlArgs &wa, int nt, bool gated, zq_error *err) {
    if (nt == 1) return gated ? launch_wl_one<TYPE, 1, true>(ctx, wa, err) : launch_wl_one<TYPE, 1, false>(ctx, wa, err);
    if (nt == 2) return gated ? launch_wl_one<TYPE, 2, true>(ctx, wa, err) : launch_wl_one<TYPE, 2, false>(ctx, wa, err);
    return gated ? launch_wl_one<TYPE, 4, true>(ctx, wa, err) : launch_wl_one<TYPE, 4, false>(ctx, wa, err);
}

static bool wl_type_ok(uint32_t t) { return t == ZQ_Q4_K || t == ZQ_Q4_0 || t == ZQ_Q8_0 || t == ZQ_IQ4_NL || t == ZQ_Q5_K || t == ZQ_Q6_K; }

bool gemv_wl_supported(const zq_ctx *ctx, const WlHostJob &j) {
    if (!j.w || !j.w->d_maps || !wl_type_ok(j.w->type) || j.m < 1 || j.m > (size_t)kMaxGemvRows) return false;
    if (j.w_up && (!j.w_up->d_maps || j.w_up->type != j.w->type || j.w_up->rows != j.w->rows || j.w_up->cols != j.w->cols)) return false;
    if ((j.w->units_per_row + kChunkUnits - 1) / kChunkUnits > 0xFFFF) return false;
    if ((size_t)2 * ctx->sm_count * kSlotFloats > ctx->gemv_partials_floats || (size_t)ctx->sm_count > ctx->gemv_counters_n) return false;
    return true;
}

// Runs the jobs (all of them supported, see gemv_wl_supported) in as few launches as their classes allow: one record
// pass per record format, then one decode launch per (weight type, column-tile count, plain / gated) class.
int launch_gemv_wl(zq_ctx *ctx, const WlHostJob *jobs, size_t n_jobs, int x_dtype, int y_dtype, zq_error *err) {
    if (n_jobs == 0) return ZQ_OK;
    // ---- records: one block per distinct (x, m, cols, record format)
    struct Src { const void *x; size_t m, cols; bool q4k; size_t rec_begin, units; };
    std::vector<Src> srcs;
    std::vector<size_t> src_of(n_jobs);
    size_t total_rec = 0;
    for (size_t i = 0; i < n_jobs; ++i) {
        const WlHostJob &j = jobs[i];
        const bool q4k = is_kclass(j.w->type);
        size_t s = 0;
        for (; s < srcs.size(); ++s)
            if (srcs[s].x == j.x && srcs[s].m == j.m && srcs[s].cols == j.w->cols && srcs[s].q4k == q4k) break;
        if (s == srcs.size()) {
            srcs.push_back({j.x, j.m, j.w->cols, q4k, total_rec, j.w->units_per_row});
            total_rec += j.m * j.w->units_per_row;
        }
        src_of[i] = s;
    }
    if (total_rec > (size_t)INT32_MAX / kRec) return set_error(err, ZQ_ERR_SHAPE, "decode work list: %zu activation records are too many for one call", total_rec);
    int rc = ensure_xq(ctx, total_rec * kRec, err);
    if (rc) return rc;
    uint8_t *xq = reinterpret_cast<uint8_t *>(ctx->xq);
    for (int cls = 0; cls < 2; ++cls) {
        WlQuantArgs qa;
        qa.x_dtype = x_dtype;
        qa.n_src = 0;
        auto flush = [&]() -> int {
            if (qa.n_src == 0) return ZQ_OK;
            // records of one launch are contiguous: the kernel's record index starts at the first block's
            const int first = qa.src[0].rec_begin;
            qa.out = xq + (size_t)first * kRec;
            for (int s = 0; s < qa.n_src; ++s) qa.src[s].rec_begin -= first;
            qa.total = qa.src[qa.n_src - 1].rec_begin + qa.src[qa.n_src - 1].m * qa.src[qa.n_src - 1].units;
            const int r = cls ? launch_wl_quantize<ZQ_Q4_0>(ctx, qa, err) : launch_wl_quantize<ZQ_Q4_K>(ctx, qa, err);
            qa.n_src = 0;
            return r;
        };
        size_t expect = 0;
        for (const Src &s : srcs) {
            if (s.q4k != (cls == 0)) continue;
            if (qa.n_src == kWlMaxJobs || (qa.n_src && s.rec_begin != expect)) {  // full, or a block of the other class lies between
                if ((rc = flush())) return rc;
            }
            qa.src[qa.n_src++] = {s.x, (int)s.m, (int)s.cols, (int)s.units, (int)s.rec_begin};
            expect = s.rec_begin + s.m * s.units;
        }
        if ((rc = flush())) return rc;
    }
    // ---- decode launches, one per class, in order of first appearance
    std::vector<char> done(n_jobs, 0);
    for (size_t i = 0; i < n_jobs; ++i) {
        if (done[i]) continue;
        const uint32_t type = jobs[i].w->type;
        const int nt = jobs[i].m <= 4 ? 1 : (jobs[i].m <= 8 ? 2 : 4);
        const bool gated = jobs[i].w_up != nullptr;
        WlArgs wa;
        wa.n_jobs = 0;
        wa.q_total = 0;
        wa.chunk_words = kChunkUnits * format_info(type).unit_bytes / 4;
        wa.y_dtype = y_dtype;
        wa.partials = ctx->gemv_partials;
        wa.counters = ctx->gemv_counters;
        wa.status = ctx->status_dev;
        int min_chunks = INT32_MAX;
        auto flush = [&]() -> int {
            if (wa.n_jobs == 0) return ZQ_OK;
            // pieces per CTA: at most one per tile boundary inside a range, plus the two ends
            const int grid = ctx->sm_count < wa.q_total ? ctx->sm_count : wa.q_total;
            const long long per_cta = (wa.q_total + grid - 1) / grid;
            if (per_cta / min_chunks + 3 > kWlMaxSegs) return set_error(err, ZQ_ERR_UNSUPPORTED, "decode work list: a CTA would walk more than %d tiles", kWlMaxSegs);
            int r;
            switch (type) {
            case ZQ_Q4_K: r = launch_wl_type<ZQ_Q4_K>(ctx, wa, nt, gated, err); break;
            case ZQ_Q5_K: r = launch_wl_type<ZQ_Q5_K>(ctx, wa, nt, gated, err); break;
            case ZQ_Q6_K: r = launch_wl_type<ZQ_Q6_K>(ctx, wa, nt, gated, err); break;
            case ZQ_Q4_0: r = launch_wl_type<ZQ_Q4_0>(ctx, wa, nt, gated, err); break;
            case ZQ_IQ4_NL: r = launch_wl_type<ZQ_IQ4_NL>(ctx, wa, nt, gated, err); break;
            default: r = launch_wl_type<ZQ_Q8_0>(ctx, wa, nt, gated, err); break;
            }
            wa.n_jobs = 0;
            wa.q_total = 0;
            min_chunks = INT32_MAX;
            return r;
        };
        for (size_t k = i; k < n_jobs; ++k) {
            const WlHostJob &j = jobs[k];
            const int nt_k = j.m <= 4 ? 1 : (j.m <= 8 ? 2 : 4);
            if (done[k] || j.w->type != type || nt_k != nt || (j.w_up != nullptr) != gated) continue;
            done[k] = 1;
            const int rows_per_tile = gated ? kTileRows / 2 : kTileRows;
            const long long tiles = (long long)((j.w->rows + rows_per_tile - 1) / rows_per_tile);
            const long long chunks = (long long)((j.w->units_per_row + kChunkUnits - 1) / kChunkUnits);
            if (wa.n_jobs == kWlMaxJobs || (long long)wa.q_total + tiles * chunks > (long long)INT32_MAX / 512) {
                if ((rc = flush())) return rc;
            }
            WlJob &d = wa.jobs[wa.n_jobs++];
            d.map_a = j.w->d_maps + (gated ? 1 : 0);
            d.map_b = gated ? j.w_up->d_maps + 1 : d.map_a;
            d.xq = xq + srcs[src_of[k]].rec_begin * kRec;
            d.y = j.y;
            d.residual = j.residual;
            d.m = (int)j.m;
            d.n_out = (int)j.w->rows;
            d.units = (int)j.w->units_per_row;
            d.chunks = (int)chunks;
            d.tiles = (int)tiles;
            d.q_begin = wa.q_total;
            d.y_dtype = j.y_dtype >= 0 ? j.y_dtype : y_dtype;
            d.pad = 0;
            wa.q_total += (int)(tiles * chunks);
            if ((int)chunks < min_chunks) min_chunks = (int)chunks;
        }
        if ((rc = flush())) return rc;
    }
    return ZQ_OK;
}

}  // namespace zq
