// MoE decode: all routed experts of a layer in two launches (gate/up + SiLU, then down), no host round trip.
//
// The per-expert form (zq_moe.cu) copies the router's ids to the host, groups them there and launches two decode
// kernels per routed expert: at 64 tokens x top-8 over 256 experts that is ~450 launches of ~10 us each and a
// pipeline drain between every pair.  Here the device does the grouping and ONE persistent kernel per projection
// walks every (expert, 8-row pass, row tile) of the layer, so the TMA ring never drains between experts:
//   moe_plan_kernel        counts, offsets, token-major stable slots (src/moe/routing.rs:136-156), per-token combine
//                          order (ascending expert id, src/backend/cpu/moe.rs:107-141), list of (expert, pass)
//   moe_quantize_kernel    activation records (zq_i8.cuh) of every routed row, grouped by expert
//   moe_grouped_kernel     integer-MMA decode over the work list; CTA c takes items c, c + grid, ...; every ring
//                          stage carries the weights of one (tile, 2 units) and the records of those units
// Arithmetic per expert is that of zq_gemv_i8.cu (16-bit integer activations, exact integer weights), the combine
// is the one of zq_moe.cu; an expert that received more than 8 rows is walked in passes of 8.
#include <cstring>

#include "zq_i8.cuh"
#include "zq_moe.cuh"

namespace zq {

constexpr int kPassRows = 8;                    // activation rows per pass (two column tiles)
constexpr int kPassUnitBytes = kPassRows * kRec;  // record slot of one unit inside a ring stage
constexpr int kItemCache = 512;                 // work items whose descriptors a CTA keeps in shared memory
constexpr int kPlanThreads = 1024;
constexpr int kGroupedThreads = kI8Threads + 32;  // 16 consumer warps and a TMA producer warp
// ring depth: the wide Q8_0 rows leave room for two stages only
__host__ __device__ constexpr int grouped_stages(uint32_t type) { return type == ZQ_Q8_0 ? 2 : (type == ZQ_Q5_K || type == ZQ_Q6_K) ? 3 : 4; }

// ---------------------------------------------------------------------------------------------------------------
// Plan: one CTA.  ids/weights are the router's [m, top_k] outputs.
//   offsets[e]        first slot of expert e (slots of an expert are in token order)
//   slot_token[s]     token whose row sits in slot s;  slot_expert[s] its expert
//   token_slots/w     per token, its top_k slots and weights in ascending expert order
//   passes[p]         {expert, m0 | rows << 16, first slot of the expert, rows of the expert}; a shared expert that
//                     rides along is expert E with one row per token in slots routes .. routes + m - 1
// ---------------------------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(kPlanThreads) moe_plan_kernel(const uint32_t *__restrict__ ids, const float *__restrict__ wts, int m, int top_k, int E, uint32_t *__restrict__ offsets, uint32_t *__restrict__ slot_token,
                                                                 uint32_t *__restrict__ slot_expert, uint32_t *__restrict__ token_slots, float *__restrict__ token_w, uint4 *__restrict__ passes, uint32_t *__restrict__ n_pass,
                                                                 int shared_rows, uint32_t *status) {
    extern __shared__ uint32_t plan_smem[];
    const int routes = m * top_k;
    uint32_t *s_cnt = plan_smem;            // [E]
    uint32_t *s_off = s_cnt + E;            // [E + 1]
    uint32_t *s_ids = s_off + E + 1;        // [routes]
    uint32_t *s_slot = s_ids + routes;      // [routes]
    pdl_launch_dependents();
    pdl_wait_prior_grid();
    for (int e = threadIdx.x; e < E; e += kPlanThreads) s_cnt[e] = 0;
    __syncthreads();
    for (int r = threadIdx.x; r < routes; r += kPlanThreads) {
        uint32_t id = ids[r];
        if (id == ZQ_MOE_NO_ROUTE) {  // an absent route: no slot, no expert work, weight 0 in the combine
            s_ids[r] = (uint32_t)E;
            s_slot[r] = 0;
            continue;
        }
        if (id >= (uint32_t)E) {  // never index out of the table: record it and park the route on the last expert
            atomicMax(status, (uint32_t)kStatusBadIndex);
            id = (uint32_t)E - 1;
        }
        s_ids[r] = id;
        atomicAdd(&s_cnt[id], 1u);
    }
    __syncthreads();
    {
        // exclusive prefix sums over the experts (E <= 1024 = one thread each): slot offsets and pass offsets
        __shared__ uint32_t warp_tot[2][32];
        const int e = threadIdx.x, lane = e & 31, wid = e >> 5;
        const uint32_t c = e < E ? s_cnt[e] : 0u;
        const uint32_t np_e = (c + kPassRows - 1) / kPassRows;
        uint32_t sc = c, sp = np_e;
#pragma unroll
        for (int d = 1; d < 32; d <<= 1) {
            const uint32_t a = __shfl_up_sync(0xffffffffu, sc, d), b = __shfl_up_sync(0xffffffffu, sp, d);
            if (lane >= d) {
                sc += a;
                sp += b;
            }
        }
        if (lane == 31) {
            warp_tot[0][wid] = sc;
            warp_tot[1][wid] = sp;
        }
        __syncthreads();
        uint32_t base_c = 0, base_p = 0;
        for (int w = 0; w < wid; ++w) {
            base_c += warp_tot[0][w];
            base_p += warp_tot[1][w];
        }
        const uint32_t first = base_c + sc - c, pfirst = base_p + sp - np_e;
        if (e < E) {
            s_off[e] = first;
            offsets[e] = first;
            for (uint32_t j = 0; j < np_e; ++j) {
                const uint32_t m0 = j * kPassRows, mc = c - m0 < (uint32_t)kPassRows ? c - m0 : (uint32_t)kPassRows;
                passes[pfirst + j] = make_uint4((uint32_t)e, m0 | (mc << 16), first, c);
            }
        }
        if (e == kPlanThreads - 1) {  // the last thread holds the totals
            s_off[E] = base_c + sc;
            offsets[E] = base_c + sc;
            // the shared expert, when it rides along: id E, every token one row, slots right behind the routed ones
            uint32_t np = base_p + sp;
            for (uint32_t m0 = 0; m0 < (uint32_t)shared_rows; m0 += kPassRows) {
                const uint32_t mc = (uint32_t)shared_rows - m0 < (uint32_t)kPassRows ? (uint32_t)shared_rows - m0 : (uint32_t)kPassRows;
                passes[np++] = make_uint4((uint32_t)E, m0 | (mc << 16), (uint32_t)routes, (uint32_t)shared_rows);  // behind ALL route places, absent ones included
            }
            *n_pass = np;
        }
    }
    __syncthreads();
    // token-major stable slots
    if (routes <= 2048) {
        // few routes (decode): every route counts the earlier routes of its expert itself: independent compares, no
        // serial walk (a quarter of the time of the walk below at 512 routes)
        for (int r = threadIdx.x; r < routes; r += kPlanThreads) {
            const uint32_t id = s_ids[r];
            if (id == (uint32_t)E) continue;
            uint32_t before = 0;
            int r2 = 0;
            for (; r2 + 4 <= r; r2 += 4) before += (s_ids[r2] == id) + (s_ids[r2 + 1] == id) + (s_ids[r2 + 2] == id) + (s_ids[r2 + 3] == id);
            for (; r2 < r; ++r2) before += s_ids[r2] == id;
            const uint32_t slot = s_off[id] + before;
            slot_token[slot] = (uint32_t)(r / top_k);
            slot_expert[slot] = id;
            s_slot[r] = slot;
        }
    } else {
        // many routes: the thread of expert e walks the routes in order
        for (int e = threadIdx.x; e < E; e += kPlanThreads) {
            if (s_cnt[e] == 0) continue;
            uint32_t slot = s_off[e];
            for (int r = 0; r < routes; ++r) {
                if (s_ids[r] == (uint32_t)e) {
                    slot_token[slot] = (uint32_t)(r / top_k);
                    slot_expert[slot] = (uint32_t)e;
                    s_slot[r] = slot++;
                }
            }
        }
    }
    __syncthreads();
    // per-token combine order: ascending expert id, stable for repeated ids (insertion sort of <= 64 entries)
    for (int t = threadIdx.x; t < m; t += kPlanThreads) {
        uint32_t ke[64], ks[64];
        float kw[64];
        for (int j = 0; j < top_k; ++j) {
            const uint32_t e = s_ids[t * top_k + j], s = s_slot[t * top_k + j];
            const float w = e == (uint32_t)E ? 0.f : wts[t * top_k + j];
            int i = j;
            while (i > 0 && ke[i - 1] > e) {
                ke[i] = ke[i - 1]; ks[i] = ks[i - 1]; kw[i] = kw[i - 1];
                --i;
            }
            ke[i] = e; ks[i] = s; kw[i] = w;
        }
        for (int j = 0; j < top_k; ++j) {
            token_slots[t * top_k + j] = ks[j];
            token_w[t * top_k + j] = kw[j];
        }
    }
}

// Records of every routed row: one warp per (slot, unit).  Record index of (expert e, unit u, local row j) is
// offsets[e] * units + u * count_e + j, so the rows of one pass of one unit are contiguous.
// row_of_slot: source row per routed slot (token of the slot), or null when the source is already in slot order.
template <uint32_t TYPE>
__global__ void __launch_bounds__(256) moe_quantize_kernel(const void *__restrict__ src, int src_dtype, const uint32_t *__restrict__ row_of_slot, const uint32_t *__restrict__ slot_expert,
                                                           const uint32_t *__restrict__ offsets, int routes, int shared_rows, int shared_id, int num_experts, int cols, int units, uint8_t *__restrict__ out) {
    pdl_launch_dependents();
    pdl_wait_prior_grid();
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int task = blockIdx.x * 8 + warp;
    if (task >= (routes + shared_rows) * units) return;  // warp-uniform
    const int slot = task / units, unit = task - slot * units;
    uint32_t first, cnt;
    size_t row;
    if (slot < routes) {
        if ((uint32_t)slot >= offsets[num_experts]) return;  // absent routes take no slot: nothing lives behind the last expert's rows
        const uint32_t e = slot_expert[slot];
        first = offsets[e];
        cnt = offsets[e + 1] - first;
        row = row_of_slot ? row_of_slot[slot] : (uint32_t)slot;
    } else {  // shared expert: slot routes + t holds token t
        (void)shared_id;
        first = (uint32_t)routes;
        cnt = (uint32_t)shared_rows;
        row = row_of_slot ? (size_t)(slot - routes) : (size_t)slot;
    }
    const size_t rec = (size_t)first * units + (size_t)unit * cnt + ((uint32_t)slot - first);
    const int k0 = unit * kUnitWeights + 8 * lane;
    float v[8];
    load_act8(src, src_dtype, row * cols + k0, k0 < cols, v);
    const RecLane o = quantize_record<TYPE>(v, lane);
    uint8_t *dst = out + rec * kRec;
    *reinterpret_cast<uint4 *>(dst + o.slot) = make_uint4(o.ph0, o.ph1, o.pl0, o.pl1);
    if (is_kclass(TYPE) && (lane & 7) == 0) *reinterpret_cast<uint2 *>(dst + kRecSums + (lane >> 3) * 8) = make_uint2(o.sw0, o.sw1);
    if (lane == 0) *reinterpret_cast<float *>(dst + kRecScale) = o.scale;
}

struct GroupedArgs {
    const CUtensorMap *maps_a;  // per expert: gate (64-row boxes) or down (128-row boxes)
    const CUtensorMap *maps_b;  // per expert: up (gated only)
    const uint4 *passes;
    const uint32_t *n_pass;
    const uint8_t *xq;          // records, grouped by expert
    float *out;                 // [slot, n_out] f32
    uint32_t *status;
    int units, chunks, chunk_words;
    int tiles;                  // row tiles per expert
    int n_out;                  // output features per expert (rows of gate, or of down)
    int shared_id;              // expert id that means "the shared expert" (its maps are below), or -1
    CUtensorMap shared_a, shared_b;
};

template <uint32_t TYPE, bool GATED>
__global__ void __launch_bounds__(kGroupedThreads, 1) moe_grouped_kernel(const __grid_constant__ GroupedArgs ga) {
    constexpr int UB = Fmt<TYPE>::unit_bytes;
    constexpr int PITCH = kChunkUnits * UB;
    constexpr int STAGE_W = kTileRows * PITCH;
    constexpr int STRIDE = STAGE_W + kChunkUnits * kPassUnitBytes;
    constexpr int STAGES = grouped_stages(TYPE);
    constexpr int RS = kPassRows;                     // activation rows a tile row can hold
    constexpr int RED_FLOATS = 2 * RS * kTileRows;    // [unit half][activation row][tile row]
    constexpr int out_rows = GATED ? kTileRows / 2 : kTileRows;
    extern __shared__ uint8_t smem_raw[];
    uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 127) & ~uintptr_t(127));
    uint8_t *ws = smem;
    float *red = reinterpret_cast<float *>(smem + STAGES * STRIDE);           // two buffers, alternating per item
    uint4 *s_pass = reinterpret_cast<uint4 *>(smem + STAGES * STRIDE + 2 * RED_FLOATS * 4);
    uint64_t *full = reinterpret_cast<uint64_t *>(smem + STAGES * STRIDE + 2 * RED_FLOATS * 4 + kItemCache * 16);
    uint64_t *empty = full + 8;
    __shared__ int s_abort;

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int G = gridDim.x, bid = blockIdx.x;
    pdl_launch_dependents();
    pdl_wait_prior_grid();  // the work list, the records and (for the down projection) nothing else precede this kernel
    const int n_items = (int)(*ga.n_pass) * ga.tiles;
    const int my_count = n_items > bid ? (n_items - bid + G - 1) / G : 0;
    const int chunks = ga.chunks;
    const long long total_q = (long long)my_count * chunks;

    for (int k = tid; k < my_count && k < kItemCache; k += kI8Threads) s_pass[k] = ga.passes[(bid + k * G) / ga.tiles];
    if (tid == 0) {
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(&full[s], 1);
            mbar_init(&empty[s], kI8Threads / 32);
        }
        fence_mbar_init();
        s_abort = 0;
    }
    __syncthreads();
    auto pass_of = [&](int k) -> uint4 { return k < kItemCache ? s_pass[k] : ga.passes[(bid + k * G) / ga.tiles]; };

    // ring item q = (k-th work item of this CTA, chunk): weights of the tile's two units and their records
    auto issue = [&](long long q, int stage) {
        const int k = (int)(q / chunks), chunk = (int)(q - (long long)k * chunks);
        const int tile = (bid + k * G) % ga.tiles;
        const uint4 pe = pass_of(k);
        const uint32_t e = pe.x, m0 = pe.y & 0xFFFFu, mc = pe.y >> 16, first = pe.z, cnt = pe.w;
        int nu = ga.units - chunk * kChunkUnits;
        if (nu > kChunkUnits) nu = kChunkUnits;
        uint8_t *dst = ws + (size_t)stage * STRIDE;
        mbar_expect_tx(&full[stage], (uint32_t)(STAGE_W + nu * mc * kRec));
        const bool sh = (int)e == ga.shared_id;
        const CUtensorMap *ma = sh ? &ga.shared_a : &ga.maps_a[e];
        if (GATED) {
            const CUtensorMap *mb = sh ? &ga.shared_b : &ga.maps_b[e];
            tma_load_2d(dst, ma, &full[stage], chunk * ga.chunk_words, tile * out_rows);
            tma_load_2d(dst + STAGE_W / 2, mb, &full[stage], chunk * ga.chunk_words, tile * out_rows);
        } else {
            tma_load_2d(dst, ma, &full[stage], chunk * ga.chunk_words, tile * out_rows);
        }
        for (int u = 0; u < nu; ++u) {
            const size_t rec = (size_t)first * ga.units + (size_t)(chunk * kChunkUnits + u) * cnt + m0;
            bulk_load_1d(dst + STAGE_W + u * kPassUnitBytes, ga.xq + rec * kRec, mc * kRec, &full[stage]);
        }
    };
    if (warp == kI8Threads / 32) {
        // ------------------------------------------------ producer warp: keeps the ring full; a stage is refilled as soon
        // as all sixteen consumer warps have released it, whichever of them is late
        if (lane == 0) {
            int pstage = 0;
            uint32_t pphase = 0;
            for (long long q = 0; q < total_q; ++q) {
                if (q >= STAGES) i8_wait_or_abort(&empty[pstage], pphase ^ 1u, &s_abort, ga.status);
                if (*(volatile int *)&s_abort) break;  // never start a copy nobody will wait for
                issue(q, pstage);
                if (++pstage == STAGES) {
                    pstage = 0;
                    pphase ^= 1u;
                }
            }
        }
        return;
    }

    const int g = lane >> 2, t = lane & 3;
    const int rs = warp & 7, ul = warp >> 3;
    const int r0 = 16 * rs + frag_row(g);
    const uint32_t w_first = smem_u32(ws) + (uint32_t)(r0 * PITCH + ul * UB);
    const uint32_t rec_first = smem_u32(ws) + STAGE_W + (uint32_t)(ul * kPassUnitBytes);
    const uint32_t xoff = (uint32_t)(16 * t + 8 * (g & 1));

    float yacc1[1][2], yacc2[2][2];
    uint32_t moff[2] = {0, 0}, soff[2] = {0, 0};
    int mc = 0, chunk = 0, k = 0, stage = 0, buf = 0;
    uint32_t phase = 0;
    for (long long q = 0; q < total_q; ++q) {
        if (chunk == 0) {  // a new work item: rows of this pass, accumulators
            const uint4 pe = pass_of(k);
            mc = (int)(pe.y >> 16);
#pragma unroll
            for (int nt = 0; nt < 2; ++nt) {
                int mb = 4 * nt + (g >> 1), ms = 4 * nt + t;
                if (mb > mc - 1) mb = mc - 1;
                if (ms > mc - 1) ms = mc - 1;
                moff[nt] = (uint32_t)(mb * kRec);
                soff[nt] = (uint32_t)(ms * kRec);
            }
            yacc1[0][0] = yacc1[0][1] = 0.f;
            yacc2[0][0] = yacc2[0][1] = yacc2[1][0] = yacc2[1][1] = 0.f;
        }
        i8_wait_or_abort(&full[stage], phase, &s_abort, ga.status);
        if (chunk * kChunkUnits + ul < ga.units) {
            const uint32_t soffs = (uint32_t)(stage * STRIDE);
            const uint32_t wq0 = w_first + soffs, wq1 = wq0 + 8 * PITCH;
            const uint32_t rb = rec_first + soffs;
            if (mc <= 4) {
                const uint32_t rec[1] = {rb + moff[0]}, srec[1] = {rb + soff[0]};
                if constexpr (TYPE == ZQ_Q6_K) consume_q6k_i8<1>(wq0, wq1, t, rec, srec, xoff, yacc1);
                else if constexpr (is_kclass(TYPE)) consume_q4k_i8<1, TYPE == ZQ_Q5_K>(wq0, wq1, t, rec, srec, xoff, yacc1);
                else consume_b32_i8<TYPE, 1>(wq0, wq1, t, rec, srec, xoff, yacc1);
            } else {
                const uint32_t rec[2] = {rb + moff[0], rb + moff[1]}, srec[2] = {rb + soff[0], rb + soff[1]};
                if constexpr (TYPE == ZQ_Q6_K) consume_q6k_i8<2>(wq0, wq1, t, rec, srec, xoff, yacc2);
                else if constexpr (is_kclass(TYPE)) consume_q4k_i8<2, TYPE == ZQ_Q5_K>(wq0, wq1, t, rec, srec, xoff, yacc2);
                else consume_b32_i8<TYPE, 2>(wq0, wq1, t, rec, srec, xoff, yacc2);
            }
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(&empty[stage]);
        if (++stage == STAGES) {
            stage = 0;
            phase ^= 1u;
        }
        if (++chunk == chunks) {
            // ------------------------------------------------ end of the work item: add the two unit halves, store
            float *rb_ = red + buf * RED_FLOATS;
            if (mc <= 4) {
                rb_[(ul * RS + t) * kTileRows + r0] = yacc1[0][0];
                rb_[(ul * RS + t) * kTileRows + r0 + 8] = yacc1[0][1];
            } else {
#pragma unroll
                for (int nt = 0; nt < 2; ++nt) {
                    rb_[(ul * RS + nt * 4 + t) * kTileRows + r0] = yacc2[nt][0];
                    rb_[(ul * RS + nt * 4 + t) * kTileRows + r0 + 8] = yacc2[nt][1];
                }
            }
            asm volatile("bar.sync 1, %0;" ::"n"(kI8Threads) : "memory");  // the consumer warps only; the other buffer is written next item, and read only after that item's barrier
            const uint4 pe = pass_of(k);
            const int tile = (bid + k * G) % ga.tiles;
            const size_t slot0 = (size_t)pe.z + (pe.y & 0xFFFFu);
            for (int i = tid; i < out_rows * mc; i += kI8Threads) {
                const int row = i & (out_rows - 1), tok = i / out_rows;
                const int n = tile * out_rows + row;
                if (n >= ga.n_out) continue;
                float v;
                if (GATED) {
                    const float gate = rb_[tok * kTileRows + row] + rb_[(RS + tok) * kTileRows + row];
                    const float up = rb_[tok * kTileRows + out_rows + row] + rb_[(RS + tok) * kTileRows + out_rows + row];
                    v = (gate / (1.0f + expf(-gate))) * up;
                } else {
                    v = rb_[tok * kTileRows + row] + rb_[(RS + tok) * kTileRows + row];
                }
                ga.out[(slot0 + tok) * ga.n_out + n] = v;
            }
            buf ^= 1;
            chunk = 0;
            ++k;
        }
    }
}

template <uint32_t TYPE>
static int launch_quantize(zq_ctx *ctx, const void *src, int src_dtype, const uint32_t *row_of_slot, const uint32_t *slot_expert, const uint32_t *offsets, size_t routes, size_t shared_rows, int shared_id, int num_experts,
                           size_t cols, size_t units, uint8_t *out, zq_error *err) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)(((routes + shared_rows) * units + 7) / 8));
    cfg.blockDim = dim3(256);
    cfg.stream = ctx->stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = ctx->disable_pdl ? 0 : 1;
    ZQ_CUDA_CHECK(cudaLaunchKernelEx(&cfg, moe_quantize_kernel<TYPE>, src, src_dtype, row_of_slot, slot_expert, offsets, (int)routes, (int)shared_rows, shared_id, num_experts, (int)cols, (int)units, out), err);
    ZQ_CUDA_CHECK(cudaGetLastError(), err);
    ctx->launches++;
    return ZQ_OK;
}

template <uint32_t TYPE, bool GATED>
static int launch_grouped(zq_ctx *ctx, const GroupedArgs &ga, zq_error *err) {
    constexpr int STAGE_W = kTileRows * kChunkUnits * Fmt<TYPE>::unit_bytes;
    constexpr int STRIDE = STAGE_W + kChunkUnits * kPassUnitBytes;
    constexpr int smem = grouped_stages(TYPE) * STRIDE + 2 * (2 * kPassRows * kTileRows) * 4 + kItemCache * 16 + 128 + 128;
    static_assert(smem <= 232448 - 256, "grouped MoE kernel: ring does not fit");
    auto kernel = moe_grouped_kernel<TYPE, GATED>;
    static bool configured[64] = {};
    if (!configured[ctx->device & 63]) {
        ZQ_CUDA_CHECK(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem), err);
        configured[ctx->device & 63] = true;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)ctx->sm_count);
    cfg.blockDim = dim3(kGroupedThreads);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = ctx->stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = ctx->disable_pdl ? 0 : 1;
    ZQ_CUDA_CHECK(cudaLaunchKernelEx(&cfg, kernel, ga), err);
    ZQ_CUDA_CHECK(cudaGetLastError(), err);
    ctx->launches++;
    return ZQ_OK;
}

bool moe_grouped_supported(const zq_moe_experts *t, size_t m, size_t top_k) {
    auto ok_type = [](uint32_t ty) { return has_i8_decode(ty); };
    const size_t routes = m * top_k;
    return t->d_gate_maps && ok_type(t->gate_type) && ok_type(t->down_type) && t->num_experts <= 1024 && top_k <= 64 && routes <= 8192 && (t->num_experts * 2 + 1 + routes * 2) * 4 <= 200 * 1024 &&
           t->inter % 64 == 0;
}

// Device-side sizes of the buffers the grouped path wants inside the MoE workspace.
size_t moe_grouped_ws_bytes(const zq_moe_experts *t, size_t m, size_t top_k, bool has_shared) {
    auto al = [](size_t v) { return (v + 255) & ~size_t(255); };
    const size_t routes = m * top_k, E = t->num_experts, H = t->hidden, I = t->inter;
    const size_t rows = routes + (has_shared ? m : 0);  // a shared expert may ride along as m more rows, or use its own buffer
    const size_t units_h = (H + kUnitWeights - 1) / kUnitWeights, units_i = (I + kUnitWeights - 1) / kUnitWeights;
    return al((E + 1) * 4) + 4 * al(routes * 4) + al((E + rows) * 16) + al(256) + al(rows * units_h * kRec) + al(rows * I * 4) + al(rows * units_i * kRec) + al(rows * H * 4) + (has_shared ? al(m * H * 4) : 0);
}

// The shared expert can ride along in the grouped launches when it looks like one more routed expert.
bool moe_shared_rides_along(const zq_moe_experts *t, const zq_weight *sg, const zq_weight *su, const zq_weight *sd) {
    return sg && su && sd && sg->type == t->gate_type && su->type == t->gate_type && sd->type == t->down_type && sg->rows == t->inter && su->rows == t->inter && sg->cols == t->hidden && su->cols == t->hidden &&
           sd->rows == t->hidden && sd->cols == t->inter;
}

// Routed experts of a layer for a decode-sized batch; `ws` holds moe_grouped_ws_bytes().  Leaves the per-slot expert
// outputs [routes, H] and the per-token combine tables in the workspace and reports where.
// `shared_*`: a shared expert that rides along (moe_shared_rides_along), or null; its output rows then follow the routed
// ones and *shared_buf points at them, otherwise *shared_buf is a separate [m, H] buffer for the caller to fill.
int moe_grouped_forward(zq_ctx *ctx, const zq_moe_experts *t, const zq_weight *shared_gate, const zq_weight *shared_up, const zq_weight *shared_down, const void *dev_x, int x_dtype, size_t m, const uint32_t *dev_ids,
                        const float *dev_weights, size_t top_k, uint8_t *ws, float **routed_out, uint32_t **token_slots_out, float **token_w_out, float **shared_buf, bool has_shared, zq_error *err) {
    auto al = [](size_t v) { return (v + 255) & ~size_t(255); };
    const size_t routes = m * top_k, E = t->num_experts, H = t->hidden, I = t->inter;
    const bool rides = shared_gate != nullptr;
    const size_t srows = rides ? m : 0, rows = routes + (has_shared ? m : 0);
    const int shared_id = rides ? (int)E : -1;
    const size_t units_h = (H + kUnitWeights - 1) / kUnitWeights, units_i = (I + kUnitWeights - 1) / kUnitWeights;
    size_t o = 0;
    uint32_t *d_offsets = reinterpret_cast<uint32_t *>(ws + o); o += al((E + 1) * 4);
    uint32_t *d_slot_token = reinterpret_cast<uint32_t *>(ws + o); o += al(routes * 4);
    uint32_t *d_slot_expert = reinterpret_cast<uint32_t *>(ws + o); o += al(routes * 4);
    uint32_t *d_token_slots = reinterpret_cast<uint32_t *>(ws + o); o += al(routes * 4);
    float *d_token_w = reinterpret_cast<float *>(ws + o); o += al(routes * 4);
    uint4 *d_passes = reinterpret_cast<uint4 *>(ws + o); o += al((E + rows) * 16);
    uint32_t *d_npass = reinterpret_cast<uint32_t *>(ws + o); o += al(256);
    uint8_t *d_xq1 = ws + o; o += al(rows * units_h * kRec);
    float *d_act = reinterpret_cast<float *>(ws + o); o += al(rows * I * 4);
    uint8_t *d_xq2 = ws + o; o += al(rows * units_i * kRec);
    float *d_out = reinterpret_cast<float *>(ws + o); o += al(rows * H * 4);
    *shared_buf = rides ? d_out + routes * H : (has_shared ? reinterpret_cast<float *>(ws + o) : nullptr);
    *routed_out = d_out;
    *token_slots_out = d_token_slots;
    *token_w_out = d_token_w;

    {
        static bool configured[64] = {};
        if (!configured[ctx->device & 63]) {
            ZQ_CUDA_CHECK(cudaFuncSetAttribute(moe_plan_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024), err);
            configured[ctx->device & 63] = true;
        }
        const size_t smem = (E * 2 + 1 + routes * 2) * 4;
        moe_plan_kernel<<<1, kPlanThreads, smem, ctx->stream>>>(dev_ids, dev_weights, (int)m, (int)top_k, (int)E, d_offsets, d_slot_token, d_slot_expert, d_token_slots, d_token_w, d_passes, d_npass, (int)srows, ctx->status_dev);
        ctx->launches++;
        ZQ_CUDA_CHECK(cudaGetLastError(), err);
    }
    int rc;
    // ---- gate/up + SiLU
    // two record formats: the K-quant column order with group sums, and the block-32 order
    if (is_kclass(t->gate_type)) rc = launch_quantize<ZQ_Q4_K>(ctx, dev_x, x_dtype, d_slot_token, d_slot_expert, d_offsets, routes, srows, shared_id, (int)E, H, units_h, d_xq1, err);
    else rc = launch_quantize<ZQ_Q4_0>(ctx, dev_x, x_dtype, d_slot_token, d_slot_expert, d_offsets, routes, srows, shared_id, (int)E, H, units_h, d_xq1, err);
    if (rc) return rc;
    GroupedArgs ga;
    ga.maps_a = t->d_gate_maps;
    ga.maps_b = t->d_up_maps;
    ga.passes = d_passes;
    ga.n_pass = d_npass;
    ga.xq = d_xq1;
    ga.out = d_act;
    ga.status = ctx->status_dev;
    ga.units = (int)units_h;
    ga.chunks = (int)((units_h + kChunkUnits - 1) / kChunkUnits);
    ga.chunk_words = kChunkUnits * format_info(t->gate_type).unit_bytes / 4;
    ga.tiles = (int)((I + kTileRows / 2 - 1) / (kTileRows / 2));
    ga.n_out = (int)I;
    ga.shared_id = shared_id;
    if (rides) {
        ga.shared_a = shared_gate->gemv_map_half;
        ga.shared_b = shared_up->gemv_map_half;
    } else {
        memset(&ga.shared_a, 0, sizeof(CUtensorMap));
        memset(&ga.shared_b, 0, sizeof(CUtensorMap));
    }
    switch (t->gate_type) {
    case ZQ_Q4_K: rc = launch_grouped<ZQ_Q4_K, true>(ctx, ga, err); break;
    case ZQ_Q5_K: rc = launch_grouped<ZQ_Q5_K, true>(ctx, ga, err); break;
    case ZQ_Q6_K: rc = launch_grouped<ZQ_Q6_K, true>(ctx, ga, err); break;
    case ZQ_Q4_0: rc = launch_grouped<ZQ_Q4_0, true>(ctx, ga, err); break;
    case ZQ_IQ4_NL: rc = launch_grouped<ZQ_IQ4_NL, true>(ctx, ga, err); break;
    default: rc = launch_grouped<ZQ_Q8_0, true>(ctx, ga, err); break;
    }
    if (rc) return rc;
    // ---- down
    if (is_kclass(t->down_type)) rc = launch_quantize<ZQ_Q4_K>(ctx, d_act, ZQ_F32, nullptr, d_slot_expert, d_offsets, routes, srows, shared_id, (int)E, I, units_i, d_xq2, err);
    else rc = launch_quantize<ZQ_Q4_0>(ctx, d_act, ZQ_F32, nullptr, d_slot_expert, d_offsets, routes, srows, shared_id, (int)E, I, units_i, d_xq2, err);
    if (rc) return rc;
    ga.maps_a = t->d_down_maps;
    ga.maps_b = t->d_down_maps;
    ga.xq = d_xq2;
    ga.out = d_out;
    ga.units = (int)units_i;
    ga.chunks = (int)((units_i + kChunkUnits - 1) / kChunkUnits);
    ga.chunk_words = kChunkUnits * format_info(t->down_type).unit_bytes / 4;
    ga.tiles = (int)((H + kTileRows - 1) / kTileRows);
    ga.n_out = (int)H;
    if (rides) {
        ga.shared_a = shared_down->gemv_map;
        ga.shared_b = shared_down->gemv_map;
    }
    switch (t->down_type) {
    case ZQ_Q4_K: rc = launch_grouped<ZQ_Q4_K, false>(ctx, ga, err); break;
    case ZQ_Q5_K: rc = launch_grouped<ZQ_Q5_K, false>(ctx, ga, err); break;
    case ZQ_Q6_K: rc = launch_grouped<ZQ_Q6_K, false>(ctx, ga, err); break;
    case ZQ_Q4_0: rc = launch_grouped<ZQ_Q4_0, false>(ctx, ga, err); break;
    case ZQ_IQ4_NL: rc = launch_grouped<ZQ_IQ4_NL, false>(ctx, ga, err); break;
    default: rc = launch_grouped<ZQ_Q8_0, false>(ctx, ga, err); break;
    }
    return rc;
}

}  // namespace zq
