// Decode GEMV on the integer tensor-core path (mma.sync m16n8k32, u8/s8 x s8 -> s32).
//
// Why integers: the packed weights ARE small integers.  Turning a 32-bit word of nibbles into an MMA operand costs
// one AND per four weights here (the low nibbles as they are, the high nibbles left in place as 16 q), against an
// AND-OR plus a scaled half-precision FMA per two weights on the f16 path, and one MMA covers a whole 32-weight
// scale group, so the group's scale is applied once to the s32 accumulator instead of to every operand pair.
// That cuts the instruction count per weight to under a third, which is what bounds these kernels.
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
// Everything up to the final scale is exact integer arithmetic; the result differs from the f32 reference only by
// the 2^-16 activation resolution and f32 rounding of the per-unit terms.
//
// Structure (ring of TMA stages, one CTA per 128-row tile and K slice, cluster reduction through distributed
// shared memory, bounded waits) is that of zq_gemv_resident.cu; up to 16 activation rows go in one pass.
#include "zq_gemv_frag.cuh"

namespace zq {

constexpr int kI8Threads = 512;
constexpr float kActMax = 32512.f;  // 127 * 256

struct I8Args {
    int stages;       // 2..5 ring stages
    int split;        // CTAs per tile (cluster size): 1, 2, 4 or 8
    int units_total;  // resident units per row (ceil(K / 256))
    int off_x, off_sx, off_sa, off_red, off_bar;  // byte offsets from the 128-byte aligned base (weights at 0)
};

__device__ __forceinline__ void i8_cluster_sync() {
    asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ float i8_ld_cluster_f32(const float *local, uint32_t rank) {
    uint32_t remote;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(smem_u32(local)), "r"(rank));
    float v;
    asm volatile("ld.shared::cluster.f32 %0, [%1];" : "=f"(v) : "r"(remote) : "memory");
    return v;
}
// Bounded wait: when the barrier does not complete (or another warp already gave up) the abort flag is raised and
// every later wait in the CTA falls through, so all warps still reach every barrier and return.
__device__ __forceinline__ void i8_wait_or_abort(uint64_t *bar, uint32_t parity, volatile int *abort_flag, uint32_t *status) {
    for (uint32_t i = 0; i < (1u << 22); ++i) {
        if (mbar_try_wait(bar, parity)) return;
        if (*abort_flag) return;
    }
    *abort_flag = 1;
    atomicMax(status, (uint32_t)kStatusTmaTimeout);
}

// Shared-memory loads by 32-bit shared address: no generic-address arithmetic, and the loads of one unit are issued
// together ahead of the MMAs that consume them.
__device__ __forceinline__ uint2 lds64(uint32_t addr) {
    uint2 v;
    asm volatile("ld.shared.v2.u32 {%0,%1}, [%2];" : "=r"(v.x), "=r"(v.y) : "r"(addr));
    return v;
}
__device__ __forceinline__ uint4 lds128(uint32_t addr) {
    uint4 v;
    asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr));
    return v;
}
__device__ __forceinline__ float lds_f32(uint32_t addr) {
    float v;
    asm volatile("ld.shared.f32 %0, [%1];" : "=f"(v) : "r"(addr));
    return v;
}
// zero-extended byte j of a word
template <int J> __device__ __forceinline__ int byte_of(uint32_t w) {
    uint32_t r;
    asm("prmt.b32 %0, %1, %2, %3;" : "=r"(r) : "r"(w), "r"(0u), "n"(0x4440 + J));
    return (int)r;
}

template <bool A_SIGNED>
__device__ __forceinline__ void imma_16832(int (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
    if constexpr (A_SIGNED) {
        asm("mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%10,%10,%10};"
                     : "=r"(d[0]), "=r"(d[1]), "=r"(d[2]), "=r"(d[3])
                     : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "r"(0));
    } else {
        asm("mma.sync.aligned.m16n8k32.row.col.s32.u8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%10,%10,%10};"
                     : "=r"(d[0]), "=r"(d[1]), "=r"(d[2]), "=r"(d[3])
                     : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "r"(0));
    }
}
// (a & b) ^ c in one LOP3
__device__ __forceinline__ uint32_t lop3_and_xor(uint32_t a, uint32_t b, uint32_t c) {
    uint32_t r;
    asm("lop3.b32 %0, %1, %2, %3, 0x6A;" : "=r"(r) : "r"(a), "r"(b), "r"(c));
    return r;
}

// Where the activation quad that starts at unit element i (a multiple of 4) sits in the B fragments:
// scale group G (one MMA each), lane-in-quad t, fragment register reg.
template <uint32_t TYPE> __device__ __forceinline__ void i8_slot(int i, int &G, int &t, int &reg) {
    G = i >> 5;
    if (TYPE == ZQ_Q4_K) {
        const int j = i & 31;  // byte of the 32-byte nibble pair; lane t reads words 2t and 2t+1
        t = j >> 3;
        reg = (j >> 2) & 1;
    } else {  // block-32 units: lane t reads the word with elements 4t..4t+3 (first half) and 16+4t.. (second half)
        const int e = i & 31;
        t = (e & 15) >> 2;
        reg = e >> 4;
    }
}

// Shared-memory layout of the quantised activations, CP = 8 NT MMA columns (columns past 2 m hold zeros):
//   x   [unit][group G][column][lane-in-quad t][register]  u32   -> one 8-byte B fragment per (G, column, t)
//   sx  [unit][column][t]                                  2 x half2 (hi limbs | lo limbs of two group sums)
//   sa  [unit][activation row 0 .. 4 NT - 1]               f32 slice scale
// All addresses below are 32-bit shared addresses.

// One Q4_K unit (256 weights) of the thread's two fragment rows.
//   wq0 / wq1  unit base of fragment rows g and g+8      xa  this lane's B fragment of group 0, column tile 0
//   sxa        this lane's group-sum fragment             saa this lane's slice scale (row t of column tile 0)
template <int NT>
__device__ __forceinline__ void consume_q4k_i8(uint32_t wq0, uint32_t wq1, int t, uint32_t xa, uint32_t sxa, uint32_t saa, float (&yacc)[NT][2]) {
    constexpr int CP = 8 * NT;
    const uint4 hdr0 = lds128(wq0), hdr1 = lds128(wq1);
    uint2 q0[4], q1[4];
#pragma unroll
    for (int pr = 0; pr < 4; ++pr) {
        q0[pr] = lds64(wq0 + 16 + 32 * pr + 8 * t);
        q1[pr] = lds64(wq1 + 16 + 32 * pr + 8 * t);
    }
    const uint32_t sc_lo0 = hdr0.y & 0x3F3F3F3Fu, sc_hi0 = (hdr0.w & 0x0F0F0F0Fu) | ((hdr0.y >> 2) & 0x30303030u);
    const uint32_t sc_lo1 = hdr1.y & 0x3F3F3F3Fu, sc_hi1 = (hdr1.w & 0x0F0F0F0Fu) | ((hdr1.y >> 2) & 0x30303030u);
    int tl[NT][4], th[NT][4];  // sum over groups of scale * MMA result: low-nibble groups, high-nibble groups
#pragma unroll
    for (int nt = 0; nt < NT; ++nt)
#pragma unroll
        for (int j = 0; j < 4; ++j) tl[nt][j] = th[nt][j] = 0;
#pragma unroll
    for (int pr = 0; pr < 4; ++pr) {
        uint2 bl[NT], bh[NT];
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) {
            bl[nt] = lds64(xa + (2 * pr) * 32 * CP + nt * 256);
            bh[nt] = lds64(xa + (2 * pr + 1) * 32 * CP + nt * 256);
        }
        const uint32_t s0w = pr < 2 ? sc_lo0 : sc_hi0, s1w = pr < 2 ? sc_lo1 : sc_hi1;
        {
            const int s0 = (pr & 1) ? byte_of<2>(s0w) : byte_of<0>(s0w), s1 = (pr & 1) ? byte_of<2>(s1w) : byte_of<0>(s1w);
            const uint32_t a0 = q0[pr].x & 0x0F0F0F0Fu, a1 = q1[pr].x & 0x0F0F0F0Fu, a2 = q0[pr].y & 0x0F0F0F0Fu, a3 = q1[pr].y & 0x0F0F0F0Fu;
#pragma unroll
            for (int nt = 0; nt < NT; ++nt) {
                int d[4];
                imma_16832<false>(d, a0, a1, a2, a3, bl[nt].x, bl[nt].y);
                tl[nt][0] += d[0] * s0;
                tl[nt][1] += d[1] * s0;
                tl[nt][2] += d[2] * s1;
                tl[nt][3] += d[3] * s1;
            }
        }
        {
            const int s0 = (pr & 1) ? byte_of<3>(s0w) : byte_of<1>(s0w), s1 = (pr & 1) ? byte_of<3>(s1w) : byte_of<1>(s1w);
            const uint32_t a0 = q0[pr].x & 0xF0F0F0F0u, a1 = q1[pr].x & 0xF0F0F0F0u, a2 = q0[pr].y & 0xF0F0F0F0u, a3 = q1[pr].y & 0xF0F0F0F0u;
#pragma unroll
            for (int nt = 0; nt < NT; ++nt) {
                int d[4];
                imma_16832<false>(d, a0, a1, a2, a3, bh[nt].x, bh[nt].y);
                th[nt][0] += d[0] * s0;
                th[nt][1] += d[1] * s0;
                th[nt][2] += d[2] * s1;
                th[nt][3] += d[3] * s1;
            }
        }
    }
    // min term: the 8 min codes of each row against the 8 group sums (hi limbs, worth 1024, in K slots 0..7; lo limbs in 8..15)
    float d2[NT][4];
    {
        const uint32_t mn_lo0 = hdr0.z & 0x3F3F3F3Fu, mn_hi0 = ((hdr0.w >> 4) & 0x0F0F0F0Fu) | ((hdr0.z >> 2) & 0x30303030u);
        const uint32_t mn_lo1 = hdr1.z & 0x3F3F3F3Fu, mn_hi1 = ((hdr1.w >> 4) & 0x0F0F0F0Fu) | ((hdr1.z >> 2) & 0x30303030u);
        const uint32_t mb = 2 * (t & 1);
        const uint32_t sel_m = 0x4040u | ((mb + 1) << 8) | mb;
        const uint32_t ma0 = hsub2_u32(prmt(t < 2 ? mn_lo0 : mn_hi0, 0x64646464u, sel_m), 0x64006400u);
        const uint32_t ma1 = hsub2_u32(prmt(t < 2 ? mn_lo1 : mn_hi1, 0x64646464u, sel_m), 0x64006400u);
        const uint32_t ma0k = hmul2_u32(ma0, 0x64006400u), ma1k = hmul2_u32(ma1, 0x64006400u);  // x 1024 (<= 64512, exact)
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) {
            const uint2 sx = lds64(sxa + nt * 256);
            mma_16816_zero(d2[nt], ma0k, ma1k, ma0, ma1, sx.x, sx.y);
        }
    }
    const __half2 dd0 = u32_as_h2(hdr0.x), dd1 = u32_as_h2(hdr1.x);
    const float d_0 = __low2float(dd0) * 0.0625f, dm_0 = __high2float(dd0), d_1 = __low2float(dd1) * 0.0625f, dm_1 = __high2float(dd1);
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) {
        // columns 2t / 2t+1 of the tile are the hi / lo limb of one activation row
        const float sa = lds_f32(saa + nt * 16);
        const float f0 = (float)((tl[nt][0] << 4) + th[nt][0]) * 256.f + (float)((tl[nt][1] << 4) + th[nt][1]);
        const float f1 = (float)((tl[nt][2] << 4) + th[nt][2]) * 256.f + (float)((tl[nt][3] << 4) + th[nt][3]);
        yacc[nt][0] += sa * (d_0 * f0 - dm_0 * d2[nt][0]);
        yacc[nt][1] += sa * (d_1 * f1 - dm_1 * d2[nt][2]);
    }
}

// One block-32 unit (8 blocks of 32 weights) of the thread's two fragment rows: Q4_0 or Q8_0.
template <uint32_t TYPE, int NT>
__device__ __forceinline__ void consume_b32_i8(uint32_t wq0, uint32_t wq1, int t, uint32_t xa, uint32_t saa, float (&yacc)[NT][2]) {
    constexpr int CP = 8 * NT;
    constexpr int H = TYPE == ZQ_Q8_0 ? 4 : 2;     // 16-byte pieces per lane
    constexpr int BPP = TYPE == ZQ_Q8_0 ? 2 : 4;   // blocks per piece
    constexpr float kPre = TYPE == ZQ_Q8_0 ? 1.f : 0.0625f;
    const uint4 hdr0 = lds128(wq0), hdr1 = lds128(wq1);
    uint4 pc0[H], pc1[H];
#pragma unroll
    for (int h = 0; h < H; ++h) {
        pc0[h] = lds128(wq0 + 16 + 16 * (t + 4 * h));
        pc1[h] = lds128(wq1 + 16 + 16 * (t + 4 * h));
    }
    const uint32_t hd0[4] = {hdr0.x, hdr0.y, hdr0.z, hdr0.w}, hd1[4] = {hdr1.x, hdr1.y, hdr1.z, hdr1.w};
    float sap[NT];
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) sap[nt] = lds_f32(saa + nt * 16) * kPre;
#pragma unroll
    for (int h = 0; h < H; ++h) {
        const uint32_t q0[4] = {pc0[h].x, pc0[h].y, pc0[h].z, pc0[h].w};
        const uint32_t q1[4] = {pc1[h].x, pc1[h].y, pc1[h].z, pc1[h].w};
        uint2 b[BPP][NT];
#pragma unroll
        for (int bb = 0; bb < BPP; ++bb)
#pragma unroll
            for (int nt = 0; nt < NT; ++nt) b[bb][nt] = lds64(xa + (BPP * h + bb) * 32 * CP + nt * 256);
#pragma unroll
        for (int bb = 0; bb < BPP; ++bb) {
            const int blk = BPP * h + bb;
            uint32_t a0, a1, a2, a3;
            if constexpr (TYPE == ZQ_Q8_0) {
                a0 = q0[2 * bb]; a1 = q1[2 * bb]; a2 = q0[2 * bb + 1]; a3 = q1[2 * bb + 1];
            } else {  // 16 (q - 8) as s8: low nibbles moved up, high nibbles in place
                a0 = lop3_and_xor(q0[bb] << 4, 0xF0F0F0F0u, 0x80808080u);
                a1 = lop3_and_xor(q1[bb] << 4, 0xF0F0F0F0u, 0x80808080u);
                a2 = lop3_and_xor(q0[bb], 0xF0F0F0F0u, 0x80808080u);
                a3 = lop3_and_xor(q1[bb], 0xF0F0F0F0u, 0x80808080u);
            }
            const __half2 s0 = u32_as_h2(hd0[blk >> 1]), s1 = u32_as_h2(hd1[blk >> 1]);
            const float sc0 = (blk & 1) ? __high2float(s0) : __low2float(s0), sc1 = (blk & 1) ? __high2float(s1) : __low2float(s1);
#pragma unroll
            for (int nt = 0; nt < NT; ++nt) {
                int d[4];
                imma_16832<true>(d, a0, a1, a2, a3, b[bb][nt].x, b[bb][nt].y);
                yacc[nt][0] += (sc0 * sap[nt]) * (float)(d[0] * 256 + d[1]);
                yacc[nt][1] += (sc1 * sap[nt]) * (float)(d[2] * 256 + d[3]);
            }
        }
    }
}

template <uint32_t TYPE, int NT, bool GATED>
__global__ void __launch_bounds__(kI8Threads, 1) gemv_i8_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b, const GemvParams p, const I8Args ia) {
    constexpr int UB = Fmt<TYPE>::unit_bytes;
    constexpr int PITCH = kChunkUnits * UB;
    constexpr int STAGE_W = kTileRows * PITCH;
    constexpr int CP = 8 * NT;
    constexpr int X_UNIT = 8 * CP * 32, SX_UNIT = CP * 32, SA_UNIT = 4 * NT * 4;  // bytes per staged unit
    extern __shared__ uint8_t smem_raw[];
    uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 127) & ~uintptr_t(127));
    uint8_t *ws = smem;
    uint32_t *xw = reinterpret_cast<uint32_t *>(smem + ia.off_x);
    uint2 *sxs = reinterpret_cast<uint2 *>(smem + ia.off_sx);
    float *sact = reinterpret_cast<float *>(smem + ia.off_sa);
    float *red = reinterpret_cast<float *>(smem + ia.off_red);
    uint64_t *full = reinterpret_cast<uint64_t *>(smem + ia.off_bar);
    uint64_t *empty = full + 8;
    __shared__ int s_abort;

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int STAGES = ia.stages;
    const int rows_per_tile = GATED ? kTileRows / 2 : kTileRows;
    const int split = ia.split;
    const int my_tile = blockIdx.x / split, my_rank = blockIdx.x % split;
    const int chunk_begin = (int)((long long)my_rank * p.chunks / split), chunk_end = (int)((long long)(my_rank + 1) * p.chunks / split);
    const int n_items = chunk_end - chunk_begin;
    const int unit0 = chunk_begin * kChunkUnits;

    if (tid == 0) {
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(&full[s], 1);
            mbar_init(&empty[s], kI8Threads / 32);
        }
        fence_mbar_init();
        tma_prefetch_desc(&map_a);
        if (GATED) tma_prefetch_desc(&map_b);
        s_abort = 0;
    }
    __syncthreads();

    auto issue_tma = [&](int local, int stage) {
        const int chunk = chunk_begin + local;
        uint8_t *dst = ws + (size_t)stage * STAGE_W;
        mbar_expect_tx(&full[stage], STAGE_W);
        if (GATED) {
            tma_load_2d(dst, &map_a, &full[stage], chunk * p.chunk_words, my_tile * rows_per_tile);
            tma_load_2d(dst + STAGE_W / 2, &map_b, &full[stage], chunk * p.chunk_words, my_tile * rows_per_tile);
        } else {
            tma_load_2d(dst, &map_a, &full[stage], chunk * p.chunk_words, my_tile * rows_per_tile);
        }
    };
    if (tid == 0) {
        const int pre = n_items < STAGES - 1 ? n_items : STAGES - 1;
        for (int s = 0; s < pre; ++s) issue_tma(s, s);
    }

    const int g = lane >> 2, t = lane & 3;
    const int rs = warp & 7, ul = warp >> 3;
    const int M = p.m;

    int slice_units = chunk_end * kChunkUnits;
    if (slice_units > ia.units_total) slice_units = ia.units_total;
    slice_units -= unit0;
    if (slice_units < 0) slice_units = 0;
    pdl_launch_dependents();
    pdl_wait_prior_grid();  // activations (and, later, outputs) belong to the previous kernel until it completes
    {
        // Quantise the activation slice: one warp per (row, 256-column slice), 8 consecutive columns per lane.  A warp
        // takes its slices four at a time, all loads first, so that their latencies overlap.  Columns past 2 m, and
        // sums and scales of rows past m, are never written: whatever they hold only reaches accumulator columns
        // that no one reads (integer MMAs cannot produce NaNs for the columns that are read).
        constexpr int kBatch = 4, kWarps = kI8Threads / 32;
        const int total = M * slice_units;
        for (int base = warp; base < total; base += kBatch * kWarps) {
            float v[kBatch][8];
            int tm[kBatch], tu[kBatch];
#pragma unroll
            for (int b = 0; b < kBatch; ++b) {
                const int task = base + b * kWarps;
                tm[b] = task < total ? task / slice_units : -1;
                tu[b] = task < total ? task - tm[b] * slice_units : 0;
#pragma unroll
                for (int j = 0; j < 8; ++j) v[b][j] = 0.f;
                const int k0 = (unit0 + tu[b]) * kUnitWeights + 8 * lane;
                if (tm[b] >= 0 && k0 < p.cols) {  // K is a multiple of 32, so a lane's 8 columns are all inside or all outside
                    const size_t o = (size_t)tm[b] * p.cols + k0;
                    if (p.x_dtype == ZQ_F32) {
                        const float4 f0 = *reinterpret_cast<const float4 *>(reinterpret_cast<const float *>(p.x) + o);
                        const float4 f1 = *reinterpret_cast<const float4 *>(reinterpret_cast<const float *>(p.x) + o + 4);
                        v[b][0] = f0.x; v[b][1] = f0.y; v[b][2] = f0.z; v[b][3] = f0.w; v[b][4] = f1.x; v[b][5] = f1.y; v[b][6] = f1.z; v[b][7] = f1.w;
                    } else {
                        const uint4 raw = *reinterpret_cast<const uint4 *>(reinterpret_cast<const uint16_t *>(p.x) + o);
                        const uint32_t rw[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
                        for (int j = 0; j < 4; ++j) {
                            if (p.x_dtype == ZQ_F16) {
                                const float2 f = __half22float2(u32_as_h2(rw[j]));
                                v[b][2 * j] = f.x; v[b][2 * j + 1] = f.y;
                            } else {  // bf16: the upper half of an f32
                                v[b][2 * j] = __uint_as_float(rw[j] << 16);
                                v[b][2 * j + 1] = __uint_as_float(rw[j] & 0xFFFF0000u);
                            }
                        }
                    }
                }
            }
#pragma unroll
            for (int b = 0; b < kBatch; ++b) {
                if (tm[b] < 0) continue;  // warp-uniform
                const int m = tm[b], unit = tu[b];
                float amax = 0.f;
#pragma unroll
                for (int j = 0; j < 8; ++j) amax = fmaxf(amax, fabsf(v[b][j]));
#pragma unroll
                for (int s = 16; s >= 1; s >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, s));
                const bool live = amax > 0.f && amax < 3.0e38f;
                const float inv = live ? __fdividef(kActMax, amax) : 0.f;
                int hi[8], lo[8], sum = 0;
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                    int xq = __float2int_rn(v[b][j] * inv);
                    xq = xq > 32512 ? 32512 : (xq < -32512 ? -32512 : xq);
                    hi[j] = (xq + 128) >> 8;
                    lo[j] = xq - (hi[j] << 8);
                    sum += xq;
                }
                const int i0 = 8 * lane;  // first of the lane's elements inside the unit
#pragma unroll
                for (int qd = 0; qd < 2; ++qd) {
                    int G, tt, reg;
                    i8_slot<TYPE>(i0 + 4 * qd, G, tt, reg);
                    const uint32_t ph = (uint32_t)(hi[4 * qd] & 0xFF) | ((uint32_t)(hi[4 * qd + 1] & 0xFF) << 8) | ((uint32_t)(hi[4 * qd + 2] & 0xFF) << 16) | ((uint32_t)(hi[4 * qd + 3] & 0xFF) << 24);
                    const uint32_t pl = (uint32_t)(lo[4 * qd] & 0xFF) | ((uint32_t)(lo[4 * qd + 1] & 0xFF) << 8) | ((uint32_t)(lo[4 * qd + 2] & 0xFF) << 16) | ((uint32_t)(lo[4 * qd + 3] & 0xFF) << 24);
                    const int slot = (((unit * 8 + G) * CP + 2 * m) * 4 + tt) * 2 + reg;
                    xw[slot] = ph;
                    xw[slot + 8] = pl;  // next column: the lo limb
                }
                // the scale actually applied: x ~ x_q / inv
                if (lane == 0) sact[unit * (4 * NT) + m] = live ? __fdividef(1.f, inv) : 0.f;
                if constexpr (TYPE == ZQ_Q4_K) {
                    // exact integer sum of each 32-column group, as two f16 limbs for the min-term MMA
                    sum += __shfl_xor_sync(0xffffffffu, sum, 1);
                    sum += __shfl_xor_sync(0xffffffffu, sum, 2);
                    if ((lane & 3) == 0) {
                        const int G8 = lane >> 2;
                        // |sum| can reach 32 * 32512, beyond f16: sum = 1024 a + r with |a| <= 1016, |r| <= 512, both exact
                        // in f16; the factor 1024 rides on the min codes of the hi-limb K slots
                        const int a = (sum + 512) >> 10, r = sum - (a << 10);
                        __half *dst = reinterpret_cast<__half *>(&sxs[(unit * CP + 2 * m) * 4 + (G8 >> 1)]);
                        dst[G8 & 1] = __int2half_rn(a);
                        dst[2 + (G8 & 1)] = __int2half_rn(r);
                    }
                }
            }
        }
    }
    __syncthreads();

    float yacc[NT][2];
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) yacc[nt][0] = yacc[nt][1] = 0.f;
    const int r0 = 16 * rs + frag_row(g);

    {
        const uint32_t w_first = smem_u32(ws) + (uint32_t)(r0 * PITCH + ul * UB);
        uint32_t xa = smem_u32(smem + ia.off_x) + (uint32_t)(ul * X_UNIT + lane * 8);
        uint32_t sxa = smem_u32(smem + ia.off_sx) + (uint32_t)(ul * SX_UNIT + lane * 8);
        uint32_t saa = smem_u32(smem + ia.off_sa) + (uint32_t)(ul * SA_UNIT + t * 4);
        int stage = 0;
        uint32_t phase = 0;
        int unit_abs = unit0 + ul;
        for (int it = 0; it < n_items; ++it) {
            {
                // refill: the stage consumed one iteration ago takes the item STAGES-1 ahead; a different warp each time
                const int nxt = it + STAGES - 1;
                if (nxt < n_items && warp == (it & 15) && lane == 0) {
                    const int nstage = stage == 0 ? STAGES - 1 : stage - 1;
                    if (it >= 1) i8_wait_or_abort(&empty[nstage], stage == 0 ? phase ^ 1u : phase, &s_abort, p.status);
                    if (!*(volatile int *)&s_abort) issue_tma(nxt, nstage);  // never start a copy nobody will wait for
                }
                __syncwarp();
            }
            i8_wait_or_abort(&full[stage], phase, &s_abort, p.status);
            if (unit_abs < ia.units_total) {
                const uint32_t wq0 = w_first + (uint32_t)(stage * STAGE_W), wq1 = wq0 + 8 * PITCH;
                if constexpr (TYPE == ZQ_Q4_K) consume_q4k_i8<NT>(wq0, wq1, t, xa, sxa, saa, yacc);
                else consume_b32_i8<TYPE, NT>(wq0, wq1, t, xa, saa, yacc);
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(&empty[stage]);
            if (++stage == STAGES) {
                stage = 0;
                phase ^= 1u;
            }
            unit_abs += kChunkUnits;
            xa += kChunkUnits * X_UNIT;
            sxa += kChunkUnits * SX_UNIT;
            saa += kChunkUnits * SA_UNIT;
        }
    }

    // ---------------------------------------------------- end of the K slice: combine and store
    {
        // Every CTA leaves its partial tile (one copy per unit half) in its own shared memory; after one barrier
        // (cluster-wide when the tile is split) the threads of rank 0 add up, for their output element, the halves
        // of every rank in rank order (deterministic), apply the epilogue and store.
        constexpr int RS = NT * 4;  // activation rows a tile row can hold
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) {
            red[(ul * RS + nt * 4 + t) * kTileRows + r0] = yacc[nt][0];  // [unit half][activation row][tile row]
            red[(ul * RS + nt * 4 + t) * kTileRows + r0 + 8] = yacc[nt][1];
        }
        if (split > 1) i8_cluster_sync();
        else __syncthreads();
        if (my_rank == 0) {
            constexpr int out_rows = GATED ? kTileRows / 2 : kTileRows;
            auto total_of = [&](int rr, int tok) -> float {
                const float *a = &red[tok * kTileRows + rr], *b = &red[(RS + tok) * kTileRows + rr];
                float v = *a + *b;
                for (int r = 1; r < split; ++r) v += i8_ld_cluster_f32(a, (uint32_t)r) + i8_ld_cluster_f32(b, (uint32_t)r);
                return v;
            };
            for (int i = tid; i < out_rows * M; i += kI8Threads) {
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
        if (split > 1) i8_cluster_sync();  // nobody leaves while rank 0 may still read its shared memory
    }
}

// Shared-memory plan: CTAs per tile (cluster size), ring depth and offsets; false when fewer than two ring stages
// fit beside the quantised activation slice.
template <uint32_t TYPE, int NT>
static bool plan_i8(int m, int units_total, int tiles, int chunks, int sm_count, I8Args &ia, int &total_bytes) {
    constexpr int STAGE_W = kTileRows * kChunkUnits * Fmt<TYPE>::unit_bytes;
    constexpr int CP = 8 * NT;  // MMA columns, padded to whole column tiles
    const int max_smem = 232448 - 256;  // 227 KB opt-in limit minus static shared and alignment slack
    const int red_bytes = 2 * kTileRows * NT * 4 * 4;
    // CTAs per tile: as many K slices as fill the SMs (any cluster size up to 8, not only powers of two); more than
    // that, i.e. more CTAs than SMs, only when the activation slice would otherwise leave no room for the ring
    int split = sm_count / (tiles > 0 ? tiles : 1);
    if (split > 8) split = 8;
    if (split > chunks) split = chunks;
    if (split < 1) split = 1;
    int room = 0, slice_chunks = 0, x_bytes = 0, sx_bytes = 0, sa_bytes = 0;  // room: ring stages that fit
    for (;; ++split) {
        slice_chunks = (chunks + split - 1) / split;
        int slice_units = slice_chunks * kChunkUnits;
        if (slice_units > units_total) slice_units = units_total;
        x_bytes = slice_units * 8 * CP * 32;
        sx_bytes = TYPE == ZQ_Q4_K ? slice_units * CP * 32 : 0;
        sa_bytes = (slice_units * 4 * NT * 4 + 127) & ~127;
        room = (max_smem - (x_bytes + sx_bytes + sa_bytes + red_bytes + 128 + 128)) / STAGE_W;
        if (room >= 3 || split >= 8 || split >= chunks) break;
    }
    if (room < 2) return false;
    int stages = room > 5 ? 5 : room;
    if (stages > slice_chunks + 1) stages = slice_chunks + 1;  // no point in more ring than work
    if (stages < 2) stages = 2;
    (void)m;
    ia.stages = stages;
    ia.split = split;
    ia.units_total = units_total;
    ia.off_x = stages * STAGE_W;
    ia.off_sx = ia.off_x + x_bytes;
    ia.off_sa = ia.off_sx + sx_bytes;
    ia.off_red = ia.off_sa + sa_bytes;
    ia.off_bar = ia.off_red + red_bytes;
    total_bytes = ia.off_bar + 128 + 128;
    return true;
}

template <uint32_t TYPE, int NT, bool GATED>
static int launch_i8_one(zq_ctx *ctx, const zq_weight *w, const zq_weight *w_up, const GemvParams &p, bool &taken, zq_error *err) {
    I8Args ia;
    int total = 0;
    taken = plan_i8<TYPE, NT>(p.m, (int)w->units_per_row, p.tiles, p.chunks, ctx->sm_count, ia, total);
    if (!taken) return ZQ_OK;
    auto kernel = gemv_i8_kernel<TYPE, NT, GATED>;
    static bool configured[64] = {};
    if (!configured[ctx->device & 63]) {
        ZQ_CUDA_CHECK(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 232448 - 256), err);
        configured[ctx->device & 63] = true;
    }
    const CUtensorMap &ma = GATED ? w->gemv_map_half : w->gemv_map;
    const CUtensorMap &mb = GATED ? w_up->gemv_map_half : w->gemv_map;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)(p.tiles * ia.split));
    cfg.blockDim = dim3(kI8Threads);
    cfg.dynamicSmemBytes = (size_t)total;
    cfg.stream = ctx->stream;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = (unsigned)ia.split;
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
    if (p.m <= 4) return gated ? launch_i8_one<TYPE, 1, true>(ctx, w, w_up, p, taken, err) : launch_i8_one<TYPE, 1, false>(ctx, w, w_up, p, taken, err);
    if (p.m <= 8) return gated ? launch_i8_one<TYPE, 2, true>(ctx, w, w_up, p, taken, err) : launch_i8_one<TYPE, 2, false>(ctx, w, w_up, p, taken, err);
    return gated ? launch_i8_one<TYPE, 4, true>(ctx, w, w_up, p, taken, err) : launch_i8_one<TYPE, 4, false>(ctx, w, w_up, p, taken, err);
}

// Tries the integer-MMA kernel for one pass of up to 16 activation rows; `taken` tells whether it was launched
// (IQ4_NL, whose codebook values would need a table lookup per weight, and slices that do not fit stay on the
// f16 kernels).
int launch_gemv_i8(zq_ctx *ctx, const zq_weight *w, const zq_weight *w_up, const GemvParams &p, bool &taken, zq_error *err) {
    taken = false;
    if (p.m < 1 || p.m > kMaxGemvRows) return ZQ_OK;
    switch (w->type) {
    case ZQ_Q4_K: return launch_i8_type<ZQ_Q4_K>(ctx, w, w_up, p, taken, err);
    case ZQ_Q4_0: return launch_i8_type<ZQ_Q4_0>(ctx, w, w_up, p, taken, err);
    case ZQ_Q8_0: return launch_i8_type<ZQ_Q8_0>(ctx, w, w_up, p, taken, err);
    default: return ZQ_OK;
    }
}

}  // namespace zq
