// Shared pieces of the decode GEMV kernels: tile constants, per-format traits, the fragment-row permutation,
// the activation-quad -> MMA-slot map, and the routine that turns one staged unit (256 weights x 16 rows) into
// tensor-core MMAs.
#pragma once
#include "zq_common.cuh"

namespace zq {

constexpr int kTileRows = 128;
constexpr int kChunkUnits = 2;
constexpr int kChunkCols = kChunkUnits * kUnitWeights;  // 512
constexpr int kGemvThreads = 512;                       // 16 warps: 8 row sub-tiles x 2 units
constexpr int kMaxGemvRows = 16;                        // 8 rows with two f16 limbs each, or 16 rows with one limb
constexpr int kSlotFloats = kTileRows * kMaxGemvRows;   // one partial tile in the fix-up scratch

template <uint32_t TYPE> struct Fmt;
template <> struct Fmt<ZQ_Q4_K> { static constexpr int unit_bytes = 144; static constexpr int stages = 4; static constexpr bool lut = false; };
template <> struct Fmt<ZQ_Q4_0> { static constexpr int unit_bytes = 144; static constexpr int stages = 4; static constexpr bool lut = false; };
template <> struct Fmt<ZQ_IQ4_NL> { static constexpr int unit_bytes = 144; static constexpr int stages = 3; static constexpr bool lut = true; };
template <> struct Fmt<ZQ_Q8_0> { static constexpr int unit_bytes = 272; static constexpr int stages = 2; static constexpr bool lut = false; };
template <> struct Fmt<ZQ_Q6_K> { static constexpr int unit_bytes = 224; static constexpr int stages = 3; static constexpr bool lut = false; };  // integer-MMA kernels only
template <> struct Fmt<ZQ_Q5_K> { static constexpr int unit_bytes = 176; static constexpr int stages = 3; static constexpr bool lut = false; };  // integer-MMA kernels only

template <uint32_t TYPE, int NT> struct GemvSmem {
    static constexpr int stages = (NT == 2 && Fmt<TYPE>::stages > 3) ? 3 : Fmt<TYPE>::stages;  // two column tiles need room
    static constexpr int pitch = kChunkUnits * Fmt<TYPE>::unit_bytes;
    static constexpr int stage_w = kTileRows * pitch;
    static constexpr int stage_x = NT * kChunkUnits * 16 * 32 * 8;
    static constexpr int stage_sx = NT * kChunkUnits * 32 * 8;  // per lane: (hi limbs, lo limbs) of two group sums
    static constexpr int off_w = 0;
    static constexpr int off_x = off_w + stages * stage_w;
    static constexpr int off_sx = off_x + stages * stage_x;
    static constexpr int off_red = off_sx + stages * stage_sx;
    static constexpr int red_bytes = 2 * kTileRows * NT * 8 * 4;  // [unit half][row][up to 8 columns per tile] f32
    static constexpr int off_lut = off_red + red_bytes;
    static constexpr int lut_bytes = Fmt<TYPE>::lut ? 256 * 32 * 4 : 0;
    static constexpr int off_bar = off_lut + lut_bytes;
    static constexpr int total = off_bar + 64 + 128;  // barriers + slack for 128-byte alignment of the base
};

struct GemvParams {
    const void *x;        // [m, cols]
    void *y;              // [m, n_out]
    const void *residual; // [m, n_out] or null
    float *partials;      // fix-up scratch
    uint32_t *counters;
    uint32_t *status;
    int x_dtype, y_dtype;
    int m;                // 1..8 rows as two f16 limbs each, or 9..16 rows as one limb each
    int limbs;            // 2 or 1
    int cols;             // logical K
    int n_out;            // output features (rows of W; for gated: rows of gate == rows of up)
    int tiles;            // ceil(n_out / rows_per_tile)
    int chunks;           // ceil(units_per_row / kChunkUnits)
    int chunk_words;      // kChunkUnits * unit_bytes / 4
};

// Fragment row g (0..7) -> row inside the warp's 16-row sub-tile.  Swapping the two low bits puts the two rows a
// quarter-warp reads 2 apart, which makes the 16-byte fragment loads bank-conflict free for row pitches that
// are 32 mod 128 bytes (288 and 544).
__device__ __forceinline__ int frag_row(int g) { return (g & 4) | ((g & 1) << 1) | ((g >> 1) & 1); }

__device__ __forceinline__ uint32_t prmt(uint32_t a, uint32_t b, uint32_t sel) {
    uint32_t r;
    asm("prmt.b32 %0, %1, %2, %3;" : "=r"(r) : "r"(a), "r"(b), "r"(sel));
    return r;
}

// Where the activation quad starting at unit element i (a multiple of 4) lands in the B-fragment staging:
// MMA step and lane-t for the whole-quad formats.
template <uint32_t TYPE> __device__ __forceinline__ void quad_slot(int i, int &step, int &t) {
    if (TYPE == ZQ_Q4_K) {
        int G = i >> 5, e = (i >> 4) & 1, ii = (i >> 2) & 3;
        int piece = 2 * (G >> 1) + e;
        t = piece & 3;
        step = 8 * (piece >> 2) + 2 * ii + (G & 1);
    } else if (TYPE == ZQ_Q8_0) {
        int blk = i >> 5, e = (i >> 4) & 1;
        t = (i >> 2) & 3;
        step = 2 * blk + e;
    } else {  // Q4_0
        int blk = i >> 5, nib = (i >> 4) & 1;
        t = (i >> 2) & 3;
        step = 8 * (blk >> 2) + 2 * (blk & 3) + nib;
    }
}


// Zero-accumulator form used when a block's sum starts fresh.
__device__ __forceinline__ void mma_16816_zero(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%10,%10,%10};"
                 : "=f"(d[0]), "=f"(d[1]), "=f"(d[2]), "=f"(d[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "f"(0.f));
}

// One unit (256 weights) of the two fragment rows a thread owns -> MMAs.
//   w0 / w1   shared-memory address of the unit in fragment rows g and g+8
//   getb      (nt, step) -> the thread's B fragment {b0, b1} of MMA step `step` for column tile nt
//   getsx     (nt) -> the thread's B fragment {hi limbs, lo limbs} of the per-group activation sums (Q4_K only);
//             the min-term MMA pairs the 8 min codes with the hi limbs (K slots 0..7) and again with the lo limbs
//             (K slots 8..15), so the sums keep two limbs whatever the activations use
//   yacc      running sums [nt][row g / row g+8][column 2t / 2t+1]; the two columns are the two limbs of one
//             activation row, or two activation rows when each row is staged as a single limb.
// Q4_K spreads its 32 dependent MMAs over CH independent accumulator chains.
template <uint32_t TYPE, int NT, class GetB, class GetSx>
__device__ __forceinline__ void consume_unit(const uint8_t *w0, const uint8_t *w1, int t, const uint32_t *lut_lane, GetB getb, GetSx getsx, float (&yacc)[NT][2][2]) {
    const uint4 hdr0 = *reinterpret_cast<const uint4 *>(w0);
    const uint4 hdr1 = *reinterpret_cast<const uint4 *>(w1);
    if constexpr (TYPE == ZQ_Q4_K) {
        constexpr int CH = NT == 1 ? 4 : 2;
        float d1[NT][CH][4], d2[NT][4];
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) {
#pragma unroll
            for (int j = 0; j < 4; ++j) d2[nt][j] = 0.f;
#pragma unroll
            for (int c = 0; c < CH; ++c)
#pragma unroll
                for (int j = 0; j < 4; ++j) d1[nt][c][j] = 0.f;
        }
        const uint32_t k1024 = 0x64006400u, k64x4 = 0x64646464u, kNeg1024 = 0xE400E400u, kNeg64 = 0xD400D400u;
        const uint32_t sc_lo0 = hdr0.y & 0x3F3F3F3Fu, sc_hi0 = (hdr0.w & 0x0F0F0F0Fu) | ((hdr0.y >> 2) & 0x30303030u);
        const uint32_t sc_lo1 = hdr1.y & 0x3F3F3F3Fu, sc_hi1 = (hdr1.w & 0x0F0F0F0Fu) | ((hdr1.y >> 2) & 0x30303030u);
        const uint32_t mn_lo0 = hdr0.z & 0x3F3F3F3Fu, mn_hi0 = ((hdr0.w >> 4) & 0x0F0F0F0Fu) | ((hdr0.z >> 2) & 0x30303030u);
        const uint32_t mn_lo1 = hdr1.z & 0x3F3F3F3Fu, mn_hi1 = ((hdr1.w >> 4) & 0x0F0F0F0Fu) | ((hdr1.z >> 2) & 0x30303030u);
        const uint32_t bidx = 2 * (t >> 1);
        const uint32_t sel_a = 0x4040u | (bidx * 0x0101u);
        const uint32_t sel_b = 0x4040u | ((bidx + 1) * 0x0101u);
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            const uint4 pc0 = *reinterpret_cast<const uint4 *>(w0 + 16 + 16 * (t + 4 * h));
            const uint4 pc1 = *reinterpret_cast<const uint4 *>(w1 + 16 + 16 * (t + 4 * h));
            const uint32_t sc0 = h ? sc_hi0 : sc_lo0, sc1 = h ? sc_hi1 : sc_lo1;
            const uint32_t sa0 = hsub2_u32(prmt(sc0, k64x4, sel_a), k1024), sb0 = hsub2_u32(prmt(sc0, k64x4, sel_b), k1024);
            const uint32_t sa1 = hsub2_u32(prmt(sc1, k64x4, sel_a), k1024), sb1 = hsub2_u32(prmt(sc1, k64x4, sel_b), k1024);
            const uint32_t oa0 = hmul2_u32(sa0, kNeg1024), ob0 = hmul2_u32(sb0, kNeg64);
            const uint32_t oa1 = hmul2_u32(sa1, kNeg1024), ob1 = hmul2_u32(sb1, kNeg64);
            const uint32_t q0[4] = {pc0.x, pc0.y, pc0.z, pc0.w};
            const uint32_t q1[4] = {pc1.x, pc1.y, pc1.z, pc1.w};
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const uint32_t x0 = q0[i], x0s = q0[i] >> 8, x1 = q1[i], x1s = q1[i] >> 8;
                uint32_t a0 = hfma2_u32(lop3_and_or(x0, 0x000F000Fu, 0x64006400u), sa0, oa0);
                uint32_t a2 = hfma2_u32(lop3_and_or(x0s, 0x000F000Fu, 0x64006400u), sa0, oa0);
                uint32_t a1 = hfma2_u32(lop3_and_or(x1, 0x000F000Fu, 0x64006400u), sa1, oa1);
                uint32_t a3 = hfma2_u32(lop3_and_or(x1s, 0x000F000Fu, 0x64006400u), sa1, oa1);
                const int step = 8 * h + 2 * i;
#pragma unroll
                for (int nt = 0; nt < NT; ++nt) {
                    const uint2 b = getb(nt, step);
                    mma_16816(d1[nt][step % CH], a0, a1, a2, a3, b.x, b.y);
                }
                a0 = hfma2_u32(lop3_and_or(x0, 0x00F000F0u, 0x54005400u), sb0, ob0);
                a2 = hfma2_u32(lop3_and_or(x0s, 0x00F000F0u, 0x54005400u), sb0, ob0);
                a1 = hfma2_u32(lop3_and_or(x1, 0x00F000F0u, 0x54005400u), sb1, ob1);
                a3 = hfma2_u32(lop3_and_or(x1s, 0x00F000F0u, 0x54005400u), sb1, ob1);
#pragma unroll
                for (int nt = 0; nt < NT; ++nt) {
                    const uint2 b = getb(nt, step + 1);
                    mma_16816(d1[nt][(step + 1) % CH], a0, a1, a2, a3, b.x, b.y);
                }
            }
        }
        {
            const uint32_t mb = 2 * (t & 1);
            const uint32_t sel_m = 0x4040u | ((mb + 1) << 8) | mb;
            const uint32_t ma0 = hsub2_u32(prmt(t < 2 ? mn_lo0 : mn_hi0, k64x4, sel_m), k1024);
            const uint32_t ma1 = hsub2_u32(prmt(t < 2 ? mn_lo1 : mn_hi1, k64x4, sel_m), k1024);
#pragma unroll
            for (int nt = 0; nt < NT; ++nt) {
                const uint2 sx = getsx(nt);
                mma_16816(d2[nt], ma0, ma1, ma0, ma1, sx.x, sx.y);
            }
        }
        const __half2 dd0 = u32_as_h2(hdr0.x), dd1 = u32_as_h2(hdr1.x);
        const float d_0 = __low2float(dd0), dm_0 = __high2float(dd0), d_1 = __low2float(dd1), dm_1 = __high2float(dd1);
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) {
            float a0 = 0.f, a1 = 0.f, b0 = 0.f, b1 = 0.f;
#pragma unroll
            for (int c = 0; c < CH; ++c) {
                a0 += d1[nt][c][0];
                a1 += d1[nt][c][1];
                b0 += d1[nt][c][2];
                b1 += d1[nt][c][3];
            }
            yacc[nt][0][0] += d_0 * a0 - dm_0 * d2[nt][0];
            yacc[nt][0][1] += d_0 * a1 - dm_0 * d2[nt][1];
            yacc[nt][1][0] += d_1 * b0 - dm_1 * d2[nt][2];
            yacc[nt][1][1] += d_1 * b1 - dm_1 * d2[nt][3];
        }
    } else if constexpr (TYPE == ZQ_Q8_0) {
        const uint32_t hd0[4] = {hdr0.x, hdr0.y, hdr0.z, hdr0.w}, hd1[4] = {hdr1.x, hdr1.y, hdr1.z, hdr1.w};
#pragma unroll
        for (int h = 0; h < 4; ++h) {
            const uint4 pc0 = *reinterpret_cast<const uint4 *>(w0 + 16 + 16 * (t + 4 * h));
            const uint4 pc1 = *reinterpret_cast<const uint4 *>(w1 + 16 + 16 * (t + 4 * h));
            const uint32_t q0[4] = {pc0.x, pc0.y, pc0.z, pc0.w};
            const uint32_t q1[4] = {pc1.x, pc1.y, pc1.z, pc1.w};
            const __half2 s0 = u32_as_h2(hd0[h]), s1 = u32_as_h2(hd1[h]);
#pragma unroll
            for (int bb = 0; bb < 2; ++bb) {
                float acc[NT][4];
#pragma unroll
                for (int e = 0; e < 2; ++e) {
                    const int j = 2 * bb + e;
                    const uint32_t u0 = q0[j] ^ 0x80808080u, u1 = q1[j] ^ 0x80808080u;
                    const uint32_t a0 = hsub2_u32(prmt(u0, 0x64646464u, 0x4240u), 0x64806480u);
                    const uint32_t a2 = hsub2_u32(prmt(u0, 0x64646464u, 0x4341u), 0x64806480u);
                    const uint32_t a1 = hsub2_u32(prmt(u1, 0x64646464u, 0x4240u), 0x64806480u);
                    const uint32_t a3 = hsub2_u32(prmt(u1, 0x64646464u, 0x4341u), 0x64806480u);
                    const int step = 4 * h + j;
#pragma unroll
                    for (int nt = 0; nt < NT; ++nt) {
                        const uint2 b = getb(nt, step);
                        if (e == 0) mma_16816_zero(acc[nt], a0, a1, a2, a3, b.x, b.y);
                        else mma_16816(acc[nt], a0, a1, a2, a3, b.x, b.y);
                    }
                }
                const float sc0 = bb ? __high2float(s0) : __low2float(s0), sc1 = bb ? __high2float(s1) : __low2float(s1);
#pragma unroll
                for (int nt = 0; nt < NT; ++nt) {
                    yacc[nt][0][0] += sc0 * acc[nt][0];
                    yacc[nt][0][1] += sc0 * acc[nt][1];
                    yacc[nt][1][0] += sc1 * acc[nt][2];
                    yacc[nt][1][1] += sc1 * acc[nt][3];
                }
            }
        }
    } else {  // Q4_0, IQ4_NL
        const uint32_t hd0[4] = {hdr0.x, hdr0.y, hdr0.z, hdr0.w}, hd1[4] = {hdr1.x, hdr1.y, hdr1.z, hdr1.w};
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            const uint4 pc0 = *reinterpret_cast<const uint4 *>(w0 + 16 + 16 * (t + 4 * h));
            const uint4 pc1 = *reinterpret_cast<const uint4 *>(w1 + 16 + 16 * (t + 4 * h));
            const uint32_t q0[4] = {pc0.x, pc0.y, pc0.z, pc0.w};
            const uint32_t q1[4] = {pc1.x, pc1.y, pc1.z, pc1.w};
#pragma unroll
            for (int bb = 0; bb < 4; ++bb) {
                float acc[NT][4];
                const uint32_t x0 = q0[bb], x1 = q1[bb];
#pragma unroll
                for (int e = 0; e < 2; ++e) {
                    uint32_t a0, a1, a2, a3;
                    if constexpr (TYPE == ZQ_Q4_0) {
                        const uint32_t mask = e ? 0x00F000F0u : 0x000F000Fu, bias = e ? 0x54005400u : 0x64006400u;
                        const uint32_t off = e ? 0x54805480u : 0x64086408u;
                        a0 = hsub2_u32(lop3_and_or(x0, mask, bias), off);
                        a2 = hsub2_u32(lop3_and_or(x0 >> 8, mask, bias), off);
                        a1 = hsub2_u32(lop3_and_or(x1, mask, bias), off);
                        a3 = hsub2_u32(lop3_and_or(x1 >> 8, mask, bias), off);
                    } else {
                        a0 = lut_lane[((x0 >> (16 * e)) & 0xFFu) * 32];
                        a2 = lut_lane[((x0 >> (16 * e + 8)) & 0xFFu) * 32];
                        a1 = lut_lane[((x1 >> (16 * e)) & 0xFFu) * 32];
                        a3 = lut_lane[((x1 >> (16 * e + 8)) & 0xFFu) * 32];
                    }
                    const int step = 8 * h + 2 * bb + e;
#pragma unroll
                    for (int nt = 0; nt < NT; ++nt) {
                        const uint2 b = getb(nt, step);
                        if (e == 0) mma_16816_zero(acc[nt], a0, a1, a2, a3, b.x, b.y);
                        else mma_16816(acc[nt], a0, a1, a2, a3, b.x, b.y);
                    }
                }
                const int blk = 4 * h + bb;
                const __half2 s0 = u32_as_h2(hd0[blk >> 1]), s1 = u32_as_h2(hd1[blk >> 1]);
                const float sc0 = (blk & 1) ? __high2float(s0) : __low2float(s0), sc1 = (blk & 1) ? __high2float(s1) : __low2float(s1);
#pragma unroll
                for (int nt = 0; nt < NT; ++nt) {
                    yacc[nt][0][0] += sc0 * acc[nt][0];
                    yacc[nt][0][1] += sc0 * acc[nt][1];
                    yacc[nt][1][0] += sc1 * acc[nt][2];
                    yacc[nt][1][1] += sc1 * acc[nt][3];
                }
            }
        }
    }
}

int launch_qmv(zq_ctx *ctx, const zq_weight *w, const GemvParams &p, bool &taken, zq_error *err);
int launch_gemv_i8(zq_ctx *ctx, const zq_weight *w, const zq_weight *w_up, const GemvParams &p, bool &taken, zq_error *err);
int launch_gemv_resident(zq_ctx *ctx, const zq_weight *w, const zq_weight *w_up, const GemvParams &p, int grid, bool &taken, zq_error *err);

}  // namespace zq
