// Pieces shared by the integer-MMA decode kernels (zq_gemv_i8.cu: one matrix per launch; zq_moe_grouped.cu: all
// routed experts of a MoE layer per launch): the activation record format and its quantiser, the shared-memory and
// cluster helpers, and the routines that turn one staged unit (256 weights x 16 rows) into m16n8k32 MMAs.
#pragma once
#include "zq_gemv_frag.cuh"

namespace zq {

constexpr int kI8Threads = 512;
constexpr float kActMax = 32512.f;  // 127 * 256
// One record per (256-column unit, activation row): 32 B-fragment slots of 16 bytes (hi-limb pair | lo-limb pair),
// 32 bytes of group sums (min-term fragment), the slice scale.
constexpr int kRec = 576, kRecSums = 512, kRecScale = 544;

struct I8Args {
    int stages;       // 2..5 ring stages
    int split;        // K slices per tile
    int tshare;       // neighbouring tiles per cluster that share the activation staging (cluster = tshare * split CTAs)
    int units_total;  // resident units per row (ceil(K / 256))
    int off_x, off_red, off_bar;  // byte offsets from the 128-byte aligned base (weights at 0)
    int stage_stride;       // bytes from one ring stage to the next (weights, plus the chunk's records when streamed)
    const uint8_t *xq;      // streamed variant: all records of the activation block in global memory
};

__device__ __forceinline__ void i8_cluster_arrive() { asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory"); }
__device__ __forceinline__ void i8_cluster_wait() { asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory"); }
__device__ __forceinline__ uint32_t i8_cluster_rank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
// shared address of `local` (a shared address of this CTA) in the CTA of cluster rank `rank`
__device__ __forceinline__ uint32_t i8_mapa(uint32_t local, uint32_t rank) {
    uint32_t remote;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(local), "r"(rank));
    return remote;
}
__device__ __forceinline__ float i8_ld_cluster_f32(uint32_t addr) {
    float v;
    asm volatile("ld.shared::cluster.f32 %0, [%1];" : "=f"(v) : "r"(addr) : "memory");
    return v;
}
__device__ __forceinline__ void i8_st_cluster_v4(uint32_t addr, uint32_t a, uint32_t b, uint32_t c, uint32_t d) {
    asm volatile("st.shared::cluster.v4.u32 [%0], {%1,%2,%3,%4};" ::"r"(addr), "r"(a), "r"(b), "r"(c), "r"(d) : "memory");
}
__device__ __forceinline__ void i8_st_cluster_v2(uint32_t addr, uint32_t a, uint32_t b) {
    asm volatile("st.shared::cluster.v2.u32 [%0], {%1,%2};" ::"r"(addr), "r"(a), "r"(b) : "memory");
}
__device__ __forceinline__ void i8_st_cluster_u32(uint32_t addr, uint32_t a) {
    asm volatile("st.shared::cluster.u32 [%0], %1;" ::"r"(addr), "r"(a) : "memory");
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
__device__ __forceinline__ uint32_t lds_f32_bits(uint32_t addr) {
    uint32_t v;
    asm volatile("ld.shared.u32 %0, [%1];" : "=r"(v) : "r"(addr));
    return v;
}
__device__ __forceinline__ float lds_f32(uint32_t addr) {
    float v;
    asm volatile("ld.shared.f32 %0, [%1];" : "=f"(v) : "r"(addr));
    return v;
}
// zero-extended byte J of a word
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
__device__ __forceinline__ uint32_t pack_s8x4(int a, int b, int c, int d) {
    return (uint32_t)(a & 0xFF) | ((uint32_t)(b & 0xFF) << 8) | ((uint32_t)(c & 0xFF) << 16) | ((uint32_t)(d & 0xFF) << 24);
}

// Reader side of a record: the B fragment (k 4t..4t+3 | k 16+4t..) of scale group G, limb l, for lane-in-quad t
// sits at byte (4 G + t) * 16 + 8 l.  Which activation columns those k stand for is the format's business:
//   Q4_K        k-th byte of the 32-byte nibble pair  ->  slot t holds columns 8t..8t+7 of the group
//   Q4_0/Q8_0   slot t holds columns 4t..4t+3 and 16+4t..16+4t+3 of the block
// (any bijection works as long as the weights use the same one; these match the resident layouts).

// One Q4_K unit (256 weights) of the thread's two fragment rows.
//   wq0 / wq1  unit base of fragment rows g and g+8 (shared addresses)
//   rec[nt]    record of the activation row this lane's B column of tile nt belongs to (row g / 2);  xoff = 16 t + 8 limb
//   srec[nt]   record of the activation row this lane's accumulator columns belong to (row t): its slice scale
// Q5_K (Q5 = true): the same super-block with a 32-byte field of high bits between the header and the quant bytes (bit g of
// byte j is bit 4 of weight j of group g, src/weight/codec/ggml.rs:425-447).  The five-bit code no longer fits the
// "16 q in place" trick of the high-nibble groups, so both groups of a pair are brought down to plain codes 0..31.
template <int NT, bool Q5 = false>
__device__ __forceinline__ void consume_q4k_i8(uint32_t wq0, uint32_t wq1, int t, const uint32_t (&rec)[NT], const uint32_t (&srec)[NT], uint32_t xoff, float (&yacc)[NT][2]) {
    constexpr uint32_t QS = Q5 ? 48 : 16;  // byte offset of the quant bytes inside the unit
    const uint4 hdr0 = lds128(wq0), hdr1 = lds128(wq1);
    uint2 q0[4], q1[4];
#pragma unroll
    for (int pr = 0; pr < 4; ++pr) {
        q0[pr] = lds64(wq0 + QS + 32 * pr + 8 * t);
        q1[pr] = lds64(wq1 + QS + 32 * pr + 8 * t);
    }
    uint2 h0 = make_uint2(0, 0), h1 = make_uint2(0, 0);
    if constexpr (Q5) {
        h0 = lds64(wq0 + 16 + 8 * t);
        h1 = lds64(wq1 + 16 + 8 * t);
    }
    // bit `g` of every byte of h, moved to bit 4
    auto hbit = [](uint32_t h, int g) -> uint32_t { return (g <= 4 ? (h << (4 - g)) : (h >> (g - 4))) & 0x10101010u; };
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
            bl[nt] = lds64(rec[nt] + xoff + (2 * pr) * 64);
            bh[nt] = lds64(rec[nt] + xoff + (2 * pr + 1) * 64);
        }
        const uint32_t s0w = pr < 2 ? sc_lo0 : sc_hi0, s1w = pr < 2 ? sc_lo1 : sc_hi1;
        {
            const int s0 = (pr & 1) ? byte_of<2>(s0w) : byte_of<0>(s0w), s1 = (pr & 1) ? byte_of<2>(s1w) : byte_of<0>(s1w);
            uint32_t a0 = q0[pr].x & 0x0F0F0F0Fu, a1 = q1[pr].x & 0x0F0F0F0Fu, a2 = q0[pr].y & 0x0F0F0F0Fu, a3 = q1[pr].y & 0x0F0F0F0Fu;
            if constexpr (Q5) {
                a0 |= hbit(h0.x, 2 * pr); a1 |= hbit(h1.x, 2 * pr); a2 |= hbit(h0.y, 2 * pr); a3 |= hbit(h1.y, 2 * pr);
            }
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
            uint32_t a0, a1, a2, a3;
            if constexpr (Q5) {  // plain codes; the factor 16 the epilogue expects of this half is put on the scale instead
                a0 = ((q0[pr].x >> 4) & 0x0F0F0F0Fu) | hbit(h0.x, 2 * pr + 1); a1 = ((q1[pr].x >> 4) & 0x0F0F0F0Fu) | hbit(h1.x, 2 * pr + 1);
                a2 = ((q0[pr].y >> 4) & 0x0F0F0F0Fu) | hbit(h0.y, 2 * pr + 1); a3 = ((q1[pr].y >> 4) & 0x0F0F0F0Fu) | hbit(h1.y, 2 * pr + 1);
            } else {
                a0 = q0[pr].x & 0xF0F0F0F0u; a1 = q1[pr].x & 0xF0F0F0F0u; a2 = q0[pr].y & 0xF0F0F0F0u; a3 = q1[pr].y & 0xF0F0F0F0u;
            }
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
            // both limb columns of a row read the row's sums; only the hi-limb column's result is used
            const uint2 sx = lds64(rec[nt] + kRecSums + 8 * t);
            mma_16816_zero(d2[nt], ma0k, ma1k, ma0, ma1, sx.x, sx.y);
        }
    }
    const __half2 dd0 = u32_as_h2(hdr0.x), dd1 = u32_as_h2(hdr1.x);
    constexpr float kHalfPre = Q5 ? 1.f : 0.0625f;  // Q4_K's high-nibble groups carry 16 q
    constexpr int kLowShift = Q5 ? 0 : 4;
    const float d_0 = __low2float(dd0) * kHalfPre, dm_0 = __high2float(dd0), d_1 = __low2float(dd1) * kHalfPre, dm_1 = __high2float(dd1);
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) {
        // columns 2t / 2t+1 of the tile are the hi / lo limb of one activation row
        const float sa = lds_f32(srec[nt] + kRecScale);
        const float f0 = (float)((tl[nt][0] << kLowShift) + th[nt][0]) * 256.f + (float)((tl[nt][1] << kLowShift) + th[nt][1]);
        const float f1 = (float)((tl[nt][2] << kLowShift) + th[nt][2]) * 256.f + (float)((tl[nt][3] << kLowShift) + th[nt][3]);
        yacc[nt][0] += sa * (d_0 * f0 - dm_0 * d2[nt][0]);
        yacc[nt][1] += sa * (d_1 * f1 - dm_1 * d2[nt][2]);
    }
}

// IQ4_NL: the 8 codebook values (src/weight/codec/ggml.rs:4) of one packed word as two s8x4 operands, `lo` for the four
// low nibbles and `hi` for the four high nibbles.  PRMT is the table lookup: its selector's low 16 bits are four
// nibbles, each picking one of 8 table bytes by its low three bits, so the low half-word looks up [lo0, hi0, lo1, hi1]
// in both halves of the table; the nibble's top bit (spread to a byte mask by PRMT's sign-replicate mode) picks between
// the halves; two more PRMTs put the low-nibble and the high-nibble results into words of their own.
__device__ __forceinline__ uint32_t prmt_b32(uint32_t a, uint32_t b, uint32_t sel) {
    uint32_t r;
    asm("prmt.b32 %0, %1, %2, %3;" : "=r"(r) : "r"(a), "r"(b), "r"(sel));
    return r;
}
__device__ __forceinline__ uint32_t lop3_select(uint32_t mask, uint32_t on, uint32_t off) {  // (mask & on) | (~mask & off)
    uint32_t r;
    asm("lop3.b32 %0, %1, %2, %3, 0xCA;" : "=r"(r) : "r"(mask), "r"(on), "r"(off));
    return r;
}
__device__ __forceinline__ void iq4nl_lookup(uint32_t w, uint32_t &lo, uint32_t &hi) {
    constexpr uint32_t T0 = 0xBFAD9881u, T1 = 0xF6EADDCFu, T2 = 0x26190D01u, T3 = 0x71594535u;  // -127 .. 113 as s8
    const uint32_t ws = w & 0x77777777u, w4 = w << 4;
    const uint32_t x = lop3_select(prmt_b32(w4, w, 0xD9C8u), prmt_b32(T2, T3, ws), prmt_b32(T0, T1, ws));
    const uint32_t ws2 = ws >> 16;
    const uint32_t y = lop3_select(prmt_b32(w4, w, 0xFBEAu), prmt_b32(T2, T3, ws2), prmt_b32(T0, T1, ws2));
    lo = prmt_b32(x, y, 0x6420u);
    hi = prmt_b32(x, y, 0x7531u);
}

// m16n8k16, s8 x s8 -> s32: one 16-weight scale group of the thread's two fragment rows (a0: row g, a1: row g + 8; k 4t..4t+3).
__device__ __forceinline__ void imma_16816_s8(int (&d)[4], uint32_t a0, uint32_t a1, uint32_t b0) {
    asm("mma.sync.aligned.m16n8k16.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5}, {%6}, {%7,%7,%7,%7};"
        : "=r"(d[0]), "=r"(d[1]), "=r"(d[2]), "=r"(d[3])
        : "r"(a0), "r"(a1), "r"(b0), "r"(0));
}
// sign-extended byte J of a word
template <int J> __device__ __forceinline__ int sbyte_of(uint32_t w) {
    uint32_t r;
    asm("prmt.b32 %0, %1, %2, %3;" : "=r"(r) : "r"(w), "r"(0u), "n"(0x8880 + 0x1111 * J));
    return (int)r;
}

// One Q6_K unit (re-laid, kQ6k* in zq_common.cuh) of the thread's two fragment rows.  Codes are stored as 6-bit two's
// complement (q - 32); moved to the top six bits of a byte they are the s8 value 4 (q - 32), so no sign extension is
// needed and the factor 4 goes onto d.  One m16n8k16 MMA per 16-column scale group; the i8 group scales multiply the s32
// results.  Records are those of the block-32 formats (slot t of block G: columns 4t..4t+3 and 16+4t..16+4t+3).
template <int NT>
__device__ __forceinline__ void consume_q6k_i8(uint32_t wq0, uint32_t wq1, int t, const uint32_t (&rec)[NT], const uint32_t (&srec)[NT], uint32_t xoff, float (&yacc)[NT][2]) {
    const uint32_t d0w = lds_f32_bits(wq0), d1w = lds_f32_bits(wq1);
    const uint4 s0 = lds128(wq0 + kQ6kScales), s1 = lds128(wq1 + kQ6kScales);
    const uint4 l0a = lds128(wq0 + kQ6kLow + 32 * t), l0b = lds128(wq0 + kQ6kLow + 32 * t + 16), l1a = lds128(wq1 + kQ6kLow + 32 * t), l1b = lds128(wq1 + kQ6kLow + 32 * t + 16);
    const uint4 h0 = lds128(wq0 + kQ6kHigh + 16 * t), h1 = lds128(wq1 + kQ6kHigh + 16 * t);
    const uint32_t lo0[8] = {l0a.x, l0a.y, l0a.z, l0a.w, l0b.x, l0b.y, l0b.z, l0b.w}, lo1[8] = {l1a.x, l1a.y, l1a.z, l1a.w, l1b.x, l1b.y, l1b.z, l1b.w};
    const uint32_t hi0[4] = {h0.x, h0.y, h0.z, h0.w}, hi1[4] = {h1.x, h1.y, h1.z, h1.w};
    const uint32_t sc0[4] = {s0.x, s0.y, s0.z, s0.w}, sc1[4] = {s1.x, s1.y, s1.z, s1.w};
    int tot[NT][4];
#pragma unroll
    for (int nt = 0; nt < NT; ++nt)
#pragma unroll
        for (int j = 0; j < 4; ++j) tot[nt][j] = 0;
#pragma unroll
    for (int G = 0; G < 8; ++G) {
        uint2 b[NT];
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) b[nt] = lds64(rec[nt] + xoff + G * 64);
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            const int x = 2 * (G & 1) + h;  // which bit pair of the high-bits word
            const uint32_t n0 = h ? (lo0[G] & 0xF0F0F0F0u) >> 2 : (lo0[G] & 0x0F0F0F0Fu) << 2;
            const uint32_t n1 = h ? (lo1[G] & 0xF0F0F0F0u) >> 2 : (lo1[G] & 0x0F0F0F0Fu) << 2;
            const uint32_t a0 = lop3_select(0xC0C0C0C0u, hi0[G >> 1] << (6 - 2 * x), n0), a1 = lop3_select(0xC0C0C0C0u, hi1[G >> 1] << (6 - 2 * x), n1);
            const int g16 = 2 * G + h;
            const int k0 = (g16 & 3) == 0 ? sbyte_of<0>(sc0[g16 >> 2]) : (g16 & 3) == 1 ? sbyte_of<1>(sc0[g16 >> 2]) : (g16 & 3) == 2 ? sbyte_of<2>(sc0[g16 >> 2]) : sbyte_of<3>(sc0[g16 >> 2]);
            const int k1 = (g16 & 3) == 0 ? sbyte_of<0>(sc1[g16 >> 2]) : (g16 & 3) == 1 ? sbyte_of<1>(sc1[g16 >> 2]) : (g16 & 3) == 2 ? sbyte_of<2>(sc1[g16 >> 2]) : sbyte_of<3>(sc1[g16 >> 2]);
#pragma unroll
            for (int nt = 0; nt < NT; ++nt) {
                int d[4];
                imma_16816_s8(d, a0, a1, h ? b[nt].y : b[nt].x);
                tot[nt][0] += d[0] * k0;
                tot[nt][1] += d[1] * k0;
                tot[nt][2] += d[2] * k1;
                tot[nt][3] += d[3] * k1;
            }
        }
    }
    const float d_0 = __half2float(__ushort_as_half((unsigned short)(d0w & 0xFFFFu))) * 0.25f, d_1 = __half2float(__ushort_as_half((unsigned short)(d1w & 0xFFFFu))) * 0.25f;
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) {
        const float sa = lds_f32(srec[nt] + kRecScale);
        yacc[nt][0] += (sa * d_0) * ((float)tot[nt][0] * 256.f + (float)tot[nt][1]);
        yacc[nt][1] += (sa * d_1) * ((float)tot[nt][2] * 256.f + (float)tot[nt][3]);
    }
}

// One block-32 unit (8 blocks of 32 weights) of the thread's two fragment rows: Q4_0, IQ4_NL or Q8_0.
template <uint32_t TYPE, int NT>
__device__ __forceinline__ void consume_b32_i8(uint32_t wq0, uint32_t wq1, int t, const uint32_t (&rec)[NT], const uint32_t (&srec)[NT], uint32_t xoff, float (&yacc)[NT][2]) {
    constexpr int H = TYPE == ZQ_Q8_0 ? 4 : 2;     // 16-byte pieces per lane
    constexpr int BPP = TYPE == ZQ_Q8_0 ? 2 : 4;   // blocks per piece
    constexpr float kPre = TYPE == ZQ_Q4_0 ? 0.0625f : 1.f;
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
    for (int nt = 0; nt < NT; ++nt) sap[nt] = lds_f32(srec[nt] + kRecScale) * kPre;
#pragma unroll
    for (int h = 0; h < H; ++h) {
        const uint32_t q0[4] = {pc0[h].x, pc0[h].y, pc0[h].z, pc0[h].w};
        const uint32_t q1[4] = {pc1[h].x, pc1[h].y, pc1[h].z, pc1[h].w};
        uint2 b[BPP][NT];
#pragma unroll
        for (int bb = 0; bb < BPP; ++bb)
#pragma unroll
            for (int nt = 0; nt < NT; ++nt) b[bb][nt] = lds64(rec[nt] + xoff + (BPP * h + bb) * 64);
#pragma unroll
        for (int bb = 0; bb < BPP; ++bb) {
            const int blk = BPP * h + bb;
            uint32_t a0, a1, a2, a3;
            if constexpr (TYPE == ZQ_Q8_0) {
                a0 = q0[2 * bb]; a1 = q1[2 * bb]; a2 = q0[2 * bb + 1]; a3 = q1[2 * bb + 1];
            } else if constexpr (TYPE == ZQ_IQ4_NL) {
                iq4nl_lookup(q0[bb], a0, a2);
                iq4nl_lookup(q1[bb], a1, a3);
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


// Eight consecutive activation columns starting at element offset o, as f32 (zeros when !valid).
__device__ __forceinline__ void load_act8(const void *x, int x_dtype, size_t o, bool valid, float (&v)[8]) {
#pragma unroll
    for (int j = 0; j < 8; ++j) v[j] = 0.f;
    if (!valid) return;
    if (x_dtype == ZQ_F32) {
        const float4 f0 = *reinterpret_cast<const float4 *>(reinterpret_cast<const float *>(x) + o);
        const float4 f1 = *reinterpret_cast<const float4 *>(reinterpret_cast<const float *>(x) + o + 4);
        v[0] = f0.x; v[1] = f0.y; v[2] = f0.z; v[3] = f0.w; v[4] = f1.x; v[5] = f1.y; v[6] = f1.z; v[7] = f1.w;
    } else {
        const uint4 raw = *reinterpret_cast<const uint4 *>(reinterpret_cast<const uint16_t *>(x) + o);
        const uint32_t rw[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            if (x_dtype == ZQ_F16) {
                const float2 f = __half22float2(u32_as_h2(rw[j]));
                v[2 * j] = f.x; v[2 * j + 1] = f.y;
            } else {  // bf16: the upper half of an f32
                v[2 * j] = __uint_as_float(rw[j] << 16);
                v[2 * j + 1] = __uint_as_float(rw[j] & 0xFFFF0000u);
            }
        }
    }
}

// What one lane contributes to a record: its 16-byte fragment slot, and (some lanes) group sums and the scale.
struct RecLane {
    uint32_t ph0, ph1, pl0, pl1;  // hi-limb pair, lo-limb pair
    uint32_t slot;                // byte offset of the 16-byte slot inside the record
    uint32_t sw0, sw1;            // Q4_K, lanes with lane % 8 == 0: min-term fragment entry lane / 8
    float scale;                  // lane 0: slice scale
};

// Quantises one record (256 columns of one activation row; the lane holds columns 8 lane .. 8 lane + 7).  All 32
// lanes of the warp must call it together.
template <uint32_t TYPE> __device__ __forceinline__ RecLane quantize_record(const float (&v)[8], int lane) {
    RecLane o;
    float amax = 0.f;
#pragma unroll
    for (int j = 0; j < 8; ++j) amax = fmaxf(amax, fabsf(v[j]));
#pragma unroll
    for (int s = 16; s >= 1; s >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, s));
    const bool live = amax > 0.f && amax < 3.0e38f;
    const float inv = live ? __fdividef(kActMax, amax) : 0.f;
    o.scale = live ? __fdividef(1.f, inv) : 0.f;  // the scale actually applied: x ~ x_q / inv
    int hi[8], lo[8], sum = 0;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
        int xq = __float2int_rn(v[j] * inv);
        xq = xq > 32512 ? 32512 : (xq < -32512 ? -32512 : xq);
        hi[j] = (xq + 128) >> 8;
        lo[j] = xq - (hi[j] << 8);
        sum += xq;
    }
    // the lane's two quads (columns 8 lane .. +3 and +4 .. +7) as packed limbs
    o.ph0 = pack_s8x4(hi[0], hi[1], hi[2], hi[3]); o.ph1 = pack_s8x4(hi[4], hi[5], hi[6], hi[7]);
    o.pl0 = pack_s8x4(lo[0], lo[1], lo[2], lo[3]); o.pl1 = pack_s8x4(lo[4], lo[5], lo[6], lo[7]);
    if constexpr (is_kclass(TYPE)) {
        o.slot = (uint32_t)lane * 16;  // group lane / 4, slot t = lane % 4: both quads are this lane's
    } else {
        // block lane / 4; the quads are (slot 2 (lane & 1) + qd, register r) with r = (lane >> 1) & 1: trade the quad of
        // the other slot for the partner's quad of this slot
        const int r = (lane >> 1) & 1;
        const uint32_t got_h = __shfl_xor_sync(0xffffffffu, r ? o.ph0 : o.ph1, 2), got_l = __shfl_xor_sync(0xffffffffu, r ? o.pl0 : o.pl1, 2);
        const uint32_t keep_h = r ? o.ph1 : o.ph0, keep_l = r ? o.pl1 : o.pl0;
        o.ph0 = r ? got_h : keep_h; o.ph1 = r ? keep_h : got_h;
        o.pl0 = r ? got_l : keep_l; o.pl1 = r ? keep_l : got_l;
        o.slot = (uint32_t)(4 * (lane >> 2) + 2 * (lane & 1) + r) * 16;
    }
    o.sw0 = o.sw1 = 0;
    if constexpr (is_kclass(TYPE)) {
        // exact integer sum of each 32-column group: |sum| can reach 32 * 32512, beyond f16, so sum = 1024 a + r with
        // |a| <= 1016, |r| <= 512, both exact in f16; the factor 1024 rides on the min codes of the hi-limb K slots.
        // Fragment entry t' = {half2(a_2t', a_2t'+1), half2(r_2t', r_2t'+1)}.
        sum += __shfl_xor_sync(0xffffffffu, sum, 1);
        sum += __shfl_xor_sync(0xffffffffu, sum, 2);
        const int a = (sum + 512) >> 10, r = sum - (a << 10);
        const int oa = __shfl_xor_sync(0xffffffffu, a, 4), orr = __shfl_xor_sync(0xffffffffu, r, 4);
        o.sw0 = h2_as_u32(__halves2half2(__int2half_rn(a), __int2half_rn(oa)));
        o.sw1 = h2_as_u32(__halves2half2(__int2half_rn(r), __int2half_rn(orr)));
    }
    return o;
}


}  // namespace zq
