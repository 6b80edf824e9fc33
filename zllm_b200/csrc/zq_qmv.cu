// Decode GEMV on the 5th-generation tensor cores: packed Q4_K rows -> exact integer f16 operand in TENSOR MEMORY ->
// tcgen05.mma against the activation limbs, per-super-block rescale in registers.  sm_100a.
//
// Why: the warp-level mma.sync path (zq_gemv*.cu) is limited on B200 by the legacy tensor pipe (one m16n8k16 per
// ~16 cycles per SM sub-partition) and by the fragment bookkeeping around it.  One tcgen05.mma covers 128 weight
// rows x 16 K-columns at a time, reads its A operand straight from tensor memory and needs no fragment shuffling,
// so the only per-weight work left is turning nibbles into f16 numbers.
//
// Operator contract and arithmetic are those of zq_gemv.cu (ggml_quant::matvec / matvec_residual,
// src/kernel/cpu/ggml_quant.rs:189-233): for every super-block the tensor core accumulates
//   D1 = sum_k (scale_g * quant_k) * x_k          (integers up to 945, exact in f16; x as two f16 limbs)
//   D2 = sum_g min_g * (sum_{k in g} x_k)          (one extra K=16 MMA against per-group activation sums)
// in f32, and the row's thread adds d * D1 - dmin * D2 to its running sums: the result carries f32-level accuracy.
//
// CTA = 13 warps, one CTA per SM, persistent over a contiguous range of work items (item = 128 rows x 1 super-block
// column, tile-major; split tiles are finished by the last arriving CTA in fixed order):
//   warp 0      TMA: packed rows of the next items into a 10-stage ring (box 36 words x 128 rows)
//   warp 1      owns tensor memory; one lane issues 17 tcgen05.mma per item (rotating over 4 accumulators) and commits
//   warps 2-4   activation staging: each handles every 3rd item: loads the item's 256 columns of up to 8 rows,
//               splits them into f16 limbs, writes the B operand (no-swizzle K-major core matrices) and the
//               per-group sums, fence.proxy.async, signals
//   warps 5-12  two dequant groups of 4 warps (one TMEM lane quarter each), alternating items: thread = weight row;
//               16-byte shared loads of its 144-byte super-block, nibble -> f16 by bit tricks, tcgen05.st into the
//               group's A buffer, signal; the item's accumulators are collected (tcgen05.ld, rescale) one own item
//               later, so the group does not wait for the tensor core right after feeding it.
// Status: parity-clean; measured slower than the warp-MMA kernels (its handshake chain costs more than the MMA
// bookkeeping it removes), so zq_linear uses it only when the context option enable_tcgen05_gemv is set.
// The order of K inside an MMA is free, so the A columns keep the order the bit tricks produce and the staging
// warps write the activations in the same order.
// Every wait is bounded and watches a CTA-wide abort flag; after an abort all roles keep walking their loops
// without waiting, so every barrier is still reached, tensor memory is released and the status word is set.
#include "zq_gemv_frag.cuh"

namespace zq {

constexpr int kQmvThreads = 13 * 32;
constexpr int kQmvRows = 8;  // activation rows per launch (two f16 limbs each fill the 16 MMA columns)
constexpr int kQmvWStages = 10;  // ~170 KB of packed rows in flight per SM: HBM latency x bandwidth needs that much
constexpr int kQmvXStages = 3;
constexpr int kQmvXWarps = 3;
constexpr int kQmvB1Bytes = 16 * 256 * 2;   // 16 operand rows (8 activation rows x 2 limbs) x 256 K
constexpr int kQmvB2Bytes = 16 * 16 * 2;    // 16 operand rows x 16 (8 group sums + 8 zero)
constexpr int kQmvXStageBytes = kQmvB1Bytes + kQmvB2Bytes;
constexpr int kQmvWStageBytes = kTileRows * 144;
constexpr int kQmvRedFloats = 2 * 2 * kQmvRows * kTileRows;  // [tile parity][group][row of x][weight row]
constexpr int kQmvOffX = kQmvWStages * kQmvWStageBytes;
constexpr int kQmvOffRed = kQmvOffX + kQmvXStages * kQmvXStageBytes;
constexpr int kQmvOffBar = kQmvOffRed + kQmvRedFloats * 4;
constexpr int kQmvSmem = kQmvOffBar + 512 + 1024;
// tensor memory columns (512 allocated): A buffers of the two groups, min-code operands, accumulators
// (the 16 dependent MMAs of an item would be latency-bound on one accumulator, so they rotate over 4)
constexpr uint32_t kTmA1 = 0, kTmA2 = 256, kTmD2 = 288, kTmD1 = 320;
constexpr int kQmvAcc = 4;

__device__ __forceinline__ void tmem_st32(uint32_t taddr, const uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31,%32};"
        ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]),
        "r"(r[16]), "r"(r[17]), "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]), "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
        : "memory");
}
__device__ __forceinline__ void tmem_st8(uint32_t taddr, const uint32_t (&r)[8]) {
    asm volatile("tcgen05.st.sync.aligned.32x32b.x8.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8};" ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]) : "memory");
}
__device__ __forceinline__ void tmem_st_wait() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tmem_ld16q(uint32_t taddr, float (&v)[16]) {
    uint32_t r[16];
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]),
                   "=r"(r[14]), "=r"(r[15])
                 : "r"(taddr)
                 : "memory");
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
    for (int j = 0; j < 16; ++j) v[j] = __uint_as_float(r[j]);
}
__device__ __forceinline__ void qmv_tmem_alloc(uint32_t *slot, uint32_t cols) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(slot)), "r"(cols) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void qmv_tmem_dealloc(uint32_t taddr, uint32_t cols) { asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(cols) : "memory"); }
__device__ __forceinline__ void qmv_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void qmv_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void qmv_commit(uint64_t *bar) { asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar)) : "memory"); }
// D[tmem] (+)= A[tmem] * B[smem descriptor]
__device__ __forceinline__ void umma_f16_ts(uint32_t tmem_d, uint32_t tmem_a, uint64_t desc_b, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}"
        ::"r"(tmem_d), "r"(tmem_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
        : "memory");
}
// K-major operand without swizzle: 8-row x 16-byte core matrices; next core matrix along K is 256 bytes away
// (leading byte offset), next 8-row group 128 bytes away (stride byte offset).
__device__ __forceinline__ uint64_t make_nosw_desc(uint32_t smem_addr) {
    uint64_t desc = 0;
    desc |= (uint64_t)((smem_addr & 0x3FFFFu) >> 4);
    desc |= (uint64_t)(256 >> 4) << 16;
    desc |= (uint64_t)(128 >> 4) << 32;
    desc |= (uint64_t)1 << 46;
    return desc;
}
__device__ __forceinline__ void named_bar(int id, int threads) { asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(threads) : "memory"); }

__device__ __forceinline__ void qmv_wait(uint64_t *bar, uint32_t parity, volatile int *abort_flag, uint32_t *status, uint32_t code) {
    if (*abort_flag) return;
    for (uint32_t i = 0; i < (1u << 22); ++i) {
        if (mbar_try_wait(bar, parity)) return;
        if (*abort_flag) return;
    }
    *abort_flag = 1;
    atomicMax(status, code);
}

__global__ void __launch_bounds__(kQmvThreads, 1) qmv_q4k_kernel(const __grid_constant__ CUtensorMap map_w, const GemvParams p) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t *ws = smem;
    uint8_t *xs = smem + kQmvOffX;
    float *red = reinterpret_cast<float *>(smem + kQmvOffRed);
    uint64_t *w_full = reinterpret_cast<uint64_t *>(smem + kQmvOffBar);
    uint64_t *w_empty = w_full + kQmvWStages;
    uint64_t *x_full = w_empty + kQmvWStages;
    uint64_t *x_empty = x_full + kQmvXStages;
    uint64_t *a_full = x_empty + kQmvXStages;
    uint64_t *d_full = a_full + 2;
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(d_full + 2);
    __shared__ int s_abort;
    __shared__ int s_flag;

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int units = p.chunks;  // super-blocks per row (this kernel's chunk is one unit)
    const long long T = (long long)p.tiles * units;
    const long long G = gridDim.x;
    const long long begin = (long long)blockIdx.x * T / G;
    const long long end = (long long)(blockIdx.x + 1) * T / G;
    const int n_items = (int)(end - begin);

    if (tid == 0) {
        for (int s = 0; s < kQmvWStages; ++s) { mbar_init(&w_full[s], 1); mbar_init(&w_empty[s], 4); }
        for (int s = 0; s < kQmvXStages; ++s) { mbar_init(&x_full[s], 1); mbar_init(&x_empty[s], 1); }
        for (int s = 0; s < 2; ++s) { mbar_init(&a_full[s], 4); mbar_init(&d_full[s], 1); }
        fence_mbar_init();
        tma_prefetch_desc(&map_w);
        s_abort = 0;
    }
    // activation ring starts zeroed: operand rows of absent activation rows must read as zero
    for (int i = tid; i < kQmvXStages * kQmvXStageBytes / 16; i += kQmvThreads) reinterpret_cast<uint4 *>(xs)[i] = make_uint4(0, 0, 0, 0);
    if (warp == 1) qmv_tmem_alloc(tmem_slot, 512);
    fence_proxy_async();
    qmv_fence_before();
    __syncthreads();
    qmv_fence_after();
    const uint32_t tmem_base = *reinterpret_cast<volatile uint32_t *>(tmem_slot);
    volatile int *abort_flag = &s_abort;

    if (warp == 0) {
        // ------------------------------------------------ TMA producer
        if (lane == 0) {
            for (int it = 0; it < n_items; ++it) {
                const int s = it % kQmvWStages;
                if (it >= kQmvWStages) qmv_wait(&w_empty[s], ((it / kQmvWStages) - 1) & 1, abort_flag, p.status, kStatusTmaTimeout);
                if (*abort_flag) break;
                const long long item = begin + it;
                const int tile = (int)(item / units), unit = (int)(item % units);
                mbar_expect_tx(&w_full[s], kQmvWStageBytes);
                tma_load_2d(ws + (size_t)s * kQmvWStageBytes, &map_w, &w_full[s], unit * 36, tile * kTileRows);
            }
        }
    } else if (warp == 1) {
        // ------------------------------------------------ MMA issuer
        if (lane == 0) {
            const uint32_t idesc = (1u << 4) | ((uint32_t)(16 >> 3) << 17) | ((uint32_t)(128 >> 4) << 24);  // f32 acc, f16 x f16, N=16, M=128
            for (int it = 0; it < n_items; ++it) {
                const int wg = it & 1, xsidx = it % kQmvXStages;
                qmv_wait(&a_full[wg], (it >> 1) & 1, abort_flag, p.status, kStatusMmaTimeout);
                qmv_wait(&x_full[xsidx], (it / kQmvXStages) & 1, abort_flag, p.status, kStatusMmaTimeout);
                if (*abort_flag) break;
                qmv_fence_after();
                const uint32_t xb = smem_u32(xs + (size_t)xsidx * kQmvXStageBytes);
                const uint64_t db1 = make_nosw_desc(xb), db2 = make_nosw_desc(xb + kQmvB1Bytes);
                const uint32_t d1 = tmem_base + kTmD1 + 16 * kQmvAcc * wg, d2 = tmem_base + kTmD2 + 16 * wg;
                const uint32_t a1 = tmem_base + kTmA1 + 128 * wg, a2 = tmem_base + kTmA2 + 16 * wg;
#pragma unroll
                for (int k = 0; k < 16; ++k) umma_f16_ts(d1 + 16 * (k % kQmvAcc), a1 + 8 * k, db1 + (uint64_t)(32 * k), idesc, k >= kQmvAcc ? 1u : 0u);  // 16 K = 8 columns of A, 512 bytes of B
                umma_f16_ts(d2, a2, db2, idesc, 0u);
                qmv_commit(&d_full[wg]);
                qmv_commit(&x_empty[xsidx]);
            }
        }
    } else if (warp < 2 + kQmvXWarps) {
        // ------------------------------------------------ activation staging: warp w handles items it = w-2, w+2, ...
        // (every 4th item); the item's activations are fetched into registers one item ahead, so the global-load
        // latency never sits between "stage released" and "stage refilled".
        const int xw = warp - 2;
        const int a = lane;  // 8-column chunk of the unit: columns 8a .. 8a+7 (group a/4, words 2(a%4), 2(a%4)+1)
        const int g = a >> 2, i0 = 2 * (a & 3);
        float v[kQmvRows][8];
        auto fetch = [&](int it) {
            const long long item = begin + it;
            const int unit = (int)(item % units);
            const size_t k0 = (size_t)unit * 256 + 8 * a;
#pragma unroll
            for (int m = 0; m < kQmvRows; ++m) {
                if (m < p.m) {
                    const size_t o = (size_t)m * p.cols + k0;
                    if (p.x_dtype == ZQ_F32) {
                        const float4 f0 = *reinterpret_cast<const float4 *>(reinterpret_cast<const float *>(p.x) + o);
                        const float4 f1 = *reinterpret_cast<const float4 *>(reinterpret_cast<const float *>(p.x) + o + 4);
                        v[m][0] = f0.x; v[m][1] = f0.y; v[m][2] = f0.z; v[m][3] = f0.w; v[m][4] = f1.x; v[m][5] = f1.y; v[m][6] = f1.z; v[m][7] = f1.w;
                    } else {
#pragma unroll
                        for (int j = 0; j < 8; ++j) v[m][j] = load_as_f32(p.x, p.x_dtype, o + j);
                    }
                }
            }
        };
        if (xw < n_items) fetch(xw);
        for (int it = xw; it < n_items; it += kQmvXWarps) {
            const int xsidx = it % kQmvXStages;
            uint8_t *stage = xs + (size_t)xsidx * kQmvXStageBytes;
            if (it >= kQmvXStages) qmv_wait(&x_empty[xsidx], ((it / kQmvXStages) - 1) & 1, abort_flag, p.status, kStatusMmaTimeout);
#pragma unroll
            for (int m = 0; m < kQmvRows; ++m) {
                if (m < p.m) {
                    __half hi[8], lo[8];
                    float sum = 0.f;
#pragma unroll
                    for (int j = 0; j < 8; ++j) {
                        hi[j] = __float2half_rn(v[m][j]);
                        lo[j] = __float2half_rn(v[m][j] - __half2float(hi[j]));
                        sum += v[m][j];
                    }
                    const int nh = 2 * m, nl = 2 * m + 1;
#pragma unroll
                    for (int wv = 0; wv < 2; ++wv) {
                        // word i of the group: its 4 columns land in 4 consecutive K slots in the order (e0, e2, e1, e3)
                        const int i = i0 + wv;
                        const int off = (8 * (g >> 1) + i) * 256 + 8 * (g & 1);
                        const uint2 qh = make_uint2(h2_as_u32(__halves2half2(hi[4 * wv + 0], hi[4 * wv + 2])), h2_as_u32(__halves2half2(hi[4 * wv + 1], hi[4 * wv + 3])));
                        const uint2 ql = make_uint2(h2_as_u32(__halves2half2(lo[4 * wv + 0], lo[4 * wv + 2])), h2_as_u32(__halves2half2(lo[4 * wv + 1], lo[4 * wv + 3])));
                        *reinterpret_cast<uint2 *>(stage + off + (nh >> 3) * 128 + (nh & 7) * 16) = qh;
                        *reinterpret_cast<uint2 *>(stage + off + (nl >> 3) * 128 + (nl & 7) * 16) = ql;
                    }
                    sum += __shfl_xor_sync(0xffffffffu, sum, 1);
                    sum += __shfl_xor_sync(0xffffffffu, sum, 2);
                    if ((a & 3) == 0) {
                        const __half shi = __float2half_rn(sum), slo = __float2half_rn(sum - __half2float(__float2half_rn(sum)));
                        __half *b2 = reinterpret_cast<__half *>(stage + kQmvB1Bytes);
                        b2[((nh >> 3) * 128 + (nh & 7) * 16) / 2 + g] = shi;
                        b2[((nl >> 3) * 128 + (nl & 7) * 16) / 2 + g] = slo;
                    }
                }
            }
            fence_proxy_async();
            __syncwarp();
            if (lane == 0) mbar_arrive(&x_full[xsidx]);
            if (it + kQmvXWarps < n_items) fetch(it + kQmvXWarps);
        }
    } else {
        // ------------------------------------------------ dequant + epilogue groups
        const int wg = (warp - 2 - kQmvXWarps) >> 2;
        const int q = warp & 3;                      // TMEM lane quarter this warp may touch
        const int row_in_tile = q * 32 + lane;       // weight row of the tile = TMEM lane
        const int gtid = tid - (2 + kQmvXWarps) * 32;  // 0..255 over both groups
        const int wtid = gtid & 127;                 // 0..127 inside the group
        const uint32_t lane_addr = tmem_base + ((uint32_t)(q * 32) << 16);
        float yacc[16];
#pragma unroll
        for (int j = 0; j < 16; ++j) yacc[j] = 0.f;
        int tile_parity = 0;
        // The accumulators of an item are collected one own-item later (or at the end of the tile), so the group
        // never waits for the tensor core right after feeding it.
        float pend_d = 0.f, pend_dmin = 0.f;
        int pend_it = -1;
        auto collect = [&]() {
            if (pend_it < 0) return;
            qmv_wait(&d_full[wg], (pend_it >> 1) & 1, abort_flag, p.status, kStatusMmaTimeout);
            qmv_fence_after();
            float v1[16], v2[16];
            tmem_ld16q(lane_addr + kTmD1 + 16 * kQmvAcc * wg, v1);
#pragma unroll
            for (int c = 1; c < kQmvAcc; ++c) {
                tmem_ld16q(lane_addr + kTmD1 + 16 * kQmvAcc * wg + 16 * c, v2);
#pragma unroll
                for (int j = 0; j < 16; ++j) v1[j] += v2[j];
            }
            tmem_ld16q(lane_addr + kTmD2 + 16 * wg, v2);
#pragma unroll
            for (int j = 0; j < 16; ++j) yacc[j] += pend_d * v1[j] - pend_dmin * v2[j];
            qmv_fence_before();
            pend_it = -1;
        };

        for (int it = 0; it < n_items; ++it) {
            const long long item = begin + it;
            const int tile = (int)(item / units);
            if ((it & 1) == wg) {
                collect();  // previous own item: its MMAs were issued a whole item ago
                const int s = it % kQmvWStages;
                qmv_wait(&w_full[s], (it / kQmvWStages) & 1, abort_flag, p.status, kStatusTmaTimeout);
                const uint8_t *wrow = ws + (size_t)s * kQmvWStageBytes + (size_t)row_in_tile * 144;
                const uint4 hdr = *reinterpret_cast<const uint4 *>(wrow);
                const uint32_t k1024 = 0x64006400u, k64x4 = 0x64646464u, kNeg1024 = 0xE400E400u, kNeg64 = 0xD400D400u;
                const uint32_t sc_lo = hdr.y & 0x3F3F3F3Fu, sc_hi = (hdr.w & 0x0F0F0F0Fu) | ((hdr.y >> 2) & 0x30303030u);
                const uint32_t mn_lo = hdr.z & 0x3F3F3F3Fu, mn_hi = ((hdr.w >> 4) & 0x0F0F0F0Fu) | ((hdr.z >> 2) & 0x30303030u);
#pragma unroll
                for (int pr = 0; pr < 4; ++pr) {
                    // group pair pr: low nibbles -> group 2pr (bias 1024), high nibbles -> group 2pr+1 (bias 64)
                    const uint4 qa = *reinterpret_cast<const uint4 *>(wrow + 16 + 32 * pr);
                    const uint4 qb = *reinterpret_cast<const uint4 *>(wrow + 32 + 32 * pr);
                    const uint32_t scw = pr < 2 ? sc_lo : sc_hi;
                    const int b = 2 * (pr & 1);
                    const uint32_t sa = hsub2_u32(prmt(scw, k64x4, 0x4040u | (b * 0x0101u)), k1024);
                    const uint32_t sb = hsub2_u32(prmt(scw, k64x4, 0x4040u | ((b + 1) * 0x0101u)), k1024);
                    const uint32_t oa = hmul2_u32(sa, kNeg1024), ob = hmul2_u32(sb, kNeg64);
                    const uint32_t qw[8] = {qa.x, qa.y, qa.z, qa.w, qb.x, qb.y, qb.z, qb.w};
                    uint32_t r[32];
#pragma unroll
                    for (int i = 0; i < 8; ++i) {
                        const uint32_t x0 = qw[i], x0s = qw[i] >> 8;
                        r[4 * i + 0] = hfma2_u32(lop3_and_or(x0, 0x000F000Fu, 0x64006400u), sa, oa);    // elements 4i, 4i+2 of group 2pr
                        r[4 * i + 1] = hfma2_u32(lop3_and_or(x0s, 0x000F000Fu, 0x64006400u), sa, oa);   // elements 4i+1, 4i+3
                        r[4 * i + 2] = hfma2_u32(lop3_and_or(x0, 0x00F000F0u, 0x54005400u), sb, ob);    // same of group 2pr+1
                        r[4 * i + 3] = hfma2_u32(lop3_and_or(x0s, 0x00F000F0u, 0x54005400u), sb, ob);
                    }
                    if (pr == 3) {
                        __syncwarp();
                        if (lane == 0) mbar_arrive(&w_empty[s]);  // the packed rows of this stage are in registers now
                    }
                    tmem_st32(lane_addr + kTmA1 + 128 * wg + 32 * pr, r);
                }
                {
                    uint32_t r[8];
                    r[0] = hsub2_u32(prmt(mn_lo, k64x4, 0x4140u), k1024);  // (m0, m1)
                    r[1] = hsub2_u32(prmt(mn_lo, k64x4, 0x4342u), k1024);  // (m2, m3)
                    r[2] = hsub2_u32(prmt(mn_hi, k64x4, 0x4140u), k1024);  // (m4, m5)
                    r[3] = hsub2_u32(prmt(mn_hi, k64x4, 0x4342u), k1024);  // (m6, m7)
                    r[4] = r[5] = r[6] = r[7] = 0u;
                    tmem_st8(lane_addr + kTmA2 + 16 * wg, r);
                }
                tmem_st_wait();
                qmv_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(&a_full[wg]);
                const __half2 dd = u32_as_h2(hdr.x);
                pend_d = __low2float(dd);
                pend_dmin = __high2float(dd);
                pend_it = it;
            }

            // ---------------- end of a tile: both groups hand in their sums, group 0 stores or hands over
            const bool tile_ends = (it == n_items - 1) || ((int)((item + 1) / units) != tile);
            if (tile_ends) {
                collect();
                float *rb = red + (size_t)tile_parity * (2 * kQmvRows * kTileRows) + (size_t)wg * (kQmvRows * kTileRows);
#pragma unroll
                for (int m = 0; m < kQmvRows; ++m) {
                    rb[m * kTileRows + row_in_tile] = yacc[2 * m] + yacc[2 * m + 1];
                    yacc[2 * m] = yacc[2 * m + 1] = 0.f;
                }
                named_bar(1, 256);
                if (wg == 0) {
                    const float *r0p = red + (size_t)tile_parity * (2 * kQmvRows * kTileRows);
                    const float *r1p = r0p + kQmvRows * kTileRows;
                    const long long tile_first = (long long)tile * units, tile_last = tile_first + units - 1;
                    const bool whole = begin <= tile_first && tile_last < end;
                    const int c_first = (int)(((tile_first + 1) * G - 1) / T), c_last = (int)(((tile_last + 1) * G - 1) / T);
                    float vals[kQmvRows];
#pragma unroll
                    for (int m = 0; m < kQmvRows; ++m) vals[m] = r0p[m * kTileRows + row_in_tile] + r1p[m * kTileRows + row_in_tile];
                    bool finish = whole;
                    if (!whole) {
                        const int which = (tile == (int)(begin / units)) ? 0 : 1;
                        float *slot = p.partials + ((size_t)blockIdx.x * 2 + which) * kSlotFloats;
                        for (int m = 0; m < p.m; ++m) slot[m * kTileRows + row_in_tile] = vals[m];
                        named_bar(2, 128);
                        if (wtid == 0) {
                            __threadfence();  // the group's stores are ordered before this thread by the barrier; one fence publishes them
                            unsigned old = atomicAdd(&p.counters[tile], 1u);
                            s_flag = (old == (unsigned)(c_last - c_first)) ? 1 : 0;
                        }
                        named_bar(2, 128);
                        finish = s_flag != 0;
                        if (finish) {
                            __threadfence();
                            for (int m = 0; m < p.m; ++m) {
                                float v = 0.f;
                                for (int c = c_first; c <= c_last; ++c) {  // fixed order: deterministic
                                    long long cb = (long long)c * T / G;
                                    int wh = (tile == (int)(cb / units)) ? 0 : 1;
                                    v += __ldcg(p.partials + ((size_t)c * 2 + wh) * kSlotFloats + m * kTileRows + row_in_tile);
                                }
                                vals[m] = v;
                            }
                            if (wtid == 0) p.counters[tile] = 0;
                        }
                        named_bar(2, 128);  // s_flag is free for the next tile
                    }
                    if (finish) {
                        const int n = tile * kTileRows + row_in_tile;
                        if (n < p.n_out) {
                            for (int m = 0; m < p.m; ++m) {
                                const size_t o = (size_t)m * p.n_out + n;
                                float v = vals[m];
                                if (p.residual) v += load_as_f32(p.residual, p.y_dtype, o);
                                store_from_f32(p.y, p.y_dtype, o, v);
                            }
                        }
                    }
                }
                tile_parity ^= 1;
            }
        }
    }
    qmv_fence_before();
    __syncthreads();
    if (warp == 1) qmv_tmem_dealloc(tmem_base, 512);
}

// One launch for up to 8 activation rows of a Q4_K weight; `taken` is false when the shape is not eligible.
int launch_qmv(zq_ctx *ctx, const zq_weight *w, const GemvParams &p_in, bool &taken, zq_error *err) {
    taken = false;
    if (w->type != ZQ_Q4_K || p_in.m > kQmvRows || p_in.limbs != 2) return ZQ_OK;
    GemvParams p = p_in;
    p.chunks = (int)w->units_per_row;
    p.tiles = (int)((w->rows + kTileRows - 1) / kTileRows);
    if ((size_t)p.tiles > ctx->gemv_counters_n) return ZQ_OK;
    long long total = (long long)p.tiles * p.chunks;
    int grid = (int)(total < ctx->sm_count ? total : ctx->sm_count);
    if (grid <= 0) return ZQ_OK;
    static bool configured[64] = {};
    if (!configured[ctx->device & 63]) {
        ZQ_CUDA_CHECK(cudaFuncSetAttribute(qmv_q4k_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kQmvSmem), err);
        configured[ctx->device & 63] = true;
    }
    qmv_q4k_kernel<<<grid, kQmvThreads, kQmvSmem, ctx->stream>>>(w->qmv_map, p);
    ctx->launches++;
    ZQ_CUDA_CHECK(cudaGetLastError(), err);
    taken = true;
    return ZQ_OK;
}

}  // namespace zq
