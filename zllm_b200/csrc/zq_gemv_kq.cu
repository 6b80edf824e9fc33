// Decode GEMV for Q5_K and Q6_K (src/weight/codec/ggml.rs:425-469; the reference's CUDA kernels for these types:
// src/kernel/cuda/linear.rs:1167-1234, 1967-2101): up to 8 activation rows straight from the packed bytes, so that
// a one-row call (the Q6_K output head of a Q4_K_M file, a Q6_K down projection) streams 0.69 / 0.82 bytes per
// weight instead of dequantising the whole matrix to f16 first.
//
// One warp per weight row, f32 arithmetic on the CUDA cores.  A lane owns one 32-bit word of a super-block's low
// quant bytes: 4 consecutive positions of two scale groups (low nibbles, high nibbles) = 8 weights, whose integer
// codes are multiplied into up to 4 activation rows at a time and scaled once per group (the codec's value
// (d*sc)*q - dmin*m resp. (d*scale)*q, with the scale factored out of the 4-element sum); the 32 lanes read a super-block's 128 low bytes as one coalesced line.  Q6_K blocks are 210 bytes, so their
// fields are only 2-byte aligned and are read as 16-bit loads.  Activations come through the read-only cache (a
// row of K floats is shared by all warps of the SM).  Sums are combined by warp shuffles; no shared memory, no
// scratch.  This is the plain form: no TMA ring, no tensor cores — a first decode path for these two types (see the
// measurements at the kernel).
#include "zq_common.cuh"

namespace zq {

__device__ __forceinline__ void kq_load_act4(const void *x, int dtype, size_t index, float (&v)[4]) {
    if (dtype == ZQ_F32) {
        const float4 f = __ldg(reinterpret_cast<const float4 *>(reinterpret_cast<const float *>(x) + index));
        v[0] = f.x; v[1] = f.y; v[2] = f.z; v[3] = f.w;
        return;
    }
    const uint2 raw = __ldg(reinterpret_cast<const uint2 *>(reinterpret_cast<const uint16_t *>(x) + index));
    if (dtype == ZQ_F16) {
        const float2 a = __half22float2(u32_as_h2(raw.x)), b = __half22float2(u32_as_h2(raw.y));
        v[0] = a.x; v[1] = a.y; v[2] = b.x; v[3] = b.y;
    } else {  // bf16: the upper half of an f32
        v[0] = __uint_as_float(raw.x << 16); v[1] = __uint_as_float(raw.x & 0xFFFF0000u);
        v[2] = __uint_as_float(raw.y << 16); v[3] = __uint_as_float(raw.y & 0xFFFF0000u);
    }
}

// Byte j of `codes` (0..255) as a float, minus `bias`: the byte is placed under the exponent of 2^23, where it is
// the integer 2^23 + byte exactly, and the subtraction is exact; no integer -> float conversion instruction.
template <int J>
__device__ __forceinline__ float kq_byte_to_float(uint32_t codes, float bias_plus_2p23) {
    uint32_t r;
    asm("prmt.b32 %0, %1, %2, %3;" : "=r"(r) : "r"(codes), "r"(0x4B000000u), "n"(0x7540 + J));
    return __fsub_rn(__uint_as_float(r), bias_plus_2p23);
}

// What lane `lane` holds of super-block `unit`: two groups of 4 integer codes (as floats, Q6_K already minus 32) at
// column offsets c0 .. c0+3 and c1 .. c1+3, and per group the factors of  weight = a * code - b.
struct KqLane {
    float q0[4], q1[4];
    float a0, b0, a1, b1;
    int c0, c1;
};

// The words a lane reads of one super-block.
struct KqRaw {
    uint32_t lo, hi;      // 4 low-quant bytes, the 4 high-bit bytes that go with them
    uint32_t s0, s1, s2;  // Q5_K: the 12 scale bytes; Q6_K: s0 = the two i8 scales (low-nibble group, high-nibble group)
    uint32_t dd;          // Q5_K: d | dmin << 16; Q6_K: d
};

template <uint32_t TYPE>
__device__ __forceinline__ KqRaw kq_lane_load(const uint8_t *unit, int lane) {
    KqRaw r;
    if constexpr (TYPE == ZQ_Q5_K) {
        // d, dmin, 12 scale bytes, 32 high-bit bytes at 16, 128 low-nibble bytes at 48; 176-byte blocks: words are aligned
        const uint32_t *u32 = reinterpret_cast<const uint32_t *>(unit);
        r.dd = u32[0];
        r.s0 = u32[1];
        r.s1 = u32[2];
        r.s2 = u32[3];
        const int pair = lane >> 3, j = (lane & 7) * 4;
        r.lo = u32[(48 + pair * 32 + j) >> 2];
        r.hi = u32[(16 + j) >> 2];
    } else {
        // 128 low-nibble bytes, 64 high-bit bytes at 128, 16 i8 scales at 192, d at 208; 210-byte blocks: 16-bit loads
        const uint16_t *u16 = reinterpret_cast<const uint16_t *>(unit);
        const int half = lane >> 4, o = (lane & 15) * 4;  // byte offset inside the half's 64 low bytes
        const int index = o & 31, odd = o >> 5;           // positions index..index+3; odd: quarters 1 and 3, else 0 and 2
        const int lw = (half * 64 + o) >> 1, hw = (128 + half * 32 + index) >> 1;
        r.lo = (uint32_t)u16[lw] | ((uint32_t)u16[lw + 1] << 16);
        r.hi = (uint32_t)u16[hw] | ((uint32_t)u16[hw + 1] << 16);
        const uint8_t *scales = unit + 192 + half * 8 + (index >> 4);
        r.s0 = (uint32_t)scales[2 * odd] | ((uint32_t)scales[2 * (odd + 2)] << 8);
        r.s1 = r.s2 = 0;
        r.dd = u16[104];
    }
    return r;
}

template <uint32_t TYPE>
__device__ __forceinline__ KqLane kq_lane_unpack(const KqRaw &r, int lane) {
    KqLane L;
    uint32_t code0, code1;  // four codes each, one per byte
    float bias;
    if constexpr (TYPE == ZQ_Q5_K) {
        const float d = __half2float(__ushort_as_half((unsigned short)(r.dd & 0xFFFFu))), dmin = __half2float(__ushort_as_half((unsigned short)(r.dd >> 16)));
        const int pair = lane >> 3, j = (lane & 7) * 4;
        // scale bytes 0..3 in s0, 4..7 in s1, 8..11 in s2 (src/weight/codec/ggml.rs:471-477)
        float dsc[2], dmn[2];
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            const int g = 2 * pair + h;
            uint32_t sc, mn;
            if (g < 4) {
                sc = (r.s0 >> (8 * g)) & 0x3Fu;
                mn = (r.s1 >> (8 * g)) & 0x3Fu;
            } else {
                const int t = 8 * (g - 4);
                sc = ((r.s2 >> t) & 0x0Fu) | (((r.s0 >> (t + 6)) & 3u) << 4);
                mn = ((r.s2 >> (t + 4)) & 0x0Fu) | (((r.s1 >> (t + 6)) & 3u) << 4);
            }
            dsc[h] = __fmul_rn(d, (float)sc);
            dmn[h] = __fmul_rn(dmin, (float)mn);
        }
        code0 = (r.lo & 0x0F0F0F0Fu) | (((r.hi >> (2 * pair)) & 0x01010101u) << 4);
        code1 = ((r.lo >> 4) & 0x0F0F0F0Fu) | (((r.hi >> (2 * pair + 1)) & 0x01010101u) << 4);
        bias = 8388608.0f;
        L.a0 = dsc[0]; L.b0 = dmn[0]; L.a1 = dsc[1]; L.b1 = dmn[1];
        L.c0 = (2 * pair) * 32 + j;
        L.c1 = L.c0 + 32;
    } else {
        const float d = __half2float(__ushort_as_half((unsigned short)r.dd));
        const int half = lane >> 4, o = (lane & 15) * 4;
        const int index = o & 31, odd = o >> 5;
        L.a0 = __fmul_rn(d, (float)(int8_t)(r.s0 & 0xFFu));
        L.a1 = __fmul_rn(d, (float)(int8_t)((r.s0 >> 8) & 0xFFu));
        L.b0 = L.b1 = 0.f;
        code0 = (r.lo & 0x0F0F0F0Fu) | (((r.hi >> (2 * odd)) & 0x03030303u) << 4);
        code1 = ((r.lo >> 4) & 0x0F0F0F0Fu) | (((r.hi >> (2 * odd + 4)) & 0x03030303u) << 4);
        bias = 8388608.0f + 32.0f;  // codes are stored plus 32
        L.c0 = half * 128 + odd * 32 + index;
        L.c1 = L.c0 + 64;
    }
    L.q0[0] = kq_byte_to_float<0>(code0, bias); L.q0[1] = kq_byte_to_float<1>(code0, bias);
    L.q0[2] = kq_byte_to_float<2>(code0, bias); L.q0[3] = kq_byte_to_float<3>(code0, bias);
    L.q1[0] = kq_byte_to_float<0>(code1, bias); L.q1[1] = kq_byte_to_float<1>(code1, bias);
    L.q1[2] = kq_byte_to_float<2>(code1, bias); L.q1[3] = kq_byte_to_float<3>(code1, bias);
    return L;
}

// Measured on 5120 -> 17408, one activation row.  Every byte unpacked by scalar shifts and integer -> float
// conversions: Q6_K 62.6 us (1.17 TB/s of packed bytes), Q5_K 74.0 us (0.83 TB/s).  The form below (four codes
// assembled at a time with word-wide masks, turned into floats by a byte permute, a group's scale applied once to
// a * sum(code * x) - b * sum(x)): 56.4 us (1.30 TB/s) and 64.5 us (0.95 TB/s).  Issuing loads ahead — one super-block
// (62.5 / 72.5 us), four super-blocks (70 / 94 us), four rows per warp (81 / 106 us) — made it slower each time:
// the extra registers cost resident warps, and a warp holds only ~210 bytes in flight per load round, so the kernel
// sits at about a sixth of the HBM roofline until it stages whole rows through shared memory the way the Q4_K
// kernels do.
template <uint32_t TYPE, int M>
__global__ void __launch_bounds__(256) gemv_kq_kernel(const uint8_t *__restrict__ data, size_t row_pitch, int units_per_row, int unit_bytes, int n_out, int cols, const void *__restrict__ x, int x_dtype,
                                                      void *__restrict__ y, int y_dtype, const void *__restrict__ residual) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    for (int row = blockIdx.x * 8 + warp; row < n_out; row += gridDim.x * 8) {
        const uint8_t *wrow = data + (size_t)row * row_pitch;
        float acc[M];
#pragma unroll
        for (int m = 0; m < M; ++m) acc[m] = 0.f;
        for (int u = 0; u < units_per_row; ++u) {
            const KqLane L = kq_lane_unpack<TYPE>(kq_lane_load<TYPE>(wrow + (size_t)u * unit_bytes, lane), lane);
            const size_t k0 = (size_t)u * kUnitWeights;
#pragma unroll
            for (int m = 0; m < M; ++m) {
                float a[4], b[4];
                kq_load_act4(x, x_dtype, (size_t)m * cols + k0 + L.c0, a);
                kq_load_act4(x, x_dtype, (size_t)m * cols + k0 + L.c1, b);
                float t0 = 0.f, t1 = 0.f;
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    t0 = fmaf(L.q0[j], a[j], t0);
                    t1 = fmaf(L.q1[j], b[j], t1);
                }
                acc[m] = fmaf(L.a0, t0, acc[m]);
                acc[m] = fmaf(L.a1, t1, acc[m]);
                if constexpr (TYPE == ZQ_Q5_K) {
                    acc[m] = fmaf(-L.b0, (a[0] + a[1]) + (a[2] + a[3]), acc[m]);
                    acc[m] = fmaf(-L.b1, (b[0] + b[1]) + (b[2] + b[3]), acc[m]);
                }
            }
        }
#pragma unroll
        for (int m = 0; m < M; ++m) {
            float v = acc[m];
#pragma unroll
            for (int s = 16; s > 0; s >>= 1) v += __shfl_xor_sync(0xFFFFFFFFu, v, s);
            if (lane == 0) {
                const size_t o = (size_t)m * n_out + row;
                if (residual) v += load_as_f32(residual, y_dtype, o);
                store_from_f32(y, y_dtype, o, v);
            }
        }
    }
}

template <uint32_t TYPE>
static int launch_kq_type(zq_ctx *ctx, const zq_weight *w, const void *x, int x_dtype, size_t m, void *y, int y_dtype, const void *residual, zq_error *err) {
    const FormatInfo f = format_info(w->type);
    const size_t xs = dtype_size(x_dtype), ys = dtype_size(y_dtype);
    for (size_t m0 = 0; m0 < m; m0 += 4) {  // up to four activation rows share one pass over the weights
        const int mm = (int)(m - m0 < 4 ? m - m0 : 4);
        size_t blocks = (w->rows + 7) / 8;
        if (blocks > (size_t)ctx->sm_count * 8) blocks = (size_t)ctx->sm_count * 8;
        const void *xp = reinterpret_cast<const uint8_t *>(x) + m0 * w->cols * xs;
        void *yp = reinterpret_cast<uint8_t *>(y) + m0 * w->rows * ys;
        const void *rp = residual ? reinterpret_cast<const uint8_t *>(residual) + m0 * w->rows * ys : nullptr;
#define ZQ_KQ_LAUNCH(MM) \
    gemv_kq_kernel<TYPE, MM><<<(unsigned)blocks, 256, 0, ctx->stream>>>(w->data, w->row_pitch, (int)w->units_per_row, f.unit_bytes, (int)w->rows, (int)w->cols, xp, x_dtype, yp, y_dtype, rp)
        switch (mm) {
        case 1: ZQ_KQ_LAUNCH(1); break;
        case 2: ZQ_KQ_LAUNCH(2); break;
        case 3: ZQ_KQ_LAUNCH(3); break;
        default: ZQ_KQ_LAUNCH(4); break;
        }
#undef ZQ_KQ_LAUNCH
        ctx->launches++;
        ZQ_CUDA_CHECK(cudaGetLastError(), err);
    }
    return ZQ_OK;
}

// y[m, n] = x[m, k] W^T (+ residual) for a Q5_K or Q6_K weight and 1..8 activation rows.  Activation rows must start
// on 16-byte (f32) or 8-byte (f16 / bf16) boundaries: true for every row when the buffer is 16-byte aligned, since
// the column count is a multiple of 256.
int launch_gemv_kq(zq_ctx *ctx, const zq_weight *w, const void *x, int x_dtype, size_t m, void *y, int y_dtype, const void *residual, zq_error *err) {
    if (m == 0 || m > 8) return set_error(err, ZQ_ERR_SHAPE, "K-quant decode kernel takes 1..8 activation rows, got %zu", m);
    if (w->type == ZQ_Q5_K) return launch_kq_type<ZQ_Q5_K>(ctx, w, x, x_dtype, m, y, y_dtype, residual, err);
    if (w->type == ZQ_Q6_K) return launch_kq_type<ZQ_Q6_K>(ctx, w, x, x_dtype, m, y, y_dtype, residual, err);
    return set_error(err, ZQ_ERR_UNSUPPORTED, "K-quant decode kernel: GGUF type %u", w->type);
}

}  // namespace zq
