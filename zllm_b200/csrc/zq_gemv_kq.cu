// Decode GEMV for Q5_K and Q6_K (src/weight/codec/ggml.rs:425-469; the reference's CUDA kernels for these types:
// src/kernel/cuda/linear.rs:1167-1234, 1967-2101): up to 8 activation rows straight from the packed bytes, so that
// a one-row call (the Q6_K output head of a Q4_K_M file, a Q6_K down projection) streams 0.69 / 0.82 bytes per
// weight instead of dequantising the whole matrix to f16 first.
//
// One warp per weight row, f32 arithmetic on the CUDA cores.  A lane owns one 32-bit word of a super-block's low
// quant bytes: 4 consecutive positions of two scale groups (low nibbles, high nibbles) = 8 weights, decoded exactly
// as the codec decodes them ((d*sc)*q - dmin*m, (d*scale)*q), then multiplied into up to 4 activation rows at a
// time; the 32 lanes read a super-block's 128 low bytes as one coalesced line.  Q6_K blocks are 210 bytes, so their
// fields are only 2-byte aligned and are read as 16-bit loads.  Activations come through the read-only cache (a
// row of K floats is shared by all warps of the SM).  Sums are combined by warp shuffles; no shared memory, no
// scratch.  This is the plain form: no TMA ring, no tensor cores, scalar unpacking of every byte — a first decode path
// for these two types, about twice as fast as dequantising the matrix to f16 for a one-row call, and far from the
// HBM roofline (see the measurement at the kernel).
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

// The 8 weights of lane `lane` in super-block `unit`: w[0..3] at column offset c0 .. c0+3, w[4..7] at c1 .. c1+3.
template <uint32_t TYPE>
__device__ __forceinline__ void kq_lane_weights(const uint8_t *unit, int lane, float (&w)[8], int &c0, int &c1) {
    if constexpr (TYPE == ZQ_Q5_K) {
        // d, dmin, 12 scale bytes, 32 high-bit bytes at 16, 128 low-nibble bytes at 48; 176-byte blocks: words are aligned
        const uint32_t dd = *reinterpret_cast<const uint32_t *>(unit);
        const float d = __half2float(__ushort_as_half((unsigned short)(dd & 0xFFFFu))), dmin = __half2float(__ushort_as_half((unsigned short)(dd >> 16)));
        const uint8_t *scales = unit + 4;
        const int pair = lane >> 3, j = (lane & 7) * 4;
        const uint32_t lo = *reinterpret_cast<const uint32_t *>(unit + 48 + pair * 32 + j);
        const uint32_t hb = *reinterpret_cast<const uint32_t *>(unit + 16 + j);
        float dsc[2], dmn[2];
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            const int g = 2 * pair + h;
            int sc, mn;
            if (g < 4) {
                sc = scales[g] & 0x3f;
                mn = scales[g + 4] & 0x3f;
            } else {
                sc = (scales[g + 4] & 0x0f) | ((scales[g - 4] >> 6) << 4);
                mn = (scales[g + 4] >> 4) | ((scales[g] >> 6) << 4);
            }
            dsc[h] = __fmul_rn(d, (float)sc);
            dmn[h] = __fmul_rn(dmin, (float)mn);
        }
#pragma unroll
        for (int b = 0; b < 4; ++b) {
            const uint32_t byte = (lo >> (8 * b)) & 0xFFu, high = (hb >> (8 * b)) & 0xFFu;
            const int q0 = (int)(byte & 0x0Fu) + (int)(((high >> (2 * pair)) & 1u) << 4);
            const int q1 = (int)(byte >> 4) + (int)(((high >> (2 * pair + 1)) & 1u) << 4);
            w[b] = __fsub_rn(__fmul_rn(dsc[0], (float)q0), dmn[0]);
            w[4 + b] = __fsub_rn(__fmul_rn(dsc[1], (float)q1), dmn[1]);
        }
        c0 = (2 * pair) * 32 + j;
        c1 = c0 + 32;
    } else {
        // 128 low-nibble bytes, 64 high-bit bytes at 128, 16 i8 scales at 192, d at 208; 210-byte blocks: 16-bit loads
        const uint16_t *u16 = reinterpret_cast<const uint16_t *>(unit);
        const float d = __half2float(__ushort_as_half(u16[104]));
        const int half = lane >> 4, o = (lane & 15) * 4;       // byte offset inside the half's 64 low bytes
        const int index = o & 31, odd = o >> 5;                // positions index..index+3; odd: quarters 1 and 3, else 0 and 2
        const uint32_t lo = (uint32_t)u16[(half * 64 + o) >> 1] | ((uint32_t)u16[((half * 64 + o) >> 1) + 1] << 16);
        const uint32_t hv = (uint32_t)u16[(128 + half * 32 + index) >> 1] | ((uint32_t)u16[((128 + half * 32 + index) >> 1) + 1] << 16);
        const int8_t *scales = reinterpret_cast<const int8_t *>(unit + 192) + half * 8 + (index >> 4);
        const float ds0 = __fmul_rn(d, (float)scales[2 * odd]), ds1 = __fmul_rn(d, (float)scales[2 * (odd + 2)]);
#pragma unroll
        for (int b = 0; b < 4; ++b) {
            const uint32_t byte = (lo >> (8 * b)) & 0xFFu, high = (hv >> (8 * b)) & 0xFFu;
            const int q0 = (int)((byte & 0x0Fu) | (((high >> (2 * odd)) & 3u) << 4)) - 32;
            const int q1 = (int)((byte >> 4) | (((high >> (2 * odd + 4)) & 3u) << 4)) - 32;
            w[b] = __fmul_rn(ds0, (float)q0);
            w[4 + b] = __fmul_rn(ds1, (float)q1);
        }
        c0 = half * 128 + odd * 32 + index;
        c1 = c0 + 64;
    }
}

// Measured on 5120 -> 17408, one activation row: Q6_K 62.6 us (1.17 TB/s of packed bytes), Q5_K 74.0 us (0.83 TB/s).
// Variants measured and not kept: the loads of 4 super-blocks issued (through the read-only path) before the first is
// decoded (1.04 / 0.65 TB/s), and 4 rows per warp with the loads of 2 super-blocks each (0.90 / 0.58) — registers cost
// more than bytes in flight win; the kernel is bound by the scalar unpacking.
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
            float w[8];
            int c0, c1;
            kq_lane_weights<TYPE>(wrow + (size_t)u * unit_bytes, lane, w, c0, c1);
            const size_t k0 = (size_t)u * kUnitWeights;
#pragma unroll
            for (int m = 0; m < M; ++m) {
                float a[4], b[4];
                kq_load_act4(x, x_dtype, (size_t)m * cols + k0 + c0, a);
                kq_load_act4(x, x_dtype, (size_t)m * cols + k0 + c1, b);
#pragma unroll
                for (int j = 0; j < 4; ++j) acc[m] = fmaf(w[j], a[j], acc[m]);
#pragma unroll
                for (int j = 0; j < 4; ++j) acc[m] = fmaf(w[4 + j], b[j], acc[m]);
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
