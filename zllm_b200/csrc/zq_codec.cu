// Codec kernels: GGUF -> resident re-layout, bit-exact dequantisation (all rows or gathered rows), and the
// device-side encoders.
//
// Reference behaviour restated here:
//   decode formulas         src/weight/codec/ggml.rs:102-109 (Q4_0), 229-234 (Q8_0), 237-244 (IQ4_NL), 408-423 (Q4_K)
//   dequantize              src/weight/codec/ggml.rs:146-160
//   gathered rows to f16    src/kernel/cuda/linear.rs:1420-1437 (gguf_rows_f16)
//   encode_q4_k             src/weight/codec/ggml.rs:188-227
#include "zq_common.cuh"

namespace zq {

// One thread per resident byte: find the GGUF byte it comes from.  Padding blocks (beyond the row's last
// GGUF block) are zero.
__global__ void repack_kernel(uint32_t type, const uint8_t *__restrict__ gguf, uint8_t *__restrict__ resident, size_t rows, size_t blocks_per_row, size_t units_per_row, int unit_bytes, int block_bytes) {
    size_t row_pitch = units_per_row * (size_t)unit_bytes;
    size_t total = rows * row_pitch;
    for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += (size_t)gridDim.x * blockDim.x) {
        size_t row = idx / row_pitch;
        size_t in_row = idx % row_pitch;
        size_t unit = in_row / unit_bytes;
        int o = (int)(in_row % unit_bytes);
        int block, src;
        if (o < 16) {
            block = o >> 1;
            src = o & 1;
        } else {
            int u = (o - 16) >> 4, w = ((o - 16) & 15) >> 2, by = o & 3;
            int t = u & 3, h = u >> 2;
            if (type == ZQ_Q8_0) {
                block = 2 * h + (w >> 1);
                src = 2 + 4 * (4 * (w & 1) + t) + by;
            } else {
                block = 4 * h + w;
                src = 2 + 4 * t + by;
            }
        }
        size_t gblock = unit * 8 + block;
        uint8_t v = 0;
        if (gblock < blocks_per_row) v = gguf[(row * blocks_per_row + gblock) * block_bytes + src];
        resident[idx] = v;
    }
}

// The 6-bit code (0..63) of column `i` of a GGUF Q6_K super-block (src/weight/codec/ggml.rs:446-469: 128 low-nibble
// bytes, 64 high-bit bytes, 16 i8 scales, d).
__device__ __forceinline__ int q6k_gguf_code(const uint8_t *block, int i) {
    const int half = i >> 7, quarter = (i >> 5) & 3, index = i & 31;
    const uint8_t lo = block[half * 64 + index + ((quarter & 1) ? 32 : 0)];
    const uint8_t hv = block[128 + half * 32 + index];
    return (int)(((quarter & 2) ? (lo >> 4) : (lo & 0x0f)) | (((hv >> (2 * quarter)) & 3) << 4));
}

// One thread per resident byte of the Q6_K units (layout: kQ6k* in zq_common.cuh).
__global__ void repack_q6k_kernel(const uint8_t *__restrict__ gguf, uint8_t *__restrict__ resident, size_t rows, size_t units_per_row) {
    const size_t total = rows * units_per_row * 224;
    for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += (size_t)gridDim.x * blockDim.x) {
        const size_t unit = idx / 224;
        const int o = (int)(idx - unit * 224);
        const uint8_t *block = gguf + unit * 210;  // rows are whole super-blocks: unit u of the tensor is block u of the file
        uint8_t v = 0;
        if (o < 2) {
            v = block[208 + o];
        } else if (o >= kQ6kScales && o < kQ6kLow) {
            v = block[192 + (o - kQ6kScales)];
        } else if (o >= kQ6kLow && o < kQ6kHigh) {
            const int r = o - kQ6kLow, t = r >> 5, G = (r >> 2) & 7, i = r & 3;
            const int c0 = (q6k_gguf_code(block, 32 * G + 4 * t + i) - 32) & 63, c1 = (q6k_gguf_code(block, 32 * G + 16 + 4 * t + i) - 32) & 63;
            v = (uint8_t)((c0 & 15) | ((c1 & 15) << 4));
        } else if (o >= kQ6kHigh) {
            const int r = o - kQ6kHigh, t = r >> 4, vv = (r >> 2) & 3, i = r & 3;
            for (int x = 0; x < 4; ++x) {
                const int G = 2 * vv + (x >> 1), h = x & 1;
                const int c = (q6k_gguf_code(block, 32 * G + 16 * h + 4 * t + i) - 32) & 63;
                v |= (uint8_t)((c >> 4) << (2 * x));
            }
        }
        resident[idx] = v;
    }
}

int launch_repack(zq_ctx *ctx, uint32_t type, const uint8_t *gguf, uint8_t *resident, size_t rows, size_t cols, zq_error *err) {
    if (type == ZQ_Q6_K) {
        const size_t units = cols / kUnitWeights, total_q6 = rows * units * 224;
        if (total_q6 == 0) return ZQ_OK;
        size_t nb = (total_q6 + 255) / 256;
        if (nb > 65535u * 16u) nb = 65535u * 16u;
        repack_q6k_kernel<<<(unsigned)nb, 256, 0, ctx->stream>>>(gguf, resident, rows, units);
        ctx->launches++;
        ZQ_CUDA_CHECK(cudaGetLastError(), err);
        return ZQ_OK;
    }
    FormatInfo f = format_info(type);
    size_t blocks_per_row = cols / f.block_elems;
    size_t units_per_row = (cols + kUnitWeights - 1) / kUnitWeights;
    size_t total = rows * units_per_row * f.unit_bytes;
    if (total == 0) return ZQ_OK;
    int threads = 256;
    size_t blocks = (total + threads - 1) / threads;
    if (blocks > 65535u * 16u) blocks = 65535u * 16u;
    repack_kernel<<<(unsigned)blocks, threads, 0, ctx->stream>>>(type, gguf, resident, rows, blocks_per_row, units_per_row, f.unit_bytes, f.block_bytes);
    ctx->launches++;
    ZQ_CUDA_CHECK(cudaGetLastError(), err);
    return ZQ_OK;
}

// Decode element `i` (0..255) of a resident unit.  Every product below is exactly representable in f32, so the
// only rounding is the reference's final subtraction; __fmul_rn/__fsub_rn keep the compiler from contracting.
__device__ __forceinline__ float decode_unit_element(uint32_t type, const uint8_t *unit, int i) {
    if (type == ZQ_Q5_K) {  // src/weight/codec/ggml.rs:425-444: d, dmin, 12 scale bytes, 32 high-bit bytes, 128 low-nibble bytes
        const __half *hd = reinterpret_cast<const __half *>(unit);
        const float d = __half2float(hd[0]), dmin = __half2float(hd[1]);
        const uint8_t *scales = unit + 4;
        const int g = i >> 5, j = i & 31;
        int sc, mn;
        if (g < 4) {
            sc = scales[g] & 0x3f;
            mn = scales[g + 4] & 0x3f;
        } else {
            sc = (scales[g + 4] & 0x0f) | ((scales[g - 4] >> 6) << 4);
            mn = (scales[g + 4] >> 4) | ((scales[g] >> 6) << 4);
        }
        const uint8_t packed = unit[48 + (g >> 1) * 32 + j];
        const int quant = ((g & 1) ? (packed >> 4) : (packed & 0x0f)) + (((unit[16 + j] >> g) & 1) << 4);
        return __fsub_rn(__fmul_rn(__fmul_rn(d, (float)sc), (float)quant), __fmul_rn(dmin, (float)mn));
    }
    if (type == ZQ_Q6_K) {  // src/weight/codec/ggml.rs:446-469 on the re-laid unit (kQ6k* in zq_common.cuh): (d * scale) * (q - 32)
        const float d = __half2float(*reinterpret_cast<const __half *>(unit));
        const int G = i >> 5, h = (i >> 4) & 1, t = (i >> 2) & 3, ii = i & 3;
        const int lo = (unit[kQ6kLow + 32 * t + 4 * G + ii] >> (4 * h)) & 15;
        const int hi = (unit[kQ6kHigh + 16 * t + 4 * (G >> 1) + ii] >> (2 * (2 * (G & 1) + h))) & 3;
        const int c = lo | (hi << 4);
        const int q = c >= 32 ? c - 64 : c;  // the stored code is (q - 32) mod 64
        const int8_t scale = (int8_t)unit[kQ6kScales + (i >> 4)];
        return __fmul_rn(__fmul_rn(d, (float)scale), (float)q);
    }
    if (type == ZQ_Q5_0 || type == ZQ_Q5_1) {  // src/weight/codec/ggml.rs:111-130; the unit is 8 GGUF blocks in file order
        const int e = i & 31;
        const uint8_t *block = unit + (i >> 5) * (type == ZQ_Q5_0 ? 22 : 24);
        const float d = __half2float(*reinterpret_cast<const __half *>(block));
        const int hoff = type == ZQ_Q5_0 ? 2 : 4;
        const uint32_t high = (uint32_t)block[hoff] | ((uint32_t)block[hoff + 1] << 8) | ((uint32_t)block[hoff + 2] << 16) | ((uint32_t)block[hoff + 3] << 24);
        const uint8_t packed = block[hoff + 4 + (e & 15)];
        const int q5 = (int)((e < 16 ? (packed & 15) : (packed >> 4)) | (((high >> e) & 1u) << 4));
        if (type == ZQ_Q5_0) return __fmul_rn(d, (float)(q5 - 16));
        return __fadd_rn(__fmul_rn(d, (float)q5), __half2float(*reinterpret_cast<const __half *>(block + 2)));
    }
    if (type == ZQ_IQ4_XS) {  // src/weight/codec/ggml.rs:246-261
        const float d = __half2float(*reinterpret_cast<const __half *>(unit));
        const uint32_t scales_h = (uint32_t)unit[2] | ((uint32_t)unit[3] << 8);
        const int ib = i >> 5, j = i & 31;
        const int ls = (int)(((unit[4 + ib / 2] >> (4 * (ib & 1))) & 0x0f) | (((scales_h >> (2 * ib)) & 3u) << 4));
        const float dl = __fmul_rn(d, __fsub_rn((float)ls, 32.0f));
        const uint8_t qb = unit[8 + ib * 16 + (j & 15)];
        return __fmul_rn(dl, (float)kIq4nlValues[j < 16 ? (qb & 0x0f) : (qb >> 4)]);
    }
    if (type == ZQ_Q3_K) {  // src/weight/codec/ggml.rs:384-406
        const uint8_t *hmask = unit, *quants = unit + 32, *scales = unit + 96;
        const float d = __half2float(*reinterpret_cast<const __half *>(unit + 108));
        const int group = i >> 4, index = i & 15;
        const int low = group < 8 ? (scales[group] & 0x0f) : (scales[group - 8] >> 4);
        const int high = (scales[8 + (group & 3)] >> (2 * (group >> 2))) & 3;
        const int scale = (low | (high << 4)) - 32;
        const int half = group >> 3, pair = group & 7;
        const int low_bits = (quants[half * 32 + (pair & 1) * 16 + index] >> (2 * (pair >> 1))) & 3;
        const int quant = low_bits - ((hmask[(pair & 1) * 16 + index] & (1u << (group >> 1))) ? 0 : 4);
        return __fmul_rn(__fmul_rn(d, (float)scale), (float)quant);
    }
    uint8_t q = unit[unit_quant_offset(type, i)];
    if (type == ZQ_Q4_K) {
        const __half *hd = reinterpret_cast<const __half *>(unit);
        float d = __half2float(hd[0]), dmin = __half2float(hd[1]);
        const uint8_t *scales = unit + 4;
        int g = i >> 5;
        int sc, mn;
        if (g < 4) {
            sc = scales[g] & 0x3f;
            mn = scales[g + 4] & 0x3f;
        } else {
            sc = (scales[g + 4] & 0x0f) | ((scales[g - 4] >> 6) << 4);
            mn = (scales[g + 4] >> 4) | ((scales[g] >> 6) << 4);
        }
        int quant = (g & 1) ? (q >> 4) : (q & 0x0f);
        return __fsub_rn(__fmul_rn(__fmul_rn(d, (float)sc), (float)quant), __fmul_rn(dmin, (float)mn));
    }
    int blk = i >> 5, e = i & 31;
    float d = __half2float(reinterpret_cast<const __half *>(unit)[blk]);
    if (type == ZQ_Q8_0) return __fmul_rn(d, (float)(int8_t)q);
    int nib = (e >> 4) ? (q >> 4) : (q & 0x0f);
    if (type == ZQ_Q4_0) return __fmul_rn((float)(nib - 8), d);
    return __fmul_rn(d, (float)kIq4nlValues[nib]);
}

// One thread per 4 consecutive output elements.
__global__ void dequantize_kernel(uint32_t type, const uint8_t *__restrict__ resident, size_t row_pitch, int unit_bytes, size_t total_rows, size_t cols, const uint32_t *__restrict__ row_ids, size_t n_rows,
                                  void *__restrict__ out, int out_dtype, uint32_t *status) {
    size_t quads_per_row = cols / 4;
    size_t total = n_rows * quads_per_row;
    for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += (size_t)gridDim.x * blockDim.x) {
        size_t orow = idx / quads_per_row;
        size_t k0 = (idx % quads_per_row) * 4;
        size_t srow = row_ids ? row_ids[orow] : orow;
        if (srow >= total_rows) {  // bad row id: record and skip, never read out of bounds
            atomicMax(status, (uint32_t)kStatusBadIndex);
            continue;
        }
        const uint8_t *unit = resident + srow * row_pitch + (k0 / kUnitWeights) * unit_bytes;
        int i0 = (int)(k0 % kUnitWeights);
        float v[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) v[j] = decode_unit_element(type, unit, i0 + j);
        size_t o = orow * cols + k0;
        if (out_dtype == ZQ_F32) {
            *reinterpret_cast<float4 *>(reinterpret_cast<float *>(out) + o) = make_float4(v[0], v[1], v[2], v[3]);
        } else {
#pragma unroll
            for (int j = 0; j < 4; ++j) store_from_f32(out, out_dtype, o + j, v[j]);
        }
    }
}

// Packed rows -> f16 [rows, cols]: the operand pass of the prefill GEMM.  Each value is the weight's f32 value rounded
// once (Q4_K: through one fused multiply-add, i.e. at least as close to the exact value as the codec's two-step form).  Up to kDequantBatch matrices of one type and shape
// per launch (MoE prefill dequantises the experts of a chunk together).  One warp per 256-weight unit, 8 consecutive elements per lane: the
// unit's packed bytes are read once with coalesced loads, the 512 output bytes are one coalesced store, and the only
// index division is one per warp.
constexpr int kDequantBatch = 96;
struct DequantBatch {
    const uint8_t *src[kDequantBatch];
    __half *dst[kDequantBatch];
};

__global__ void __launch_bounds__(256) dequantize_f16_batch_kernel(const __grid_constant__ DequantBatch batch, uint32_t type, size_t row_pitch, int unit_bytes, int rows, int cols, int units_per_row) {
    const uint8_t *resident = batch.src[blockIdx.y];
    __half *out = batch.dst[blockIdx.y];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int total_units = rows * units_per_row;
    for (int u = blockIdx.x * 8 + warp; u < total_units; u += gridDim.x * 8) {
        const int row = u / units_per_row, ur = u - row * units_per_row;
        const int k0 = ur * kUnitWeights + 8 * lane;
        if (k0 >= cols) continue;  // padded tail of the last unit (cols is a multiple of 32, so all 8 or none)
        const uint8_t *unit = resident + (size_t)row * row_pitch + (size_t)ur * unit_bytes;
        const int i0 = 8 * lane;
        float v[8];
        if (type == ZQ_Q4_K) {
            const uint4 hdr = *reinterpret_cast<const uint4 *>(unit);
            const __half2 dd = *reinterpret_cast<const __half2 *>(&hdr.x);
            const float d = __low2float(dd), dmin = __high2float(dd);
            const uint8_t *scales = reinterpret_cast<const uint8_t *>(&hdr.y);
            const int g = i0 >> 5, j0 = i0 & 31;
            int sc, mn;
            if (g < 4) {
                sc = scales[g] & 0x3f;
                mn = scales[g + 4] & 0x3f;
            } else {
                sc = (scales[g + 4] & 0x0f) | ((scales[g - 4] >> 6) << 4);
                mn = (scales[g + 4] >> 4) | ((scales[g] >> 6) << 4);
            }
            // operand value: fma(d*sc, q, -(dmin*m)), one rounding (the fused GEMM kernel forms the same bits)
            const float dsc = __fmul_rn(d, (float)sc), ndm = -__fmul_rn(dmin, (float)mn);
            const uint2 qw = *reinterpret_cast<const uint2 *>(unit + 16 + (g >> 1) * 32 + j0);
            const int shift = (g & 1) * 4;
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                const uint32_t word = j < 4 ? qw.x : qw.y;
                const int q = (word >> (8 * (j & 3) + shift)) & 0x0f;
                v[j] = fmaf(dsc, (float)q, ndm);
            }
        } else {
#pragma unroll
            for (int j = 0; j < 8; ++j) v[j] = decode_unit_element(type, unit, i0 + j);
        }
        uint4 packed;
        packed.x = h2_as_u32(__floats2half2_rn(v[0], v[1]));
        packed.y = h2_as_u32(__floats2half2_rn(v[2], v[3]));
        packed.z = h2_as_u32(__floats2half2_rn(v[4], v[5]));
        packed.w = h2_as_u32(__floats2half2_rn(v[6], v[7]));
        *reinterpret_cast<uint4 *>(out + (size_t)row * cols + k0) = packed;
    }
}

// weights[i] -> outs[i], all of one type and shape.
int launch_dequantize_f16_batch(zq_ctx *ctx, const zq_weight *const *weights, __half *const *outs, size_t count, zq_error *err) {
    for (size_t first = 0; first < count; first += kDequantBatch) {
        const size_t n = count - first < (size_t)kDequantBatch ? count - first : (size_t)kDequantBatch;
        const zq_weight *w0 = weights[first];
        if (w0->cols % 8) return set_error(err, ZQ_ERR_SHAPE, "f16 operand pass needs columns aligned to 8, got %zu", w0->cols);
        DequantBatch batch;
        for (size_t i = 0; i < n; ++i) {
            const zq_weight *w = weights[first + i];
            if (w->type != w0->type || w->rows != w0->rows || w->cols != w0->cols) return set_error(err, ZQ_ERR_SHAPE, "batched dequantisation needs matrices of one type and shape");
            batch.src[i] = w->data;
            batch.dst[i] = outs[first + i];
        }
        const FormatInfo f = format_info(w0->type);
        const size_t units = w0->rows * w0->units_per_row;
        size_t bx = (units + 7) / 8;
        const size_t cap = ((size_t)ctx->sm_count * 64 + n - 1) / n;  // enough blocks in total to fill the machine a few times over
        if (bx > cap) bx = cap;
        if (bx == 0) bx = 1;
        dequantize_f16_batch_kernel<<<dim3((unsigned)bx, (unsigned)n), 256, 0, ctx->stream>>>(batch, w0->type, w0->row_pitch, f.unit_bytes, (int)w0->rows, (int)w0->cols, (int)w0->units_per_row);
        ctx->launches++;
        ZQ_CUDA_CHECK(cudaGetLastError(), err);
    }
    return ZQ_OK;
}

int launch_dequantize_f16(zq_ctx *ctx, const zq_weight *w, __half *out, zq_error *err) {
    if (w->rows == 0 || w->cols == 0) return ZQ_OK;
    return launch_dequantize_f16_batch(ctx, &w, &out, 1, err);
}

int launch_dequantize(zq_ctx *ctx, const zq_weight *w, const uint32_t *row_ids, size_t n_rows, void *out, int out_dtype, zq_error *err) {
    size_t total = n_rows * (w->cols / 4);
    if (total == 0) return ZQ_OK;
    int threads = 256;
    size_t blocks = (total + threads - 1) / threads;
    if (blocks > (size_t)ctx->sm_count * 64) blocks = (size_t)ctx->sm_count * 64;
    FormatInfo f = format_info(w->type);
    dequantize_kernel<<<(unsigned)blocks, threads, 0, ctx->stream>>>(w->type, w->data, w->row_pitch, f.unit_bytes, w->rows, w->cols, row_ids, n_rows, out, out_dtype, ctx->status_dev);
    ctx->launches++;
    ZQ_CUDA_CHECK(cudaGetLastError(), err);
    return ZQ_OK;
}

// ---------------------------------------------------------------------------------------------------------------
// Encoders (GGUF layout out).
// ---------------------------------------------------------------------------------------------------------------

__device__ __forceinline__ float f16_round(float v) { return __half2float(__float2half_rn(v)); }
__device__ __forceinline__ float clampf(float v, float lo, float hi) { return v < lo ? lo : (v > hi ? hi : v); }

// encode_q4_k, one thread per super-block, same operation order as the reference (f32 throughout, f16 rounding
// of d and dmin, round-half-away-from-zero codes).
__global__ void quantize_q4_k_kernel(const float *__restrict__ values, uint8_t *__restrict__ out, size_t blocks) {
    size_t b = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (b >= blocks) return;
    const float *v = values + b * 256;
    uint8_t *block = out + b * 144;
    float scales[8], minimums[8];
    for (int g = 0; g < 8; ++g) {
        float minimum = INFINITY, maximum = -INFINITY;
        for (int i = 0; i < 32; ++i) {
            float x = v[g * 32 + i];
            minimum = fminf(minimum, x);
            maximum = fmaxf(maximum, x);
        }
        minimums[g] = fmaxf(-minimum, 0.0f);
        scales[g] = __fdiv_rn(fmaxf(__fadd_rn(maximum, minimums[g]), 0.0f), 15.0f);
    }
    float max_scale = 0.0f, max_min = 0.0f;
    for (int g = 0; g < 8; ++g) {
        max_scale = fmaxf(max_scale, scales[g]);
        max_min = fmaxf(max_min, minimums[g]);
    }
    float d = f16_round(__fdiv_rn(max_scale, 63.0f));
    float dmin = f16_round(__fdiv_rn(max_min, 63.0f));
    for (int i = 0; i < 144; ++i) block[i] = 0;
    __half dh = __float2half_rn(d), dmh = __float2half_rn(dmin);
    // blocks start on even addresses: the two f16 fields go out as 16-bit stores
    reinterpret_cast<uint16_t *>(block)[0] = __half_as_ushort(dh);
    reinterpret_cast<uint16_t *>(block)[1] = __half_as_ushort(dmh);
    uint8_t sc[8], mc[8];
    for (int g = 0; g < 8; ++g) {
        sc[g] = d == 0.0f ? 0 : (uint8_t)clampf(roundf(__fdiv_rn(scales[g], d)), 0.0f, 63.0f);
        mc[g] = dmin == 0.0f ? 0 : (uint8_t)clampf(roundf(__fdiv_rn(minimums[g], dmin)), 0.0f, 63.0f);
    }
    for (int g = 0; g < 4; ++g) {
        block[4 + g] = (uint8_t)((sc[g] & 0x3f) | ((sc[g + 4] >> 4) << 6));
        block[8 + g] = (uint8_t)((mc[g] & 0x3f) | ((mc[g + 4] >> 4) << 6));
        block[12 + g] = (uint8_t)((sc[g + 4] & 0x0f) | ((mc[g + 4] & 0x0f) << 4));
    }
    for (int g = 0; g < 8; ++g) {
        float scale = __fmul_rn(d, (float)sc[g]);
        float minimum = __fmul_rn(dmin, (float)mc[g]);
        for (int i = 0; i < 32; ++i) {
            uint8_t quant = 0;
            if (scale != 0.0f) quant = (uint8_t)clampf(roundf(__fdiv_rn(__fadd_rn(v[g * 32 + i], minimum), scale)), 0.0f, 15.0f);
            int target = 16 + (g / 2) * 32 + i;
            if ((g & 1) == 0) block[target] = quant;
            else block[target] |= (uint8_t)(quant << 4);
        }
    }
}

// Round-to-nearest encoders for the 32-weight block types (synthetic-input generators; the reference has none).
//   Q8_0:   d = f16(max|v| / 127), q = rint(v / d)
//   Q4_0:   d = f16(v_at_max_abs / -8), code = nearest of -8..7 to v / d
//   IQ4_NL: d = f16(v_at_max_abs / -127), code = nearest codebook entry to v / d
__global__ void quantize_block32_kernel(uint32_t type, const float *__restrict__ values, uint8_t *__restrict__ out, size_t blocks) {
    size_t b = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (b >= blocks) return;
    const float *v = values + b * 32;
    float amax = 0.0f, smax = 0.0f;
    for (int i = 0; i < 32; ++i) {
        float a = fabsf(v[i]);
        if (a > amax) { amax = a; smax = v[i]; }
    }
    if (type == ZQ_Q8_0) {
        uint8_t *block = out + b * 34;
        float d = f16_round(__fdiv_rn(amax, 127.0f));
        float inv = d > 0.0f ? __fdiv_rn(1.0f, d) : 0.0f;
        __half dh = __float2half_rn(d);
        reinterpret_cast<uint16_t *>(block)[0] = __half_as_ushort(dh);
        for (int i = 0; i < 32; ++i) block[2 + i] = (uint8_t)(int8_t)clampf(rintf(__fmul_rn(v[i], inv)), -127.0f, 127.0f);
        return;
    }
    uint8_t *block = out + b * 18;
    float d = f16_round(__fdiv_rn(smax, type == ZQ_Q4_0 ? -8.0f : -127.0f));
    float inv = d != 0.0f ? __fdiv_rn(1.0f, d) : 0.0f;
    __half dh = __float2half_rn(d);
    reinterpret_cast<uint16_t *>(block)[0] = __half_as_ushort(dh);
    uint8_t codes[32];
    for (int i = 0; i < 32; ++i) {
        float s = __fmul_rn(v[i], inv);
        int best = 0;
        float best_err = INFINITY;
        for (int c = 0; c < 16; ++c) {
            float target = type == ZQ_Q4_0 ? (float)(c - 8) : (float)kIq4nlValues[c];
            float e = fabsf(__fsub_rn(s, target));
            if (e < best_err) { best_err = e; best = c; }
        }
        codes[i] = (uint8_t)best;
    }
    for (int i = 0; i < 16; ++i) block[2 + i] = (uint8_t)(codes[i] | (codes[i + 16] << 4));
}

int launch_quantize(zq_ctx *ctx, uint32_t type, const float *values, size_t rows, size_t cols, void *out, zq_error *err) {
    FormatInfo f = format_info(type);
    size_t blocks = rows * cols / f.block_elems;
    if (blocks == 0) return ZQ_OK;
    int threads = 128;
    unsigned grid = (unsigned)((blocks + threads - 1) / threads);
    if (type == ZQ_Q4_K) quantize_q4_k_kernel<<<grid, threads, 0, ctx->stream>>>(values, reinterpret_cast<uint8_t *>(out), blocks);
    else quantize_block32_kernel<<<grid, threads, 0, ctx->stream>>>(type, values, reinterpret_cast<uint8_t *>(out), blocks);
    ctx->launches++;
    ZQ_CUDA_CHECK(cudaGetLastError(), err);
    return ZQ_OK;
}

}  // namespace zq
