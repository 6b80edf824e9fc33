// MoE entry points: router (logits + softmax top-k), resident expert table, routed forward.
//
// Reference behaviour restated here:
//   router logits + softmax top-k      src/kernel/cuda/routing.rs:15-62, 167-210; src/moe/routing.rs:25-39
//                                      (ordering: logit descending, ties to the lower expert id)
//   token-major stable grouping        src/moe/routing.rs:136-156
//   expert = gate/up + SiLU, then down src/kernel/cpu/moe.rs:122-138
//   weighted combine, per token in     src/backend/cpu/moe.rs:107-141 (no atomics; fixed order)
//     ascending expert order
//   shared expert added to the sum     src/moe/topk_moe.rs:84-104
//
// Two orchestrations.  Decode-sized batches (a few rows per expert) stay on the device: grouping, both projections of
// all routed experts and the combine are seven launches with no host round trip (zq_moe_grouped.cu).  Larger
// batches keep the reference CUDA backend's orchestration (router ids come back to the host,
// src/kernel/cuda/routing.rs:208; the host groups routes and issues the expert kernels,
// src/backend/cuda/expert.rs:787-917): the per-expert projections are calls into the prefill GEMM of this library
// over gathered token rows.
#include <algorithm>

#include "zq_i8.cuh"
#include "zq_moe.cuh"

using namespace zq;

namespace zq {

constexpr int kRouterTokens = 4;     // tokens per CTA
constexpr int kRouterThreads = 256;

// Softmax top-k of one token from its logits in shared memory (the logits are consumed): repeated arg-max with ties
// to the lower expert id; one warp per token.
// Raw score of the bias-corrected routers (src/moe/routing.rs:43-81): sigmoid, or sqrt(softplus) in its stable form.
__device__ __forceinline__ float router_raw_score(float logit, int scoring) {
    if (scoring == ZQ_ROUTE_SIGMOID_BIAS) return 1.0f / (1.0f + expf(-logit));
    const float softplus = logit > 0.0f ? logit + log1pf(expf(-logit)) : log1pf(expf(logit));
    return sqrtf(softplus);
}

// Bias-corrected top-k (route_bias_corrected_logits, src/moe/routing.rs:45-67): every expert has a raw score; the bias
// takes part in the SELECTION only (raw + bias, descending, ties to the lower id); the selected experts' raw scores are
// normalised to sum 1 and scaled.  `l` holds the logits (left untouched); one warp per token; each lane owns experts
// lane, lane + 32, ... and remembers the ones already taken in a bit mask (num_experts <= 1024).
__device__ __forceinline__ void router_select_bias(const float *l, const float *bias, int scoring, int lane, int num_experts, int top_k, float scaling, uint32_t *ids_out, float *weights_out, uint32_t *status) {
    uint32_t taken = 0;
    float sel_raw = 0.f, sum_raw = 0.f;
    uint32_t sel_id = 0;
    for (int slot = 0; slot < top_k; ++slot) {
        float best = -INFINITY;
        int best_e = 0x7fffffff;
        for (int e = lane, i = 0; e < num_experts; e += 32, ++i) {
            if ((taken >> i) & 1u) continue;
            const float v = router_raw_score(l[e], scoring) + (bias ? bias[e] : 0.f);
            if (v > best || (v == best && e < best_e)) { best = v; best_e = e; }
        }
        for (int o = 16; o > 0; o >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, best, o);
            const int oe = __shfl_xor_sync(0xffffffffu, best_e, o);
            if (ov > best || (ov == best && oe < best_e)) { best = ov; best_e = oe; }
        }
        if (best_e < 0 || best_e >= num_experts) {  // warp-uniform: nothing comparable left (NaN scores): a valid id, and a report
            best_e = slot;
            if (lane == 0) atomicMax(status, (uint32_t)kStatusBadIndex);
        }
        if ((best_e & 31) == lane) taken |= 1u << (best_e >> 5);
        const float raw = router_raw_score(l[best_e], scoring);
        if (lane == slot) { sel_raw = raw; sel_id = (uint32_t)best_e; }
        sum_raw += raw;
    }
    if (lane < top_k) {
        ids_out[lane] = sel_id;
        weights_out[lane] = sel_raw / sum_raw * scaling;
    }
}

// A row whose logits are all NaN (NaN in the activations, the router matrix or the bias) has no arg-max: such a slot
// takes expert id `slot` (always a valid id), the status word records it, and the weights come out NaN.
__device__ __forceinline__ void router_select(float *l, int lane, int num_experts, int top_k, float scaling, int normalize_selected, uint32_t *ids_out, float *weights_out, uint32_t *status, int scoring = ZQ_ROUTE_SOFTMAX,
                                              const float *bias = nullptr) {
    if (scoring != ZQ_ROUTE_SOFTMAX) {
        router_select_bias(l, bias, scoring, lane, num_experts, top_k, scaling, ids_out, weights_out, status);
        return;
    }
    float maximum = -INFINITY;
    for (int e = lane; e < num_experts; e += 32) maximum = fmaxf(maximum, l[e]);
    for (int o = 16; o > 0; o >>= 1) maximum = fmaxf(maximum, __shfl_xor_sync(0xffffffffu, maximum, o));
    float denom_all = 0.f;
    if (!normalize_selected) {
        for (int e = lane; e < num_experts; e += 32) denom_all += expf(l[e] - maximum);
        for (int o = 16; o > 0; o >>= 1) denom_all += __shfl_xor_sync(0xffffffffu, denom_all, o);
    }
    float sel_logit = 0.f, denom_sel = 0.f;  // lane j keeps the j-th selected logit (top_k <= 32)
    uint32_t sel_id = 0;
    for (int slot = 0; slot < top_k; ++slot) {
        float best = -INFINITY;
        int best_e = 0x7fffffff;
        for (int e = lane; e < num_experts; e += 32) {
            float v = l[e];
            if (v > best || (v == best && e < best_e)) { best = v; best_e = e; }
        }
        for (int o = 16; o > 0; o >>= 1) {
            float ov = __shfl_xor_sync(0xffffffffu, best, o);
            int oe = __shfl_xor_sync(0xffffffffu, best_e, o);
            if (ov > best || (ov == best && oe < best_e)) { best = ov; best_e = oe; }
        }
        if (best_e < 0 || best_e >= num_experts) {  // warp-uniform: no comparable logit left in the row
            best_e = slot;
            if (lane == 0) atomicMax(status, (uint32_t)kStatusBadIndex);
        }
        if (lane == slot) { sel_logit = best; sel_id = (uint32_t)best_e; }
        if (lane == 0) l[best_e] = -INFINITY;
        __syncwarp();
        denom_sel += expf(best - maximum);
    }
    const float denom = normalize_selected ? denom_sel : denom_all;
    if (lane < top_k) {
        ids_out[lane] = sel_id;
        weights_out[lane] = expf(sel_logit - maximum) / denom * scaling;
    }
}

// logits[t, e] = x[t] . router[e] (+ bias[e]) in f32, then softmax top-k per token.
// One CTA per 4 tokens and per block of `experts_per_cta` experts; each warp owns experts warp, warp + 8, ... of the
// block; lanes stride the hidden dimension.  With one expert block per token block the CTA selects right away;
// with several (few tokens: the expert blocks are what fills the machine) the logits go to `logits_g` and
// router_select_kernel finishes.
__global__ void __launch_bounds__(kRouterThreads) router_topk_kernel(const void *__restrict__ x, int x_dtype, int m, int hidden, const float *__restrict__ router, const float *__restrict__ bias, int num_experts, int top_k,
                                                                      float scaling, int normalize_selected, uint32_t *__restrict__ ids, float *__restrict__ weights, int experts_per_cta, float *__restrict__ logits_g, uint32_t *status, int scoring) {
    extern __shared__ float rsm[];
    float *xs = rsm;                                 // [kRouterTokens][hidden]
    float *logits = rsm + (size_t)kRouterTokens * hidden;  // [kRouterTokens][num_experts]
    const int tok0 = blockIdx.x * kRouterTokens;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int e_begin = blockIdx.y * experts_per_cta;
    const int e_end = e_begin + experts_per_cta < num_experts ? e_begin + experts_per_cta : num_experts;
    if ((hidden & 7) == 0) {  // 8 columns per thread and step: 16- or 32-byte loads, no index division
        for (int t = 0; t < kRouterTokens; ++t) {
            const bool live = tok0 + t < m;
            for (int c = threadIdx.x * 8; c < hidden; c += kRouterThreads * 8) {
                float v[8];
                const size_t o = (size_t)(tok0 + t) * hidden + c;
                if (!live) {
#pragma unroll
                    for (int j = 0; j < 8; ++j) v[j] = 0.f;
                } else if (x_dtype == ZQ_F32) {
                    const float4 f0 = *reinterpret_cast<const float4 *>(reinterpret_cast<const float *>(x) + o), f1 = *reinterpret_cast<const float4 *>(reinterpret_cast<const float *>(x) + o + 4);
                    v[0] = f0.x; v[1] = f0.y; v[2] = f0.z; v[3] = f0.w; v[4] = f1.x; v[5] = f1.y; v[6] = f1.z; v[7] = f1.w;
                } else {
                    const uint4 raw = *reinterpret_cast<const uint4 *>(reinterpret_cast<const uint16_t *>(x) + o);
                    const uint32_t rw[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        if (x_dtype == ZQ_F16) {
                            const float2 f = __half22float2(u32_as_h2(rw[j]));
                            v[2 * j] = f.x; v[2 * j + 1] = f.y;
                        } else {
                            v[2 * j] = __uint_as_float(rw[j] << 16);
                            v[2 * j + 1] = __uint_as_float(rw[j] & 0xFFFF0000u);
                        }
                    }
                }
                float4 *dst = reinterpret_cast<float4 *>(xs + t * hidden + c);
                dst[0] = make_float4(v[0], v[1], v[2], v[3]);
                dst[1] = make_float4(v[4], v[5], v[6], v[7]);
            }
        }
    } else {
        for (int i = threadIdx.x; i < kRouterTokens * hidden; i += kRouterThreads) {
            int t = i / hidden, c = i - t * hidden;
            xs[i] = (tok0 + t < m) ? load_as_f32(x, x_dtype, (size_t)(tok0 + t) * hidden + c) : 0.f;
        }
    }
    __syncthreads();
    for (int e = e_begin + warp; e < e_end; e += kRouterThreads / 32) {
        const float *w = router + (size_t)e * hidden;
        float acc[kRouterTokens];
#pragma unroll
        for (int t = 0; t < kRouterTokens; ++t) acc[t] = 0.f;
        if ((hidden & 127) == 0) {  // 16-byte loads of the router row, several in flight per lane
            const float4 *w4 = reinterpret_cast<const float4 *>(w);
#pragma unroll 8
            for (int c4 = lane; c4 < hidden / 4; c4 += 32) {
                const float4 wv = __ldg(w4 + c4);
#pragma unroll
                for (int t = 0; t < kRouterTokens; ++t) {
                    const float4 xv = reinterpret_cast<const float4 *>(xs + t * hidden)[c4];
                    acc[t] = fmaf(xv.w, wv.w, fmaf(xv.z, wv.z, fmaf(xv.y, wv.y, fmaf(xv.x, wv.x, acc[t]))));
                }
            }
        } else {
#pragma unroll 8
            for (int c = lane; c < hidden; c += 32) {
                const float wv = w[c];
#pragma unroll
                for (int t = 0; t < kRouterTokens; ++t) acc[t] = fmaf(xs[t * hidden + c], wv, acc[t]);
            }
        }
#pragma unroll
        for (int t = 0; t < kRouterTokens; ++t) {
            float v = acc[t];
            for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
            if (lane == 0) {
                if (scoring == ZQ_ROUTE_SOFTMAX) v += bias ? bias[e] : 0.f;  // the other routers use the bias for the selection only
                if (logits_g) {
                    if (tok0 + t < m) logits_g[(size_t)(tok0 + t) * num_experts + e] = v;
                } else {
                    logits[t * num_experts + e] = v;
                }
            }
        }
    }
    if (logits_g) return;
    __syncthreads();
    if (warp < kRouterTokens && tok0 + warp < m)
        router_select(logits + warp * num_experts, lane, num_experts, top_k, scaling, normalize_selected, ids + (size_t)(tok0 + warp) * top_k, weights + (size_t)(tok0 + warp) * top_k, status, scoring, bias);
}

// Few tokens with f16 / bf16 activations (MoE decode): eight tokens per CTA kept as 16-bit values in shared memory
// (half the footprint of the f32 staging above, so half as many token blocks re-read the router matrix), one expert per
// warp and round, 16-byte loads of the router row.  Writes logits only; router_select_kernel finishes.
constexpr int kRouter16Tokens = 8;
__global__ void __launch_bounds__(kRouterThreads) router_logits16_kernel(const uint16_t *__restrict__ x, int x_dtype, int m, int hidden, const float *__restrict__ router, int num_experts, int experts_per_cta,
                                                                          float *__restrict__ logits_g) {
    extern __shared__ float rsm[];
    uint16_t *xs = reinterpret_cast<uint16_t *>(rsm);  // [kRouter16Tokens][hidden]
    const int tok0 = blockIdx.x * kRouter16Tokens;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int e_begin = blockIdx.y * experts_per_cta;
    const int e_end = e_begin + experts_per_cta < num_experts ? e_begin + experts_per_cta : num_experts;
    const int vec_per_row = hidden / 8;
    // the eight rows are contiguous in x: a flat copy, four 16-byte loads in flight per thread
    const int live_vec = (m - tok0 < kRouter16Tokens ? m - tok0 : kRouter16Tokens) * vec_per_row, all_vec = kRouter16Tokens * vec_per_row;
    const uint4 *src = reinterpret_cast<const uint4 *>(x + (size_t)tok0 * hidden);
    uint4 *dst = reinterpret_cast<uint4 *>(xs);
    for (int i = threadIdx.x; i < all_vec; i += 4 * kRouterThreads) {
        uint4 raw[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int k = i + j * kRouterThreads;
            raw[j] = k < live_vec ? __ldg(src + k) : make_uint4(0, 0, 0, 0);
        }
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int k = i + j * kRouterThreads;
            if (k < all_vec) dst[k] = raw[j];
        }
    }
    __syncthreads();
    for (int e = e_begin + warp; e < e_end; e += kRouterThreads / 32) {
        const float4 *w4 = reinterpret_cast<const float4 *>(router + (size_t)e * hidden);
        float acc[kRouter16Tokens];
#pragma unroll
        for (int t = 0; t < kRouter16Tokens; ++t) acc[t] = 0.f;
        const int hv = hidden / 4;
        for (int base = lane; base < hv; base += 32 * 8) {  // eight 16-byte loads of the router row in flight, then the arithmetic
            float4 wv[8];
#pragma unroll
            for (int j = 0; j < 8; ++j) wv[j] = base + 32 * j < hv ? __ldg(w4 + base + 32 * j) : make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                const int c4 = base + 32 * j;
                if (c4 >= hv) break;
#pragma unroll
                for (int t = 0; t < kRouter16Tokens; ++t) {
                    const uint2 raw = reinterpret_cast<const uint2 *>(xs + (size_t)t * hidden)[c4];
                    float x0, x1, x2, x3;
                    if (x_dtype == ZQ_F16) {
                        const float2 a = __half22float2(u32_as_h2(raw.x)), b = __half22float2(u32_as_h2(raw.y));
                        x0 = a.x; x1 = a.y; x2 = b.x; x3 = b.y;
                    } else {  // bf16: the upper half of an f32
                        x0 = __uint_as_float(raw.x << 16); x1 = __uint_as_float(raw.x & 0xFFFF0000u);
                        x2 = __uint_as_float(raw.y << 16); x3 = __uint_as_float(raw.y & 0xFFFF0000u);
                    }
                    acc[t] = fmaf(x3, wv[j].w, fmaf(x2, wv[j].z, fmaf(x1, wv[j].y, fmaf(x0, wv[j].x, acc[t]))));
                }
            }
        }
#pragma unroll
        for (int t = 0; t < kRouter16Tokens; ++t) {
            float v = acc[t];
            for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
            if (lane == 0 && tok0 + t < m) logits_g[(size_t)(tok0 + t) * num_experts + e] = v;
        }
    }
}

// Router logits on the tensor cores for prefill-sized batches.  f16 operands alone would move logits by ~1e-3 and
// flip top-k choices, so both operands are split into two f16 limbs (v = hi + lo, 22 bits) and the three products
// that matter ride in ONE GEMM over a 3x longer K: x -> [hi | hi | lo], w -> [hi | lo | hi]; the products of f16
// numbers are exact in the f32 accumulator, the dropped lo*lo term is 2^-22 of a product.
// The operands are stored cut into `chunks` slices of that K, slice c of all rows together ([chunk][rows][kc]; one slice =
// the plain [rows][3 K] layout):
// with few tokens one GEMM over the whole K has too few tiles for the machine, so the slices become the "matrices" of a
// grouped GEMM whose partial logits router_select_kernel adds in ascending order.
__global__ void split_f16_chunked_kernel(const void *__restrict__ src, int dtype, size_t rows, int cols, int pattern, int kc, __half *__restrict__ dst) {
    // eight consecutive columns per thread (cols and kc are multiples of 8, so they never straddle a slice): one 16- or
    // 32-byte load, three 16-byte stores
    const int groups = cols / 8;
    const size_t total = rows * (size_t)groups;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
        const size_t r = i / groups;
        const int c = (int)(i - r * groups) * 8;
        float v[8];
        load_act8(src, dtype, r * (size_t)cols + c, true, v);
        __align__(16) __half hi[8], lo[8];
#pragma unroll
        for (int q = 0; q < 8; ++q) {
            hi[q] = __float2half_rn(v[q]);
            lo[q] = __float2half_rn(v[q] - __half2float(hi[q]));
        }
        const uint4 vh = *reinterpret_cast<const uint4 *>(hi), vl = *reinterpret_cast<const uint4 *>(lo);
        const uint4 seg[3] = {vh, pattern == 0 ? vh : vl, pattern == 0 ? vl : vh};
#pragma unroll
        for (int sgm = 0; sgm < 3; ++sgm) {
            const int g = sgm * cols + c, chunk = g / kc, kcol = g - chunk * kc;
            *reinterpret_cast<uint4 *>(dst + ((size_t)chunk * rows + r) * kc + kcol) = seg[sgm];
        }
    }
}

// work list of that grouped GEMM: item = {slice, first expert row, first token row, end of the slice's token rows}
__global__ void router_items_kernel(int chunks, int row_tiles, int tok_tiles, int m, int4 *__restrict__ items) {
    const int n = chunks * row_tiles * tok_tiles;
    for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < n; i += gridDim.x * blockDim.x) {
        const int c = i / (row_tiles * tok_tiles), rem = i - c * row_tiles * tok_tiles, rt = rem / tok_tiles, tt = rem - rt * tok_tiles;
        items[i] = make_int4(c, rt * 128, c * m + tt * 256, c * m + m);
    }
}

// Second half of the split router: one warp per token, logits from global memory.
// `chunks` > 1: the logits arrive as that many partial sums over slices of the hidden dimension ([chunk][m][experts]) and are
// added here in ascending order.
__global__ void __launch_bounds__(kRouterThreads) router_select_kernel(const float *__restrict__ logits_g, const float *__restrict__ bias, int m, int num_experts, int top_k, float scaling, int normalize_selected,
                                                                        uint32_t *__restrict__ ids, float *__restrict__ weights, uint32_t *status, int scoring, int chunks = 1) {
    extern __shared__ float rsm[];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int tok = blockIdx.x * (kRouterThreads / 32) + warp;
    if (tok >= m) return;
    float *l = rsm + warp * num_experts;
    for (int e = lane; e < num_experts; e += 32) {
        float v = logits_g[(size_t)tok * num_experts + e];
        for (int c = 1; c < chunks; ++c) v += logits_g[((size_t)c * m + tok) * num_experts + e];
        l[e] = v + ((bias && scoring == ZQ_ROUTE_SOFTMAX) ? bias[e] : 0.f);
    }
    __syncwarp();
    router_select(l, lane, num_experts, top_k, scaling, normalize_selected, ids + (size_t)tok * top_k, weights + (size_t)tok * top_k, status, scoring, bias);
}

__global__ void gather_rows_kernel(const void *__restrict__ x, int dtype, const uint32_t *__restrict__ tokens, size_t n_rows, int hidden, void *__restrict__ out) {
    const size_t esz = dtype_size(dtype);
    const size_t row_bytes = (size_t)hidden * esz;  // multiple of 16: hidden is a multiple of 32
    const size_t vec_per_row = row_bytes / 16;
    const size_t total = n_rows * vec_per_row;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
        size_t r = i / vec_per_row, v = i - r * vec_per_row;
        reinterpret_cast<uint4 *>(out)[i] = reinterpret_cast<const uint4 *>(reinterpret_cast<const uint8_t *>(x) + (size_t)tokens[r] * row_bytes)[v];
    }
}

// y[t] = ((sum_j w[t,j] * out[slot[t,j]]) + shared[t]) + residual[t]; slots of a token are in ascending expert order.
// Four columns per thread (hidden is a multiple of 32).  With a sink (expert-parallel owner side) the rows go to the source
// ranks' return buffers instead of y.
__global__ void __launch_bounds__(256) combine_kernel(const float *__restrict__ routed, const uint32_t *__restrict__ slots, const float *__restrict__ w, int top_k, const float *__restrict__ shared,
                                                      const void *__restrict__ residual, void *__restrict__ y, int y_dtype, size_t m, int hidden, const PeerRowSink sink) {
    const int hv = hidden / 4;
    const size_t total = m * (size_t)hv;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
        const size_t t = i / hv;
        const int c = (int)(i - t * hv);
        float *sink_row = nullptr;
        if (sink.world) {
            const int s = (int)(t / sink.cap), r = (int)(t - (size_t)s * sink.cap);
            if (r >= sink.counts[s]) continue;  // nothing was sent for this place
            sink_row = sink.base[s] + (size_t)r * hidden;
        }
        float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
        for (int j = 0; j < top_k; ++j) {
            const float wj = w[t * top_k + j];
            if (wj == 0.f) continue;  // an absent route (ZQ_MOE_NO_ROUTE) has no slot: nothing is read for it
            const float4 v = __ldcs(reinterpret_cast<const float4 *>(routed + (size_t)slots[t * top_k + j] * hidden) + c);
            acc.x = __fadd_rn(acc.x, __fmul_rn(v.x, wj));
            acc.y = __fadd_rn(acc.y, __fmul_rn(v.y, wj));
            acc.z = __fadd_rn(acc.z, __fmul_rn(v.z, wj));
            acc.w = __fadd_rn(acc.w, __fmul_rn(v.w, wj));
        }
        float vv[4] = {acc.x, acc.y, acc.z, acc.w};
        const size_t o = t * (size_t)hidden + 4 * (size_t)c;
        if (shared) {
            const float4 sh = *reinterpret_cast<const float4 *>(shared + o);
            vv[0] = __fadd_rn(vv[0], sh.x); vv[1] = __fadd_rn(vv[1], sh.y); vv[2] = __fadd_rn(vv[2], sh.z); vv[3] = __fadd_rn(vv[3], sh.w);
        }
        if (residual) {
#pragma unroll
            for (int q = 0; q < 4; ++q) vv[q] = __fadd_rn(vv[q], load_as_f32(residual, y_dtype, o + q));
        }
        if (sink_row) {
            reinterpret_cast<float4 *>(sink_row)[c] = make_float4(vv[0], vv[1], vv[2], vv[3]);
        } else if (y_dtype == ZQ_F32) {
            *reinterpret_cast<float4 *>(reinterpret_cast<float *>(y) + o) = make_float4(vv[0], vv[1], vv[2], vv[3]);
        } else {
#pragma unroll
            for (int q = 0; q < 4; ++q) store_from_f32(y, y_dtype, o + q, vv[q]);
        }
    }
    if (sink.world) {  // rows first, then the flags: every CTA fences its peer stores, the last one to arrive announces them
        __threadfence_system();
        __syncthreads();
        __shared__ int s_last;
        if (threadIdx.x == 0) s_last = atomicAdd(sink.done, 1u) == gridDim.x - 1;
        __syncthreads();
        if (s_last) {
            __threadfence_system();
            if ((int)threadIdx.x < sink.world) asm volatile("st.release.sys.global.v2.u32 [%0], {%1,%2};" ::"l"(sink.flag[threadIdx.x]), "r"(0u), "r"(sink.epoch) : "memory");
            if (threadIdx.x == 0) *sink.done = 0;
        }
    }
}

// out[rows[i]] += weights[i] * in[i]: scatter_add_rows_f32 (src/kernel/cuda/routing.rs:112-125).  Atomic adds, like the
// reference's: the rows of one call are distinct targets in every use the runtime makes of it (the tokens of one expert),
// so the sum each target receives per call is a single addition and the result does not depend on scheduling.
__global__ void scatter_add_rows_kernel(const void *__restrict__ in, int dtype, const uint32_t *__restrict__ rows, const float *__restrict__ w, size_t n, int hidden, size_t out_rows, float *__restrict__ out, uint32_t *status) {
    const size_t total = n * (size_t)hidden;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
        const size_t r = i / hidden;
        const uint32_t target = rows[r];
        if (target >= out_rows) {  // never write out of range: record it and skip
            atomicMax(status, (uint32_t)kStatusBadIndex);
            continue;
        }
        atomicAdd(out + (size_t)target * hidden + (i - r * hidden), load_as_f32(in, dtype, i) * (w ? w[r] : 1.0f));
    }
}

__global__ void gather_rows_checked_kernel(const void *__restrict__ x, int dtype, const uint32_t *__restrict__ tokens, size_t n_rows, size_t x_rows, int hidden, void *__restrict__ out, uint32_t *status) {
    const size_t esz = dtype_size(dtype);
    const size_t row_bytes = (size_t)hidden * esz, vec_per_row = row_bytes / 16, total = n_rows * vec_per_row;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
        const size_t r = i / vec_per_row, v = i - r * vec_per_row;
        const uint32_t src = tokens[r];
        if (src >= x_rows) {
            atomicMax(status, (uint32_t)kStatusBadIndex);
            reinterpret_cast<uint4 *>(out)[i] = make_uint4(0, 0, 0, 0);
            continue;
        }
        reinterpret_cast<uint4 *>(out)[i] = reinterpret_cast<const uint4 *>(reinterpret_cast<const uint8_t *>(x) + (size_t)src * row_bytes)[v];
    }
}

// ---------------------------------------------------------------------------------------------------------------
// Prefill grouping on the device (src/moe/routing.rs:136-156: token-major stable grouping; per-token combine order
// ascending expert id, src/backend/cpu/moe.rs:107-141).  A stable counting sort over chunks of whole tokens:
//   count   per chunk, how many routes go to each expert
//   scan    one CTA, thread per expert: the chunk's first slot inside each expert's range, the experts' ranges, and
//           the two work lists of the grouped GEMMs (one item per expert, 256-token tile, 128-row tile) with their counts
//   place   per chunk: slot of every route (the thread of an expert walks the chunk's routes in order), the
//           slot -> token table, and each token's slots and weights in combine order
// Nothing returns to the host: the GEMM kernels read their item counts from device memory.
// ---------------------------------------------------------------------------------------------------------------
constexpr int kGroupThreads = 1024;

__global__ void __launch_bounds__(kGroupThreads) moe_prefill_count_kernel(const uint32_t *__restrict__ ids, int m, int top_k, int E, int tokens_per_chunk, uint32_t *__restrict__ hist, uint32_t *status) {
    extern __shared__ uint32_t grp_smem[];
    uint32_t *s_cnt = grp_smem;
    for (int e = threadIdx.x; e < E; e += kGroupThreads) s_cnt[e] = 0;
    __syncthreads();
    const int t0 = blockIdx.x * tokens_per_chunk, t1 = min(m, t0 + tokens_per_chunk);
    const int r0 = t0 * top_k, nr = (t1 - t0) * top_k;
    for (int r = threadIdx.x; r < nr; r += kGroupThreads) {
        uint32_t id = ids[r0 + r];
        if (id == ZQ_MOE_NO_ROUTE) continue;
        if (id >= (uint32_t)E) {  // never index out of the table: record it and park the route on the last expert
            atomicMax(status, (uint32_t)kStatusBadIndex);
            id = (uint32_t)E - 1;
        }
        atomicAdd(&s_cnt[id], 1u);
    }
    __syncthreads();
    for (int e = threadIdx.x; e < E; e += kGroupThreads) hist[(size_t)blockIdx.x * E + e] = s_cnt[e];
}

// counts: [0] items of the gated launch, [1] items of the down launch, [2] routed rows in all
__global__ void __launch_bounds__(kGroupThreads) moe_prefill_scan_kernel(uint32_t *__restrict__ hist, int chunks, int E, uint32_t *__restrict__ offsets, int rt_gated, int rt_down, int4 *__restrict__ items_gated,
                                                                         int4 *__restrict__ items_down, int *__restrict__ counts) {
    __shared__ uint32_t warp_tot[2][32];
    const int e = threadIdx.x, lane = e & 31, wid = e >> 5;
    uint32_t c = 0;
    if (e < E)
        for (int b = 0; b < chunks; ++b) {  // exclusive prefix over the chunks: where chunk b's routes start inside expert e's range
            const uint32_t v = hist[(size_t)b * E + e];
            hist[(size_t)b * E + e] = c;
            c += v;
        }
    const uint32_t nt = (c + 255u) / 256u;  // 256-token tiles of this expert
    uint32_t sc = c, st = nt;
#pragma unroll
    for (int d = 1; d < 32; d <<= 1) {
        const uint32_t a = __shfl_up_sync(0xffffffffu, sc, d), b = __shfl_up_sync(0xffffffffu, st, d);
        if (lane >= d) {
            sc += a;
            st += b;
        }
    }
    if (lane == 31) {
        warp_tot[0][wid] = sc;
        warp_tot[1][wid] = st;
    }
    __syncthreads();
    uint32_t base_c = 0, base_t = 0;
    for (int w = 0; w < wid; ++w) {
        base_c += warp_tot[0][w];
        base_t += warp_tot[1][w];
    }
    const uint32_t first = base_c + sc - c, tfirst = base_t + st - nt;
    if (e < E) {
        offsets[e] = first;
        for (uint32_t tt = 0; tt < nt; ++tt) {
            const int t0 = (int)(first + tt * 256u), end = (int)(first + c);
            for (int rt = 0; rt < rt_gated; ++rt) items_gated[(size_t)(tfirst + tt) * rt_gated + rt] = make_int4(e, rt * 128, t0, end);
            for (int rt = 0; rt < rt_down; ++rt) items_down[(size_t)(tfirst + tt) * rt_down + rt] = make_int4(e, rt * 128, t0, end);
        }
    }
    if (e == kGroupThreads - 1) {  // the last thread holds the totals
        offsets[E] = base_c + sc;
        const uint32_t tiles = base_t + st;
        counts[0] = (int)(tiles * (uint32_t)rt_gated);
        counts[1] = (int)(tiles * (uint32_t)rt_down);
        counts[2] = (int)(base_c + sc);
    }
}

__global__ void __launch_bounds__(kGroupThreads) moe_prefill_place_kernel(const uint32_t *__restrict__ ids, const float *__restrict__ wts, int m, int top_k, int E, int tokens_per_chunk, const uint32_t *__restrict__ hist,
                                                                          const uint32_t *__restrict__ offsets, uint32_t *__restrict__ slot_token, uint32_t *__restrict__ token_slots, float *__restrict__ token_w) {
    extern __shared__ uint32_t grp_smem[];
    const int cap = tokens_per_chunk * top_k;
    uint32_t *s_ids = grp_smem;         // [cap]
    uint32_t *s_slot = s_ids + cap;     // [cap]
    uint32_t *s_cnt = s_slot + cap;     // [E]
    for (int e = threadIdx.x; e < E; e += kGroupThreads) s_cnt[e] = 0;
    __syncthreads();
    const int t0 = blockIdx.x * tokens_per_chunk, t1 = min(m, t0 + tokens_per_chunk);
    const int r0 = t0 * top_k, nr = (t1 - t0) * top_k;
    for (int r = threadIdx.x; r < nr; r += kGroupThreads) {
        uint32_t id = ids[r0 + r];
        s_slot[r] = 0;
        if (id == ZQ_MOE_NO_ROUTE) {  // an absent route: no slot, weight 0 in the combine
            s_ids[r] = (uint32_t)E;
            continue;
        }
        if (id >= (uint32_t)E) id = (uint32_t)E - 1;  // reported by the count kernel
        s_ids[r] = id;
        atomicAdd(&s_cnt[id], 1u);
    }
    __syncthreads();
    // every route counts the earlier routes of its expert inside the chunk itself (independent compares over at most
    // 1024 entries, instead of a serial walk per expert)
    for (int r = threadIdx.x; r < nr; r += kGroupThreads) {
        const uint32_t id = s_ids[r];
        if (id == (uint32_t)E) continue;
        uint32_t before = 0;
        int r2 = 0;
        for (; r2 + 4 <= r; r2 += 4) before += (s_ids[r2] == id) + (s_ids[r2 + 1] == id) + (s_ids[r2 + 2] == id) + (s_ids[r2 + 3] == id);
        for (; r2 < r; ++r2) before += s_ids[r2] == id;
        const uint32_t slot = offsets[id] + hist[(size_t)blockIdx.x * E + id] + before;
        slot_token[slot] = (uint32_t)((r0 + r) / top_k);
        s_slot[r] = slot;
    }
    __syncthreads();
    for (int t = threadIdx.x; t < t1 - t0; t += kGroupThreads) {
        uint32_t ke[64], ks[64];
        float kw[64];
        for (int j = 0; j < top_k; ++j) {
            const uint32_t e = s_ids[t * top_k + j], s = s_slot[t * top_k + j];
            const float w = e == (uint32_t)E ? 0.f : wts[r0 + t * top_k + j];
            int i = j;
            while (i > 0 && ke[i - 1] > e) {
                ke[i] = ke[i - 1]; ks[i] = ks[i - 1]; kw[i] = kw[i - 1];
                --i;
            }
            ke[i] = e; ks[i] = s; kw[i] = w;
        }
        for (int j = 0; j < top_k; ++j) {
            token_slots[(size_t)(t0 + t) * top_k + j] = ks[j];
            token_w[(size_t)(t0 + t) * top_k + j] = kw[j];
        }
    }
}

// out16[s] = f16(x[slot_token[s]]) for the slots that exist (their number is on the device); 8 elements per thread
__global__ void gather_rows_f16_kernel(const void *__restrict__ x, int dtype, const uint32_t *__restrict__ slot_token, const int *__restrict__ n_rows_dev, int hidden, __half *__restrict__ out) {
    const size_t vec_per_row = (size_t)hidden / 8, total = (size_t)*n_rows_dev * vec_per_row;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
        const size_t r = i / vec_per_row, v = i - r * vec_per_row;
        const size_t src = (size_t)slot_token[r] * hidden + v * 8;
        __align__(16) __half h[8];
        if (dtype == ZQ_F16) {
            *reinterpret_cast<uint4 *>(h) = *reinterpret_cast<const uint4 *>(reinterpret_cast<const __half *>(x) + src);
        } else {
#pragma unroll
            for (int j = 0; j < 8; ++j) h[j] = __float2half_rn(load_as_f32(x, dtype, src + j));
        }
        reinterpret_cast<uint4 *>(out)[i] = *reinterpret_cast<const uint4 *>(h);
    }
}

static unsigned grid_for(zq_ctx *ctx, size_t total, int threads) {
    size_t blocks = (total + threads - 1) / threads;
    size_t cap = (size_t)ctx->sm_count * 32;
    if (blocks > cap) blocks = cap;
    if (blocks == 0) blocks = 1;
    return (unsigned)blocks;
}

static int ensure_moe_ws(zq_ctx *ctx, size_t bytes, zq_error *err) {
    if (bytes <= ctx->moe_ws_bytes) return ZQ_OK;
    ZQ_CUDA_CHECK(cudaStreamSynchronize(ctx->stream), err);
    if (ctx->moe_ws) cudaFree(ctx->moe_ws);
    ctx->moe_ws = nullptr;
    ctx->moe_ws_bytes = 0;
    size_t rounded = (bytes + (size_t(1) << 20) - 1) & ~((size_t(1) << 20) - 1);
    ZQ_CUDA_CHECK(cudaMalloc(&ctx->moe_ws, rounded), err);
    ctx->moe_ws_bytes = rounded;
    return ZQ_OK;
}

// MoE prefill with Q4_K experts, everything on the device: grouping (three small kernels), one gather that also
// converts to f16, the two grouped fused GEMMs (their item counts read from device memory), shared expert, combine.
static int moe_prefill_device(zq_ctx *ctx, const zq_moe_experts *experts, const zq_weight *shared_gate, const zq_weight *shared_up, const zq_weight *shared_down, const void *dev_x, int x_dtype, size_t m, const uint32_t *dev_ids,
                              const float *dev_weights, size_t top_k, void *dev_y, int y_dtype, const void *dev_residual, zq_error *err) {
    const size_t E = experts->num_experts, H = experts->hidden, I = experts->inter, routes = m * top_k;
    const bool has_shared = shared_gate != nullptr;
    const int tokens_per_chunk = (int)(kGroupThreads / top_k > 0 ? kGroupThreads / top_k : 1);
    const int chunks = (int)((m + tokens_per_chunk - 1) / tokens_per_chunk);
    const int rt_i = (int)((I + 127) / 128), rt_h = (int)((H + 127) / 128);
    const size_t max_tiles = routes / 256 + E;  // sum over experts of ceil(count / 256)
    auto al = [](size_t v) { return (v + 255) & ~size_t(255); };
    // tables and f32 results
    const size_t o_hist = 0, o_offsets = o_hist + al((size_t)chunks * E * 4), o_counts = o_offsets + al((E + 1) * 4), o_slot_token = o_counts + al(16), o_token_slots = o_slot_token + al(routes * 4);
    const size_t o_token_w = o_token_slots + al(routes * 4), o_out = o_token_w + al(routes * 4), o_shared = o_out + al(routes * H * 4), total = o_shared + (has_shared ? al(m * H * 4) : 0);
    int rc = ensure_moe_ws(ctx, total, err);
    if (rc) return rc;
    uint8_t *ws = reinterpret_cast<uint8_t *>(ctx->moe_ws);
    uint32_t *d_hist = reinterpret_cast<uint32_t *>(ws + o_hist), *d_offsets = reinterpret_cast<uint32_t *>(ws + o_offsets), *d_slot_token = reinterpret_cast<uint32_t *>(ws + o_slot_token);
    uint32_t *d_token_slots = reinterpret_cast<uint32_t *>(ws + o_token_slots);
    int *d_counts = reinterpret_cast<int *>(ws + o_counts);
    float *d_token_w = reinterpret_cast<float *>(ws + o_token_w), *d_out = reinterpret_cast<float *>(ws + o_out), *d_shared = has_shared ? reinterpret_cast<float *>(ws + o_shared) : nullptr;
    // f16 operands and work lists
    auto al2 = [](size_t v) { return (v + 1023) & ~size_t(1023); };
    const size_t x16_bytes = al2(routes * H * sizeof(__half)), act16_bytes = al2(routes * I * sizeof(__half)), items_g_bytes = al2(max_tiles * rt_i * sizeof(int4)), items_d_bytes = al2(max_tiles * rt_h * sizeof(int4));
    rc = ensure_workspace(ctx, x16_bytes + act16_bytes + items_g_bytes + items_d_bytes, err);
    if (rc) return rc;
    uint8_t *wsb = reinterpret_cast<uint8_t *>(ctx->workspace);
    __half *x16 = reinterpret_cast<__half *>(wsb), *act16 = reinterpret_cast<__half *>(wsb + x16_bytes);
    int4 *d_items_g = reinterpret_cast<int4 *>(wsb + x16_bytes + act16_bytes), *d_items_d = reinterpret_cast<int4 *>(wsb + x16_bytes + act16_bytes + items_g_bytes);

    static bool configured[64] = {};
    const size_t place_smem = ((size_t)tokens_per_chunk * top_k * 2 + E) * 4;
    if (!configured[ctx->device & 63]) {
        ZQ_CUDA_CHECK(cudaFuncSetAttribute(moe_prefill_place_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 64 * 1024), err);
        configured[ctx->device & 63] = true;
    }
    moe_prefill_count_kernel<<<chunks, kGroupThreads, E * 4, ctx->stream>>>(dev_ids, (int)m, (int)top_k, (int)E, tokens_per_chunk, d_hist, ctx->status_dev);
    moe_prefill_scan_kernel<<<1, kGroupThreads, 0, ctx->stream>>>(d_hist, chunks, (int)E, d_offsets, rt_i, rt_h, d_items_g, d_items_d, d_counts);
    moe_prefill_place_kernel<<<chunks, kGroupThreads, place_smem, ctx->stream>>>(dev_ids, dev_weights, (int)m, (int)top_k, (int)E, tokens_per_chunk, d_hist, d_offsets, d_slot_token, d_token_slots, d_token_w);
    gather_rows_f16_kernel<<<grid_for(ctx, routes * (H / 8), 256), 256, 0, ctx->stream>>>(dev_x, x_dtype, d_slot_token, d_counts + 2, (int)H, x16);
    ctx->launches += 4;
    ZQ_CUDA_CHECK(cudaGetLastError(), err);
    rc = launch_gemm_fused_grouped(ctx, experts->d_gate_qmaps, experts->d_up_qmaps, I, H, x16, routes, d_items_g, (int)(max_tiles * rt_i), d_counts, act16, ZQ_F16, err);
    if (rc) return rc;
    rc = launch_gemm_fused_grouped(ctx, experts->d_down_qmaps, nullptr, H, I, act16, routes, d_items_d, (int)(max_tiles * rt_h), d_counts + 1, d_out, ZQ_F32, err);
    if (rc) return rc;
    if (has_shared) {
        rc = zq_gated_mlp(ctx, shared_gate, shared_up, shared_down, dev_x, x_dtype, m, d_shared, ZQ_F32, nullptr, err);
        if (rc) return rc;
    }
    combine_kernel<<<grid_for(ctx, m * (H / 4), 256), 256, 0, ctx->stream>>>(d_out, d_token_slots, d_token_w, (int)top_k, d_shared, dev_residual, dev_y, y_dtype, m, (int)H, ctx->moe_row_sink ? *reinterpret_cast<const PeerRowSink *>(ctx->moe_row_sink) : PeerRowSink());
    ctx->launches++;
    ZQ_CUDA_CHECK(cudaGetLastError(), err);
    return ZQ_OK;
}

}  // namespace zq

extern "C" {

int zq_moe_route_softmax_topk(zq_ctx *ctx, const void *dev_x, int x_dtype, size_t m, size_t hidden, const float *dev_router_f32, const float *dev_bias_f32, size_t num_experts, size_t top_k, float scaling_factor, int normalize_selected,
                              uint32_t *dev_ids, float *dev_weights, zq_error *err) {
    return zq_moe_route_topk(ctx, ZQ_ROUTE_SOFTMAX, dev_x, x_dtype, m, hidden, dev_router_f32, dev_bias_f32, num_experts, top_k, scaling_factor, normalize_selected, dev_ids, dev_weights, err);
}

int zq_moe_route_topk(zq_ctx *ctx, int scoring, const void *dev_x, int x_dtype, size_t m, size_t hidden, const float *dev_router_f32, const float *dev_bias_f32, size_t num_experts, size_t top_k, float scaling_factor,
                      int normalize_selected, uint32_t *dev_ids, float *dev_weights, zq_error *err) {
    if (!ctx || !dev_x || !dev_router_f32 || !dev_ids || !dev_weights) return set_error(err, ZQ_ERR_ARG, "zq_moe_route_topk: null argument");
    if (scoring != ZQ_ROUTE_SOFTMAX && scoring != ZQ_ROUTE_SIGMOID_BIAS && scoring != ZQ_ROUTE_SQRT_SOFTPLUS_BIAS) return set_error(err, ZQ_ERR_ARG, "zq_moe_route_topk: unknown scoring %d", scoring);
    // same limits as the reference's device router (src/kernel/cuda/routing.rs:177): experts <= 1024, 0 < top_k <= experts
    if (num_experts == 0 || num_experts > 1024 || top_k == 0 || top_k > num_experts || top_k > 32) return set_error(err, ZQ_ERR_SHAPE, "softmax router: experts=%zu top_k=%zu outside the supported range (experts <= 1024, top_k <= 32)", num_experts, top_k);
    if (!(scaling_factor == scaling_factor) || scaling_factor > 3.0e38f || scaling_factor < -3.0e38f) return set_error(err, ZQ_ERR_ARG, "softmax router: scaling factor is not finite");
    if (m == 0 || hidden == 0) return set_error(err, ZQ_ERR_SHAPE, "softmax router: empty input");
    if (x_dtype != ZQ_F32 && x_dtype != ZQ_F16 && x_dtype != ZQ_BF16) return set_error(err, ZQ_ERR_ARG, "softmax router: unknown input dtype %d", x_dtype);
    // the kernels read x and the router matrix with 16-byte loads whenever hidden is a multiple of 8
    if ((reinterpret_cast<uintptr_t>(dev_x) & 15) || (reinterpret_cast<uintptr_t>(dev_router_f32) & 15)) return set_error(err, ZQ_ERR_ARG, "softmax router: x and the router matrix must be 16-byte aligned");
    if ((reinterpret_cast<uintptr_t>(dev_ids) & 3) || (reinterpret_cast<uintptr_t>(dev_weights) & 3) || (reinterpret_cast<uintptr_t>(dev_bias_f32) & 3)) return set_error(err, ZQ_ERR_ARG, "softmax router: ids, weights and bias must be 4-byte aligned");
    if (int rc = use_device(ctx, err)) return rc;
    size_t smem = ((size_t)kRouterTokens * hidden + (size_t)kRouterTokens * num_experts) * sizeof(float);
    if (smem > 200 * 1024) return set_error(err, ZQ_ERR_UNSUPPORTED, "softmax router: hidden=%zu does not fit the router kernel's shared memory", hidden);
    static bool configured[64] = {};
    if (!configured[ctx->device & 63]) {
        ZQ_CUDA_CHECK(cudaFuncSetAttribute(router_topk_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024), err);
        configured[ctx->device & 63] = true;
    }
    const unsigned grid = (unsigned)((m + kRouterTokens - 1) / kRouterTokens);
    // few tokens: split the experts over CTAs too, so that the router matrix is read by the whole machine
    size_t blocks_y = 1, per_cta = num_experts;
    if (grid < (unsigned)ctx->sm_count) {
        blocks_y = (2 * (size_t)ctx->sm_count + grid - 1) / grid;
        per_cta = ((num_experts + blocks_y - 1) / blocks_y + 7) & ~size_t(7);  // whole rounds of the 8 warps
        blocks_y = (num_experts + per_cta - 1) / per_cta;
    }
    if (m >= 256 && hidden % 8 == 0) {
        auto al = [](size_t v) { return (v + 255) & ~size_t(255); };
        // slices of K as separate tiles while the whole-K tiles would leave most SMs idle
        const int row_tiles = (int)((num_experts + 127) / 128), tok_tiles = (int)((m + 255) / 256);
        int chunks = 1;
        if (hidden % 64 == 0)
            for (int c = 16; c >= 2; --c)
                if ((3 * hidden / 64) % c == 0 && row_tiles * tok_tiles * c <= 2 * ctx->sm_count) {
                    chunks = c;
                    break;
                }
        const int n_items = chunks * row_tiles * tok_tiles;
        const size_t xb = al(m * 3 * hidden * sizeof(__half)), wb = al(num_experts * 3 * hidden * sizeof(__half)), lb = al((size_t)chunks * m * num_experts * sizeof(float));
        int rc = ensure_moe_ws(ctx, xb + wb + lb + al((size_t)n_items * sizeof(int4)), err);
        if (rc) return rc;
        uint8_t *ws = reinterpret_cast<uint8_t *>(ctx->moe_ws);
        __half *x3 = reinterpret_cast<__half *>(ws), *w3 = reinterpret_cast<__half *>(ws + xb);
        float *logits_g = reinterpret_cast<float *>(ws + xb + wb);
        int4 *d_items = reinterpret_cast<int4 *>(ws + xb + wb + lb);
        const unsigned sel_grid = (unsigned)((m + kRouterThreads / 32 - 1) / (kRouterThreads / 32));
        if (chunks > 1) {
            const int kc = (int)(3 * hidden / chunks);
            split_f16_chunked_kernel<<<grid_for(ctx, m * hidden / 8, 256), 256, 0, ctx->stream>>>(dev_x, x_dtype, m, (int)hidden, 0, kc, x3);
            split_f16_chunked_kernel<<<grid_for(ctx, num_experts * hidden / 8, 256), 256, 0, ctx->stream>>>(dev_router_f32, ZQ_F32, num_experts, (int)hidden, 1, kc, w3);
            router_items_kernel<<<(n_items + 255) / 256, 256, 0, ctx->stream>>>(chunks, row_tiles, tok_tiles, (int)m, d_items);
            ctx->launches += 3;
            ZQ_CUDA_CHECK(cudaGetLastError(), err);
            rc = launch_gemm_grouped(ctx, w3, nullptr, (size_t)chunks, num_experts, (size_t)kc, x3, (size_t)chunks * m, d_items, n_items, logits_g, ZQ_F32, err);
            if (rc) return rc;
        } else {
            split_f16_chunked_kernel<<<grid_for(ctx, m * hidden / 8, 256), 256, 0, ctx->stream>>>(dev_x, x_dtype, m, (int)hidden, 0, (int)(3 * hidden), x3);  // one slice: the plain [rows][3 K] layout
            split_f16_chunked_kernel<<<grid_for(ctx, num_experts * hidden / 8, 256), 256, 0, ctx->stream>>>(dev_router_f32, ZQ_F32, num_experts, (int)hidden, 1, (int)(3 * hidden), w3);
            ctx->launches += 2;
            ZQ_CUDA_CHECK(cudaGetLastError(), err);
            rc = launch_gemm_f16(ctx, w3, num_experts, 3 * hidden, x3, m, logits_g, ZQ_F32, err);
            if (rc) return rc;
        }
        router_select_kernel<<<sel_grid, kRouterThreads, (kRouterThreads / 32) * num_experts * sizeof(float), ctx->stream>>>(logits_g, dev_bias_f32, (int)m, (int)num_experts, (int)top_k, scaling_factor, normalize_selected, dev_ids,
                                                                                                                            dev_weights, ctx->status_dev, scoring, chunks);
        ctx->launches++;
        ZQ_CUDA_CHECK(cudaGetLastError(), err);
        return ZQ_OK;
    }
    if (blocks_y > 1 && x_dtype != ZQ_F32 && hidden % 128 == 0 && (size_t)kRouter16Tokens * hidden * 2 <= 200 * 1024) {
        int rc = ensure_moe_ws(ctx, m * num_experts * sizeof(float), err);
        if (rc) return rc;
        float *logits_g = reinterpret_cast<float *>(ctx->moe_ws);
        static bool configured16[64] = {};
        if (!configured16[ctx->device & 63]) {
            ZQ_CUDA_CHECK(cudaFuncSetAttribute(router_logits16_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024), err);
            configured16[ctx->device & 63] = true;
        }
        const size_t grid16 = (m + kRouter16Tokens - 1) / kRouter16Tokens;
        size_t by = (2 * (size_t)ctx->sm_count + grid16 - 1) / grid16;
        size_t per16 = ((num_experts + by - 1) / by + 7) & ~size_t(7);  // whole rounds of the 8 warps
        by = (num_experts + per16 - 1) / per16;
        router_logits16_kernel<<<dim3((unsigned)grid16, (unsigned)by), kRouterThreads, (size_t)kRouter16Tokens * hidden * 2, ctx->stream>>>(reinterpret_cast<const uint16_t *>(dev_x), x_dtype, (int)m, (int)hidden, dev_router_f32,
                                                                                                                                         (int)num_experts, (int)per16, logits_g);
        ctx->launches++;
        ZQ_CUDA_CHECK(cudaGetLastError(), err);
        const unsigned sel_grid = (unsigned)((m + kRouterThreads / 32 - 1) / (kRouterThreads / 32));
        router_select_kernel<<<sel_grid, kRouterThreads, (kRouterThreads / 32) * num_experts * sizeof(float), ctx->stream>>>(logits_g, dev_bias_f32, (int)m, (int)num_experts, (int)top_k, scaling_factor, normalize_selected, dev_ids,
                                                                                                                            dev_weights, ctx->status_dev, scoring);
        ctx->launches++;
        ZQ_CUDA_CHECK(cudaGetLastError(), err);
        return ZQ_OK;
    }
    if (blocks_y > 1) {
        int rc = ensure_moe_ws(ctx, m * num_experts * sizeof(float), err);  // the logits; consumed before anything else uses the buffer
        if (rc) return rc;
        float *logits_g = reinterpret_cast<float *>(ctx->moe_ws);
        router_topk_kernel<<<dim3(grid, (unsigned)blocks_y), kRouterThreads, smem, ctx->stream>>>(dev_x, x_dtype, (int)m, (int)hidden, dev_router_f32, dev_bias_f32, (int)num_experts, (int)top_k, scaling_factor, normalize_selected,
                                                                                                   dev_ids, dev_weights, (int)per_cta, logits_g, ctx->status_dev, scoring);
        ctx->launches++;
        ZQ_CUDA_CHECK(cudaGetLastError(), err);
        const unsigned sel_grid = (unsigned)((m + kRouterThreads / 32 - 1) / (kRouterThreads / 32));
        router_select_kernel<<<sel_grid, kRouterThreads, (kRouterThreads / 32) * num_experts * sizeof(float), ctx->stream>>>(logits_g, scoring == ZQ_ROUTE_SOFTMAX ? nullptr : dev_bias_f32, (int)m, (int)num_experts, (int)top_k, scaling_factor, normalize_selected, dev_ids, dev_weights, ctx->status_dev, scoring);
        ctx->launches++;
        ZQ_CUDA_CHECK(cudaGetLastError(), err);
        return ZQ_OK;
    }
    router_topk_kernel<<<grid, kRouterThreads, smem, ctx->stream>>>(dev_x, x_dtype, (int)m, (int)hidden, dev_router_f32, dev_bias_f32, (int)num_experts, (int)top_k, scaling_factor, normalize_selected, dev_ids, dev_weights,
                                                                    (int)num_experts, nullptr, ctx->status_dev, scoring);
    ctx->launches++;
    ZQ_CUDA_CHECK(cudaGetLastError(), err);
    return ZQ_OK;
}

int zq_moe_gather_rows(zq_ctx *ctx, const void *dev_x, int dtype, size_t x_rows, size_t hidden, const uint32_t *dev_row_ids, size_t n_rows, void *dev_out, zq_error *err) {
    if (!ctx || !dev_x || !dev_row_ids || !dev_out) return set_error(err, ZQ_ERR_ARG, "zq_moe_gather_rows: null argument");
    if (dtype != ZQ_F32 && dtype != ZQ_F16 && dtype != ZQ_BF16) return set_error(err, ZQ_ERR_ARG, "zq_moe_gather_rows: unknown dtype %d", dtype);
    if (n_rows == 0 || hidden == 0 || (hidden * dtype_size(dtype)) % 16) return set_error(err, ZQ_ERR_SHAPE, "zq_moe_gather_rows: rows=%zu hidden=%zu (a row must be a multiple of 16 bytes)", n_rows, hidden);
    if ((reinterpret_cast<uintptr_t>(dev_x) & 15) || (reinterpret_cast<uintptr_t>(dev_out) & 15)) return set_error(err, ZQ_ERR_ARG, "zq_moe_gather_rows: buffers must be 16-byte aligned");
    if (int rc = use_device(ctx, err)) return rc;
    gather_rows_checked_kernel<<<grid_for(ctx, n_rows * (hidden * dtype_size(dtype) / 16), 256), 256, 0, ctx->stream>>>(dev_x, dtype, dev_row_ids, n_rows, x_rows, (int)hidden, dev_out, ctx->status_dev);
    ctx->launches++;
    ZQ_CUDA_CHECK(cudaGetLastError(), err);
    return ZQ_OK;
}

int zq_moe_scatter_add_rows(zq_ctx *ctx, const void *dev_rows, int dtype, const uint32_t *dev_row_ids, const float *dev_weights, size_t n_rows, size_t hidden, float *dev_out_f32, size_t out_rows, zq_error *err) {
    if (!ctx || !dev_rows || !dev_row_ids || !dev_out_f32) return set_error(err, ZQ_ERR_ARG, "zq_moe_scatter_add_rows: null argument");
    if (dtype != ZQ_F32 && dtype != ZQ_F16 && dtype != ZQ_BF16) return set_error(err, ZQ_ERR_ARG, "zq_moe_scatter_add_rows: unknown dtype %d", dtype);
    if (n_rows == 0 || hidden == 0 || out_rows == 0 || hidden > (size_t)INT32_MAX) return set_error(err, ZQ_ERR_SHAPE, "zq_moe_scatter_add_rows: rows=%zu hidden=%zu targets=%zu", n_rows, hidden, out_rows);
    if (int rc = use_device(ctx, err)) return rc;
    scatter_add_rows_kernel<<<grid_for(ctx, n_rows * hidden, 256), 256, 0, ctx->stream>>>(dev_rows, dtype, dev_row_ids, dev_weights, n_rows, (int)hidden, out_rows, dev_out_f32, ctx->status_dev);
    ctx->launches++;
    ZQ_CUDA_CHECK(cudaGetLastError(), err);
    return ZQ_OK;
}

int zq_moe_experts_create(zq_ctx *ctx, const zq_weight *const *gate, const zq_weight *const *up, const zq_weight *const *down, size_t num_experts, zq_moe_experts **out, zq_error *err) {
    if (!ctx || !gate || !up || !down || !out || num_experts == 0) return set_error(err, ZQ_ERR_ARG, "zq_moe_experts_create: null or empty argument");
    zq_moe_experts *t = new zq_moe_experts();
    t->ctx = ctx;
    t->num_experts = num_experts;
    for (size_t e = 0; e < num_experts; ++e) {
        const zq_weight *g = gate[e], *u = up[e], *d = down[e];
        if (!g || !u || !d || g->ctx != ctx || u->ctx != ctx || d->ctx != ctx) {
            delete t;
            return set_error(err, ZQ_ERR_ARG, "expert %zu: missing weight or weight from another context", e);
        }
        if (e == 0) {
            t->hidden = g->cols;
            t->inter = g->rows;
        }
        if (g->cols != t->hidden || g->rows != t->inter || u->cols != t->hidden || u->rows != t->inter || d->cols != t->inter || d->rows != t->hidden || g->type != u->type) {
            delete t;
            return set_error(err, ZQ_ERR_SHAPE, "expert %zu: gate [%zu,%zu] up [%zu,%zu] down [%zu,%zu] do not form hidden=%zu intermediate=%zu", e, g->rows, g->cols, u->rows, u->cols, d->rows, d->cols, t->hidden, t->inter);
        }
        t->gate.push_back(g);
        t->up.push_back(u);
        t->down.push_back(d);
    }
    // grouped decode path: needs one gate/up type and one down type across the table
    bool uniform = true;
    t->gate_type = gate[0]->type;
    t->down_type = down[0]->type;
    for (size_t e = 0; e < num_experts; ++e) uniform = uniform && gate[e]->type == t->gate_type && down[e]->type == t->down_type;
    if (uniform) {
        std::vector<CUtensorMap> hg(num_experts), hu(num_experts), hd(num_experts), qg(num_experts), qu(num_experts), qd(num_experts);
        for (size_t e = 0; e < num_experts; ++e) {
            hg[e] = gate[e]->gemv_map_half;
            hu[e] = up[e]->gemv_map_half;
            hd[e] = down[e]->gemv_map;
            qg[e] = gate[e]->qmv_map;
            qu[e] = up[e]->qmv_map;
            qd[e] = down[e]->qmv_map;
        }
        const size_t bytes = num_experts * sizeof(CUtensorMap);
        cudaError_t ce = cudaMalloc(&t->d_gate_maps, bytes);
        if (ce == cudaSuccess) ce = cudaMalloc(&t->d_up_maps, bytes);
        if (ce == cudaSuccess) ce = cudaMalloc(&t->d_down_maps, bytes);
        if (ce == cudaSuccess) ce = cudaMalloc(&t->d_gate_qmaps, bytes);
        if (ce == cudaSuccess) ce = cudaMalloc(&t->d_up_qmaps, bytes);
        if (ce == cudaSuccess) ce = cudaMalloc(&t->d_down_qmaps, bytes);
        if (ce == cudaSuccess) ce = cudaMemcpy(t->d_gate_maps, hg.data(), bytes, cudaMemcpyHostToDevice);
        if (ce == cudaSuccess) ce = cudaMemcpy(t->d_up_maps, hu.data(), bytes, cudaMemcpyHostToDevice);
        if (ce == cudaSuccess) ce = cudaMemcpy(t->d_down_maps, hd.data(), bytes, cudaMemcpyHostToDevice);
        if (ce == cudaSuccess) ce = cudaMemcpy(t->d_gate_qmaps, qg.data(), bytes, cudaMemcpyHostToDevice);
        if (ce == cudaSuccess) ce = cudaMemcpy(t->d_up_qmaps, qu.data(), bytes, cudaMemcpyHostToDevice);
        if (ce == cudaSuccess) ce = cudaMemcpy(t->d_down_qmaps, qd.data(), bytes, cudaMemcpyHostToDevice);
        if (ce != cudaSuccess) {
            zq_moe_experts_destroy(t);
            return set_error(err, ZQ_ERR_CUDA, "zq_moe_experts_create: tensor-map table: %s", cudaGetErrorString(ce));
        }
    }
    *out = t;
    return ZQ_OK;
}

void zq_moe_experts_destroy(zq_moe_experts *experts) {
    if (!experts) return;
    if (experts->d_gate_maps) cudaFree(experts->d_gate_maps);
    if (experts->d_up_maps) cudaFree(experts->d_up_maps);
    if (experts->d_down_maps) cudaFree(experts->d_down_maps);
    if (experts->d_gate_qmaps) cudaFree(experts->d_gate_qmaps);
    if (experts->d_up_qmaps) cudaFree(experts->d_up_qmaps);
    if (experts->d_down_qmaps) cudaFree(experts->d_down_qmaps);
    delete experts;
}

int zq_moe_forward(zq_ctx *ctx, const zq_moe_experts *experts, const zq_weight *shared_gate, const zq_weight *shared_up, const zq_weight *shared_down, const void *dev_x, int x_dtype, size_t m, const uint32_t *dev_ids,
                   const float *dev_weights, size_t top_k, void *dev_y, int y_dtype, const void *dev_residual, zq_error *err) {
    if (!ctx || !experts || !dev_x || !dev_ids || !dev_weights || !dev_y) return set_error(err, ZQ_ERR_ARG, "zq_moe_forward: null argument");
    if (experts->ctx != ctx) return set_error(err, ZQ_ERR_ARG, "zq_moe_forward: expert table belongs to another context");
    if (m == 0 || top_k == 0) return set_error(err, ZQ_ERR_SHAPE, "zq_moe_forward: empty routing (rows=%zu top_k=%zu)", m, top_k);
    if (x_dtype != ZQ_F32 && x_dtype != ZQ_F16 && x_dtype != ZQ_BF16) return set_error(err, ZQ_ERR_ARG, "zq_moe_forward: unknown input dtype %d", x_dtype);
    if (y_dtype != ZQ_F32 && y_dtype != ZQ_F16 && y_dtype != ZQ_BF16) return set_error(err, ZQ_ERR_ARG, "zq_moe_forward: unknown output dtype %d", y_dtype);
    // rows are gathered and stored with 16-byte accesses
    if ((reinterpret_cast<uintptr_t>(dev_x) & 15) || (reinterpret_cast<uintptr_t>(dev_y) & 15) || (reinterpret_cast<uintptr_t>(dev_residual) & 15)) return set_error(err, ZQ_ERR_ARG, "zq_moe_forward: x, y and residual must be 16-byte aligned");
    if ((reinterpret_cast<uintptr_t>(dev_ids) & 3) || (reinterpret_cast<uintptr_t>(dev_weights) & 3)) return set_error(err, ZQ_ERR_ARG, "zq_moe_forward: ids and weights must be 4-byte aligned");
    if (experts->hidden % 32 || experts->inter % 32) return set_error(err, ZQ_ERR_SHAPE, "zq_moe_forward: hidden=%zu and intermediate=%zu must be multiples of 32", experts->hidden, experts->inter);
    if (int rc = use_device(ctx, err)) return rc;
    {
        cudaError_t stale = cudaGetLastError();  // an error some earlier call of this thread left behind is not this call's
        if (stale != cudaSuccess) return set_error(err, ZQ_ERR_CUDA, "zq_moe_forward: the CUDA runtime already held an error on entry: %s", cudaGetErrorString(stale));
    }
    const bool has_shared = shared_gate || shared_up || shared_down;
    if (has_shared && !(shared_gate && shared_up && shared_down)) return set_error(err, ZQ_ERR_ARG, "zq_moe_forward: shared expert needs gate, up and down");
    const size_t E = experts->num_experts, H = experts->hidden, I = experts->inter, routes = m * top_k;
    if (has_shared && (shared_gate->cols != H || shared_down->rows != H || shared_down->cols != shared_gate->rows)) return set_error(err, ZQ_ERR_SHAPE, "zq_moe_forward: shared expert shapes do not match hidden=%zu", H);

    // ---- decode-sized batch: everything stays on the device
    if (!ctx->force_moe_per_expert && moe_grouped_supported(experts, m, top_k) && routes <= 16 * E) {
        int rc = ensure_moe_ws(ctx, moe_grouped_ws_bytes(experts, m, top_k, has_shared), err);
        if (rc) return rc;
        float *d_out = nullptr, *d_token_w = nullptr, *d_shared = nullptr;
        uint32_t *d_token_slots = nullptr;
        // a shared expert shaped like the routed ones is one more entry of the work list (one row per token)
        const bool rides = has_shared && moe_shared_rides_along(experts, shared_gate, shared_up, shared_down);
        rc = moe_grouped_forward(ctx, experts, rides ? shared_gate : nullptr, rides ? shared_up : nullptr, rides ? shared_down : nullptr, dev_x, x_dtype, m, dev_ids, dev_weights, top_k,
                                 reinterpret_cast<uint8_t *>(ctx->moe_ws), &d_out, &d_token_slots, &d_token_w, &d_shared, has_shared, err);
        if (rc) return rc;
        if (has_shared && !rides) {
            rc = zq_gated_mlp(ctx, shared_gate, shared_up, shared_down, dev_x, x_dtype, m, d_shared, ZQ_F32, nullptr, err);
            if (rc) return rc;
        }
        combine_kernel<<<grid_for(ctx, m * (H / 4), 256), 256, 0, ctx->stream>>>(d_out, d_token_slots, d_token_w, (int)top_k, d_shared, dev_residual, dev_y, y_dtype, m, (int)H, ctx->moe_row_sink ? *reinterpret_cast<const PeerRowSink *>(ctx->moe_row_sink) : PeerRowSink());
        ctx->launches++;
        ZQ_CUDA_CHECK(cudaGetLastError(), err);
        return ZQ_OK;
    }

    // ---- prefill with Q4_K experts: grouping, gather and the two grouped GEMMs stay on the device
    if (!ctx->force_moe_per_expert && !ctx->force_moe_host_grouping && !ctx->disable_fused_gemm && routes >= 32 * E && E <= (size_t)kGroupThreads && top_k <= 64 && experts->d_gate_qmaps &&
        experts->gate_type == ZQ_Q4_K && experts->down_type == ZQ_Q4_K && H % kUnitWeights == 0 && I % kUnitWeights == 0)
        return moe_prefill_device(ctx, experts, shared_gate, shared_up, shared_down, dev_x, x_dtype, m, dev_ids, dev_weights, top_k, dev_y, y_dtype, dev_residual, err);

    // ---- routing back to the host, token-major stable grouping (src/moe/routing.rs:136-156)
    std::vector<uint32_t> ids(routes);
    std::vector<float> wts(routes);
    ZQ_CUDA_CHECK(cudaMemcpyAsync(ids.data(), dev_ids, routes * sizeof(uint32_t), cudaMemcpyDeviceToHost, ctx->stream), err);
    ZQ_CUDA_CHECK(cudaMemcpyAsync(wts.data(), dev_weights, routes * sizeof(float), cudaMemcpyDeviceToHost, ctx->stream), err);
    ZQ_CUDA_CHECK(cudaStreamSynchronize(ctx->stream), err);
    std::vector<uint32_t> offsets(E + 1, 0);
    for (size_t r = 0; r < routes; ++r) {
        if (ids[r] == ZQ_MOE_NO_ROUTE) continue;  // an absent route: no expert runs for it, its weight counts as 0
        if (ids[r] >= E) return set_error(err, ZQ_ERR_SHAPE, "router returned expert %u, table holds %zu", ids[r], E);
        offsets[ids[r] + 1]++;
    }
    for (size_t e = 0; e < E; ++e) offsets[e + 1] += offsets[e];
    std::vector<uint32_t> cursor(offsets.begin(), offsets.end() - 1);
    std::vector<uint32_t> slot_token(routes), token_slots(routes);
    std::vector<float> token_w(routes);
    std::vector<uint32_t> fill(m, 0);
    // visiting routes token-major and experts ascending keeps, per token, its slots in ascending expert order
    std::vector<std::pair<uint32_t, uint32_t>> order(top_k);
    for (size_t t = 0; t < m; ++t) {
        for (size_t j = 0; j < top_k; ++j) {
            uint32_t e = ids[t * top_k + j];
            if (e == ZQ_MOE_NO_ROUTE) {  // sorts behind every real expert; slot 0 is never read for a zero weight
                order[j] = {e, (uint32_t)j};
                token_slots[t * top_k + j] = 0;
                wts[t * top_k + j] = 0.f;
                continue;
            }
            uint32_t slot = cursor[e]++;
            slot_token[slot] = (uint32_t)t;
            order[j] = {e, (uint32_t)j};
            token_slots[t * top_k + j] = slot;
        }
        // per-token combine order: ascending expert id (src/backend/cpu/moe.rs:107-141); stable for repeated ids
        std::stable_sort(order.begin(), order.end(), [](const std::pair<uint32_t, uint32_t> &a, const std::pair<uint32_t, uint32_t> &b) { return a.first < b.first; });
        uint32_t tmp_s[64];
        float tmp_w[64];
        if (top_k > 64) return set_error(err, ZQ_ERR_SHAPE, "zq_moe_forward: top_k=%zu above 64", top_k);
        for (size_t j = 0; j < top_k; ++j) {
            tmp_s[j] = token_slots[t * top_k + order[j].second];
            tmp_w[j] = wts[t * top_k + order[j].second];
        }
        for (size_t j = 0; j < top_k; ++j) {
            token_slots[t * top_k + j] = tmp_s[j];
            token_w[t * top_k + j] = tmp_w[j];
        }
    }

    // ---- workspace: [slot_token | token_slots | token_w | gathered x | activated | routed out | shared out]
    const size_t esz = dtype_size(x_dtype);
    auto al = [](size_t v) { return (v + 255) & ~size_t(255); };
    const size_t o_slot_token = 0, o_token_slots = o_slot_token + al(routes * 4), o_token_w = o_token_slots + al(routes * 4);
    const size_t o_xs = o_token_w + al(routes * 4), o_act = o_xs + al(routes * H * esz), o_out = o_act + al(routes * I * 4);
    const size_t o_shared = o_out + al(routes * H * 4), total = o_shared + (has_shared ? al(m * H * 4) : 0);
    int rc = ensure_moe_ws(ctx, total, err);
    if (rc) return rc;
    uint8_t *ws = reinterpret_cast<uint8_t *>(ctx->moe_ws);
    uint32_t *d_slot_token = reinterpret_cast<uint32_t *>(ws + o_slot_token), *d_token_slots = reinterpret_cast<uint32_t *>(ws + o_token_slots);
    float *d_token_w = reinterpret_cast<float *>(ws + o_token_w);
    uint8_t *d_xs = ws + o_xs;
    float *d_act = reinterpret_cast<float *>(ws + o_act), *d_out = reinterpret_cast<float *>(ws + o_out), *d_shared = has_shared ? reinterpret_cast<float *>(ws + o_shared) : nullptr;
    ZQ_CUDA_CHECK(cudaMemcpyAsync(d_slot_token, slot_token.data(), routes * 4, cudaMemcpyHostToDevice, ctx->stream), err);
    ZQ_CUDA_CHECK(cudaMemcpyAsync(d_token_slots, token_slots.data(), routes * 4, cudaMemcpyHostToDevice, ctx->stream), err);
    ZQ_CUDA_CHECK(cudaMemcpyAsync(d_token_w, token_w.data(), routes * 4, cudaMemcpyHostToDevice, ctx->stream), err);
    ZQ_CUDA_CHECK(cudaStreamSynchronize(ctx->stream), err);  // the host vectors go out of scope at return

    gather_rows_kernel<<<grid_for(ctx, routes * (H * esz / 16), 256), 256, 0, ctx->stream>>>(dev_x, x_dtype, d_slot_token, routes, (int)H, d_xs);
    ctx->launches++;
    ZQ_CUDA_CHECK(cudaGetLastError(), err);

    // ---- experts, ascending id (src/moe/routing.rs:180-213: gather rows, expert batch, weighted scatter)
    const bool grouped_gemm = !ctx->force_moe_per_expert && routes >= 32 * E && H % 8 == 0 && I % 8 == 0;
    const bool fused_gemm = grouped_gemm && !ctx->disable_fused_gemm && experts->d_gate_qmaps && experts->gate_type == ZQ_Q4_K && experts->down_type == ZQ_Q4_K && H % kUnitWeights == 0 && I % kUnitWeights == 0;
    if (fused_gemm) {
        // Prefill, Q4_K experts: two launches for the whole layer.  The fused tensor-core GEMM dequantises the packed
        // tiles of whichever expert a work item names (per-expert tensor maps in a device table), so there is no f16
        // copy of any expert.  Work list: one item per (expert, 256-token tile, 128-row tile); tokens are the gathered
        // slot rows, so outputs land in slot order as the combine expects.
        auto al2 = [](size_t v) { return (v + 1023) & ~size_t(1023); };
        std::vector<int4> items;
        const int rt_i = (int)((I + 127) / 128), rt_h = (int)((H + 127) / 128);
        for (size_t e = 0; e < E; ++e) {
            const int first = (int)offsets[e], end = (int)offsets[e + 1];
            for (int t0 = first; t0 < end; t0 += 256)
                for (int rt = 0; rt < rt_i; ++rt) items.push_back(make_int4((int)e, rt * 128, t0, end));
        }
        const int n_gated = (int)items.size();
        for (size_t e = 0; e < E; ++e) {
            const int first = (int)offsets[e], end = (int)offsets[e + 1];
            for (int t0 = first; t0 < end; t0 += 256)
                for (int rt = 0; rt < rt_h; ++rt) items.push_back(make_int4((int)e, rt * 128, t0, end));
        }
        const int n_down = (int)items.size() - n_gated;
        const size_t x16_bytes = al2(routes * H * sizeof(__half)), act16_bytes = al2(routes * I * sizeof(__half)), items_bytes = al2(items.size() * sizeof(int4));
        rc = ensure_workspace(ctx, x16_bytes + act16_bytes + items_bytes, err);
        if (rc) return rc;
        uint8_t *wsb = reinterpret_cast<uint8_t *>(ctx->workspace);
        __half *x16 = reinterpret_cast<__half *>(wsb), *act16 = reinterpret_cast<__half *>(wsb + x16_bytes);
        int4 *d_items = reinterpret_cast<int4 *>(wsb + x16_bytes + act16_bytes);
        ZQ_CUDA_CHECK(cudaMemcpyAsync(d_items, items.data(), items.size() * sizeof(int4), cudaMemcpyHostToDevice, ctx->stream), err);
        ZQ_CUDA_CHECK(cudaStreamSynchronize(ctx->stream), err);  // the host vector goes out of scope at return
        const __half *xin = reinterpret_cast<const __half *>(d_xs);
        if (x_dtype != ZQ_F16) {
            rc = launch_to_f16(ctx, d_xs, x_dtype, x16, routes * H, err);
            if (rc) return rc;
            xin = x16;
        }
        rc = launch_gemm_fused_grouped(ctx, experts->d_gate_qmaps, experts->d_up_qmaps, I, H, xin, routes, d_items, n_gated, nullptr, act16, ZQ_F16, err);
        if (rc) return rc;
        rc = launch_gemm_fused_grouped(ctx, experts->d_down_qmaps, nullptr, H, I, act16, routes, d_items + n_gated, n_down, nullptr, d_out, ZQ_F32, err);
        if (rc) return rc;
    } else if (grouped_gemm) {
        // Prefill: one grouped tensor-core GEMM per projection and chunk of experts instead of two launches per
        // expert (an expert's own GEMM has 16-56 tiles for 148 SMs).  The chunk's packed weights are dequantised to
        // f16 stacks [chunk][rows][K] in the workspace; the work list holds one item per (expert, token tile, row
        // tile); tokens are the gathered slot rows, so outputs land in slot order as the combine expects.
        const size_t per_expert = 3 * I * H * sizeof(__half);
        size_t chunk = (size_t(3) << 30) / per_expert;  // ~3 GB of f16 operands at a time
        if (chunk < 1) chunk = 1;
        if (chunk > E) chunk = E;
        auto al2 = [](size_t v) { return (v + 1023) & ~size_t(1023); };
        const size_t w_stack = al2(chunk * I * H * sizeof(__half));
        const size_t x16_bytes = al2(routes * H * sizeof(__half)), act16_bytes = al2(routes * I * sizeof(__half));
        std::vector<int4> items;
        struct ChunkPlan { size_t e0, e1; int gated_first, gated_n, down_first, down_n; };
        std::vector<ChunkPlan> plans;
        const int rt_i = (int)((I + 127) / 128), rt_h = (int)((H + 127) / 128);
        for (size_t e0 = 0; e0 < E; e0 += chunk) {
            ChunkPlan cp;
            cp.e0 = e0;
            cp.e1 = e0 + chunk < E ? e0 + chunk : E;
            cp.gated_first = (int)items.size();
            for (size_t e = cp.e0; e < cp.e1; ++e) {
                const int first = (int)offsets[e], end = (int)offsets[e + 1];
                for (int t0 = first; t0 < end; t0 += 256)
                    for (int rt = 0; rt < rt_i; ++rt) items.push_back(make_int4((int)(e - e0), rt * 128, t0, end));
            }
            cp.gated_n = (int)items.size() - cp.gated_first;
            cp.down_first = (int)items.size();
            for (size_t e = cp.e0; e < cp.e1; ++e) {
                const int first = (int)offsets[e], end = (int)offsets[e + 1];
                for (int t0 = first; t0 < end; t0 += 256)
                    for (int rt = 0; rt < rt_h; ++rt) items.push_back(make_int4((int)(e - e0), rt * 128, t0, end));
            }
            cp.down_n = (int)items.size() - cp.down_first;
            plans.push_back(cp);
        }
        const size_t items_bytes = al2(items.size() * sizeof(int4));
        rc = ensure_workspace(ctx, 3 * w_stack + x16_bytes + act16_bytes + items_bytes, err);
        if (rc) return rc;
        uint8_t *wsb = reinterpret_cast<uint8_t *>(ctx->workspace);
        __half *wg16 = reinterpret_cast<__half *>(wsb), *wu16 = reinterpret_cast<__half *>(wsb + w_stack), *wd16 = reinterpret_cast<__half *>(wsb + 2 * w_stack);
        __half *x16 = reinterpret_cast<__half *>(wsb + 3 * w_stack), *act16 = reinterpret_cast<__half *>(wsb + 3 * w_stack + x16_bytes);
        int4 *d_items = reinterpret_cast<int4 *>(wsb + 3 * w_stack + x16_bytes + act16_bytes);
        ZQ_CUDA_CHECK(cudaMemcpyAsync(d_items, items.data(), items.size() * sizeof(int4), cudaMemcpyHostToDevice, ctx->stream), err);
        ZQ_CUDA_CHECK(cudaStreamSynchronize(ctx->stream), err);  // the host vector goes out of scope at return
        const __half *xin = reinterpret_cast<const __half *>(d_xs);
        if (x_dtype != ZQ_F16) {
            rc = launch_to_f16(ctx, d_xs, x_dtype, x16, routes * H, err);
            if (rc) return rc;
            xin = x16;
        }
        for (const ChunkPlan &cp : plans) {
            if (cp.gated_n == 0) continue;
            std::vector<const zq_weight *> wl_gu, wl_d;
            std::vector<__half *> ol_gu, ol_d;
            for (size_t e = cp.e0; e < cp.e1; ++e) {
                if (offsets[e + 1] == offsets[e]) continue;
                const size_t z = e - cp.e0;
                wl_gu.push_back(experts->gate[e]); ol_gu.push_back(wg16 + z * I * H);
                wl_gu.push_back(experts->up[e]); ol_gu.push_back(wu16 + z * I * H);
                wl_d.push_back(experts->down[e]); ol_d.push_back(wd16 + z * H * I);
            }
            // gate and up share shape but may differ in type from expert to expert only if the table was built so;
            // the batched pass wants one type per launch, so fall back to single launches when they differ
            bool uniform = true;
            for (const zq_weight *w : wl_gu) uniform = uniform && w->type == wl_gu[0]->type;
            for (const zq_weight *w : wl_d) uniform = uniform && w->type == wl_d[0]->type;
            if (uniform) {
                rc = launch_dequantize_f16_batch(ctx, wl_gu.data(), ol_gu.data(), wl_gu.size(), err);
                if (!rc) rc = launch_dequantize_f16_batch(ctx, wl_d.data(), ol_d.data(), wl_d.size(), err);
                if (rc) return rc;
            } else {
                for (size_t i = 0; i < wl_gu.size(); ++i) {
                    rc = launch_dequantize_f16(ctx, wl_gu[i], ol_gu[i], err);
                    if (rc) return rc;
                }
                for (size_t i = 0; i < wl_d.size(); ++i) {
                    rc = launch_dequantize_f16(ctx, wl_d[i], ol_d[i], err);
                    if (rc) return rc;
                }
            }
            rc = launch_gemm_grouped(ctx, wg16, wu16, cp.e1 - cp.e0, I, H, xin, routes, d_items + cp.gated_first, cp.gated_n, act16, ZQ_F16, err);
            if (rc) return rc;
            rc = launch_gemm_grouped(ctx, wd16, nullptr, cp.e1 - cp.e0, H, I, act16, routes, d_items + cp.down_first, cp.down_n, d_out, ZQ_F32, err);
            if (rc) return rc;
        }
    } else {
    for (size_t e = 0; e < E; ++e) {
        const size_t first = offsets[e], count = offsets[e + 1] - offsets[e];
        if (!count) continue;
        rc = zq_gated_silu(ctx, experts->gate[e], experts->up[e], d_xs + first * H * esz, x_dtype, count, d_act + first * I, ZQ_F32, err);
        if (rc) return rc;
        rc = zq_linear(ctx, experts->down[e], d_act + first * I, ZQ_F32, count, d_out + first * H, ZQ_F32, nullptr, err);
        if (rc) return rc;
    }
    }
    if (has_shared) {
        rc = zq_gated_mlp(ctx, shared_gate, shared_up, shared_down, dev_x, x_dtype, m, d_shared, ZQ_F32, nullptr, err);
        if (rc) return rc;
    }
    combine_kernel<<<grid_for(ctx, m * (H / 4), 256), 256, 0, ctx->stream>>>(d_out, d_token_slots, d_token_w, (int)top_k, d_shared, dev_residual, dev_y, y_dtype, m, (int)H, ctx->moe_row_sink ? *reinterpret_cast<const PeerRowSink *>(ctx->moe_row_sink) : PeerRowSink());
    ctx->launches++;
    ZQ_CUDA_CHECK(cudaGetLastError(), err);
    return ZQ_OK;
}

}  // extern "C"
