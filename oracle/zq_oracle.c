/*
 * CPU oracle for the GGUF block-quantized linear path.  TEST INFRASTRUCTURE ONLY.
 *
 * This file restates, in plain C with AVX2/FMA intrinsics, the CPU algorithm of the
 * zLLM reference for this path.  It is the checker for the CUDA library and the timed
 * CPU baseline; nothing in the shipped product may link or call it.
 *
 * Parity pin: the reference is Rust and cannot be compiled in this environment, so the
 * oracle is pinned against the reference's own known-answer unit tests (restated in
 * tests/test_oracle_kat.py) rather than against outputs of the reference binary.
 *
 * Every function cites the reference file:line it follows (paths relative to the
 * reference project root).
 *
 * Third-party arithmetic restated here:
 *   half 2.7.1   f16::from_bits().to_f32()  -> exact widening (F16C _cvtsh_ss)
 *                f16::from_f32()            -> round-to-nearest-even (F16C _cvtss_sh)
 *   wide 0.7.33  f32x8::exp (polynomial)    -> NOT reproducible from the source tree;
 *                libm expf is used instead (the reference's own test allows 1e-5 abs).
 *   rayon 1.12   parallel iteration only    -> pthread static partition over rows;
 *                per-row results do not depend on the partition.
 */
#define _GNU_SOURCE
#include <immintrin.h>
#include <math.h>
#include <pthread.h>
#include <sched.h>
#include <stdint.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#define QK_K 256

/* src/weight/codec/ggml.rs:4 */
static const int8_t KVALUES_IQ4NL[16] = {-127, -104, -83, -65, -49, -35, -22, -10, 1, 13, 25, 38, 53, 69, 89, 113};

/* ------------------------------------------------------------------ f16 helpers */

/* half::f16::from_bits(bits).to_f32(): exact widening (src/weight/codec/ggml.rs:475-477). */
float zqo_f16_to_f32(uint16_t bits) { return _cvtsh_ss(bits); }

/* half::f16::from_f32(value).to_bits(): round to nearest even (src/weight/codec/ggml.rs:198-202). */
uint16_t zqo_f32_to_f16(float value) { return _cvtss_sh(value, _MM_FROUND_TO_NEAREST_INT | _MM_FROUND_NO_EXC); }

static inline float read_f16(const uint8_t *bytes, size_t offset) {
    return zqo_f16_to_f32((uint16_t)(bytes[offset] | (bytes[offset + 1] << 8)));
}

/* ------------------------------------------------------------------ layouts */

/* src/weight/codec/ggml.rs:33-71 (block_layout), the four types on the path plus Q5_K/Q6_K. */
int zqo_block_layout(uint32_t tensor_type, size_t *elements, size_t *bytes) {
    switch (tensor_type) {
    case 0: *elements = 1; *bytes = 4; return 0;
    case 1: *elements = 1; *bytes = 2; return 0;
    case 2: *elements = 32; *bytes = 18; return 0;
    case 6: *elements = 32; *bytes = 22; return 0;
    case 7: *elements = 32; *bytes = 24; return 0;
    case 8: *elements = 32; *bytes = 34; return 0;
    case 11: *elements = QK_K; *bytes = 110; return 0;
    case 12: *elements = QK_K; *bytes = 144; return 0;
    case 13: *elements = QK_K; *bytes = 176; return 0;
    case 14: *elements = QK_K; *bytes = 210; return 0;
    case 20: *elements = 32; *bytes = 18; return 0;
    case 23: *elements = QK_K; *bytes = 136; return 0;
    default: return -1;
    }
}

/* ------------------------------------------------------------------ block decode */

/* src/weight/codec/ggml.rs:102-109 */
static void decode_q4_0(const uint8_t *block, float *output) {
    float scale = read_f16(block, 0);
    for (int index = 0; index < 16; ++index) {
        uint8_t pair = block[2 + index];
        output[index] = (float)((int)(pair & 0x0f) - 8) * scale;
        output[index + 16] = (float)((int)(pair >> 4) - 8) * scale;
    }
}

/* src/weight/codec/ggml.rs:229-234 */
static void decode_q8_0(const uint8_t *block, float *output) {
    float d = read_f16(block, 0);
    for (int index = 0; index < 32; ++index) output[index] = d * (float)(int8_t)block[2 + index];
}

/* src/weight/codec/ggml.rs:237-244 */
static void decode_iq4_nl(const uint8_t *block, float *output) {
    float d = read_f16(block, 0);
    for (int j = 0; j < 16; ++j) {
        uint8_t q = block[2 + j];
        output[j] = d * (float)KVALUES_IQ4NL[q & 0x0f];
        output[j + 16] = d * (float)KVALUES_IQ4NL[q >> 4];
    }
}

/* src/weight/codec/ggml.rs:471-473 (scale_min_k4) */
static inline void scale_min_k4(int group, const uint8_t *scales, uint8_t *scale, uint8_t *min) {
    if (group < 4) {
        *scale = scales[group] & 0x3f;
        *min = scales[group + 4] & 0x3f;
    } else {
        *scale = (uint8_t)((scales[group + 4] & 0x0f) | ((scales[group - 4] >> 6) << 4));
        *min = (uint8_t)((scales[group + 4] >> 4) | ((scales[group] >> 6) << 4));
    }
}

/* src/weight/codec/ggml.rs:408-423: value = d*scale*quant - dmin*min, evaluated left to right in f32. */
static void decode_q4_k(const uint8_t *block, float *output) {
    float d = read_f16(block, 0);
    float dmin = read_f16(block, 2);
    const uint8_t *scales = block + 4;
    const uint8_t *quants = block + 16;
    for (int group = 0; group < 8; ++group) {
        uint8_t scale, min;
        scale_min_k4(group, scales, &scale, &min);
        int source = (group / 2) * 32;
        for (int index = 0; index < 32; ++index) {
            uint8_t packed = quants[source + index];
            uint8_t quant = (group % 2 == 0) ? (packed & 0x0f) : (packed >> 4);
            volatile float left = d * (float)scale;   /* volatile: forbid FMA contraction, keep Rust's order */
            volatile float prod = left * (float)quant;
            volatile float right = dmin * (float)min;
            output[group * 32 + index] = prod - right;
        }
    }
}

/* src/weight/codec/ggml.rs:425-444 */
static void decode_q5_k(const uint8_t *block, float *output) {
    float d = read_f16(block, 0);
    float dmin = read_f16(block, 2);
    const uint8_t *scales = block + 4;
    const uint8_t *high_bits = block + 16;
    const uint8_t *low_bits = block + 48;
    for (int group = 0; group < 8; ++group) {
        uint8_t scale, min;
        scale_min_k4(group, scales, &scale, &min);
        int source = (group / 2) * 32;
        uint8_t high_mask = (uint8_t)(1u << group);
        for (int index = 0; index < 32; ++index) {
            uint8_t packed = low_bits[source + index];
            uint8_t low = (group % 2 == 0) ? (packed & 0x0f) : (packed >> 4);
            uint8_t quant = (uint8_t)(low + ((high_bits[index] & high_mask) ? 16 : 0));
            volatile float left = d * (float)scale;
            volatile float prod = left * (float)quant;
            volatile float right = dmin * (float)min;
            output[group * 32 + index] = prod - right;
        }
    }
}

/* src/weight/codec/ggml.rs:446-469 */
static void decode_q6_k(const uint8_t *block, float *output) {
    const uint8_t *low_bits = block;
    const uint8_t *high_bits = block + 128;
    const int8_t *scales = (const int8_t *)(block + 192);
    float d = read_f16(block, 208);
    for (int half = 0; half < 2; ++half) {
        int low = half * 64, high = half * 32, scale = half * 8, target = half * 128;
        for (int index = 0; index < 32; ++index) {
            int scale_index = index / 16;
            uint8_t high_value = high_bits[high + index];
            int q1 = (int)((low_bits[low + index] & 0x0f) | ((high_value & 3) << 4)) - 32;
            int q2 = (int)((low_bits[low + index + 32] & 0x0f) | (((high_value >> 2) & 3) << 4)) - 32;
            int q3 = (int)((low_bits[low + index] >> 4) | (((high_value >> 4) & 3) << 4)) - 32;
            int q4 = (int)((low_bits[low + index + 32] >> 4) | (((high_value >> 6) & 3) << 4)) - 32;
            volatile float s1 = d * (float)scales[scale + scale_index];
            volatile float s2 = d * (float)scales[scale + scale_index + 2];
            volatile float s3 = d * (float)scales[scale + scale_index + 4];
            volatile float s4 = d * (float)scales[scale + scale_index + 6];
            output[target + index] = s1 * (float)q1;
            output[target + index + 32] = s2 * (float)q2;
            output[target + index + 64] = s3 * (float)q3;
            output[target + index + 96] = s4 * (float)q4;
        }
    }
}

/* src/weight/codec/ggml.rs:73-100 (decode_block) */
/* src/weight/codec/ggml.rs:111-119 (Q5_0: f16 scale, 32 high bits, 16 nibble bytes; value = d * (q5 - 16)) */
static void decode_q5_0(const uint8_t *block, float *output) {
    const float scale = read_f16(block, 0);
    uint32_t high;
    memcpy(&high, block + 2, 4);
    for (int index = 0; index < 32; ++index) {
        const uint8_t packed = block[6 + index % 16];
        const uint32_t low = index < 16 ? (uint32_t)(packed & 15) : (uint32_t)(packed >> 4);
        output[index] = scale * (float)((int32_t)(low | (((high >> index) & 1u) << 4)) - 16);
    }
}

/* src/weight/codec/ggml.rs:121-130 (Q5_1: f16 scale, f16 minimum, 32 high bits, 16 nibble bytes; value = d * q5 + m) */
static void decode_q5_1(const uint8_t *block, float *output) {
    const float scale = read_f16(block, 0), minimum = read_f16(block, 2);
    uint32_t high;
    memcpy(&high, block + 4, 4);
    for (int index = 0; index < 16; ++index) {
        const uint8_t low = block[8 + index];
        volatile float a = scale * (float)((uint32_t)(low & 15) | (((high >> index) & 1u) << 4));
        volatile float b = scale * (float)((uint32_t)(low >> 4) | (((high >> (index + 16)) & 1u) << 4));
        output[index] = a + minimum;
        output[index + 16] = b + minimum;
    }
}

/* src/weight/codec/ggml.rs:246-261 (IQ4_XS: f16 d, 16 high scale bits, 4 low scale bytes, 128 nibble bytes; each block of
 * 32 has a 6-bit scale ls, value = d * (ls - 32) * codebook[nibble]) */
static void decode_iq4_xs(const uint8_t *block, float *output) {
    const float d = read_f16(block, 0);
    const uint16_t scales_h = (uint16_t)(block[2] | (block[3] << 8));
    const uint8_t *scales_l = block + 4, *quants = block + 8;
    for (int ib = 0; ib < 8; ++ib) {
        const int ls = ((scales_l[ib / 2] >> (4 * (ib % 2))) & 0x0f) | (((scales_h >> (2 * ib)) & 0x03) << 4);
        const float dl = d * ((float)ls - 32.0f);
        for (int j = 0; j < 16; ++j) {
            const uint8_t q = quants[ib * 16 + j];
            output[ib * 32 + j] = dl * (float)KVALUES_IQ4NL[q & 0x0f];
            output[ib * 32 + j + 16] = dl * (float)KVALUES_IQ4NL[q >> 4];
        }
    }
}

/* src/weight/codec/ggml.rs:384-406 (Q3_K: 32 high-bit mask bytes, 64 two-bit bytes, 12 scale bytes, f16 d; 16 groups of
 * 16 with a 6-bit scale - 32; value = d * scale * (q2 - (high bit clear ? 4 : 0)), multiplied left to right) */
static void decode_q3_k(const uint8_t *block, float *output) {
    const uint8_t *hmask = block, *quants = block + 32, *scales = block + 96;
    const float d = read_f16(block, 108);
    for (int group = 0; group < 16; ++group) {
        const uint8_t low = group < 8 ? (uint8_t)(scales[group] & 0x0f) : (uint8_t)(scales[group - 8] >> 4);
        const uint8_t high = (uint8_t)((scales[8 + group % 4] >> (2 * (group / 4))) & 0x03);
        const int scale = (int)(low | (high << 4)) - 32;
        const int half = group / 8, pair = group % 8;
        const int source = half * 32 + (pair % 2) * 16, mask_source = (pair % 2) * 16, shift = 2 * (pair / 2);
        const uint8_t mask = (uint8_t)(1u << (group / 2));
        for (int index = 0; index < 16; ++index) {
            const int low_bits = (quants[source + index] >> shift) & 0x03;
            const int quant = low_bits - ((hmask[mask_source + index] & mask) == 0 ? 4 : 0);
            volatile float ds = d * (float)scale;
            output[group * 16 + index] = ds * (float)quant;
        }
    }
}

int zqo_decode_block(uint32_t tensor_type, const uint8_t *bytes, size_t nbytes, float *output, size_t noutput) {
    size_t elements, block_bytes;
    if (zqo_block_layout(tensor_type, &elements, &block_bytes)) return -1;
    if (nbytes != block_bytes || noutput != elements) return -2;
    switch (tensor_type) {
    case 0: memcpy(output, bytes, 4); return 0;
    case 1: output[0] = read_f16(bytes, 0); return 0;
    case 2: decode_q4_0(bytes, output); return 0;
    case 6: decode_q5_0(bytes, output); return 0;
    case 7: decode_q5_1(bytes, output); return 0;
    case 8: decode_q8_0(bytes, output); return 0;
    case 11: decode_q3_k(bytes, output); return 0;
    case 12: decode_q4_k(bytes, output); return 0;
    case 13: decode_q5_k(bytes, output); return 0;
    case 14: decode_q6_k(bytes, output); return 0;
    case 20: decode_iq4_nl(bytes, output); return 0;
    case 23: decode_iq4_xs(bytes, output); return 0;
    default: return -1;
    }
}

/* src/weight/codec/ggml.rs:146-160 (dequantize): errors on misaligned element count or byte count. */
int zqo_dequantize(uint32_t tensor_type, const uint8_t *bytes, size_t nbytes, size_t elements, float *output) {
    size_t block_elements, block_bytes;
    if (zqo_block_layout(tensor_type, &block_elements, &block_bytes)) return -1;
    if (elements % block_elements) return -2;
    if (nbytes != elements / block_elements * block_bytes) return -3;
    for (size_t block = 0; block < elements / block_elements; ++block)
        zqo_decode_block(tensor_type, bytes + block * block_bytes, block_bytes, output + block * block_elements, block_elements);
    return 0;
}

/* ------------------------------------------------------------------ Q4_K encoder */

/* Rust f32::round: half away from zero == C roundf. Rust f32::clamp(lo,hi) on non-NaN == fminf(fmaxf()). */
static inline float clampf(float v, float lo, float hi) { return v < lo ? lo : (v > hi ? hi : v); }

/* src/weight/codec/ggml.rs:188-227 (encode_q4_k) */
void zqo_encode_q4_k(const float *values, uint8_t *block) {
    float scales[8], minimums[8];
    for (int group = 0; group < 8; ++group) {
        const float *v = values + group * 32;
        float minimum = INFINITY, maximum = -INFINITY;
        for (int i = 0; i < 32; ++i) {
            minimum = fminf(minimum, v[i]);
            maximum = fmaxf(maximum, v[i]);
        }
        minimums[group] = fmaxf(-minimum, 0.0f);
        scales[group] = fmaxf(maximum + minimums[group], 0.0f) / 15.0f;
    }
    float max_scale = 0.0f, max_min = 0.0f;
    for (int group = 0; group < 8; ++group) {
        max_scale = fmaxf(max_scale, scales[group]);
        max_min = fmaxf(max_min, minimums[group]);
    }
    float d = zqo_f16_to_f32(zqo_f32_to_f16(max_scale / 63.0f));
    float dmin = zqo_f16_to_f32(zqo_f32_to_f16(max_min / 63.0f));
    memset(block, 0, 144);
    uint16_t d_bits = zqo_f32_to_f16(d), dmin_bits = zqo_f32_to_f16(dmin);
    block[0] = (uint8_t)d_bits; block[1] = (uint8_t)(d_bits >> 8);
    block[2] = (uint8_t)dmin_bits; block[3] = (uint8_t)(dmin_bits >> 8);
    uint8_t scale_codes[8], minimum_codes[8];
    for (int group = 0; group < 8; ++group) {
        scale_codes[group] = d == 0.0f ? 0 : (uint8_t)clampf(roundf(scales[group] / d), 0.0f, 63.0f);
        minimum_codes[group] = dmin == 0.0f ? 0 : (uint8_t)clampf(roundf(minimums[group] / dmin), 0.0f, 63.0f);
    }
    for (int group = 0; group < 4; ++group) {
        block[4 + group] = (uint8_t)((scale_codes[group] & 0x3f) | ((scale_codes[group + 4] >> 4) << 6));
        block[8 + group] = (uint8_t)((minimum_codes[group] & 0x3f) | ((minimum_codes[group + 4] >> 4) << 6));
        block[12 + group] = (uint8_t)((scale_codes[group + 4] & 0x0f) | ((minimum_codes[group + 4] & 0x0f) << 4));
    }
    for (int group = 0; group < 8; ++group) {
        volatile float scale = d * (float)scale_codes[group];
        volatile float minimum = dmin * (float)minimum_codes[group];
        for (int index = 0; index < 32; ++index) {
            uint8_t quant = 0;
            if (scale != 0.0f) {
                volatile float shifted = values[group * 32 + index] + minimum;
                quant = (uint8_t)clampf(roundf(shifted / scale), 0.0f, 15.0f);
            }
            int target = 16 + (group / 2) * 32 + index;
            if (group % 2 == 0) block[target] = quant;
            else block[target] |= (uint8_t)(quant << 4);
        }
    }
}

/* src/weight/codec/ggml.rs:163-186 (requantize_q4_k): sources Q8_0, Q4_K (copy), Q5_K. */
int zqo_requantize_q4_k(uint32_t tensor_type, const uint8_t *bytes, size_t nbytes, size_t elements, uint8_t *output) {
    size_t source_elements, source_bytes;
    if (zqo_block_layout(tensor_type, &source_elements, &source_bytes)) return -1;
    if (!(tensor_type == 8 || tensor_type == 12 || tensor_type == 13) || elements % QK_K || QK_K % source_elements) return -2;
    if (nbytes != elements / source_elements * source_bytes) return -3;
    if (tensor_type == 12) { memcpy(output, bytes, nbytes); return 0; }
    float values[QK_K];
    size_t per = QK_K / source_elements;
    for (size_t block = 0; block < elements / QK_K; ++block) {
        for (size_t source = 0; source < per; ++source)
            zqo_decode_block(tensor_type, bytes + (block * per + source) * source_bytes, source_bytes, values + source * source_elements, source_elements);
        zqo_encode_q4_k(values, output + block * 144);
    }
    return 0;
}

/* ------------------------------------------------------------------ thread team */

static int g_threads = 0;

/* Cores in the process affinity mask (the reference's allowed_parallelism, src/kernel/cpu/mod.rs:29-44). */
int zqo_allowed_parallelism(void) {
    cpu_set_t set;
    if (sched_getaffinity(0, sizeof(set), &set) == 0) {
        int n = CPU_COUNT(&set);
        if (n > 0) return n;
    }
    return 1;
}

void zqo_set_threads(int threads) { g_threads = threads; }
int zqo_get_threads(void) { return g_threads > 0 ? g_threads : zqo_allowed_parallelism(); }

typedef void (*row_fn)(size_t row, void *ctx);
typedef struct { row_fn fn; void *ctx; size_t begin, end; } row_task;

static void *row_worker(void *arg) {
    row_task *task = (row_task *)arg;
    for (size_t row = task->begin; row < task->end; ++row) task->fn(row, task->ctx);
    return NULL;
}

/* Stand-in for rayon's par_chunks_exact over weight rows: static contiguous partition. */
static void parallel_rows(size_t rows, row_fn fn, void *ctx) {
    int threads = zqo_get_threads();
    if (threads > 256) threads = 256;
    if ((size_t)threads > rows) threads = (int)(rows ? rows : 1);
    if (threads <= 1) {
        for (size_t row = 0; row < rows; ++row) fn(row, ctx);
        return;
    }
    pthread_t handles[256];
    row_task tasks[256];
    for (int t = 0; t < threads; ++t) {
        tasks[t].fn = fn; tasks[t].ctx = ctx;
        tasks[t].begin = rows * (size_t)t / (size_t)threads;
        tasks[t].end = rows * (size_t)(t + 1) / (size_t)threads;
        pthread_create(&handles[t], NULL, row_worker, &tasks[t]);
    }
    for (int t = 0; t < threads; ++t) pthread_join(handles[t], NULL);
}

/* ------------------------------------------------------------------ AVX2 dots */

/* src/kernel/cpu/ggml_quant.rs:157-165 (horizontal_sum_avx2) */
static inline float horizontal_sum_avx2(__m256 value) {
    __m128 halves = _mm_add_ps(_mm256_castps256_ps128(value), _mm256_extractf128_ps(value, 1));
    __m128 pairs = _mm_add_ps(halves, _mm_movehl_ps(halves, halves));
    return _mm_cvtss_f32(_mm_add_ss(pairs, _mm_shuffle_ps(pairs, pairs, 0x55)));
}

/* src/kernel/cpu/ggml_quant.rs:15-43 (dot_f32_avx2): four accumulators over 32-element strides, scalar tail. */
static float dot_f32_avx2(const float *left, const float *right, size_t len) {
    size_t index = 0;
    __m256 sum0 = _mm256_setzero_ps(), sum1 = _mm256_setzero_ps(), sum2 = _mm256_setzero_ps(), sum3 = _mm256_setzero_ps();
    while (index + 32 <= len) {
        sum0 = _mm256_fmadd_ps(_mm256_loadu_ps(left + index), _mm256_loadu_ps(right + index), sum0);
        sum1 = _mm256_fmadd_ps(_mm256_loadu_ps(left + index + 8), _mm256_loadu_ps(right + index + 8), sum1);
        sum2 = _mm256_fmadd_ps(_mm256_loadu_ps(left + index + 16), _mm256_loadu_ps(right + index + 16), sum2);
        sum3 = _mm256_fmadd_ps(_mm256_loadu_ps(left + index + 24), _mm256_loadu_ps(right + index + 24), sum3);
        index += 32;
    }
    __m256 sum = _mm256_add_ps(_mm256_add_ps(sum0, sum1), _mm256_add_ps(sum2, sum3));
    float total = horizontal_sum_avx2(sum);
    while (index < len) {
        volatile float product = left[index] * right[index];
        total += product;
        index += 1;
    }
    return total;
}

/* src/kernel/cpu/ggml_quant.rs:58-80 (q8_0_dot_avx2) */
static float q8_0_dot_avx2(const uint8_t *block, const float *input) {
    __m256 scale = _mm256_set1_ps(read_f16(block, 0));
    __m256i quants = _mm256_loadu_si256((const __m256i *)(block + 2));
    __m128i halves[2] = {_mm256_castsi256_si128(quants), _mm256_extracti128_si256(quants, 1)};
    __m256 total = _mm256_setzero_ps();
    for (int half = 0; half < 2; ++half) {
        __m128i chunks[2] = {halves[half], _mm_srli_si128(halves[half], 8)};
        for (int chunk = 0; chunk < 2; ++chunk) {
            __m256 quant = _mm256_cvtepi32_ps(_mm256_cvtepi8_epi32(chunks[chunk]));
            __m256 weight = _mm256_mul_ps(quant, scale);
            __m256 activation = _mm256_loadu_ps(input + half * 16 + chunk * 8);
            total = _mm256_fmadd_ps(activation, weight, total);
        }
    }
    return horizontal_sum_avx2(total);
}

/* src/kernel/cpu/ggml_quant.rs:82-112 (q4_k_dot_avx2): weight = quant*(d*scale) - dmin*min, fmadd into one accumulator. */
static float q4_k_dot_avx2(const uint8_t *block, const float *input) {
    float d = read_f16(block, 0), dmin = read_f16(block, 2);
    __m256i nibble_mask = _mm256_set1_epi8(15);
    __m256 total = _mm256_setzero_ps();
    for (int group = 0; group < 8; ++group) {
        uint8_t scale_code, min_code;
        scale_min_k4(group, block + 4, &scale_code, &min_code);
        __m256i packed = _mm256_loadu_si256((const __m256i *)(block + 16 + (group / 2) * 32));
        __m256i quants = (group % 2 == 0) ? _mm256_and_si256(packed, nibble_mask) : _mm256_and_si256(_mm256_srli_epi16(packed, 4), nibble_mask);
        __m128i halves[2] = {_mm256_castsi256_si128(quants), _mm256_extracti128_si256(quants, 1)};
        volatile float scale_f = d * (float)scale_code;
        volatile float minimum_f = dmin * (float)min_code;
        __m256 scale = _mm256_set1_ps(scale_f);
        __m256 minimum = _mm256_set1_ps(minimum_f);
        for (int half = 0; half < 2; ++half) {
            __m128i chunks[2] = {halves[half], _mm_srli_si128(halves[half], 8)};
            for (int chunk = 0; chunk < 2; ++chunk) {
                __m256 quant = _mm256_cvtepi32_ps(_mm256_cvtepu8_epi32(chunks[chunk]));
                __m256 weight = _mm256_sub_ps(_mm256_mul_ps(quant, scale), minimum);
                __m256 activation = _mm256_loadu_ps(input + group * 32 + half * 16 + chunk * 8);
                total = _mm256_fmadd_ps(activation, weight, total);
            }
        }
    }
    return horizontal_sum_avx2(total);
}

/* src/kernel/cpu/ggml_quant.rs:167-178 (direct_quant_dot): AVX2 kernels exist for types 8 and 12 only. */
typedef float (*quant_dot_fn)(const uint8_t *, const float *);
static quant_dot_fn direct_quant_dot(uint32_t tensor_type) {
    if (tensor_type == 8) return q8_0_dot_avx2;
    if (tensor_type == 12) return q4_k_dot_avx2;
    return NULL;
}

/* ------------------------------------------------------------------ matvec family */

typedef struct {
    uint32_t tensor_type;
    const uint8_t *bytes, *bytes2;
    size_t rows, columns, input_rows, block_elements, block_bytes, row_bytes;
    const float *input;
    float *output, *scratch, *scratch2;
} mv_ctx;

/* One output row of matvec (src/kernel/cpu/ggml_quant.rs:203-218): per-block dot, scalar sum across blocks. */
static float matvec_row(const mv_ctx *c, const uint8_t *row, const float *input) {
    float decoded[256];
    quant_dot_fn quant_dot = direct_quant_dot(c->tensor_type);
    float sum = 0.0f;
    for (size_t block = 0; block < c->columns / c->block_elements; ++block) {
        const uint8_t *b = row + block * c->block_bytes;
        const float *x = input + block * c->block_elements;
        if (quant_dot) {
            sum += quant_dot(b, x);
        } else {
            zqo_decode_block(c->tensor_type, b, c->block_bytes, decoded, c->block_elements);
            sum += dot_f32_avx2(decoded, x, c->block_elements);
        }
    }
    return sum;
}

static void matvec_task(size_t row, void *ctx) {
    mv_ctx *c = (mv_ctx *)ctx;
    c->output[row] = matvec_row(c, c->bytes + row * c->row_bytes, c->input);
}

static int check_shape(uint32_t tensor_type, size_t nbytes, size_t rows, size_t columns, mv_ctx *c) {
    if (zqo_block_layout(tensor_type, &c->block_elements, &c->block_bytes)) return -1;
    if (columns % c->block_elements) return -2;
    c->row_bytes = columns / c->block_elements * c->block_bytes;
    if (nbytes != c->row_bytes * rows) return -3;
    c->tensor_type = tensor_type; c->rows = rows; c->columns = columns;
    return 0;
}

/* src/kernel/cpu/ggml_quant.rs:189-219 (matvec). input_len/output_len mirror the Rust slice-length checks. */
int zqo_matvec(uint32_t tensor_type, const uint8_t *bytes, size_t nbytes, size_t rows, size_t columns, const float *input, size_t input_len, float *output, size_t output_len) {
    if (input_len != columns || output_len != rows) return -4;
    mv_ctx c; memset(&c, 0, sizeof(c));
    int rc = check_shape(tensor_type, nbytes, rows, columns, &c);
    if (rc) return rc;
    c.bytes = bytes; c.input = input; c.output = output;
    parallel_rows(rows, matvec_task, &c);
    return 0;
}

/* src/kernel/cpu/ggml_quant.rs:224-233 (matvec_residual) */
int zqo_matvec_residual(uint32_t tensor_type, const uint8_t *bytes, size_t nbytes, size_t rows, size_t columns, const float *input, size_t input_len, float *output, size_t output_len, const float *residual, size_t residual_len) {
    if (residual_len != rows) return -5;
    int rc = zqo_matvec(tensor_type, bytes, nbytes, rows, columns, input, input_len, output, output_len);
    if (rc) return rc;
    for (size_t row = 0; row < rows; ++row) output[row] += residual[row];
    return 0;
}

/* src/kernel/cpu/ggml_quant.rs:114-155 (q4_k_pair_dot_avx2) computes the two dots with the same per-lane
 * operations and order as two q4_k_dot_avx2 calls, so the pair path is restated as two single dots; the
 * reference asserts bit-equality of the two forms (ggml_quant.rs:481-516). */
static void gated_matvec_task(size_t row, void *ctx) {
    mv_ctx *c = (mv_ctx *)ctx;
    float gate_sum = matvec_row(c, c->bytes + row * c->row_bytes, c->input);
    float up_sum = matvec_row(c, c->bytes2 + row * c->row_bytes, c->input);
    /* src/kernel/cpu/ggml_quant.rs:274 */
    c->output[row] = (gate_sum / (1.0f + expf(-gate_sum))) * up_sum;
}

/* src/kernel/cpu/ggml_quant.rs:236-277 (gated_silu_matvec) */
int zqo_gated_silu_matvec(uint32_t tensor_type, const uint8_t *gate, size_t gate_bytes, const uint8_t *up, size_t up_bytes, size_t rows, size_t columns, const float *input, size_t input_len, float *output, size_t output_len) {
    if (input_len != columns || output_len != rows) return -4;
    mv_ctx c; memset(&c, 0, sizeof(c));
    int rc = check_shape(tensor_type, gate_bytes, rows, columns, &c);
    if (rc) return rc;
    if (up_bytes != gate_bytes) return -3;
    c.bytes = gate; c.bytes2 = up; c.input = input; c.output = output;
    parallel_rows(rows, gated_matvec_task, &c);
    return 0;
}

/* One weight row of matmul (src/kernel/cpu/ggml_quant.rs:298-308): each block decoded once, dotted with every token. */
static void matmul_row(const mv_ctx *c, const uint8_t *weight_row, float *sums) {
    float decoded[256];
    for (size_t block = 0; block < c->columns / c->block_elements; ++block) {
        zqo_decode_block(c->tensor_type, weight_row + block * c->block_bytes, c->block_bytes, decoded, c->block_elements);
        size_t column = block * c->block_elements;
        for (size_t token = 0; token < c->input_rows; ++token)
            sums[token] += dot_f32_avx2(decoded, c->input + token * c->columns + column, c->block_elements);
    }
}

static void matmul_task(size_t row, void *ctx) {
    mv_ctx *c = (mv_ctx *)ctx;
    matmul_row(c, c->bytes + row * c->row_bytes, c->scratch + row * c->input_rows);
}

/* src/kernel/cpu/ggml_quant.rs:280-315 (matmul): row-major [rows, input_rows] temp, then transpose to Y[token*rows+row]. */
int zqo_matmul(uint32_t tensor_type, const uint8_t *bytes, size_t nbytes, size_t rows, size_t columns, size_t input_rows, const float *input, size_t input_len, float *output, size_t output_len) {
    if (input_rows == 0 || input_len != input_rows * columns || output_len != input_rows * rows) return -4;
    mv_ctx c; memset(&c, 0, sizeof(c));
    int rc = check_shape(tensor_type, nbytes, rows, columns, &c);
    if (rc) return rc;
    c.bytes = bytes; c.input = input; c.input_rows = input_rows;
    c.scratch = (float *)calloc(rows * input_rows, sizeof(float));
    if (!c.scratch) return -6;
    parallel_rows(rows, matmul_task, &c);
    for (size_t row = 0; row < rows; ++row)
        for (size_t token = 0; token < input_rows; ++token) output[token * rows + row] = c.scratch[row * input_rows + token];
    free(c.scratch);
    return 0;
}

static void gated_matmul_task(size_t row, void *ctx) {
    mv_ctx *c = (mv_ctx *)ctx;
    float gate_decoded[256], up_decoded[256];
    float *gate_sums = c->scratch + row * c->input_rows, *up_sums = c->scratch2 + row * c->input_rows;
    const uint8_t *gate_row = c->bytes + row * c->row_bytes, *up_row = c->bytes2 + row * c->row_bytes;
    for (size_t block = 0; block < c->columns / c->block_elements; ++block) {
        zqo_decode_block(c->tensor_type, gate_row + block * c->block_bytes, c->block_bytes, gate_decoded, c->block_elements);
        zqo_decode_block(c->tensor_type, up_row + block * c->block_bytes, c->block_bytes, up_decoded, c->block_elements);
        size_t column = block * c->block_elements;
        for (size_t token = 0; token < c->input_rows; ++token) {
            const float *x = c->input + token * c->columns + column;
            gate_sums[token] += dot_f32_avx2(gate_decoded, x, c->block_elements);
            up_sums[token] += dot_f32_avx2(up_decoded, x, c->block_elements);
        }
    }
    for (size_t token = 0; token < c->input_rows; ++token) {
        float gate = gate_sums[token];
        gate_sums[token] = (gate / (1.0f + expf(-gate))) * up_sums[token]; /* ggml_quant.rs:352 */
    }
}

/* src/kernel/cpu/ggml_quant.rs:319-362 (gated_silu_matmul) */
int zqo_gated_silu_matmul(uint32_t tensor_type, const uint8_t *gate, size_t gate_bytes, const uint8_t *up, size_t up_bytes, size_t rows, size_t columns, size_t input_rows, const float *input, size_t input_len, float *output, size_t output_len) {
    if (input_rows == 0 || input_len != input_rows * columns || output_len != input_rows * rows) return -4;
    mv_ctx c; memset(&c, 0, sizeof(c));
    int rc = check_shape(tensor_type, gate_bytes, rows, columns, &c);
    if (rc) return rc;
    if (up_bytes != gate_bytes) return -3;
    c.bytes = gate; c.bytes2 = up; c.input = input; c.input_rows = input_rows;
    c.scratch = (float *)calloc(rows * input_rows, sizeof(float));
    c.scratch2 = (float *)calloc(rows * input_rows, sizeof(float));
    if (!c.scratch || !c.scratch2) { free(c.scratch); free(c.scratch2); return -6; }
    parallel_rows(rows, gated_matmul_task, &c);
    for (size_t row = 0; row < rows; ++row)
        for (size_t token = 0; token < input_rows; ++token) output[token * rows + row] = c.scratch[row * input_rows + token];
    free(c.scratch); free(c.scratch2);
    return 0;
}

/* CpuContext::linear dispatch (src/backend/cpu/context.rs:184-198): one token -> matvec, several -> matmul. */
int zqo_linear(uint32_t tensor_type, const uint8_t *bytes, size_t nbytes, size_t rows, size_t columns, size_t input_rows, const float *input, float *output) {
    if (input_rows == 1) return zqo_matvec(tensor_type, bytes, nbytes, rows, columns, input, columns, output, rows);
    return zqo_matmul(tensor_type, bytes, nbytes, rows, columns, input_rows, input, input_rows * columns, output, input_rows * rows);
}

/* ------------------------------------------------------------------ SiLU */

void zqo_silu_mul(const float *gate, const float *up, float *out, size_t len);

/* CpuContext::gated_linear with Activation::Silu (src/backend/cpu/context.rs:450-469): Q4_K pairs take the fused
 * kernels; every other type runs two linears followed by silu_mul (gated_activation). */
int zqo_gated_linear(uint32_t tensor_type, const uint8_t *gate, size_t gate_bytes, const uint8_t *up, size_t up_bytes, size_t rows, size_t columns, size_t input_rows, const float *input, float *output) {
    if (tensor_type == 12) {
        if (input_rows == 1) return zqo_gated_silu_matvec(12, gate, gate_bytes, up, up_bytes, rows, columns, input, columns, output, rows);
        return zqo_gated_silu_matmul(12, gate, gate_bytes, up, up_bytes, rows, columns, input_rows, input, input_rows * columns, output, input_rows * rows);
    }
    float *g = (float *)malloc(input_rows * rows * sizeof(float));
    float *u = (float *)malloc(input_rows * rows * sizeof(float));
    int rc = zqo_linear(tensor_type, gate, gate_bytes, rows, columns, input_rows, input, g);
    if (!rc) rc = zqo_linear(tensor_type, up, up_bytes, rows, columns, input_rows, input, u);
    if (!rc) zqo_silu_mul(g, u, output, input_rows * rows);
    free(g); free(u);
    return rc;
}

/* src/kernel/cpu/silu.rs:8-21 (silu_mul): full 8-lane chunks use g*sigmoid(g)*u with
 * sigmoid from src/kernel/cpu/silu.rs:116-122; the tail uses g/(1+exp(-g))*u.  wide's polynomial
 * exp is replaced by libm expf. */
void zqo_silu_mul(const float *gate, const float *up, float *out, size_t len) {
    size_t full = len / 8 * 8;
    for (size_t i = 0; i < full; ++i) {
        float g = gate[i];
        float e = expf(-fabsf(g));
        float denominator = 1.0f + e;
        float s = signbit(g) ? e / denominator : 1.0f / denominator;
        if (isnan(g)) s = g;
        volatile float gs = g * s;
        out[i] = gs * up[i];
    }
    for (size_t i = full; i < len; ++i) {
        volatile float silu = gate[i] / (1.0f + expf(-gate[i]));
        out[i] = silu * up[i];
    }
}

/* ------------------------------------------------------------------ MoE */

/* src/kernel/cpu/moe.rs:38-55 (router_logits): eight-lane accumulate (separate multiply and add), then a
 * lane reduction.  wide's reduce_add order is not visible from the reference tree; pairwise order is used. */
void zqo_router_logits(const float *input, const float *weight, size_t hidden, size_t num_experts, float *logits) {
    for (size_t e = 0; e < num_experts; ++e) {
        const float *w = weight + e * hidden;
        __m256 acc = _mm256_setzero_ps();
        for (size_t i = 0; i + 8 <= hidden; i += 8) acc = _mm256_add_ps(acc, _mm256_mul_ps(_mm256_loadu_ps(input + i), _mm256_loadu_ps(w + i)));
        logits[e] = horizontal_sum_avx2(acc);
    }
}

typedef struct { float logit; uint32_t expert; } ranked_t;

/* Ordering of src/moe/routing.rs:31: logit descending by total_cmp, then expert id ascending. */
static int32_t total_key(float value) {
    int32_t bits; memcpy(&bits, &value, 4);
    return bits ^ (int32_t)(((uint32_t)(bits >> 31)) >> 1);
}
static int ranked_cmp(const void *a, const void *b) {
    const ranked_t *l = (const ranked_t *)a, *r = (const ranked_t *)b;
    int32_t lk = total_key(l->logit), rk = total_key(r->logit);
    if (lk != rk) return rk > lk ? 1 : -1;
    return l->expert < r->expert ? -1 : (l->expert > r->expert ? 1 : 0);
}

/* src/moe/routing.rs:25-39 (route_softmax_logits).  The ordering is total, so select_nth + sort equals a full sort. */
int zqo_route_softmax_logits(const float *logits, size_t num_experts, size_t top_k, float scaling_factor, int normalize_selected, uint32_t *experts, float *weights) {
    if (num_experts == 0 || top_k == 0 || top_k > num_experts || !isfinite(scaling_factor)) return -1;
    ranked_t *ranked = (ranked_t *)malloc(num_experts * sizeof(ranked_t));
    for (size_t e = 0; e < num_experts; ++e) { ranked[e].logit = logits[e]; ranked[e].expert = (uint32_t)e; }
    qsort(ranked, num_experts, sizeof(ranked_t), ranked_cmp);
    float max_logit = ranked[0].logit;
    float denominator = 0.0f;
    if (normalize_selected) for (size_t k = 0; k < top_k; ++k) denominator += expf(ranked[k].logit - max_logit);
    else for (size_t e = 0; e < num_experts; ++e) denominator += expf(logits[e] - max_logit);
    if (!isfinite(denominator) || denominator <= 0.0f) { free(ranked); return -2; }
    for (size_t k = 0; k < top_k; ++k) {
        experts[k] = ranked[k].expert;
        volatile float p = expf(ranked[k].logit - max_logit) / denominator;
        weights[k] = p * scaling_factor;
    }
    free(ranked);
    return 0;
}

/* src/kernel/cpu/moe.rs:61-63 (route_softmax) over every token row (src/backend/cpu/moe.rs:36-64). */
int zqo_moe_route_softmax(const float *input, size_t rows, size_t hidden, const float *router, size_t num_experts, size_t top_k, float scaling_factor, int normalize_selected, uint32_t *expert_ids, float *weights) {
    if (hidden % 8) return -3;
    float *logits = (float *)malloc(num_experts * sizeof(float));
    for (size_t row = 0; row < rows; ++row) {
        zqo_router_logits(input + row * hidden, router, hidden, num_experts, logits);
        int rc = zqo_route_softmax_logits(logits, num_experts, top_k, scaling_factor, normalize_selected, expert_ids + row * top_k, weights + row * top_k);
        if (rc) { free(logits); return rc; }
    }
    free(logits);
    return 0;
}

/* src/moe/routing.rs:136-156 (group_routing): token-major stable grouping.  Output is CSR: offsets[E+1],
 * tokens[routes], route_weights[routes].  Returns -1 on an out-of-range expert id. */
int zqo_group_routing(const uint32_t *expert_ids, const float *weights, size_t routes, size_t top_k, size_t expert_count, uint32_t *offsets, uint32_t *tokens, float *route_weights) {
    if (top_k == 0 || routes % top_k) return -2;
    memset(offsets, 0, (expert_count + 1) * sizeof(uint32_t));
    for (size_t r = 0; r < routes; ++r) {
        if (expert_ids[r] >= expert_count) return -1;
        offsets[expert_ids[r] + 1] += 1;
    }
    for (size_t e = 0; e < expert_count; ++e) offsets[e + 1] += offsets[e];
    uint32_t *cursor = (uint32_t *)malloc(expert_count * sizeof(uint32_t));
    memcpy(cursor, offsets, expert_count * sizeof(uint32_t));
    for (size_t r = 0; r < routes; ++r) {
        uint32_t slot = cursor[expert_ids[r]]++;
        tokens[slot] = (uint32_t)(r / top_k);
        route_weights[slot] = weights[r];
    }
    free(cursor);
    return 0;
}

typedef struct {
    uint32_t tensor_type;
    const uint8_t *bytes;
    size_t nbytes, rows, columns;
} zqo_matrix;

/* src/kernel/cpu/moe.rs:129-138 (gguf_matmul_batch): one matvec per token row. */
static int gguf_matmul_batch(const zqo_matrix *w, const float *input, size_t input_rows, float *output) {
    for (size_t t = 0; t < input_rows; ++t) {
        int rc = zqo_matvec(w->tensor_type, w->bytes, w->nbytes, w->rows, w->columns, input + t * w->columns, w->columns, output + t * w->rows, w->rows);
        if (rc) return rc;
    }
    return 0;
}

/* src/kernel/cpu/moe.rs:122-127 (gguf_expert_batch) with Activation::Silu (src/kernel/cpu/moe.rs:74-77). */
int zqo_gguf_expert_batch(const zqo_matrix *gate, const zqo_matrix *up, const zqo_matrix *down, const float *input, size_t input_rows, float *output) {
    if (gate->columns != up->columns || gate->rows != up->rows || down->columns != gate->rows) return -7;
    size_t inter = gate->rows;
    float *g = (float *)malloc(input_rows * inter * sizeof(float));
    float *u = (float *)malloc(input_rows * inter * sizeof(float));
    float *a = (float *)malloc(input_rows * inter * sizeof(float));
    int rc = gguf_matmul_batch(gate, input, input_rows, g);
    if (!rc) rc = gguf_matmul_batch(up, input, input_rows, u);
    if (!rc) {
        zqo_silu_mul(g, u, a, input_rows * inter);
        rc = gguf_matmul_batch(down, a, input_rows, output);
    }
    free(g); free(u); free(a);
    return rc;
}

/* Routed MoE forward on the CPU path:
 *   routing  src/moe/prefill.rs:128-205 -> moe_route_rows -> grouped (src/moe/routing.rs:126-156)
 *   experts  src/moe/routing.rs:180-213 (execute_routed_experts): gather rows, expert batch, weighted scatter
 *   scatter  src/backend/cpu/moe.rs:107-141: per target row, contributions in ascending active-expert order,
 *            out[row] += y * weight
 *   shared   src/moe/topk_moe.rs:84-104 (gated_linear -> linear(down)), added to the routed sum
 * output[rows, hidden] = routed (+ shared) (+ residual).  expert arrays hold num_experts entries each. */
int zqo_moe_forward(const zqo_matrix *gates, const zqo_matrix *ups, const zqo_matrix *downs, size_t num_experts,
                    const zqo_matrix *shared_gate, const zqo_matrix *shared_up, const zqo_matrix *shared_down,
                    const float *input, size_t rows, size_t hidden, const uint32_t *expert_ids, const float *weights, size_t top_k,
                    const float *residual, float *output) {
    size_t routes = rows * top_k;
    uint32_t *offsets = (uint32_t *)malloc((num_experts + 1) * sizeof(uint32_t));
    uint32_t *tokens = (uint32_t *)malloc(routes * sizeof(uint32_t));
    float *rweights = (float *)malloc(routes * sizeof(float));
    int rc = zqo_group_routing(expert_ids, weights, routes, top_k, num_experts, offsets, tokens, rweights);
    if (rc) { free(offsets); free(tokens); free(rweights); return rc; }
    memset(output, 0, rows * hidden * sizeof(float));
    for (size_t e = 0; e < num_experts && !rc; ++e) {
        size_t count = offsets[e + 1] - offsets[e];
        if (!count) continue;
        float *gathered = (float *)malloc(count * hidden * sizeof(float));
        float *computed = (float *)malloc(count * hidden * sizeof(float));
        for (size_t i = 0; i < count; ++i) memcpy(gathered + i * hidden, input + (size_t)tokens[offsets[e] + i] * hidden, hidden * sizeof(float));
        rc = zqo_gguf_expert_batch(&gates[e], &ups[e], &downs[e], gathered, count, computed);
        for (size_t i = 0; i < count && !rc; ++i) {
            float *target = output + (size_t)tokens[offsets[e] + i] * hidden;
            float w = rweights[offsets[e] + i];
            for (size_t c = 0; c < hidden; ++c) {
                volatile float product = computed[i * hidden + c] * w;
                target[c] += product;
            }
        }
        free(gathered); free(computed);
    }
    if (!rc && shared_gate) {
        size_t inter = shared_gate->rows;
        float *activated = (float *)malloc(rows * inter * sizeof(float));
        float *shared = (float *)malloc(rows * hidden * sizeof(float));
        rc = zqo_gated_linear(shared_gate->tensor_type, shared_gate->bytes, shared_gate->nbytes, shared_up->bytes, shared_up->nbytes, inter, hidden, rows, input, activated);
        if (!rc) rc = zqo_linear(shared_down->tensor_type, shared_down->bytes, shared_down->nbytes, shared_down->rows, shared_down->columns, rows, activated, shared);
        for (size_t i = 0; i < rows * hidden && !rc; ++i) output[i] += shared[i];
        free(activated); free(shared);
    }
    if (!rc && residual) for (size_t i = 0; i < rows * hidden; ++i) output[i] += residual[i];
    free(offsets); free(tokens); free(rweights);
    return rc;
}

/* ------------------------------------------------------------------ RoPE on projection outputs */

/* attention::rope::apply_f32 (src/attention/rope.rs:120-165), the arithmetic behind Backend::rope / rope_prefix /
 * rope_prefix_qk (src/backend/mod.rs:545-583; CPU: src/backend/cpu/context.rs:590-625, whose 8-lane fast path keeps the
 * same mul / sub / add order).  layout 0 = SplitHalf (pair p = elements p and half + p), 1 = Interleaved (2p, 2p + 1);
 * placement 0 = Prefix (the head's first rotary_dim elements), 1 = Suffix (its last).  In place.
 * Returns 0, or 1 for the parameter errors the reference reports. */
int zqo_rope(float *data, size_t rows, size_t columns, size_t head_count, size_t rotary_dim, size_t position, const float *cos_table, const float *sin_table, size_t table_len, int layout, int placement) {
    if (head_count == 0 || rotary_dim == 0 || rotary_dim % 2 || columns % head_count) return 1;
    const size_t head_dim = columns / head_count;
    if (rotary_dim > head_dim) return 1;
    const size_t half = rotary_dim / 2;
    if ((position + rows) * half > table_len) return 1;
    float *source = (float *)malloc(rotary_dim * sizeof(float));
    for (size_t row = 0; row < rows; ++row) {
        const float *cos_row = cos_table + (position + row) * half, *sin_row = sin_table + (position + row) * half;
        for (size_t head = 0; head < head_count; ++head) {
            const size_t head_start = row * columns + head * head_dim;
            const size_t start = placement == 0 ? head_start : head_start + head_dim - rotary_dim;
            memcpy(source, data + start, rotary_dim * sizeof(float));
            for (size_t pair = 0; pair < half; ++pair) {
                const size_t ri = layout == 0 ? pair : pair * 2, ii = layout == 0 ? half + pair : pair * 2 + 1;
                const float real = source[ri], imaginary = source[ii];
                /* separate roundings, as the reference's scalar code (this file is built with -ffp-contract=off) */
                volatile float a = real * cos_row[pair], b = imaginary * sin_row[pair];
                volatile float c = imaginary * cos_row[pair], d = real * sin_row[pair];
                data[start + ri] = a - b;
                data[start + ii] = c + d;
            }
        }
    }
    free(source);
    return 0;
}

/* ------------------------------------------------------------------ bias-corrected routers */

/* route_bias_corrected_logits (src/moe/routing.rs:45-67) behind route_sigmoid_bias_logits (:74, kind 1) and
 * route_sqrt_softplus_bias_logits (:79, kind 2; sqrt_softplus_score :70-73): every expert has a raw score; raw + bias ranks
 * the experts (descending, ties to the lower id); the top_k raw scores are normalised to sum 1 and scaled.
 * Returns 0, or 1 for the parameter / mass errors the reference reports. */
static float raw_router_score(float logit, int kind) {
    if (kind == 1) return 1.0f / (1.0f + expf(-logit));
    const float softplus = logit > 0.0f ? logit + log1pf(expf(-logit)) : log1pf(expf(logit));
    return sqrtf(softplus);
}

int zqo_route_bias_corrected_logits(const float *logits, const float *bias, size_t num_experts, size_t top_k, float scaling_factor, int kind, uint32_t *experts, float *weights) {
    if (num_experts == 0 || top_k == 0 || top_k > num_experts || !isfinite(scaling_factor) || (kind != 1 && kind != 2)) return 1;
    float *raw = (float *)malloc(num_experts * sizeof(float));
    float *corrected = (float *)malloc(num_experts * sizeof(float));
    char *taken = (char *)calloc(num_experts, 1);
    for (size_t e = 0; e < num_experts; ++e) {
        raw[e] = raw_router_score(logits[e], kind);
        corrected[e] = raw[e] + bias[e];
    }
    float sum_raw = 0.0f;
    for (size_t slot = 0; slot < top_k; ++slot) {  /* repeated arg-max = a stable descending sort's first top_k entries */
        size_t best = num_experts;
        for (size_t e = 0; e < num_experts; ++e) {
            if (taken[e]) continue;
            if (best == num_experts || corrected[e] > corrected[best]) best = e;
        }
        taken[best] = 1;
        experts[slot] = (uint32_t)best;
        sum_raw += raw[best];
    }
    int rc = 0;
    if (!isfinite(sum_raw) || sum_raw <= 0.0f) rc = 1;
    for (size_t slot = 0; slot < top_k && !rc; ++slot) weights[slot] = raw[experts[slot]] / sum_raw * scaling_factor;
    free(raw); free(corrected); free(taken);
    return rc;
}
