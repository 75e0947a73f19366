/*
 * CPU oracle for the gpurs dense matrix-multiply path.  TEST INFRASTRUCTURE ONLY.
 *
 * This file restates, in plain C, the host-side arithmetic that the reference (1jmdev/gpurs, Rust)
 * uses to check its tensor-core GEMM examples, plus the storage-format conversions those checks
 * depend on.  It is linked or loaded only by the test-suite, by the smoke check and by the
 * "cpu baseline" / "reference" legs of the benchmark; nothing in the shipped library calls it.
 *
 * Reference locations restated here (paths are relative to the gpurs source tree):
 *   examples/matrix_benchmark.rs:5-14     deterministic example inputs
 *   examples/matrix_benchmark.rs:36-51    fp64 check loop  C[r,c] = sum_k A[r,k] * B[c,k]
 *   crates/gpurs/src/gpu/float16.rs:19-64 binary16  from_f32 / to_f32
 *   crates/gpurs/src/gpu/float16.rs:71-83 bfloat16  from_f32 / to_f32
 *   crates/gpurs/src/gpu/float8.rs:20-74  E4M3      from_f32 / to_f32
 *   crates/gpurs/src/gpu/float8.rs:233-262 TF32     from_f32
 *   crates/gpurs/src/gpu/tensor/warp/instruction.rs:14-17  int8 products accumulate in wrapping int32
 *
 * Parity status: the reference holds no golden vectors and cannot be compiled where this oracle is
 * developed (it needs a nightly Rust toolchain), so the oracle is pinned (a) against independent
 * implementations of the same formats (numpy / torch) through the fixtures under tests/golden and
 * (b) through the exactness property of the reference's own example inputs: every partial sum of
 * those inputs is representable in fp32, so any correct fp32-accumulating GEMM must reproduce the
 * fp64 loop bit for bit.  For the int8, FP8 block-scaled, fp32 and 2:4-sparse variants the
 * reference ships no kernel and no check at all: for those, parity is unpinned and this oracle is
 * the definition.
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#define API __attribute__((visibility("default")))

/* ---------------------------------------------------------------------------------------------
 * Storage formats
 * ------------------------------------------------------------------------------------------- */

static inline uint32_t f32_bits(float v) { uint32_t b; memcpy(&b, &v, 4); return b; }
static inline float bits_f32(uint32_t b) { float v; memcpy(&v, &b, 4); return v; }

/* binary16, round to nearest even, overflow to infinity (float16.rs:19-47). */
API uint16_t gpurs_oracle_f16_from_f32(float value) {
    uint32_t bits = f32_bits(value);
    uint32_t sign = (bits >> 16) & 0x8000u;
    uint32_t mantissa = bits & 0x7fffffu;
    int32_t exponent = (int32_t)((bits >> 23) & 0xff) - 127 + 15;
    if (exponent == 0xff - 127 + 15) {
        uint32_t quiet = mantissa == 0 ? 0 : 0x200u;
        return (uint16_t)(sign | 0x7c00u | quiet);
    }
    if (exponent >= 0x1f) return (uint16_t)(sign | 0x7c00u);
    if (exponent < -10) return (uint16_t)sign;
    uint32_t shift;
    if (exponent > 0) {
        shift = 13;
    } else {
        mantissa |= 0x800000u;
        shift = (uint32_t)(14 - exponent);
    }
    uint32_t kept_exponent = exponent > 0 ? (uint32_t)exponent : 0u;
    uint32_t truncated = (kept_exponent << 10) | (mantissa >> shift);
    uint32_t remainder = mantissa & ((1u << shift) - 1u);
    uint32_t midpoint = 1u << (shift - 1);
    uint32_t round = remainder > midpoint || (remainder == midpoint && (truncated & 1u));
    return (uint16_t)(sign | (truncated + round));
}

/* float16.rs:49-64 */
API float gpurs_oracle_f16_to_f32(uint16_t half) {
    uint32_t bits = half;
    uint32_t sign = (bits & 0x8000u) << 16;
    uint32_t exponent = (bits >> 10) & 0x1f;
    uint32_t mantissa = bits & 0x3ffu;
    if (exponent == 0 && mantissa == 0) return bits_f32(sign);
    if (exponent == 0) {
        uint32_t shift = (uint32_t)__builtin_clz(mantissa) - 21u;
        return bits_f32(sign | ((113u - shift) << 23) | (((mantissa << shift) & 0x3ffu) << 13));
    }
    if (exponent == 0x1f) return bits_f32(sign | 0x7f800000u | (mantissa << 13));
    return bits_f32(sign | ((exponent + 112u) << 23) | (mantissa << 13));
}

/* bfloat16, round to nearest even, NaN quieted (float16.rs:71-83). */
API uint16_t gpurs_oracle_bf16_from_f32(float value) {
    uint32_t bits = f32_bits(value);
    if (value != value) return (uint16_t)((bits >> 16) | 0x40u);
    return (uint16_t)((bits + 0x7fffu + ((bits >> 16) & 1u)) >> 16);
}

API float gpurs_oracle_bf16_to_f32(uint16_t v) { return bits_f32((uint32_t)v << 16); }

/* float8.rs:54-73 */
API float gpurs_oracle_e4m3_to_f32(uint8_t v) {
    uint32_t magnitude = v & 0x7fu;
    uint32_t sign = ((uint32_t)v & 0x80u) << 24;
    if (magnitude == 127) return bits_f32(sign | 0x7fc00000u);
    uint32_t exponent = magnitude >> 3;
    uint32_t fraction = magnitude & 7u;
    float value = exponent == 0 ? (float)fraction * bits_f32(118u << 23)
                                : bits_f32(((exponent + 120u) << 23) | (fraction << 20));
    return bits_f32(sign | f32_bits(value));
}

/* E4M3: nearest even, finite saturation at 448, NaN -> 0x7f (float8.rs:20-52).  The reference
 * finds the largest code not above |value| by bisection and then rounds on the midpoint. */
API uint8_t gpurs_oracle_e4m3_from_f32(float value) {
    uint8_t sign = (uint8_t)((f32_bits(value) >> 24) & 0x80u);
    if (value != value) return 127;
    float magnitude = fabsf(value);
    uint8_t low = 0, high = 126;
    while (low < high) {
        uint8_t midpoint = (uint8_t)(low + (high - low + 1) / 2);
        if (gpurs_oracle_e4m3_to_f32(midpoint) <= magnitude) low = midpoint;
        else high = (uint8_t)(midpoint - 1);
    }
    if (low < 126) {
        float lo = gpurs_oracle_e4m3_to_f32(low), hi = gpurs_oracle_e4m3_to_f32((uint8_t)(low + 1));
        float midpoint = (float)(((double)lo + (double)hi) * 0.5);
        if (magnitude > midpoint || (magnitude == midpoint && (low & 1))) low++;
    }
    return (uint8_t)(sign | low);
}

/* TF32: nearest, ties away from zero; infinities stay, NaN quieted (float8.rs:241-247). */
API uint32_t gpurs_oracle_tf32_from_f32(float value) {
    uint32_t bits = f32_bits(value);
    if ((bits & 0x7f800000u) == 0x7f800000u) return bits | (value != value ? 0x400000u : 0u);
    return (bits + 0x1000u) & ~0x1fffu;
}

/* Vector forms used by the tests and by the input generators. */
API void gpurs_oracle_f16_from_f32_n(const float *s, uint16_t *d, size_t n) { for (size_t i = 0; i < n; i++) d[i] = gpurs_oracle_f16_from_f32(s[i]); }
API void gpurs_oracle_f16_to_f32_n(const uint16_t *s, float *d, size_t n) { for (size_t i = 0; i < n; i++) d[i] = gpurs_oracle_f16_to_f32(s[i]); }
API void gpurs_oracle_bf16_from_f32_n(const float *s, uint16_t *d, size_t n) { for (size_t i = 0; i < n; i++) d[i] = gpurs_oracle_bf16_from_f32(s[i]); }
API void gpurs_oracle_bf16_to_f32_n(const uint16_t *s, float *d, size_t n) { for (size_t i = 0; i < n; i++) d[i] = gpurs_oracle_bf16_to_f32(s[i]); }
API void gpurs_oracle_e4m3_from_f32_n(const float *s, uint8_t *d, size_t n) { for (size_t i = 0; i < n; i++) d[i] = gpurs_oracle_e4m3_from_f32(s[i]); }
API void gpurs_oracle_e4m3_to_f32_n(const uint8_t *s, float *d, size_t n) { for (size_t i = 0; i < n; i++) d[i] = gpurs_oracle_e4m3_to_f32(s[i]); }
API void gpurs_oracle_tf32_from_f32_n(const float *s, uint32_t *d, size_t n) { for (size_t i = 0; i < n; i++) d[i] = gpurs_oracle_tf32_from_f32(s[i]); }

/* ---------------------------------------------------------------------------------------------
 * Inputs
 * ------------------------------------------------------------------------------------------- */

/* Element formats understood by the generators and the GEMM loops. */
enum { FMT_F16 = 0, FMT_BF16 = 1, FMT_F32 = 2, FMT_I8 = 3, FMT_E4M3 = 4 };

/* The reference example's inputs (matrix_benchmark.rs:5-14): left[i] = (i*13 mod 31)/16 - 1,
 * right[i] = (i*7 mod 29)/16 - 1, stored as 16-bit floats.  `format` selects binary16 or bfloat16;
 * the values are multiples of 1/16 in [-1, 1) and exact in both. */
API void gpurs_oracle_example_inputs(int format, size_t count, uint16_t *left, uint16_t *right) {
#pragma omp parallel for schedule(static)
    for (size_t i = 0; i < count; i++) {
        float l = (float)(i * 13 % 31) / 16.0f - 1.0f;
        float r = (float)(i * 7 % 29) / 16.0f - 1.0f;
        left[i] = format == FMT_F16 ? gpurs_oracle_f16_from_f32(l) : gpurs_oracle_bf16_from_f32(l);
        right[i] = format == FMT_F16 ? gpurs_oracle_f16_from_f32(r) : gpurs_oracle_bf16_from_f32(r);
    }
}

/* Counter-based generator: one 64-bit word per (seed, index), splitmix64 finaliser. */
static inline uint64_t word(uint64_t seed, uint64_t index) {
    uint64_t z = (seed + 1) * 0x9E3779B97F4A7C15ull + index * 0xD1B54A32D192ED03ull;
    z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
    z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
    return z ^ (z >> 31);
}

/* Uniform on [-1, 1) with 24 random bits. */
static inline float uniform_pm1(uint64_t seed, uint64_t index) {
    return (float)(word(seed, index) >> 40) * (2.0f / 16777216.0f) - 1.0f;
}

/* Standard normal by Box-Muller on the two 24-bit halves of one word. */
static inline float normal(uint64_t seed, uint64_t index) {
    uint64_t z = word(seed, index);
    double u1 = ((double)(z >> 40) + 1.0) / 16777216.0;
    double u2 = (double)((z >> 16) & 0xffffffu) / 16777216.0;
    return (float)(sqrt(-2.0 * log(u1)) * cos(6.283185307179586476925 * u2));
}

API void gpurs_oracle_fill_uniform_f32(float *out, size_t count, uint64_t seed) {
#pragma omp parallel for schedule(static)
    for (size_t i = 0; i < count; i++) out[i] = uniform_pm1(seed, i);
}

API void gpurs_oracle_fill_normal_f32(float *out, size_t count, uint64_t seed) {
#pragma omp parallel for schedule(static)
    for (size_t i = 0; i < count; i++) out[i] = normal(seed, i);
}

/* N(0,1) rounded to binary16 or bfloat16 with the reference's host conversion. */
API void gpurs_oracle_fill_normal_16(int format, uint16_t *out, size_t count, uint64_t seed) {
#pragma omp parallel for schedule(static)
    for (size_t i = 0; i < count; i++) {
        float v = normal(seed, i);
        out[i] = format == FMT_F16 ? gpurs_oracle_f16_from_f32(v) : gpurs_oracle_bf16_from_f32(v);
    }
}

/* Uniform integers in [-128, 127]. */
API void gpurs_oracle_fill_int8(int8_t *out, size_t count, uint64_t seed) {
#pragma omp parallel for schedule(static)
    for (size_t i = 0; i < count; i++) out[i] = (int8_t)(word(seed, i) >> 56);
}

/* A rows x columns bfloat16 matrix with exactly two non-zeros in every aligned group of four
 * along the columns: the pair of positions is one of the six possible, chosen from the seed; the
 * values are N(0,1) (a value that rounds to zero is replaced by 1 so the pattern stays exact). */
API void gpurs_oracle_fill_sparse24_bf16(uint16_t *out, size_t rows, size_t columns, uint64_t seed) {
    static const uint8_t pairs[6][2] = {{0, 1}, {0, 2}, {0, 3}, {1, 2}, {1, 3}, {2, 3}};
    size_t groups = rows * (columns / 4);
#pragma omp parallel for schedule(static)
    for (size_t g = 0; g < groups; g++) {
        uint32_t choice = (uint32_t)((word(seed ^ 0x5eedull, g) >> 32) % 6u);
        uint16_t *group = out + g * 4;
        group[0] = group[1] = group[2] = group[3] = 0;
        for (int j = 0; j < 2; j++) {
            size_t position = pairs[choice][j];
            uint16_t v = gpurs_oracle_bf16_from_f32(normal(seed, g * 4 + position));
            if ((v & 0x7fffu) == 0) v = 0x3f80u;
            group[position] = v;
        }
    }
}

/* ---------------------------------------------------------------------------------------------
 * FP8 block quantisation and 2:4 compression (host restatements of the device helpers)
 * ------------------------------------------------------------------------------------------- */

/* Quantise a rows x depth fp32 matrix to E4M3 with one fp32 scale per block of block_rows x 128
 * elements (block_rows = 1 for the left operand, 128 for the right one).  scale = absmax / 448, or
 * 1 for an all-zero block; q = E4M3(x / scale).  Scales are stored row-major as
 * [ceil(rows / block_rows)][ceil(depth / 128)]. */
API void gpurs_oracle_quantize_e4m3(const float *source, size_t rows, size_t depth, size_t block_rows,
                                    uint8_t *quantized, float *scales) {
    size_t row_blocks = (rows + block_rows - 1) / block_rows;
    size_t depth_blocks = (depth + 127) / 128;
#pragma omp parallel for schedule(static) collapse(2)
    for (size_t rb = 0; rb < row_blocks; rb++) {
        for (size_t kb = 0; kb < depth_blocks; kb++) {
            size_t r0 = rb * block_rows, r1 = r0 + block_rows < rows ? r0 + block_rows : rows;
            size_t k0 = kb * 128, k1 = k0 + 128 < depth ? k0 + 128 : depth;
            float absmax = 0.0f;
            for (size_t r = r0; r < r1; r++)
                for (size_t k = k0; k < k1; k++) absmax = fmaxf(absmax, fabsf(source[r * depth + k]));
            float scale = absmax > 0.0f ? absmax / 448.0f : 1.0f;
            scales[rb * depth_blocks + kb] = scale;
            for (size_t r = r0; r < r1; r++)
                for (size_t k = k0; k < k1; k++)
                    quantized[r * depth + k] = gpurs_oracle_e4m3_from_f32(source[r * depth + k] / scale);
        }
    }
}

/* Compress a 2:4-sparse 16-bit matrix: keep the two non-zeros of every group of four (a group with
 * fewer than two non-zeros keeps zeros in the lowest free positions, so the kept positions are
 * always ascending) and record their positions.  values: rows x depth/2; indices: one byte per
 * group, low two bits = first kept position, next two bits = second kept position.  Returns the
 * number of groups that held more than two non-zeros (0 for a valid 2:4 matrix). */
API size_t gpurs_oracle_compress_24(const uint16_t *dense, size_t rows, size_t depth, uint16_t *values,
                                    uint8_t *indices) {
    size_t groups_per_row = depth / 4, violations = 0;
#pragma omp parallel for schedule(static) reduction(+ : violations)
    for (size_t r = 0; r < rows; r++) {
        for (size_t g = 0; g < groups_per_row; g++) {
            const uint16_t *group = dense + r * depth + g * 4;
            int kept[2], count = 0, nonzero = 0;
            for (int p = 0; p < 4; p++) nonzero += (group[p] & 0x7fffu) != 0;
            if (nonzero > 2) violations++;
            for (int p = 0; p < 4 && count < 2; p++)
                if ((group[p] & 0x7fffu) != 0) kept[count++] = p;
            /* pad with zero positions, keeping the pair ascending and distinct */
            for (int p = 0; p < 4 && count < 2; p++) {
                int used = 0;
                for (int j = 0; j < count; j++) used |= kept[j] == p;
                if (!used && (group[p] & 0x7fffu) == 0) kept[count++] = p;
            }
            if (kept[0] > kept[1]) { int t = kept[0]; kept[0] = kept[1]; kept[1] = t; }
            values[r * (depth / 2) + g * 2 + 0] = group[kept[0]];
            values[r * (depth / 2) + g * 2 + 1] = group[kept[1]];
            indices[r * groups_per_row + g] = (uint8_t)(kept[0] | (kept[1] << 2));
        }
    }
    return violations;
}

/* ---------------------------------------------------------------------------------------------
 * The check loop: C[r,c] = sum_k A[r,k] * B[c,k], both operands depth-major (matrix_benchmark.rs:40-45)
 * ------------------------------------------------------------------------------------------- */

static inline double element(int format, const void *base, size_t index) {
    switch (format) {
    case FMT_F16: return (double)gpurs_oracle_f16_to_f32(((const uint16_t *)base)[index]);
    case FMT_BF16: return (double)gpurs_oracle_bf16_to_f32(((const uint16_t *)base)[index]);
    case FMT_F32: return (double)((const float *)base)[index];
    case FMT_I8: return (double)((const int8_t *)base)[index];
    case FMT_E4M3: return (double)gpurs_oracle_e4m3_to_f32(((const uint8_t *)base)[index]);
    default: return 0.0;
    }
}

static void widen_row(int format, const void *base, size_t row, size_t depth, double *out) {
    for (size_t k = 0; k < depth; k++) out[k] = element(format, base, row * depth + k);
}

/* Dot product with k ascending, as the reference's iterator sum does.  With scales, every 128-deep
 * block of the product is weighted by left_scale[block] * right_scale[block] (the dequantised
 * product of a block-scaled FP8 GEMM). */
static inline double dot(const double *a, const double *b, size_t depth, const float *left_scale,
                         const float *right_scale) {
    double sum = 0.0;
    if (!left_scale) {
        for (size_t k = 0; k < depth; k++) sum += a[k] * b[k];
        return sum;
    }
    for (size_t k0 = 0, kb = 0; k0 < depth; k0 += 128, kb++) {
        size_t k1 = k0 + 128 < depth ? k0 + 128 : depth;
        double weight = (double)left_scale[kb] * (double)right_scale[kb];
        for (size_t k = k0; k < k1; k++) sum += (a[k] * weight) * b[k];
    }
    return sum;
}

/* expected[i * columns + c] for the listed rows and every column c.  left is rows x depth, right is
 * columns x depth (the reference's "right_transposed" operand).  left_scales is [rows][ceil(depth/128)]
 * and right_scales is [ceil(columns/128)][ceil(depth/128)], or both NULL. */
API void gpurs_oracle_matmul_rows(int format, const void *left, const void *right, size_t columns,
                                  size_t depth, const int64_t *row_list, size_t row_count,
                                  const float *left_scales, const float *right_scales, double *expected) {
    size_t depth_blocks = (depth + 127) / 128;
    double *left_rows = (double *)malloc(row_count * depth * sizeof(double));
    for (size_t i = 0; i < row_count; i++) widen_row(format, left, (size_t)row_list[i], depth, left_rows + i * depth);
#pragma omp parallel
    {
        double *right_row = (double *)malloc(depth * sizeof(double));
#pragma omp for schedule(static)
        for (size_t c = 0; c < columns; c++) {
            widen_row(format, right, c, depth, right_row);
            for (size_t i = 0; i < row_count; i++) {
                const float *ls = left_scales ? left_scales + (size_t)row_list[i] * depth_blocks : NULL;
                const float *rs = right_scales ? right_scales + (c / 128) * depth_blocks : NULL;
                expected[i * columns + c] = dot(left_rows + i * depth, right_row, depth, ls, rs);
            }
        }
        free(right_row);
    }
    free(left_rows);
}

/* expected[i] for the listed flat output indices (row = index / columns, column = index % columns):
 * the sampled form of the reference's check (matrix_benchmark.rs:36-39). */
API void gpurs_oracle_matmul_samples(int format, const void *left, const void *right, size_t columns,
                                     size_t depth, const int64_t *index_list, size_t index_count,
                                     const float *left_scales, const float *right_scales, double *expected) {
    size_t depth_blocks = (depth + 127) / 128;
#pragma omp parallel
    {
        double *a = (double *)malloc(depth * sizeof(double));
        double *b = (double *)malloc(depth * sizeof(double));
#pragma omp for schedule(static)
        for (size_t i = 0; i < index_count; i++) {
            size_t row = (size_t)index_list[i] / columns, column = (size_t)index_list[i] % columns;
            widen_row(format, left, row, depth, a);
            widen_row(format, right, column, depth, b);
            const float *ls = left_scales ? left_scales + row * depth_blocks : NULL;
            const float *rs = right_scales ? right_scales + (column / 128) * depth_blocks : NULL;
            expected[i] = dot(a, b, depth, ls, rs);
        }
        free(a);
        free(b);
    }
}

/* Exact integer form for int8 operands: int64 accumulation of the listed rows, all columns. */
API void gpurs_oracle_matmul_rows_i8(const int8_t *left, const int8_t *right, size_t columns, size_t depth,
                                     const int64_t *row_list, size_t row_count, int64_t *expected) {
#pragma omp parallel for schedule(static)
    for (size_t c = 0; c < columns; c++) {
        const int8_t *b = right + c * depth;
        for (size_t i = 0; i < row_count; i++) {
            const int8_t *a = left + (size_t)row_list[i] * depth;
            int64_t sum = 0;
            for (size_t k = 0; k < depth; k++) sum += (int64_t)a[k] * (int64_t)b[k];
            expected[i * columns + c] = sum;
        }
    }
}

/* Number of threads the loops above run on. */
#ifdef _OPENMP
#include <omp.h>
API int gpurs_oracle_threads(void) { return omp_get_max_threads(); }
/* Sets it (a launcher such as torch.distributed.run exports OMP_NUM_THREADS=1 to its children; the timed CPU baseline
 * is meant to use every core the process may run on). */
API void gpurs_oracle_set_threads(int count) { omp_set_num_threads(count > 0 ? count : 1); }
#else
API int gpurs_oracle_threads(void) { return 1; }
API void gpurs_oracle_set_threads(int n) { (void)n; }
#endif
