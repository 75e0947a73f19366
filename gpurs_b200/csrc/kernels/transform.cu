// Element-wise helpers that run before a GEMM.  All are HBM-bound streaming kernels: 16-byte loads and
// stores, consecutive threads on consecutive addresses, grid-stride loops sized by the host to a
// multiple of the SM count.
#include <cstdint>

// These kernels are launched with the programmatic-serialization attribute: they may be scheduled while the previous
// kernel of the stream still runs, wait here for it to complete before touching memory, and let the next kernel in.
#define GPURS_AFTER_PREVIOUS_KERNEL() asm volatile("griddepcontrol.wait;\n\tgriddepcontrol.launch_dependents;" ::: "memory")

// Splits fp32 values for a three-pass TF32 product.  Each x becomes hi = tf32(x) (round to nearest,
// the `cvt.rna.tf32.f32` the reference uses for its TF32 operands, crates/gpurs/src/gpu/float8.rs:250-256)
// and lo = tf32(x - hi); x - hi is exact in fp32.  The destination row is three K-wide segments,
//   order 0 (left operand):  [hi | hi | lo]
//   order 1 (right operand): [hi | lo | hi]
// so that one K-major product over 3K gives hi*hi + hi*lo + lo*hi, which differs from the fp32 product
// by about 2^-21 relative.
extern "C" __global__ void __launch_bounds__(256)
gpurs_split_tf32(const float *__restrict__ source, long long source_pitch, float *__restrict__ destination, int rows, int k, int order) {
    GPURS_AFTER_PREVIOUS_KERNEL();
    const long long quads_per_row = k / 4;
    const long long total = (long long)rows * quads_per_row;
    for (long long index = blockIdx.x * (long long)blockDim.x + threadIdx.x; index < total; index += (long long)gridDim.x * blockDim.x) {
        const long long row = index / quads_per_row, quad = index - row * quads_per_row;
        const float4 x = *reinterpret_cast<const float4 *>(source + row * source_pitch + quad * 4);
        float4 hi, lo;
        uint32_t bits;
#define GPURS_SPLIT(component)                                                              \
    asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(bits) : "f"(x.component));                         \
    hi.component = __uint_as_float(bits);                                                     \
    asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(bits) : "f"(x.component - hi.component));          \
    lo.component = __uint_as_float(bits);
        GPURS_SPLIT(x)
        GPURS_SPLIT(y)
        GPURS_SPLIT(z)
        GPURS_SPLIT(w)
#undef GPURS_SPLIT
        float *out = destination + row * 3ll * k + quad * 4;
        *reinterpret_cast<float4 *>(out) = hi;
        *reinterpret_cast<float4 *>(out + k) = order == 0 ? hi : lo;
        *reinterpret_cast<float4 *>(out + 2ll * k) = order == 0 ? lo : hi;
    }
}

// Both operands of a product in one launch (left operand order 0, right operand order 1): quads of the left operand first.
extern "C" __global__ void __launch_bounds__(256)
gpurs_split_tf32_pair(const float *__restrict__ left, long long left_pitch, float *__restrict__ left_destination, int left_rows,
                      const float *__restrict__ right, long long right_pitch, float *__restrict__ right_destination, int right_rows, int k) {
    GPURS_AFTER_PREVIOUS_KERNEL();
    const long long quads_per_row = k / 4;
    const long long left_total = (long long)left_rows * quads_per_row, total = left_total + (long long)right_rows * quads_per_row;
    for (long long index = blockIdx.x * (long long)blockDim.x + threadIdx.x; index < total; index += (long long)gridDim.x * blockDim.x) {
        const bool is_left = index < left_total;
        const long long local = is_left ? index : index - left_total;
        const long long row = local / quads_per_row, quad = local - row * quads_per_row;
        const float *source = is_left ? left + row * left_pitch : right + row * right_pitch;
        const float4 x = *reinterpret_cast<const float4 *>(source + quad * 4);
        float4 hi, lo;
        uint32_t bits;
#define GPURS_SPLIT(component)                                                              \
    asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(bits) : "f"(x.component));                         \
    hi.component = __uint_as_float(bits);                                                     \
    asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(bits) : "f"(x.component - hi.component));          \
    lo.component = __uint_as_float(bits);
        GPURS_SPLIT(x)
        GPURS_SPLIT(y)
        GPURS_SPLIT(z)
        GPURS_SPLIT(w)
#undef GPURS_SPLIT
        float *out = (is_left ? left_destination : right_destination) + row * 3ll * k + quad * 4;
        *reinterpret_cast<float4 *>(out) = hi;
        *reinterpret_cast<float4 *>(out + k) = is_left ? hi : lo;
        *reinterpret_cast<float4 *>(out + 2ll * k) = is_left ? lo : hi;
    }
}

// The same split for a right operand stored K x N (row-major B of C = A * B): tiles of 32 x 32 elements go through shared
// memory, so that the reads run along N and the writes along K, and the destination is the N x 3K array [hi | lo | hi] the
// product reads K-major.  Block = 32 x 8 threads, one tile per block and grid-stride step.
extern "C" __global__ void __launch_bounds__(256)
gpurs_split_tf32_transposed(const float *__restrict__ source, long long source_pitch, float *__restrict__ destination, int n, int k) {
    GPURS_AFTER_PREVIOUS_KERNEL();
    __shared__ float tile[32][33];
    const int tiles_n = (n + 31) / 32, tiles_k = (k + 31) / 32;
    const int x = threadIdx.x % 32, y = threadIdx.x / 32;
    for (long long t = blockIdx.x; t < (long long)tiles_n * tiles_k; t += gridDim.x) {
        const int tile_k = int(t / tiles_n), tile_n = int(t - (long long)tile_k * tiles_n);
#pragma unroll
        for (int i = 0; i < 4; i++) {
            const int kk = tile_k * 32 + y + 8 * i, nn = tile_n * 32 + x;
            tile[y + 8 * i][x] = (kk < k && nn < n) ? source[kk * source_pitch + nn] : 0.0f;
        }
        __syncthreads();
#pragma unroll
        for (int i = 0; i < 4; i++) {
            const int nn = tile_n * 32 + y + 8 * i, kk = tile_k * 32 + x;
            if (nn < n && kk < k) {
                const float value = tile[x][y + 8 * i];
                uint32_t bits;
                asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(bits) : "f"(value));
                const float hi = __uint_as_float(bits);
                asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(bits) : "f"(value - hi));
                const float lo = __uint_as_float(bits);
                float *out = destination + nn * 3ll * k + kk;
                out[0] = hi, out[k] = lo, out[2ll * k] = hi;
            }
        }
        __syncthreads();
    }
}

// A right operand stored K x N copied as N x K (what the kernels without an N-major read take): tiles of 32 x 32 elements
// through shared memory, reads along N, writes along K.  Block = 32 x 8 threads, one tile per block and grid-stride step.
template <typename T>
__device__ __forceinline__ void transpose_body(const T *__restrict__ source, long long source_pitch, T *__restrict__ destination, int n, int k) {
    __shared__ T tile[32][33];
    const int tiles_n = (n + 31) / 32, tiles_k = (k + 31) / 32;
    const int x = threadIdx.x % 32, y = threadIdx.x / 32;
    for (long long t = blockIdx.x; t < (long long)tiles_n * tiles_k; t += gridDim.x) {
        const int tile_k = int(t / tiles_n), tile_n = int(t - (long long)tile_k * tiles_n);
#pragma unroll
        for (int i = 0; i < 4; i++) {
            const int kk = tile_k * 32 + y + 8 * i, nn = tile_n * 32 + x;
            if (kk < k && nn < n) tile[y + 8 * i][x] = source[kk * source_pitch + nn];
        }
        __syncthreads();
#pragma unroll
        for (int i = 0; i < 4; i++) {
            const int nn = tile_n * 32 + y + 8 * i, kk = tile_k * 32 + x;
            if (nn < n && kk < k) destination[(long long)nn * k + kk] = tile[x][y + 8 * i];
        }
        __syncthreads();
    }
}

extern "C" __global__ void __launch_bounds__(256)
gpurs_transpose_b8(const uint8_t *__restrict__ source, long long source_pitch, uint8_t *__restrict__ destination, int n, int k) {
    GPURS_AFTER_PREVIOUS_KERNEL();
    transpose_body(source, source_pitch, destination, n, k);
}
extern "C" __global__ void __launch_bounds__(256)
gpurs_transpose_b16(const uint16_t *__restrict__ source, long long source_pitch, uint16_t *__restrict__ destination, int n, int k) {
    GPURS_AFTER_PREVIOUS_KERNEL();
    transpose_body(source, source_pitch, destination, n, k);
}
extern "C" __global__ void __launch_bounds__(256)
gpurs_transpose_b32(const uint32_t *__restrict__ source, long long source_pitch, uint32_t *__restrict__ destination, int n, int k) {
    GPURS_AFTER_PREVIOUS_KERNEL();
    transpose_body(source, source_pitch, destination, n, k);
}

#include "gemm_sparse_tcgen05.cuh"

// 2:4 compression of a 16-bit matrix (no counterpart in the reference, which has no sparse path).  One
// thread handles 16 consecutive logical K of one row: 32 bytes in, the 8 kept values (16 bytes) and 16 bits of
// metadata out.  In every group of four the first two non-zeros are kept; a group with fewer than two
// non-zeros keeps zeros from its lowest free positions, so the kept positions are distinct and ascending.
// A group with more than two non-zeros is not 2:4: it is counted in *violations (if given) and loses its
// later non-zeros.  Metadata goes to the block layout of gemm::metadata_offset.
extern "C" __global__ void __launch_bounds__(256)
gpurs_compress_24(const uint16_t *__restrict__ dense, long long pitch, uint16_t *__restrict__ values, uint8_t *__restrict__ metadata,
                  unsigned int *violations, int rows, int k) {
    GPURS_AFTER_PREVIOUS_KERNEL();
    const long long spans_per_row = k / 16;
    const long long total = (long long)rows * spans_per_row;
    const int k_blocks = (k + gemm::SPARSE_STAGE_K - 1) / gemm::SPARSE_STAGE_K;
    unsigned int bad = 0;
    for (long long index = blockIdx.x * (long long)blockDim.x + threadIdx.x; index < total; index += (long long)gridDim.x * blockDim.x) {
        const long long row = index / spans_per_row;
        const int span = int(index - row * spans_per_row);
        const uint4 *source = reinterpret_cast<const uint4 *>(dense + row * pitch + span * 16);
        const uint4 lo = source[0], hi = source[1];
        const uint32_t words[8] = {lo.x, lo.y, lo.z, lo.w, hi.x, hi.y, hi.z, hi.w};
        uint32_t kept_words[4];
        uint32_t nibbles = 0;
#pragma unroll
        for (int group = 0; group < 4; group++) {
            const uint16_t v[4] = {uint16_t(words[2 * group]), uint16_t(words[2 * group] >> 16), uint16_t(words[2 * group + 1]),
                                   uint16_t(words[2 * group + 1] >> 16)};
            int first = -1, second = -1, nonzero = 0;
#pragma unroll
            for (int position = 0; position < 4; position++)
                if ((v[position] & 0x7fffu) != 0) {
                    if (nonzero == 0) first = position;
                    else if (nonzero == 1) second = position;
                    nonzero++;
                }
            bad += nonzero > 2;
#pragma unroll
            for (int position = 0; position < 4; position++)
                if ((v[position] & 0x7fffu) == 0) {
                    if (first < 0) first = position;
                    else if (second < 0 && position != first) second = position;
                }
            if (first > second) { const int t = first; first = second; second = t; }
            kept_words[group] = uint32_t(v[first]) | (uint32_t(v[second]) << 16);
            nibbles |= uint32_t(first | (second << 2)) << (4 * group);
        }
        *reinterpret_cast<uint4 *>(values + row * (long long)(k / 2) + span * 8) = make_uint4(kept_words[0], kept_words[1], kept_words[2], kept_words[3]);
        const long long block = (row / 128) * k_blocks + (span * 16) / gemm::SPARSE_STAGE_K;
        const int offset = gemm::metadata_offset(int(row % 128), (span * 16) % gemm::SPARSE_STAGE_K);
        *reinterpret_cast<uint16_t *>(metadata + block * gemm::METADATA_BLOCK_BYTES + offset) = uint16_t(nibbles);
    }
    if (violations != nullptr && bad != 0) atomicAdd(violations, bad);
}

#include <cuda_fp8.h>

// Block quantisation of an fp32 matrix to E4M3 with one fp32 scale per block of BLOCK_ROWS x 128 elements
// (BLOCK_ROWS = 1 for a left operand, 128 for a right one): scale = absmax / 448, or 1 for an all-zero block,
// code = E4M3(x / scale) with round-to-nearest-even and saturation, the conversion the reference's host code
// performs in crates/gpurs/src/gpu/float8.rs:20-52 (`cvt.rn.satfinite.e4m3x2.f32` on the device, float8.rs:96-101).
// One warp owns 128 consecutive elements of a row (a float4 per lane); for 128-row blocks a CTA of 32 warps owns
// the block, each warp four of its rows, and the block maximum goes through shared memory.
template <int BLOCK_ROWS>
__device__ __forceinline__ void quantize_e4m3_body(const float *__restrict__ source, long long pitch, uint8_t *__restrict__ codes,
                                                    float *__restrict__ scales, int rows, int k) {
    constexpr int ROWS_PER_WARP = BLOCK_ROWS == 1 ? 1 : 4;
    __shared__ float warp_max[32];
    const int lane = threadIdx.x % 32, warp = threadIdx.x / 32;
    const int k_blocks = (k + 127) / 128;
    const long long row_blocks = (rows + BLOCK_ROWS - 1) / BLOCK_ROWS;
    // BLOCK_ROWS == 1: a "block" per warp, blockDim.x / 32 of them per CTA; otherwise one block per CTA.
    const long long blocks_total = row_blocks * k_blocks;
    const int per_cta = BLOCK_ROWS == 1 ? blockDim.x / 32 : 1;
    for (long long first = (long long)blockIdx.x * per_cta; first < blocks_total; first += (long long)gridDim.x * per_cta) {
        const long long block = BLOCK_ROWS == 1 ? first + warp : first;
        const bool active = block < blocks_total;
        const long long row_block = active ? block / k_blocks : 0;
        const int k_block = active ? int(block - row_block * k_blocks) : 0;
        const int column = k_block * 128 + lane * 4;
        float4 values[ROWS_PER_WARP];
        float absmax = 0.0f;
#pragma unroll
        for (int i = 0; i < ROWS_PER_WARP; i++) {
            const long long row = row_block * BLOCK_ROWS + (BLOCK_ROWS == 1 ? 0 : warp * ROWS_PER_WARP + i);
            values[i] = make_float4(0.f, 0.f, 0.f, 0.f);
            if (active && row < rows && column < k) {   // k is a multiple of 4, so a float4 is all in or all out
                values[i] = *reinterpret_cast<const float4 *>(source + row * pitch + column);
                absmax = fmaxf(absmax, fmaxf(fmaxf(fabsf(values[i].x), fabsf(values[i].y)), fmaxf(fabsf(values[i].z), fabsf(values[i].w))));
            }
        }
#pragma unroll
        for (int offset = 16; offset > 0; offset >>= 1) absmax = fmaxf(absmax, __shfl_xor_sync(0xffffffffu, absmax, offset));
        if constexpr (BLOCK_ROWS != 1) {
            if (lane == 0) warp_max[warp] = absmax;
            __syncthreads();
            absmax = warp_max[lane];
#pragma unroll
            for (int offset = 16; offset > 0; offset >>= 1) absmax = fmaxf(absmax, __shfl_xor_sync(0xffffffffu, absmax, offset));
            __syncthreads();
        }
        const float scale = absmax > 0.0f ? __fdiv_rn(absmax, 448.0f) : 1.0f;
        if (active && lane == 0 && (BLOCK_ROWS == 1 || warp == 0)) scales[block] = scale;
#pragma unroll
        for (int i = 0; i < ROWS_PER_WARP; i++) {
            const long long row = row_block * BLOCK_ROWS + (BLOCK_ROWS == 1 ? 0 : warp * ROWS_PER_WARP + i);
            if (active && row < rows && column < k) {
                const __nv_fp8x2_storage_t low = __nv_cvt_float2_to_fp8x2(make_float2(__fdiv_rn(values[i].x, scale), __fdiv_rn(values[i].y, scale)), __NV_SATFINITE, __NV_E4M3);
                const __nv_fp8x2_storage_t high = __nv_cvt_float2_to_fp8x2(make_float2(__fdiv_rn(values[i].z, scale), __fdiv_rn(values[i].w, scale)), __NV_SATFINITE, __NV_E4M3);
                *reinterpret_cast<uint32_t *>(codes + row * (long long)k + column) = uint32_t(low) | (uint32_t(high) << 16);
            }
        }
    }
}

extern "C" __global__ void __launch_bounds__(256)
gpurs_quantize_e4m3_rows(const float *source, long long pitch, uint8_t *codes, float *scales, int rows, int k) {
    GPURS_AFTER_PREVIOUS_KERNEL();
    quantize_e4m3_body<1>(source, pitch, codes, scales, rows, k);
}

extern "C" __global__ void __launch_bounds__(1024)
gpurs_quantize_e4m3_tiles(const float *source, long long pitch, uint8_t *codes, float *scales, int rows, int k) {
    GPURS_AFTER_PREVIOUS_KERNEL();
    quantize_e4m3_body<128>(source, pitch, codes, scales, rows, k);
}


#include "gemm_mx_tcgen05.cuh"

// MX quantiser: fp32 -> E4M3 codes with one power-of-two scale (UE8M0 byte = exponent + 127) per 32 elements of a row,
// the scale being the smallest power of two that brings the group's largest magnitude to 448 or below (1 for an all-zero
// group); dividing by a power of two is exact, so code = E4M3(x * 2^-e), round to nearest even with saturation like the
// reference's host conversion (crates/gpurs/src/gpu/float8.rs:20-52).  Scales are written in the tiled order of
// gemm::mx_scale_index for the left or the right operand.  One warp per 128 elements of a row (8 lanes per group).
extern "C" __global__ void __launch_bounds__(256)
gpurs_quantize_mx_e4m3(const float *__restrict__ source, long long pitch, uint8_t *__restrict__ codes, uint8_t *__restrict__ scales, int rows, int k,
                       int right_operand) {
    GPURS_AFTER_PREVIOUS_KERNEL();
    const int lane = threadIdx.x % 32;
    const int k_blocks = (k + 127) / 128;
    const long long spans = (long long)rows * k_blocks;
    for (long long span = (long long)blockIdx.x * (blockDim.x / 32) + threadIdx.x / 32; span < spans; span += (long long)gridDim.x * (blockDim.x / 32)) {
        const long long row = span / k_blocks;
        const int column = int(span - row * k_blocks) * 128 + lane * 4;
        float4 x = make_float4(0.f, 0.f, 0.f, 0.f);
        if (column < k) x = *reinterpret_cast<const float4 *>(source + row * pitch + column);   // k is a multiple of 4
        float absmax = fmaxf(fmaxf(fabsf(x.x), fabsf(x.y)), fmaxf(fabsf(x.z), fabsf(x.w)));
#pragma unroll
        for (int offset = 4; offset > 0; offset >>= 1) absmax = fmaxf(absmax, __shfl_xor_sync(0xffffffffu, absmax, offset));
        // absmax = f * 2^x with 1 <= f < 2; 448 = 1.75 * 2^8: e = x - 8 if f <= 1.75, else x - 7
        int exponent = 0;
        if (absmax > 0.0f && absmax <= 3.0e38f) {
            int x2;
            const float fraction = frexpf(absmax, &x2) * 2.0f;      // frexpf gives [0.5, 1)
            exponent = (x2 - 1) - (fraction <= 1.75f ? 8 : 7);
            exponent = max(-127, min(127, exponent));
        }
        if (column < k) {
            const __nv_fp8x2_storage_t low = __nv_cvt_float2_to_fp8x2(make_float2(scalbnf(x.x, -exponent), scalbnf(x.y, -exponent)), __NV_SATFINITE, __NV_E4M3);
            const __nv_fp8x2_storage_t high = __nv_cvt_float2_to_fp8x2(make_float2(scalbnf(x.z, -exponent), scalbnf(x.w, -exponent)), __NV_SATFINITE, __NV_E4M3);
            *reinterpret_cast<uint32_t *>(codes + row * (long long)k + column) = uint32_t(low) | (uint32_t(high) << 16);
            if (lane % 8 == 0) scales[gemm::mx_scale_index(right_operand != 0, row, column, k_blocks)] = uint8_t(exponent + 127);
        }
    }
}
