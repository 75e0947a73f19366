// Element-wise helpers that run before a GEMM.  All are HBM-bound streaming kernels: 16-byte loads and
// stores, consecutive threads on consecutive addresses, grid-stride loops sized by the host to a
// multiple of the SM count.
#include <cstdint>

// Splits fp32 values for a three-pass TF32 product.  Each x becomes hi = tf32(x) (round to nearest,
// the `cvt.rna.tf32.f32` the reference uses for its TF32 operands, crates/gpurs/src/gpu/float8.rs:250-256)
// and lo = tf32(x - hi); x - hi is exact in fp32.  The destination row is three K-wide segments,
//   order 0 (left operand):  [hi | hi | lo]
//   order 1 (right operand): [hi | lo | hi]
// so that one K-major product over 3K gives hi*hi + hi*lo + lo*hi, which differs from the fp32 product
// by about 2^-21 relative.
extern "C" __global__ void __launch_bounds__(256)
gpurs_split_tf32(const float *__restrict__ source, long long source_pitch, float *__restrict__ destination, int rows, int k, int order) {
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
