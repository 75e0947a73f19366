// gpurs_matmul_f32_static: the fp32 product for callers that must not allocate device memory.
//
// The regular fp32 path (gpurs_matmul with GPURS_F32 operands) splits both operands into TF32 hi / lo
// parts and needs scratch memory for the split copies, which it takes from a block that grows with
// cuMemAlloc / cuMemFree.  Some hosts cannot afford that: a serving loop that has handed every byte of
// the device to its own pool (a direct driver allocation then fails, or succeeds only by fragmenting the
// pool's address space), and latency-bound callers for which the implicit device-wide synchronisation of
// cuMemAlloc / cuMemFree is itself the problem.  For them this file keeps the split copies in a fixed
// array that is part of the loaded library image: GPURS_STATIC_SCRATCH_BYTES on every GPU that loads the
// library, held until the process exits, and nothing is allocated or freed by a call.
//
// Consequences a caller has to know:
//   * problems whose split copies do not fit the array are rejected (GPURS_E_SIZE_OVERFLOW);
//   * every call on a device shares the one array and overwrites what the previous call left there.  Calls
//     that can run at the same time on the GPU (different streams, no ordering between them) race on it;
//     calls on one stream are ordered by the stream and are safe;
//   * nothing in the array has to start at zero: the split kernel writes every element the GEMM reads,
//     rows past the end of a tile come from the TMA unit's out-of-range fill, not from the array;
//   * every call asks the CUDA runtime for the array's device address (a host-side lookup that allocates
//     nothing once the library image is loaded on the device) and hands that one address to both kernels,
//     so a handle that was closed and reopened, or a context that was torn down and rebuilt in between,
//     can never leave a stale address behind.  The first call on each device also loads the kernels; make
//     that first call before starting any stream capture.
#include "gemm_launch.hpp"

#include <cuda_runtime.h>

#include <algorithm>
#include <cstdio>

namespace {

// The scratch itself.  In host code this name is only a handle for cudaGetSymbolAddress: it is not a
// device address and must never be passed to a kernel or to the TMA descriptor encoder.
static __device__ __align__(256) float static_scratch[GPURS_STATIC_SCRATCH_BYTES / sizeof(float)];

// Same split as the regular path's kernel: x -> hi = tf32(x), lo = tf32(x - hi), written as three K-wide
// segments per row, [hi | hi | lo] for the left operand and [hi | lo | hi] for the right one, so that one
// K-major product over 3K gives hi*hi + hi*lo + lo*hi.  Both operands are handled by one launch and the
// destination is the static array at the address the host resolved for this call (`scratch`, the same pointer the
// product's TMA descriptors are built from): rows of A first, rows of B from `b_offset` floats on.
__global__ void __launch_bounds__(256)
split_tf32_static(const float *__restrict__ a, const float *__restrict__ b, float *__restrict__ scratch, int m, int n, int k, long long b_offset) {
    const long long quads_per_row = k / 4;
    const long long total = (long long)(m + n) * quads_per_row;
    for (long long index = blockIdx.x * (long long)blockDim.x + threadIdx.x; index < total; index += (long long)gridDim.x * blockDim.x) {
        const long long row = index / quads_per_row, quad = index - row * quads_per_row;
        const bool left = row < m;
        const float *source = left ? a + row * (long long)k : b + (row - m) * (long long)k;
        float *out = left ? scratch + row * 3ll * k : scratch + b_offset + (row - m) * 3ll * k;
        const float4 x = *reinterpret_cast<const float4 *>(source + quad * 4);
        const float in[4] = {x.x, x.y, x.z, x.w};
        float hi[4], lo[4];
#pragma unroll
        for (int i = 0; i < 4; i++) {
            uint32_t bits;
            asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(bits) : "f"(in[i]));
            hi[i] = __uint_as_float(bits);
            asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(bits) : "f"(in[i] - hi[i]));
            lo[i] = __uint_as_float(bits);
        }
        const float4 high = make_float4(hi[0], hi[1], hi[2], hi[3]), low = make_float4(lo[0], lo[1], lo[2], lo[3]);
        out += quad * 4;
        *reinterpret_cast<float4 *>(out) = high;
        *reinterpret_cast<float4 *>(out + k) = left ? high : low;
        *reinterpret_cast<float4 *>(out + 2ll * k) = left ? low : high;
    }
}

int fail_runtime(const char *operation, cudaError_t code) {
    return runtime::fail(operation, int(code), cudaGetErrorString(code));
}

bool overlap(uint64_t a, uint64_t a_bytes, uint64_t b, uint64_t b_bytes) { return a < b + b_bytes && b < a + a_bytes; }

}  // namespace

extern "C" int gpurs_matmul_f32_static(gpurs_stream *stream, uint64_t m, uint64_t n, uint64_t k, gpurs_device_ptr a,
                                       gpurs_device_ptr b, gpurs_device_ptr c) {
    const char *const op = "gpurs_matmul_f32_static";
    if (!stream) return runtime::fail(op, GPURS_E_INVALID_ARGUMENT, "null stream");
    gpurs_gpu *gpu = stream->gpu;
    if (m > 0x7fffffffull || n > 0x7fffffffull || k > 0x7fffffffull / 3)
        return runtime::fail(op, GPURS_E_SIZE_OVERFLOW, "a matrix dimension exceeds what the kernels index");
    if (m == 0 || n == 0) return GPURS_OK;
    if (k == 0 || k % 4) return runtime::fail(op, GPURS_E_INVALID_VIEW, "k must be a positive multiple of 4 (16-byte rows)");
    if (!a || !b || !c) return runtime::fail(op, GPURS_E_INVALID_ARGUMENT, "null operand or output");
    if (a % 16 || b % 16 || c % 4) return runtime::fail(op, GPURS_E_INVALID_VIEW, "operands must be 16-byte aligned, the output 4-byte aligned");
    // Split copies: m x 3k floats, then (256-byte aligned) n x 3k floats.
    const uint64_t a_split = (m * 3 * k * 4 + 255) & ~uint64_t(255), b_split = n * 3 * k * 4;
    // each term is below 2^64 for dimensions below 2^31 (3k included); their sum need not be: compare without adding
    if (a_split > uint64_t(GPURS_STATIC_SCRATCH_BYTES) || b_split > uint64_t(GPURS_STATIC_SCRATCH_BYTES) - a_split) {
        static thread_local char message[160];
        std::snprintf(message, sizeof message, "the split operands need %llu bytes but the static scratch holds %llu: use gpurs_matmul",
                      (unsigned long long)(a_split + std::min<uint64_t>(b_split, ~uint64_t(0) - a_split)), (unsigned long long)GPURS_STATIC_SCRATCH_BYTES);
        return runtime::fail(op, GPURS_E_SIZE_OVERFLOW, message);
    }
    const uint64_t a_bytes = m * k * 4, b_bytes = n * k * 4, c_bytes = m * n * 4;
    if (overlap(c, c_bytes, a, a_bytes) || overlap(c, c_bytes, b, b_bytes))
        return runtime::fail(op, GPURS_E_ALIASING, "the output overlaps an operand");

    runtime::Enter enter(gpu);   // the gpu's (primary) context is current from here on, for both APIs
    // With that device current: ask the runtime where the array lives in this context.  Asked on every call, never
    // cached: the answer belongs to the context that is current now.
    float *scratch = nullptr;
    const cudaError_t found = cudaGetSymbolAddress(reinterpret_cast<void **>(&scratch), static_scratch);
    if (found != cudaSuccess) return fail_runtime("cudaGetSymbolAddress", found);
    if (!scratch) return runtime::fail(op, GPURS_E_INVALID_ARGUMENT, "the static scratch has no device address");

    const uint64_t quads = (m + n) * (k / 4);
    const unsigned blocks = unsigned(std::max<uint64_t>(1, std::min<uint64_t>((quads + 255) / 256, uint64_t(gpu->multiprocessors) * 8)));
    split_tf32_static<<<blocks, 256, 0, reinterpret_cast<cudaStream_t>(stream->handle)>>>(
        reinterpret_cast<const float *>(a), reinterpret_cast<const float *>(b), scratch, int(m), int(n), int(k), (long long)(a_split / 4));
    const cudaError_t launched = cudaGetLastError();
    if (launched != cudaSuccess) return fail_runtime("split_tf32_static", launched);
    gpu->launches++;

    launcher::Gemm gemm;
    gemm.stem = "gpurs_gemm_tf32_promoted_f32";
    gemm.element_type = GPURS_F32;
    gemm.element_bytes = 4;
    gemm.output_bytes = 4;
    gemm.a = reinterpret_cast<gpurs_device_ptr>(scratch);
    gemm.b = reinterpret_cast<gpurs_device_ptr>(scratch) + a_split;
    gemm.c = c;
    gemm.lda = gemm.ldb = 3 * k;
    gemm.ldc = n;
    gemm.m = m, gemm.n = n, gemm.k = 3 * k;
    gemm.cta_group = 1;
    gemm.raster_rows = 0;
    gemm.max_ctas = 0;
    gemm.threads = gemm::SCALED_THREADS;
    gemm.whole_tiles = true;      // tiles split along K would borrow the handle's workspace, which is allocated memory
    return launcher::launch_gemm(stream, gemm);
}
