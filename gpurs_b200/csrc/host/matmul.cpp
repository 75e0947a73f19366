// gpurs_matmul: the host half of the matrix-multiply path.  It plays the part of the launcher that
// the reference's `#[gpu]` macro generates for a kernel (crates/macros/src/launcher.rs:110-223) plus the
// example's own set-up (examples/blackwell/examples/blackwell_matrix.rs:58-83): check the arguments,
// describe A and B to the TMA unit, pick the launch geometry and enqueue one kernel.
#include "../kernels/gemm_params.hpp"
#include "runtime.hpp"

#include <algorithm>
#include <cstdio>
#include <cstring>

namespace {

using runtime::fail;

struct Choice {
    const char *stem;      // kernel entry name without the tile suffix
    int element_bytes;     // bytes per element of A and B
    int output_bytes;      // bytes per element of C
};

bool choose(int a_type, int c_type, Choice &choice) {
    struct Row { int a, c; Choice choice; };
    static const Row table[] = {
        {GPURS_F16, GPURS_F32, {"gpurs_gemm_f16_f32", 2, 4}},   {GPURS_F16, GPURS_F16, {"gpurs_gemm_f16_f16", 2, 2}},
        {GPURS_BF16, GPURS_F32, {"gpurs_gemm_bf16_f32", 2, 4}}, {GPURS_BF16, GPURS_BF16, {"gpurs_gemm_bf16_bf16", 2, 2}},
        {GPURS_F32, GPURS_F32, {"gpurs_gemm_tf32_f32", 4, 4}},  {GPURS_I8, GPURS_I32, {"gpurs_gemm_i8_i32", 1, 4}},
        {GPURS_E4M3, GPURS_F32, {"gpurs_gemm_e4m3_f32", 1, 4}}, {GPURS_E4M3, GPURS_BF16, {"gpurs_gemm_e4m3_bf16", 1, 2}},
    };
    for (const Row &row : table)
        if (row.a == a_type && row.c == c_type) {
            choice = row.choice;
            return true;
        }
    return false;
}

// Half-open byte ranges [begin, end) overlap?
bool overlap(uint64_t a, uint64_t a_bytes, uint64_t b, uint64_t b_bytes) { return a < b + b_bytes && b < a + a_bytes; }

}  // namespace

extern "C" int gpurs_matmul(gpurs_stream *stream, const gpurs_matmul_desc *desc, gpurs_device_ptr a, gpurs_device_ptr b,
                            gpurs_device_ptr c) {
    const char *const op = "gpurs_matmul";
    if (!stream || !desc) return fail(op, GPURS_E_INVALID_ARGUMENT, "null stream or descriptor");
    gpurs_gpu *gpu = stream->gpu;
    Choice choice;
    if (!choose(desc->a_type, desc->c_type, choice))
        return fail(op, GPURS_E_INVALID_ARGUMENT, "unsupported combination of operand and output types");
    const uint64_t m = desc->m, n = desc->n, k = desc->k;
    if (m > 0x7fffffffull || n > 0x7fffffffull || k > 0x7fffffffull)
        return fail(op, GPURS_E_SIZE_OVERFLOW, "a matrix dimension exceeds 2^31 - 1");
    const uint64_t lda = desc->lda ? desc->lda : k, ldb = desc->ldb ? desc->ldb : k, ldc = desc->ldc ? desc->ldc : n;
    if (lda < k || ldb < k || ldc < n) return fail(op, GPURS_E_INVALID_VIEW, "a row pitch is smaller than the row");
    // Extent of each operand in elements: the last row ends at (rows - 1) * pitch + columns.
    const uint64_t a_extent = m ? (m - 1) * lda + k : 0, b_extent = n ? (n - 1) * ldb + k : 0, c_extent = m ? (m - 1) * ldc + n : 0;
    if ((desc->a_len && desc->a_len < a_extent) || (desc->b_len && desc->b_len < b_extent) || (desc->c_len && desc->c_len < c_extent))
        return fail(op, GPURS_E_LENGTH_MISMATCH, "a slice is shorter than the matrix it is said to hold");
    if (m == 0 || n == 0) return GPURS_OK;
    if (!c) return fail(op, GPURS_E_INVALID_ARGUMENT, "null output");
    const uint64_t eb = uint64_t(choice.element_bytes), ob = uint64_t(choice.output_bytes);
    runtime::Enter enter(gpu);
    if (k == 0) {
        // An empty sum: the product is all zeros.
        for (uint64_t row = 0; row < (ldc == n ? 1 : m); row++)
            GPURS_TRY(gpu->api, cuMemsetD8Async(c + row * ldc * ob, 0, (ldc == n ? m * n : n) * ob, stream->handle));
        return GPURS_OK;
    }
    if (!a || !b) return fail(op, GPURS_E_INVALID_ARGUMENT, "null operand");
    // Writing C while reading it as an operand is rejected, as the reference's launchers reject
    // aliasing arguments (crates/gpurs/src/host/launch/kernel.rs:322-355).
    if (overlap(c, c_extent * ob, a, a_extent * eb) || overlap(c, c_extent * ob, b, b_extent * eb))
        return fail(op, GPURS_E_ALIASING, "the output overlaps an operand");
    // TMA wants 16-byte aligned bases and row pitches; rows shorter than that cannot be described
    // (`validate`, crates/gpurs/src/gpu/tensor/hopper/cursor.rs:110-116, asks for whole 128-byte rows).
    if (a % 16 || b % 16 || (lda * eb) % 16 || (ldb * eb) % 16)
        return fail(op, GPURS_E_INVALID_VIEW, "operand bases and row pitches must be multiples of 16 bytes");
    if (c % ob) return fail(op, GPURS_E_INVALID_VIEW, "the output is not aligned to its element size");
    if ((desc->scale_a != 0) != (desc->scale_b != 0))
        return fail(op, GPURS_E_INVALID_ARGUMENT, "both scale arrays or neither must be given");
    if (desc->scale_a) return fail(op, GPURS_E_INVALID_ARGUMENT, "block-scaled operands are not supported by this build");

    int group = desc->algorithm;
    if (group == GPURS_ALGO_AUTO) group = m > 128 ? GPURS_ALGO_CTA_PAIR : GPURS_ALGO_SINGLE_CTA;
    if (group != GPURS_ALGO_SINGLE_CTA && group != GPURS_ALGO_CTA_PAIR) return fail(op, GPURS_E_INVALID_ARGUMENT, "unknown algorithm");
    const int cta_group = group == GPURS_ALGO_CTA_PAIR ? 2 : 1;

    char name[96];
    std::snprintf(name, sizeof name, "%s_cg%d", choice.stem, cta_group);
    const uint32_t shared_bytes = cta_group == 2 ? gemm::SharedLayout<gemm::BLOCK_N, 2, gemm::STAGES_PAIR>::DYNAMIC_BYTES
                                                 : gemm::SharedLayout<gemm::BLOCK_N, 1, gemm::STAGES_SINGLE>::DYNAMIC_BYTES;
    gpurs_kernel *kernel = nullptr;
    int result = runtime::builtin_kernel(gpu, name, shared_bytes, &kernel);
    if (result != GPURS_OK) return result;

    // The two operand descriptors: rows of 128 bytes of K, 128-byte swizzle, out-of-range reads as
    // zero, the same form the reference encodes (crates/driver/src/memory.rs:325-354) with boxes of
    // 128 rows of A and 256 (or, per CTA of a pair, 128) rows of B.
    const uint32_t block_k = uint32_t(gemm::ROW_BYTES / choice.element_bytes);
    alignas(64) CUtensorMap map_a, map_b;
    const uint64_t dims_a[2] = {k, m}, dims_b[2] = {k, n};
    const uint64_t stride_a[1] = {lda * eb}, stride_b[1] = {ldb * eb};
    const uint32_t box_a[2] = {block_k, uint32_t(gemm::BLOCK_M)}, box_b[2] = {block_k, uint32_t(gemm::BLOCK_N / cta_group)};
    result = gpurs_tensor_map_encode(gpu, &map_a, desc->a_type, 2, a, dims_a, stride_a, box_a, 3, 3);
    if (result != GPURS_OK) return result;
    result = gpurs_tensor_map_encode(gpu, &map_b, desc->a_type, 2, b, dims_b, stride_b, box_b, 3, 3);
    if (result != GPURS_OK) return result;

    gemm::Params params;
    std::memset(&params, 0, sizeof params);
    params.c = reinterpret_cast<void *>(c);
    params.ldc = (long long)ldc;
    params.m = int(m);
    params.n = int(n);
    params.k = int(k);
    const uint64_t tile_rows = uint64_t(gemm::BLOCK_M) * cta_group;
    params.tiles_m = int((m + tile_rows - 1) / tile_rows);
    params.tiles_n = int((n + gemm::BLOCK_N - 1) / gemm::BLOCK_N);
    // Bands of 2048 rows: with one tile per SM in flight, the tiles running together then cover about
    // 2048 x 2304 outputs, whose A and B panels stay within the L2.
    params.raster_rows = 16 / cta_group;
    params.vector_stores = (c % 16 == 0 && (ldc * ob) % 16 == 0) ? 1 : 0;
    params.status = reinterpret_cast<unsigned int *>(gpu->status);

    const uint64_t tiles = uint64_t(params.tiles_m) * uint64_t(params.tiles_n);
    uint64_t ctas = desc->max_ctas > 0 ? uint64_t(desc->max_ctas) : uint64_t(gpu->multiprocessors);
    uint64_t clusters = std::max<uint64_t>(1, ctas / cta_group);
    clusters = std::min(clusters, tiles);
    gpurs_launch_config config;
    std::memset(&config, 0, sizeof config);
    config.grid[0] = uint32_t(clusters * cta_group);
    config.grid[1] = config.grid[2] = 1;
    config.block[0] = gemm::NUM_THREADS;
    config.block[1] = config.block[2] = 1;
    config.shared_bytes = shared_bytes;
    config.cluster[0] = uint32_t(cta_group);
    config.cluster[1] = config.cluster[2] = 1;
    void *arguments[3] = {&map_a, &map_b, &params};
    return runtime::launch(kernel, stream, &config, arguments);
}
