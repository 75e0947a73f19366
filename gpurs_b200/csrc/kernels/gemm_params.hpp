// Types shared by the GEMM kernels and the host code that launches them: the kernel parameter block,
// the shared-memory layout of a pipeline, and the status codes of the bounded device waits.
#pragma once
#include <cstdint>

namespace gemm {

// Output element types.
enum : int { OUT_F32 = 0, OUT_BF16 = 1, OUT_F16 = 2, OUT_I32 = 3 };

// Device status codes written to the status word when a bounded wait gives up.
enum : uint32_t {
    STATUS_OK = 0,
    STATUS_PRODUCER_TIMEOUT = 1,
    STATUS_MMA_TIMEOUT = 2,
    STATUS_EPILOGUE_TIMEOUT = 3,
    STATUS_PROBE_TIMEOUT = 4,     // the self-test kernel (diagnostics.cu)
};

// Kernel parameter block of the tile kernels (after the TMA descriptors).  Hosts that launch an entry themselves
// through the module door fill it field by field; its layout is part of the kernel image's interface.
struct Params {
    void *c;                 // output, row-major M x N with row pitch ldc (elements)
    long long ldc;
    int m, n, k;
    int tiles_m, tiles_n;    // in units of (128 * CTA_GROUP) x BLOCK_N tiles
    int raster_rows;         // tile rows walked together so concurrent tiles share operands in L2
    int vector_stores;       // 1 when every output row start is 16-byte aligned (16-byte stores, and TMA stores where a
                             // kernel takes a descriptor of C)
    int b_row_major;         // dense kernels: 0 = B is N x K (K contiguous, the reference's layout), 1 = B is K x N (N contiguous)
    unsigned int *status;    // [0] first failure code, [1] block, [2] tile, [3] K-block
    const float *scale_a;    // block-scaled FP8 only: [M][ceil(K/128)]
    const float *scale_b;    // block-scaled FP8 only: [ceil(N/128)][ceil(K/128)]
    const float *bias;       // optional fp32 [N], added to every row before the output rounding (float outputs), or null
    int l2_policy;           // dense kernels: 0 no hint; 1 keep A (evict last), stream B (evict first); 2 the reverse; 3 keep both
    int batches;             // batched entries: number of matrices (0 or 1 = one); every other entry ignores it
    // Epilogue algebra on float outputs, applied in this order before the output rounding (each optional):
    //     value * alpha * row_scale[row] * column_scale[column] + bias[column]
    const float *row_scale;     // fp32 [M] or null: e.g. a per-token activation scale
    const float *column_scale;  // fp32 [N] or null: e.g. a per-channel weight scale
    float alpha;                // used when scaled_by_alpha != 0
    int scaled_by_alpha;
    long long batch_stride_c;   // batched entries: elements between successive outputs (for the per-lane store path)
    float *row_absmax;          // dense tile kernels, float outputs: fp32 [M] or null; max |value| of each output row (after the
                                // algebra above, before the output rounding) is folded in with an atomic max, so the caller
                                // zeroes it first.  What a per-row quantiser of C needs, without reading C again.
    // Stream-K entries only: scratch for the partial tiles of the split round, [split tile][contributor][tile rows][BLOCK_N]
    // 32-bit sums; one arrival counter per split tile and epilogue warp (zero between launches); contributors allotted per tile.
    void *partials;
    unsigned int *split_counters;
    int max_contributors;
    int split_tiles;            // tiles of the last round that are split (the host's decision, gemm_schedule.hpp)
    // More epilogue algebra on float outputs, after the bias and before the output rounding (each optional):
    //     value + row_bias[row] + beta * residual[row, column]
    const float *row_bias;      // fp32 [M] or null: one value added to every element of the row
    const void *residual;       // matrix of C's element type with row pitch ldr (elements), or null; it may be C itself
    long long ldr;
    float beta;                 // factor of the residual
    int accumulate;             // fp32 output only: 1 = add the result to what C holds (atomic adds) instead of storing it
    float *row_sum;             // fp32 [M] or null: the sum of each output row's values (after the algebra, before the output
                                // rounding) is added in with atomic adds, one per row and tile; the caller zeroes it first
};
static_assert(sizeof(Params) == 192, "the parameter block is part of the kernel image's interface");

constexpr int MAX_PUSH_TARGETS = 8;   // GPUs of one box

constexpr int BLOCK_M = 128;       // rows per CTA (= TMEM lanes)
constexpr int ROW_BYTES = 128;     // bytes of K per stage row: one 128-byte swizzle span
constexpr int MMA_K_BYTES = 32;    // bytes of K per tcgen05.mma
constexpr int NUM_THREADS = 192;
constexpr int EPILOGUE_WARPS = 4;
constexpr int GROUPED_THREADS = 320;  // grouped kernel: weight producer, MMA issuer, 4 epilogue warps, 4 gather warps
constexpr int SCALED_THREADS = 384;  // promotion kernels: warpgroup 0 (producer warp, MMA warp, two idle), 8 promotion warps
constexpr int BLOCK_N = 256;       // columns per tile
constexpr int STAGES_SINGLE = 4;   // pipeline depth of the one-CTA kernels (48 KiB per stage)
constexpr int STAGES_PAIR = 6;     // pipeline depth of the CTA-pair kernels (32 KiB per stage and CTA)

// Dynamic shared memory of the CTA-pair block-scaled FP8 entries (gemm_blockscaled_tcgen05.cuh): 6 stages of 32 KiB, 24 barriers,
// one 4 KiB output box per promotion warp, alignment slack.
constexpr int BLOCKSCALED_SHARED = ((6 * 32768 + (2 * 6 + 12) * 8 + 8 + 16 + 1023) / 1024) * 1024 + 8 * 32 * 128 + 1024;

// Dynamic shared memory of the 256 x 512 CTA-pair entries (gemm_wide_tcgen05.cuh): 4 stages of 48 KiB, 12 barriers, 32 KiB of
// output staging, alignment slack.
constexpr int WIDE_NUM_THREADS = 320;     // producer warp, MMA warp, eight epilogue warps
constexpr int WIDE_SHARED = ((4 * 49152 + (2 * 4 + 4) * 8 + 8 + 1023) / 1024) * 1024 + 4 * 2 * 32 * 128 + 1024;

template <int BLOCK_N, int CTA_GROUP, int STAGES>
struct SharedLayout {
    static constexpr int A_BYTES = BLOCK_M * ROW_BYTES;
    static constexpr int B_ROWS = BLOCK_N / CTA_GROUP;   // rows of the B tile this CTA loads
    static constexpr int B_BYTES = B_ROWS * ROW_BYTES;
    static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
    static constexpr int BARRIER_OFFSET = STAGES * STAGE_BYTES;
    // full[STAGES], empty[STAGES], accumulator_full[4], accumulator_empty[4] (the dense kernels use two of each),
    // then the TMEM base word
    static constexpr int NUM_BARRIERS = 2 * STAGES + 8;
    static constexpr int TMEM_SLOT_OFFSET = BARRIER_OFFSET + NUM_BARRIERS * 8;
    static constexpr int ABORT_OFFSET = TMEM_SLOT_OFFSET + 4;
    // Epilogue staging for TMA stores: per epilogue warp two buffers of 32 rows x 128 bytes (128-byte swizzle).
    static constexpr int STAGING_OFFSET = ((ABORT_OFFSET + 4 + 1023) / 1024) * 1024;
    static constexpr int STAGING_BYTES = EPILOGUE_WARPS * 2 * 32 * ROW_BYTES;
    static constexpr int TOTAL = STAGING_OFFSET + STAGING_BYTES;
    static constexpr int DYNAMIC_BYTES = TOTAL + 1024;   // slack to align the stages to 1024 bytes
    static_assert(DYNAMIC_BYTES <= 232448, "more than the 227 KiB a CTA may have");
};

// Skinny kernels (gemm_skinny_tcgen05.cuh): 8 stages of 128 rows of the big operand + the padded small one.
constexpr int skinny_shared_bytes(int tokens) { return 8 * (BLOCK_M * ROW_BYTES + ((tokens * ROW_BYTES + 1023) / 1024) * 1024) + (2 * 8 + 1) * 8 + 8 + 1024; }
constexpr int SKINNY_MAX_ROWS = 64;      // m up to which the skinny kernels are used
constexpr int SKINNY_MAX_TILES = 4096;   // turn counters kept per gpu handle

// 2:4 sparse kernels (gemm_sparse_tcgen05.cuh).  Their tiles are 224 columns wide: two accumulators of 224 columns and the
// 16 metadata columns of the pipeline stages fit the 512 columns of tensor memory (2 x 256 + 16 would not), so that a
// tile's epilogue overlaps the next tile's main loop.  Dynamic shared memory of the one-CTA (2 stages of 74 KiB) and
// CTA-pair (4 stages of 46 KiB) entries, and the size of one metadata block (128 rows x 128 logical K).
constexpr int SPARSE_BLOCK_N = 224;
constexpr int SPARSE_SHARED_SINGLE = 2 * (BLOCK_M * ROW_BYTES + 2 * SPARSE_BLOCK_N * ROW_BYTES + 2048) + (2 * 2 + 4) * 8 + 8 + 1024;
constexpr int SPARSE_SHARED_PAIR = 4 * (BLOCK_M * ROW_BYTES + SPARSE_BLOCK_N * ROW_BYTES + 2048) + (2 * 4 + 4) * 8 + 8 + 1024;
// the CTA-pair push entry adds 32 KiB of output staging behind the stages (1024-byte aligned)
constexpr int SPARSE_SHARED_PAIR_PUSH = ((SPARSE_SHARED_PAIR - 1024 + 1023) / 1024) * 1024 + 4 * 2 * 32 * ROW_BYTES + 1024;
// 512 x 224 pair tiles: three stages of two A tiles, the CTA's half of B and two metadata blocks
constexpr int SPARSE_TALL_NUM_THREADS = 320;     // producer warp, MMA warp, eight epilogue warps
constexpr int SPARSE_TALL_SHARED = 3 * (2 * BLOCK_M * ROW_BYTES + SPARSE_BLOCK_N * ROW_BYTES + 2 * 2048) + (2 * 3 + 4) * 8 + 8 + 1024;
constexpr int SPARSE_METADATA_BLOCK_BYTES = 2048;
constexpr int SPARSE_BLOCK_K = 128;

// MX (hardware block-scaled FP8) kernels (gemm_mx_tcgen05.cuh): 224-column tiles; per stage A (16 KiB), B (28 KiB, or 14 KiB per
// CTA of a pair) and 2 KiB of scales; 12 columns of tensor memory per stage hold the scales, which bounds the depth.
constexpr int MX_BLOCK_N = 224;
constexpr int MX_STAGES_SINGLE = 4, MX_STAGES_PAIR = 5;
constexpr int MX_SHARED_SINGLE = MX_STAGES_SINGLE * (BLOCK_M * ROW_BYTES + MX_BLOCK_N * ROW_BYTES + 2048) + (2 * MX_STAGES_SINGLE + 4) * 8 + 8 + 1024;
constexpr int MX_SHARED_PAIR = MX_STAGES_PAIR * (BLOCK_M * ROW_BYTES + MX_BLOCK_N / 2 * ROW_BYTES + 2048) + (2 * MX_STAGES_PAIR + 4) * 8 + 8 + 1024;

}  // namespace gemm
