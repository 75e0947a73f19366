// gpurs_matmul: the host half of the matrix-multiply path.  It plays the part of the launcher that
// the reference's `#[gpu]` macro generates for a kernel (crates/macros/src/launcher.rs:110-223) plus the
// example's own set-up (examples/blackwell/examples/blackwell_matrix.rs:58-83): check the arguments,
// describe A and B to the TMA unit, pick the launch geometry and enqueue one kernel.
#include "gemm_launch.hpp"
#include "../kernels/gemm_schedule.hpp"

#include <algorithm>
#include <cstdio>
#include <cstring>
#include <utility>
#include <vector>

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

// Host mirror of gemm::PushTargets (kernels/gemm_tcgen05.cuh).
struct PushTargets {
    alignas(64) CUtensorMap maps[gemm::MAX_PUSH_TARGETS];
    int count;
    int row_offset;
    int first;
    int reserved;
};

// Host mirror of gemm::SparsePushTargets (kernels/gemm_sparse_tcgen05.cuh).
struct SparsePushTargets {
    alignas(64) CUtensorMap maps[gemm::MAX_PUSH_TARGETS];
    alignas(64) CUtensorMap half_maps[gemm::MAX_PUSH_TARGETS];
    int count;
    int row_offset;
    int first;
    int reserved;
};

// The caller's explicit geometry against the kernel that was chosen: block and shared memory must fit it, the grid is a
// whole number of clusters.  Returns the number of CTAs to launch at most (0 = the caller has no say).
int explicit_ctas(const char *op, const gpurs_launch_config *launch, int cta_group, uint32_t threads, uint32_t shared_bytes, uint64_t &ctas) {
    ctas = 0;
    if (!launch) return GPURS_OK;
    const uint64_t grid = uint64_t(launch->grid[0] ? launch->grid[0] : 1) * (launch->grid[1] ? launch->grid[1] : 1) * (launch->grid[2] ? launch->grid[2] : 1);
    if (launch->grid[0] == 0) return fail(op, GPURS_E_INVALID_VIEW, "empty launch geometry");
    if (grid % uint64_t(cta_group) || grid > 0x7fffffffull) return fail(op, GPURS_E_INVALID_VIEW, "the grid must be a whole number of clusters");
    if (launch->block[0] != 0 && (launch->block[0] != threads || launch->block[1] > 1 || launch->block[2] > 1))
        return fail(op, GPURS_E_INVALID_VIEW, "the block size differs from the kernel's thread count");
    if (launch->shared_bytes != 0 && launch->shared_bytes < shared_bytes)
        return fail(op, GPURS_E_INVALID_VIEW, "less shared memory than the kernel needs");
    if (launch->shared_bytes > 232448) return fail(op, GPURS_E_INVALID_VIEW, "more shared memory than a CTA may have");
    if (launch->cluster[0] > 1 && int(launch->cluster[0]) != cta_group) return fail(op, GPURS_E_INVALID_VIEW, "the cluster size differs from the tile algorithm's");
    if (launch->cluster[1] > 1 || launch->cluster[2] > 1) return fail(op, GPURS_E_INVALID_VIEW, "clusters are one-dimensional");
    ctas = grid;
    return GPURS_OK;
}

// Dynamic shared memory of the tile kernel a Gemm selects.
uint32_t shared_for(const launcher::Gemm &g) {
    if (g.metadata != 0) return uint32_t(g.gather ? gemm::SPARSE_SHARED_PAIR_PUSH : g.cta_group == 2 ? gemm::SPARSE_SHARED_PAIR : gemm::SPARSE_SHARED_SINGLE);
    return g.cta_group == 2 ? gemm::SharedLayout<gemm::BLOCK_N, 2, gemm::STAGES_PAIR>::DYNAMIC_BYTES
                            : gemm::SharedLayout<gemm::BLOCK_N, 1, gemm::STAGES_SINGLE>::DYNAMIC_BYTES;
}

// Half-open byte ranges [begin, end) overlap?
bool overlap(uint64_t a, uint64_t a_bytes, uint64_t b, uint64_t b_bytes) { return a < b + b_bytes && b < a + a_bytes; }

}  // namespace

using launcher::Gemm;

namespace {

// How a dense or promoted tile product divides its tiles over the grid: which tiles (if any) are split along K.
struct SplitPlan {
    uint64_t all_tiles, wanted_ctas, grid_clusters;
    int depth_blocks, split_tiles;
    bool promoted_kernel;
    gemm::StreamSchedule schedule;
    // scratch for the parts of the split tiles
    size_t partial_bytes(int cta_group) const {
        return split_tiles > 0 ? size_t(schedule.split_tiles) * gemm::max_contributors(schedule) * (size_t(gemm::BLOCK_M) * cta_group) * gemm::BLOCK_N * 4 : 0;
    }
};

SplitPlan plan_split(const gpurs_gpu *gpu, const Gemm &g, uint64_t explicit_grid, uint64_t tile_columns = 0) {
    SplitPlan plan;
    const int cta_group = g.cta_group;
    const uint64_t eb = uint64_t(g.element_bytes);
    const bool batched = g.batches > 1;
    const uint64_t tile_rows = uint64_t(gemm::BLOCK_M) * cta_group;
    const bool sparse = g.metadata != 0;       // 224-column tiles, stages of 128 logical K
    const uint64_t block_n = tile_columns ? tile_columns : sparse ? uint64_t(gemm::SPARSE_BLOCK_N) : uint64_t(gemm::BLOCK_N);
    const uint64_t all_tiles = ((g.m + tile_rows - 1) / tile_rows) * ((g.n + block_n - 1) / block_n);
    const uint64_t wanted_ctas = explicit_grid ? explicit_grid : g.max_ctas > 0 ? uint64_t(g.max_ctas) : uint64_t(gpu->multiprocessors);
    const uint64_t full_clusters = std::max<uint64_t>(1, wanted_ctas / cta_group);
    uint64_t grid_clusters = std::min(full_clusters, std::max<uint64_t>(all_tiles, 1));
    const int depth_blocks = sparse ? int((g.k + gemm::SPARSE_BLOCK_K - 1) / gemm::SPARSE_BLOCK_K) : int((g.k * eb + gemm::ROW_BYTES - 1) / gemm::ROW_BYTES);
    const bool promoted_kernel = !sparse && g.threads == gemm::SCALED_THREADS;      // promotes every K-block to registers: same schedule
    const bool may_split = !g.whole_tiles && !batched && !g.gather && (g.threads == gemm::NUM_THREADS || promoted_kernel) && all_tiles <= 0x7fffffffull;
    int split_tiles = may_split ? gemm::stream_split_tiles(int(all_tiles), depth_blocks, int(grid_clusters), g.force_split) : 0;
    // Fewer tiles than CTA groups and a deep K (the reference's SplitDepth case, crates/gpurs/src/gpu/tensor/schedule): every tile
    // is split along K among up to STREAM_MAX_SHARE groups, which the same schedule expresses as "all tiles belong to the split
    // round".  It must pay for the parts' trip through memory (about 30 K-blocks' time, as above).
    if (may_split && split_tiles == 0 && !explicit_grid && all_tiles > 0 && all_tiles * 2 <= full_clusters && depth_blocks >= 2) {
        const uint64_t shares = std::min<uint64_t>(std::min<uint64_t>(gemm::STREAM_MAX_SHARE, full_clusters / all_tiles), uint64_t(depth_blocks));
        const uint64_t saved = uint64_t(depth_blocks) - (uint64_t(depth_blocks) + shares - 1) / shares;
        if (shares >= 2 && (g.force_split || saved >= 40)) {
            split_tiles = int(all_tiles);
            grid_clusters = all_tiles * shares;
        }
    }
    plan.all_tiles = all_tiles, plan.wanted_ctas = wanted_ctas, plan.grid_clusters = grid_clusters;
    plan.depth_blocks = depth_blocks, plan.split_tiles = split_tiles, plan.promoted_kernel = promoted_kernel;
    plan.schedule = gemm::make_stream_schedule(int(std::min<uint64_t>(all_tiles, 0x7fffffff)), depth_blocks, int(grid_clusters), split_tiles);
    return plan;
}

}  // namespace

int launcher::launch_gemm(gpurs_stream *stream, const Gemm &g) {
    gpurs_gpu *gpu = stream->gpu;
    const int cta_group = g.cta_group;
    const uint64_t eb = uint64_t(g.element_bytes), ob = uint64_t(g.output_bytes);
    char name[96];
    const bool batched = g.batches > 1;
    // Stream-K: decided here from the tile count and the grid, by the same arithmetic the kernel uses to find its work.
    const uint64_t tile_rows_ = uint64_t(gemm::BLOCK_M) * cta_group;
    uint64_t explicit_grid = 0;
    {
        const int checked = explicit_ctas("gpurs_matmul", g.launch, cta_group, uint32_t(g.threads), shared_for(g), explicit_grid);
        if (checked != GPURS_OK) return checked;
    }
    const SplitPlan plan = plan_split(gpu, g, explicit_grid);
    const uint64_t all_tiles = plan.all_tiles, wanted_ctas = plan.wanted_ctas, grid_clusters = plan.grid_clusters;
    const int split_tiles = plan.split_tiles;
    const bool promoted_kernel = plan.promoted_kernel;
    const gemm::StreamSchedule schedule = plan.schedule;
    bool stream_k = split_tiles > 0;
    // 256 x 512 tiles (kernels/gemm_wide_tcgen05.cuh): a quarter less operand traffic from L2 per flop, which is what bounds the
    // 256 x 256 tiles.  Plain products on CTA pairs, n x k right operand, C rows on 16-byte boundaries.  By default they are used
    // where the tile count fills the rounds of the grid nearly as well as the square tiles do (a round of wide tiles is twice as
    // long; they are taken to be 7 % faster per flop when weighing rounds against each other).
    const bool algebra_ = g.bias || g.row_scale || g.column_scale || (g.alpha != 0.0f && g.alpha != 1.0f) || g.row_absmax || g.row_bias || g.residual ||
                          g.row_sum || g.accumulate;
    // the wide kernel's epilogue has the element-wise algebra (its `_ep` entries, float outputs), not the row reductions nor the
    // accumulation into C
    const bool unstaged_algebra = g.row_absmax || g.row_sum || g.accumulate || (algebra_ && g.output_type == GPURS_I32);
    bool wide = false;
    uint64_t wide_columns = 512;
    if (g.tile_width != 256 && !g.force_split && cta_group == 2 && g.metadata == 0 && g.threads == gemm::NUM_THREADS && !batched && !g.gather && !g.b_row_major &&
        !unstaged_algebra && g.element_type != GPURS_F32 && g.l2_policy == 0 && g.n > 256 && g.c % 16 == 0 && (g.ldc * ob) % 16 == 0 &&
        (!g.launch || g.launch->block[0] == 0)) {      // that kernel has its own block size
        const uint64_t wide_tiles = ((g.m + tile_rows_ - 1) / tile_rows_) * ((g.n + 511) / 512);
        const uint64_t pairs = std::max<uint64_t>(1, wanted_ctas / 2);
        // measured on bf16 8192^3 (14 rounds of square tiles against 7 of wide ones): +8.6 %; on f16 4096^3, where the square tiles'
        // last round is split along K (3.46 rounds) and wide tiles need 2 whole rounds for 1.73: -6 %
        const double square_cost = stream_k ? double(all_tiles) / double(pairs) + 0.15 : double((all_tiles + grid_clusters - 1) / std::max<uint64_t>(grid_clusters, 1));
        const double wide_cost = 2.0 * 0.93 * double((wide_tiles + pairs - 1) / pairs);
        // (a single partial round of wide tiles counts as a whole one: 64 wide tiles on 74 pairs, the 1024-row shard of int8
        // 8192^3, measured 49.2 us against 51.1 us for 128 square tiles with the last round split along K)
        wide = g.tile_width == 512 || (all_tiles > pairs && wide_cost <= square_cost);
        if (wide_tiles > 0x7fffffffull) wide = false;
        // 256 x 480 tiles (second half 224 columns; 32-bit outputs, no output algebra) where they need fewer rounds x columns than
        // the 512-wide ones: 8192 columns on 1024 rows are 64 tiles of 512 for 74 pairs, one round either way, or 72 of 480
        if (wide && g.tile_width != 512 && g.output_bytes == 4 && !algebra_) {
            const uint64_t narrower_tiles = ((g.m + tile_rows_ - 1) / tile_rows_) * ((g.n + 479) / 480);
            if (480 * ((narrower_tiles + pairs - 1) / pairs) < 512 * ((wide_tiles + pairs - 1) / pairs)) wide_columns = 480;
        }
    }
    if (wide) stream_k = false;
    // 512 x 224 tiles of the 2:4-sparse product (kernels/gemm_sparse_tall_tcgen05.cuh): B, most of the sparse kernel's operand
    // traffic, is fetched once for two row blocks.  Used where they fill the grid's rounds no worse than the 256-row tiles do,
    // for plain products (that kernel has no output algebra) without an explicit launch geometry (it has its own block size).
    bool tall = false;
    if (g.metadata != 0 && cta_group == 2 && !g.gather && g.tile_width != 256 && !algebra_ && !g.launch) {
        const uint64_t columns = (g.n + gemm::SPARSE_BLOCK_N - 1) / gemm::SPARSE_BLOCK_N;
        const uint64_t pairs = std::max<uint64_t>(1, wanted_ctas / 2);
        const uint64_t short_rounds = (((g.m + 255) / 256) * columns + pairs - 1) / pairs, tall_rounds = (((g.m + 511) / 512) * columns + pairs - 1) / pairs;
        tall = g.tile_width == 512 || (!g.force_split && g.m > 256 && 2.0 * 0.8 * double(tall_rounds) <= double(short_rounds));
    }
    if (tall) stream_k = false;
    // The dense tile kernels come without and with the output algebra compiled in ("_ep"): a plain product runs the lean entry.
    const bool algebra = g.bias || g.row_scale || g.column_scale || (g.alpha != 0.0f && g.alpha != 1.0f) || g.row_absmax || g.row_bias || g.residual ||
                         g.row_sum || g.accumulate;
    const bool dense_tile = g.metadata == 0 && g.threads == gemm::NUM_THREADS;
    const char *form = g.gather ? "%s_push_cg%d" : batched ? "%s_batched_cg%d" : tall ? "%s_t512_cg%d" : wide ? (wide_columns == 480 ? "%s_w480_cg%d" : algebra ? "%s_w512_ep_cg%d" : "%s_w512_cg%d") : stream_k ? ((algebra && dense_tile) ? "%s_sk_ep_cg%d" : "%s_sk_cg%d")
                       : (algebra && dense_tile) ? "%s_ep_cg%d" : "%s_cg%d";
    std::snprintf(name, sizeof name, form, g.stem, cta_group);
    const bool sparse = g.metadata != 0;
    const uint32_t shared_bytes = std::max(wide ? uint32_t(gemm::WIDE_SHARED) : tall ? uint32_t(gemm::SPARSE_TALL_SHARED) : shared_for(g), g.launch ? g.launch->shared_bytes : 0u);
    gpurs_kernel *kernel = nullptr;
    int result = runtime::builtin_kernel(gpu, name, shared_bytes, &kernel);
    if (result != GPURS_OK) return result;

    // The two operand descriptors: rows of 128 bytes of K, 128-byte swizzle, out-of-range reads as
    // zero, the same form the reference encodes (crates/driver/src/memory.rs:325-354) with boxes of
    // 128 rows of A and 256 (or, per CTA of a pair, 128) rows of B.
    const uint32_t block_k = uint32_t(gemm::ROW_BYTES / g.element_bytes);
    alignas(64) CUtensorMap map_a, map_b, map_e;
    // A sparse A is stored as its kept half: k/2 values per row.
    const uint64_t dims_a[2] = {sparse ? g.k / 2 : g.k, g.m};
    const uint64_t stride_a[1] = {g.lda * eb}, stride_b[1] = {g.ldb * eb};
    const uint32_t box_a[2] = {block_k, uint32_t(gemm::BLOCK_M)};
    // B as n x k: one box of (128 bytes of k) x (the tile's rows of n).  B as k x n: boxes of (128 bytes of n) x (block_k rows of k).
    // columns of one tile: 256, or 224 for the sparse kernels (two accumulators plus metadata in tensor memory)
    const uint64_t block_n = sparse ? uint64_t(gemm::SPARSE_BLOCK_N) : wide ? wide_columns : uint64_t(gemm::BLOCK_N);
    uint64_t dims_b[2] = {g.k, g.n};
    uint32_t box_b[2] = {block_k, wide ? 128u : uint32_t(block_n / cta_group)};      // wide tiles: the CTA's 128 rows of either half
    if (g.b_row_major) {
        dims_b[0] = g.n, dims_b[1] = g.k;
        box_b[0] = uint32_t(gemm::ROW_BYTES / g.element_bytes), box_b[1] = block_k;
    }
    if (batched) {
        // rank 3: (k, rows, batch), boxes one matrix deep; rows beyond a matrix read as zero, not as the next matrix
        const uint64_t dims_a3[3] = {g.k, g.m, g.batches}, dims_b3[3] = {g.k, g.n, g.batches};
        const uint64_t stride_a3[2] = {g.lda * eb, g.stride_a * eb}, stride_b3[2] = {g.ldb * eb, g.stride_b * eb};
        const uint32_t box_a3[3] = {box_a[0], box_a[1], 1}, box_b3[3] = {box_b[0], box_b[1], 1};
        result = gpurs_tensor_map_encode(gpu, &map_a, g.element_type, 3, g.a, dims_a3, stride_a3, box_a3, 3, 3);
        if (result != GPURS_OK) return result;
        result = gpurs_tensor_map_encode(gpu, &map_b, g.element_type, 3, g.b, dims_b3, stride_b3, box_b3, 3, 3);
        if (result != GPURS_OK) return result;
    } else {
        result = gpurs_tensor_map_encode(gpu, &map_a, g.element_type, 2, g.a, dims_a, stride_a, box_a, 3, 3);
        if (result != GPURS_OK) return result;
        result = gpurs_tensor_map_encode(gpu, &map_b, g.element_type, 2, g.b, dims_b, stride_b, box_b, 3, 3);
        if (result != GPURS_OK) return result;
    }

    if (sparse) {
        // The metadata as rows of 16 bytes, 128 rows per block, no swizzle: block (row block, K block) starts at
        // row (row_block * k_blocks + k_block) * 128.
        const uint64_t blocks = ((g.m + 127) / 128) * ((g.k + gemm::SPARSE_BLOCK_K - 1) / gemm::SPARSE_BLOCK_K);
        const uint64_t dims_e[2] = {16, blocks * 128}, stride_e[1] = {16};
        const uint32_t box_e[2] = {16, 128};
        result = gpurs_tensor_map_encode(gpu, &map_e, GPURS_I8, 2, g.metadata, dims_e, stride_e, box_e, 0, 3);
        if (result != GPURS_OK) return result;
    }

    gemm::Params params;
    std::memset(&params, 0, sizeof params);
    params.c = reinterpret_cast<void *>(g.c);
    params.ldc = (long long)g.ldc;
    params.m = int(g.m);
    params.n = int(g.n);
    params.k = int(g.k);
    const uint64_t tile_rows = tall ? 512 : uint64_t(gemm::BLOCK_M) * cta_group;
    params.tiles_m = int((g.m + tile_rows - 1) / tile_rows);
    params.tiles_n = int((g.n + block_n - 1) / block_n);
    // Bands of 2048 rows by default: with one tile per SM in flight, the tiles running together then
    // cover about 2048 x 2304 outputs, a near-square patch whose A and B panels are shared through L2.
    params.raster_rows = g.raster_rows > 0 ? g.raster_rows : 16 / cta_group;
    params.vector_stores = (g.c % 16 == 0 && (g.ldc * ob) % 16 == 0 && (!batched || (g.stride_c * ob) % 16 == 0)) ? 1 : 0;
    params.batches = int(g.batches);
    params.batch_stride_c = (long long)g.stride_c;
    params.status = reinterpret_cast<unsigned int *>(gpu->status);
    params.scale_a = reinterpret_cast<const float *>(g.scale_a);
    params.scale_b = reinterpret_cast<const float *>(g.scale_b);
    params.l2_policy = g.l2_policy;
    params.b_row_major = g.b_row_major ? 1 : 0;
    params.bias = reinterpret_cast<const float *>(g.bias);
    params.row_scale = reinterpret_cast<const float *>(g.row_scale);
    params.column_scale = reinterpret_cast<const float *>(g.column_scale);
    params.alpha = g.alpha;
    params.scaled_by_alpha = (g.alpha != 0.0f && g.alpha != 1.0f) ? 1 : 0;
    params.row_absmax = reinterpret_cast<float *>(g.row_absmax);
    params.row_bias = reinterpret_cast<const float *>(g.row_bias);
    params.residual = reinterpret_cast<const void *>(g.residual);
    params.ldr = (long long)g.ldr;
    params.beta = g.beta;
    params.row_sum = reinterpret_cast<float *>(g.row_sum);
    params.accumulate = g.accumulate ? 1 : 0;

    const uint64_t tiles = uint64_t(params.tiles_m) * uint64_t(params.tiles_n) * g.batches;
    if (tiles > 0x7fffffffull) return fail("gpurs_matmul", GPURS_E_SIZE_OVERFLOW, "too many tiles");
    uint64_t ctas = wanted_ctas;
    uint64_t clusters = std::max<uint64_t>(1, ctas / cta_group);
    clusters = stream_k ? grid_clusters : std::min(clusters, tiles);      // a split round may use more groups than there are tiles
    gpurs_launch_config config;
    std::memset(&config, 0, sizeof config);
    config.grid[0] = uint32_t(clusters * cta_group);
    config.grid[1] = config.grid[2] = 1;
    config.block[0] = tall ? uint32_t(gemm::SPARSE_TALL_NUM_THREADS) : wide ? uint32_t(gemm::WIDE_NUM_THREADS) : uint32_t(g.threads);
    config.block[1] = config.block[2] = 1;
    config.shared_bytes = shared_bytes;
    config.cluster[0] = uint32_t(cta_group);
    config.cluster[1] = config.cluster[2] = 1;
    // The dense tile kernels also take a descriptor of C: boxes of 32 rows x 128 bytes for their TMA-store epilogue
    // (used when every row of C starts on a 16-byte boundary; otherwise the descriptor is ignored).
    const bool takes_output_map = !sparse && g.threads == gemm::NUM_THREADS;
    alignas(64) CUtensorMap map_c;
    std::memset(&map_c, 0, sizeof map_c);
    if (takes_output_map && params.vector_stores == 1) {
        const uint64_t dims_c[3] = {g.n, g.m, g.batches}, stride_c[2] = {g.ldc * ob, g.stride_c * ob};
        const uint32_t box_c[3] = {uint32_t(gemm::ROW_BYTES / g.output_bytes), 32, 1};
        result = gpurs_tensor_map_encode(gpu, &map_c, g.output_type, batched ? 3 : 2, g.c, dims_c, stride_c, box_c, 3, 3);
        if (result != GPURS_OK) return result;
    }
    if (g.gather && sparse) {
        // as below, with a second, unswizzled descriptor per GPU for the 32-column box that ends a 224-column tile
        SparsePushTargets targets;
        std::memset(&targets, 0, sizeof targets);
        const uint64_t pitch = g.gather->ld_full ? g.gather->ld_full : g.n;
        const uint64_t dims_c[2] = {g.n, g.gather->total_rows}, stride_c[1] = {pitch * ob};
        const uint32_t box_c[2] = {64, 32}, half_box_c[2] = {32, 32};
        for (uint32_t t = 0; t < g.gather->world; t++) {
            result = gpurs_tensor_map_encode(gpu, &targets.maps[t], g.output_type, 2, g.gather->full[t], dims_c, stride_c, box_c, 3, 3);
            if (result != GPURS_OK) return result;
            result = gpurs_tensor_map_encode(gpu, &targets.half_maps[t], g.output_type, 2, g.gather->full[t], dims_c, stride_c, half_box_c, 0, 3);
            if (result != GPURS_OK) return result;
        }
        targets.count = int(g.gather->world);
        targets.row_offset = int(g.gather->row_offset);
        targets.first = int((g.gather->rank + 1) % g.gather->world);
        void *push_arguments[5] = {&map_a, &map_b, &map_e, &targets, &params};
        return runtime::launch(kernel, stream, &config, push_arguments, true);
    }
    if (g.gather) {
        // One descriptor of the whole gathered matrix per GPU; the kernel stores each box of its block to all of them.
        PushTargets targets;
        std::memset(&targets, 0, sizeof targets);
        const uint64_t pitch = g.gather->ld_full ? g.gather->ld_full : g.n;
        const uint64_t dims_c[2] = {g.n, g.gather->total_rows}, stride_c[1] = {pitch * ob};
        const uint32_t box_c[2] = {uint32_t(gemm::ROW_BYTES / g.output_bytes), 32};
        for (uint32_t t = 0; t < g.gather->world; t++) {
            result = gpurs_tensor_map_encode(gpu, &targets.maps[t], g.output_type, 2, g.gather->full[t], dims_c, stride_c, box_c, 3, 3);
            if (result != GPURS_OK) return result;
        }
        targets.count = int(g.gather->world);
        targets.row_offset = int(g.gather->row_offset);
        targets.first = int((g.gather->rank + 1) % g.gather->world);
        void *push_arguments[4] = {&map_a, &map_b, &targets, &params};
        return runtime::launch(kernel, stream, &config, push_arguments, true);
    }
    if (stream_k) {
        // scratch for the partial tiles and their arrival counters, borrowed from the handle for this launch
        const int most = gemm::max_contributors(schedule);
        const size_t partial_bytes = plan.partial_bytes(cta_group);
        CUdeviceptr partials = g.partials, counters = 0;
        const bool borrowed_here = partials == 0;       // a caller that holds the workspace already passes its own room for the parts
        if (!borrowed_here && g.partials_bytes < partial_bytes) return fail("gpurs_matmul", GPURS_E_INVALID_ARGUMENT, "too little room for the partial tiles");
        if (borrowed_here) result = runtime::workspace_acquire(stream, partial_bytes, &partials);
        if (result != GPURS_OK) return result;
        // one arrival counter per tile and warp that finishes rows of it: 4 epilogue warps per CTA, 8 promotion warps
        result = runtime::turns_acquire(stream, std::max<size_t>(size_t(schedule.split_tiles) * (promoted_kernel ? 8 : 4) * cta_group * sizeof(uint32_t), 4096), &counters);
        if (result != GPURS_OK) {
            if (borrowed_here) runtime::workspace_release(stream);     // nothing was enqueued: the next borrower need not wait for this one
            return result;
        }
        params.partials = reinterpret_cast<void *>(partials);
        params.split_counters = reinterpret_cast<unsigned int *>(counters);
        params.max_contributors = most;
        params.split_tiles = split_tiles;
        void *stream_arguments[4] = {&map_a, &map_b, &map_c, &params};
        void *promoted_arguments[3] = {&map_a, &map_b, &params};
        void *sparse_stream_arguments[4] = {&map_a, &map_b, &map_e, &params};
        result = runtime::launch(kernel, stream, &config, sparse ? sparse_stream_arguments : promoted_kernel ? promoted_arguments : stream_arguments, true);
        const int released = borrowed_here ? runtime::workspace_release(stream) : GPURS_OK, turned = runtime::turns_release(stream);
        return result != GPURS_OK ? result : released != GPURS_OK ? released : turned;
    }
    void *arguments[3] = {&map_a, &map_b, &params};
    void *dense_arguments[4] = {&map_a, &map_b, &map_c, &params};
    void *sparse_arguments[4] = {&map_a, &map_b, &map_e, &params};
    return runtime::launch(kernel, stream, &config, sparse ? sparse_arguments : takes_output_map ? dense_arguments : arguments, true);
}

namespace {

using launcher::launch_gemm;

// The FP8 product with the tensor core's own block scaling (kernels/gemm_mx_tcgen05.cuh): operand descriptors as for the
// dense kernels (224-row boxes of B), plus the two tiled scale arrays as rows of 16 bytes.
int launch_mx(gpurs_stream *stream, const launcher::Gemm &g) {
    gpurs_gpu *gpu = stream->gpu;
    const int cta_group = g.cta_group;
    const uint32_t shared_bytes = uint32_t(cta_group == 2 ? gemm::MX_SHARED_PAIR : gemm::MX_SHARED_SINGLE);
    uint64_t explicit_grid = 0;
    int result = explicit_ctas("gpurs_matmul", g.launch, cta_group, uint32_t(gemm::NUM_THREADS), shared_bytes, explicit_grid);
    if (result != GPURS_OK) return result;
    // the schedule of the dense kernels on this kernel's 224-column tiles: the last round, or every tile of a small deep product,
    // split along K
    const SplitPlan plan = plan_split(gpu, g, explicit_grid, gemm::MX_BLOCK_N);
    const bool stream_k = plan.split_tiles > 0;
    char name[96];
    std::snprintf(name, sizeof name, stream_k ? "%s_sk_cg%d" : "%s_cg%d", g.stem, cta_group);
    gpurs_kernel *kernel = nullptr;
    result = runtime::builtin_kernel(gpu, name, shared_bytes, &kernel);
    if (result != GPURS_OK) return result;
    const uint64_t tile_rows = uint64_t(gemm::BLOCK_M) * cta_group;
    const uint64_t k_blocks = (g.k + 127) / 128, tiles_m = (g.m + tile_rows - 1) / tile_rows, tiles_n = (g.n + gemm::MX_BLOCK_N - 1) / gemm::MX_BLOCK_N;
    alignas(64) CUtensorMap map_a, map_b, map_sa, map_sb;
    const uint64_t dims_a[2] = {g.k, g.m}, dims_b[2] = {g.k, g.n}, stride_a[1] = {g.lda}, stride_b[1] = {g.ldb};
    const uint32_t box_a[2] = {128, uint32_t(gemm::BLOCK_M)}, box_b[2] = {128, uint32_t(gemm::MX_BLOCK_N / cta_group)};
    result = gpurs_tensor_map_encode(gpu, &map_a, GPURS_E4M3, 2, g.a, dims_a, stride_a, box_a, 3, 3);
    if (result != GPURS_OK) return result;
    result = gpurs_tensor_map_encode(gpu, &map_b, GPURS_E4M3, 2, g.b, dims_b, stride_b, box_b, 3, 3);
    if (result != GPURS_OK) return result;
    const uint64_t dims_sa[2] = {16, ((g.m + 127) / 128) * k_blocks * 32}, dims_sb[2] = {16, tiles_n * k_blocks * 64}, stride_s[1] = {16};
    const uint32_t box_sa[2] = {16, 32}, box_sb[2] = {16, 64};
    result = gpurs_tensor_map_encode(gpu, &map_sa, GPURS_I8, 2, g.scale_a, dims_sa, stride_s, box_sa, 0, 3);
    if (result != GPURS_OK) return result;
    result = gpurs_tensor_map_encode(gpu, &map_sb, GPURS_I8, 2, g.scale_b, dims_sb, stride_s, box_sb, 0, 3);
    if (result != GPURS_OK) return result;

    gemm::Params params;
    std::memset(&params, 0, sizeof params);
    params.c = reinterpret_cast<void *>(g.c);
    params.ldc = (long long)g.ldc;
    params.m = int(g.m), params.n = int(g.n), params.k = int(g.k);
    params.tiles_m = int(tiles_m), params.tiles_n = int(tiles_n);
    params.raster_rows = g.raster_rows > 0 ? g.raster_rows : 16 / cta_group;
    params.vector_stores = (g.c % 16 == 0 && (g.ldc * uint64_t(g.output_bytes)) % 16 == 0) ? 1 : 0;
    params.status = reinterpret_cast<unsigned int *>(gpu->status);
    params.bias = reinterpret_cast<const float *>(g.bias);
    params.row_scale = reinterpret_cast<const float *>(g.row_scale);
    params.column_scale = reinterpret_cast<const float *>(g.column_scale);
    params.alpha = g.alpha;
    params.scaled_by_alpha = (g.alpha != 0.0f && g.alpha != 1.0f) ? 1 : 0;
    params.row_bias = reinterpret_cast<const float *>(g.row_bias);
    params.residual = reinterpret_cast<const void *>(g.residual);
    params.ldr = (long long)g.ldr;
    params.beta = g.beta;
    params.accumulate = g.accumulate ? 1 : 0;
    const uint64_t tiles = tiles_m * tiles_n;
    if (tiles > 0x7fffffffull) return fail("gpurs_matmul", GPURS_E_SIZE_OVERFLOW, "too many tiles");
    const uint64_t ctas = explicit_grid ? explicit_grid : g.max_ctas > 0 ? uint64_t(g.max_ctas) : uint64_t(gpu->multiprocessors);
    gpurs_launch_config config;
    std::memset(&config, 0, sizeof config);
    const uint64_t clusters = stream_k ? plan.grid_clusters : std::min(std::max<uint64_t>(1, ctas / cta_group), tiles);
    config.grid[0] = uint32_t(clusters * cta_group);
    config.block[0] = uint32_t(gemm::NUM_THREADS);
    config.shared_bytes = shared_bytes;
    config.cluster[0] = uint32_t(cta_group);
    config.cluster[1] = config.cluster[2] = 1;
    void *arguments[5] = {&map_a, &map_b, &map_sa, &map_sb, &params};
    if (!stream_k) return runtime::launch(kernel, stream, &config, arguments, true);
    // scratch for the partial tiles and their arrival counters, borrowed from the handle for this launch
    CUdeviceptr partials = 0, counters = 0;
    result = runtime::workspace_acquire(stream, plan.partial_bytes(cta_group), &partials);
    if (result != GPURS_OK) return result;
    result = runtime::turns_acquire(stream, std::max<size_t>(size_t(plan.schedule.split_tiles) * 4 * cta_group * sizeof(uint32_t), 4096), &counters);
    if (result != GPURS_OK) {
        runtime::workspace_release(stream);
        return result;
    }
    params.partials = reinterpret_cast<void *>(partials);
    params.split_counters = reinterpret_cast<unsigned int *>(counters);
    params.max_contributors = gemm::max_contributors(plan.schedule);
    params.split_tiles = plan.split_tiles;
    result = runtime::launch(kernel, stream, &config, arguments, true);
    const int released = runtime::workspace_release(stream), turned = runtime::turns_release(stream);
    return result != GPURS_OK ? result : released != GPURS_OK ? released : turned;
}

// The block-scaled FP8 product on CTA pairs (kernels/gemm_blockscaled_tcgen05.cuh): 256 x 256 tiles, every K-block issued as two
// products of 128 columns.  Each CTA loads its 128 rows of A and, of each 128-column half of the B tile, its 64 rows.
int launch_blockscaled(gpurs_stream *stream, const launcher::Gemm &g) {
    gpurs_gpu *gpu = stream->gpu;
    const uint32_t shared_bytes = std::max(uint32_t(gemm::BLOCKSCALED_SHARED), g.launch ? g.launch->shared_bytes : 0u);
    uint64_t explicit_grid = 0;
    int result = explicit_ctas("gpurs_matmul", g.launch, 2, uint32_t(gemm::SCALED_THREADS), uint32_t(gemm::BLOCKSCALED_SHARED), explicit_grid);
    if (result != GPURS_OK) return result;
    char name[96];
    std::snprintf(name, sizeof name, "%s_cg2", g.stem);
    gpurs_kernel *kernel = nullptr;
    result = runtime::builtin_kernel(gpu, name, shared_bytes, &kernel);
    if (result != GPURS_OK) return result;
    const uint64_t ob = uint64_t(g.output_bytes);
    alignas(64) CUtensorMap map_a, map_b, map_c;
    const uint64_t dims_a[2] = {g.k, g.m}, dims_b[2] = {g.k, g.n}, stride_a[1] = {g.lda}, stride_b[1] = {g.ldb};
    const uint32_t box_a[2] = {128, uint32_t(gemm::BLOCK_M)}, box_b[2] = {128, 64};
    result = gpurs_tensor_map_encode(gpu, &map_a, GPURS_E4M3, 2, g.a, dims_a, stride_a, box_a, 3, 3);
    if (result != GPURS_OK) return result;
    result = gpurs_tensor_map_encode(gpu, &map_b, GPURS_E4M3, 2, g.b, dims_b, stride_b, box_b, 3, 3);
    if (result != GPURS_OK) return result;
    gemm::Params params;
    std::memset(&params, 0, sizeof params);
    params.c = reinterpret_cast<void *>(g.c);
    params.ldc = (long long)g.ldc;
    params.m = int(g.m), params.n = int(g.n), params.k = int(g.k);
    params.tiles_m = int((g.m + 255) / 256), params.tiles_n = int((g.n + 255) / 256);
    params.raster_rows = g.raster_rows > 0 ? g.raster_rows : 8;
    params.vector_stores = (g.c % 16 == 0 && (g.ldc * ob) % 16 == 0) ? 1 : 0;
    params.status = reinterpret_cast<unsigned int *>(gpu->status);
    params.scale_a = reinterpret_cast<const float *>(g.scale_a);
    params.scale_b = reinterpret_cast<const float *>(g.scale_b);
    params.bias = reinterpret_cast<const float *>(g.bias);
    params.row_scale = reinterpret_cast<const float *>(g.row_scale);
    params.column_scale = reinterpret_cast<const float *>(g.column_scale);
    params.alpha = g.alpha;
    params.scaled_by_alpha = (g.alpha != 0.0f && g.alpha != 1.0f) ? 1 : 0;
    params.row_bias = reinterpret_cast<const float *>(g.row_bias);
    params.residual = reinterpret_cast<const void *>(g.residual);
    params.ldr = (long long)g.ldr;
    params.beta = g.beta;
    std::memset(&map_c, 0, sizeof map_c);
    if (params.vector_stores == 1) {
        const uint64_t dims_c[2] = {g.n, g.m}, stride_c[1] = {g.ldc * ob};
        const uint32_t box_c[2] = {uint32_t(gemm::ROW_BYTES / g.output_bytes), 32};
        result = gpurs_tensor_map_encode(gpu, &map_c, g.output_type, 2, g.c, dims_c, stride_c, box_c, 3, 3);
        if (result != GPURS_OK) return result;
    }
    const uint64_t tiles = uint64_t(params.tiles_m) * uint64_t(params.tiles_n);
    if (tiles > 0x7fffffffull) return fail("gpurs_matmul", GPURS_E_SIZE_OVERFLOW, "too many tiles");
    const uint64_t ctas = explicit_grid ? explicit_grid : g.max_ctas > 0 ? uint64_t(g.max_ctas) : uint64_t(gpu->multiprocessors);
    const uint64_t pairs = std::min(std::max<uint64_t>(1, ctas / 2), tiles);
    // the kernel numbers the 128-column products of one CTA pair with 32 bits
    if (((tiles + pairs - 1) / pairs) * ((g.k + 127) / 128) * 2 > 0xffffffffull) return fail("gpurs_matmul", GPURS_E_SIZE_OVERFLOW, "too many K-blocks per CTA pair");
    gpurs_launch_config config;
    std::memset(&config, 0, sizeof config);
    config.grid[0] = uint32_t(pairs * 2);
    config.block[0] = uint32_t(gemm::SCALED_THREADS);
    config.shared_bytes = shared_bytes;
    config.cluster[0] = 2;
    config.cluster[1] = config.cluster[2] = 1;
    void *arguments[4] = {&map_a, &map_b, &map_c, &params};
    return runtime::launch(kernel, stream, &config, arguments, true);
}

// Host mirror of gemm::SkinnyParams (kernels/gemm_skinny_tcgen05.cuh).
struct SkinnyParams {
    float *c;
    long long ldc;
    const float *bias;
    unsigned int *turns;
    float *partials;
    unsigned int *status;
    int m, n, k, tiles, splits, k_blocks_per_split;
};

// The decode-shaped product: m <= 64 rows of A against all of B, K split among CTAs, ordered reduction.
int launch_skinny(gpurs_stream *stream, const launcher::Gemm &g) {
    gpurs_gpu *gpu = stream->gpu;
    const int tokens = g.m <= 16 ? 16 : (g.m <= 32 ? 32 : 64);
    char name[96];
    std::snprintf(name, sizeof name, "gpurs_gemm_skinny_%s_f32_t%d", g.element_type == GPURS_F16 ? "f16" : "bf16", tokens);
    const uint32_t shared_bytes = uint32_t(gemm::skinny_shared_bytes(tokens));
    gpurs_kernel *kernel = nullptr;
    int result = runtime::builtin_kernel(gpu, name, shared_bytes, &kernel);
    if (result != GPURS_OK) return result;
    alignas(64) CUtensorMap map_big, map_small;
    const uint64_t dims_big[2] = {g.k, g.n}, dims_small[2] = {g.k, g.m};
    const uint64_t stride_big[1] = {g.ldb * 2}, stride_small[1] = {g.lda * 2};
    const uint32_t box_big[2] = {64, uint32_t(gemm::BLOCK_M)}, box_small[2] = {64, uint32_t(tokens)};
    result = gpurs_tensor_map_encode(gpu, &map_big, g.element_type, 2, g.b, dims_big, stride_big, box_big, 3, 3);
    if (result != GPURS_OK) return result;
    result = gpurs_tensor_map_encode(gpu, &map_small, g.element_type, 2, g.a, dims_small, stride_small, box_small, 3, 3);
    if (result != GPURS_OK) return result;

    SkinnyParams params;
    std::memset(&params, 0, sizeof params);
    params.c = reinterpret_cast<float *>(g.c);
    params.ldc = (long long)g.ldc;
    params.bias = reinterpret_cast<const float *>(g.bias);
    params.status = reinterpret_cast<unsigned int *>(gpu->status);
    params.m = int(g.m), params.n = int(g.n), params.k = int(g.k);
    params.tiles = int((g.n + gemm::BLOCK_M - 1) / gemm::BLOCK_M);
    // One CTA per multiprocessor at most (each keeps 8 stages in flight), each with a whole number of 64-deep K-blocks.
    const int k_blocks = int((g.k + 63) / 64);
    const int ctas = g.max_ctas > 0 ? g.max_ctas : gpu->multiprocessors;
    int splits = std::max(1, std::min(k_blocks, ctas / params.tiles));
    params.k_blocks_per_split = (k_blocks + splits - 1) / splits;
    splits = (k_blocks + params.k_blocks_per_split - 1) / params.k_blocks_per_split;   // no empty trailing split
    params.splits = splits;
    CUdeviceptr turns = 0, partials = 0;
    if (splits > 1) {
        result = runtime::turns_acquire(stream, size_t(gemm::SKINNY_MAX_TILES) * 4 * sizeof(unsigned int), &turns);
        if (result != GPURS_OK) return result;
        result = runtime::workspace_acquire(stream, size_t(params.tiles) * splits * tokens * gemm::BLOCK_M * sizeof(float), &partials);
        if (result != GPURS_OK) {
            runtime::turns_release(stream);
            return result;
        }
    }
    params.turns = reinterpret_cast<unsigned int *>(turns);
    params.partials = reinterpret_cast<float *>(partials);
    gpurs_launch_config config;
    std::memset(&config, 0, sizeof config);
    config.grid[0] = uint32_t(params.tiles) * uint32_t(splits);
    config.block[0] = gemm::NUM_THREADS;
    config.shared_bytes = shared_bytes;
    void *arguments[3] = {&map_big, &map_small, &params};
    result = runtime::launch(kernel, stream, &config, arguments, true);
    if (splits > 1) {
        const int released = runtime::turns_release(stream), freed = runtime::workspace_release(stream);
        if (result == GPURS_OK) result = released != GPURS_OK ? released : freed;
    }
    return result;
}

// Enqueues the hi/lo split of a rows x k fp32 matrix into a rows x 3k one (kernels/transform.cu).
int split_tf32(gpurs_stream *stream, gpurs_device_ptr source, uint64_t pitch, gpurs_device_ptr destination, uint64_t rows, uint64_t k, int order) {
    gpurs_gpu *gpu = stream->gpu;
    gpurs_kernel *kernel = nullptr;
    int result = runtime::builtin_kernel(gpu, "gpurs_split_tf32", 0, &kernel);
    if (result != GPURS_OK) return result;
    const uint64_t quads = rows * (k / 4);
    gpurs_launch_config config;
    std::memset(&config, 0, sizeof config);
    // a whole number of waves: up to 8 blocks of 256 threads per multiprocessor
    const uint64_t blocks = std::min<uint64_t>((quads + 255) / 256, uint64_t(gpu->multiprocessors) * 8);
    config.grid[0] = uint32_t(std::max<uint64_t>(1, blocks));
    config.block[0] = 256;
    const void *source_pointer = reinterpret_cast<const void *>(source);
    void *destination_pointer = reinterpret_cast<void *>(destination);
    long long source_pitch = (long long)pitch;
    int row_count = int(rows), depth = int(k);
    void *arguments[6] = {&source_pointer, &source_pitch, &destination_pointer, &row_count, &depth, &order};
    return runtime::launch(kernel, stream, &config, arguments, true);
}

// Both operands (n x k right operand) in one launch.
int split_tf32_pair(gpurs_stream *stream, gpurs_device_ptr left, uint64_t left_pitch, gpurs_device_ptr left_destination, uint64_t left_rows,
                    gpurs_device_ptr right, uint64_t right_pitch, gpurs_device_ptr right_destination, uint64_t right_rows, uint64_t k) {
    gpurs_gpu *gpu = stream->gpu;
    gpurs_kernel *kernel = nullptr;
    int result = runtime::builtin_kernel(gpu, "gpurs_split_tf32_pair", 0, &kernel);
    if (result != GPURS_OK) return result;
    const uint64_t quads = (left_rows + right_rows) * (k / 4);
    gpurs_launch_config config;
    std::memset(&config, 0, sizeof config);
    const uint64_t blocks = std::min<uint64_t>((quads + 255) / 256, uint64_t(gpu->multiprocessors) * 8);
    config.grid[0] = uint32_t(std::max<uint64_t>(1, blocks));
    config.block[0] = 256;
    const void *left_pointer = reinterpret_cast<const void *>(left), *right_pointer = reinterpret_cast<const void *>(right);
    void *left_out = reinterpret_cast<void *>(left_destination), *right_out = reinterpret_cast<void *>(right_destination);
    long long left_stride = (long long)left_pitch, right_stride = (long long)right_pitch;
    int left_count = int(left_rows), right_count = int(right_rows), depth = int(k);
    void *arguments[9] = {&left_pointer, &left_stride, &left_out, &left_count, &right_pointer, &right_stride, &right_out, &right_count, &depth};
    return runtime::launch(kernel, stream, &config, arguments, true);
}

// The same split for a right operand stored k x n: written transposed, as the n x 3k array the product reads K-major.
int split_tf32_transposed(gpurs_stream *stream, gpurs_device_ptr source, uint64_t pitch, gpurs_device_ptr destination, uint64_t n, uint64_t k) {
    gpurs_gpu *gpu = stream->gpu;
    gpurs_kernel *kernel = nullptr;
    int result = runtime::builtin_kernel(gpu, "gpurs_split_tf32_transposed", 0, &kernel);
    if (result != GPURS_OK) return result;
    const uint64_t tiles = ((n + 31) / 32) * ((k + 31) / 32);
    gpurs_launch_config config;
    std::memset(&config, 0, sizeof config);
    config.grid[0] = uint32_t(std::max<uint64_t>(1, std::min<uint64_t>(tiles, uint64_t(gpu->multiprocessors) * 8)));
    config.block[0] = 256;
    const void *source_pointer = reinterpret_cast<const void *>(source);
    void *destination_pointer = reinterpret_cast<void *>(destination);
    long long source_pitch = (long long)pitch;
    int columns = int(n), depth = int(k);
    void *arguments[5] = {&source_pointer, &source_pitch, &destination_pointer, &columns, &depth};
    return runtime::launch(kernel, stream, &config, arguments, true);
}

// A k x n right operand copied as n x k (pitch k) for the kernels that read B K-major only.
int transpose_copy(gpurs_stream *stream, gpurs_device_ptr source, uint64_t pitch, gpurs_device_ptr destination, uint64_t n, uint64_t k, uint64_t element_bytes) {
    gpurs_gpu *gpu = stream->gpu;
    gpurs_kernel *kernel = nullptr;
    int result = runtime::builtin_kernel(gpu, element_bytes == 1 ? "gpurs_transpose_b8" : element_bytes == 2 ? "gpurs_transpose_b16" : "gpurs_transpose_b32", 0, &kernel);
    if (result != GPURS_OK) return result;
    const uint64_t tiles = ((n + 31) / 32) * ((k + 31) / 32);
    gpurs_launch_config config;
    std::memset(&config, 0, sizeof config);
    config.grid[0] = uint32_t(std::max<uint64_t>(1, std::min<uint64_t>(tiles, uint64_t(gpu->multiprocessors) * 8)));
    config.block[0] = 256;
    const void *source_pointer = reinterpret_cast<const void *>(source);
    void *destination_pointer = reinterpret_cast<void *>(destination);
    long long source_pitch = (long long)pitch;
    int columns = int(n), depth = int(k);
    void *arguments[5] = {&source_pointer, &source_pitch, &destination_pointer, &columns, &depth};
    return runtime::launch(kernel, stream, &config, arguments, true);
}

}  // namespace

namespace {

// The checks and the dispatch shared by gpurs_matmul and gpurs_matmul_allgather (`gather` non-null: C is this call's
// block of rows of a matrix that every GPU of the box keeps, and the kernel stores the block to all of them).
// `checks_only`: return after the checks, before anything is enqueued.
int matmul_checked(const char *op, gpurs_stream *stream, const gpurs_matmul_desc *desc, gpurs_device_ptr a, gpurs_device_ptr b,
                   gpurs_device_ptr c, const gpurs_gather_desc *gather, bool checks_only = false) {
    if (!stream || !desc) return fail(op, GPURS_E_INVALID_ARGUMENT, "null stream or descriptor");
    gpurs_gpu *gpu = stream->gpu;
    Choice choice;
    if (!choose(desc->a_type, desc->c_type, choice))
        return fail(op, GPURS_E_INVALID_ARGUMENT, "unsupported combination of operand and output types");
    const uint64_t m = desc->m, n = desc->n, k = desc->k;
    if (m > 0x7fffffffull || n > 0x7fffffffull || k > 0x7fffffffull)
        return fail(op, GPURS_E_SIZE_OVERFLOW, "a matrix dimension exceeds 2^31 - 1");
    const bool sparse = desc->metadata != 0;
    if (sparse && desc->a_type != GPURS_F16 && desc->a_type != GPURS_BF16)
        return fail(op, GPURS_E_INVALID_ARGUMENT, "2:4-sparse A is supported for 16-bit operands");
    if (sparse && (desc->a_type == GPURS_F16) && desc->c_type != GPURS_F32)
        return fail(op, GPURS_E_INVALID_ARGUMENT, "unsupported combination of operand and output types");
    if (sparse && k % 128) return fail(op, GPURS_E_INVALID_VIEW, "the depth of a 2:4-sparse product must be a multiple of 128");
    if (sparse && desc->metadata % 16) return fail(op, GPURS_E_INVALID_VIEW, "the metadata must be 16-byte aligned");
    const uint64_t a_columns = sparse ? k / 2 : k;   // stored elements per row of A
    if (desc->b_row_major != 0 && desc->b_row_major != 1) return fail(op, GPURS_E_INVALID_ARGUMENT, "b_row_major must be 0 or 1");
    const bool b_row_major = desc->b_row_major == 1;
    // B is n rows of k (the reference's layout) or, row-major as in C = A * B, k rows of n.
    const uint64_t b_rows = b_row_major ? k : n, b_columns = b_row_major ? n : k;
    const uint64_t lda = desc->lda ? desc->lda : a_columns, ldb = desc->ldb ? desc->ldb : b_columns, ldc = desc->ldc ? desc->ldc : n;
    if (lda < a_columns || ldb < b_columns || ldc < n) return fail(op, GPURS_E_INVALID_VIEW, "a row pitch is smaller than the row");
    // Extent of each operand in elements: the last row ends at (rows - 1) * pitch + columns.
    uint64_t a_extent = m ? (m - 1) * lda + a_columns : 0, b_extent = b_rows ? (b_rows - 1) * ldb + b_columns : 0,
             c_extent = m ? (m - 1) * ldc + n : 0;
    // A batch: matrix i starts stride_* elements after matrix i - 1 (packed when 0); matrices of one operand may not overlap.
    if (desc->batches < 0 || desc->batches > 65535) return fail(op, GPURS_E_INVALID_ARGUMENT, "batches must be 0..65535");
    const uint64_t batches = desc->batches > 1 ? uint64_t(desc->batches) : 1;
    const uint64_t stride_a = desc->stride_a ? desc->stride_a : m * lda, stride_b = desc->stride_b ? desc->stride_b : b_rows * ldb,
                   stride_c = desc->stride_c ? desc->stride_c : m * ldc;
    if (batches > 1) {
        if (stride_a < a_extent || stride_b < b_extent || stride_c < c_extent)
            return fail(op, GPURS_E_INVALID_VIEW, "a batch stride is smaller than the matrix");
        a_extent += (batches - 1) * stride_a, b_extent += (batches - 1) * stride_b, c_extent += (batches - 1) * stride_c;
    }
    if ((desc->a_len && desc->a_len < a_extent) || (desc->b_len && desc->b_len < b_extent) || (desc->c_len && desc->c_len < c_extent))
        return fail(op, GPURS_E_LENGTH_MISMATCH, "a slice is shorter than the matrix it is said to hold");
    if (m == 0 || n == 0) return GPURS_OK;
    if (!c) return fail(op, GPURS_E_INVALID_ARGUMENT, "null output");
    const uint64_t eb = uint64_t(choice.element_bytes), ob = uint64_t(choice.output_bytes);
    runtime::Enter enter(gpu);
    int result = GPURS_OK;
    if (k == 0) {
        // An empty sum: the product is all zeros.
        // (for a gathering product: the block of every GPU's copy)
        for (uint32_t target = 0; target < (gather ? gather->world : 1u); target++) {
            const gpurs_device_ptr block = gather ? c - gather->full[gather->rank] + gather->full[target] : c;
            for (uint64_t batch = 0; batch < batches; batch++)
                for (uint64_t row = 0; row < (ldc == n ? 1 : m); row++)
                    GPURS_TRY(gpu->api, cuMemsetD8Async(block + (batch * stride_c + row * ldc) * ob, 0, (ldc == n ? m * n : n) * ob, stream->handle));
        }
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
    if (desc->scale_a && desc->a_type != GPURS_E4M3) return fail(op, GPURS_E_INVALID_ARGUMENT, "scales are for E4M3 operands only");
    if (desc->scale_a && (desc->scale_a % 4 || desc->scale_b % 4)) return fail(op, GPURS_E_INVALID_VIEW, "scale arrays must be 4-byte aligned");
    if (desc->scale_kind != GPURS_SCALES_FP32_BLOCKS && desc->scale_kind != GPURS_SCALES_MX) return fail(op, GPURS_E_INVALID_ARGUMENT, "unknown scale kind");
    // A k x n right operand (the reference's row-major B of C = A * B): the dense 16-bit and 8-bit kernels read it in place and
    // the full-precision fp32 product transposes it while splitting it; every other kernel (2:4-sparse, scaled FP8, one-pass
    // TF32) reads B K-major only and gets a transposed copy in the handle's workspace first, then runs as an n x k product on
    // whole tiles (tiles split along K would need the workspace as well).
    if (b_row_major && gpu && !gather && batches == 1 &&
        (sparse || desc->scale_a != 0 || (desc->a_type == GPURS_F32 && desc->precision != GPURS_PRECISION_DEFAULT))) {
        if ((k * eb) % 16) return fail(op, GPURS_E_INVALID_VIEW, "operand bases and row pitches must be multiples of 16 bytes");
        if (m == 0 || n == 0 || k == 0) return GPURS_OK;
        if (n > (1ull << 40) / k) return fail(op, GPURS_E_SIZE_OVERFLOW, "the transposed copy of the right operand would exceed 2^40 elements");
        gpurs_matmul_desc local = *desc;
        local.b_row_major = 0, local.ldb = 0, local.b_len = 0;
        local.algorithm = (local.algorithm & ~GPURS_ALGO_SPLIT_LAST_ROUND) | GPURS_ALGO_WHOLE_TILES;
        // a rejected call launches nothing: the n x k product is checked before B is copied (B's own address stands in for the
        // copy's: n * k elements from there lie within B, which has been checked against C above)
        int result = matmul_checked(op, stream, &local, a, b, c, nullptr, true);
        if (result != GPURS_OK || checks_only) return result;
        runtime::Enter enter(gpu);
        CUdeviceptr copy = 0;
        result = runtime::workspace_acquire(stream, n * k * eb, &copy);
        if (result != GPURS_OK) return result;
        result = transpose_copy(stream, b, ldb, copy, n, k, eb);
        if (result == GPURS_OK) result = matmul_checked(op, stream, &local, a, copy, c, nullptr);
        const int released = runtime::workspace_release(stream);
        return result != GPURS_OK ? result : released;
    }
    if (desc->scale_kind == GPURS_SCALES_MX) {
        // Power-of-two scales per 32 elements, applied by the tensor core: its own kernel, dispatched here.
        if (!desc->scale_a) return fail(op, GPURS_E_INVALID_ARGUMENT, "both scale arrays or neither must be given");
        if (desc->c_type != GPURS_BF16 && desc->c_type != GPURS_F32)
            return fail(op, GPURS_E_INVALID_ARGUMENT, "unsupported combination of operand and output types");
        if (sparse || b_row_major || batches > 1 || gather || desc->row_absmax || (desc->algorithm & 0xff) > GPURS_ALGO_CTA_PAIR)
            return fail(op, GPURS_E_INVALID_ARGUMENT, "the MX-scaled product is a single dense n x k product on the tile kernels");
        if (k % 128) return fail(op, GPURS_E_INVALID_VIEW, "the depth of an MX-scaled product must be a multiple of 128");
        if (desc->scale_a % 16 || desc->scale_b % 16) return fail(op, GPURS_E_INVALID_VIEW, "MX scale arrays must be 16-byte aligned");
        if (desc->bias % 4 || desc->row_scale % 4 || desc->column_scale % 4) return fail(op, GPURS_E_INVALID_VIEW, "epilogue vectors must be 4-byte aligned");
        if (desc->alpha != desc->alpha) return fail(op, GPURS_E_INVALID_ARGUMENT, "alpha is not a number");
        if (desc->row_sum) return fail(op, GPURS_E_INVALID_ARGUMENT, "the row reduction is for single dense products with float outputs on the tile kernels");
        if (desc->accumulate != 0 && (desc->accumulate != 1 || desc->c_type != GPURS_F32)) return fail(op, GPURS_E_INVALID_ARGUMENT, "accumulating into the output needs an fp32 output");
        if (desc->row_bias % 4) return fail(op, GPURS_E_INVALID_VIEW, "epilogue vectors must be 4-byte aligned");
        const uint64_t mx_ldr = desc->ldr ? desc->ldr : n;
        if (desc->residual) {
            if (mx_ldr < n) return fail(op, GPURS_E_INVALID_VIEW, "a row pitch is smaller than the row");
            if (desc->residual % ob) return fail(op, GPURS_E_INVALID_VIEW, "the residual is not aligned to its element size");
            if (!(desc->residual == c && mx_ldr == ldc) && overlap(desc->residual, ((m - 1) * mx_ldr + n) * ob, c, c_extent * ob))
                return fail(op, GPURS_E_ALIASING, "the residual overlaps the output without being the output");
        }
        if ((desc->algorithm & GPURS_ALGO_WHOLE_TILES) && (desc->algorithm & GPURS_ALGO_SPLIT_LAST_ROUND))
            return fail(op, GPURS_E_INVALID_ARGUMENT, "whole tiles and a split last round exclude each other");
        if (checks_only) return GPURS_OK;
        Gemm mx;
        mx.stem = desc->c_type == GPURS_BF16 ? "gpurs_gemm_e4m3_mx_bf16" : "gpurs_gemm_e4m3_mx_f32";
        mx.element_type = desc->a_type, mx.element_bytes = 1, mx.output_bytes = choice.output_bytes, mx.output_type = desc->c_type;
        mx.a = a, mx.b = b, mx.c = c;
        mx.lda = lda, mx.ldb = ldb, mx.ldc = ldc;
        mx.m = m, mx.n = n, mx.k = k;
        const int wanted = desc->algorithm & 0xff;
        mx.cta_group = wanted == GPURS_ALGO_CTA_PAIR || (wanted == GPURS_ALGO_AUTO && m > 128) ? 2 : 1;
        mx.raster_rows = desc->raster_rows, mx.max_ctas = desc->max_ctas;
        mx.scale_a = desc->scale_a, mx.scale_b = desc->scale_b;
        mx.bias = desc->bias, mx.row_scale = desc->row_scale, mx.column_scale = desc->column_scale, mx.alpha = desc->alpha;
        mx.row_bias = desc->row_bias, mx.residual = desc->residual, mx.ldr = mx_ldr, mx.beta = desc->beta == 0.0f ? 1.0f : desc->beta;
        mx.accumulate = desc->accumulate == 1, mx.launch = desc->launch;
        mx.whole_tiles = (desc->algorithm & GPURS_ALGO_WHOLE_TILES) != 0, mx.force_split = (desc->algorithm & GPURS_ALGO_SPLIT_LAST_ROUND) != 0;
        return launch_mx(stream, mx);
    }

    int group = desc->algorithm & 0xff;
    if (desc->algorithm & ~(0xff | GPURS_ALGO_WHOLE_TILES | GPURS_ALGO_SPLIT_LAST_ROUND | GPURS_ALGO_WIDE_TILES | GPURS_ALGO_SQUARE_TILES)) return fail(op, GPURS_E_INVALID_ARGUMENT, "unknown algorithm");
    if ((desc->algorithm & GPURS_ALGO_WHOLE_TILES) && (desc->algorithm & GPURS_ALGO_SPLIT_LAST_ROUND))
        return fail(op, GPURS_E_INVALID_ARGUMENT, "whole tiles and a split last round exclude each other");
    if ((desc->algorithm & GPURS_ALGO_WIDE_TILES) && (desc->algorithm & GPURS_ALGO_SQUARE_TILES))
        return fail(op, GPURS_E_INVALID_ARGUMENT, "wide tiles and square tiles exclude each other");
    // Kernels that promote K-blocks to registers hand an accumulator back and forth between the tensor core and the CUDA cores.
    const bool promoted = desc->scale_a != 0 || (desc->a_type == GPURS_F32 && desc->precision == GPURS_PRECISION_DEFAULT);
    // Few rows of A, 16-bit operands, fp32 output: the split-K kernel that streams B once with every multiprocessor.
    const bool skinny_possible = m <= uint64_t(gemm::SKINNY_MAX_ROWS) && (desc->a_type == GPURS_F16 || desc->a_type == GPURS_BF16) &&
                                 desc->c_type == GPURS_F32 && !sparse && !desc->scale_a && !b_row_major && (n + 127) / 128 <= uint64_t(gemm::SKINNY_MAX_TILES) &&
                                 c % 4 == 0 && batches == 1 && !desc->row_absmax && !desc->row_scale && !desc->column_scale && (desc->alpha == 0.0f || desc->alpha == 1.0f) &&
                                 !desc->row_bias && !desc->residual && !desc->row_sum && !desc->accumulate;
    // N-major reading of 32-bit elements needs a different shared-memory swizzle (32-byte atoms) that these kernels
    // do not set up; measured: the plain 128-byte swizzle yields zeros for TF32.
    // fp32 operands at full precision are copied (split) before the product anyway: the copy of a k x n right operand is
    // written transposed, and the product reads it K-major like any other.
    const bool transposing_split = b_row_major && desc->a_type == GPURS_F32 && desc->precision == GPURS_PRECISION_DEFAULT && !sparse && !desc->scale_a;
    if (b_row_major && !transposing_split && (sparse || promoted || desc->a_type == GPURS_F32))
        return fail(op, GPURS_E_INVALID_ARGUMENT, "a k x n right operand is supported by the dense 16-bit and 8-bit tile kernels and by full-precision fp32 products");
    if (group == GPURS_ALGO_SKINNY && !skinny_possible)
        return fail(op, GPURS_E_INVALID_ARGUMENT, "the skinny algorithm needs m <= 64, 16-bit dense operands and fp32 output");
    if (batches > 1) {
        const bool typed = (desc->a_type == GPURS_F16 || desc->a_type == GPURS_BF16) && (desc->c_type == GPURS_F32 || desc->c_type == desc->a_type);
        if (!typed || sparse || promoted || b_row_major || gather || desc->l2_policy % 4 != 0)
            return fail(op, GPURS_E_INVALID_ARGUMENT, "a batch is supported for dense f16 / bf16 operands (n x k right operand, no L2 hints)");
        if ((stride_a * eb) % 16 || (stride_b * eb) % 16) return fail(op, GPURS_E_INVALID_VIEW, "operand bases and row pitches must be multiples of 16 bytes");
        if ((stride_c * ob) % ob) return fail(op, GPURS_E_INVALID_VIEW, "the output is not aligned to its element size");
        if (group == GPURS_ALGO_SKINNY) return fail(op, GPURS_E_INVALID_ARGUMENT, "the skinny algorithm takes a single product");
    }
    if (gather) {
        // The push epilogue exists for the CTA-pair tile kernels of these type pairs, and it stores whole boxes of 32 rows.
        const bool typed = (desc->a_type == GPURS_BF16 && desc->c_type == GPURS_BF16) || (desc->a_type == GPURS_F16 && desc->c_type == GPURS_F32) ||
                           (desc->a_type == GPURS_I8 && desc->c_type == GPURS_I32) || (desc->a_type == GPURS_E4M3 && desc->c_type == GPURS_BF16);
        if (!typed || promoted || (sparse && desc->a_type != GPURS_BF16))
            return fail(op, GPURS_E_INVALID_ARGUMENT, "the gathering product supports bf16->bf16 (dense or 2:4 sparse), f16->f32, i8->i32 and unscaled e4m3->bf16");
        if (group != GPURS_ALGO_AUTO && group != GPURS_ALGO_CTA_PAIR)
            return fail(op, GPURS_E_INVALID_ARGUMENT, "the gathering product runs on the CTA-pair kernels only");
        group = GPURS_ALGO_CTA_PAIR;
    }
    // An explicit geometry speaks for the tile kernels: its cluster size picks between them when the caller left that open.
    if (group == GPURS_ALGO_AUTO && desc->launch && (desc->launch->cluster[0] == 1 || desc->launch->cluster[0] == 2) && !promoted)
        group = desc->launch->cluster[0] == 2 ? GPURS_ALGO_CTA_PAIR : GPURS_ALGO_SINGLE_CTA;
    if (group == GPURS_ALGO_AUTO && skinny_possible && !desc->launch) group = GPURS_ALGO_SKINNY;
    // The promoted products (fp32 as three TF32 passes, block-scaled FP8) stay on one-CTA tiles: their accumulator hand-offs then
    // never cross to another CTA.  The block-scaled product also has a CTA-pair kernel (four accumulators in flight, chosen with
    // GPURS_ALGO_CTA_PAIR); measured side by side on one box it is the slower one (4096 x 7168 x 7168: 1745-1755 against
    // 1882-1913 TFLOP/s; 8192^3: 1950 against 2075).
    if (group == GPURS_ALGO_AUTO) group = (m > 128 && !promoted) ? GPURS_ALGO_CTA_PAIR : GPURS_ALGO_SINGLE_CTA;
    if (group != GPURS_ALGO_SINGLE_CTA && group != GPURS_ALGO_CTA_PAIR && group != GPURS_ALGO_SKINNY)
        return fail(op, GPURS_E_INVALID_ARGUMENT, "unknown algorithm");
    if (desc->bias && desc->c_type == GPURS_I32) return fail(op, GPURS_E_INVALID_ARGUMENT, "a bias is for floating-point outputs");
    if (desc->bias % 4) return fail(op, GPURS_E_INVALID_VIEW, "the bias must be 4-byte aligned");
    const bool scaled_output = desc->row_scale || desc->column_scale || (desc->alpha != 0.0f && desc->alpha != 1.0f);
    if (scaled_output && desc->c_type == GPURS_I32) return fail(op, GPURS_E_INVALID_ARGUMENT, "output scales are for floating-point outputs");
    if (desc->row_scale % 4 || desc->column_scale % 4) return fail(op, GPURS_E_INVALID_VIEW, "output scales must be 4-byte aligned");
    if (desc->alpha != desc->alpha) return fail(op, GPURS_E_INVALID_ARGUMENT, "alpha is not a number");
    if (desc->row_absmax) {
        if (desc->c_type == GPURS_I32 || sparse || promoted || batches > 1 || group == GPURS_ALGO_SKINNY)
            return fail(op, GPURS_E_INVALID_ARGUMENT, "the row reduction is for single dense products with float outputs on the tile kernels");
        if (desc->row_absmax % 4) return fail(op, GPURS_E_INVALID_VIEW, "the row reduction must be 4-byte aligned");
        if (overlap(desc->row_absmax, m * sizeof(float), c, c_extent * ob))
            return fail(op, GPURS_E_ALIASING, "the row reduction overlaps the output");
    }
    if (desc->precision != GPURS_PRECISION_DEFAULT && desc->precision != GPURS_PRECISION_TF32)
        return fail(op, GPURS_E_INVALID_ARGUMENT, "unknown precision");
    if (desc->accumulate != 0 && desc->accumulate != 1) return fail(op, GPURS_E_INVALID_ARGUMENT, "accumulate must be 0 or 1");
    if (desc->reserved != 0) return fail(op, GPURS_E_INVALID_ARGUMENT, "reserved fields must be 0");
    const uint64_t ldr = desc->ldr ? desc->ldr : n;
    if (desc->row_bias || desc->residual || desc->row_sum || desc->accumulate) {
        if (desc->c_type == GPURS_I32) return fail(op, GPURS_E_INVALID_ARGUMENT, "the output algebra is for floating-point outputs");
        if (group == GPURS_ALGO_SKINNY) return fail(op, GPURS_E_INVALID_ARGUMENT, "the skinny algorithm takes a bias only");
        if (desc->row_bias % 4 || desc->row_sum % 4) return fail(op, GPURS_E_INVALID_VIEW, "epilogue vectors must be 4-byte aligned");
    }
    if (desc->residual) {
        if (batches > 1 || gather) return fail(op, GPURS_E_INVALID_ARGUMENT, "a residual is for single products");
        if (ldr < n) return fail(op, GPURS_E_INVALID_VIEW, "a row pitch is smaller than the row");
        if (desc->residual % ob) return fail(op, GPURS_E_INVALID_VIEW, "the residual is not aligned to its element size");
        if (desc->beta != desc->beta) return fail(op, GPURS_E_INVALID_ARGUMENT, "beta is not a number");
        // C itself (updated in place, element by element) or memory that does not touch C
        const bool in_place = desc->residual == c && ldr == ldc;
        if (!in_place && overlap(desc->residual, ((m - 1) * ldr + n) * ob, c, c_extent * ob))
            return fail(op, GPURS_E_ALIASING, "the residual overlaps the output without being the output");
    }
    if (desc->row_sum) {
        if (sparse || promoted || batches > 1) return fail(op, GPURS_E_INVALID_ARGUMENT, "the row reduction is for single dense products with float outputs on the tile kernels");
        if (overlap(desc->row_sum, m * sizeof(float), c, c_extent * ob)) return fail(op, GPURS_E_ALIASING, "the row reduction overlaps the output");
    }
    if (desc->accumulate) {
        if (desc->c_type != GPURS_F32) return fail(op, GPURS_E_INVALID_ARGUMENT, "accumulating into the output needs an fp32 output");
        if (batches > 1 || gather) return fail(op, GPURS_E_INVALID_ARGUMENT, "accumulating into the output is for single products");
        if (c % 4) return fail(op, GPURS_E_INVALID_VIEW, "the output is not aligned to its element size");
    }
    if (desc->launch) {
        if (group == GPURS_ALGO_SKINNY) return fail(op, GPURS_E_INVALID_ARGUMENT, "the skinny algorithm sizes its own grid");
        if (gather) return fail(op, GPURS_E_INVALID_ARGUMENT, "the gathering product sizes its own grid");
    }
    if (desc->l2_policy < 0 || desc->l2_policy > 4) return fail(op, GPURS_E_INVALID_ARGUMENT, "unknown L2 policy");
    if (sparse && desc->scale_a) return fail(op, GPURS_E_INVALID_ARGUMENT, "a sparse product takes no scales");
    if (checks_only) return GPURS_OK;
    Gemm gemm;
    gemm.stem = choice.stem;
    gemm.element_type = desc->a_type;
    gemm.element_bytes = choice.element_bytes;
    gemm.output_bytes = choice.output_bytes;
    gemm.output_type = desc->c_type;
    gemm.a = a, gemm.b = b, gemm.c = c;
    gemm.lda = lda, gemm.ldb = ldb, gemm.ldc = ldc;
    gemm.m = m, gemm.n = n, gemm.k = k;
    gemm.cta_group = group == GPURS_ALGO_CTA_PAIR ? 2 : 1;
    gemm.raster_rows = desc->raster_rows;
    gemm.max_ctas = desc->max_ctas;
    gemm.bias = desc->bias;
    gemm.row_scale = desc->row_scale, gemm.column_scale = desc->column_scale, gemm.alpha = desc->alpha;
    gemm.row_absmax = desc->row_absmax;
    gemm.row_bias = desc->row_bias, gemm.residual = desc->residual, gemm.ldr = ldr, gemm.beta = desc->beta == 0.0f ? 1.0f : desc->beta;
    gemm.row_sum = desc->row_sum, gemm.accumulate = desc->accumulate == 1, gemm.launch = desc->launch;
    gemm.whole_tiles = (desc->algorithm & GPURS_ALGO_WHOLE_TILES) != 0;
    gemm.force_split = (desc->algorithm & GPURS_ALGO_SPLIT_LAST_ROUND) != 0;
    gemm.tile_width = (desc->algorithm & GPURS_ALGO_WIDE_TILES) ? 512 : (desc->algorithm & GPURS_ALGO_SQUARE_TILES) ? 256 : 0;
    gemm.b_row_major = b_row_major;
    gemm.gather = gather;
    gemm.batches = batches, gemm.stride_a = stride_a, gemm.stride_b = stride_b, gemm.stride_c = stride_c;
    if (group == GPURS_ALGO_SKINNY) return launch_skinny(stream, gemm);
    gemm.l2_policy = desc->l2_policy == 4 ? 0 : desc->l2_policy;   // library default: no hints
    if (sparse) {
        gemm.stem = desc->a_type == GPURS_F16 ? "gpurs_gemm_sparse_f16_f32"
                    : desc->c_type == GPURS_BF16 ? "gpurs_gemm_sparse_bf16_bf16" : "gpurs_gemm_sparse_bf16_f32";
        gemm.metadata = desc->metadata;
    }
    if (desc->scale_a) {
        // per-K-block promotion kernel: fp32 scales [m][ceil(k/128)] and [ceil(n/128)][ceil(k/128)]
        gemm.stem = desc->c_type == GPURS_BF16 ? "gpurs_gemm_e4m3_scaled_bf16" : "gpurs_gemm_e4m3_scaled_f32";
        gemm.scale_a = desc->scale_a;
        gemm.scale_b = desc->scale_b;
        gemm.threads = gemm::SCALED_THREADS;
        if (gemm.cta_group == 2 && !gemm.accumulate) {
            // CTA pairs: the kernel that keeps four accumulators in flight
            gemm.stem = desc->c_type == GPURS_BF16 ? "gpurs_gemm_e4m3_blockscaled_bf16" : "gpurs_gemm_e4m3_blockscaled_f32";
            return launch_blockscaled(stream, gemm);
        }
    }

    if (desc->a_type == GPURS_F32 && desc->precision == GPURS_PRECISION_DEFAULT) {
        // fp32 operands at fp32-like accuracy: split both operands into TF32 hi and lo parts in scratch
        // memory, laid out so that ONE K-major product over 3K sums hi*hi + hi*lo + lo*hi.
        if (k % 4) return fail(op, GPURS_E_INVALID_VIEW, "operand bases and row pitches must be multiples of 16 bytes");
        // the split operands are 3k deep, and the kernels index the depth with 32-bit integers
        if (k > 0x7fffffffull / 3) return fail(op, GPURS_E_SIZE_OVERFLOW, "the depth of a full-precision fp32 product exceeds (2^31 - 1) / 3");
        const uint64_t a_split = m * 3 * k * sizeof(float), b_split = n * 3 * k * sizeof(float);
        {
            // the geometry is checked before the split kernels are enqueued: a rejected call launches nothing
            gemm.threads = gemm::SCALED_THREADS;
            uint64_t unused = 0;
            result = explicit_ctas(op, desc->launch, gemm.cta_group, uint32_t(gemm.threads), shared_for(gemm), unused);
            if (result != GPURS_OK) return result;
        }
        // the product may split tiles along K: the parts share the borrowed workspace with the split operands
        gemm.lda = gemm.ldb = 3 * k;
        gemm.k = 3 * k;
        gemm.b_row_major = false;     // the split copy is n x 3k whatever B was
        uint64_t explicit_grid = 0;
        explicit_ctas(op, desc->launch, gemm.cta_group, uint32_t(gemm.threads), shared_for(gemm), explicit_grid);
        const uint64_t operands = (a_split + b_split + 255) / 256 * 256;
        const size_t parts = plan_split(gpu, gemm, explicit_grid).partial_bytes(gemm.cta_group);
        CUdeviceptr scratch = 0;
        result = runtime::workspace_acquire(stream, operands + parts, &scratch);
        if (result != GPURS_OK) return result;
        gemm.partials = parts ? scratch + operands : 0, gemm.partials_bytes = parts;
        if (b_row_major) {
            result = split_tf32(stream, a, lda, scratch, m, k, 0);
            if (result == GPURS_OK) result = split_tf32_transposed(stream, b, ldb, scratch + a_split, n, k);
        } else {
            result = split_tf32_pair(stream, a, lda, scratch, m, b, ldb, scratch + a_split, n, k);
        }
        gemm.a = scratch, gemm.b = scratch + a_split;
        // The tensor core's fp32 accumulator truncates after every instruction; promoting each K-block to
        // registers keeps the sum round-to-nearest, which the 1e-4 bound needs once K reaches thousands.
        gemm.stem = "gpurs_gemm_tf32_promoted_f32";
        gemm.threads = gemm::SCALED_THREADS;
        if (result == GPURS_OK) result = launch_gemm(stream, gemm);
        int released = runtime::workspace_release(stream);
        return result != GPURS_OK ? result : released;
    }
    return launch_gemm(stream, gemm);
}

}  // namespace

extern "C" int gpurs_matmul(gpurs_stream *stream, const gpurs_matmul_desc *desc, gpurs_device_ptr a, gpurs_device_ptr b,
                            gpurs_device_ptr c) {
    return matmul_checked("gpurs_matmul", stream, desc, a, b, c, nullptr);
}

extern "C" int gpurs_matmul_allgather(gpurs_stream *stream, const gpurs_matmul_desc *desc, const gpurs_gather_desc *gather,
                                      gpurs_device_ptr a, gpurs_device_ptr b) {
    const char *const op = "gpurs_matmul_allgather";
    if (!stream || !desc || !gather) return fail(op, GPURS_E_INVALID_ARGUMENT, "null stream or descriptor");
    if (gather->world < 1 || gather->world > uint32_t(gemm::MAX_PUSH_TARGETS) || gather->rank >= gather->world)
        return fail(op, GPURS_E_INVALID_ARGUMENT, "world must be 1..8 and rank below it");
    const uint64_t m = desc->m, n = desc->n;
    const uint64_t pitch = gather->ld_full ? gather->ld_full : n;
    if (pitch < n) return fail(op, GPURS_E_INVALID_VIEW, "a row pitch is smaller than the row");
    if (gather->total_rows > 0x7fffffffull) return fail(op, GPURS_E_SIZE_OVERFLOW, "a matrix dimension exceeds 2^31 - 1");
    if (gather->row_offset > gather->total_rows || m > gather->total_rows - gather->row_offset)
        return fail(op, GPURS_E_LENGTH_MISMATCH, "the block of rows does not fit in the gathered matrix");
    // The epilogue stores boxes of 32 rows: a block that ended inside a box would overwrite the next block's first rows.
    if (gather->row_offset + m != gather->total_rows && m % 32)
        return fail(op, GPURS_E_INVALID_VIEW, "every block of rows but the last must be a multiple of 32 rows");
    if (desc->ldc && desc->ldc != pitch) return fail(op, GPURS_E_INVALID_VIEW, "ldc must be 0 or the pitch of the gathered matrix");
    const uint64_t ob = (desc->c_type == GPURS_BF16 || desc->c_type == GPURS_F16) ? 2 : 4;
    for (uint32_t t = 0; t < gather->world; t++) {
        if (!gather->full[t]) return fail(op, GPURS_E_INVALID_ARGUMENT, "null output");
        if (gather->full[t] % 16 || (pitch * ob) % 16)
            return fail(op, GPURS_E_INVALID_VIEW, "the gathered matrices need 16-byte aligned bases and row pitches");
    }
    // No copy of the result may lie over an operand (the rank's own copy is checked again with exact extents below).
    const uint64_t eb = desc->a_type == GPURS_F32 ? 4 : (desc->a_type == GPURS_F16 || desc->a_type == GPURS_BF16) ? 2 : 1;
    const uint64_t a_bytes = m * (desc->lda ? desc->lda : (desc->metadata ? desc->k / 2 : desc->k)) * eb;
    const uint64_t b_bytes = (desc->b_row_major == 1 ? desc->k * (desc->ldb ? desc->ldb : n) : n * (desc->ldb ? desc->ldb : desc->k)) * eb;
    for (uint32_t t = 0; t < gather->world; t++)
        if (overlap(gather->full[t], gather->total_rows * pitch * ob, a, a_bytes) || overlap(gather->full[t], gather->total_rows * pitch * ob, b, b_bytes))
            return fail(op, GPURS_E_ALIASING, "the output overlaps an operand");
    gpurs_matmul_desc local = *desc;
    local.ldc = pitch;
    local.c_len = 0;
    const gpurs_device_ptr mine = gather->full[gather->rank] + gather->row_offset * pitch * ob;
    if (!(desc->algorithm & GPURS_ALGO_GATHER_BY_COPIES)) return matmul_checked(op, stream, &local, a, b, mine, gather);

    // Copy-engine form: the block is multiplied in up to four bands of rows (whole 512-row tiles) by the plain kernels, into
    // this GPU's copy; when a band is complete, one helper stream per peer copies it to that peer over NVLink while the next
    // band is multiplied.  The caller's stream continues after all copies (they are its work).
    local.algorithm &= ~GPURS_ALGO_GATHER_BY_COPIES;
    if (desc->batches > 1) return fail(op, GPURS_E_INVALID_ARGUMENT, "the gathering product takes a single product");
    gpurs_gpu *gpu = stream->gpu;
    runtime::Enter enter(gpu);
    const driver::Api *api = gpu->api;
    const uint32_t peers = gather->world - 1;
    const uint64_t granule = 512;
    const uint64_t bands = std::min<uint64_t>(4, std::max<uint64_t>(1, m / granule));
    const uint64_t band_rows = ((m + bands - 1) / bands + granule - 1) / granule * granule;
    int result = runtime::copy_pipeline(gpu, bands + peers);
    if (result == GPURS_OK) result = runtime::peer_pipeline(gpu, peers);
    if (result != GPURS_OK) return result;
    const uint64_t a_pitch = desc->lda ? desc->lda : (desc->metadata ? desc->k / 2 : desc->k);
    const uint64_t metadata_per_row_block = desc->metadata ? (desc->k / 128) * uint64_t(gemm::SPARSE_METADATA_BLOCK_BYTES) : 0;
    bool copied = false;
    for (uint64_t band = 0; band * band_rows < m && result == GPURS_OK; band++) {
        const uint64_t first = band * band_rows, rows = std::min(band_rows, m - first);
        gpurs_matmul_desc part = local;
        part.m = rows;
        if (desc->metadata) part.metadata = desc->metadata + (first / 128) * metadata_per_row_block;
        // fp32 block scales: one per row and 128 of K; MX scales: tiles of 512 bytes per 128 rows and 128 of K (bands are whole tiles)
        if (desc->scale_a)
            part.scale_a = desc->scale_a + (desc->scale_kind == GPURS_SCALES_MX ? (first / 128) * ((desc->k + 127) / 128) * 512
                                                                                 : first * ((desc->k + 127) / 128) * sizeof(float));
        if (desc->row_scale) part.row_scale = desc->row_scale + first * sizeof(float);
        if (desc->row_bias) part.row_bias = desc->row_bias + first * sizeof(float);
        if (desc->row_absmax) part.row_absmax = desc->row_absmax + first * sizeof(float);
        if (desc->row_sum) part.row_sum = desc->row_sum + first * sizeof(float);
        if (desc->residual) part.residual = desc->residual + first * (desc->ldr ? desc->ldr : n) * ob;
        const uint64_t c_offset = first * pitch * ob;
        result = matmul_checked(op, stream, &part, a + first * a_pitch * eb, b, mine + c_offset, nullptr);
        if (result != GPURS_OK) break;
        CUevent multiplied = gpu->events[band];
        CUresult code = api->cuEventRecord(multiplied, stream->handle);
        for (uint32_t i = 0; i < peers && code == CUDA_SUCCESS; i++) {
            const uint32_t target = (gather->rank + 1 + i) % gather->world;
            const CUdeviceptr to = gather->full[target] + gather->row_offset * pitch * ob + c_offset;
            code = api->cuStreamWaitEvent(gpu->peer_streams[i], multiplied, 0);
            if (code != CUDA_SUCCESS) break;
            if (pitch == n) {
                code = api->cuMemcpyDtoDAsync(to, mine + c_offset, rows * n * ob, gpu->peer_streams[i]);
            } else {
                CUDA_MEMCPY2D copy;
                std::memset(&copy, 0, sizeof copy);
                copy.srcMemoryType = copy.dstMemoryType = CU_MEMORYTYPE_DEVICE;
                copy.srcDevice = mine + c_offset, copy.dstDevice = to;
                copy.srcPitch = copy.dstPitch = pitch * ob;
                copy.WidthInBytes = n * ob;
                copy.Height = rows;
                code = api->cuMemcpy2DAsync(&copy, gpu->peer_streams[i]);
            }
            copied = true;
        }
        if (code != CUDA_SUCCESS) result = runtime::fail_driver(api, "gpurs_matmul_allgather copy", code);
    }
    // whatever happened, the caller's stream continues only after the helper streams have drained
    for (uint32_t i = 0; i < peers && copied; i++) {
        CUevent sent = gpu->events[bands + i];
        CUresult code = api->cuEventRecord(sent, gpu->peer_streams[i]);
        if (code == CUDA_SUCCESS) code = api->cuStreamWaitEvent(stream->handle, sent, 0);
        if (code != CUDA_SUCCESS && result == GPURS_OK) result = runtime::fail_driver(api, "gpurs_matmul_allgather join", code);
    }
    return result;
}

// Operands and result in HOST memory: copy in, multiply, copy out, with the three overlapped.  One operand goes up whole,
// the other in blocks; each block is multiplied as soon as it has arrived and its part of C starts its way back while
// the next block is still arriving, so the call costs about the longer of the two transfer directions instead of
// their sum plus the product.  The reference's host writes the same steps one after the other
// (examples/blackwell/examples/blackwell_matrix.rs:58-83: upload, upload, zeros, launch, download).
extern "C" int gpurs_matmul_host(gpurs_stream *stream, const gpurs_matmul_desc *desc, const void *host_a, const void *host_b, void *host_c,
                                 gpurs_device_ptr a, gpurs_device_ptr b, gpurs_device_ptr c) {
    const char *const op = "gpurs_matmul_host";
    if (!stream || !desc) return fail(op, GPURS_E_INVALID_ARGUMENT, "null stream or descriptor");
    Choice choice;
    if (!choose(desc->a_type, desc->c_type, choice))
        return fail(op, GPURS_E_INVALID_ARGUMENT, "unsupported combination of operand and output types");
    if (desc->metadata) return fail(op, GPURS_E_INVALID_ARGUMENT, "a 2:4-sparse operand is prepared on the device: use gpurs_matmul");
    if (desc->batches > 1) return fail(op, GPURS_E_INVALID_ARGUMENT, "the host-buffer product takes a single product");
    if (desc->scale_kind != GPURS_SCALES_FP32_BLOCKS) return fail(op, GPURS_E_INVALID_ARGUMENT, "the host-buffer product takes fp32 block scales only");
    const uint64_t m = desc->m, n = desc->n, k = desc->k;
    if (m > 0x7fffffffull || n > 0x7fffffffull || k > 0x7fffffffull)
        return fail(op, GPURS_E_SIZE_OVERFLOW, "a matrix dimension exceeds 2^31 - 1");
    if (m == 0 || n == 0) return GPURS_OK;
    if (!host_c || !c || (k && (!host_a || !host_b || !a || !b))) return fail(op, GPURS_E_INVALID_ARGUMENT, "null operand");
    const bool b_row_major = desc->b_row_major == 1;
    const uint64_t b_rows = b_row_major ? k : n, b_columns = b_row_major ? n : k;
    const uint64_t lda = desc->lda ? desc->lda : k, ldb = desc->ldb ? desc->ldb : b_columns, ldc = desc->ldc ? desc->ldc : n;
    if (lda < k || ldb < b_columns || ldc < n) return fail(op, GPURS_E_INVALID_VIEW, "a row pitch is smaller than the row");
    const uint64_t eb = uint64_t(choice.element_bytes), ob = uint64_t(choice.output_bytes);
    gpurs_gpu *gpu = stream->gpu;
    runtime::Enter enter(gpu);

    // The smaller operand goes up whole, the larger one in about eight blocks (measured on bf16 8192^3: 4, 8, 16, 32
    // blocks take 6.1, 5.9, 6.1, 6.7 ms) (of rows of A, or of rows of B = columns
    // of C), whole 256-wide tiles each; every block is multiplied when it has arrived and its part of C starts back at
    // once.  Products that prepare B per call (fp32 operands, whose split copy of B would be rebuilt for every block)
    // and small ones go in one piece.
    // (a k x n right operand of a kernel that reads B K-major only is copied transposed per call as well)
    const bool in_one_piece = (desc->a_type == GPURS_F32 && desc->precision == GPURS_PRECISION_DEFAULT) ||
                              (b_row_major && (desc->metadata != 0 || desc->scale_a != 0 || desc->a_type == GPURS_F32));
    const bool by_columns = !in_one_piece && !b_row_major && n > m;
    const uint64_t extent = by_columns ? n : m;
    const uint64_t block_extent = (in_one_piece || extent <= 512) ? extent : std::max<uint64_t>(256, ((extent + 7) / 8 + 255) / 256 * 256);
    // The last block's product and its way back to the host follow the last copy in and overlap nothing: the blocks taper off at
    // the end (the last full-size block goes as a half and two quarters, whole 256-wide tiles each).
    std::vector<std::pair<uint64_t, uint64_t>> pieces;      // first row (or column) and extent of every block
    for (uint64_t first = 0; first < extent;) {
        const uint64_t left = extent - first;
        uint64_t count = std::min(block_extent, left);
        if (!in_one_piece && !pieces.empty() && left <= block_extent && left >= 512) count = ((left / 2 + 255) / 256) * 256;
        pieces.emplace_back(first, count);
        first += count;
    }
    const uint64_t blocks = pieces.size();
    int result = runtime::copy_pipeline(gpu, 3 * blocks + 8);
    if (result != GPURS_OK) return result;
    const driver::Api *api = gpu->api;
    CUevent *events = gpu->events.data();
    CUevent begun = events[0], whole_arrived = events[1], finished = events[2];
    size_t next_event = 3;

    // Both helper streams start after the work already on the caller's stream (it may still be using the buffers).
    GPURS_TRY(api, cuEventRecord(begun, stream->handle));
    GPURS_TRY(api, cuStreamWaitEvent(gpu->copy_in, begun, 0));
    GPURS_TRY(api, cuStreamWaitEvent(gpu->copy_out, begun, 0));
    auto join = [&]() -> int {
        // whatever happened, the caller's stream continues only after both helper streams have drained
        GPURS_TRY(api, cuEventRecord(finished, gpu->copy_out));
        GPURS_TRY(api, cuStreamWaitEvent(stream->handle, finished, 0));
        GPURS_TRY(api, cuEventRecord(finished, gpu->copy_in));
        GPURS_TRY(api, cuStreamWaitEvent(stream->handle, finished, 0));
        return GPURS_OK;
    };
    // Copies of `rows` rows of `row_bytes` bytes at a pitch of `pitch` bytes on both sides: only the rows move, whatever
    // lies between them (in host or device memory) stays as it is.
    auto copy_rows = [&](bool to_device, CUdeviceptr device, const void *host, uint64_t rows, uint64_t row_bytes, uint64_t pitch, CUstream on) -> CUresult {
        if (pitch == row_bytes)
            return to_device ? api->cuMemcpyHtoDAsync(device, host, rows * row_bytes, on)
                             : api->cuMemcpyDtoHAsync(const_cast<void *>(host), device, rows * row_bytes, on);
        CUDA_MEMCPY2D copy;
        std::memset(&copy, 0, sizeof copy);
        copy.srcMemoryType = to_device ? CU_MEMORYTYPE_HOST : CU_MEMORYTYPE_DEVICE;
        copy.dstMemoryType = to_device ? CU_MEMORYTYPE_DEVICE : CU_MEMORYTYPE_HOST;
        if (to_device) copy.srcHost = host, copy.dstDevice = device;
        else copy.srcDevice = device, copy.dstHost = const_cast<void *>(host);
        copy.srcPitch = copy.dstPitch = pitch;
        copy.WidthInBytes = row_bytes;
        copy.Height = rows;
        return api->cuMemcpy2DAsync(&copy, on);
    };
    auto driver_failed = [&](CUresult code) { return runtime::fail_driver(api, "gpurs_matmul_host copy", code); };
    // From here on no exit may skip join(): a failure is remembered in `result` and the loops stop.
    auto checked = [&](CUresult code, const char *what) { return code == CUDA_SUCCESS ? int(GPURS_OK) : runtime::fail_driver(api, what, code); };
    const uint8_t *bytes_a = static_cast<const uint8_t *>(host_a), *bytes_b = static_cast<const uint8_t *>(host_b);
    uint8_t *bytes_c = static_cast<uint8_t *>(host_c);
    const uint64_t k_blocks = (k + 127) / 128;
    const uint64_t ldr = desc->ldr ? desc->ldr : n;

    // Rows [first, first + count) of an operand (A, or B stored n x k) go up; the caller's stream waits for them.
    auto upload = [&](bool left, uint64_t first, uint64_t count) -> int {
        const uint64_t pitch = left ? lda : ldb, offset = first * pitch * eb;
        const CUresult code = copy_rows(true, (left ? a : b) + offset, (left ? bytes_a : bytes_b) + offset, count, k * eb, pitch * eb, gpu->copy_in);
        if (code) return driver_failed(code);
        CUevent arrived = events[next_event++];
        int status = checked(api->cuEventRecord(arrived, gpu->copy_in), "cuEventRecord");
        if (status == GPURS_OK) status = checked(api->cuStreamWaitEvent(stream->handle, arrived, 0), "cuStreamWaitEvent");
        return status;
    };
    // C[row .. row + rows, column .. column + columns) = A's rows times B's rows (columns of C), every vector and matrix of the
    // output algebra moved along; then that part of C starts its way back.
    auto multiply_and_return = [&](uint64_t row, uint64_t rows, uint64_t column, uint64_t columns) -> int {
        gpurs_matmul_desc local = *desc;
        local.a_len = local.b_len = local.c_len = 0;
        local.lda = lda, local.ldb = ldb, local.ldc = ldc;
        local.m = rows, local.n = columns;
        if (desc->bias) local.bias = desc->bias + column * sizeof(float);
        if (desc->column_scale) local.column_scale = desc->column_scale + column * sizeof(float);
        if (desc->scale_b) local.scale_b = desc->scale_b + (column / 128) * k_blocks * sizeof(float);
        if (desc->row_scale) local.row_scale = desc->row_scale + row * sizeof(float);
        if (desc->scale_a) local.scale_a = desc->scale_a + row * k_blocks * sizeof(float);
        if (desc->row_bias) local.row_bias = desc->row_bias + row * sizeof(float);
        if (desc->row_absmax) local.row_absmax = desc->row_absmax + row * sizeof(float);
        if (desc->row_sum) local.row_sum = desc->row_sum + row * sizeof(float);
        if (desc->residual) local.residual = desc->residual + (row * ldr + column) * ob, local.ldr = ldr;
        const uint64_t b_offset = b_row_major ? column * eb : column * ldb * eb, c_offset = (row * ldc + column) * ob;
        int status = matmul_checked(op, stream, &local, a + row * lda * eb, b + b_offset, c + c_offset, nullptr);
        if (status != GPURS_OK) return status;
        CUevent c_ready = events[next_event++];
        status = checked(api->cuEventRecord(c_ready, stream->handle), "cuEventRecord");
        if (status == GPURS_OK) status = checked(api->cuStreamWaitEvent(gpu->copy_out, c_ready, 0), "cuStreamWaitEvent");
        if (status != GPURS_OK) return status;
        const CUresult code = copy_rows(false, c + c_offset, bytes_c + c_offset, rows, columns * ob, ldc * ob, gpu->copy_out);
        return code ? driver_failed(code) : int(GPURS_OK);
    };

    {
        if (k) {
            const CUresult code = by_columns ? copy_rows(true, a, host_a, m, k * eb, lda * eb, gpu->copy_in)
                                             : copy_rows(true, b, host_b, b_rows, b_columns * eb, ldb * eb, gpu->copy_in);
            if (code) result = driver_failed(code);
            if (result == GPURS_OK) result = checked(api->cuEventRecord(whole_arrived, gpu->copy_in), "cuEventRecord");
            if (result == GPURS_OK) result = checked(api->cuStreamWaitEvent(stream->handle, whole_arrived, 0), "cuStreamWaitEvent");
        }
        for (uint64_t block = 0; block < blocks && result == GPURS_OK; block++) {
            const uint64_t first = pieces[block].first, count = pieces[block].second;
            if (k) result = upload(!by_columns, first, count);
            if (result != GPURS_OK) break;
            result = by_columns ? multiply_and_return(0, m, first, count) : multiply_and_return(first, count, 0, n);
        }
    }
    const int joined = join();
    return result != GPURS_OK ? result : joined;
}

extern "C" size_t gpurs_metadata_bytes(uint64_t m, uint64_t k) {
    return size_t(((m + 127) / 128) * ((k + gemm::SPARSE_BLOCK_K - 1) / gemm::SPARSE_BLOCK_K) * gemm::SPARSE_METADATA_BLOCK_BYTES);
}

extern "C" int gpurs_compress_24(gpurs_stream *stream, int element_type, uint64_t m, uint64_t k, gpurs_device_ptr dense, uint64_t ld,
                                 gpurs_device_ptr values, gpurs_device_ptr metadata, gpurs_device_ptr violations) {
    const char *const op = "gpurs_compress_24";
    if (!stream) return fail(op, GPURS_E_INVALID_ARGUMENT, "null stream");
    if (element_type != GPURS_F16 && element_type != GPURS_BF16) return fail(op, GPURS_E_INVALID_ARGUMENT, "16-bit element types only");
    if (m > 0x7fffffffull || k > 0x7fffffffull) return fail(op, GPURS_E_SIZE_OVERFLOW, "a matrix dimension exceeds 2^31 - 1");
    if (m == 0 || k == 0) return GPURS_OK;
    if (k % 128) return fail(op, GPURS_E_INVALID_VIEW, "the depth must be a multiple of 128");
    const uint64_t pitch = ld ? ld : k;
    if (pitch < k) return fail(op, GPURS_E_INVALID_VIEW, "a row pitch is smaller than the row");
    if (!dense || !values || !metadata) return fail(op, GPURS_E_INVALID_ARGUMENT, "null argument");
    if (dense % 16 || (pitch * 2) % 16 || values % 16 || metadata % 16 || violations % 4)
        return fail(op, GPURS_E_INVALID_VIEW, "buffers and the row pitch must be multiples of 16 bytes");
    if (overlap(values, m * k, dense, ((m - 1) * pitch + k) * 2) || overlap(metadata, gpurs_metadata_bytes(m, k), dense, ((m - 1) * pitch + k) * 2))
        return fail(op, GPURS_E_ALIASING, "an output overlaps the input");
    gpurs_gpu *gpu = stream->gpu;
    runtime::Enter enter(gpu);
    gpurs_kernel *kernel = nullptr;
    int result = runtime::builtin_kernel(gpu, "gpurs_compress_24", 0, &kernel);
    if (result != GPURS_OK) return result;
    const uint64_t spans = m * (k / 16);
    gpurs_launch_config config;
    std::memset(&config, 0, sizeof config);
    config.grid[0] = uint32_t(std::max<uint64_t>(1, std::min<uint64_t>((spans + 255) / 256, uint64_t(gpu->multiprocessors) * 8)));
    config.block[0] = 256;
    const void *source = reinterpret_cast<const void *>(dense);
    void *value_pointer = reinterpret_cast<void *>(values), *metadata_pointer = reinterpret_cast<void *>(metadata);
    void *violation_pointer = reinterpret_cast<void *>(violations);
    long long source_pitch = (long long)pitch;
    int rows = int(m), depth = int(k);
    void *arguments[7] = {&source, &source_pitch, &value_pointer, &metadata_pointer, &violation_pointer, &rows, &depth};
    return runtime::launch(kernel, stream, &config, arguments, true);
}

extern "C" int gpurs_quantize_e4m3(gpurs_stream *stream, uint64_t rows, uint64_t k, gpurs_device_ptr source, uint64_t ld, uint32_t block_rows,
                                   gpurs_device_ptr codes, gpurs_device_ptr scales) {
    const char *const op = "gpurs_quantize_e4m3";
    if (!stream) return fail(op, GPURS_E_INVALID_ARGUMENT, "null stream");
    if (block_rows != 1 && block_rows != 128) return fail(op, GPURS_E_INVALID_ARGUMENT, "block_rows must be 1 or 128");
    if (rows > 0x7fffffffull || k > 0x7fffffffull) return fail(op, GPURS_E_SIZE_OVERFLOW, "a matrix dimension exceeds 2^31 - 1");
    if (rows == 0 || k == 0) return GPURS_OK;
    const uint64_t pitch = ld ? ld : k;
    if (pitch < k) return fail(op, GPURS_E_INVALID_VIEW, "a row pitch is smaller than the row");
    if (!source || !codes || !scales) return fail(op, GPURS_E_INVALID_ARGUMENT, "null argument");
    if (k % 4 || source % 16 || (pitch * 4) % 16 || codes % 4 || scales % 4)
        return fail(op, GPURS_E_INVALID_VIEW, "k must be a multiple of 4, the source 16-byte aligned, the outputs 4-byte aligned");
    const uint64_t k_blocks = (k + 127) / 128, row_blocks = (rows + block_rows - 1) / block_rows;
    const uint64_t source_bytes = ((rows - 1) * pitch + k) * 4;
    if (overlap(codes, rows * k, source, source_bytes) || overlap(scales, row_blocks * k_blocks * 4, source, source_bytes))
        return fail(op, GPURS_E_ALIASING, "an output overlaps the input");
    gpurs_gpu *gpu = stream->gpu;
    runtime::Enter enter(gpu);
    gpurs_kernel *kernel = nullptr;
    int result = runtime::builtin_kernel(gpu, block_rows == 1 ? "gpurs_quantize_e4m3_rows" : "gpurs_quantize_e4m3_tiles", 0, &kernel);
    if (result != GPURS_OK) return result;
    const uint64_t blocks = row_blocks * k_blocks;
    gpurs_launch_config config;
    std::memset(&config, 0, sizeof config);
    // rows form: 8 warps = 8 blocks per CTA of 256 threads; tiles form: one 128 x 128 block per CTA of 1024 threads
    const uint64_t ctas = block_rows == 1 ? (blocks + 7) / 8 : blocks;
    config.grid[0] = uint32_t(std::max<uint64_t>(1, std::min<uint64_t>(ctas, uint64_t(gpu->multiprocessors) * (block_rows == 1 ? 8 : 2))));
    config.block[0] = block_rows == 1 ? 256 : 1024;
    const void *source_pointer = reinterpret_cast<const void *>(source);
    void *code_pointer = reinterpret_cast<void *>(codes), *scale_pointer = reinterpret_cast<void *>(scales);
    long long source_pitch = (long long)pitch;
    int row_count = int(rows), depth = int(k);
    void *arguments[6] = {&source_pointer, &source_pitch, &code_pointer, &scale_pointer, &row_count, &depth};
    return runtime::launch(kernel, stream, &config, arguments, true);
}

extern "C" size_t gpurs_mx_scale_bytes(uint64_t rows, uint64_t k, int right_operand) {
    const uint64_t k_blocks = (k + 127) / 128;
    return right_operand ? size_t(((rows + gemm::MX_BLOCK_N - 1) / gemm::MX_BLOCK_N) * k_blocks * 1024) : size_t(((rows + 127) / 128) * k_blocks * 512);
}

extern "C" int gpurs_quantize_mx_e4m3(gpurs_stream *stream, uint64_t rows, uint64_t k, gpurs_device_ptr source, uint64_t ld, int right_operand,
                                      gpurs_device_ptr codes, gpurs_device_ptr scales) {
    const char *const op = "gpurs_quantize_mx_e4m3";
    if (!stream) return fail(op, GPURS_E_INVALID_ARGUMENT, "null stream");
    if (right_operand != 0 && right_operand != 1) return fail(op, GPURS_E_INVALID_ARGUMENT, "right_operand must be 0 or 1");
    if (rows > 0x7fffffffull || k > 0x7fffffffull) return fail(op, GPURS_E_SIZE_OVERFLOW, "a matrix dimension exceeds 2^31 - 1");
    if (rows == 0 || k == 0) return GPURS_OK;
    const uint64_t pitch = ld ? ld : k;
    if (pitch < k) return fail(op, GPURS_E_INVALID_VIEW, "a row pitch is smaller than the row");
    if (!source || !codes || !scales) return fail(op, GPURS_E_INVALID_ARGUMENT, "null argument");
    if (k % 4 || source % 16 || (pitch * 4) % 16 || codes % 4 || scales % 16)
        return fail(op, GPURS_E_INVALID_VIEW, "k must be a multiple of 4, the source and the scales 16-byte aligned, the codes 4-byte aligned");
    const uint64_t source_bytes = ((rows - 1) * pitch + k) * 4, scale_bytes = gpurs_mx_scale_bytes(rows, k, right_operand);
    if (overlap(codes, rows * k, source, source_bytes) || overlap(scales, scale_bytes, source, source_bytes) || overlap(scales, scale_bytes, codes, rows * k))
        return fail(op, GPURS_E_ALIASING, "an output overlaps the input or the other output");
    gpurs_gpu *gpu = stream->gpu;
    runtime::Enter enter(gpu);
    gpurs_kernel *kernel = nullptr;
    int result = runtime::builtin_kernel(gpu, "gpurs_quantize_mx_e4m3", 0, &kernel);
    if (result != GPURS_OK) return result;
    // entries of the tiled array that no element maps to (rows past the matrix, the unused quarter of B's second block): scale 1
    GPURS_TRY(gpu->api, cuMemsetD8Async(scales, 127, scale_bytes, stream->handle));
    const uint64_t spans = rows * ((k + 127) / 128);
    gpurs_launch_config config;
    std::memset(&config, 0, sizeof config);
    config.grid[0] = uint32_t(std::max<uint64_t>(1, std::min<uint64_t>((spans + 7) / 8, uint64_t(gpu->multiprocessors) * 8)));
    config.block[0] = 256;
    const void *source_pointer = reinterpret_cast<const void *>(source);
    void *code_pointer = reinterpret_cast<void *>(codes), *scale_pointer = reinterpret_cast<void *>(scales);
    long long source_pitch = (long long)pitch;
    int row_count = int(rows), depth = int(k), right = right_operand;
    void *arguments[7] = {&source_pointer, &source_pitch, &code_pointer, &scale_pointer, &row_count, &depth, &right};
    return runtime::launch(kernel, stream, &config, arguments, true);
}

extern "C" int gpurs_self_test_timeout(gpurs_stream *stream) {
    if (!stream) return fail("gpurs_self_test_timeout", GPURS_E_INVALID_ARGUMENT, "null stream");
    gpurs_gpu *gpu = stream->gpu;
    runtime::Enter enter(gpu);
    gpurs_kernel *kernel = nullptr;
    int result = runtime::builtin_kernel(gpu, "gpurs_wait_probe", 0, &kernel);
    if (result != GPURS_OK) return result;
    gpurs_launch_config config;
    std::memset(&config, 0, sizeof config);
    config.grid[0] = 1;
    config.block[0] = 32;
    void *status = reinterpret_cast<void *>(gpu->status);
    void *arguments[1] = {&status};
    return runtime::launch(kernel, stream, &config, arguments);
}

namespace {
// Host mirror of gemm::GroupedParams (kernels/gemm_grouped_tcgen05.cuh).
struct GroupedParams {
    void *c;
    long long ldc;
    const void *input;
    long long lda;
    const unsigned int *routes;
    const unsigned int *offsets;
    unsigned int *status;
    int rows, tokens, n, k, experts, tiles_n, vector_stores;
};
}  // namespace

extern "C" int gpurs_matmul_grouped(gpurs_stream *stream, const gpurs_grouped_desc *desc, gpurs_device_ptr input, gpurs_device_ptr routes,
                                    gpurs_device_ptr offsets, gpurs_device_ptr weight, gpurs_device_ptr output) {
    const char *const op = "gpurs_matmul_grouped";
    if (!stream || !desc) return fail(op, GPURS_E_INVALID_ARGUMENT, "null stream or descriptor");
    if (desc->a_type != GPURS_F16 && desc->a_type != GPURS_BF16) return fail(op, GPURS_E_INVALID_ARGUMENT, "16-bit operands only");
    if (desc->c_type != desc->a_type && desc->c_type != GPURS_F32) return fail(op, GPURS_E_INVALID_ARGUMENT, "unsupported output type");
    const uint64_t rows = desc->rows, tokens = desc->tokens, n = desc->n, k = desc->k, experts = desc->experts;
    if (rows > 0x7fffffffull || tokens > 0x7fffffffull || k > 0x7fffffffull || experts > 65536 || experts * n > 0x7fffffffull)
        return fail(op, GPURS_E_SIZE_OVERFLOW, "a dimension exceeds what the kernel indexes");
    if (rows == 0 || n == 0 || experts == 0) return GPURS_OK;
    if (k == 0 || tokens == 0) return fail(op, GPURS_E_INVALID_VIEW, "empty depth or no input rows");
    const uint64_t lda = desc->lda ? desc->lda : k, ldc = desc->ldc ? desc->ldc : n;
    if (lda < k || ldc < n) return fail(op, GPURS_E_INVALID_VIEW, "a row pitch is smaller than the row");
    if (!input || !routes || !offsets || !weight || !output) return fail(op, GPURS_E_INVALID_ARGUMENT, "null argument");
    const uint64_t ob = desc->c_type == GPURS_F32 ? 4 : 2;
    if (k % 8 || input % 16 || weight % 16 || (lda * 2) % 16 || routes % 4 || offsets % 4 || output % ob)
        return fail(op, GPURS_E_INVALID_VIEW, "k must be a multiple of 8, operands 16-byte aligned with 16-byte row pitches");
    const uint64_t out_bytes = ((rows - 1) * ldc + n) * ob;
    if (overlap(output, out_bytes, input, ((tokens - 1) * lda + k) * 2) || overlap(output, out_bytes, weight, experts * n * k * 2) ||
        overlap(output, out_bytes, routes, rows * 4) || overlap(output, out_bytes, offsets, (experts + 1) * 4))
        return fail(op, GPURS_E_ALIASING, "the output overlaps an input");
    gpurs_gpu *gpu = stream->gpu;
    runtime::Enter enter(gpu);
    char name[96];
    std::snprintf(name, sizeof name, "gpurs_gemm_grouped_%s_%s", desc->a_type == GPURS_F16 ? "f16" : "bf16",
                  desc->c_type == GPURS_F32 ? "f32" : (desc->a_type == GPURS_F16 ? "f16" : "bf16"));
    const uint32_t shared_bytes = gemm::SharedLayout<gemm::BLOCK_N, 1, gemm::STAGES_SINGLE>::DYNAMIC_BYTES;
    gpurs_kernel *kernel = nullptr;
    int result = runtime::builtin_kernel(gpu, name, shared_bytes, &kernel);
    if (result != GPURS_OK) return result;
    alignas(64) CUtensorMap map_w;
    const uint64_t dims_w[2] = {k, experts * n}, stride_w[1] = {k * 2};
    const uint32_t box_w[2] = {64, uint32_t(gemm::BLOCK_N)};
    result = gpurs_tensor_map_encode(gpu, &map_w, desc->a_type, 2, weight, dims_w, stride_w, box_w, 3, 3);
    if (result != GPURS_OK) return result;
    GroupedParams params;
    std::memset(&params, 0, sizeof params);
    params.c = reinterpret_cast<void *>(output);
    params.ldc = (long long)ldc;
    params.input = reinterpret_cast<const void *>(input);
    params.lda = (long long)lda;
    params.routes = reinterpret_cast<const unsigned int *>(routes);
    params.offsets = reinterpret_cast<const unsigned int *>(offsets);
    params.status = reinterpret_cast<unsigned int *>(gpu->status);
    params.rows = int(rows), params.tokens = int(tokens), params.n = int(n), params.k = int(k), params.experts = int(experts);
    params.tiles_n = int((n + gemm::BLOCK_N - 1) / gemm::BLOCK_N);
    params.vector_stores = (output % 16 == 0 && (ldc * ob) % 16 == 0) ? 1 : 0;
    // The tile count depends on the offsets, which live on the device: at most one ragged tile per expert beyond
    // rows / 128.  The persistent blocks stop at the real count.
    const uint64_t tile_bound = ((rows + gemm::BLOCK_M - 1) / gemm::BLOCK_M + experts) * uint64_t(params.tiles_n);
    gpurs_launch_config config;
    std::memset(&config, 0, sizeof config);
    config.grid[0] = uint32_t(std::min<uint64_t>(tile_bound, uint64_t(gpu->multiprocessors)));
    config.block[0] = gemm::GROUPED_THREADS;
    config.shared_bytes = shared_bytes;
    void *arguments[2] = {&map_w, &params};
    return runtime::launch(kernel, stream, &config, arguments, true);
}
