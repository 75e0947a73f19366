// Block-scaled FP8 (E4M3) GEMM for sm_100a:
//
//     C[m, n] = sum_kb  sA[m, kb] * sB[n / 128, kb] * ( sum_{k in block kb} A[m, k] * B[n, k] )
//
// A is M x K with one fp32 scale per row and 128-deep K-block, B is N x K with one fp32 scale per
// 128 x 128 block.  The reference only ships the raw FP8 instruction for this
// (crates/gpurs/src/gpu/tensor/blackwell/instruction.rs:13-21, tensor_memory.rs:136-165) and no kernel.
//
// The scales change with every K-block, so the tensor core cannot accumulate across blocks.  Instead each
// 128-deep block is multiplied into a fresh TMEM accumulator (one pipeline stage = one block = 4
// tcgen05.mma of K = 32), and the epilogue warps promote it: TMEM -> registers, times the block's scale,
// added into fp32 register accumulators, while the tensor core already works on the next block in the
// other TMEM accumulator.  Eight epilogue warps share the work: warps 2..5 own columns 0..127 of the
// tile, warps 6..9 columns 128..255 (one 128-wide scale block of B each), each warp its 32 TMEM lanes.
#pragma once
#include "gemm_tcgen05.cuh"

namespace gemm {

constexpr int SCALED_EPILOGUE_WARPS = 8;
constexpr int PRODUCER_REGISTERS = 40;      // warpgroup 0 after setmaxnreg.dec
constexpr int PROMOTION_REGISTERS = 232;    // warpgroups 1 and 2 after setmaxnreg.inc: 128 sums + 64 staged values + addressing
static_assert(128 * PRODUCER_REGISTERS + 256 * PROMOTION_REGISTERS <= 65536, "register budgets exceed the register file");
constexpr int SCALE_BLOCK = 128;             // K-depth and B-row extent of one scale

// KIND / ELEMENT_FORMAT as in gemm_body.  SCALED = true multiplies every 128-byte K-block by
// scale_a[row][block] * scale_b[column / 128][block]; SCALED = false only promotes (scale 1): the fp32
// accumulator of the tensor core truncates after every instruction, so a long K loop drifts towards
// zero, while sums promoted to registers every K-block are added with round-to-nearest.  The fp32
// (three-pass TF32) product uses the unscaled form.
// STREAMK: the K-blocks of the tiles of a split round are spread over the CTA groups (gemm_schedule.hpp), as in gemm_body: a
// group's share of a tile is promoted like a whole tile, written to scratch as a 32-bit partial tile, and whichever
// promotion warp brings the last part of its 32 rows x 128 columns adds the parts in the contributors' order and stores.
template <int KIND, int ELEMENT_FORMAT, int OUT, bool SCALED, int CTA_GROUP, int STAGES, bool STREAMK = false>
__device__ __forceinline__ void gemm_promoted_body(const CUtensorMap *map_a, const CUtensorMap *map_b, const Params &p) {
    constexpr int BN = BLOCK_N;
    using L = SharedLayout<BN, CTA_GROUP, STAGES>;
    constexpr uint32_t TMEM_COLUMNS = 2 * BN;
    // SPLIT issues every K-block as two products of 128 columns, each into its own accumulator with its own pair of
    // barriers (four accumulators in flight instead of two).
    constexpr bool SPLIT = false;   // measured: two 128-column products per block ran slower (1359 vs 1665 TFLOP/s) than one of 256
    constexpr int HALVES = SPLIT ? 2 : 1;
    // K-blocks multiplied into one TMEM accumulator before it is promoted.  Scales change with every block, so a scaled
    // product promotes every block.  The unscaled form only has to keep the tensor core's truncating fp32 adds short: four
    // blocks (16 instructions) per accumulator keep that error near 1e-6 relative and cost a quarter of the hand-offs.
    constexpr int PERIOD = SCALED ? 1 : 4;
    static_assert(!SPLIT, "the two-halves variant was measured slower and is not wired into the loops below");
    constexpr int MMA_N = BN / HALVES;
    constexpr uint32_t IDESC = instruction_descriptor(1, ELEMENT_FORMAT, BLOCK_M * CTA_GROUP, MMA_N);   // f32 accumulate
    // A tcgen05.commit costs the issuing thread about 250 cycles, half of what the tensor core needs for a K-block.  Where an
    // accumulator holds exactly one K-block (the scaled product on one CTA), its completion is also the moment the K-block's
    // shared-memory stage is free: a promotion warp that has seen the accumulator complete hands the stage back to the
    // producer, and the MMA thread issues one commit per K-block instead of two.
    constexpr bool PROMOTION_FREES_STAGES = SCALED && CTA_GROUP == 1;
    constexpr int ELEMENT_BYTES = KIND == ptx::KIND_F16 ? 2 : (KIND == ptx::KIND_TF32 ? 4 : 1);
    constexpr int BLOCK_K = ROW_BYTES / ELEMENT_BYTES;   // elements of K per stage (128 for FP8: one scale block)

    extern __shared__ uint8_t raw_shared[];
    const uint32_t base = (ptx::smem_u32(raw_shared) + 1023u) & ~1023u;
    uint8_t *aligned = raw_shared + (base - ptx::smem_u32(raw_shared));
    volatile uint32_t *tmem_slot = reinterpret_cast<volatile uint32_t *>(aligned + L::TMEM_SLOT_OFFSET);
    volatile uint32_t *abort_flag = reinterpret_cast<volatile uint32_t *>(aligned + L::ABORT_OFFSET);

    auto stage_a = [&](int s) { return base + uint32_t(s) * L::STAGE_BYTES; };
    auto stage_b = [&](int s) { return base + uint32_t(s) * L::STAGE_BYTES + L::A_BYTES; };
    auto full_bar = [&](int s) { return base + L::BARRIER_OFFSET + uint32_t(s) * 8; };
    auto empty_bar = [&](int s) { return base + L::BARRIER_OFFSET + uint32_t(STAGES + s) * 8; };
    auto acc_full_bar = [&](int a) { return base + L::BARRIER_OFFSET + uint32_t(2 * STAGES + a) * 8; };
    auto acc_empty_bar = [&](int a) { return base + L::BARRIER_OFFSET + uint32_t(2 * STAGES + 4 + a) * 8; };

    const int warp = threadIdx.x / 32;
    const uint32_t lane = ptx::lane_id();
    const uint32_t cta_rank = CTA_GROUP == 2 ? ptx::cluster_cta_rank() : 0u;
    const bool leader = cta_rank == 0;
    const int cluster_id = blockIdx.x / CTA_GROUP;
    const int cluster_count = gridDim.x / CTA_GROUP;
    const int tile_count = p.tiles_m * p.tiles_n;
    const int k_blocks = (p.k + BLOCK_K - 1) / BLOCK_K;

    if (threadIdx.x == 0) {
        *abort_flag = 0;
        for (int s = 0; s < STAGES; s++) {
            ptx::mbarrier_init(full_bar(s), 1);
            ptx::mbarrier_init(empty_bar(s), 1);
        }
        for (int a = 0; a < 4; a++) {
            ptx::mbarrier_init(acc_full_bar(a), 1);
            ptx::mbarrier_init(acc_empty_bar(a), SCALED_EPILOGUE_WARPS / HALVES * CTA_GROUP);
        }
        ptx::fence_mbarrier_init();
        ptx::prefetch_tensor_map(map_a);
        ptx::prefetch_tensor_map(map_b);
    }
    if (warp == 1) {
        ptx::tmem_alloc<CTA_GROUP>(ptx::smem_u32(const_cast<uint32_t *>(tmem_slot)), TMEM_COLUMNS);
        ptx::tmem_relinquish<CTA_GROUP>();
    }
    ptx::tcgen05_fence_before();
    __syncthreads();
    if constexpr (CTA_GROUP == 2) {
        ptx::cluster_arrive();
        ptx::cluster_wait();
    }
    ptx::tcgen05_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    // Everything above touched no global memory and may have overlapped the previous kernel of the stream.
    ptx::grid_dependency_wait();
    ptx::grid_dependency_launch();

    if (warp < 4) ptx::registers_decrease<PRODUCER_REGISTERS>();
    if (warp == 0) {
        // ------------------------------------------------------------------ producer (as in the dense kernel)
        if (lane == 0) {
            int stage = 0;
            uint32_t phase = 0;
            bool ok = true;
            WorkWalker<STREAMK> walker(tile_count, k_blocks, cluster_id, cluster_count, p.split_tiles);
            WorkItem item;
            while (ok && walker.next(item)) {
                const int tile = item.tile;
                int tile_m, tile_n;
                tile_position(tile, p, tile_m, tile_n);
                const int row_a = (tile_m * CTA_GROUP + int(cta_rank)) * BLOCK_M;
                const int row_b = tile_n * BN + int(cta_rank) * L::B_ROWS;
                for (int kb = item.kb_begin; kb < item.kb_end; kb++) {
                    if (!ptx::mbarrier_wait(empty_bar(stage), phase ^ 1, abort_flag)) {
                        report(p, abort_flag, STATUS_PRODUCER_TIMEOUT, tile, kb);
                        ok = false;
                        break;
                    }
                    if constexpr (CTA_GROUP == 1) {
                        ptx::mbarrier_arrive_expect_tx(full_bar(stage), L::STAGE_BYTES);
                        ptx::tma_load_2d(stage_a(stage), map_a, kb * BLOCK_K, row_a, full_bar(stage));
                        ptx::tma_load_2d(stage_b(stage), map_b, kb * BLOCK_K, row_b, full_bar(stage));
                    } else {
                        if (leader) ptx::mbarrier_arrive_expect_tx(full_bar(stage), 2 * L::STAGE_BYTES);
                        const uint32_t leader_bar = ptx::map_to_cta(full_bar(stage), 0);
                        ptx::tma_load_2d_pair(stage_a(stage), map_a, kb * BLOCK_K, row_a, leader_bar);
                        ptx::tma_load_2d_pair(stage_b(stage), map_b, kb * BLOCK_K, row_b, leader_bar);
                    }
                    if (++stage == STAGES) { stage = 0; phase ^= 1; }
                }
            }
            for (int s = 0; s < STAGES && ok; s++) {
                ok = ptx::mbarrier_wait(empty_bar(stage), phase ^ 1, abort_flag);
                if (++stage == STAGES) { stage = 0; phase ^= 1; }
            }
        }
    } else if (warp == 1) {
        // ------------------------------------------------------------------ MMA issuer: one accumulator per K-block
        if (lane == 0 && leader) {
            int stage = 0;
            uint32_t phase = 0;
            int acc = 0;
            uint32_t acc_phase = 0;
            bool ok = true;
            const uint64_t a_desc0 = ptx::smem_descriptor_k_major_sw128(stage_a(0)), b_desc0 = ptx::smem_descriptor_k_major_sw128(stage_b(0));
            constexpr uint64_t STAGE_STEP = uint64_t(L::STAGE_BYTES >> 4);
            WorkWalker<STREAMK> walker(tile_count, k_blocks, cluster_id, cluster_count, p.split_tiles);
            WorkItem item;
            while (ok && walker.next(item)) {
                const int tile = item.tile;
                for (int first = item.kb_begin; first < item.kb_end && ok; first += PERIOD) {
                    // one accumulator takes PERIOD K-blocks, then goes to the promotion warps
                    const int slot = acc * 2;
                    if (!ptx::mbarrier_wait<CTA_GROUP == 2>(acc_empty_bar(slot), acc_phase ^ 1, abort_flag)) {
                        report(p, abort_flag, STATUS_MMA_TIMEOUT, tile, first);
                        ok = false;
                        break;
                    }
                    ptx::tcgen05_fence_after();
                    const uint32_t d_tmem = tmem_base + uint32_t(acc) * BN;
                    const int last = min(first + PERIOD, item.kb_end);
                    for (int kb = first; kb < last; kb++) {
                        if (!ptx::mbarrier_wait(full_bar(stage), phase, abort_flag)) {
                            report(p, abort_flag, STATUS_MMA_TIMEOUT, tile, kb);
                            ok = false;
                            break;
                        }
                        ptx::tcgen05_fence_after();
                        const uint64_t a_desc = a_desc0 + uint64_t(stage) * STAGE_STEP, b_desc = b_desc0 + uint64_t(stage) * STAGE_STEP;
                        ptx::tcgen05_mma<KIND, CTA_GROUP>(d_tmem, a_desc, b_desc, IDESC, uint32_t(kb != first));
#pragma unroll
                        for (int j = 1; j < ROW_BYTES / MMA_K_BYTES; j++)
                            ptx::tcgen05_mma_accumulate<KIND, CTA_GROUP>(d_tmem, a_desc + uint64_t(j * (MMA_K_BYTES >> 4)), b_desc + uint64_t(j * (MMA_K_BYTES >> 4)), IDESC);
                        if constexpr (PROMOTION_FREES_STAGES) {}
                        else if constexpr (CTA_GROUP == 1) ptx::tcgen05_commit(empty_bar(stage));
                        else ptx::tcgen05_commit_pair(empty_bar(stage), 0x3);
                        if (++stage == STAGES) { stage = 0; phase ^= 1; }
                    }
                    if (!ok) break;
                    if constexpr (CTA_GROUP == 1) ptx::tcgen05_commit(acc_full_bar(slot));
                    else ptx::tcgen05_commit_pair(acc_full_bar(slot), 0x3);
                    if (++acc == 2) { acc = 0; acc_phase ^= 1; }
                }
            }
        }
    } else if (warp >= 4) {
        // ------------------------------------------------------------------ promotion + epilogue
        ptx::registers_increase<PROMOTION_REGISTERS>();
        const int epilogue_warp = warp - 4;
        const int quadrant = warp % 4;             // TMEM lanes this warp may read
        const int half = epilogue_warp / 4;        // which 128 columns of the tile
        const int scale_pitch = k_blocks;
        int acc = 0;
        uint32_t acc_phase = 0;
        int release_stage = 0;
        bool ok = true;
        WorkWalker<STREAMK> walker(tile_count, k_blocks, cluster_id, cluster_count, p.split_tiles);
        WorkItem item;
        while (ok && walker.next(item)) {
            const int tile = item.tile;
            int tile_m, tile_n;
            tile_position(tile, p, tile_m, tile_n);
            const int row = (tile_m * CTA_GROUP + int(cta_rank)) * BLOCK_M + quadrant * 32 + int(lane);
            const int column = tile_n * BN + half * SCALE_BLOCK;
            const float *row_scales = SCALED ? p.scale_a + size_t(min(row, p.m - 1)) * scale_pitch : nullptr;
            const float *block_scales = SCALED ? p.scale_b + size_t(min(column, p.n - 1) / SCALE_BLOCK) * scale_pitch : nullptr;
            float sums[SCALE_BLOCK];
#pragma unroll
            for (int i = 0; i < SCALE_BLOCK; i++) sums[i] = 0.0f;
            float scale = SCALED ? __ldg(row_scales + item.kb_begin) * __ldg(block_scales + item.kb_begin) : 1.0f;
            // Scales are fetched two blocks ahead and multiplied one block ahead: a warp issues in order, and a product placed
            // right behind its loads would hold the warp for the whole trip to L2.
            const int second = min(item.kb_begin + 1, k_blocks - 1);
            float row_part = SCALED ? __ldg(row_scales + second) : 1.0f, block_part = SCALED ? __ldg(block_scales + second) : 1.0f;
            for (int kb = item.kb_begin; kb < item.kb_end; kb += PERIOD) {
                const float next_scale = row_part * block_part;
                if constexpr (SCALED) {
                    const int ahead = min(kb + 2, k_blocks - 1);
                    row_part = __ldg(row_scales + ahead), block_part = __ldg(block_scales + ahead);
                }
                const int slot = acc * 2 + (SPLIT ? half : 0);
                const bool ready = ptx::mbarrier_wait(acc_full_bar(slot), acc_phase, abort_flag);
                if (!__all_sync(0xffffffffu, ready)) {
                    if (lane == 0) report(p, abort_flag, STATUS_EPILOGUE_TIMEOUT, tile, kb);
                    ok = false;
                    break;
                }
                ptx::tcgen05_fence_after();
                if constexpr (PROMOTION_FREES_STAGES) {
                    // the K-block's products are complete: its stage goes back to the producer
                    if (epilogue_warp == 0 && lane == 0) ptx::mbarrier_arrive(empty_bar(release_stage));
                    if (++release_stage == STAGES) release_stage = 0;
                }
                const uint32_t address = tmem_base + (uint32_t(quadrant * 32) << 16) + uint32_t(acc) * BN + uint32_t(half * SCALE_BLOCK);
#pragma unroll
                for (int pair = 0; pair < SCALE_BLOCK / 64; pair++) {
                    // two 32-column loads in flight per wait: the TMEM round trip is paid twice per block, not four times
                    uint32_t first[32], second[32];
                    ptx::tmem_load_32x32(address + uint32_t(pair * 64), first);
                    ptx::tmem_load_32x32(address + uint32_t(pair * 64 + 32), second);
                    ptx::tmem_load_wait();
                    if (pair == SCALE_BLOCK / 64 - 1) {
                        // the last values have left the accumulator: hand it back before the remaining arithmetic
                        ptx::tcgen05_fence_before();
                        __syncwarp();
                        if (lane == 0) {
                            // nothing is published through ordinary memory (the accumulator has been read out when
                            // tcgen05.wait::ld returns): no release, which at cluster scope would wait for this thread's stores
                            if (CTA_GROUP == 1 || leader) ptx::mbarrier_arrive(acc_empty_bar(slot));
                            else ptx::mbarrier_arrive_cluster_relaxed(ptx::map_to_cta(acc_empty_bar(slot), 0));
                        }
                    }
#pragma unroll
                    for (int i = 0; i < 32; i += 2) {
                        // two columns per instruction (fma.rn.f32x2): half the issue slots of scalar FMAs
                        ptx::fma2(sums[pair * 64 + i], sums[pair * 64 + i + 1], first[i], first[i + 1], scale);
                        ptx::fma2(sums[pair * 64 + 32 + i], sums[pair * 64 + 32 + i + 1], second[i], second[i + 1], scale);
                    }
                }
                if (++acc == 2) { acc = 0; acc_phase ^= 1; }
                scale = next_scale;
            }
            if (!ok) break;
            if (STREAMK && item.split_tile >= 0) {
                // This group multiplied only its share of the tile's K-blocks: the sums go to scratch as one part of the tile, laid
                // out as in gemm_body ([group of four columns][row] x 16 bytes), and the warp that brings the last part of these
                // 32 rows x 128 columns adds the parts up in the contributors' order and stores.  Nobody waits for anybody.
                constexpr int TILE_ROWS = BLOCK_M * CTA_GROUP;
                constexpr size_t PART = size_t(TILE_ROWS) * BN / 4;      // one part, in 16-byte units
                const int row_in_tile = int(cta_rank) * BLOCK_M + quadrant * 32 + int(lane);
                uint4 *parts = reinterpret_cast<uint4 *>(p.partials) + size_t(item.split_tile) * p.max_contributors * PART + size_t(half) * (SCALE_BLOCK / 4) * TILE_ROWS +
                               row_in_tile;
                uint4 *mine = parts + size_t(item.contributor) * PART;
#pragma unroll
                for (int i = 0; i < SCALE_BLOCK / 4; i++)
                    mine[size_t(i) * TILE_ROWS] = make_uint4(__float_as_uint(sums[4 * i]), __float_as_uint(sums[4 * i + 1]), __float_as_uint(sums[4 * i + 2]),
                                                             __float_as_uint(sums[4 * i + 3]));
                unsigned int *counter = p.split_counters + item.split_tile * (8 * CTA_GROUP) + int(cta_rank) * 8 + half * 4 + quadrant;
                __threadfence();
                __syncwarp();
                unsigned int earlier = 0;
                if (lane == 0) earlier = atomicAdd(counter, 1u);
                earlier = __shfl_sync(0xffffffffu, earlier, 0);
                if (earlier == unsigned(item.contributors - 1)) {
                    __threadfence();
                    if (lane == 0) *counter = 0;       // ready for the next launch
#pragma unroll 1
                    for (int chunk = 0; chunk < SCALE_BLOCK / 32; chunk++) {
                        uint32_t sum[32];
#pragma unroll
                        for (int i = 0; i < 32; i++) sum[i] = 0;    // +0.0f: the first part is added to it exactly
                        for (int q = 0; q < item.contributors; q++) {
                            uint4 loaded[8];
#pragma unroll
                            for (int i = 0; i < 8; i++) loaded[i] = __ldcg(parts + size_t(q) * PART + size_t(chunk * 8 + i) * TILE_ROWS);
#pragma unroll
                            for (int i = 0; i < 8; i++) {
                                const uint32_t w[4] = {loaded[i].x, loaded[i].y, loaded[i].z, loaded[i].w};
#pragma unroll
                                for (int j = 0; j < 4; j++) sum[4 * i + j] = __float_as_uint(__fadd_rn(__uint_as_float(sum[4 * i + j]), __uint_as_float(w[j])));
                            }
                        }
                        store_chunk<OUT>(p, sum, row, column + chunk * 32);
                    }
                }
            } else {
#pragma unroll
                for (int chunk = 0; chunk < SCALE_BLOCK / 32; chunk++) {
                    uint32_t values[32];
#pragma unroll
                    for (int i = 0; i < 32; i++) values[i] = __float_as_uint(sums[chunk * 32 + i]);
                    store_chunk<OUT>(p, values, row, column + chunk * 32);
                }
            }
        }
    }

    // ---------------------------------------------------------------------- teardown
    __syncwarp();
    ptx::tcgen05_fence_before();
    __syncthreads();
    if (*abort_flag != 0 && threadIdx.x == 0) {
        const unsigned long long start = ptx::global_timer();
        while (ptx::global_timer() - start < 2000000ull) __nanosleep(1000);
    }
    __syncwarp();
    if constexpr (CTA_GROUP == 2) {
        ptx::cluster_arrive();
        ptx::cluster_wait();
    } else {
        __syncthreads();
    }
    if (warp == 1) {
        ptx::tcgen05_fence_after();
        ptx::tmem_dealloc<CTA_GROUP>(tmem_base, TMEM_COLUMNS);
    }
}

}  // namespace gemm
