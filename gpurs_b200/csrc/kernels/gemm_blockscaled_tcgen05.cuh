// Block-scaled FP8 (E4M3) GEMM on CTA pairs, four accumulators in flight:
//
//     C[m, n] = sum_kb  sA[m, kb] * sB[n / 128, kb] * ( sum_{k in block kb} A[m, k] * B[n, k] )
//
// Same arithmetic as gemm_promoted_body (gemm_scaled_tcgen05.cuh): every 128-deep K-block is multiplied into a fresh
// accumulator in tensor memory and promoted -- TMEM -> registers, times the block's scale, added in fp32 -- by the CUDA
// cores.  What bounds that scheme is the hand-off of the accumulator: from the last tcgen05.mma of a block to the first
// of the block that reuses its columns, the completion, the wake-up of the promotion warps, the drain and the hand-back
// take about 1300 cycles, and with two 256-column accumulators only 512 cycles of tensor work cover them.  Here a CTA pair
// shares a 256 x 256 tile and every K-block is issued as TWO products of 128 columns (cta_group::2, M = 256, N = 128), each
// into its own quarter of tensor memory with its own pair of barriers: four accumulators are in flight, three products
// (768 cycles) run between the end of one and the reuse of its columns, and the pair keeps the operand traffic of a
// 256 x 256 tile (64 bytes per clock and SM from L2; a 128-column product on ONE CTA would read shared memory at its full
// bandwidth, which is why the one-CTA kernel cannot be split this way).
//
// Two more things had to go for that to pay, both found with clock stamps inside the kernel:
//   * a hand-back with `mbarrier.arrive.release.cluster` makes the arriving thread wait for every memory operation it has
//     in flight, about 1300 cycles per product; the promotion warps of the leader arrive on their own CTA's barrier, those of
//     the other CTA with a relaxed remote arrive (they publish nothing through ordinary memory: the accumulator has been read
//     out when tcgen05.wait::ld returns);
//   * every tcgen05.commit costs the thread that issues it about 250 cycles, as much as the tensor core needs for one whole
//     product, so one issuing thread is outrun by the tensor core.  THREE threads (warps 1..3 of the leader) issue the
//     products in rotation, each tracking its own products with its own commits, and the shared-memory stages are handed back
//     to the producer by the promotion warps (a stage is free when the products of both halves have been seen complete)
//     instead of by a third commit per K-block.
//
// Roles (384 threads): warp 0 TMA producer, warps 1..3 MMA issuers (leader CTA), warps 4..11 promotion: warp w owns TMEM
// lanes 32 * (w % 4) .. +31 and the columns of half (w - 4) / 4, which are exactly one 128-wide scale block of B.  The
// epilogue stages boxes of 32 rows x 128 bytes in shared memory and hands them to the TMA unit.
#pragma once
#include "gemm_tcgen05.cuh"

namespace gemm {

constexpr int SCALE_BLOCK_COLUMNS = 128;           // columns of C (rows of B) that share one scale of B
constexpr int BLOCKSCALED_THREADS = 384;
constexpr int BLOCKSCALED_STAGES = 6;              // 6 x 32 KiB of operands per CTA
constexpr int BLOCKSCALED_PRODUCER_REGISTERS = 40;
constexpr int BLOCKSCALED_PROMOTION_REGISTERS = 232;

struct BlockScaledLayout {
    static constexpr int A_BYTES = BLOCK_M * ROW_BYTES;              // this CTA's 128 rows of A
    static constexpr int B_HALF_BYTES = 64 * ROW_BYTES;              // this CTA's 64 rows of one 128-column half of the B tile
    static constexpr int STAGE_BYTES = A_BYTES + 2 * B_HALF_BYTES;   // 32 KiB
    static constexpr int BARRIER_OFFSET = BLOCKSCALED_STAGES * STAGE_BYTES;
    // full[STAGES], empty[STAGES], accumulator_full[4], accumulator_empty[4] (+ 4 spare)
    static constexpr int NUM_BARRIERS = 2 * BLOCKSCALED_STAGES + 12;
    static constexpr int TMEM_SLOT_OFFSET = BARRIER_OFFSET + NUM_BARRIERS * 8;
    static constexpr int ABORT_OFFSET = TMEM_SLOT_OFFSET + 4;
    static constexpr int ISSUED_OFFSET = ABORT_OFFSET + 4;           // products issued so far into each of the four accumulators
    static constexpr int STAGING_OFFSET = ((ISSUED_OFFSET + 16 + 1023) / 1024) * 1024;
    static constexpr int STAGING_BYTES = 8 * 32 * ROW_BYTES;         // one box of 32 rows x 128 bytes per promotion warp
    static constexpr int TOTAL = STAGING_OFFSET + STAGING_BYTES;
    static constexpr int DYNAMIC_BYTES = TOTAL + 1024;
    static_assert(DYNAMIC_BYTES <= 232448, "more than the 227 KiB a CTA may have");
    static_assert(DYNAMIC_BYTES == BLOCKSCALED_SHARED, "the host sizes the launch from gemm_params.hpp");
};

constexpr int BLOCKSCALED_ISSUERS = 3;             // threads that issue the products in rotation

template <int OUT>
__device__ __forceinline__ void gemm_blockscaled_body(const CUtensorMap *map_a, const CUtensorMap *map_b, const CUtensorMap *map_c, const Params &p) {
    using L = BlockScaledLayout;
    constexpr int BN = 256, HALF = 128, STAGES = BLOCKSCALED_STAGES;
    constexpr uint32_t IDESC = instruction_descriptor(1, 0, 2 * BLOCK_M, HALF);     // f32 accumulate, E4M3 operands, M = 256, N = 128
    constexpr int BLOCK_K = ROW_BYTES;                                              // 128 elements: one scale block

    extern __shared__ uint8_t raw_shared[];
    const uint32_t base = (ptx::smem_u32(raw_shared) + 1023u) & ~1023u;
    uint8_t *aligned = raw_shared + (base - ptx::smem_u32(raw_shared));
    volatile uint32_t *tmem_slot = reinterpret_cast<volatile uint32_t *>(aligned + L::TMEM_SLOT_OFFSET);
    volatile uint32_t *abort_flag = reinterpret_cast<volatile uint32_t *>(aligned + L::ABORT_OFFSET);
    volatile uint32_t *issued = reinterpret_cast<volatile uint32_t *>(aligned + L::ISSUED_OFFSET);

    auto stage_a = [&](int s) { return base + uint32_t(s) * L::STAGE_BYTES; };
    auto stage_b = [&](int s, int half) { return base + uint32_t(s) * L::STAGE_BYTES + L::A_BYTES + uint32_t(half) * L::B_HALF_BYTES; };
    auto full_bar = [&](int s) { return base + L::BARRIER_OFFSET + uint32_t(s) * 8; };
    auto empty_bar = [&](int s) { return base + L::BARRIER_OFFSET + uint32_t(STAGES + s) * 8; };
    auto acc_full_bar = [&](int a) { return base + L::BARRIER_OFFSET + uint32_t(2 * STAGES + a) * 8; };
    auto acc_empty_bar = [&](int a) { return base + L::BARRIER_OFFSET + uint32_t(2 * STAGES + 4 + a) * 8; };

    const int warp = threadIdx.x / 32;
    const uint32_t lane = ptx::lane_id();
    const uint32_t cta_rank = ptx::cluster_cta_rank();
    const bool leader = cta_rank == 0;
    const int cluster_id = blockIdx.x / 2;
    const int cluster_count = gridDim.x / 2;
    const int tile_count = p.tiles_m * p.tiles_n;
    const int k_blocks = (p.k + BLOCK_K - 1) / BLOCK_K;
    // K-blocks this pair multiplies in all: the stage ring, the accumulators and their barriers run through them without a
    // break at tile borders
    const int my_tiles = cluster_id < tile_count ? (tile_count - cluster_id + cluster_count - 1) / cluster_count : 0;
    const long long all_blocks = (long long)my_tiles * k_blocks;      // the host keeps 2 * all_blocks below 2^32

    if (threadIdx.x == 0) {
        *abort_flag = 0;
        for (int a = 0; a < 4; a++) issued[a] = 0;
        for (int s = 0; s < STAGES; s++) {
            ptx::mbarrier_init(full_bar(s), 1);
            ptx::mbarrier_init(empty_bar(s), 2);          // one promotion warp of either half has seen its product of the stage complete
        }
        for (int a = 0; a < 4; a++) {
            ptx::mbarrier_init(acc_full_bar(a), 1);
            ptx::mbarrier_init(acc_empty_bar(a), 8);      // four promotion warps of either CTA
        }
        ptx::fence_mbarrier_init();
        ptx::prefetch_tensor_map(map_a);
        ptx::prefetch_tensor_map(map_b);
    }
    if (warp == 1) {
        ptx::tmem_alloc<2>(ptx::smem_u32(const_cast<uint32_t *>(tmem_slot)), 512);
        ptx::tmem_relinquish<2>();
    }
    ptx::tcgen05_fence_before();
    __syncthreads();
    ptx::cluster_arrive();
    ptx::cluster_wait();
    ptx::tcgen05_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    // Everything above touched no global memory and may have overlapped the previous kernel of the stream.
    ptx::grid_dependency_wait();
    ptx::grid_dependency_launch();

    if (warp < 4) ptx::registers_decrease<BLOCKSCALED_PRODUCER_REGISTERS>();
    if (warp == 0) {
        // ------------------------------------------------------------------ producer
        if (lane == 0) {
            int stage = 0;
            uint32_t phase = 0;
            bool ok = true;
            for (int tile = cluster_id; tile < tile_count && ok; tile += cluster_count) {
                int tile_m, tile_n;
                tile_position(tile, p, tile_m, tile_n);
                const int row_a = (tile_m * 2 + int(cta_rank)) * BLOCK_M;
                // half h of the tile is columns [128 h, 128 h + 128): the leader holds the first 64 rows of B of each half, the
                // other CTA the last 64, so that a product of N = 128 reads 64 rows from either CTA at one shared-memory offset
                const int row_b = tile_n * BN + int(cta_rank) * 64;
                for (int kb = 0; kb < k_blocks; kb++) {
                    if (!ptx::mbarrier_wait(empty_bar(stage), phase ^ 1, abort_flag)) {
                        report(p, abort_flag, STATUS_PRODUCER_TIMEOUT, tile, kb);
                        ok = false;
                        break;
                    }
                    if (leader) ptx::mbarrier_arrive_expect_tx(full_bar(stage), 2 * L::STAGE_BYTES);
                    const uint32_t leader_bar = ptx::map_to_cta(full_bar(stage), 0);
                    ptx::tma_load_2d_pair(stage_a(stage), map_a, kb * BLOCK_K, row_a, leader_bar);
                    ptx::tma_load_2d_pair(stage_b(stage, 0), map_b, kb * BLOCK_K, row_b, leader_bar);
                    ptx::tma_load_2d_pair(stage_b(stage, 1), map_b, kb * BLOCK_K, row_b + HALF, leader_bar);
                    if (++stage == STAGES) { stage = 0; phase ^= 1; }
                }
            }
            for (int s = 0; s < STAGES && ok; s++) {
                ok = ptx::mbarrier_wait(empty_bar(stage), phase ^ 1, abort_flag);
                if (++stage == STAGES) { stage = 0; phase ^= 1; }
            }
        }
    } else if (warp < 4) {
        // ------------------------------------------------------------------ MMA issuers: products g = issuer, issuer + 3, ...
        // Product g is half g & 1 of K-block g >> 1 (counted over all tiles of this pair), in accumulator g & 3.
        if (lane == 0 && leader) {
            const uint64_t a_desc0 = ptx::smem_descriptor_k_major_sw128(stage_a(0));
            const uint64_t b_desc0 = ptx::smem_descriptor_k_major_sw128(stage_b(0, 0));
            constexpr uint64_t STAGE_STEP = uint64_t(L::STAGE_BYTES >> 4), HALF_STEP = uint64_t(L::B_HALF_BYTES >> 4);
            const uint32_t products = uint32_t(2 * all_blocks);
            for (uint32_t g = uint32_t(warp - 1); g < products; g += BLOCKSCALED_ISSUERS) {
                const uint32_t block = g >> 1;
                const int half = int(g & 1), slot = int(g & 3);
                const int stage = int(block % uint32_t(STAGES));
                const uint32_t stage_phase = (block / uint32_t(STAGES)) & 1, use = block >> 1, use_phase = use & 1;
                // An accumulator's barrier tells its phases apart by one bit, and the previous product into this accumulator came
                // from another thread (three issuers, four accumulators): until that product has been issued, the hand-back this
                // thread is about to wait for belongs to a phase the barrier has not begun, and the parity test would pass at once.
                bool ok = true;
                if (issued[slot] < use) {
                    const unsigned long long start = ptx::global_timer();
                    while (issued[slot] < use && ok) ok = *abort_flag == 0 && ptx::global_timer() - start < ptx::WAIT_LIMIT_NS;
                }
                if (!ok || !ptx::mbarrier_wait(full_bar(stage), stage_phase, abort_flag) || !ptx::mbarrier_wait(acc_empty_bar(slot), use_phase ^ 1, abort_flag)) {
                    report(p, abort_flag, STATUS_MMA_TIMEOUT, int(block / uint32_t(k_blocks)), int(block % uint32_t(k_blocks)));
                    break;
                }
                ptx::tcgen05_fence_after();
                const uint64_t a_desc = a_desc0 + uint64_t(stage) * STAGE_STEP, b_desc = b_desc0 + uint64_t(stage) * STAGE_STEP + uint64_t(half) * HALF_STEP;
                const uint32_t d_tmem = tmem_base + uint32_t(slot) * HALF;
                ptx::tcgen05_mma<ptx::KIND_F8F6F4, 2>(d_tmem, a_desc, b_desc, IDESC, 0u);
#pragma unroll
                for (int j = 1; j < ROW_BYTES / MMA_K_BYTES; j++)
                    ptx::tcgen05_mma_accumulate<ptx::KIND_F8F6F4, 2>(d_tmem, a_desc + uint64_t(j * (MMA_K_BYTES >> 4)), b_desc + uint64_t(j * (MMA_K_BYTES >> 4)), IDESC);
                ptx::tcgen05_commit_pair(acc_full_bar(slot), 0x3);
                issued[slot] = use + 1;
            }
        }
    } else {
        // ------------------------------------------------------------------ promotion + epilogue
        ptx::registers_increase<BLOCKSCALED_PROMOTION_REGISTERS>();
        const int quadrant = warp % 4;             // TMEM lanes this warp may read
        const int half = (warp - 4) / 4;           // which 128 columns of the tile: one scale block of B
        const int scale_pitch = k_blocks;
        const uint32_t staging = base + L::STAGING_OFFSET + uint32_t(warp - 4) * 32 * ROW_BYTES;
        uint32_t block = 0;
        int stage = 0;
        bool ok = true;
        for (int tile = cluster_id; tile < tile_count && ok; tile += cluster_count) {
            int tile_m, tile_n;
            tile_position(tile, p, tile_m, tile_n);
            const int warp_row = (tile_m * 2 + int(cta_rank)) * BLOCK_M + quadrant * 32;
            const int row = warp_row + int(lane);
            const int column = tile_n * BN + half * HALF;
            const float *row_scales = p.scale_a + size_t(min(row, p.m - 1)) * scale_pitch;
            const float *block_scales = p.scale_b + size_t(min(column, p.n - 1) / SCALE_BLOCK_COLUMNS) * scale_pitch;
            float sums[HALF];
#pragma unroll
            for (int i = 0; i < HALF; i++) sums[i] = 0.0f;
            // The scales are fetched two blocks ahead and multiplied one block ahead: a warp issues in order, so a product placed
            // right behind its loads would hold the warp for the whole trip to L2 (the rows' scales are 4 bytes out of every
            // 128-byte line a lane touches; they miss the small L1 that a full shared-memory carve-out leaves).
            float scale = __ldg(row_scales) * __ldg(block_scales);
            float row_part = __ldg(row_scales + min(1, k_blocks - 1)), block_part = __ldg(block_scales + min(1, k_blocks - 1));
            for (int kb = 0; kb < k_blocks; kb++, block++) {
                const int ahead = min(kb + 2, k_blocks - 1);
                const int slot = int(block & 1) * 2 + half;
                const bool ready = ptx::mbarrier_wait(acc_full_bar(slot), (block >> 1) & 1, abort_flag);
                if (!__all_sync(0xffffffffu, ready)) {
                    if (lane == 0) report(p, abort_flag, STATUS_EPILOGUE_TIMEOUT, tile, kb);
                    ok = false;
                    break;
                }
                ptx::tcgen05_fence_after();
                // this half's product of the stage is complete: with the other half's warp saying the same, the stage is free
                if (quadrant == 0 && lane == 0) ptx::mbarrier_arrive(empty_bar(stage));
                if (++stage == STAGES) stage = 0;
                const uint32_t address = tmem_base + (uint32_t(quadrant * 32) << 16) + uint32_t(slot) * HALF;
                // two 32-column loads per wait, the second pair issued as soon as the first buffer is free
                uint32_t first[32], second[32];
                ptx::tmem_load_32x32(address, first);
                ptx::tmem_load_32x32(address + 32, second);
                ptx::tmem_load_wait();
#pragma unroll
                for (int i = 0; i < 32; i += 2) ptx::fma2(sums[i], sums[i + 1], first[i], first[i + 1], scale);
                ptx::tmem_load_32x32(address + 64, first);
#pragma unroll
                for (int i = 0; i < 32; i += 2) ptx::fma2(sums[32 + i], sums[32 + i + 1], second[i], second[i + 1], scale);
                ptx::tmem_load_32x32(address + 96, second);
                ptx::tmem_load_wait();
                // the last values have left the accumulator: hand it back before the remaining arithmetic
                ptx::tcgen05_fence_before();
                __syncwarp();
                if (lane == 0) {
                    if (leader) ptx::mbarrier_arrive(acc_empty_bar(slot));                      // the barrier is in this CTA
                    else ptx::mbarrier_arrive_cluster_relaxed(ptx::map_to_cta(acc_empty_bar(slot), 0));
                }
                const float scale_next = row_part * block_part;          // loaded during the previous block: long since arrived
                row_part = __ldg(row_scales + ahead), block_part = __ldg(block_scales + ahead);
#pragma unroll
                for (int i = 0; i < 32; i += 2) {
                    ptx::fma2(sums[64 + i], sums[64 + i + 1], first[i], first[i + 1], scale);
                    ptx::fma2(sums[96 + i], sums[96 + i + 1], second[i], second[i + 1], scale);
                }
                scale = scale_next;
            }
            if (!ok) break;
            // ---- epilogue of this warp's 32 rows x 128 columns
            if (p.vector_stores == 1) {
                constexpr int COLUMNS_PER_BOX = OUT == OUT_F32 ? 32 : 64;
#pragma unroll
                for (int box = 0; box < HALF / COLUMNS_PER_BOX; box++) {
                    const int box_column = column + box * COLUMNS_PER_BOX;
                    uint32_t packed[32];
                    if constexpr (COLUMNS_PER_BOX == 32) {
#pragma unroll
                        for (int i = 0; i < 32; i++) packed[i] = __float_as_uint(sums[box * 32 + i]);
                        apply_epilogue<OUT>(p, packed, row, box_column);
                    } else {
                        uint32_t low[32], high[32];
#pragma unroll
                        for (int i = 0; i < 32; i++) {
                            low[i] = __float_as_uint(sums[box * 64 + i]);
                            high[i] = __float_as_uint(sums[box * 64 + 32 + i]);
                        }
                        apply_epilogue<OUT>(p, low, row, box_column);
                        apply_epilogue<OUT>(p, high, row, box_column + 32);
#pragma unroll
                        for (int i = 0; i < 16; i++) {
                            packed[i] = pack_pair<OUT>(low[2 * i], low[2 * i + 1]);
                            packed[16 + i] = pack_pair<OUT>(high[2 * i], high[2 * i + 1]);
                        }
                    }
                    if (warp_row < p.m && box_column < p.n) {      // warp-uniform: boxes wholly outside C are skipped
                        if (lane == 0) ptx::tma_store_wait_read<0>();       // the previous box has left the buffer
                        __syncwarp();
#pragma unroll
                        for (int j = 0; j < 8; j++)                          // lane = row; 16-byte piece j goes to slot j ^ (row % 8)
                            ptx::store_shared_v4(staging + lane * ROW_BYTES + uint32_t((j ^ int(lane & 7)) * 16), packed[4 * j], packed[4 * j + 1],
                                                 packed[4 * j + 2], packed[4 * j + 3]);
                        ptx::fence_async_shared();
                        __syncwarp();
                        if (lane == 0) {
                            ptx::tma_store_2d(map_c, box_column, warp_row, staging);
                            ptx::tma_store_commit();
                        }
                    }
                }
            } else {
#pragma unroll
                for (int chunk = 0; chunk < HALF / 32; chunk++) {
                    uint32_t values[32];
#pragma unroll
                    for (int i = 0; i < 32; i++) values[i] = __float_as_uint(sums[chunk * 32 + i]);
                    store_chunk<OUT>(p, values, row, column + chunk * 32);
                }
            }
        }
        if (lane == 0) ptx::tma_store_wait_read<0>();   // the stores have read their source; the grid's completion orders their writes
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
    ptx::cluster_arrive();
    ptx::cluster_wait();
    if (warp == 1) {
        ptx::tcgen05_fence_after();
        ptx::tmem_dealloc<2>(tmem_base, 512);
    }
}

}  // namespace gemm
