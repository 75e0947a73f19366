// The dense GEMM on 256 x 512 CTA-pair tiles.
//
// Every dense kernel of this library with 256 x 256 pair tiles was measured to draw 11 to 12 TB/s from L2 (bf16 8192^3:
// 8.59 GB of tile loads in 0.70 to 0.74 ms; int8 and FP8 the same rate), which is what the path from L2 to the 148 SMs
// delivers: about 64 bytes per clock and SM.  At that rate the operands of a 256 x 256 tile arrive exactly as fast as the
// tensor cores consume them, and the fabric, not the tensor pipe, sets the time.  A 256 x 512 tile needs 48 bytes per clock and
// SM for the same flops (A is fetched once for twice the columns), and DRAM sees fewer re-reads for the same reason.
//
// Such a tile is all 512 columns of tensor memory: there is no second accumulator to multiply into while the first is
// stored.  The two 256-column halves are handed over separately instead: each has its own full / empty barriers, every
// K-block is two products of N = 256 (half 0, then half 1, A read twice from shared memory), and at a tile border the next
// tile's products into half 0 start as soon as half 0 has been read out, while half 1 is still being stored.  What stays
// exposed per tile is about the read-out of one half, against 1024 tensor cycles per K-block.
//
// Layout per stage and CTA: 128 rows of A (16 KiB), then the CTA's 128 rows of either half of the B tile (2 x 16 KiB): the
// leader holds the first 128 rows of B of each half, the other CTA the last 128, so that a product of N = 256 finds 128 rows
// in either CTA at one shared-memory offset.  4 stages of 48 KiB, 32 KiB of output staging.  Roles: warp 0 producer, warp 1 MMA
// issuer (leader), warps 2..9 epilogue: two warps per quadrant of tensor-memory lanes, one for the first and one for the second
// 128 columns of either half, one staging box each.  (A launch of one round ends with every tile's read-out exposed at once;
// with four epilogue warps that tail was measured at 6.6 us for 32-bit outputs, which a 1024-row shard of an 8192^3 product
// cannot afford.)  Epilogue: round, stage, TMA store, with the element-wise output algebra in the `_ep` entries; C with 16-byte aligned
// rows; row reductions, accumulation into C and everything else take the 256-column kernels.
//
// What paces the read-out is the SM's path to L2 for stores, 32 bytes per clock (a tile's 256 KiB of 32-bit outputs: 4.5 us,
// measured the same with one CTA pair running and with 72).  Between tiles the epilogue therefore empties tensor memory into
// registers first and stores afterwards, so that the next tile's products do not wait for stores; the last tile of a CTA pair
// is read out box by box, so that its stores never pause.
#pragma once
#include "gemm_tcgen05.cuh"

namespace gemm {

constexpr int WIDE_BLOCK_N = 512, WIDE_STAGES = 4;
constexpr int WIDE_EPILOGUE_WARPS = 8;
constexpr int WIDE_THREADS = 64 + 32 * WIDE_EPILOGUE_WARPS;
static_assert(WIDE_THREADS == WIDE_NUM_THREADS, "the host sizes the launch from gemm_params.hpp");

struct WideLayout {
    static constexpr int A_BYTES = BLOCK_M * ROW_BYTES;
    static constexpr int B_HALF_BYTES = 128 * ROW_BYTES;
    static constexpr int STAGE_BYTES = A_BYTES + 2 * B_HALF_BYTES;     // 48 KiB
    static constexpr int BARRIER_OFFSET = WIDE_STAGES * STAGE_BYTES;
    // full[STAGES], empty[STAGES], accumulator_full[2], accumulator_empty[2]
    static constexpr int NUM_BARRIERS = 2 * WIDE_STAGES + 4;
    static constexpr int TMEM_SLOT_OFFSET = BARRIER_OFFSET + NUM_BARRIERS * 8;
    static constexpr int ABORT_OFFSET = TMEM_SLOT_OFFSET + 4;
    static constexpr int STAGING_OFFSET = ((ABORT_OFFSET + 4 + 1023) / 1024) * 1024;
    static constexpr int STAGING_BYTES = WIDE_EPILOGUE_WARPS * 32 * ROW_BYTES;      // one box of 32 rows x 128 bytes per epilogue warp
    static constexpr int TOTAL = STAGING_OFFSET + STAGING_BYTES;
    static constexpr int DYNAMIC_BYTES = TOTAL + 1024;
    static_assert(DYNAMIC_BYTES <= 232448, "more than the 227 KiB a CTA may have");
    static_assert(DYNAMIC_BYTES == WIDE_SHARED, "the host sizes the launch from gemm_params.hpp");
};

// ALGEBRA: the epilogue applies the element-wise output algebra of Params (alpha, row and column scales, bias, row bias,
// residual) as the 256-column kernels do; the entries without it are the ones a plain product runs.
// SECOND: columns of the tile's second half, 256 or 224.  A 256 + 224 = 480-column tile exists for shapes whose 512-wide tiles
// fill the grid badly (8192 columns on 1024 rows: 64 tiles of 512 for 74 CTA pairs, 72 of 480); its second half is a product of
// N = 224 on 112 rows of B per CTA (the 128-row box is loaded all the same), and its outputs are 32-bit (whole 32-column boxes).
template <int KIND, int ELEMENT_FORMAT, int ACC_FORMAT, int OUT, bool ALGEBRA = false, int SECOND = 256>
__device__ __forceinline__ void gemm_wide_body(const CUtensorMap *map_a, const CUtensorMap *map_b, const CUtensorMap *map_c, const Params &p) {
    using L = WideLayout;
    constexpr int STAGES = WIDE_STAGES, HALF = 256, TILE_N = HALF + SECOND;
    static_assert(SECOND == 256 || (SECOND == 224 && (OUT == OUT_F32 || OUT == OUT_I32)), "second half: 256 columns, or 224 with 32-bit outputs");
    constexpr uint32_t IDESC_FIRST = instruction_descriptor(ACC_FORMAT, ELEMENT_FORMAT, 2 * BLOCK_M, HALF);
    constexpr uint32_t IDESC_SECOND = instruction_descriptor(ACC_FORMAT, ELEMENT_FORMAT, 2 * BLOCK_M, SECOND);

    extern __shared__ uint8_t raw_shared[];
    const uint32_t base = (ptx::smem_u32(raw_shared) + 1023u) & ~1023u;
    uint8_t *aligned = raw_shared + (base - ptx::smem_u32(raw_shared));
    volatile uint32_t *tmem_slot = reinterpret_cast<volatile uint32_t *>(aligned + L::TMEM_SLOT_OFFSET);
    volatile uint32_t *abort_flag = reinterpret_cast<volatile uint32_t *>(aligned + L::ABORT_OFFSET);

    auto stage_a = [&](int s) { return base + uint32_t(s) * L::STAGE_BYTES; };
    auto stage_b = [&](int s, int half) { return base + uint32_t(s) * L::STAGE_BYTES + L::A_BYTES + uint32_t(half) * L::B_HALF_BYTES; };
    auto full_bar = [&](int s) { return base + L::BARRIER_OFFSET + uint32_t(s) * 8; };
    auto empty_bar = [&](int s) { return base + L::BARRIER_OFFSET + uint32_t(STAGES + s) * 8; };
    auto acc_full_bar = [&](int h) { return base + L::BARRIER_OFFSET + uint32_t(2 * STAGES + h) * 8; };
    auto acc_empty_bar = [&](int h) { return base + L::BARRIER_OFFSET + uint32_t(2 * STAGES + 2 + h) * 8; };
    const uint32_t staging = base + L::STAGING_OFFSET;

    const int warp = threadIdx.x / 32;
    const uint32_t lane = ptx::lane_id();
    const uint32_t cta_rank = ptx::cluster_cta_rank();
    const bool leader = cta_rank == 0;
    const int cluster_id = blockIdx.x / 2;
    const int cluster_count = gridDim.x / 2;
    const int tile_count = p.tiles_m * p.tiles_n;
    const int element_bytes = KIND == ptx::KIND_F16 ? 2 : (KIND == ptx::KIND_TF32 ? 4 : 1);
    const int block_k = ROW_BYTES / element_bytes;
    const int k_blocks = (p.k + block_k - 1) / block_k;

    if (threadIdx.x == 0) {
        *abort_flag = 0;
        for (int s = 0; s < STAGES; s++) {
            ptx::mbarrier_init(full_bar(s), 1);
            ptx::mbarrier_init(empty_bar(s), 1);
        }
        for (int h = 0; h < 2; h++) {
            ptx::mbarrier_init(acc_full_bar(h), 1);
            ptx::mbarrier_init(acc_empty_bar(h), WIDE_EPILOGUE_WARPS * 2);
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
                const int row_b = tile_n * TILE_N + int(cta_rank) * 128;
                const int row_b_second = tile_n * TILE_N + HALF + int(cta_rank) * (SECOND / 2);
                for (int kb = 0; kb < k_blocks; kb++) {
                    if (!ptx::mbarrier_wait(empty_bar(stage), phase ^ 1, abort_flag)) {
                        report(p, abort_flag, STATUS_PRODUCER_TIMEOUT, tile, kb);
                        ok = false;
                        break;
                    }
                    if (leader) ptx::mbarrier_arrive_expect_tx(full_bar(stage), 2 * L::STAGE_BYTES);
                    const uint32_t leader_bar = ptx::map_to_cta(full_bar(stage), 0);
                    ptx::tma_load_2d_pair(stage_a(stage), map_a, kb * block_k, row_a, leader_bar);
                    ptx::tma_load_2d_pair(stage_b(stage, 0), map_b, kb * block_k, row_b, leader_bar);
                    ptx::tma_load_2d_pair(stage_b(stage, 1), map_b, kb * block_k, row_b_second, leader_bar);
                    if (++stage == STAGES) { stage = 0; phase ^= 1; }
                }
            }
            // Before leaving, see every stage released once more, so that no commit can arrive on a barrier of a CTA that has exited.
            for (int s = 0; s < STAGES && ok; s++) {
                ok = ptx::mbarrier_wait(empty_bar(stage), phase ^ 1, abort_flag);
                if (++stage == STAGES) { stage = 0; phase ^= 1; }
            }
        }
    } else if (warp == 1) {
        // ------------------------------------------------------------------ MMA issuer
        if (lane == 0 && leader) {
            int stage = 0;
            uint32_t phase = 0, tile_phase = 0;
            bool ok = true;
            const uint64_t a_desc0 = ptx::smem_descriptor_k_major_sw128(stage_a(0)), b_desc0 = ptx::smem_descriptor_k_major_sw128(stage_b(0, 0));
            constexpr uint64_t STAGE_STEP = uint64_t(L::STAGE_BYTES >> 4), HALF_STEP = uint64_t(L::B_HALF_BYTES >> 4), K_STEP = uint64_t(MMA_K_BYTES >> 4);
            for (int tile = cluster_id; tile < tile_count && ok; tile += cluster_count) {
                for (int kb = 0; kb < k_blocks && ok; kb++) {
                    if (!ptx::mbarrier_wait(full_bar(stage), phase, abort_flag)) {
                        report(p, abort_flag, STATUS_MMA_TIMEOUT, tile, kb);
                        ok = false;
                        break;
                    }
                    ptx::tcgen05_fence_after();
                    const uint64_t a_desc = a_desc0 + uint64_t(stage) * STAGE_STEP, b_desc = b_desc0 + uint64_t(stage) * STAGE_STEP;
#pragma unroll
                    for (int half = 0; half < 2; half++) {
                        if (kb == 0) {
                            // the half must have been read out before the first product of a tile overwrites it
                            if (!ptx::mbarrier_wait<true>(acc_empty_bar(half), tile_phase ^ 1, abort_flag)) {
                                report(p, abort_flag, STATUS_MMA_TIMEOUT, tile, -1 - half);
                                ok = false;
                                break;
                            }
                            ptx::tcgen05_fence_after();
                        }
                        const uint32_t d_tmem = tmem_base + uint32_t(half) * HALF;
                        const uint64_t b_half = b_desc + uint64_t(half) * HALF_STEP;
                        const uint32_t idesc = half == 0 ? IDESC_FIRST : IDESC_SECOND;
                        ptx::tcgen05_mma<KIND, 2>(d_tmem, a_desc, b_half, idesc, uint32_t(kb != 0));
#pragma unroll
                        for (int j = 1; j < ROW_BYTES / MMA_K_BYTES; j++)
                            ptx::tcgen05_mma_accumulate<KIND, 2>(d_tmem, a_desc + uint64_t(j) * K_STEP, b_half + uint64_t(j) * K_STEP, idesc);
                        if (kb == k_blocks - 1) ptx::tcgen05_commit_pair(acc_full_bar(half), 0x3);      // this half of the tile is complete
                    }
                    if (!ok) break;
                    ptx::tcgen05_commit_pair(empty_bar(stage), 0x3);
                    if (++stage == STAGES) { stage = 0; phase ^= 1; }
                }
                tile_phase ^= 1;
            }
        }
    } else {
        // ------------------------------------------------------------------ epilogue: half 0, then half 1
        const int quadrant = warp % 4;                 // the 32 lanes of tensor memory this warp may read
        const int side = (warp - 2) / 4;               // 0: the first 128 columns of either half, 1: the last 128
        const uint32_t buffer = staging + uint32_t(warp - 2) * 32 * ROW_BYTES;
        constexpr int COLUMNS_PER_BOX = (OUT == OUT_F32 || OUT == OUT_I32) ? 32 : 64;
        constexpr int BOXES = 128 / COLUMNS_PER_BOX;   // per warp and half: 32 registers each once rounded
        uint32_t tile_phase = 0;
        bool ok = true;
        // A warp's 128 columns of a half are read from tensor memory in one go and the half is handed back before anything of it
        // is stored: stores leave an SM at 32 bytes per clock (a 4 KiB box of each of the eight warps: 1024 clocks), and a half
        // that waited for its staging buffer kept the next tile's products waiting with it (measured on bf16 8192^3: +1.3 %).
        // With 16-bit outputs the last box of half 0 stays in registers while half 1 is read, so that half 1 waits for one box of
        // half 0 only; 32-bit outputs fill the registers with one half (128 per lane of the 168 a CTA of ten warps gets).
        for (int tile = cluster_id; tile < tile_count && ok; tile += cluster_count) {
            int tile_m, tile_n;
            tile_position(tile, p, tile_m, tile_n);
            const int warp_row = (tile_m * 2 + int(cta_rank)) * BLOCK_M + quadrant * 32;
            const int column0 = tile_n * TILE_N + side * 128;
            // one box: 32 rows x 128 bytes from registers to the warp's staging buffer, then to C
            auto store_box = [&](const uint32_t (&box)[32], int column) {
                if (warp_row < p.m && column < p.n) {    // warp-uniform: boxes wholly outside C are skipped
                    if (lane == 0) ptx::tma_store_wait_read<0>();       // the previous store has read the buffer
                    __syncwarp();
#pragma unroll
                    for (int j = 0; j < 8; j++)                          // lane = row; 16-byte piece j goes to slot j ^ (row % 8)
                        ptx::store_shared_v4(buffer + lane * ROW_BYTES + uint32_t((j ^ int(lane & 7)) * 16), box[4 * j], box[4 * j + 1],
                                             box[4 * j + 2], box[4 * j + 3]);
                    ptx::fence_async_shared();
                    __syncwarp();
                    if (lane == 0) {
                        ptx::tma_store_2d(map_c, column, warp_row, buffer);
                        ptx::tma_store_commit();
                    }
                }
            };
            // reads the warp's 128 columns of a half (of a 224-column half: the last 32 are columns no product writes and no
            // box stores), hands the half back and rounds (plain products only: see below)
            auto read_half = [&](int half, uint32_t (&boxes)[BOXES][32]) -> bool {
                const bool ready = ptx::mbarrier_wait(acc_full_bar(half), tile_phase, abort_flag);
                if (!__all_sync(0xffffffffu, ready)) {
                    if (lane == 0) report(p, abort_flag, STATUS_EPILOGUE_TIMEOUT, tile, -1 - half);
                    return false;
                }
                ptx::tcgen05_fence_after();
                const uint32_t lane_base = tmem_base + (uint32_t(quadrant * 32) << 16) + uint32_t(half * HALF + side * 128);
                if constexpr (COLUMNS_PER_BOX == 32) {
#pragma unroll
                    for (int chunk = 0; chunk < 4; chunk++) ptx::tmem_load_32x32(lane_base + uint32_t(chunk * 32), boxes[chunk]);
                    ptx::tmem_load_wait();
                } else {
                    uint32_t values[4][32];
#pragma unroll
                    for (int chunk = 0; chunk < 4; chunk++) ptx::tmem_load_32x32(lane_base + uint32_t(chunk * 32), values[chunk]);
                    ptx::tmem_load_wait();
#pragma unroll
                    for (int chunk = 0; chunk < 4; chunk++) {
#pragma unroll
                        for (int i = 0; i < 16; i++) boxes[chunk / 2][(chunk % 2) * 16 + i] = pack_pair<OUT>(values[chunk][2 * i], values[chunk][2 * i + 1]);
                    }
                }
                // this warp's part of the half has left tensor memory: once all sixteen warps of the pair have said so, the next
                // tile's products may overwrite it
                ptx::tcgen05_fence_before();
                __syncwarp();
                if (lane == 0) {
                    if (leader) ptx::mbarrier_arrive(acc_empty_bar(half));
                    else ptx::mbarrier_arrive_cluster_relaxed(ptx::map_to_cta(acc_empty_bar(half), 0));
                }
                return true;
            };
            // boxes of the second half: 128 columns' worth, or what is left of a 224-column second half
            const int second_boxes = side == 1 ? (SECOND - 128) / COLUMNS_PER_BOX : BOXES;
            const bool last_tile = tile + cluster_count >= tile_count;
            if (ALGEBRA || last_tile) {
                // The pair's last tile: no product waits for tensor memory any more, and what counts is that the stores never
                // pause (in a launch of one round this read-out is all exposed: 256 KiB at 32 bytes per clock).  Box by box, the
                // read of the next box in flight while one is staged and stored.  The entries with the output algebra read every
                // tile this way: the algebra's registers on top of a whole half's spilled (bf16 8192^3 with a bias: -1.2 %).
                for (int half = 0; half < 2 && ok; half++) {
                    const bool ready = ptx::mbarrier_wait(acc_full_bar(half), tile_phase, abort_flag);
                    if (!__all_sync(0xffffffffu, ready)) {
                        if (lane == 0) report(p, abort_flag, STATUS_EPILOGUE_TIMEOUT, tile, -1 - half);
                        ok = false;
                        break;
                    }
                    ptx::tcgen05_fence_after();
                    const uint32_t lane_base = tmem_base + (uint32_t(quadrant * 32) << 16) + uint32_t(half * HALF + side * 128);
                    const int boxes = half == 1 ? second_boxes : BOXES;
                    uint32_t low[32], high[32];
                    ptx::tmem_load_32x32(lane_base, low);
                    if constexpr (COLUMNS_PER_BOX == 64) ptx::tmem_load_32x32(lane_base + 32, high);
#pragma unroll
                    for (int box = 0; box < BOXES; box++) {
                        if (box >= boxes) break;
                        const int column = column0 + half * HALF + box * COLUMNS_PER_BOX;
                        uint32_t packed[32];
                        ptx::tmem_load_wait();
                        if constexpr (COLUMNS_PER_BOX == 32) {
                            if constexpr (ALGEBRA) apply_epilogue<OUT>(p, low, warp_row + int(lane), column);
#pragma unroll
                            for (int i = 0; i < 32; i++) packed[i] = low[i];
                            if (box + 1 < boxes) ptx::tmem_load_32x32(lane_base + uint32_t((box + 1) * 32), low);
                        } else {
                            if constexpr (ALGEBRA) {
                                apply_epilogue<OUT>(p, low, warp_row + int(lane), column);
                                apply_epilogue<OUT>(p, high, warp_row + int(lane), column + 32);
                            }
#pragma unroll
                            for (int i = 0; i < 16; i++) {
                                packed[i] = pack_pair<OUT>(low[2 * i], low[2 * i + 1]);
                                packed[16 + i] = pack_pair<OUT>(high[2 * i], high[2 * i + 1]);
                            }
                            if (box + 1 < boxes) {
                                ptx::tmem_load_32x32(lane_base + uint32_t((box + 1) * 64), low);
                                ptx::tmem_load_32x32(lane_base + uint32_t((box + 1) * 64 + 32), high);
                            }
                        }
                        if (box == boxes - 1) {
                            ptx::tcgen05_fence_before();
                            __syncwarp();
                            if (lane == 0) {
                                if (leader) ptx::mbarrier_arrive(acc_empty_bar(half));
                                else ptx::mbarrier_arrive_cluster_relaxed(ptx::map_to_cta(acc_empty_bar(half), 0));
                            }
                        }
                        store_box(packed, column);
                    }
                }
                if (last_tile) break;
                tile_phase ^= 1;
                continue;
            }
            uint32_t first[BOXES][32], second[BOXES][32];
            ok = read_half(0, first);
            if (!ok) break;
            constexpr int CARRIED = COLUMNS_PER_BOX == 64 ? 1 : 0;
#pragma unroll
            for (int box = 0; box < BOXES - CARRIED; box++) store_box(first[box], column0 + box * COLUMNS_PER_BOX);
            ok = read_half(1, second);
            if (!ok) break;
            if constexpr (CARRIED == 1) store_box(first[BOXES - 1], column0 + (BOXES - 1) * COLUMNS_PER_BOX);
#pragma unroll
            for (int box = 0; box < BOXES; box++)
                if (box < second_boxes) store_box(second[box], column0 + HALF + box * COLUMNS_PER_BOX);
            tile_phase ^= 1;
        }
        // the stores have read their shared-memory source; the grid's completion orders their writes before whatever follows
        if (lane == 0) ptx::tma_store_wait_read<0>();
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
