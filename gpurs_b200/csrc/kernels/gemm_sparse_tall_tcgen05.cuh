// The 2:4-sparse GEMM on 512 x 224 CTA-pair tiles.
//
// The 256 x 224 kernel (gemm_sparse_tcgen05.cuh) moves 46 KiB per CTA and stage for 448 tensor cycles, 105 bytes per clock and
// SM at full rate, and the path from L2 to the SMs delivers about 64 (gemm_wide_tcgen05.cuh says how that was found): its
// tensor pipe was measured 59 % busy.  B is most of those bytes, and B is what two row blocks can share: here a CTA pair takes
// TWO 256-row blocks of A per tile, each into its own 224-column accumulator, against one load of the B tile: 64 KiB per CTA
// and stage for 896 tensor cycles, 73 bytes per clock and SM.
//
// Both accumulators then belong to one tile, and both are written in every stage, so a tile's epilogue cannot hide behind the
// next tile's main loop the way it does with two tiles' accumulators in turn: the tensor core waits while they are read.  That
// wait is kept short instead: EIGHT epilogue warps (two per lane quadrant, 128 and 96 columns each) copy an accumulator to
// registers in one go and hand it back before they convert and store anything; the stores then run beside the next tile's
// products.  Measured with four warps that stored before they released: +8 % over the 256-row tiles on 8192^3 where the
// operand traffic promised 30 %.  The kernel applies no output algebra (the launcher keeps such products on the 256-row tiles).
//
// Per stage (128 logical K) and CTA: two tiles of compressed A (its 128 rows of either row block, 16 KiB each), the two
// 64-deep halves of its 112 rows of B (14 KiB each), two metadata blocks (2 KiB each): 64 KiB, three stages.  The MMA thread
// copies both metadata blocks to tensor memory (8 columns per stage behind the accumulators) and issues 2 x 4 tcgen05.mma.sp.
#pragma once
#include "gemm_sparse_tcgen05.cuh"

namespace gemm {

constexpr int SPARSE_TALL_STAGES = 3;
constexpr int SPARSE_TALL_EPILOGUE_WARPS = 8;
constexpr int SPARSE_TALL_THREADS = 64 + 32 * SPARSE_TALL_EPILOGUE_WARPS;
static_assert(SPARSE_TALL_THREADS == SPARSE_TALL_NUM_THREADS, "the host sizes the launch from gemm_params.hpp");

struct SparseTallLayout {
    static constexpr int A_BYTES = BLOCK_M * ROW_BYTES;                   // one row block: 128 rows x 64 kept elements
    static constexpr int B_HALF_BYTES = (SPARSE_BLOCK_N / 2) * ROW_BYTES; // this CTA's 112 rows of one 64-deep half of the B tile
    static constexpr int STAGE_BYTES = 2 * A_BYTES + 2 * B_HALF_BYTES + 2 * METADATA_BLOCK_BYTES;      // 64 KiB
    static constexpr int BARRIER_OFFSET = SPARSE_TALL_STAGES * STAGE_BYTES;
    static constexpr int NUM_BARRIERS = 2 * SPARSE_TALL_STAGES + 4;
    static constexpr int TMEM_SLOT_OFFSET = BARRIER_OFFSET + NUM_BARRIERS * 8;
    static constexpr int ABORT_OFFSET = TMEM_SLOT_OFFSET + 4;
    static constexpr int DYNAMIC_BYTES = ABORT_OFFSET + 4 + 1024;
    static_assert(STAGE_BYTES % 1024 == 0, "stages must keep the 1024-byte alignment of the swizzled tiles");
    static_assert(DYNAMIC_BYTES == SPARSE_TALL_SHARED, "the host sizes the launch from gemm_params.hpp");
};

// ELEMENT_FORMAT: 0 = f16, 1 = bf16.  map_e describes the metadata as rows of 16 bytes (box 16 x 128).
template <int ELEMENT_FORMAT, int OUT>
__device__ __forceinline__ void gemm_sparse_tall_body(const CUtensorMap *map_a, const CUtensorMap *map_b, const CUtensorMap *map_e, const Params &p) {
    using L = SparseTallLayout;
    constexpr int BN = SPARSE_BLOCK_N, STAGES = SPARSE_TALL_STAGES;
    constexpr uint32_t METADATA_COLUMN = 2 * BN;      // metadata of stage s, row block r: columns 2 * BN + 8 * s + 4 * r .. + 3
    static_assert(2 * BN + 8 * STAGES <= 512, "two accumulators and the metadata must fit tensor memory");
    constexpr uint32_t IDESC = instruction_descriptor(1, ELEMENT_FORMAT, 2 * BLOCK_M, BN) | (1u << 2);       // sparse flag: bit 2

    extern __shared__ uint8_t raw_shared[];
    const uint32_t base = (ptx::smem_u32(raw_shared) + 1023u) & ~1023u;
    uint8_t *aligned = raw_shared + (base - ptx::smem_u32(raw_shared));
    volatile uint32_t *tmem_slot = reinterpret_cast<volatile uint32_t *>(aligned + L::TMEM_SLOT_OFFSET);
    volatile uint32_t *abort_flag = reinterpret_cast<volatile uint32_t *>(aligned + L::ABORT_OFFSET);

    auto stage_a = [&](int s, int r) { return base + uint32_t(s) * L::STAGE_BYTES + uint32_t(r) * L::A_BYTES; };
    auto stage_b = [&](int s, int half) { return base + uint32_t(s) * L::STAGE_BYTES + 2 * L::A_BYTES + uint32_t(half) * L::B_HALF_BYTES; };
    auto stage_e = [&](int s, int r) { return base + uint32_t(s) * L::STAGE_BYTES + 2 * L::A_BYTES + 2 * L::B_HALF_BYTES + uint32_t(r) * METADATA_BLOCK_BYTES; };
    auto full_bar = [&](int s) { return base + L::BARRIER_OFFSET + uint32_t(s) * 8; };
    auto empty_bar = [&](int s) { return base + L::BARRIER_OFFSET + uint32_t(STAGES + s) * 8; };
    auto acc_full_bar = [&](int a) { return base + L::BARRIER_OFFSET + uint32_t(2 * STAGES + a) * 8; };
    auto acc_empty_bar = [&](int a) { return base + L::BARRIER_OFFSET + uint32_t(2 * STAGES + 2 + a) * 8; };

    const int warp = threadIdx.x / 32;
    const uint32_t lane = ptx::lane_id();
    const uint32_t cta_rank = ptx::cluster_cta_rank();
    const bool leader = cta_rank == 0;
    const int cluster_id = blockIdx.x / 2;
    const int cluster_count = gridDim.x / 2;
    const int tile_count = p.tiles_m * p.tiles_n;
    const int k_blocks = (p.k + SPARSE_STAGE_K - 1) / SPARSE_STAGE_K;     // p.k is the logical depth
    // 128-row block of A (and of C) that row block r of tile row tile_m is on this CTA: the pair's products cover 256 rows each,
    // the leader's 128 first
    auto row_block = [&](int tile_m, int r) { return tile_m * 4 + r * 2 + int(cta_rank); };

    if (threadIdx.x == 0) {
        *abort_flag = 0;
        for (int s = 0; s < STAGES; s++) {
            ptx::mbarrier_init(full_bar(s), 1);
            ptx::mbarrier_init(empty_bar(s), 1);
        }
        for (int a = 0; a < 2; a++) {
            ptx::mbarrier_init(acc_full_bar(a), 1);
            ptx::mbarrier_init(acc_empty_bar(a), SPARSE_TALL_EPILOGUE_WARPS * 2);
        }
        ptx::fence_mbarrier_init();
        ptx::prefetch_tensor_map(map_a);
        ptx::prefetch_tensor_map(map_b);
        ptx::prefetch_tensor_map(map_e);
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
        // ------------------------------------------------------------------ producer: two tiles of A, two halves of B, two metadata blocks
        if (lane == 0) {
            int stage = 0;
            uint32_t phase = 0;
            bool ok = true;
            for (int tile = cluster_id; tile < tile_count && ok; tile += cluster_count) {
                int tile_m, tile_n;
                tile_position(tile, p, tile_m, tile_n);
                const int row_b = tile_n * BN + int(cta_rank) * (BN / 2);
                for (int kb = 0; kb < k_blocks; kb++) {
                    if (!ptx::mbarrier_wait(empty_bar(stage), phase ^ 1, abort_flag)) {
                        report(p, abort_flag, STATUS_PRODUCER_TIMEOUT, tile, kb);
                        ok = false;
                        break;
                    }
                    const int k_logical = kb * SPARSE_STAGE_K;
                    if (leader) ptx::mbarrier_arrive_expect_tx(full_bar(stage), 2 * L::STAGE_BYTES);
                    const uint32_t leader_bar = ptx::map_to_cta(full_bar(stage), 0);
#pragma unroll
                    for (int r = 0; r < 2; r++) {
                        const int block = row_block(tile_m, r);
                        ptx::tma_load_2d_pair(stage_a(stage, r), map_a, k_logical / 2, block * BLOCK_M, leader_bar);
                        // rows past the matrix: the block index may run past the metadata array, whose descriptor then fills zeros
                        ptx::tma_load_2d_pair(stage_e(stage, r), map_e, 0, (block * k_blocks + kb) * 128, leader_bar);
                    }
                    ptx::tma_load_2d_pair(stage_b(stage, 0), map_b, k_logical, row_b, leader_bar);
                    ptx::tma_load_2d_pair(stage_b(stage, 1), map_b, k_logical + 64, row_b, leader_bar);
                    if (++stage == STAGES) { stage = 0; phase ^= 1; }
                }
            }
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
            for (int tile = cluster_id; tile < tile_count && ok; tile += cluster_count) {
                for (int kb = 0; kb < k_blocks && ok; kb++) {
                    if (!ptx::mbarrier_wait(full_bar(stage), phase, abort_flag)) {
                        report(p, abort_flag, STATUS_MMA_TIMEOUT, tile, kb);
                        ok = false;
                        break;
                    }
                    ptx::tcgen05_fence_after();
#pragma unroll
                    for (int r = 0; r < 2; r++) {
                        if (kb == 0) {
                            // the accumulator must have been read out before the first product of a tile overwrites it
                            if (!ptx::mbarrier_wait<true>(acc_empty_bar(r), tile_phase ^ 1, abort_flag)) {
                                report(p, abort_flag, STATUS_MMA_TIMEOUT, tile, -1 - r);
                                ok = false;
                                break;
                            }
                            ptx::tcgen05_fence_after();
                        }
                        const uint32_t d_tmem = tmem_base + uint32_t(r) * BN;
                        const uint32_t metadata_tmem = tmem_base + METADATA_COLUMN + uint32_t(stage) * 8 + uint32_t(r) * 4;
                        ptx::tcgen05_copy_128x128b<2>(metadata_tmem, ptx::smem_descriptor_rows16(stage_e(stage, r)));
                        const uint64_t a_desc = ptx::smem_descriptor_k_major_sw128(stage_a(stage, r));
#pragma unroll
                        for (int j = 0; j < 4; j++) {
                            // instruction j: 32 logical K = 32 bytes of compressed A, 64 bytes of B (half j / 2, offset j % 2)
                            const uint64_t b_desc = ptx::smem_descriptor_k_major_sw128(stage_b(stage, j / 2)) + uint64_t((j % 2) * (64 >> 4));
                            const uint32_t column = metadata_tmem + uint32_t(j);      // the even column of the pair + a selector bit
                            ptx::tcgen05_mma_sparse_f16<2>(d_tmem, a_desc + uint64_t(j * (MMA_K_BYTES >> 4)), b_desc, column & ~1u, IDESC | (column & 1u),
                                                           uint32_t((kb | j) != 0));
                        }
                        if (kb == k_blocks - 1) ptx::tcgen05_commit_pair(acc_full_bar(r), 0x3);      // this row block of the tile is complete
                    }
                    if (!ok) break;
                    ptx::tcgen05_commit_pair(empty_bar(stage), 0x3);
                    if (++stage == STAGES) { stage = 0; phase ^= 1; }
                }
                tile_phase ^= 1;
            }
        }
    } else {
        // ------------------------------------------------------------------ epilogue: row block 0, then row block 1
        const int quadrant = warp % 4;                                    // the 32 lanes of tensor memory this warp may read
        const int first_chunk = warp < 6 ? 0 : 4;                         // warps 2-5: columns 0-127; warps 6-9: columns 128-223
        const int chunks = warp < 6 ? 4 : BN / 32 - 4;
        uint32_t tile_phase = 0;
        bool ok = true;
        for (int tile = cluster_id; tile < tile_count && ok; tile += cluster_count) {
            int tile_m, tile_n;
            tile_position(tile, p, tile_m, tile_n);
#pragma unroll 1
            for (int r = 0; r < 2 && ok; r++) {
                const bool ready = ptx::mbarrier_wait(acc_full_bar(r), tile_phase, abort_flag);
                if (!__all_sync(0xffffffffu, ready)) {
                    if (lane == 0) report(p, abort_flag, STATUS_EPILOGUE_TIMEOUT, tile, -1 - r);
                    ok = false;
                    break;
                }
                ptx::tcgen05_fence_after();
                const int row = row_block(tile_m, r) * BLOCK_M + quadrant * 32 + int(lane);
                const uint32_t lane_base = tmem_base + (uint32_t(quadrant * 32) << 16) + uint32_t(r) * BN + uint32_t(first_chunk * 32);
                uint32_t values[4][32];
#pragma unroll
                for (int c = 0; c < 4; c++)
                    if (c < chunks) ptx::tmem_load_32x32(lane_base + uint32_t(c * 32), values[c]);
                ptx::tmem_load_wait();
                ptx::tcgen05_fence_before();
                __syncwarp();
                if (lane == 0) {
                    if (leader) ptx::mbarrier_arrive(acc_empty_bar(r));
                    else ptx::mbarrier_arrive_cluster_relaxed(ptx::map_to_cta(acc_empty_bar(r), 0));
                }
#pragma unroll
                for (int c = 0; c < 4; c++)
                    if (c < chunks) store_chunk<OUT, false, false>(p, values[c], row, tile_n * BN + (first_chunk + c) * 32);
            }
            tile_phase ^= 1;
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
    ptx::cluster_arrive();
    ptx::cluster_wait();
    if (warp == 1) {
        ptx::tcgen05_fence_after();
        ptx::tmem_dealloc<2>(tmem_base, 512);
    }
}

}  // namespace gemm
