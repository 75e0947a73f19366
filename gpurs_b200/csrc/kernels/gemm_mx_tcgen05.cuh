// FP8 (E4M3) GEMM with the tensor core's own block scaling, for sm_100a:
//
//     C[m, n] = sum_k  A[m, k] * 2^(sA[m, k / 32] - 127)  *  B[n, k] * 2^(sB[n, k / 32] - 127)
//
// sA and sB hold one power-of-two scale (UE8M0: a biased exponent byte) per 32 elements of K, per row of A and per row of B
// (the MX "microscaling" format).  The reference has only the raw unscaled FP8 instruction
// (crates/gpurs/src/gpu/tensor/blackwell/instruction.rs:13-21); the product with fp32 scales per 128-deep block
// (gemm_scaled_tcgen05.cuh) must leave the tensor core after every K-block, which bounds it at about two thirds of the
// unscaled rate.  Power-of-two scales per 32 elements are applied inside `tcgen05.mma.kind::mxf8f6f4.block_scale`, so this
// kernel accumulates over all of K in tensor memory like the unscaled one.
//
// Scales arrive "tiled" (gpurs_quantize_mx_e4m3 writes them so): 512-byte blocks of 128 rows x 128 K, and inside a block
// the scale of row r (0..127) and 32-element group g (0..3) at byte (r % 32) * 16 + (r / 32) * 4 + g  (mx_scale_offset).
// A's blocks follow its 128-row tiles: block (row / 128, k / 128), ordered [row block][K block].  B's follow THIS kernel's
// 224-row tiles, two blocks per tile and K-block (rows 0..127 and 128..223 of the tile), ordered [tile][K block][2]
// (mx_scale_index), because the instruction indexes B's scales by the column within the tile.
// That is the order the instruction reads them from tensor memory after `tcgen05.cp.32x128b.warpx4` has copied the block
// (32 rows of 16 bytes) to four columns of all four lane quadrants (found by experiment: each byte of the block given a
// distinct power of two, the factor of every output row and K group solved for).  Instruction j of a stage (32 of its 128
// K) selects byte j of the columns through the scale ids of its descriptor.
//
// Tiles are 224 columns wide (128 rows for one CTA, 256 for a CTA pair): two accumulators of 224 columns plus 12 scale
// columns per stage (4 for the CTA's 128 rows of A, 8 for B's 224 columns in two blocks) fit the 512 columns of tensor
// memory for 4 (5) stages.  In a pair each CTA loads the scale block of its own rows of A and BOTH blocks of B (its
// tensor core multiplies its 128 rows by all 224 columns), and the leader's `tcgen05.cp.cta_group::2` copies each CTA's
// shared-memory blocks into that CTA's own tensor memory.
#pragma once
#include "gemm_tcgen05.cuh"

namespace gemm {

constexpr int MX_SCALE_BLOCK_BYTES = 512;     // 128 rows x 4 groups of 32 K

__host__ __device__ inline int mx_scale_offset(int row, int k) {
    return (row % 32) * 16 + ((row / 32) % 4) * 4 + (k / 32) % 4;
}

// Byte index of the scale of (row, k) in the tiled array of the left (right_operand = false) or right operand; k_blocks =
// ceil(K / 128).
__host__ __device__ inline long long mx_scale_index(bool right_operand, long long row, int k, int k_blocks) {
    const int k_block = k / 128;
    if (!right_operand) return ((row / 128) * k_blocks + k_block) * MX_SCALE_BLOCK_BYTES + mx_scale_offset(int(row % 128), k);
    const long long tile = row / MX_BLOCK_N;
    const int inside = int(row % MX_BLOCK_N);
    return ((tile * k_blocks + k_block) * 2 + inside / 128) * MX_SCALE_BLOCK_BYTES + mx_scale_offset(inside % 128, k);
}

template <int CTA_GROUP, int STAGES>
struct MxLayout {
    static constexpr int A_BYTES = BLOCK_M * ROW_BYTES;
    static constexpr int B_ROWS = MX_BLOCK_N / CTA_GROUP;
    static constexpr int B_BYTES = B_ROWS * ROW_BYTES;
    static constexpr int SCALE_BYTES = 3 * MX_SCALE_BLOCK_BYTES + 512;           // A's block, B's two blocks, padding to 1024
    static constexpr int STAGE_BYTES = A_BYTES + B_BYTES + SCALE_BYTES;
    static constexpr int BARRIER_OFFSET = ((STAGES * STAGE_BYTES + 1023) / 1024) * 1024;
    static constexpr int NUM_BARRIERS = 2 * STAGES + 4;
    static constexpr int TMEM_SLOT_OFFSET = BARRIER_OFFSET + NUM_BARRIERS * 8;
    static constexpr int ABORT_OFFSET = TMEM_SLOT_OFFSET + 4;
    static constexpr int DYNAMIC_BYTES = ABORT_OFFSET + 4 + 1024;
};
static_assert(MxLayout<1, MX_STAGES_SINGLE>::DYNAMIC_BYTES == MX_SHARED_SINGLE, "host and kernel disagree on shared memory");
static_assert(MxLayout<2, MX_STAGES_PAIR>::DYNAMIC_BYTES == MX_SHARED_PAIR, "host and kernel disagree on shared memory");

template <int CTA_GROUP>
__device__ __forceinline__ void tcgen05_mma_mx(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t scale_a_tmem,
                                               uint32_t scale_b_tmem, uint32_t accumulate) {
    if constexpr (CTA_GROUP == 1)
        asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %6, 0;\n\t"
                     "tcgen05.mma.cta_group::1.kind::mxf8f6f4.block_scale.scale_vec::1X [%0], %1, %2, %3, [%4], [%5], p;\n\t}"
                     ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(scale_a_tmem), "r"(scale_b_tmem), "r"(accumulate) : "memory");
    else
        asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %6, 0;\n\t"
                     "tcgen05.mma.cta_group::2.kind::mxf8f6f4.block_scale.scale_vec::1X [%0], %1, %2, %3, [%4], [%5], p;\n\t}"
                     ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(scale_a_tmem), "r"(scale_b_tmem), "r"(accumulate) : "memory");
}

// 32 rows of 16 bytes from shared memory to 4 columns of tensor memory, the same in all four lane quadrants.
template <int CTA_GROUP>
__device__ __forceinline__ void tcgen05_copy_32x128b_warpx4(uint32_t tmem_address, uint64_t smem_descriptor) {
    if constexpr (CTA_GROUP == 1) asm volatile("tcgen05.cp.cta_group::1.32x128b.warpx4 [%0], %1;" ::"r"(tmem_address), "l"(smem_descriptor) : "memory");
    else asm volatile("tcgen05.cp.cta_group::2.32x128b.warpx4 [%0], %1;" ::"r"(tmem_address), "l"(smem_descriptor) : "memory");
}

// map_sa / map_sb describe the tiled scales as rows of 16 bytes: box 16 x 32 (one block of A's), 16 x 64 (B's two blocks).
// STREAMK: the K-blocks of the tiles of a split round are spread over the CTA groups (gemm_schedule.hpp) and the parts are added
// up by whoever arrives last, as in gemm_body; a part is laid out like a dense tile's (256 columns wide, 224 used).
template <int OUT, int CTA_GROUP, int STAGES, bool STREAMK = false>
__device__ __forceinline__ void gemm_mx_body(const CUtensorMap *map_a, const CUtensorMap *map_b, const CUtensorMap *map_sa, const CUtensorMap *map_sb,
                                             const Params &p) {
    using L = MxLayout<CTA_GROUP, STAGES>;
    constexpr int BN = MX_BLOCK_N;
    constexpr uint32_t TMEM_COLUMNS = 512;
    constexpr uint32_t SCALE_COLUMN = 2 * BN;         // stage s: A's scales at 2*BN + 12*s .. +3, B's at +4 .. +11
    static_assert(2 * BN + 12 * STAGES <= 512 && BN % 32 == 0 && BN > 128 && BN <= 256, "accumulators and scales must fit tensor memory");
    // Block-scaled instruction descriptor: operand formats E4M3 (0) at bits 7 and 10, N >> 3 at bit 17, scale format UE8M0
    // at bit 23, M >> 4 at bit 24; the scale ids (which byte of the scale columns) go to bits 4..5 (B) and 29..30 (A).
    constexpr uint32_t IDESC = (uint32_t(BN >> 3) << 17) | (1u << 23) | (uint32_t((BLOCK_M * CTA_GROUP) >> 4) << 24);
    static_assert(L::STAGE_BYTES % 1024 == 0, "stages must keep the 1024-byte alignment of the swizzled tiles");

    extern __shared__ uint8_t raw_shared[];
    const uint32_t base = (ptx::smem_u32(raw_shared) + 1023u) & ~1023u;
    uint8_t *aligned = raw_shared + (base - ptx::smem_u32(raw_shared));
    volatile uint32_t *tmem_slot = reinterpret_cast<volatile uint32_t *>(aligned + L::TMEM_SLOT_OFFSET);
    volatile uint32_t *abort_flag = reinterpret_cast<volatile uint32_t *>(aligned + L::ABORT_OFFSET);

    auto stage_a = [&](int s) { return base + uint32_t(s) * L::STAGE_BYTES; };
    auto stage_b = [&](int s) { return base + uint32_t(s) * L::STAGE_BYTES + L::A_BYTES; };
    auto stage_scales = [&](int s, int block) { return base + uint32_t(s) * L::STAGE_BYTES + L::A_BYTES + L::B_BYTES + uint32_t(block) * MX_SCALE_BLOCK_BYTES; };
    auto full_bar = [&](int s) { return base + L::BARRIER_OFFSET + uint32_t(s) * 8; };
    auto empty_bar = [&](int s) { return base + L::BARRIER_OFFSET + uint32_t(STAGES + s) * 8; };
    auto acc_full_bar = [&](int a) { return base + L::BARRIER_OFFSET + uint32_t(2 * STAGES + a) * 8; };
    auto acc_empty_bar = [&](int a) { return base + L::BARRIER_OFFSET + uint32_t(2 * STAGES + 2 + a) * 8; };

    const int warp = threadIdx.x / 32;
    const uint32_t lane = ptx::lane_id();
    const uint32_t cta_rank = CTA_GROUP == 2 ? ptx::cluster_cta_rank() : 0u;
    const bool leader = cta_rank == 0;
    const int cluster_id = blockIdx.x / CTA_GROUP;
    const int cluster_count = gridDim.x / CTA_GROUP;
    const int tile_count = p.tiles_m * p.tiles_n;
    const int k_blocks = (p.k + ROW_BYTES - 1) / ROW_BYTES;           // 128 one-byte elements per stage

    if (threadIdx.x == 0) {
        *abort_flag = 0;
        for (int s = 0; s < STAGES; s++) {
            ptx::mbarrier_init(full_bar(s), 1);
            ptx::mbarrier_init(empty_bar(s), 1);
        }
        for (int a = 0; a < 2; a++) {
            ptx::mbarrier_init(acc_full_bar(a), 1);
            ptx::mbarrier_init(acc_empty_bar(a), EPILOGUE_WARPS * CTA_GROUP);
        }
        ptx::fence_mbarrier_init();
        ptx::prefetch_tensor_map(map_a);
        ptx::prefetch_tensor_map(map_b);
        ptx::prefetch_tensor_map(map_sa);
        ptx::prefetch_tensor_map(map_sb);
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

    if (warp == 0) {
        // ------------------------------------------------------------------ producer: A, B, one scale block of A, two of B
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
                const int row_block = tile_m * CTA_GROUP + int(cta_rank);          // 128-row block of A this CTA owns
                const int row_a = row_block * BLOCK_M, row_b = tile_n * BN + int(cta_rank) * L::B_ROWS;
                for (int kb = item.kb_begin; kb < item.kb_end; kb++) {
                    if (!ptx::mbarrier_wait(empty_bar(stage), phase ^ 1, abort_flag)) {
                        report(p, abort_flag, STATUS_PRODUCER_TIMEOUT, tile, kb);
                        ok = false;
                        break;
                    }
                    constexpr uint32_t BYTES = L::A_BYTES + L::B_BYTES + 3 * MX_SCALE_BLOCK_BYTES;
                    if constexpr (CTA_GROUP == 1) {
                        ptx::mbarrier_arrive_expect_tx(full_bar(stage), BYTES);
                        ptx::tma_load_2d(stage_a(stage), map_a, kb * ROW_BYTES, row_a, full_bar(stage));
                        ptx::tma_load_2d(stage_b(stage), map_b, kb * ROW_BYTES, row_b, full_bar(stage));
                        ptx::tma_load_2d(stage_scales(stage, 0), map_sa, 0, (row_block * k_blocks + kb) * 32, full_bar(stage));
                        ptx::tma_load_2d(stage_scales(stage, 1), map_sb, 0, (tile_n * k_blocks + kb) * 64, full_bar(stage));
                    } else {
                        if (leader) ptx::mbarrier_arrive_expect_tx(full_bar(stage), 2 * BYTES);
                        const uint32_t leader_bar = ptx::map_to_cta(full_bar(stage), 0);
                        ptx::tma_load_2d_pair(stage_a(stage), map_a, kb * ROW_BYTES, row_a, leader_bar);
                        ptx::tma_load_2d_pair(stage_b(stage), map_b, kb * ROW_BYTES, row_b, leader_bar);
                        ptx::tma_load_2d_pair(stage_scales(stage, 0), map_sa, 0, (row_block * k_blocks + kb) * 32, leader_bar);
                        ptx::tma_load_2d_pair(stage_scales(stage, 1), map_sb, 0, (tile_n * k_blocks + kb) * 64, leader_bar);
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
        // ------------------------------------------------------------------ MMA issuer
        if (lane == 0 && leader) {
            int stage = 0, acc = 0;
            uint32_t phase = 0, acc_phase = 0;
            bool ok = true;
            WorkWalker<STREAMK> walker(tile_count, k_blocks, cluster_id, cluster_count, p.split_tiles);
            WorkItem item;
            while (ok && walker.next(item)) {
                const int tile = item.tile;
                if (!ptx::mbarrier_wait<CTA_GROUP == 2>(acc_empty_bar(acc), acc_phase ^ 1, abort_flag)) {
                    report(p, abort_flag, STATUS_MMA_TIMEOUT, tile, -1);
                    break;
                }
                ptx::tcgen05_fence_after();
                const uint32_t d_tmem = tmem_base + uint32_t(acc) * BN;
                for (int kb = item.kb_begin; kb < item.kb_end; kb++) {
                    if (!ptx::mbarrier_wait(full_bar(stage), phase, abort_flag)) {
                        report(p, abort_flag, STATUS_MMA_TIMEOUT, tile, kb);
                        ok = false;
                        break;
                    }
                    ptx::tcgen05_fence_after();
                    const uint32_t scale_a_tmem = tmem_base + SCALE_COLUMN + uint32_t(stage) * 12, scale_b_tmem = scale_a_tmem + 4;
                    tcgen05_copy_32x128b_warpx4<CTA_GROUP>(scale_a_tmem, ptx::smem_descriptor_rows16(stage_scales(stage, 0)));
                    tcgen05_copy_32x128b_warpx4<CTA_GROUP>(scale_b_tmem, ptx::smem_descriptor_rows16(stage_scales(stage, 1)));
                    tcgen05_copy_32x128b_warpx4<CTA_GROUP>(scale_b_tmem + 4, ptx::smem_descriptor_rows16(stage_scales(stage, 2)));
                    const uint64_t a_desc = ptx::smem_descriptor_k_major_sw128(stage_a(stage));
                    const uint64_t b_desc = ptx::smem_descriptor_k_major_sw128(stage_b(stage));
#pragma unroll
                    for (int j = 0; j < ROW_BYTES / MMA_K_BYTES; j++)
                        tcgen05_mma_mx<CTA_GROUP>(d_tmem, a_desc + uint64_t(j * (MMA_K_BYTES >> 4)), b_desc + uint64_t(j * (MMA_K_BYTES >> 4)),
                                       IDESC | (uint32_t(j) << 29) | (uint32_t(j) << 4), scale_a_tmem, scale_b_tmem, uint32_t(kb != item.kb_begin || j != 0));
                    if constexpr (CTA_GROUP == 1) ptx::tcgen05_commit(empty_bar(stage));
                    else ptx::tcgen05_commit_pair(empty_bar(stage), 0x3);
                    if (++stage == STAGES) { stage = 0; phase ^= 1; }
                }
                if (!ok) break;
                if constexpr (CTA_GROUP == 1) ptx::tcgen05_commit(acc_full_bar(acc));
                else ptx::tcgen05_commit_pair(acc_full_bar(acc), 0x3);
                if (++acc == 2) { acc = 0; acc_phase ^= 1; }
            }
        }
    } else {
        // ------------------------------------------------------------------ epilogue
        const int quadrant = warp % 4;
        uint32_t acc_phase = 0;
        int acc = 0;
        WorkWalker<STREAMK> walker(tile_count, k_blocks, cluster_id, cluster_count, p.split_tiles);
        WorkItem item;
        while (walker.next(item)) {
            const int tile = item.tile;
            int tile_m, tile_n;
            tile_position(tile, p, tile_m, tile_n);
            const bool ready = ptx::mbarrier_wait(acc_full_bar(acc), acc_phase, abort_flag);
            if (!__all_sync(0xffffffffu, ready)) {
                if (lane == 0) report(p, abort_flag, STATUS_EPILOGUE_TIMEOUT, tile, -1);
                break;
            }
            ptx::tcgen05_fence_after();
            const int row = (tile_m * CTA_GROUP + int(cta_rank)) * BLOCK_M + quadrant * 32 + int(lane);
            const uint32_t lane_base = tmem_base + (uint32_t(quadrant * 32) << 16) + uint32_t(acc) * BN;
            constexpr int TILE_ROWS = BLOCK_M * CTA_GROUP;
            constexpr size_t PART = size_t(TILE_ROWS) * BLOCK_N / 4;      // one part, in 16-byte units (a dense tile's extent)
            const int row_in_tile = int(cta_rank) * BLOCK_M + quadrant * 32 + int(lane);
            const bool shared_tile = STREAMK && item.split_tile >= 0;
            uint4 *parts = shared_tile ? reinterpret_cast<uint4 *>(p.partials) + size_t(item.split_tile) * p.max_contributors * PART + row_in_tile : nullptr;
#pragma unroll 1
            for (int chunk = 0; chunk < BN / 32; chunk++) {
                uint32_t values[32];
                ptx::tmem_load_32x32(lane_base + uint32_t(chunk * 32), values);
                ptx::tmem_load_wait();
                if (shared_tile) {
                    // this group's share of the tile's K-blocks: the 32-bit sums go to scratch as they are
                    uint4 *mine = parts + size_t(item.contributor) * PART;
#pragma unroll
                    for (int i = 0; i < 8; i++)
                        mine[size_t(chunk * 8 + i) * TILE_ROWS] = make_uint4(values[4 * i], values[4 * i + 1], values[4 * i + 2], values[4 * i + 3]);
                } else {
                    store_chunk<OUT>(p, values, row, tile_n * BN + chunk * 32);
                }
            }
            if (shared_tile) {
                // the accumulator goes back first; then whoever brings the last part of these 32 rows adds the parts up in the
                // contributors' order and stores.  Nobody waits for anybody.
                ptx::tcgen05_fence_before();
                __syncwarp();
                if (lane == 0) {
                    if (CTA_GROUP == 1 || leader) ptx::mbarrier_arrive(acc_empty_bar(acc));
                    else ptx::mbarrier_arrive_cluster_relaxed(ptx::map_to_cta(acc_empty_bar(acc), 0));
                }
                if (++acc == 2) { acc = 0; acc_phase ^= 1; }
                unsigned int *counter = p.split_counters + item.split_tile * (4 * CTA_GROUP) + int(cta_rank) * 4 + quadrant;
                __threadfence();
                __syncwarp();
                unsigned int earlier = 0;
                if (lane == 0) earlier = atomicAdd(counter, 1u);
                earlier = __shfl_sync(0xffffffffu, earlier, 0);
                if (earlier == unsigned(item.contributors - 1)) {
                    __threadfence();
                    if (lane == 0) *counter = 0;       // ready for the next launch
#pragma unroll 1
                    for (int chunk = 0; chunk < BN / 32; chunk++) {
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
                        store_chunk<OUT>(p, sum, row, tile_n * BN + chunk * 32);
                    }
                }
                continue;
            }
            ptx::tcgen05_fence_before();
            __syncwarp();
            if (lane == 0) {
                // no release needed: the accumulator has been read out, nothing is published through ordinary memory
                if (CTA_GROUP == 1 || leader) ptx::mbarrier_arrive(acc_empty_bar(acc));
                else ptx::mbarrier_arrive_cluster_relaxed(ptx::map_to_cta(acc_empty_bar(acc), 0));
            }
            if (++acc == 2) { acc = 0; acc_phase ^= 1; }
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
