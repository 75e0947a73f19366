// 2:4 structured-sparse GEMM for sm_100a (16-bit operands):
//
//     C[m, n] = sum_k A[m, k] * B[n, k],     A has at most 2 non-zeros in every aligned group of 4 along K.
//
// The reference has nothing for this (no sparse instruction, kernel or test); the definition is the dense
// product of the densified A.  A arrives compressed: `values` is M x K/2 (the kept pair of every group, in
// order) and `metadata` holds, per group, the two 2-bit positions of the kept elements (low bits first),
// arranged in 2048-byte blocks, one per 128 rows x 128 logical K, in the order the tensor core reads them
// from tensor memory (see metadata_offset below; gpurs_compress_24 in transform.cu produces both).
//
// One pipeline stage is 128 logical K: 128 bytes of compressed A per row, two 128-byte-swizzled tiles of B
// (logical K 0..63 and 64..127) and one metadata block.  The MMA thread copies the block into tensor memory
// (tcgen05.cp, 4 columns) and issues 4 tcgen05.mma.sp of 32 logical K each, one metadata column apiece.
// Tensor memory: two accumulators of 224 columns (tiles are 224 columns wide for that reason: the epilogue of a tile
// overlaps the main loop of the next) plus 4 metadata columns per stage.  With one 256-column accumulator the exposed
// epilogue and hand-over cost about 4 us per tile, 15 % at K = 8192 (measured by varying K).
#pragma once
#include "gemm_tcgen05.cuh"

namespace gemm {

constexpr int SPARSE_STAGE_K = 128;            // logical K per stage
constexpr int METADATA_BLOCK_BYTES = 2048;     // 128 rows x 128 logical K x 4 bits per group of 4

// Byte offset, inside its 2048-byte block, of the metadata of logical element (row, k) of a 128 x 128 block,
// and the nibble within that byte.  Row r = r0 + 8*r1 + 16*r2 (r0 < 8, r1 < 2), k = k0 + 16*k1 + 32*k2
// (k0 < 16, k1 < 2, k2 < 4):  offset = 16*r0 + 2*r1 + 256*r2 + 128*k1 + 4*k2 + k0/8, nibble = (k0 % 8) / 4.
// Read as 128 units of 16 bytes, unit u = r0 + 8*k1 + 16*r2 lands in TMEM lane u, and its four 32-bit words are
// the metadata columns of the stage's four instructions (k2): low half-word row r1 = 0, high half-word r1 = 1.
__host__ __device__ inline int metadata_offset(int row, int k) {
    return 16 * (row % 8) + 2 * ((row / 8) % 2) + 256 * (row / 16) + 128 * ((k / 16) % 2) + 4 * (k / 32) + (k % 16) / 8;
}

template <int CTA_GROUP, int STAGES>
struct SparseLayout {
    static constexpr int A_BYTES = BLOCK_M * ROW_BYTES;                   // 128 rows x 64 kept elements
    static constexpr int B_ROWS = SPARSE_BLOCK_N / CTA_GROUP;
    static constexpr int B_HALF_BYTES = B_ROWS * ROW_BYTES;               // one 64-deep half of the B tile
    static constexpr int STAGE_BYTES = A_BYTES + 2 * B_HALF_BYTES + METADATA_BLOCK_BYTES;
    static constexpr int BARRIER_OFFSET = ((STAGES * STAGE_BYTES + 1023) / 1024) * 1024;
    static constexpr int NUM_BARRIERS = 2 * STAGES + 4;                   // full, empty, two accumulators' full / empty
    static constexpr int TMEM_SLOT_OFFSET = BARRIER_OFFSET + NUM_BARRIERS * 8;
    static constexpr int ABORT_OFFSET = TMEM_SLOT_OFFSET + 4;
    static constexpr int DYNAMIC_BYTES = ABORT_OFFSET + 4 + 1024;
    // the push entries stage their output boxes behind everything else: two 4 KiB buffers per epilogue warp
    static constexpr int STAGING_OFFSET = ((ABORT_OFFSET + 4 + 1023) / 1024) * 1024;
    static constexpr int PUSH_DYNAMIC_BYTES = STAGING_OFFSET + EPILOGUE_WARPS * 2 * 32 * ROW_BYTES + 1024;
};

// Destinations of the push epilogue of the sparse kernels (bf16 output): as gemm::PushTargets, with a second descriptor per
// GPU whose boxes are 32 columns wide and unswizzled, for the last 32 of a tile's 224 columns.
struct SparsePushTargets {
    CUtensorMap maps[MAX_PUSH_TARGETS];        // boxes of 32 rows x 64 columns, 128-byte swizzle
    CUtensorMap half_maps[MAX_PUSH_TARGETS];   // boxes of 32 rows x 32 columns, rows of 64 bytes back to back
    int count;
    int row_offset;
    int first;
    int reserved;
};

constexpr int SPARSE_STAGES_SINGLE = 2;   // 74 KiB per stage
constexpr int SPARSE_STAGES_PAIR = 4;     // 46 KiB per stage and CTA
static_assert(SparseLayout<1, SPARSE_STAGES_SINGLE>::DYNAMIC_BYTES == SPARSE_SHARED_SINGLE, "host and kernel disagree on shared memory");
static_assert(SparseLayout<2, SPARSE_STAGES_PAIR>::DYNAMIC_BYTES == SPARSE_SHARED_PAIR, "host and kernel disagree on shared memory");
static_assert(SparseLayout<2, SPARSE_STAGES_PAIR>::PUSH_DYNAMIC_BYTES == SPARSE_SHARED_PAIR_PUSH, "host and kernel disagree on shared memory");
static_assert(METADATA_BLOCK_BYTES == SPARSE_METADATA_BLOCK_BYTES && SPARSE_STAGE_K == SPARSE_BLOCK_K, "host and kernel disagree on the metadata block");

// ELEMENT_FORMAT: 0 = f16, 1 = bf16.  map_e describes the metadata as rows of 16 bytes (box 16 x 128).
// PUSH (bf16 output): every finished box of C is stored to all GPUs' copies of the gathered matrix (PushTargets) by TMA
// stores from shared staging, as the dense push kernels do.  A 224-column tile is three boxes of 64 columns (128-byte
// swizzled staging) and one of 32 (staged as plain 64-byte rows, its own descriptors): writing columns 160..191 twice with a
// fourth full box instead was measured at 8 GPUs and cost the 14 % more bytes it sends.
// STREAMK: the K-blocks of the tiles of a split round are spread over the CTA groups (gemm_schedule.hpp) and the parts are added
// up by whoever arrives last, as in gemm_body; a part is laid out like a dense tile's (256 columns wide, 224 used).
template <int ELEMENT_FORMAT, int OUT, int CTA_GROUP, int STAGES, bool PUSH = false, bool STREAMK = false>
__device__ __forceinline__ void gemm_sparse_body(const CUtensorMap *map_a, const CUtensorMap *map_b, const CUtensorMap *map_e, const Params &p,
                                                 const SparsePushTargets *targets = nullptr) {
    static_assert(!PUSH || OUT == OUT_BF16, "the push epilogue of the sparse kernels writes bf16");
    static_assert(!(PUSH && STREAMK), "the push epilogue stores whole tiles");
    using L = SparseLayout<CTA_GROUP, STAGES>;
    constexpr int BN = SPARSE_BLOCK_N;
    constexpr uint32_t TMEM_COLUMNS = 512;
    constexpr uint32_t METADATA_COLUMN = 2 * BN;  // metadata of stage s: columns 2*BN + 4*s .. +3, after the two accumulators
    static_assert(2 * BN + 4 * STAGES <= 512 && BN % 32 == 0, "two accumulators and the metadata must fit tensor memory");
    // sparse flag (bit 2) on top of the dense descriptor
    constexpr uint32_t IDESC = instruction_descriptor(1, ELEMENT_FORMAT, BLOCK_M * CTA_GROUP, BN) | (1u << 2);
    static_assert(L::STAGE_BYTES % 1024 == 0, "stages must keep the 1024-byte alignment of the swizzled tiles");

    extern __shared__ uint8_t raw_shared[];
    const uint32_t base = (ptx::smem_u32(raw_shared) + 1023u) & ~1023u;
    uint8_t *aligned = raw_shared + (base - ptx::smem_u32(raw_shared));
    volatile uint32_t *tmem_slot = reinterpret_cast<volatile uint32_t *>(aligned + L::TMEM_SLOT_OFFSET);
    volatile uint32_t *abort_flag = reinterpret_cast<volatile uint32_t *>(aligned + L::ABORT_OFFSET);

    auto stage_a = [&](int s) { return base + uint32_t(s) * L::STAGE_BYTES; };
    auto stage_b = [&](int s, int half) { return base + uint32_t(s) * L::STAGE_BYTES + L::A_BYTES + uint32_t(half) * L::B_HALF_BYTES; };
    auto stage_e = [&](int s) { return base + uint32_t(s) * L::STAGE_BYTES + L::A_BYTES + 2 * L::B_HALF_BYTES; };
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
    const int k_blocks = (p.k + SPARSE_STAGE_K - 1) / SPARSE_STAGE_K;     // p.k is the logical depth

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
        ptx::prefetch_tensor_map(map_e);
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
        // ------------------------------------------------------------------ producer: A, two halves of B, metadata
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
                const int row_a = row_block * BLOCK_M;
                const int row_b = tile_n * BN + int(cta_rank) * L::B_ROWS;
                for (int kb = item.kb_begin; kb < item.kb_end; kb++) {
                    if (!ptx::mbarrier_wait(empty_bar(stage), phase ^ 1, abort_flag)) {
                        report(p, abort_flag, STATUS_PRODUCER_TIMEOUT, tile, kb);
                        ok = false;
                        break;
                    }
                    const int k_logical = kb * SPARSE_STAGE_K;
                    const int metadata_row = (row_block * k_blocks + kb) * 128;     // 128 rows of 16 bytes per block
                    if constexpr (CTA_GROUP == 1) {
                        ptx::mbarrier_arrive_expect_tx(full_bar(stage), L::STAGE_BYTES);
                        ptx::tma_load_2d(stage_a(stage), map_a, k_logical / 2, row_a, full_bar(stage));
                        ptx::tma_load_2d(stage_b(stage, 0), map_b, k_logical, row_b, full_bar(stage));
                        ptx::tma_load_2d(stage_b(stage, 1), map_b, k_logical + 64, row_b, full_bar(stage));
                        ptx::tma_load_2d(stage_e(stage), map_e, 0, metadata_row, full_bar(stage));
                    } else {
                        if (leader) ptx::mbarrier_arrive_expect_tx(full_bar(stage), 2 * L::STAGE_BYTES);
                        const uint32_t leader_bar = ptx::map_to_cta(full_bar(stage), 0);
                        ptx::tma_load_2d_pair(stage_a(stage), map_a, k_logical / 2, row_a, leader_bar);
                        ptx::tma_load_2d_pair(stage_b(stage, 0), map_b, k_logical, row_b, leader_bar);
                        ptx::tma_load_2d_pair(stage_b(stage, 1), map_b, k_logical + 64, row_b, leader_bar);
                        ptx::tma_load_2d_pair(stage_e(stage), map_e, 0, metadata_row, leader_bar);
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
            int stage = 0;
            uint32_t phase = 0, acc_phase = 0;
            int acc = 0;
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
                    const uint32_t metadata_tmem = tmem_base + METADATA_COLUMN + uint32_t(stage) * 4;
                    ptx::tcgen05_copy_128x128b<CTA_GROUP>(metadata_tmem, ptx::smem_descriptor_rows16(stage_e(stage)));
                    const uint64_t a_desc = ptx::smem_descriptor_k_major_sw128(stage_a(stage));
#pragma unroll
                    for (int j = 0; j < 4; j++) {
                        // instruction j: 32 logical K = 32 bytes of compressed A, 64 bytes of B (half j / 2, offset j % 2)
                        const uint64_t b_desc = ptx::smem_descriptor_k_major_sw128(stage_b(stage, j / 2)) + uint64_t((j % 2) * (64 >> 4));
                        // The instruction takes the metadata column pair (an even column address) and, in bits 0..1 of
                        // its descriptor, which column of the pair to use.
                        const uint32_t column = metadata_tmem + uint32_t(j);
                        ptx::tcgen05_mma_sparse_f16<CTA_GROUP>(d_tmem, a_desc + uint64_t(j * (MMA_K_BYTES >> 4)), b_desc,
                                                               column & ~1u, IDESC | (column & 1u), uint32_t(kb != item.kb_begin || j != 0));
                    }
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
        [[maybe_unused]] int stores = 0;     // push epilogue: TMA stores issued by this warp, picks the staging buffer
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
            if constexpr (PUSH) {
                const int warp_row = (tile_m * CTA_GROUP + int(cta_rank)) * BLOCK_M + quadrant * 32;
                const uint32_t staging = base + L::STAGING_OFFSET;
#pragma unroll 1
                for (int box = 0; box < (BN + 63) / 64; box++) {
                    const int column = tile_n * BN + box * 64;
                    const bool half = box * 64 + 64 > BN;            // the tile's last 32 columns
                    uint32_t low[32], high[32], packed[32];
                    ptx::tmem_load_32x32(lane_base + uint32_t(box * 64), low);
                    if (!half) ptx::tmem_load_32x32(lane_base + uint32_t(box * 64 + 32), high);
                    ptx::tmem_load_wait();
                    apply_epilogue<OUT>(p, low, row, column);
                    if (!half) apply_epilogue<OUT>(p, high, row, column + 32);
#pragma unroll
                    for (int i = 0; i < 16; i++) {
                        packed[i] = pack_pair<OUT>(low[2 * i], low[2 * i + 1]);
                        packed[16 + i] = half ? 0u : pack_pair<OUT>(high[2 * i], high[2 * i + 1]);
                    }
                    if (warp_row < p.m && column < p.n) {
                        const uint32_t buffer = staging + uint32_t(((warp - 2) * 2 + (stores & 1)) * 32 * ROW_BYTES);
                        stores++;
                        if (lane == 0) ptx::tma_store_wait_read<1>();
                        __syncwarp();
                        if (half) {
#pragma unroll
                            for (int j = 0; j < 4; j++)                      // rows of 64 bytes back to back, no swizzle
                                ptx::store_shared_v4(buffer + lane * 64u + uint32_t(j * 16), packed[4 * j], packed[4 * j + 1], packed[4 * j + 2], packed[4 * j + 3]);
                        } else {
#pragma unroll
                            for (int j = 0; j < 8; j++)                      // lane = row; 16-byte piece j goes to slot j ^ (row % 8)
                                ptx::store_shared_v4(buffer + lane * ROW_BYTES + uint32_t((j ^ int(lane & 7)) * 16), packed[4 * j], packed[4 * j + 1],
                                                     packed[4 * j + 2], packed[4 * j + 3]);
                        }
                        ptx::fence_async_shared();
                        __syncwarp();
                        if (lane == 0) {
                            for (int t = 0; t < targets->count; t++) {
                                const int target = targets->first + t < targets->count ? targets->first + t : targets->first + t - targets->count;
                                ptx::tma_store_2d(half ? &targets->half_maps[target] : &targets->maps[target], column, targets->row_offset + warp_row, buffer);
                            }
                            ptx::tma_store_commit();
                        }
                    }
                }
            } else {
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
        if constexpr (PUSH) {
            if (lane == 0) ptx::tma_store_wait<0>();   // this warp's stores have been performed before the block exits
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
