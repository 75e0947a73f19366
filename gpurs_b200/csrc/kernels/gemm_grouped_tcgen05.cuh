// Grouped (mixture-of-experts) GEMM for sm_100a:
//
//     output[r, :] = input[routes[r], :] * weight[e]^T      for offsets[e] <= r < offsets[e + 1],
//
// the reference's `experts` example (examples/ada/examples/grouped_matrix.rs:30-60): rows routed to expert e are
// gathered by index straight from the activations and multiplied by that expert's own N x K weight (weight is
// [experts][N][K], K contiguous).  Tiles never straddle two experts: expert e's rows are cut into tiles of 128 starting
// at offsets[e] (the reference's Grouped scheduler, crates/gpurs/src/gpu/tensor/schedule/grouped.rs:13-68); the number
// of tiles is only known on the device, so the persistent CTAs walk tile indices until they run past it.
//
// Roles (320 threads): warp 0 loads the weight tile with TMA; warps 6..9 gather the 128 activation rows of the stage
// with asynchronous 16-byte copies (cp.async; 8 threads per 128-byte row, whole lines) straight into shared memory in the
// 128-byte swizzle the tensor core expects (the reference's gather cursor, crates/gpurs/src/gpu/tensor/global/gather.rs:19-115),
// rows past the end of the group as zeros; warp 1 issues tcgen05.mma into one of two TMEM accumulators; warps 2..5
// round and store finished tiles while the next one is being multiplied.
#pragma once
#include "gemm_tcgen05.cuh"

namespace gemm {

constexpr int GATHER_THREADS = 128;

struct GroupedParams {
    void *c;                      // rows x n output, row pitch ldc
    long long ldc;
    const void *input;            // tokens x k, row pitch lda (elements), the rows `routes` picks from
    long long lda;
    const unsigned int *routes;   // [rows]: input row of every output row
    const unsigned int *offsets;  // [experts + 1]: output rows of expert e are offsets[e] .. offsets[e + 1]
    unsigned int *status;
    int rows, tokens, n, k, experts;
    int tiles_n;                  // ceil(n / 256)
    int vector_stores;
};

// Tile index -> (expert, first output row, end of the expert's rows, tile column).  Tiles are numbered expert by expert,
// row tile by row tile, column fastest.  Returns false past the last tile.
__device__ __forceinline__ bool grouped_tile(const GroupedParams &p, int tile, int &expert, int &first_row, int &end_row, int &tile_n) {
    int row_tile = tile / p.tiles_n;
    tile_n = tile - row_tile * p.tiles_n;
    for (int e = 0; e < p.experts; e++) {
        const int begin = int(__ldg(p.offsets + e)), end = int(__ldg(p.offsets + e + 1));
        const int tiles = (end - begin + BLOCK_M - 1) / BLOCK_M;
        if (row_tile < tiles) {
            expert = e;
            first_row = begin + row_tile * BLOCK_M;
            end_row = end;
            return true;
        }
        row_tile -= tiles;
    }
    return false;
}

template <int ELEMENT_FORMAT, int OUT, int STAGES>
__device__ __forceinline__ void gemm_grouped_body(const CUtensorMap *map_w, const GroupedParams &p) {
    using L = SharedLayout<BLOCK_N, 1, STAGES>;
    constexpr uint32_t TMEM_COLUMNS = 2 * BLOCK_N;
    constexpr uint32_t IDESC = instruction_descriptor(1, ELEMENT_FORMAT, BLOCK_M, BLOCK_N);
    constexpr int BLOCK_K = ROW_BYTES / 2;

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
    const int k_blocks = (p.k + BLOCK_K - 1) / BLOCK_K;

    if (threadIdx.x == 0) {
        *abort_flag = 0;
        for (int s = 0; s < STAGES; s++) {
            ptx::mbarrier_init(full_bar(s), 1 + GATHER_THREADS);     // the weight load's arrive + every gathering thread
            ptx::mbarrier_init(empty_bar(s), 1);
        }
        for (int a = 0; a < 2; a++) {
            ptx::mbarrier_init(acc_full_bar(a), 1);
            ptx::mbarrier_init(acc_empty_bar(a), EPILOGUE_WARPS);
        }
        ptx::fence_mbarrier_init();
        ptx::prefetch_tensor_map(map_w);
    }
    if (warp == 1) {
        ptx::tmem_alloc<1>(ptx::smem_u32(const_cast<uint32_t *>(tmem_slot)), TMEM_COLUMNS);
        ptx::tmem_relinquish<1>();
    }
    ptx::tcgen05_fence_before();
    __syncthreads();
    ptx::tcgen05_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    // Everything above touched no global memory and may have overlapped the previous kernel of the stream.
    ptx::grid_dependency_wait();
    ptx::grid_dependency_launch();

    int expert, first_row, end_row, tile_n;
    if (warp == 0) {
        // ------------------------------------------------------------------ weight producer (TMA)
        if (lane == 0) {
            int stage = 0;
            uint32_t phase = 0;
            bool ok = true;
            for (int tile = blockIdx.x; ok && grouped_tile(p, tile, expert, first_row, end_row, tile_n); tile += gridDim.x) {
                const int weight_row = expert * p.n + tile_n * BLOCK_N;    // rows of the [experts * n][k] weight
                for (int kb = 0; kb < k_blocks; kb++) {
                    if (!ptx::mbarrier_wait(empty_bar(stage), phase ^ 1, abort_flag)) {
                        report_status(p.status, abort_flag, STATUS_PRODUCER_TIMEOUT, tile, kb);
                        ok = false;
                        break;
                    }
                    ptx::mbarrier_arrive_expect_tx(full_bar(stage), L::B_BYTES);
                    // rows past this expert's n columns belong to the next expert: the epilogue never stores them
                    ptx::tma_load_2d(stage_b(stage), map_w, kb * BLOCK_K, weight_row, full_bar(stage));
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
        if (lane == 0) {
            int stage = 0, acc = 0;
            uint32_t phase = 0, acc_phase = 0;
            bool ok = true;
            for (int tile = blockIdx.x; ok && grouped_tile(p, tile, expert, first_row, end_row, tile_n); tile += gridDim.x) {
                if (!ptx::mbarrier_wait(acc_empty_bar(acc), acc_phase ^ 1, abort_flag)) {
                    report_status(p.status, abort_flag, STATUS_MMA_TIMEOUT, tile, -1);
                    break;
                }
                ptx::tcgen05_fence_after();
                const uint32_t d_tmem = tmem_base + uint32_t(acc) * BLOCK_N;
                for (int kb = 0; kb < k_blocks; kb++) {
                    if (!ptx::mbarrier_wait(full_bar(stage), phase, abort_flag)) {
                        report_status(p.status, abort_flag, STATUS_MMA_TIMEOUT, tile, kb);
                        ok = false;
                        break;
                    }
                    ptx::tcgen05_fence_after();
                    const uint64_t a_desc = ptx::smem_descriptor_k_major_sw128(stage_a(stage));
                    const uint64_t b_desc = ptx::smem_descriptor_k_major_sw128(stage_b(stage));
#pragma unroll
                    for (int j = 0; j < ROW_BYTES / MMA_K_BYTES; j++)
                        ptx::tcgen05_mma<ptx::KIND_F16, 1>(d_tmem, a_desc + uint64_t(j * (MMA_K_BYTES >> 4)), b_desc + uint64_t(j * (MMA_K_BYTES >> 4)),
                                                           IDESC, uint32_t((kb | j) != 0));
                    ptx::tcgen05_commit(empty_bar(stage));
                    if (++stage == STAGES) { stage = 0; phase ^= 1; }
                }
                if (!ok) break;
                ptx::tcgen05_commit(acc_full_bar(acc));
                if (++acc == 2) { acc = 0; acc_phase ^= 1; }
            }
        }
    } else if (warp < 6) {
        // ------------------------------------------------------------------ epilogue
        const int quadrant = warp % 4;
        int acc = 0;
        uint32_t acc_phase = 0;
        Params out{};                     // what store_chunk reads: the output, clipped to this expert's rows; no algebra (all zero)
        out.c = p.c, out.ldc = p.ldc, out.n = p.n, out.vector_stores = p.vector_stores;
        for (int tile = blockIdx.x; grouped_tile(p, tile, expert, first_row, end_row, tile_n); tile += gridDim.x) {
            const bool ready = ptx::mbarrier_wait(acc_full_bar(acc), acc_phase, abort_flag);
            if (!__all_sync(0xffffffffu, ready)) {
                if (lane == 0) report_status(p.status, abort_flag, STATUS_EPILOGUE_TIMEOUT, tile, -1);
                break;
            }
            ptx::tcgen05_fence_after();
            out.m = end_row;
            const int row = first_row + quadrant * 32 + int(lane);
            const uint32_t lane_base = tmem_base + (uint32_t(quadrant * 32) << 16) + uint32_t(acc) * BLOCK_N;
#pragma unroll 1
            for (int chunk = 0; chunk < BLOCK_N / 32; chunk++) {
                uint32_t values[32];
                ptx::tmem_load_32x32(lane_base + uint32_t(chunk * 32), values);
                ptx::tmem_load_wait();
                store_chunk<OUT>(out, values, row, tile_n * BLOCK_N + chunk * 32);
            }
            ptx::tcgen05_fence_before();
            __syncwarp();
            if (lane == 0) ptx::mbarrier_arrive(acc_empty_bar(acc));
            if (++acc == 2) { acc = 0; acc_phase ^= 1; }
        }
    } else {
        // ------------------------------------------------------------------ gather producer
        // thread g of 128: 16-byte piece g % 8 of rows g / 8 + 16 * i (i = 0..7): a warp instruction reads four whole rows
        const int g = int(threadIdx.x) - 6 * 32;
        const int piece = g % 8;
        const uint16_t *input = reinterpret_cast<const uint16_t *>(p.input);
        int stage = 0;
        uint32_t phase = 0;
        bool ok = true;
        for (int tile = blockIdx.x; ok && grouped_tile(p, tile, expert, first_row, end_row, tile_n); tile += gridDim.x) {
            const uint16_t *source[8];
#pragma unroll
            for (int i = 0; i < 8; i++) {
                const int row = first_row + g / 8 + 16 * i;
                source[i] = row < end_row ? input + size_t(min(__ldg(p.routes + row), uint32_t(p.tokens - 1))) * p.lda + piece * 8 : nullptr;
            }
            for (int kb = 0; kb < k_blocks; kb++) {
                if (!ptx::mbarrier_wait(empty_bar(stage), phase ^ 1, abort_flag)) {
                    if (g == 0) report_status(p.status, abort_flag, STATUS_PRODUCER_TIMEOUT, tile, kb);
                    ok = false;
                    break;
                }
                // Asynchronous 16-byte copies straight into the swizzled tile: nothing is waited for here, so the gather
                // runs as many stages ahead as the ring allows and the latency of the scattered rows is hidden by it.
                const bool inside = kb * BLOCK_K + piece * 8 < p.k;
#pragma unroll
                for (int i = 0; i < 8; i++) {
                    const int r = g / 8 + 16 * i;                // row of the tile: 128 bytes per row, piece j at slot j ^ (r % 8)
                    const bool valid = inside && source[i] != nullptr;
                    ptx::copy_async_16(stage_a(stage) + uint32_t(r * ROW_BYTES + ((piece ^ (r & 7)) * 16)),
                                       valid ? static_cast<const void *>(source[i] + kb * BLOCK_K) : p.input, valid ? 16u : 0u);
                }
                ptx::copy_async_arrive(full_bar(stage));         // arrives when this thread's copies have landed
                if (++stage == STAGES) { stage = 0; phase ^= 1; }
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
    __syncthreads();
    if (warp == 1) {
        ptx::tcgen05_fence_after();
        ptx::tmem_dealloc<1>(tmem_base, TMEM_COLUMNS);
    }
}

}  // namespace gemm
