// Decode-shaped ("skinny") GEMM for sm_100a: few rows of A against a large B, plus a bias,
//
//     C[m, n] = bias[n] + sum_k A[m, k] * B[n, k],        m <= 64, fp32 output,
//
// the reference's `project` example (examples/ada/examples/skinny_matrix.rs:35-68: 16 tokens x a 4096 x 4096 f16
// weight + bias).  Like the reference the operands are swapped so that the big one fills the tensor core's row
// operand: 128 rows of B become the 128 TMEM lanes of a tcgen05.mma with M = 128 and N = TOKENS, A's rows are the
// instruction's N.  The work is bound by streaming B from HBM once, so K is split among several CTAs per 128-row
// tile (the reference's SplitDepth, crates/gpurs/src/gpu/tensor/schedule/split.rs:11-62) to put every SM on the
// stream.  Every split parks its partial sums in scratch and counts in on a per-tile counter; the warp that counts
// in last adds all partials, always in split order, plus the bias, and writes C.  The result therefore does not
// depend on timing, and no second launch is needed: the two properties the reference gets from its TileLock
// (crates/gpurs/src/gpu/tensor/output/reduction.rs:21-129), which passes the output from split to split in turn.
// (A turn-by-turn hand-over was tried first: each hop cost about 5 us, 57 us for 10 splits.)
#pragma once
#include "gemm_tcgen05.cuh"

namespace gemm {

constexpr int SKINNY_STAGES = 8;   // 8 x 18 KiB in flight per CTA: a short K range is fetched in one or two round trips

// Kernel parameter block of the skinny entries (mirrored by the host in matmul.cpp).
struct SkinnyParams {
    float *c;                  // m x n row-major, pitch ldc
    long long ldc;
    const float *bias;         // [n] or null
    unsigned int *turns;       // four counters per 128-row tile of B (one per 32 columns); zero before and after every launch
    float *partials;           // [tiles][splits][TOKENS][128] partial sums of the splits (splits > 1)
    unsigned int *status;
    int m, n, k;
    int tiles;                 // ceil(n / 128)
    int splits;                // CTAs per tile
    int k_blocks_per_split;    // in stages of 128 bytes of K
};

template <int TOKENS>
struct SkinnyLayout {
    static constexpr int B_BYTES = BLOCK_M * ROW_BYTES;        // 128 rows of the big operand
    static constexpr int A_BYTES = TOKENS * ROW_BYTES;         // the few rows of the small one
    static constexpr int STAGE_BYTES = B_BYTES + ((A_BYTES + 1023) / 1024) * 1024;
    static constexpr int BARRIER_OFFSET = SKINNY_STAGES * STAGE_BYTES;
    static constexpr int NUM_BARRIERS = 2 * SKINNY_STAGES + 1;
    static constexpr int TMEM_SLOT_OFFSET = BARRIER_OFFSET + NUM_BARRIERS * 8;
    static constexpr int ABORT_OFFSET = TMEM_SLOT_OFFSET + 4;
    static constexpr int DYNAMIC_BYTES = ABORT_OFFSET + 4 + 1024;
    static_assert(DYNAMIC_BYTES == skinny_shared_bytes(TOKENS), "host and kernel disagree on shared memory");
};

// ELEMENT_FORMAT: 0 = f16, 1 = bf16.  map_big describes B (box 64 x 128), map_small A (box 64 x TOKENS).
template <int ELEMENT_FORMAT, int TOKENS>
__device__ __forceinline__ void gemm_skinny_body(const CUtensorMap *map_big, const CUtensorMap *map_small, const SkinnyParams &p) {
    using L = SkinnyLayout<TOKENS>;
    static_assert(TOKENS == 16 || TOKENS == 32 || TOKENS == 64, "the small operand is padded to 16, 32 or 64 rows");
    constexpr uint32_t TMEM_COLUMNS = TOKENS < 32 ? 32 : TOKENS;
    constexpr uint32_t IDESC = instruction_descriptor(1, ELEMENT_FORMAT, BLOCK_M, TOKENS);
    constexpr int BLOCK_K = ROW_BYTES / 2;

    extern __shared__ uint8_t raw_shared[];
    const uint32_t base = (ptx::smem_u32(raw_shared) + 1023u) & ~1023u;
    uint8_t *aligned = raw_shared + (base - ptx::smem_u32(raw_shared));
    volatile uint32_t *tmem_slot = reinterpret_cast<volatile uint32_t *>(aligned + L::TMEM_SLOT_OFFSET);
    volatile uint32_t *abort_flag = reinterpret_cast<volatile uint32_t *>(aligned + L::ABORT_OFFSET);
    auto stage_big = [&](int s) { return base + uint32_t(s) * L::STAGE_BYTES; };
    auto stage_small = [&](int s) { return base + uint32_t(s) * L::STAGE_BYTES + L::B_BYTES; };
    auto full_bar = [&](int s) { return base + L::BARRIER_OFFSET + uint32_t(s) * 8; };
    auto empty_bar = [&](int s) { return base + L::BARRIER_OFFSET + uint32_t(SKINNY_STAGES + s) * 8; };
    const uint32_t done_bar = base + L::BARRIER_OFFSET + uint32_t(2 * SKINNY_STAGES) * 8;

    const int warp = threadIdx.x / 32;
    const uint32_t lane = ptx::lane_id();
    const int split = blockIdx.x / p.tiles, tile = blockIdx.x % p.tiles;     // split-major numbering
    const int k_blocks_total = (p.k + BLOCK_K - 1) / BLOCK_K;
    const int first_block = split * p.k_blocks_per_split;
    const int k_blocks = max(0, min(p.k_blocks_per_split, k_blocks_total - first_block));

    if (threadIdx.x == 0) {
        *abort_flag = 0;
        for (int s = 0; s < SKINNY_STAGES; s++) {
            ptx::mbarrier_init(full_bar(s), 1);
            ptx::mbarrier_init(empty_bar(s), 1);
        }
        ptx::mbarrier_init(done_bar, 1);
        ptx::fence_mbarrier_init();
        ptx::prefetch_tensor_map(map_big);
        ptx::prefetch_tensor_map(map_small);
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

    if (warp == 0) {
        if (lane == 0) {
            int stage = 0;
            uint32_t phase = 0;
            for (int kb = 0; kb < k_blocks; kb++) {
                if (!ptx::mbarrier_wait(empty_bar(stage), phase ^ 1, abort_flag)) {
                    report_status(p.status, abort_flag, STATUS_PRODUCER_TIMEOUT, tile, kb);
                    break;
                }
                ptx::mbarrier_arrive_expect_tx(full_bar(stage), L::B_BYTES + L::A_BYTES);
                ptx::tma_load_2d(stage_big(stage), map_big, (first_block + kb) * BLOCK_K, tile * BLOCK_M, full_bar(stage));
                ptx::tma_load_2d(stage_small(stage), map_small, (first_block + kb) * BLOCK_K, 0, full_bar(stage));
                if (++stage == SKINNY_STAGES) { stage = 0; phase ^= 1; }
            }
            // see every stage released before leaving: no commit may arrive on a barrier of a block that has exited
            for (int s = 0; s < SKINNY_STAGES; s++) {
                if (!ptx::mbarrier_wait(empty_bar(stage), phase ^ 1, abort_flag)) break;
                if (++stage == SKINNY_STAGES) { stage = 0; phase ^= 1; }
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            int stage = 0;
            uint32_t phase = 0;
            bool ok = true;
            for (int kb = 0; kb < k_blocks; kb++) {
                if (!ptx::mbarrier_wait(full_bar(stage), phase, abort_flag)) {
                    report_status(p.status, abort_flag, STATUS_MMA_TIMEOUT, tile, kb);
                    ok = false;
                    break;
                }
                ptx::tcgen05_fence_after();
                const uint64_t big = ptx::smem_descriptor_k_major_sw128(stage_big(stage));
                const uint64_t small = ptx::smem_descriptor_k_major_sw128(stage_small(stage));
#pragma unroll
                for (int j = 0; j < ROW_BYTES / MMA_K_BYTES; j++)
                    ptx::tcgen05_mma<ptx::KIND_F16, 1>(tmem_base, big + uint64_t(j * (MMA_K_BYTES >> 4)), small + uint64_t(j * (MMA_K_BYTES >> 4)),
                                                       IDESC, uint32_t((kb | j) != 0));
                ptx::tcgen05_commit(empty_bar(stage));
                if (++stage == SKINNY_STAGES) { stage = 0; phase ^= 1; }
            }
            if (ok) ptx::tcgen05_commit(done_bar);
        }
    } else {
        // ------------------------------------------------------------------ epilogue: ordered split reduction
        const int quadrant = warp % 4;
        const int column_base = tile * BLOCK_M + quadrant * 32;
        const int column = column_base + int(lane);                        // output column = row of the big operand
        uint32_t values[TOKENS];
#pragma unroll
        for (int i = 0; i < TOKENS; i++) values[i] = 0u;
        bool ok = true;
        if (k_blocks > 0) {
            ok = __all_sync(0xffffffffu, ptx::mbarrier_wait(done_bar, 0, abort_flag));
            if (ok) {
                ptx::tcgen05_fence_after();
                tmem_load_columns<TOKENS>(tmem_base + (uint32_t(quadrant * 32) << 16), values);
                ptx::tmem_load_wait();
            } else if (lane == 0) {
                report_status(p.status, abort_flag, STATUS_EPILOGUE_TIMEOUT, tile, -1);
            }
        }
        if (ok && column_base < p.n) {
            if (p.splits == 1) {
                const float first = (p.bias != nullptr && column < p.n) ? __ldg(p.bias + column) : 0.0f;
#pragma unroll
                for (int token = 0; token < TOKENS; token++)
                    if (token < p.m && column < p.n) p.c[size_t(token) * p.ldc + column] = first + __uint_as_float(values[token]);
            } else {
                // Park this split's partial sums (32 lanes -> 32 consecutive floats per token), then count in.
                float *mine = p.partials + ((size_t(tile) * p.splits + split) * TOKENS) * BLOCK_M + quadrant * 32 + lane;
#pragma unroll
                for (int token = 0; token < TOKENS; token++)
                    if (token < p.m) __stcg(mine + size_t(token) * BLOCK_M, __uint_as_float(values[token]));
                __syncwarp();
                unsigned int arrived = 0;
                if (lane == 0) {
                    __threadfence();                                             // the partials before the count
                    arrived = atomicAdd(p.turns + tile * 4 + quadrant, 1u);
                    if (arrived == uint32_t(p.splits) - 1u) {
                        p.turns[tile * 4 + quadrant] = 0;                        // ready for the next launch
                        __threadfence();                                         // the count before the others' partials
                    }
                }
                arrived = __shfl_sync(0xffffffffu, arrived, 0);
                if (arrived == uint32_t(p.splits) - 1u && column < p.n) {
                    // The last warp to arrive for these 32 columns adds every split's partial, always in split order.
                    const float first = p.bias != nullptr ? __ldg(p.bias + column) : 0.0f;
                    const float *all = p.partials + (size_t(tile) * p.splits * TOKENS) * BLOCK_M + quadrant * 32 + lane;
                    float sums[TOKENS];
#pragma unroll
                    for (int token = 0; token < TOKENS; token++) sums[token] = first;
                    for (int s = 0; s < p.splits; s++) {
                        // TOKENS independent loads per split are in flight together; the additions stay in split order
#pragma unroll
                        for (int token = 0; token < TOKENS; token++)
                            if (token < p.m) sums[token] += __ldcg(all + (size_t(s) * TOKENS + token) * BLOCK_M);
                    }
#pragma unroll
                    for (int token = 0; token < TOKENS; token++)
                        if (token < p.m) p.c[size_t(token) * p.ldc + column] = sums[token];
                }
            }
        }
    }

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
