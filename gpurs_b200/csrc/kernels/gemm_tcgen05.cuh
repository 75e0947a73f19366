// The dense GEMM of the gpurs matrix-multiply path, rebuilt for sm_100a:
//
//     C[m, n] = sum_k A[m, k] * B[n, k]          A is M x K, B is N x K, both K-major,
//
// the operand convention of the reference's tensor-core examples
// (examples/blackwell/examples/blackwell_matrix.rs:32-56, crates/gpurs/src/gpu/tensor/layout.rs:1-2).
//
// Structure (one persistent CTA, or CTA pair, per SM):
//   warp 0      producer: waits for a free stage, arms its barrier and issues the two TMA tile loads
//   warp 1      MMA issuer: waits for a full stage, issues 4 tcgen05.mma (32 bytes of K each) into one
//               of two TMEM accumulators, commits the stage back to the producer, and after the last
//               K-block commits the accumulator to the epilogue
//   warps 2..5  epilogue: tcgen05.ld the finished accumulator (warp w owns TMEM lanes 32*(w%4)..+31),
//               round to the output type, store 16 bytes per instruction; then hand the accumulator back
// so the tensor pipe never waits for a TMA round trip or for the epilogue of the previous tile.  The
// reference's kernel does all three jobs with one thread and one accumulator
// (crates/gpurs/src/gpu/tensor/hopper/ring.rs:144-209, blackwell/tensor_memory.rs:91-121,232-278).
//
// With CTA_GROUP == 2 two CTAs of a cluster share one 256 x BLOCK_N tile: each loads its own 128 rows
// of A and its own half of the B tile, and the leader (cluster rank 0) issues tcgen05.mma.cta_group::2,
// which reads B from both CTAs' shared memory and writes each CTA's 128 accumulator rows into that
// CTA's own tensor memory.  No TMA load is multicast; every CTA fetches its own operands.
#pragma once
#include "gemm_params.hpp"
#include "gemm_schedule.hpp"
#include "sm100_ptx.cuh"
#include <cuda_bf16.h>
#include <cuda_fp16.h>

namespace gemm {

// Destinations of the "push" epilogue of an M-sharded product: a descriptor of the whole gathered matrix on every GPU
// of the box (this GPU's own copy included).  Every finished box of C is stored to all of them, `row_offset` rows down,
// so that when the kernels of all ranks have finished every GPU holds the complete matrix: the all-gather that would
// follow the GEMM rides on the GEMM's own epilogue, tile by tile, as plain remote stores over NVLink.
struct PushTargets {
    CUtensorMap maps[MAX_PUSH_TARGETS];
    int count;
    int row_offset;
    int first;       // the copy a box goes to first (the rank after this one): the ranks do not all start on the same GPU
    int reserved;
};

// Instruction descriptor: accumulator format (1 = f32, 2 = s32) at bit 4, A and B element formats at
// bits 7 and 10, both operands K-major, N/8 at bit 17, M/16 at bit 24 (M counts both CTAs of a pair).
__host__ __device__ constexpr uint32_t instruction_descriptor(int accumulator_format, int element_format, int mma_m, int mma_n) {
    return (uint32_t(accumulator_format) << 4) | (uint32_t(element_format) << 7) | (uint32_t(element_format) << 10) |
           (uint32_t(mma_n >> 3) << 17) | (uint32_t(mma_m >> 4) << 24);
}

// Tile index -> (tile row, tile column): bands of `raster_rows` tile rows are walked column by column,
// the same idea as the reference's Swizzle<8> raster (crates/gpurs/src/gpu/tensor/schedule/grid.rs:55-82).
// Odd bands walk their columns backwards, so that the columns of B in L2 at the end of a band are the first
// ones the next band asks for.
__device__ __forceinline__ void tile_position(int tile, const Params &p, int &tile_m, int &tile_n) {
    int band_tiles = p.raster_rows * p.tiles_n;
    int band = tile / band_tiles;
    int first_row = band * p.raster_rows;
    int rows = min(p.raster_rows, p.tiles_m - first_row);
    int local = tile - band * band_tiles;
    tile_m = first_row + local % rows;
    tile_n = (band & 1) ? p.tiles_n - 1 - local / rows : local / rows;
}

__device__ __forceinline__ void report_status(unsigned int *status, volatile uint32_t *abort_flag, uint32_t code, int tile, int k_block) {
    *abort_flag = code;
    if (atomicCAS(status, 0u, code) == 0u) {
        status[1] = blockIdx.x;
        status[2] = uint32_t(tile);
        status[3] = uint32_t(k_block);
    }
}

__device__ __forceinline__ void report(const Params &p, volatile uint32_t *abort_flag, uint32_t code, int tile, int k_block) {
    report_status(p.status, abort_flag, code, tile, k_block);
}

// COLUMNS (16, 32 or 64) consecutive accumulator columns of this warp's 32 TMEM lanes.
template <int COLUMNS>
__device__ __forceinline__ void tmem_load_columns(uint32_t address, uint32_t (&values)[COLUMNS]) {
    if constexpr (COLUMNS == 16) ptx::tmem_load_32x16(address, values);
    else if constexpr (COLUMNS == 32) ptx::tmem_load_32x32(address, values);
    else ptx::tmem_load_32x64(address, values);
}

// One element of the residual matrix (stored in C's element type) as fp32.  Plain loads: the residual may be C itself,
// which this kernel writes (every element is read by the thread that later writes it, before it writes it).
template <int OUT>
__device__ __forceinline__ float residual_element(const Params &p, int row, int column) {
    const size_t index = size_t(row) * size_t(p.ldr) + size_t(column);
    if constexpr (OUT == OUT_BF16) return __bfloat162float(reinterpret_cast<const __nv_bfloat16 *>(p.residual)[index]);
    else if constexpr (OUT == OUT_F16) return __half2float(reinterpret_cast<const __half *>(p.residual)[index]);
    else return reinterpret_cast<const float *>(p.residual)[index];
}

// The epilogue algebra on 32 accumulator columns of one output row, starting at `column`:
// value * (alpha * row_scale[row]) * column_scale[column] + bias[column] + row_bias[row] + beta * residual[row, column],
// each part optional (float outputs only), every step rounded to fp32 on its own (no fused multiply-add), so that a host
// can reproduce the result exactly.  The reference offers the same steps on its accumulator tiles: scale, scale_rows,
// scale_columns, add_columns, add_rows and add of another tile (crates/gpurs/src/gpu/tensor/warp/accumulators.rs:82-110).
template <int OUT>
__device__ __forceinline__ void apply_epilogue(const Params &p, uint32_t (&acc)[32], int row, int column) {
    if constexpr (OUT != OUT_I32) {
        if (p.scaled_by_alpha != 0 || p.row_scale != nullptr) {
            float factor = p.scaled_by_alpha != 0 ? p.alpha : 1.0f;
            if (p.row_scale != nullptr) factor = __fmul_rn(factor, __ldg(p.row_scale + min(row, p.m - 1)));
#pragma unroll
            for (int i = 0; i < 32; i++) acc[i] = __float_as_uint(__fmul_rn(__uint_as_float(acc[i]), factor));
        }
        // the 32 values of a per-column vector are fetched as eight 16-byte loads where the chunk is whole and the vector
        // aligned (a quarter of the load instructions; the arithmetic is the same)
        const bool whole_chunk = column + 32 <= p.n;
        if (p.column_scale != nullptr) {
            if (whole_chunk && (reinterpret_cast<uintptr_t>(p.column_scale + column) & 15) == 0) {
                const float4 *vector = reinterpret_cast<const float4 *>(p.column_scale + column);
#pragma unroll
                for (int i = 0; i < 8; i++) {
                    const float4 v = __ldg(vector + i);
                    acc[4 * i] = __float_as_uint(__fmul_rn(__uint_as_float(acc[4 * i]), v.x));
                    acc[4 * i + 1] = __float_as_uint(__fmul_rn(__uint_as_float(acc[4 * i + 1]), v.y));
                    acc[4 * i + 2] = __float_as_uint(__fmul_rn(__uint_as_float(acc[4 * i + 2]), v.z));
                    acc[4 * i + 3] = __float_as_uint(__fmul_rn(__uint_as_float(acc[4 * i + 3]), v.w));
                }
            } else {
#pragma unroll
                for (int i = 0; i < 32; i++)
                    if (column + i < p.n) acc[i] = __float_as_uint(__fmul_rn(__uint_as_float(acc[i]), __ldg(p.column_scale + column + i)));
            }
        }
        if (p.bias != nullptr) {
            if (whole_chunk && (reinterpret_cast<uintptr_t>(p.bias + column) & 15) == 0) {
                const float4 *vector = reinterpret_cast<const float4 *>(p.bias + column);
#pragma unroll
                for (int i = 0; i < 8; i++) {
                    const float4 v = __ldg(vector + i);
                    acc[4 * i] = __float_as_uint(__fadd_rn(__uint_as_float(acc[4 * i]), v.x));
                    acc[4 * i + 1] = __float_as_uint(__fadd_rn(__uint_as_float(acc[4 * i + 1]), v.y));
                    acc[4 * i + 2] = __float_as_uint(__fadd_rn(__uint_as_float(acc[4 * i + 2]), v.z));
                    acc[4 * i + 3] = __float_as_uint(__fadd_rn(__uint_as_float(acc[4 * i + 3]), v.w));
                }
            } else {
#pragma unroll
                for (int i = 0; i < 32; i++)
                    if (column + i < p.n) acc[i] = __float_as_uint(__fadd_rn(__uint_as_float(acc[i]), __ldg(p.bias + column + i)));
            }
        }
        if (p.row_bias != nullptr) {
            const float addend = __ldg(p.row_bias + min(row, p.m - 1));
#pragma unroll
            for (int i = 0; i < 32; i++) acc[i] = __float_as_uint(__fadd_rn(__uint_as_float(acc[i]), addend));
        }
        if (p.residual != nullptr && row < p.m) {
            constexpr int ELEMENT_BYTES = OUT == OUT_F32 ? 4 : 2;
            const uint8_t *source = reinterpret_cast<const uint8_t *>(p.residual) + (size_t(row) * size_t(p.ldr) + size_t(column)) * ELEMENT_BYTES;
            if (whole_chunk && (reinterpret_cast<uintptr_t>(source) & 15) == 0) {
                // the row's 32 elements as 16-byte loads (plain loads: the residual may be C itself)
                const uint4 *vector = reinterpret_cast<const uint4 *>(source);
#pragma unroll
                for (int i = 0; i < 32 * ELEMENT_BYTES / 16; i++) {
                    const uint4 v = vector[i];
                    const uint32_t words[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
                    for (int j = 0; j < 4; j++) {
                        if constexpr (OUT == OUT_F32) {
                            const int e = 4 * i + j;
                            acc[e] = __float_as_uint(__fadd_rn(__uint_as_float(acc[e]), __fmul_rn(p.beta, __uint_as_float(words[j]))));
                        } else {
                            const int e = 8 * i + 2 * j;
                            float low, high;
                            if constexpr (OUT == OUT_BF16) {
                                low = __uint_as_float(words[j] << 16), high = __uint_as_float(words[j] & 0xffff0000u);
                            } else {
                                const __half2 pair = *reinterpret_cast<const __half2 *>(&words[j]);
                                low = __low2float(pair), high = __high2float(pair);
                            }
                            acc[e] = __float_as_uint(__fadd_rn(__uint_as_float(acc[e]), __fmul_rn(p.beta, low)));
                            acc[e + 1] = __float_as_uint(__fadd_rn(__uint_as_float(acc[e + 1]), __fmul_rn(p.beta, high)));
                        }
                    }
                }
            } else {
#pragma unroll
                for (int i = 0; i < 32; i++)
                    if (column + i < p.n)
                        acc[i] = __float_as_uint(__fadd_rn(__uint_as_float(acc[i]), __fmul_rn(p.beta, residual_element<OUT>(p, row, column + i))));
            }
        }
    }
}

// running + the values of this chunk's columns that exist, added in column order (`reduce_rows` with + as the operation).
__device__ __forceinline__ float fold_sum(const Params &p, const uint32_t (&acc)[32], int column, float running) {
#pragma unroll
    for (int i = 0; i < 32; i++)
        if (column + i < p.n) running = __fadd_rn(running, __uint_as_float(acc[i]));
    return running;
}

// Two fp32 accumulators rounded to nearest even and packed into one word of bf16 or f16.
template <int OUT>
__device__ __forceinline__ uint32_t pack_pair(uint32_t low, uint32_t high) {
    if constexpr (OUT == OUT_BF16) {
        __nv_bfloat162 v = __floats2bfloat162_rn(__uint_as_float(low), __uint_as_float(high));
        return *reinterpret_cast<uint32_t *>(&v);
    } else {
        __half2 v = __floats2half2_rn(__uint_as_float(low), __uint_as_float(high));
        return *reinterpret_cast<uint32_t *>(&v);
    }
}

// max(running, |acc[i]|) over the columns of this chunk that exist (`reduce_rows` of the reference's accumulator tiles,
// crates/gpurs/src/gpu/tensor/warp/accumulators.rs:112-128, with max |.| as the operation).
__device__ __forceinline__ float fold_absmax(const Params &p, const uint32_t (&acc)[32], int column, float running) {
#pragma unroll
    for (int i = 0; i < 32; i++)
        if (column + i < p.n) running = fmaxf(running, fabsf(__uint_as_float(acc[i])));
    return running;
}

template <int OUT, bool APPLY = true, bool ATOMIC = true>
__device__ __forceinline__ void store_chunk(const Params &p, const uint32_t (&source)[32], int row, int column, long long element_offset = 0) {
    if (row >= p.m || column >= p.n) return;
    const bool whole = column + 32 <= p.n && p.vector_stores;
    uint32_t acc[32];
#pragma unroll
    for (int i = 0; i < 32; i++) acc[i] = source[i];
    if constexpr (APPLY) apply_epilogue<OUT>(p, acc, row, column);
    if constexpr (OUT == OUT_F32 || OUT == OUT_I32) {
        uint32_t *out = reinterpret_cast<uint32_t *>(p.c) + element_offset + size_t(row) * p.ldc + column;
        if constexpr (OUT == OUT_F32 && ATOMIC) {
            if (p.accumulate != 0) {
                // `accumulate` of the reference's f32 output matrix (crates/gpurs/src/gpu/tensor/output/reduction.rs:157-202):
                // one atomic add per element, so that any number of products may add into the same C at once
#pragma unroll
                for (int i = 0; i < 32; i++)
                    if (column + i < p.n) atomicAdd(reinterpret_cast<float *>(out) + i, __uint_as_float(acc[i]));
                return;
            }
        }
        if (whole) {
#pragma unroll
            for (int i = 0; i < 8; i++)
                reinterpret_cast<uint4 *>(out)[i] = make_uint4(acc[4 * i], acc[4 * i + 1], acc[4 * i + 2], acc[4 * i + 3]);
        } else {
#pragma unroll
            for (int i = 0; i < 32; i++)
                if (column + i < p.n) out[i] = acc[i];
        }
    } else {
        uint32_t packed[16];
#pragma unroll
        for (int i = 0; i < 16; i++) {
            float lo = __uint_as_float(acc[2 * i]), hi = __uint_as_float(acc[2 * i + 1]);
            if constexpr (OUT == OUT_BF16) {
                __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
                packed[i] = *reinterpret_cast<uint32_t *>(&v);
            } else {
                __half2 v = __floats2half2_rn(lo, hi);
                packed[i] = *reinterpret_cast<uint32_t *>(&v);
            }
        }
        uint16_t *out = reinterpret_cast<uint16_t *>(p.c) + element_offset + size_t(row) * p.ldc + column;
        if (whole) {
#pragma unroll
            for (int i = 0; i < 4; i++)
                reinterpret_cast<uint4 *>(out)[i] = make_uint4(packed[4 * i], packed[4 * i + 1], packed[4 * i + 2], packed[4 * i + 3]);
        } else {
#pragma unroll
            for (int i = 0; i < 32; i++)
                if (column + i < p.n) out[i] = uint16_t(packed[i / 2] >> (16 * (i & 1)));
        }
    }
}

// One piece of work of a CTA group: K-blocks [kb_begin, kb_end) of a tile.  split_tile >= 0 marks a tile of the split round
// that `contributors` groups share; this group is number `contributor` of them.
struct WorkItem {
    int tile, kb_begin, kb_end;
    int split_tile, contributor, contributors;
};

// Walks the work of one CTA group in order: with STREAMK first its share of the K-blocks of the split round (first, so that
// adding the parts up overlaps the whole tiles that follow instead of ending the kernel), then its whole tiles (tile =
// group, group + groups, ...).  All three roles of a CTA walk the same sequence.
template <bool STREAMK>
struct WorkWalker {
    StreamSchedule schedule;
    int group, groups, next_tile, whole_tiles;
    long long unit, unit_end;

    __device__ __forceinline__ WorkWalker(int tile_count, int k_blocks, int group_, int groups_, int split_tiles) : group(group_), groups(groups_), next_tile(group_) {
        schedule.k_blocks = k_blocks;
        whole_tiles = tile_count;
        unit = unit_end = 0;
        if constexpr (STREAMK) {
            schedule = make_stream_schedule(tile_count, k_blocks, groups_, split_tiles);
            whole_tiles = schedule.whole_tiles;
            if (schedule.split_tiles > 0 && group_ < schedule.clusters) {
                unit = schedule.first_unit(group_);
                unit_end = schedule.first_unit(group_ + 1);
            }
        }
    }

    __device__ __forceinline__ bool next(WorkItem &item) {
        if constexpr (STREAMK) {
            if (unit < unit_end) {
                const int r = int(unit / schedule.k_blocks);
                item.tile = whole_tiles + r;
                item.kb_begin = int(unit - (long long)r * schedule.k_blocks);
                const long long take = min((long long)(schedule.k_blocks - item.kb_begin), unit_end - unit);
                item.kb_end = item.kb_begin + int(take);
                item.contributors = schedule.contributors(r);
                item.contributor = group - schedule.first_contributor(r);
                item.split_tile = item.contributors > 1 ? r : -1;
                unit += take;
                return true;
            }
        }
        if (next_tile < whole_tiles) {
            item.tile = next_tile, item.kb_begin = 0, item.kb_end = schedule.k_blocks;
            item.split_tile = -1, item.contributor = 0, item.contributors = 1;
            next_tile += groups;
            return true;
        }
        return false;
    }
};

// KIND: ptx::KIND_*; ELEMENT_FORMAT: the 3-bit format code of the operands for that kind;
// ACC_FORMAT: 1 = f32, 2 = s32; OUT: OUT_*.
// PUSH: the epilogue stores every box to all GPUs' copies (PushTargets).  BATCHED: the operands and the output are batches
// of matrices described by rank-3 tensor maps (z = batch); tiles are numbered batch by batch.
// STREAMK: the tiles of the last, partial round are split along K over all CTA groups (gemm_schedule.hpp).
// ALGEBRA: the epilogue applies the optional output algebra and row reductions of Params.  The entries without it are
// the ones a plain product runs: their epilogue is load, round, stage, store, and nothing else is compiled in.
template <int KIND, int ELEMENT_FORMAT, int ACC_FORMAT, int OUT, int BLOCK_N, int CTA_GROUP, int STAGES, bool PUSH = false, bool BATCHED = false,
          bool STREAMK = false, bool ALGEBRA = true>
__device__ __forceinline__ void gemm_body(const CUtensorMap *map_a, const CUtensorMap *map_b, const CUtensorMap *map_c, const Params &p,
                                          const PushTargets *targets = nullptr) {
    using L = SharedLayout<BLOCK_N, CTA_GROUP, STAGES>;
    static_assert(BLOCK_N == 128 || BLOCK_N == 256, "two accumulators of BLOCK_N columns must fit 512 TMEM columns");
    constexpr uint32_t TMEM_COLUMNS = 2 * BLOCK_N;
    constexpr uint32_t IDESC = instruction_descriptor(ACC_FORMAT, ELEMENT_FORMAT, BLOCK_M * CTA_GROUP, BLOCK_N);

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
    const uint32_t staging = base + L::STAGING_OFFSET;

    const int warp = threadIdx.x / 32;
    const uint32_t lane = ptx::lane_id();
    const uint32_t cta_rank = CTA_GROUP == 2 ? ptx::cluster_cta_rank() : 0u;
    const bool leader = cta_rank == 0;
    const int cluster_id = blockIdx.x / CTA_GROUP;
    const int cluster_count = gridDim.x / CTA_GROUP;
    const int tiles_per_matrix = p.tiles_m * p.tiles_n;
    const int tile_count = BATCHED ? tiles_per_matrix * max(p.batches, 1) : tiles_per_matrix;
    const int element_bytes = KIND == ptx::KIND_F16 ? 2 : (KIND == ptx::KIND_TF32 ? 4 : 1);
    const int block_k = ROW_BYTES / element_bytes;
    const int k_blocks = (p.k + block_k - 1) / block_k;
    // K x N storage of B: one TMA box is 128 bytes of N (n_per_box elements) by block_k rows of K.
    const int n_per_box = ROW_BYTES / element_bytes;
    const uint32_t box_bytes = uint32_t(block_k) * ROW_BYTES;

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
    }
    if (warp == 1) {
        ptx::tmem_alloc<CTA_GROUP>(ptx::smem_u32(const_cast<uint32_t *>(tmem_slot)), TMEM_COLUMNS);
        ptx::tmem_relinquish<CTA_GROUP>();
    }
    ptx::tcgen05_fence_before();
    __syncthreads();
    if constexpr (CTA_GROUP == 2) {
        // The peer's TMA loads and the leader's commits signal barriers of this CTA: both CTAs must
        // have initialised theirs before either starts.
        ptx::cluster_arrive();
        ptx::cluster_wait();
    }
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
            // L2 residency: the operand whose panel is shared by the tiles of successive waves can be asked to
            // stay (evict last) while the other streams through (evict first).
            const bool hinted = p.l2_policy != 0;
            const uint64_t policy_a = (p.l2_policy == 1 || p.l2_policy == 3) ? ptx::l2_policy_evict_last() : ptx::l2_policy_evict_first();
            const uint64_t policy_b = (p.l2_policy == 2 || p.l2_policy == 3) ? ptx::l2_policy_evict_last() : ptx::l2_policy_evict_first();
            WorkWalker<STREAMK> walker(tile_count, k_blocks, cluster_id, cluster_count, p.split_tiles);
            WorkItem item;
            while (ok && walker.next(item)) {
                const int tile = item.tile;
                int tile_m, tile_n;
                const int batch = BATCHED ? tile / tiles_per_matrix : 0;
                tile_position(tile - batch * tiles_per_matrix, p, tile_m, tile_n);
                const int row_a = (tile_m * CTA_GROUP + int(cta_rank)) * BLOCK_M;
                const int row_b = tile_n * BLOCK_N + int(cta_rank) * L::B_ROWS;
                for (int kb = item.kb_begin; kb < item.kb_end; kb++) {
                    if (!ptx::mbarrier_wait(empty_bar(stage), phase ^ 1, abort_flag)) {
                        report(p, abort_flag, STATUS_PRODUCER_TIMEOUT, tile, kb);
                        ok = false;
                        break;
                    }
                    if constexpr (BATCHED) {
                        if constexpr (CTA_GROUP == 1) {
                            ptx::mbarrier_arrive_expect_tx(full_bar(stage), L::STAGE_BYTES);
                            ptx::tma_load_3d(stage_a(stage), map_a, kb * block_k, row_a, batch, full_bar(stage));
                            ptx::tma_load_3d(stage_b(stage), map_b, kb * block_k, row_b, batch, full_bar(stage));
                        } else {
                            if (leader) ptx::mbarrier_arrive_expect_tx(full_bar(stage), 2 * L::STAGE_BYTES);
                            const uint32_t leader_bar = ptx::map_to_cta(full_bar(stage), 0);
                            ptx::tma_load_3d_pair(stage_a(stage), map_a, kb * block_k, row_a, batch, leader_bar);
                            ptx::tma_load_3d_pair(stage_b(stage), map_b, kb * block_k, row_b, batch, leader_bar);
                        }
                    } else if constexpr (CTA_GROUP == 1) {
                        ptx::mbarrier_arrive_expect_tx(full_bar(stage), L::STAGE_BYTES);
                        if (hinted) {
                            ptx::tma_load_2d_hint(stage_a(stage), map_a, kb * block_k, row_a, full_bar(stage), policy_a);
                            ptx::tma_load_2d_hint(stage_b(stage), map_b, kb * block_k, row_b, full_bar(stage), policy_b);
                        } else if (p.b_row_major) {
                            ptx::tma_load_2d(stage_a(stage), map_a, kb * block_k, row_a, full_bar(stage));
                            // K x N storage: boxes of 128 bytes of N by block_k rows of K, side by side
                            for (int i = 0; i < L::B_ROWS / n_per_box; i++)
                                ptx::tma_load_2d(stage_b(stage) + uint32_t(i) * box_bytes, map_b, row_b + i * n_per_box, kb * block_k, full_bar(stage));
                        } else {
                            ptx::tma_load_2d(stage_a(stage), map_a, kb * block_k, row_a, full_bar(stage));
                            ptx::tma_load_2d(stage_b(stage), map_b, kb * block_k, row_b, full_bar(stage));
                        }
                    } else {
                        // Both CTAs' loads are counted on the leader's barrier, which the leader arms
                        // for the bytes of the pair.
                        if (leader) ptx::mbarrier_arrive_expect_tx(full_bar(stage), 2 * L::STAGE_BYTES);
                        const uint32_t leader_bar = ptx::map_to_cta(full_bar(stage), 0);
                        if (hinted) {
                            ptx::tma_load_2d_pair_hint(stage_a(stage), map_a, kb * block_k, row_a, leader_bar, policy_a);
                            ptx::tma_load_2d_pair_hint(stage_b(stage), map_b, kb * block_k, row_b, leader_bar, policy_b);
                        } else if (p.b_row_major) {
                            ptx::tma_load_2d_pair(stage_a(stage), map_a, kb * block_k, row_a, leader_bar);
                            for (int i = 0; i < L::B_ROWS / n_per_box; i++)
                                ptx::tma_load_2d_pair(stage_b(stage) + uint32_t(i) * box_bytes, map_b, row_b + i * n_per_box, kb * block_k, leader_bar);
                        } else {
                            ptx::tma_load_2d_pair(stage_a(stage), map_a, kb * block_k, row_a, leader_bar);
                            ptx::tma_load_2d_pair(stage_b(stage), map_b, kb * block_k, row_b, leader_bar);
                        }
                    }
                    if (++stage == STAGES) { stage = 0; phase ^= 1; }
                }
            }
            // Before leaving, see every stage released once more, so that no commit can arrive on a
            // barrier of a CTA that has already exited.
            for (int s = 0; s < STAGES && ok; s++) {
                ok = ptx::mbarrier_wait(empty_bar(stage), phase ^ 1, abort_flag);
                if (++stage == STAGES) { stage = 0; phase ^= 1; }
            }
        }
    } else if (warp == 1) {
        // ------------------------------------------------------------------ MMA issuer
        if (lane == 0 && leader) {
            int stage = 0;
            uint32_t phase = 0;
            int acc = 0;
            uint32_t acc_phase = 0;
            bool ok = true;
            WorkWalker<STREAMK> walker(tile_count, k_blocks, cluster_id, cluster_count, p.split_tiles);
            WorkItem item;
            // Everything that does not change from stage to stage is computed here, once.  (Releasing the stages in pairs with one
            // commit per two K-blocks was measured on bf16 8192^3 and changed nothing: this kernel is not bound by its issuing thread.)
            // B as N x K: K-major like A, 32 bytes of K per instruction inside the swizzle span.  B as K x N: N-major
            // (bit 16 of the instruction descriptor), an instruction's K is MMA_K rows of 128 bytes.
            const uint64_t a_desc0 = ptx::smem_descriptor_k_major_sw128(stage_a(0));
            const uint64_t b_desc0 = p.b_row_major ? ptx::smem_descriptor_mn_major_sw128(stage_b(0), box_bytes) : ptx::smem_descriptor_k_major_sw128(stage_b(0));
            const uint64_t b_step = p.b_row_major ? uint64_t(((MMA_K_BYTES / element_bytes) * ROW_BYTES) >> 4) : uint64_t(MMA_K_BYTES >> 4);
            const uint32_t idesc = p.b_row_major ? (IDESC | (1u << 16)) : IDESC;
            constexpr uint64_t STAGE_STEP = uint64_t(L::STAGE_BYTES >> 4);        // one stage further, in descriptor address units
            while (ok && walker.next(item)) {
                const int tile = item.tile;
                if (!ptx::mbarrier_wait<CTA_GROUP == 2>(acc_empty_bar(acc), acc_phase ^ 1, abort_flag)) {
                    report(p, abort_flag, STATUS_MMA_TIMEOUT, tile, -1);
                    break;
                }
                ptx::tcgen05_fence_after();
                const uint32_t d_tmem = tmem_base + uint32_t(acc) * BLOCK_N;
                for (int kb = item.kb_begin; kb < item.kb_end; kb++) {
                    if (!ptx::mbarrier_wait(full_bar(stage), phase, abort_flag)) {
                        report(p, abort_flag, STATUS_MMA_TIMEOUT, tile, kb);
                        ok = false;
                        break;
                    }
                    ptx::tcgen05_fence_after();
                    const uint64_t a_desc = a_desc0 + uint64_t(stage) * STAGE_STEP, b_desc = b_desc0 + uint64_t(stage) * STAGE_STEP;
                    // advancing A's start address by 32 bytes steps through K inside the swizzle span
                    ptx::tcgen05_mma<KIND, CTA_GROUP>(d_tmem, a_desc, b_desc, idesc, uint32_t(kb != item.kb_begin));
#pragma unroll
                    for (int j = 1; j < ROW_BYTES / MMA_K_BYTES; j++)
                        ptx::tcgen05_mma_accumulate<KIND, CTA_GROUP>(d_tmem, a_desc + uint64_t(j * (MMA_K_BYTES >> 4)), b_desc + uint64_t(j) * b_step, idesc);
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
        const int quadrant = warp % 4;   // the TMEM lanes this warp may read
        int acc = 0;
        uint32_t acc_phase = 0;
        int stores = 0;                  // TMA stores issued by this warp: picks the staging buffer
        WorkWalker<STREAMK> walker(tile_count, k_blocks, cluster_id, cluster_count, p.split_tiles);
        WorkItem item;
        while (walker.next(item)) {
            const int tile = item.tile;
            int tile_m, tile_n;
            const int batch = BATCHED ? tile / tiles_per_matrix : 0;
            tile_position(tile - batch * tiles_per_matrix, p, tile_m, tile_n);
            // Every lane waits (each needs the barrier's acquire); the vote keeps the warp together
            // for the warp-wide tcgen05.ld that follows.
            const bool ready = ptx::mbarrier_wait(acc_full_bar(acc), acc_phase, abort_flag);
            if (!__all_sync(0xffffffffu, ready)) {
                if (lane == 0) report(p, abort_flag, STATUS_EPILOGUE_TIMEOUT, tile, -1);
                break;
            }
            ptx::tcgen05_fence_after();
            const int row = (tile_m * CTA_GROUP + int(cta_rank)) * BLOCK_M + quadrant * 32 + int(lane);
            const uint32_t lane_base = tmem_base + (uint32_t(quadrant * 32) << 16) + uint32_t(acc) * BLOCK_N;
            const bool reduce = ALGEBRA && OUT != OUT_I32 && p.row_absmax != nullptr;
            const bool summing = ALGEBRA && OUT != OUT_I32 && p.row_sum != nullptr;
            float row_max = 0.0f, row_total = 0.0f;
            const bool shared_tile = STREAMK && item.split_tile >= 0;
            // A tile of the split round holds only this group's K-blocks: its 32-bit sums go to scratch as they are.
            constexpr int TILE_ROWS = BLOCK_M * CTA_GROUP;
            const int row_in_tile = int(cta_rank) * BLOCK_M + quadrant * 32 + int(lane);
            if (shared_tile) {
                // one part = [BLOCK_N / 4 groups of four columns][TILE_ROWS rows] of 16 bytes: the 32 lanes (rows) of a
                // warp write, and later read, 512 contiguous bytes per instruction
                uint4 *mine = reinterpret_cast<uint4 *>(p.partials) +
                              (size_t(item.split_tile) * p.max_contributors + item.contributor) * (TILE_ROWS * BLOCK_N / 4) + row_in_tile;
#pragma unroll 1
                for (int chunk = 0; chunk < BLOCK_N / 32; chunk++) {
                    uint32_t values[32];
                    ptx::tmem_load_32x32(lane_base + uint32_t(chunk * 32), values);
                    ptx::tmem_load_wait();
#pragma unroll
                    for (int i = 0; i < 8; i++)
                        mine[size_t(chunk * 8 + i) * TILE_ROWS] = make_uint4(values[4 * i], values[4 * i + 1], values[4 * i + 2], values[4 * i + 3]);
                }
            } else if (p.vector_stores == 1) {
                // Coalesced path: every 128 bytes of 32 output rows are staged in shared memory (128-byte swizzle, so
                // the 32 lanes writing their rows do not collide on banks) and written by one TMA store, which also
                // clips the box at the edges of C.  Two staging buffers per warp: the next box is filled while the
                // previous store still reads its buffer.
                constexpr int COLUMNS_PER_BOX = (OUT == OUT_F32 || OUT == OUT_I32) ? 32 : 64;
                const int warp_row = (tile_m * CTA_GROUP + int(cta_rank)) * BLOCK_M + quadrant * 32;
                // the read of box b + 1 is in flight while box b is staged and stored
                constexpr int BOXES = BLOCK_N / COLUMNS_PER_BOX;
                uint32_t low[32], high[32];
                ptx::tmem_load_32x32(lane_base, low);
                if constexpr (COLUMNS_PER_BOX == 64) ptx::tmem_load_32x32(lane_base + 32, high);
#pragma unroll 1
                for (int box = 0; box < BOXES; box++) {
                    const int column = tile_n * BLOCK_N + box * COLUMNS_PER_BOX;
                    uint32_t packed[32];
                    ptx::tmem_load_wait();
                    if constexpr (COLUMNS_PER_BOX == 32) {
                        if constexpr (ALGEBRA) apply_epilogue<OUT>(p, low, row, column);
                        if (reduce) row_max = fold_absmax(p, low, column, row_max);
                        if (summing) row_total = fold_sum(p, low, column, row_total);
#pragma unroll
                        for (int i = 0; i < 32; i++) packed[i] = low[i];
                        if (box + 1 < BOXES) ptx::tmem_load_32x32(lane_base + uint32_t((box + 1) * 32), low);
                    } else {
                        if constexpr (ALGEBRA) {
                            apply_epilogue<OUT>(p, low, row, column);
                            apply_epilogue<OUT>(p, high, row, column + 32);
                        }
                        if (reduce) row_max = fold_absmax(p, high, column + 32, fold_absmax(p, low, column, row_max));
                        if (summing) row_total = fold_sum(p, high, column + 32, fold_sum(p, low, column, row_total));
#pragma unroll
                        for (int i = 0; i < 16; i++) {
                            packed[i] = pack_pair<OUT>(low[2 * i], low[2 * i + 1]);
                            packed[16 + i] = pack_pair<OUT>(high[2 * i], high[2 * i + 1]);
                        }
                        if (box + 1 < BOXES) {
                            ptx::tmem_load_32x32(lane_base + uint32_t((box + 1) * 64), low);
                            ptx::tmem_load_32x32(lane_base + uint32_t((box + 1) * 64 + 32), high);
                        }
                    }
                    if (warp_row < p.m && column < p.n) {    // warp-uniform: boxes wholly outside C are skipped
                        const uint32_t buffer = staging + uint32_t(((warp - 2) * 2 + (stores & 1)) * 32 * ROW_BYTES);
                        stores++;
                        if (lane == 0) ptx::tma_store_wait_read<1>();       // the store that used this buffer two boxes ago
                        __syncwarp();
#pragma unroll
                        for (int j = 0; j < 8; j++)                          // lane = row; 16-byte piece j goes to slot j ^ (row % 8)
                            ptx::store_shared_v4(buffer + lane * ROW_BYTES + uint32_t((j ^ int(lane & 7)) * 16), packed[4 * j], packed[4 * j + 1],
                                                 packed[4 * j + 2], packed[4 * j + 3]);
                        ptx::fence_async_shared();
                        __syncwarp();
                        if (lane == 0) {
                            if constexpr (PUSH) {
                                // one staged box, one store per GPU of the box (remote ones travel over NVLink)
                                for (int t = 0; t < targets->count; t++) {
                                    const int target = targets->first + t < targets->count ? targets->first + t : targets->first + t - targets->count;
                                    ptx::tma_store_2d(&targets->maps[target], column, targets->row_offset + warp_row, buffer);
                                }
                            } else if constexpr (BATCHED) {
                                ptx::tma_store_3d(map_c, column, warp_row, batch, buffer);
                            } else if (ALGEBRA && OUT == OUT_F32 && p.accumulate != 0) {
                                // the staged box is added to C by the TMA unit (element-wise atomic f32 adds)
                                ptx::tma_reduce_add_2d(map_c, column, warp_row, buffer);
                            } else {
                                ptx::tma_store_2d(map_c, column, warp_row, buffer);
                            }
                            ptx::tma_store_commit();
                        }
                    }
                }
            } else {
#pragma unroll 1
                for (int chunk = 0; chunk < BLOCK_N / 32; chunk++) {
                    uint32_t values[32];
                    ptx::tmem_load_32x32(lane_base + uint32_t(chunk * 32), values);
                    ptx::tmem_load_wait();
                    if constexpr (ALGEBRA) apply_epilogue<OUT>(p, values, row, tile_n * BLOCK_N + chunk * 32);
                    if (reduce) row_max = fold_absmax(p, values, tile_n * BLOCK_N + chunk * 32, row_max);
                    if (summing) row_total = fold_sum(p, values, tile_n * BLOCK_N + chunk * 32, row_total);
                    store_chunk<OUT, false, ALGEBRA>(p, values, row, tile_n * BLOCK_N + chunk * 32, BATCHED ? batch * p.batch_stride_c : 0ll);
                }
            }
            // non-negative floats order like their bit patterns, so an unsigned atomic max folds the tile's part in
            if (reduce && row < p.m) atomicMax(reinterpret_cast<unsigned int *>(p.row_absmax) + row, __float_as_uint(row_max));
            if (summing && row < p.m && !shared_tile) atomicAdd(p.row_sum + row, row_total);
            ptx::tcgen05_fence_before();
            __syncwarp();
            if (lane == 0) {
                // The accumulator has been read out (tcgen05.wait::ld returned): nothing is published through ordinary memory, so
                // the hand-back needs no release, which at cluster scope would first wait for every store this thread has in flight.
                if (CTA_GROUP == 1 || leader) ptx::mbarrier_arrive(acc_empty_bar(acc));
                else ptx::mbarrier_arrive_cluster_relaxed(ptx::map_to_cta(acc_empty_bar(acc), 0));
            }
            if (++acc == 2) { acc = 0; acc_phase ^= 1; }
            if constexpr (STREAMK) {
                if (shared_tile) {
                    // Whoever brings the last part of these 32 rows adds the parts up, in the contributors' order (so the
                    // sum does not depend on who was last), and finishes the rows.  Nobody waits for anybody.
                    unsigned int *counter = p.split_counters + item.split_tile * (4 * CTA_GROUP) + int(cta_rank) * 4 + quadrant;
                    __threadfence();
                    __syncwarp();
                    unsigned int earlier = 0;
                    if (lane == 0) earlier = atomicAdd(counter, 1u);
                    earlier = __shfl_sync(0xffffffffu, earlier, 0);
                    if (earlier == unsigned(item.contributors - 1)) {
                        __threadfence();
                        if (lane == 0) *counter = 0;       // ready for the next launch
                        const uint4 *parts = reinterpret_cast<const uint4 *>(p.partials) +
                                             size_t(item.split_tile) * p.max_contributors * (TILE_ROWS * BLOCK_N / 4) + row_in_tile;
                        constexpr size_t PART = size_t(TILE_ROWS) * BLOCK_N / 4;      // one part, in 16-byte units
#pragma unroll 1
                        for (int chunk = 0; chunk < BLOCK_N / 32; chunk++) {
                            uint32_t sum[32];
#pragma unroll
                            for (int i = 0; i < 32; i++) sum[i] = 0;    // +0.0f / 0: the first part is added to it exactly
                            // four parts' loads in flight at a time, added in the contributors' order
                            for (int first = 0; first < item.contributors; first += 4) {
                                uint4 loaded[4][8];
#pragma unroll
                                for (int q = 0; q < 4; q++)
                                    if (first + q < item.contributors) {
#pragma unroll
                                        for (int i = 0; i < 8; i++) loaded[q][i] = __ldcg(parts + size_t(first + q) * PART + size_t(chunk * 8 + i) * TILE_ROWS);
                                    }
#pragma unroll
                                for (int q = 0; q < 4; q++)
                                    if (first + q < item.contributors) {
#pragma unroll
                                        for (int i = 0; i < 8; i++) {
                                            const uint32_t w[4] = {loaded[q][i].x, loaded[q][i].y, loaded[q][i].z, loaded[q][i].w};
#pragma unroll
                                            for (int j = 0; j < 4; j++) {
                                                if constexpr (ACC_FORMAT == 2) sum[4 * i + j] += w[j];      // s32 sums wrap like the tensor core's
                                                else sum[4 * i + j] = __float_as_uint(__fadd_rn(__uint_as_float(sum[4 * i + j]), __uint_as_float(w[j])));
                                            }
                                        }
                                    }
                            }
                            const int column = tile_n * BLOCK_N + chunk * 32;
                            if constexpr (ALGEBRA) apply_epilogue<OUT>(p, sum, row, column);
                            if (reduce) row_max = fold_absmax(p, sum, column, row_max);
                            if (summing) row_total = fold_sum(p, sum, column, row_total);
                            store_chunk<OUT, false, ALGEBRA>(p, sum, row, column);
                        }
                        if (reduce && row < p.m) atomicMax(reinterpret_cast<unsigned int *>(p.row_absmax) + row, __float_as_uint(row_max));
                        if (summing && row < p.m) atomicAdd(p.row_sum + row, row_total);
                    }
                }
            }
        }
        if (lane == 0) {
            // PUSH: the stores travel to other GPUs, and the kernel's completion is what tells the host they have been performed.
            // Otherwise it is enough that the stores have read their shared-memory source before the block exits: the grid's
            // completion orders their writes before whatever follows on the stream.
            if constexpr (PUSH) ptx::tma_store_wait<0>();
            else ptx::tma_store_wait_read<0>();
        }
    }

    // ---------------------------------------------------------------------- teardown
    __syncwarp();
    ptx::tcgen05_fence_before();
    __syncthreads();
    if (*abort_flag != 0 && threadIdx.x == 0) {
        // A wait gave up: give copies that may still be in flight a bounded time to land before the
        // shared memory they target is released.
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
