// TEST INFRASTRUCTURE ONLY: a CUDA restatement of the DESIGN of the reference's own sm_100a matrix-multiply kernel, so that
// the product's kernels can be timed beside it on the same GPU.  The reference (1jmdev/gpurs) is Rust compiled to PTX by its
// own toolchain, which is not available where this is built; this file is not its binary and not a translation of its
// code generator's output, only the same schedule written in CUDA:
//
//   examples/blackwell/examples/blackwell_matrix.rs:32-56   one CTA of 128 threads per 128 x 256 output tile (grid = tiles,
//                                                           tile rows walked in groups of eight, schedule/grid.rs:55-82),
//                                                           K in steps of 64, a four-stage ring, one 256-column accumulator
//   crates/gpurs/src/gpu/tensor/hopper/ring.rs:144-209      per step, thread 0: commit the previous step's stage to its
//                                                           `empty` barrier, all threads wait for this step's `full` barrier,
//                                                           thread 0 waits for the stage it just committed to be released
//                                                           (that is: for the previous step's products to finish), refills it
//                                                           by TMA, then issues this step's four tcgen05.mma
//   blackwell/tensor_memory.rs:91-121                       the four products of K = 16, accumulate flag off for the first
//   blackwell/tensor_memory.rs:232-278, output/direct.rs:59-88   epilogue: commit and wait, then every warp reads its 32 lanes
//                                                           in two halves of 16 with tcgen05.ld.16x256b.x8 (64 columns a call)
//                                                           and writes pairs of fp32 with bounds-checked 8-byte stores
//
// Differences, all deliberate: every wait is bounded (the reference's spin without limit, hopper/intrinsics.rs:15-16) and on
// expiry the block records a status word and leaves; descriptors arrive by value.  Nothing in the shipped library uses this.
#include "../gpurs_b200/csrc/kernels/sm100_ptx.cuh"

namespace {

constexpr int TILE_ROWS = 128, TILE_COLUMNS = 256, DEPTH = 64, STAGES = 4, THREADS = 128;
constexpr int A_BYTES = TILE_ROWS * DEPTH * 2, B_BYTES = TILE_COLUMNS * DEPTH * 2, STAGE_BYTES = A_BYTES + B_BYTES;

__device__ __forceinline__ void load_16x256b_x8(uint32_t address, uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.16x256b.x8.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
          "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
          "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
          "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(address)
        : "memory");
}

}  // namespace

extern "C" __global__ void __launch_bounds__(THREADS, 1)
gpurs_reference_design_f16_f32(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b, float *output, int m, int n,
                               int k, unsigned int *status) {
    extern __shared__ uint8_t raw_shared[];
    const uint32_t base = (ptx::smem_u32(raw_shared) + 1023u) & ~1023u;
    uint8_t *aligned = raw_shared + (base - ptx::smem_u32(raw_shared));
    const uint32_t barriers = base + STAGES * STAGE_BYTES;
    auto full = [&](uint32_t i) { return barriers + (i % STAGES) * 8; };
    auto empty = [&](uint32_t i) { return barriers + (STAGES + i % STAGES) * 8; };
    const uint32_t done = barriers + 2 * STAGES * 8;
    volatile uint32_t *tmem_slot = reinterpret_cast<volatile uint32_t *>(aligned + STAGES * STAGE_BYTES + (2 * STAGES + 1) * 8);
    volatile uint32_t *abort_flag = tmem_slot + 1;

    // blockIdx.x -> tile: groups of eight tile rows walked column by column
    const int tiles_m = (m + TILE_ROWS - 1) / TILE_ROWS, tiles_n = (n + TILE_COLUMNS - 1) / TILE_COLUMNS;
    const int group_tiles = 8 * tiles_n, group = blockIdx.x / group_tiles, first_row = group * 8, rows = min(8, tiles_m - first_row);
    const int local = blockIdx.x - group * group_tiles;
    const int tile_m = first_row + local % rows, tile_n = local / rows;
    const int steps = (k + DEPTH - 1) / DEPTH;
    const int warp = threadIdx.x / 32;
    const uint32_t lane = ptx::lane_id();

    if (threadIdx.x == 0) {
        *abort_flag = 0;
        for (int s = 0; s < STAGES; s++) {
            ptx::mbarrier_init(full(s), 1);
            ptx::mbarrier_init(empty(s), 1);
        }
        ptx::mbarrier_init(done, 1);
        ptx::fence_mbarrier_init();
    }
    if (warp == 0) {
        ptx::tmem_alloc<1>(ptx::smem_u32(const_cast<uint32_t *>(tmem_slot)), TILE_COLUMNS);
        ptx::tmem_relinquish<1>();
    }
    ptx::tcgen05_fence_before();
    __syncthreads();
    ptx::tcgen05_fence_after();
    const uint32_t tmem = *tmem_slot;
    constexpr uint32_t IDESC = (1u << 4) | (uint32_t(TILE_COLUMNS >> 3) << 17) | (8u << 24);      // f32 accumulate, f16 operands, 128 x 256

    auto fill = [&](uint32_t index) {        // thread 0: one stage's two tile copies
        const uint32_t stage = base + (index % STAGES) * STAGE_BYTES;
        ptx::mbarrier_arrive_expect_tx(full(index), STAGE_BYTES);
        ptx::tma_load_2d(stage, &map_a, int(index) * DEPTH, tile_m * TILE_ROWS, full(index));
        ptx::tma_load_2d(stage + A_BYTES, &map_b, int(index) * DEPTH, tile_n * TILE_COLUMNS, full(index));
    };
    uint32_t filled = 0;
    if (threadIdx.x == 0)
        for (; filled < uint32_t(min(STAGES - 1, steps)); filled++) fill(filled);

    for (int step = 0; step < steps; step++) {
        if (threadIdx.x == 0 && step > 0) ptx::tcgen05_commit(empty(uint32_t(step - 1)));      // released when the previous step's products finish
        // every thread waits for this step's tiles, as the reference's ring has all 128 threads do
        if (!ptx::mbarrier_wait(full(uint32_t(step)), (uint32_t(step) / STAGES) & 1, abort_flag)) {
            if (atomicCAS(status, 0u, 101u) == 0u) status[1] = blockIdx.x, status[2] = uint32_t(step);
            *abort_flag = 1;
        }
        if (*abort_flag) break;
        if (threadIdx.x == 0) {
            const uint32_t next = uint32_t(step) + STAGES - 1;
            if (next < uint32_t(steps)) {
                // the stage to refill is the one just committed: wait for the previous step's products before issuing this step's
                if (next >= STAGES && !ptx::mbarrier_wait(empty(next), (next / STAGES - 1) & 1, abort_flag)) {
                    if (atomicCAS(status, 0u, 102u) == 0u) status[1] = blockIdx.x, status[2] = uint32_t(step);
                    *abort_flag = 1;
                } else {
                    fill(next);
                }
            }
            ptx::tcgen05_fence_after();
            const uint32_t stage = base + (uint32_t(step) % STAGES) * STAGE_BYTES;
            const uint64_t a_desc = ptx::smem_descriptor_k_major_sw128(stage), b_desc = ptx::smem_descriptor_k_major_sw128(stage + A_BYTES);
            for (int depth = 0; depth < 4; depth++)
                ptx::tcgen05_mma<ptx::KIND_F16, 1>(tmem, a_desc + uint64_t(depth * 2), b_desc + uint64_t(depth * 2), IDESC, uint32_t(step > 0 || depth > 0));
        }
        __syncwarp();
    }
    // complete: commit everything issued and wait for it
    if (threadIdx.x == 0) ptx::tcgen05_commit(done);
    const bool finished = ptx::mbarrier_wait(done, 0, abort_flag);
    if (!finished && threadIdx.x == 0 && atomicCAS(status, 0u, 103u) == 0u) status[1] = blockIdx.x;
    ptx::tcgen05_fence_after();
    if (finished && *abort_flag == 0) {
        const int row = tile_m * TILE_ROWS + (warp % 4) * 32 + int(lane / 4);
        const uint32_t lane_base = uint32_t(warp % 4) * 32;
        for (int half = 0; half < 2; half++)
            for (int chunk = 0; chunk < TILE_COLUMNS / 64; chunk++) {
                uint32_t values[32];
                load_16x256b_x8(tmem + ((lane_base + uint32_t(half) * 16) << 16) + uint32_t(chunk) * 64, values);
                ptx::tmem_load_wait();
                for (int index = 0; index < 8; index++) {
                    const int column = tile_n * TILE_COLUMNS + (chunk * 8 + index) * 8 + int(lane % 4) * 2;
                    for (int pair = 0; pair < 2; pair++) {      // rows r and r + 8 of the fragment
                        const int r = row + half * 16 + pair * 8;
                        if (r < m && column + 1 < n)
                            *reinterpret_cast<float2 *>(output + size_t(r) * n + column) =
                                make_float2(__uint_as_float(values[index * 4 + pair * 2]), __uint_as_float(values[index * 4 + pair * 2 + 1]));
                        else if (r < m && column < n)
                            output[size_t(r) * n + column] = __uint_as_float(values[index * 4 + pair * 2]);
                    }
                }
            }
    }
    ptx::tcgen05_fence_before();
    __syncthreads();
    if (*abort_flag != 0 && threadIdx.x == 0) {
        // a wait gave up: give copies that may still be in flight a bounded time to land before the shared memory is released
        const unsigned long long start = ptx::global_timer();
        while (ptx::global_timer() - start < 2000000ull) __nanosleep(1000);
    }
    __syncthreads();
    if (warp == 0) {
        ptx::tcgen05_fence_after();
        ptx::tmem_dealloc<1>(tmem, TILE_COLUMNS);
    }
}
