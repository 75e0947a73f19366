// Entry points of the 2:4 structured-sparse GEMM (see gemm_sparse_tcgen05.cuh).
#include "gemm_sparse_tcgen05.cuh"
#include "gemm_sparse_tall_tcgen05.cuh"

#define GPURS_SPARSE_KERNEL(NAME, FORMAT, OUT, GROUP, STAGES)                                                         \
    extern "C" __global__ void __launch_bounds__(gemm::NUM_THREADS, 1)                                               \
    NAME(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,                       \
         const __grid_constant__ CUtensorMap map_e, const __grid_constant__ gemm::Params params) {                   \
        gemm::gemm_sparse_body<FORMAT, OUT, GROUP, STAGES>(&map_a, &map_b, &map_e, params);                          \
    }

GPURS_SPARSE_KERNEL(gpurs_gemm_sparse_bf16_bf16_cg1, 1, gemm::OUT_BF16, 1, gemm::SPARSE_STAGES_SINGLE)
GPURS_SPARSE_KERNEL(gpurs_gemm_sparse_bf16_bf16_cg2, 1, gemm::OUT_BF16, 2, gemm::SPARSE_STAGES_PAIR)
GPURS_SPARSE_KERNEL(gpurs_gemm_sparse_bf16_f32_cg1, 1, gemm::OUT_F32, 1, gemm::SPARSE_STAGES_SINGLE)
GPURS_SPARSE_KERNEL(gpurs_gemm_sparse_bf16_f32_cg2, 1, gemm::OUT_F32, 2, gemm::SPARSE_STAGES_PAIR)
GPURS_SPARSE_KERNEL(gpurs_gemm_sparse_f16_f32_cg1, 0, gemm::OUT_F32, 1, gemm::SPARSE_STAGES_SINGLE)
GPURS_SPARSE_KERNEL(gpurs_gemm_sparse_f16_f32_cg2, 0, gemm::OUT_F32, 2, gemm::SPARSE_STAGES_PAIR)

// Push entry (see gemm::SparsePushTargets): the M-sharded sparse product whose epilogue stores every box of C into all
// GPUs' copies of the gathered matrix.
extern "C" __global__ void __launch_bounds__(gemm::NUM_THREADS, 1)
gpurs_gemm_sparse_bf16_bf16_push_cg2(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                                     const __grid_constant__ CUtensorMap map_e, const __grid_constant__ gemm::SparsePushTargets targets,
                                     const __grid_constant__ gemm::Params params) {
    gemm::gemm_sparse_body<1, gemm::OUT_BF16, 2, gemm::SPARSE_STAGES_PAIR, true>(&map_a, &map_b, &map_e, params, &targets);
}

// 512 x 224 CTA-pair tiles (see gemm_sparse_tall_tcgen05.cuh).
#define GPURS_SPARSE_TALL_KERNEL(NAME, FORMAT, OUT)                                                                   \
    extern "C" __global__ void __launch_bounds__(gemm::SPARSE_TALL_THREADS, 1)                                       \
    NAME(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,                       \
         const __grid_constant__ CUtensorMap map_e, const __grid_constant__ gemm::Params params) {                   \
        gemm::gemm_sparse_tall_body<FORMAT, OUT>(&map_a, &map_b, &map_e, params);                                    \
    }

GPURS_SPARSE_TALL_KERNEL(gpurs_gemm_sparse_bf16_bf16_t512_cg2, 1, gemm::OUT_BF16)
GPURS_SPARSE_TALL_KERNEL(gpurs_gemm_sparse_bf16_f32_t512_cg2, 1, gemm::OUT_F32)
GPURS_SPARSE_TALL_KERNEL(gpurs_gemm_sparse_f16_f32_t512_cg2, 0, gemm::OUT_F32)

// Stream-K entries: the K-blocks of the tiles of a split round are spread over the grid (gemm_schedule.hpp).
#define GPURS_SPARSE_STREAMK_KERNEL(NAME, FORMAT, OUT, GROUP, STAGES)                                                 \
    extern "C" __global__ void __launch_bounds__(gemm::NUM_THREADS, 1)                                               \
    NAME(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,                       \
         const __grid_constant__ CUtensorMap map_e, const __grid_constant__ gemm::Params params) {                   \
        gemm::gemm_sparse_body<FORMAT, OUT, GROUP, STAGES, false, true>(&map_a, &map_b, &map_e, params);             \
    }

GPURS_SPARSE_STREAMK_KERNEL(gpurs_gemm_sparse_bf16_bf16_sk_cg1, 1, gemm::OUT_BF16, 1, gemm::SPARSE_STAGES_SINGLE)
GPURS_SPARSE_STREAMK_KERNEL(gpurs_gemm_sparse_bf16_bf16_sk_cg2, 1, gemm::OUT_BF16, 2, gemm::SPARSE_STAGES_PAIR)
GPURS_SPARSE_STREAMK_KERNEL(gpurs_gemm_sparse_bf16_f32_sk_cg1, 1, gemm::OUT_F32, 1, gemm::SPARSE_STAGES_SINGLE)
GPURS_SPARSE_STREAMK_KERNEL(gpurs_gemm_sparse_bf16_f32_sk_cg2, 1, gemm::OUT_F32, 2, gemm::SPARSE_STAGES_PAIR)
GPURS_SPARSE_STREAMK_KERNEL(gpurs_gemm_sparse_f16_f32_sk_cg1, 0, gemm::OUT_F32, 1, gemm::SPARSE_STAGES_SINGLE)
GPURS_SPARSE_STREAMK_KERNEL(gpurs_gemm_sparse_f16_f32_sk_cg2, 0, gemm::OUT_F32, 2, gemm::SPARSE_STAGES_PAIR)
