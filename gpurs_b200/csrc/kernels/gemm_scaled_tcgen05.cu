// Entry points of the GEMMs that promote every K-block to registers (see gemm_scaled_tcgen05.cuh): the
// block-scaled FP8 product and the fp32 product built from three TF32 passes.
#include "gemm_scaled_tcgen05.cuh"

#define GPURS_PROMOTED_KERNEL(NAME, KIND, FORMAT, OUT, SCALED, GROUP, STAGES)                                                         \
    extern "C" __global__ void __launch_bounds__(gemm::SCALED_THREADS, 1)                                      \
    NAME(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,                 \
         const __grid_constant__ gemm::Params params) {                                                        \
        gemm::gemm_promoted_body<KIND, FORMAT, OUT, SCALED, GROUP, STAGES>(&map_a, &map_b, params);            \
    }

GPURS_PROMOTED_KERNEL(gpurs_gemm_e4m3_scaled_bf16_cg1, ptx::KIND_F8F6F4, 0, gemm::OUT_BF16, true, 1, gemm::STAGES_SINGLE)
GPURS_PROMOTED_KERNEL(gpurs_gemm_e4m3_scaled_bf16_cg2, ptx::KIND_F8F6F4, 0, gemm::OUT_BF16, true, 2, gemm::STAGES_PAIR)
GPURS_PROMOTED_KERNEL(gpurs_gemm_e4m3_scaled_f32_cg1, ptx::KIND_F8F6F4, 0, gemm::OUT_F32, true, 1, gemm::STAGES_SINGLE)
GPURS_PROMOTED_KERNEL(gpurs_gemm_e4m3_scaled_f32_cg2, ptx::KIND_F8F6F4, 0, gemm::OUT_F32, true, 2, gemm::STAGES_PAIR)
GPURS_PROMOTED_KERNEL(gpurs_gemm_tf32_promoted_f32_cg1, ptx::KIND_TF32, 2, gemm::OUT_F32, false, 1, gemm::STAGES_SINGLE)
GPURS_PROMOTED_KERNEL(gpurs_gemm_tf32_promoted_f32_cg2, ptx::KIND_TF32, 2, gemm::OUT_F32, false, 2, gemm::STAGES_PAIR)

// Stream-K entries: the K-blocks of the tiles of a split round are spread over the grid (gemm_schedule.hpp).
#define GPURS_PROMOTED_STREAMK_KERNEL(NAME, KIND, FORMAT, OUT, SCALED, GROUP, STAGES)                                               \
    extern "C" __global__ void __launch_bounds__(gemm::SCALED_THREADS, 1)                                      \
    NAME(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,                 \
         const __grid_constant__ gemm::Params params) {                                                        \
        gemm::gemm_promoted_body<KIND, FORMAT, OUT, SCALED, GROUP, STAGES, true>(&map_a, &map_b, params);      \
    }

GPURS_PROMOTED_STREAMK_KERNEL(gpurs_gemm_e4m3_scaled_bf16_sk_cg1, ptx::KIND_F8F6F4, 0, gemm::OUT_BF16, true, 1, gemm::STAGES_SINGLE)
GPURS_PROMOTED_STREAMK_KERNEL(gpurs_gemm_e4m3_scaled_bf16_sk_cg2, ptx::KIND_F8F6F4, 0, gemm::OUT_BF16, true, 2, gemm::STAGES_PAIR)
GPURS_PROMOTED_STREAMK_KERNEL(gpurs_gemm_e4m3_scaled_f32_sk_cg1, ptx::KIND_F8F6F4, 0, gemm::OUT_F32, true, 1, gemm::STAGES_SINGLE)
GPURS_PROMOTED_STREAMK_KERNEL(gpurs_gemm_e4m3_scaled_f32_sk_cg2, ptx::KIND_F8F6F4, 0, gemm::OUT_F32, true, 2, gemm::STAGES_PAIR)
GPURS_PROMOTED_STREAMK_KERNEL(gpurs_gemm_tf32_promoted_f32_sk_cg1, ptx::KIND_TF32, 2, gemm::OUT_F32, false, 1, gemm::STAGES_SINGLE)
GPURS_PROMOTED_STREAMK_KERNEL(gpurs_gemm_tf32_promoted_f32_sk_cg2, ptx::KIND_TF32, 2, gemm::OUT_F32, false, 2, gemm::STAGES_PAIR)
