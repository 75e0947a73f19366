// Entry points of the FP8 GEMM with the tensor core's own (MX, power-of-two) block scaling (see gemm_mx_tcgen05.cuh).
#include "gemm_mx_tcgen05.cuh"

#define GPURS_MX_KERNEL(NAME, OUT, GROUP, STAGES)                                                                    \
    extern "C" __global__ void __launch_bounds__(gemm::NUM_THREADS, 1)                                               \
    NAME(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,                       \
         const __grid_constant__ CUtensorMap map_sa, const __grid_constant__ CUtensorMap map_sb,                     \
         const __grid_constant__ gemm::Params params) {                                                              \
        gemm::gemm_mx_body<OUT, GROUP, STAGES>(&map_a, &map_b, &map_sa, &map_sb, params);                            \
    }

GPURS_MX_KERNEL(gpurs_gemm_e4m3_mx_bf16_cg1, gemm::OUT_BF16, 1, gemm::MX_STAGES_SINGLE)
GPURS_MX_KERNEL(gpurs_gemm_e4m3_mx_bf16_cg2, gemm::OUT_BF16, 2, gemm::MX_STAGES_PAIR)
GPURS_MX_KERNEL(gpurs_gemm_e4m3_mx_f32_cg1, gemm::OUT_F32, 1, gemm::MX_STAGES_SINGLE)
GPURS_MX_KERNEL(gpurs_gemm_e4m3_mx_f32_cg2, gemm::OUT_F32, 2, gemm::MX_STAGES_PAIR)

// Stream-K entries: the K-blocks of the tiles of a split round are spread over the grid (gemm_schedule.hpp).
#define GPURS_MX_STREAMK_KERNEL(NAME, OUT, GROUP, STAGES)                                                            \
    extern "C" __global__ void __launch_bounds__(gemm::NUM_THREADS, 1)                                               \
    NAME(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,                       \
         const __grid_constant__ CUtensorMap map_sa, const __grid_constant__ CUtensorMap map_sb,                     \
         const __grid_constant__ gemm::Params params) {                                                              \
        gemm::gemm_mx_body<OUT, GROUP, STAGES, true>(&map_a, &map_b, &map_sa, &map_sb, params);                      \
    }

GPURS_MX_STREAMK_KERNEL(gpurs_gemm_e4m3_mx_bf16_sk_cg1, gemm::OUT_BF16, 1, gemm::MX_STAGES_SINGLE)
GPURS_MX_STREAMK_KERNEL(gpurs_gemm_e4m3_mx_bf16_sk_cg2, gemm::OUT_BF16, 2, gemm::MX_STAGES_PAIR)
GPURS_MX_STREAMK_KERNEL(gpurs_gemm_e4m3_mx_f32_sk_cg1, gemm::OUT_F32, 1, gemm::MX_STAGES_SINGLE)
GPURS_MX_STREAMK_KERNEL(gpurs_gemm_e4m3_mx_f32_sk_cg2, gemm::OUT_F32, 2, gemm::MX_STAGES_PAIR)
