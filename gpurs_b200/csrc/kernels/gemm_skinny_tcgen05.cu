// Entry points of the skinny (decode-shaped) GEMM (see gemm_skinny_tcgen05.cuh).
#include "gemm_skinny_tcgen05.cuh"

#define GPURS_SKINNY_KERNEL(NAME, FORMAT, TOKENS)                                                                  \
    extern "C" __global__ void __launch_bounds__(gemm::NUM_THREADS)                                                \
    NAME(const __grid_constant__ CUtensorMap map_big, const __grid_constant__ CUtensorMap map_small,              \
         const __grid_constant__ gemm::SkinnyParams params) {                                                      \
        gemm::gemm_skinny_body<FORMAT, TOKENS>(&map_big, &map_small, params);                                      \
    }

GPURS_SKINNY_KERNEL(gpurs_gemm_skinny_f16_f32_t16, 0, 16)
GPURS_SKINNY_KERNEL(gpurs_gemm_skinny_f16_f32_t32, 0, 32)
GPURS_SKINNY_KERNEL(gpurs_gemm_skinny_f16_f32_t64, 0, 64)
GPURS_SKINNY_KERNEL(gpurs_gemm_skinny_bf16_f32_t16, 1, 16)
GPURS_SKINNY_KERNEL(gpurs_gemm_skinny_bf16_f32_t32, 1, 32)
GPURS_SKINNY_KERNEL(gpurs_gemm_skinny_bf16_f32_t64, 1, 64)
