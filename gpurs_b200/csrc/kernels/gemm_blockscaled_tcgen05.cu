// Entry points of the CTA-pair block-scaled FP8 product with four accumulators in flight (gemm_blockscaled_tcgen05.cuh).
#include "gemm_blockscaled_tcgen05.cuh"

#define GPURS_BLOCKSCALED_KERNEL(NAME, OUT)                                                                        \
    extern "C" __global__ void __launch_bounds__(gemm::BLOCKSCALED_THREADS, 1)                                     \
    NAME(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,                     \
         const __grid_constant__ CUtensorMap map_c, const __grid_constant__ gemm::Params params) {                 \
        gemm::gemm_blockscaled_body<OUT>(&map_a, &map_b, &map_c, params);                                          \
    }

GPURS_BLOCKSCALED_KERNEL(gpurs_gemm_e4m3_blockscaled_bf16_cg2, gemm::OUT_BF16)
GPURS_BLOCKSCALED_KERNEL(gpurs_gemm_e4m3_blockscaled_f32_cg2, gemm::OUT_F32)
