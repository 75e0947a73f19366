// Entry points of the grouped (mixture-of-experts) GEMM (see gemm_grouped_tcgen05.cuh).
#include "gemm_grouped_tcgen05.cuh"

#define GPURS_GROUPED_KERNEL(NAME, FORMAT, OUT)                                                                    \
    extern "C" __global__ void __launch_bounds__(gemm::GROUPED_THREADS, 1)                                         \
    NAME(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ gemm::GroupedParams params) {          \
        gemm::gemm_grouped_body<FORMAT, OUT, gemm::STAGES_SINGLE>(&map_w, params);                                 \
    }

GPURS_GROUPED_KERNEL(gpurs_gemm_grouped_f16_f16, 0, gemm::OUT_F16)
GPURS_GROUPED_KERNEL(gpurs_gemm_grouped_f16_f32, 0, gemm::OUT_F32)
GPURS_GROUPED_KERNEL(gpurs_gemm_grouped_bf16_bf16, 1, gemm::OUT_BF16)
GPURS_GROUPED_KERNEL(gpurs_gemm_grouped_bf16_f32, 1, gemm::OUT_F32)
