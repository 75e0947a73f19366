// Entry points of the dense GEMM on 256 x 512 CTA-pair tiles (gemm_wide_tcgen05.cuh): plain epilogue, n x k right operand.
#include "gemm_wide_tcgen05.cuh"

#define GPURS_WIDE_ENTRY(NAME, KIND, FORMAT, ACC, OUT, ALGEBRA)                                                    \
    extern "C" __global__ void __launch_bounds__(gemm::WIDE_THREADS, 1)                                            \
    NAME(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,                     \
         const __grid_constant__ CUtensorMap map_c, const __grid_constant__ gemm::Params params) {                 \
        gemm::gemm_wide_body<KIND, FORMAT, ACC, OUT, ALGEBRA>(&map_a, &map_b, &map_c, params);                     \
    }
// the lean entry a plain product runs, and the one with the output algebra compiled in (float outputs)
#define GPURS_WIDE_KERNEL(STEM, KIND, FORMAT, ACC, OUT)                                                            \
    GPURS_WIDE_ENTRY(STEM##_w512_cg2, KIND, FORMAT, ACC, OUT, false)                                               \
    GPURS_WIDE_ENTRY(STEM##_w512_ep_cg2, KIND, FORMAT, ACC, OUT, true)

// Operand format codes and accumulator codes as in gemm_tcgen05.cu.
GPURS_WIDE_KERNEL(gpurs_gemm_f16_f32, ptx::KIND_F16, 0, 1, gemm::OUT_F32)
GPURS_WIDE_KERNEL(gpurs_gemm_f16_f16, ptx::KIND_F16, 0, 1, gemm::OUT_F16)
GPURS_WIDE_KERNEL(gpurs_gemm_bf16_f32, ptx::KIND_F16, 1, 1, gemm::OUT_F32)
GPURS_WIDE_KERNEL(gpurs_gemm_bf16_bf16, ptx::KIND_F16, 1, 1, gemm::OUT_BF16)
GPURS_WIDE_ENTRY(gpurs_gemm_i8_i32_w512_cg2, ptx::KIND_I8, 1, 2, gemm::OUT_I32, false)
GPURS_WIDE_KERNEL(gpurs_gemm_e4m3_f32, ptx::KIND_F8F6F4, 0, 1, gemm::OUT_F32)
GPURS_WIDE_KERNEL(gpurs_gemm_e4m3_bf16, ptx::KIND_F8F6F4, 0, 1, gemm::OUT_BF16)

// 256 x 480 tiles (second half 224 columns), 32-bit outputs
#define GPURS_WIDE_480_ENTRY(NAME, KIND, FORMAT, ACC, OUT)                                                         \
    extern "C" __global__ void __launch_bounds__(gemm::WIDE_THREADS, 1)                                            \
    NAME(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,                     \
         const __grid_constant__ CUtensorMap map_c, const __grid_constant__ gemm::Params params) {                 \
        gemm::gemm_wide_body<KIND, FORMAT, ACC, OUT, false, 224>(&map_a, &map_b, &map_c, params);                  \
    }

GPURS_WIDE_480_ENTRY(gpurs_gemm_f16_f32_w480_cg2, ptx::KIND_F16, 0, 1, gemm::OUT_F32)
GPURS_WIDE_480_ENTRY(gpurs_gemm_bf16_f32_w480_cg2, ptx::KIND_F16, 1, 1, gemm::OUT_F32)
GPURS_WIDE_480_ENTRY(gpurs_gemm_i8_i32_w480_cg2, ptx::KIND_I8, 1, 2, gemm::OUT_I32)
GPURS_WIDE_480_ENTRY(gpurs_gemm_e4m3_f32_w480_cg2, ptx::KIND_F8F6F4, 0, 1, gemm::OUT_F32)
