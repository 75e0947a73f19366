// Entry points of the tcgen05 GEMM family.  Each is an `extern "C"` kernel so that the host side can
// find it by name in the module it loads with cuModuleLoadData, which is also how the reference's
// interop layer would load it (crates/gpurs/src/raw/module.rs:64-92).
#include "gemm_tcgen05.cuh"

#define GPURS_GEMM_KERNEL(NAME, KIND, FORMAT, ACC, OUT, BLOCK_N, GROUP, STAGES, ALGEBRA)                          \
    extern "C" __global__ void __launch_bounds__(gemm::NUM_THREADS, 1)                                           \
    NAME(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,                   \
         const __grid_constant__ CUtensorMap map_c, const __grid_constant__ gemm::Params params) {               \
        gemm::gemm_body<KIND, FORMAT, ACC, OUT, BLOCK_N, GROUP, STAGES, false, false, false, ALGEBRA>(&map_a, &map_b, &map_c, params); \
    }

// Operand format codes inside each kind: f16 = 0, bf16 = 1, tf32 = 2 (kind f16 / tf32); signed int8 = 1
// (kind i8); e4m3 = 0 (kind f8f6f4).  Accumulator: 1 = f32, 2 = s32.
// STEM_cg{1,2}: the plain product (no output algebra compiled in); STEM_ep_cg{1,2}: with the epilogue algebra of Params
// (alpha, row / column scales, bias, row bias, residual, row reductions, accumulation into C).  Integer outputs take no
// algebra and have the plain entries only.
#define GPURS_GEMM_PAIR(STEM, KIND, FORMAT, ACC, OUT)                                  \
    GPURS_GEMM_KERNEL(STEM##_cg1, KIND, FORMAT, ACC, OUT, gemm::BLOCK_N, 1, gemm::STAGES_SINGLE, false)            \
    GPURS_GEMM_KERNEL(STEM##_cg2, KIND, FORMAT, ACC, OUT, gemm::BLOCK_N, 2, gemm::STAGES_PAIR, false)
#define GPURS_GEMM_PAIR_EP(STEM, KIND, FORMAT, ACC, OUT)                               \
    GPURS_GEMM_PAIR(STEM, KIND, FORMAT, ACC, OUT)                                      \
    GPURS_GEMM_KERNEL(STEM##_ep_cg1, KIND, FORMAT, ACC, OUT, gemm::BLOCK_N, 1, gemm::STAGES_SINGLE, true)          \
    GPURS_GEMM_KERNEL(STEM##_ep_cg2, KIND, FORMAT, ACC, OUT, gemm::BLOCK_N, 2, gemm::STAGES_PAIR, true)

GPURS_GEMM_PAIR_EP(gpurs_gemm_f16_f32, ptx::KIND_F16, 0, 1, gemm::OUT_F32)
GPURS_GEMM_PAIR_EP(gpurs_gemm_f16_f16, ptx::KIND_F16, 0, 1, gemm::OUT_F16)
GPURS_GEMM_PAIR_EP(gpurs_gemm_bf16_f32, ptx::KIND_F16, 1, 1, gemm::OUT_F32)
GPURS_GEMM_PAIR_EP(gpurs_gemm_bf16_bf16, ptx::KIND_F16, 1, 1, gemm::OUT_BF16)
GPURS_GEMM_PAIR_EP(gpurs_gemm_tf32_f32, ptx::KIND_TF32, 2, 1, gemm::OUT_F32)
GPURS_GEMM_PAIR(gpurs_gemm_i8_i32, ptx::KIND_I8, 1, 2, gemm::OUT_I32)
GPURS_GEMM_PAIR_EP(gpurs_gemm_e4m3_f32, ptx::KIND_F8F6F4, 0, 1, gemm::OUT_F32)
GPURS_GEMM_PAIR_EP(gpurs_gemm_e4m3_bf16, ptx::KIND_F8F6F4, 0, 1, gemm::OUT_BF16)

// "Push" entries: the CTA-pair kernels with an epilogue that stores every box of C to all GPUs of the box (see
// gemm::PushTargets).  They require 16-byte aligned output rows (the TMA-store epilogue).
#define GPURS_GEMM_PUSH_KERNEL(NAME, KIND, FORMAT, ACC, OUT)                                                        \
    extern "C" __global__ void __launch_bounds__(gemm::NUM_THREADS, 1)                                              \
    NAME(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,                      \
         const __grid_constant__ gemm::PushTargets targets, const __grid_constant__ gemm::Params params) {          \
        gemm::gemm_body<KIND, FORMAT, ACC, OUT, gemm::BLOCK_N, 2, gemm::STAGES_PAIR, true>(&map_a, &map_b, nullptr, params, &targets); \
    }

GPURS_GEMM_PUSH_KERNEL(gpurs_gemm_bf16_bf16_push_cg2, ptx::KIND_F16, 1, 1, gemm::OUT_BF16)
GPURS_GEMM_PUSH_KERNEL(gpurs_gemm_f16_f32_push_cg2, ptx::KIND_F16, 0, 1, gemm::OUT_F32)
GPURS_GEMM_PUSH_KERNEL(gpurs_gemm_i8_i32_push_cg2, ptx::KIND_I8, 1, 2, gemm::OUT_I32)
GPURS_GEMM_PUSH_KERNEL(gpurs_gemm_e4m3_bf16_push_cg2, ptx::KIND_F8F6F4, 0, 1, gemm::OUT_BF16)

// Batched entries: rank-3 descriptors (z = batch) for A, B and C; tiles of all matrices share one persistent grid.
#define GPURS_GEMM_BATCHED_KERNEL(NAME, KIND, FORMAT, ACC, OUT, GROUP, STAGES)                                      \
    extern "C" __global__ void __launch_bounds__(gemm::NUM_THREADS, 1)                                              \
    NAME(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,                      \
         const __grid_constant__ CUtensorMap map_c, const __grid_constant__ gemm::Params params) {                  \
        gemm::gemm_body<KIND, FORMAT, ACC, OUT, gemm::BLOCK_N, GROUP, STAGES, false, true>(&map_a, &map_b, &map_c, params); \
    }

GPURS_GEMM_BATCHED_KERNEL(gpurs_gemm_bf16_bf16_batched_cg1, ptx::KIND_F16, 1, 1, gemm::OUT_BF16, 1, gemm::STAGES_SINGLE)
GPURS_GEMM_BATCHED_KERNEL(gpurs_gemm_bf16_bf16_batched_cg2, ptx::KIND_F16, 1, 1, gemm::OUT_BF16, 2, gemm::STAGES_PAIR)
GPURS_GEMM_BATCHED_KERNEL(gpurs_gemm_bf16_f32_batched_cg1, ptx::KIND_F16, 1, 1, gemm::OUT_F32, 1, gemm::STAGES_SINGLE)
GPURS_GEMM_BATCHED_KERNEL(gpurs_gemm_bf16_f32_batched_cg2, ptx::KIND_F16, 1, 1, gemm::OUT_F32, 2, gemm::STAGES_PAIR)
GPURS_GEMM_BATCHED_KERNEL(gpurs_gemm_f16_f16_batched_cg1, ptx::KIND_F16, 0, 1, gemm::OUT_F16, 1, gemm::STAGES_SINGLE)
GPURS_GEMM_BATCHED_KERNEL(gpurs_gemm_f16_f16_batched_cg2, ptx::KIND_F16, 0, 1, gemm::OUT_F16, 2, gemm::STAGES_PAIR)
GPURS_GEMM_BATCHED_KERNEL(gpurs_gemm_f16_f32_batched_cg1, ptx::KIND_F16, 0, 1, gemm::OUT_F32, 1, gemm::STAGES_SINGLE)
GPURS_GEMM_BATCHED_KERNEL(gpurs_gemm_f16_f32_batched_cg2, ptx::KIND_F16, 0, 1, gemm::OUT_F32, 2, gemm::STAGES_PAIR)

// Stream-K entries: the tiles of the last, partial round are split along K over the whole grid (gemm_schedule.hpp).
#define GPURS_GEMM_STREAMK_KERNEL(NAME, KIND, FORMAT, ACC, OUT, GROUP, STAGES, ALGEBRA)                             \
    extern "C" __global__ void __launch_bounds__(gemm::NUM_THREADS, 1)                                              \
    NAME(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,                      \
         const __grid_constant__ CUtensorMap map_c, const __grid_constant__ gemm::Params params) {                  \
        gemm::gemm_body<KIND, FORMAT, ACC, OUT, gemm::BLOCK_N, GROUP, STAGES, false, false, true, ALGEBRA>(&map_a, &map_b, &map_c, params); \
    }
#define GPURS_GEMM_STREAMK_PAIR(STEM, KIND, FORMAT, ACC, OUT)                                       \
    GPURS_GEMM_STREAMK_KERNEL(STEM##_sk_cg1, KIND, FORMAT, ACC, OUT, 1, gemm::STAGES_SINGLE, false)  \
    GPURS_GEMM_STREAMK_KERNEL(STEM##_sk_cg2, KIND, FORMAT, ACC, OUT, 2, gemm::STAGES_PAIR, false)
#define GPURS_GEMM_STREAMK_PAIR_EP(STEM, KIND, FORMAT, ACC, OUT)                                    \
    GPURS_GEMM_STREAMK_PAIR(STEM, KIND, FORMAT, ACC, OUT)                                           \
    GPURS_GEMM_STREAMK_KERNEL(STEM##_sk_ep_cg1, KIND, FORMAT, ACC, OUT, 1, gemm::STAGES_SINGLE, true) \
    GPURS_GEMM_STREAMK_KERNEL(STEM##_sk_ep_cg2, KIND, FORMAT, ACC, OUT, 2, gemm::STAGES_PAIR, true)

GPURS_GEMM_STREAMK_PAIR_EP(gpurs_gemm_f16_f32, ptx::KIND_F16, 0, 1, gemm::OUT_F32)
GPURS_GEMM_STREAMK_PAIR_EP(gpurs_gemm_f16_f16, ptx::KIND_F16, 0, 1, gemm::OUT_F16)
GPURS_GEMM_STREAMK_PAIR_EP(gpurs_gemm_bf16_f32, ptx::KIND_F16, 1, 1, gemm::OUT_F32)
GPURS_GEMM_STREAMK_PAIR_EP(gpurs_gemm_bf16_bf16, ptx::KIND_F16, 1, 1, gemm::OUT_BF16)
GPURS_GEMM_STREAMK_PAIR(gpurs_gemm_i8_i32, ptx::KIND_I8, 1, 2, gemm::OUT_I32)
GPURS_GEMM_STREAMK_PAIR_EP(gpurs_gemm_tf32_f32, ptx::KIND_TF32, 2, 1, gemm::OUT_F32)
GPURS_GEMM_STREAMK_PAIR_EP(gpurs_gemm_e4m3_f32, ptx::KIND_F8F6F4, 0, 1, gemm::OUT_F32)
GPURS_GEMM_STREAMK_PAIR_EP(gpurs_gemm_e4m3_bf16, ptx::KIND_F8F6F4, 0, 1, gemm::OUT_BF16)
