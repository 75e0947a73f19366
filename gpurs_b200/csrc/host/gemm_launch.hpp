// The validated description of one tcgen05 GEMM launch and the function that enqueues it (matmul.cpp).
#pragma once
#include "../kernels/gemm_params.hpp"
#include "runtime.hpp"

namespace launcher {

// One launch of a tcgen05 GEMM entry: everything the kernel needs, already validated.
struct Gemm {
    const char *stem;
    int element_type, element_bytes, output_bytes;
    int output_type = GPURS_F32;                 // element type of C
    gpurs_device_ptr a, b, c;
    uint64_t lda, ldb, ldc, m, n, k;
    int cta_group, raster_rows, max_ctas;
    gpurs_device_ptr scale_a = 0, scale_b = 0;   // block-scaled E4M3 only
    int threads = gemm::NUM_THREADS;
    gpurs_device_ptr bias = 0;                   // optional fp32 [n]
    gpurs_device_ptr row_scale = 0, column_scale = 0;   // optional fp32 [m] and [n]
    float alpha = 0.0f;                          // 0 = none
    gpurs_device_ptr row_absmax = 0;             // optional fp32 [m], atomic max of |C[row, :]|
    gpurs_device_ptr row_bias = 0;               // optional fp32 [m]
    gpurs_device_ptr residual = 0;               // optional m x n matrix of C's type, pitch ldr, added as beta * residual
    uint64_t ldr = 0;
    float beta = 1.0f;
    gpurs_device_ptr row_sum = 0;                // optional fp32 [m], atomic add of the row's sum
    bool accumulate = false;                     // fp32 output: atomic adds into C instead of stores
    const gpurs_launch_config *launch = nullptr; // the caller's explicit geometry, already checked for plausibility
    uint64_t batches = 1, stride_a = 0, stride_b = 0, stride_c = 0;   // batched entries: matrices and the elements between them
    bool whole_tiles = false;                    // never split the last round's tiles along K
    int tile_width = 0;                          // 0 the launcher's choice, 512 wide tiles wherever possible, 256 never wide
    bool force_split = false;                    // split it whenever it is not full, whether or not that pays
    bool b_row_major = false;                    // B stored k x n
    int l2_policy = 0;                           // Params::l2_policy
    gpurs_device_ptr metadata = 0;               // 2:4-sparse A only: `a` then holds the kept values, k the logical depth
    gpurs_device_ptr partials = 0;               // room for the parts of tiles split along K, if the caller already holds the workspace
    uint64_t partials_bytes = 0;
    const gpurs_gather_desc *gather = nullptr;   // push epilogue: C is a block of rows of a matrix kept on every GPU of the box
};

// Encodes the operand descriptors, picks the geometry and enqueues the kernel on `stream`.  The
// caller has made the gpu's context current.
int launch_gemm(gpurs_stream *stream, const Gemm &g);

}  // namespace launcher
