/*
 * gpurs_b200 — C ABI of the B200-native matrix-multiply path of gpurs.
 *
 * This is the boundary a gpurs host binds instead of (or beside) its own `crates/driver` FFI block
 * (crates/driver/src/ffi.rs:47-214): plain pointers and sizes, opaque handles, `int` results.  Every
 * function returns 0 on success, the raw CUresult of the failing CUDA driver call (1..99999), or one
 * of the GPURS_E_* codes below, which mirror the variants of the reference's runtime error enum
 * (crates/gpurs/src/error.rs:13-71).  Nothing throws, aborts or exits across this boundary.
 *
 * Threading follows the reference (crates/gpurs/src/lib.rs:7-9): a handle belongs to the host thread
 * that created it; use one gpurs_gpu per device and thread.  Every call makes the handle's context
 * current for its duration and restores the caller's on return
 * (crates/driver/src/context.rs:117-129).
 *
 * Device memory handed to gpurs_matmul is borrowed until the stream has passed the launch
 * (the contract of `Stream::submit_external`, crates/gpurs/src/raw/interop.rs:37-59).
 */
#ifndef GPURS_B200_H
#define GPURS_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif
#if defined(__GNUC__)
#pragma GCC visibility push(default)
#endif

typedef struct gpurs_gpu gpurs_gpu;
typedef struct gpurs_stream gpurs_stream;
typedef struct gpurs_event gpurs_event;
typedef struct gpurs_module gpurs_module;
typedef struct gpurs_kernel gpurs_kernel;
typedef uint64_t gpurs_device_ptr; /* `DevicePointer = u64`, crates/driver/src/ffi.rs:10 */

/* Library result codes (driver failures keep their CUresult value). */
enum {
    GPURS_OK = 0,
    GPURS_E_CONTEXT_MISMATCH = 100001,   /* Error::ContextMismatch  */
    GPURS_E_SIZE_OVERFLOW = 100002,      /* Error::SizeOverflow     */
    GPURS_E_LENGTH_MISMATCH = 100003,    /* Error::LengthMismatch   */
    GPURS_E_OVERLAP = 100004,            /* Error::Overlap          */
    GPURS_E_INVALID_VIEW = 100005,       /* Error::InvalidView      */
    GPURS_E_ALIASING = 100006,           /* Error::Aliasing         */
    GPURS_E_UNKNOWN_KERNEL = 100007,     /* Error::UnknownKernel    */
    GPURS_E_INCOMPATIBLE_DEVICE = 100008,/* Error::IncompatibleDevice */
    GPURS_E_INVALID_ARGUMENT = 100009,   /* null handle / unknown enum value */
    GPURS_E_DEVICE_TIMEOUT = 100010,     /* a bounded device-side wait gave up (no reference counterpart:
                                            the reference's waits are unbounded) */
    GPURS_E_DRIVER_UNAVAILABLE = 100011, /* libcuda could not be loaded */
    GPURS_E_COLLECTIVE = 100012          /* libnccl could not be loaded, or an NCCL call failed (its text is in gpurs_last_error) */
};

/* Element types.  The values of the first three match the TMA data-type codes the reference uses
 * (crates/gpurs/src/gpu/tensor/element.rs:48,78,113). */
enum {
    GPURS_F16 = 6,
    GPURS_F32 = 7,
    GPURS_BF16 = 9,
    GPURS_I8 = 100,
    GPURS_I32 = 101,
    GPURS_E4M3 = 102
};

/* ---- context, streams, events ---------------------------------------------------------------- */

/* `Gpu::new(ordinal)` (crates/gpurs/src/host/context.rs:69): retains the device's primary context.
 * Fails with GPURS_E_INCOMPATIBLE_DEVICE unless the device is compute capability 10.0, the only
 * target the embedded sm_100a image supports (crates/artifact/src/target.rs:68-72). */
int gpurs_gpu_new(int ordinal, gpurs_gpu **out);
void gpurs_gpu_free(gpurs_gpu *gpu);
int gpurs_gpu_properties(gpurs_gpu *gpu, int *major, int *minor, int *multiprocessors, size_t *total_bytes);

/* `gpu.stream()` (context.rs:125-130): a new non-blocking stream. */
int gpurs_stream_new(gpurs_gpu *gpu, gpurs_stream **out);
/* Borrow a CUstream created elsewhere (`AsRaw` / `Stream::submit_external`, crates/gpurs/src/raw/interop.rs:45-59).
 * `raw` may be NULL for the legacy default stream. */
int gpurs_stream_borrow(gpurs_gpu *gpu, void *raw, gpurs_stream **out);
void gpurs_stream_free(gpurs_stream *stream);
void *gpurs_stream_raw(gpurs_stream *stream);
/* `Stream::synchronize` (crates/gpurs/src/host/stream.rs).  Also collects the device status word:
 * returns GPURS_E_DEVICE_TIMEOUT if a kernel's bounded wait gave up since the last call. */
int gpurs_stream_synchronize(gpurs_stream *stream);

/* `Stream::record_timed` / `Event::elapsed` (crates/gpurs/src/host/stream.rs:109-115,184-186). */
int gpurs_event_record_timed(gpurs_stream *stream, gpurs_event **out);
int gpurs_event_synchronize(gpurs_event *event);
int gpurs_event_elapsed_ms(gpurs_event *start, gpurs_event *end, float *milliseconds);
void gpurs_event_free(gpurs_event *event);

/* ---- memory ---------------------------------------------------------------------------------- */

/* `Gpu::allocate` (crates/gpurs/src/raw/allocation.rs:54-74): uninitialised device memory. */
int gpurs_alloc(gpurs_gpu *gpu, size_t bytes, gpurs_device_ptr *out);
int gpurs_free(gpurs_gpu *gpu, gpurs_device_ptr pointer);
/* `gpu.upload(&host)` (context.rs:132-149): allocate, copy, and wait for the copy. */
int gpurs_upload(gpurs_gpu *gpu, const void *host, size_t bytes, gpurs_device_ptr *out);
/* `gpu.zeros::<T>(n)` (context.rs:151-168): allocate and clear. */
int gpurs_zeros(gpurs_gpu *gpu, size_t bytes, gpurs_device_ptr *out);
/* `DeviceSlice::download` (crates/gpurs/src/host/memory/buffer.rs:251-271): copy back and wait. */
int gpurs_download(gpurs_gpu *gpu, gpurs_device_ptr source, void *host, size_t bytes);
/* Stream-ordered copies between existing buffers (`copy_from_host` / `copy_to_host`,
 * crates/driver/src/memory.rs); the host side should be pinned for the copy to be asynchronous. */
int gpurs_copy_to_device(gpurs_stream *stream, gpurs_device_ptr destination, const void *host, size_t bytes);
int gpurs_copy_to_host(gpurs_stream *stream, void *host, gpurs_device_ptr source, size_t bytes);
int gpurs_fill_u8(gpurs_stream *stream, gpurs_device_ptr destination, uint8_t value, size_t bytes);
/* Free and total device memory in bytes as the driver reports them now (`cuMemGetInfo`; the reference exposes the
 * same pair through `Gpu::memory_info`, crates/driver/src/memory.rs).  Does not wait for the device. */
int gpurs_memory_info(gpurs_gpu *gpu, size_t *free_bytes, size_t *total_bytes);
/* Page-locked host memory (`PinnedBuffer`, crates/gpurs/src/host/memory/pinned.rs). */
int gpurs_host_alloc(gpurs_gpu *gpu, size_t bytes, void **out);
int gpurs_host_free(gpurs_gpu *gpu, void *pointer);

/* ---- graphs ------------------------------------------------------------------------------------------ */

/* Record the operations enqueued on `stream` between begin and end (products, quantiser, compressor, copies, fills)
 * instead of running them, then replay the recording with one submission: `Stream::capture` + `Graph::instantiate` +
 * `GraphExec::launch` of the reference (crates/gpurs/src/host/graph/capture.rs:110-149,272-282; graph/exec.rs:48-72).
 * The recording keeps the addresses and shapes it was made with; the caller keeps those buffers alive and unchanged in
 * place while the graph exists.  One capture at a time per gpu handle.  Products that borrow the handle's scratch (fp32
 * operands at full precision, split-K, a last round of tiles split along K) must have run once with the same shapes before they are captured, because the
 * scratch cannot grow inside a capture (GPURS_E_INVALID_ARGUMENT otherwise); a replay takes its turn on the scratch like
 * any other call.  Calls that wait for the device (download, status_read, stream_synchronize) are not capturable. */
typedef struct gpurs_graph gpurs_graph;
int gpurs_stream_capture_begin(gpurs_stream *stream);
/* Ends the capture and instantiates the recording. */
int gpurs_stream_capture_end(gpurs_stream *stream, gpurs_graph **out);
/* Enqueues one replay of the whole recording on `stream`; does not wait. */
int gpurs_graph_launch(gpurs_graph *graph, gpurs_stream *stream);
void gpurs_graph_free(gpurs_graph *graph);

/* ---- sharing device memory between the processes of one box (no counterpart in the reference, which is
 *      single-process and single-GPU) ------------------------------------------------------------------ */

/* A 64-byte handle another process on the same machine can open to reach `pointer` (an allocation made with
 * gpurs_alloc / gpurs_upload / gpurs_zeros), and the reverse.  A pointer returned by gpurs_ipc_open addresses the peer
 * GPU's memory over NVLink and must be closed before the owner frees the allocation. */
int gpurs_ipc_export(gpurs_gpu *gpu, gpurs_device_ptr pointer, uint8_t handle[64]);
int gpurs_ipc_open(gpurs_gpu *gpu, const uint8_t handle[64], gpurs_device_ptr *out);
int gpurs_ipc_close(gpurs_gpu *gpu, gpurs_device_ptr pointer);

/* ---- TMA descriptors ------------------------------------------------------------------------- */

/* Generalises `driver::try_tensor_map` (crates/driver/src/memory.rs:325-354), which is fixed to rank 2,
 * SWIZZLE_128B, L2 promotion 256 B and zero fill.  `descriptor` receives the 128-byte CUtensorMap and
 * must be 64-byte aligned.  dims / box are innermost first; strides_bytes has rank-1 entries (the
 * innermost dimension is contiguous).  swizzle: 0 none, 1 32 B, 2 64 B, 3 128 B.  l2_promotion:
 * 0 none, 1 64 B, 2 128 B, 3 256 B.  Element types: GPURS_F16/F32/BF16/I32, and GPURS_I8 / GPURS_E4M3
 * (both encoded as bytes). */
int gpurs_tensor_map_encode(gpurs_gpu *gpu, void *descriptor, int element_type, uint32_t rank,
                            gpurs_device_ptr address, const uint64_t *dims, const uint64_t *strides_bytes,
                            const uint32_t *box, int swizzle, int l2_promotion);

/* ---- external modules: the reference's drop-in door ------------------------------------------- */

/* `LaunchConfig` (crates/gpurs/src/host/stream.rs:28-52) plus the cluster dimension the driver crate
 * already models (crates/driver/src/launch.rs:21,43-49) but the reference's raw launch never sets
 * (crates/gpurs/src/raw/module.rs:195). */
typedef struct gpurs_launch_config {
    uint32_t grid[3];
    uint32_t block[3];
    uint32_t shared_bytes;
    uint32_t cluster[3]; /* all zero or all one: no cluster attribute */
} gpurs_launch_config;

/* `Gpu::load_module` / `Module::kernel` / `Kernel::reserve_shared` / `Kernel::launch`
 * (crates/gpurs/src/raw/module.rs:64-67,86-92,143-146,158-207).  `params` is the driver's
 * array-of-pointers form (crates/driver/src/launch.rs:83-110). */
int gpurs_module_load(gpurs_gpu *gpu, const void *image, size_t bytes, gpurs_module **out);
void gpurs_module_free(gpurs_module *module);
int gpurs_module_kernel(gpurs_module *module, const char *name, gpurs_kernel **out);
int gpurs_kernel_reserve_shared(gpurs_kernel *kernel, uint32_t bytes);
int gpurs_kernel_registers(gpurs_kernel *kernel, int *registers);
int gpurs_kernel_launch(gpurs_kernel *kernel, gpurs_stream *stream, const gpurs_launch_config *config, void **params);
/* The sm_100a kernel image built into this library, for hosts that prefer to load it through their
 * own module path (the reference's `Gpu::load_module(&[u8])`). */
const void *gpurs_kernel_image(size_t *bytes);

/* ---- the matrix multiply --------------------------------------------------------------------- */

/* Tile / algorithm choice.  AUTO is what a caller should use. */
enum {
    GPURS_ALGO_AUTO = 0,
    GPURS_ALGO_SINGLE_CTA = 1,  /* 128 x 256 tiles, one CTA per tile (tcgen05 cta_group::1) */
    GPURS_ALGO_CTA_PAIR = 2,    /* 256 x 256 tiles shared by a 2-CTA cluster (tcgen05 cta_group::2) */
    GPURS_ALGO_SKINNY = 3,      /* m <= 64, 16-bit operands, fp32 output: B fills the tensor core's rows, K is split among CTAs
                                   and the splits add in order (the reference's SplitDepth + TileLock); AUTO picks it */
    /* Flags, or-ed to one of the above.  By default, when the tile count leaves the last round of the persistent grid
     * idle enough to pay for it (and at least one whole round precedes it), the dense tile kernels split the K-blocks of
     * that round's tiles over the grid and add the parts up in a fixed order ("stream-K", the reference's
     * schedule/stream.rs): faster, deterministic for a given shape, but the low bits of a floating-point result then
     * depend on the shape.  WHOLE_TILES: every tile is multiplied whole by one CTA or CTA pair.  SPLIT_LAST_ROUND: the
     * last round is split whenever it is not full, whether or not that pays. */
    GPURS_ALGO_WHOLE_TILES = 0x100,
    GPURS_ALGO_SPLIT_LAST_ROUND = 0x200,
    /* CTA-pair tiles are 256 x 256 or, for plain products whose tile count fills the grid well that way, 256 x 512 (a quarter less
     * operand traffic from L2 per flop, which is what bounds the 256 x 256 tiles).  WIDE_TILES: 256 x 512 wherever that kernel
     * can run at all; SQUARE_TILES: never.  A 2:4-sparse product has the same choice between its 256 x 224 and 512 x 224 pair
     * tiles (the right operand fetched once for two row blocks).  The result does not depend on the choice. */
    GPURS_ALGO_WIDE_TILES = 0x400,
    GPURS_ALGO_SQUARE_TILES = 0x800,
    /* gpurs_matmul_allgather only: multiply the block in bands of rows with the plain kernels and send every finished band to
     * the other GPUs with the copy engines (one helper stream per peer) while the next band is multiplied, instead of storing
     * to all GPUs from the product's epilogue.  The call is stream-ordered as always: work enqueued on `stream` after it sees
     * this GPU's copies sent.  This form takes every single product gpurs_matmul takes (the epilogue form has kernels for four
     * type pairs). */
    GPURS_ALGO_GATHER_BY_COPIES = 0x1000
};

/* What the scale arrays of an E4M3 product hold. */
enum {
    GPURS_SCALES_FP32_BLOCKS = 0,    /* fp32, one per 1 x 128 block of A and per 128 x 128 block of B (promoted every K-block in registers) */
    GPURS_SCALES_MX = 1              /* power-of-two (UE8M0) bytes, one per 32 elements of K of every row of A and of B, in the tiled order
                                        gpurs_quantize_mx_e4m3 writes: applied by the tensor core itself (kind::mxf8f6f4.block_scale),
                                        k a multiple of 128, n x k right operand */
};

/* How fp32 operands are multiplied.  The tensor cores take TF32 (10-bit mantissa) inputs. */
enum {
    GPURS_PRECISION_DEFAULT = 0, /* fp32 operands: three TF32 passes over a hi/lo split, about 2^-21 relative */
    GPURS_PRECISION_TF32 = 1     /* fp32 operands: one TF32 pass, what the reference's `f32` tensor element
                                    does (crates/gpurs/src/gpu/tensor/element.rs:75-110); about 2^-11 relative */
};

/* C[m, n] = sum_k A[m, k] * B[n, k]: A is m x k, B is n x k ("right_transposed",
 * examples/blackwell/examples/blackwell_matrix.rs:35,64), C is m x n, all row-major.  A zeroed
 * descriptor with the three types and m, n, k set describes the dense contiguous case. */
typedef struct gpurs_matmul_desc {
    int32_t a_type;   /* element type of A and of B: GPURS_F16, GPURS_BF16, GPURS_F32, GPURS_I8, GPURS_E4M3 */
    int32_t c_type;   /* GPURS_F32, GPURS_BF16, GPURS_F16 (float inputs) or GPURS_I32 (GPURS_I8 inputs) */
    uint64_t m, n, k;
    uint64_t lda, ldb, ldc;          /* row pitches in elements; 0 = contiguous (k, k, n) */
    uint64_t a_len, b_len, c_len;    /* slice lengths in elements for the bounds check; 0 = not checked */
    int32_t algorithm;               /* GPURS_ALGO_* */
    int32_t max_ctas;                /* upper bound on resident CTAs (0 = one per multiprocessor) */
    int32_t precision;               /* GPURS_PRECISION_* (fp32 operands only) */
    int32_t raster_rows;             /* tile rows walked together for L2 reuse (0 = library default) */
    gpurs_device_ptr scale_a;        /* GPURS_E4M3 block-scaled: fp32 [m][ceil(k/128)], else 0 */
    gpurs_device_ptr scale_b;        /* GPURS_E4M3 block-scaled: fp32 [ceil(n/128)][ceil(k/128)], else 0 */
    gpurs_device_ptr metadata;       /* 2:4-sparse A (GPURS_F16 / GPURS_BF16): the metadata from gpurs_compress_24; then `a`
                                        is the m x k/2 array of kept values, k stays the logical depth (a multiple of
                                        128), lda counts kept values (0 = k/2).  0 = dense A */
    int32_t l2_policy;               /* L2 residency hint of the operand loads (dense kernels): 0 library default,
                                        1 keep A / stream B, 2 stream A / keep B, 3 keep both, 4 no hints */
    int32_t b_row_major;             /* 0: B is n x k, k contiguous (the reference's "right_transposed" operand); 1: B is k x n,
                                        n contiguous (C = A * B with all three row-major), ldb >= n.  The dense 16-bit and 8-bit
                                        tile kernels read it in place and the full-precision fp32 product transposes it while
                                        splitting it; the other kernels (2:4-sparse, scaled FP8, one-pass TF32) get a transposed
                                        copy in the handle's workspace first (one more launch; k * element size a multiple of
                                        16 bytes; single products, not the gathering one) */
    gpurs_device_ptr bias;           /* optional fp32 [n] added to every row of C before the output rounding (float outputs;
                                        the epilogue of the reference's skinny example, examples/ada/examples/skinny_matrix.rs:60-64) */
    /* More epilogue algebra for float outputs, the steps the reference offers on accumulator tiles (`scale`, `scale_rows`,
     * `scale_columns`, crates/gpurs/src/gpu/tensor/warp/accumulators.rs:86-110).  Applied before the bias and the output
     * rounding: C = acc * alpha * row_scale[row] * column_scale[column] + bias[column].  Tile kernels only (a product with
     * any of the three does not take the split-K path). */
    gpurs_device_ptr row_scale;      /* optional fp32 [m], e.g. a per-token activation scale */
    gpurs_device_ptr column_scale;   /* optional fp32 [n], e.g. a per-channel weight scale */
    float alpha;                     /* scalar factor; 0 is read as 1, so that a zeroed descriptor scales by nothing */
    /* A batch of products of one shape, C[i] = A[i] * B[i]^T for i < batches, as ONE launch whose persistent grid walks the
     * tiles of all matrices (`OutputMatrix::batched` + `Tile::batch`, crates/gpurs/src/gpu/tensor/output/matrix.rs:94-99,
     * schedule/grid.rs:57-66).  Matrix i of each operand starts stride_* elements after matrix i - 1; 0 = packed (m * lda,
     * n * ldb, m * ldc).  Dense f16 / bf16 operands on the tile kernels; strides must keep every matrix 16-byte aligned.
     * bias, row_scale and column_scale, if given, apply to every matrix alike; a_len / b_len / c_len cover the whole batch. */
    int32_t batches;                 /* 0 or 1 = a single product */
    uint64_t stride_a, stride_b, stride_c;
    /* Row reduction of the result (`reduce_rows` on the reference's accumulator tiles, warp/accumulators.rs:112-128, with
     * max |.| as the operation): fp32 [m], folded in with an atomic max of |C[row, :]| taken after the algebra above and
     * before the output rounding.  The caller zeroes the array first; it may be folded into by several products.  What a
     * per-row quantiser of C needs without reading C again.  Dense tile kernels, float outputs, single products. */
    gpurs_device_ptr row_absmax;
    int32_t scale_kind;              /* what scale_a / scale_b hold: GPURS_SCALES_* */
    /* 1: the product is ADDED to what C holds instead of replacing it, with atomic adds, so that several products (for
     * instance the parts of a depth split across launches or streams) may add into one C at once: `accumulate` of the
     * reference's f32 output matrix (`red.global.add.f32`, crates/gpurs/src/gpu/tensor/output/reduction.rs:157-202).  fp32
     * output only; single products on the tile kernels.  The order of the additions, and so the last bits, is not fixed. */
    int32_t accumulate;
    /* The rest of the accumulator-tile algebra of the reference (`add_rows`, and `add` of another tile,
     * crates/gpurs/src/gpu/tensor/warp/accumulators.rs:82-105), applied after the bias, each step rounded on its own:
     *     C = acc * alpha * row_scale[row] * column_scale[column] + bias[column] + row_bias[row] + beta * residual[row, column] */
    gpurs_device_ptr row_bias;       /* optional fp32 [m]: one value added to every element of its row */
    gpurs_device_ptr residual;       /* optional m x n matrix of C's element type: a skip connection, or beta * C_in when it is C
                                        itself (then ldr must equal ldc); otherwise it must not overlap C.  Single products. */
    uint64_t ldr;                    /* its row pitch in elements; 0 = n */
    float beta;                      /* factor of the residual; 0 is read as 1 */
    int32_t reserved;                /* 0 */
    /* `reduce_rows` with + (warp/accumulators.rs:112-128): fp32 [m], zeroed by the caller; the sum of each row of the
     * result (after the algebra, before the output rounding) is added in with one atomic add per row and tile, so the
     * last bits depend on the order the tiles finish in.  Dense tile kernels, float outputs, single products. */
    gpurs_device_ptr row_sum;
    /* An explicit launch geometry, as `stream.launch(LaunchConfig)` gives a launcher in the reference
     * (crates/gpurs/src/host/stream.rs:28-52,142-148), or NULL to let the library pick.  The kernels are persistent, so the
     * grid says how many CTAs walk the tiles: grid[0] * grid[1] * grid[2] CTAs (a multiple of the cluster size, at most one
     * per multiprocessor is useful).  cluster[0] 1 or 2 picks one-CTA or CTA-pair tiles when `algorithm` is AUTO and must
     * agree with it otherwise (0 = no say).  block[0], if not 0, must be the thread count of the kernel that will run, and
     * shared_bytes, if not 0, at least what it needs: a mismatch is GPURS_E_INVALID_VIEW and nothing is launched.
     * Tile kernels only (the split-K decode kernel sizes its own grid). */
    const gpurs_launch_config *launch;
} gpurs_matmul_desc;

/* The launcher behind `matmul(&stream, &a, &b, &mut c, ...)`.  It validates like the reference's
 * generated launchers do before submitting (lengths, views, aliasing:
 * crates/gpurs/src/host/launch/kernel.rs:178-255,322-355), encodes the TMA descriptors
 * (crates/gpurs/src/host/argument/tensor_map.rs:24-60), and enqueues one kernel on `stream`.
 * It does not wait. */
int gpurs_matmul(gpurs_stream *stream, const gpurs_matmul_desc *desc, gpurs_device_ptr a, gpurs_device_ptr b,
                 gpurs_device_ptr c);

/* The same product with operands and result in HOST memory, staged through the caller's device buffers a, b, c (sized
 * and pitched exactly like the host arrays): what the reference's example writes as upload, upload, zeros, launch,
 * download (examples/blackwell/examples/blackwell_matrix.rs:58-83), as one call that overlaps the three.  The smaller
 * operand is copied first, then the larger one in blocks (rows of A, or rows of B = columns of C); every block is
 * multiplied as soon as it has arrived, and its part of C travels back while the next block is still on its way, so the
 * call costs about the longer transfer direction instead of both plus the product.  Rows at a pitch are copied row by
 * row: bytes between rows are left alone in host and device memory.  Copies run on two streams of the handle, tied to `stream` by events: everything is ordered after
 * the work already on `stream`, and `stream` continues after the last copy; the call does not wait.  The host arrays
 * must stay valid until then and should be page-locked (gpurs_host_alloc), or the copies do not overlap.  Scales and
 * bias in `desc` are device-resident as for gpurs_matmul; a 2:4-sparse operand is not accepted (it is prepared on the
 * device).  a_len / b_len / c_len of `desc` are ignored. */
int gpurs_matmul_host(gpurs_stream *stream, const gpurs_matmul_desc *desc, const void *host_a, const void *host_b, void *host_c,
                      gpurs_device_ptr a, gpurs_device_ptr b, gpurs_device_ptr c);

/* ---- FP8 block quantisation ------------------------------------------------------------------------ */

/* Quantises a row-major rows x k fp32 matrix (pitch `ld` elements, 0 = k; k a multiple of 4) to E4M3 with one fp32
 * scale per block of block_rows x 128 elements, block_rows = 1 (left operand) or 128 (right operand): scale =
 * absmax / 448 (1 for an all-zero block), code = E4M3(x / scale), round to nearest even with saturation — the host
 * conversion of the reference (crates/gpurs/src/gpu/float8.rs:20-52); the reference has no block quantiser.
 * `codes` receives rows x k bytes, `scales` [ceil(rows / block_rows)][ceil(k / 128)] floats: the operand and scale
 * layout gpurs_matmul takes for GPURS_E4M3 with scales. */
int gpurs_quantize_e4m3(gpurs_stream *stream, uint64_t rows, uint64_t k, gpurs_device_ptr source, uint64_t ld, uint32_t block_rows,
                        gpurs_device_ptr codes, gpurs_device_ptr scales);

/* MX quantiser (no counterpart in the reference): fp32 rows x k (pitch `ld`, 0 = k; k a multiple of 4) -> E4M3 codes
 * (rows x k bytes) and one power-of-two scale per 32 elements of a row: the smallest power of two that brings the group's
 * largest magnitude to 448 or below (1 for an all-zero group), stored as its biased exponent (UE8M0).  `scales` receives
 * gpurs_mx_scale_bytes(rows, k, right_operand) bytes in the order the MX-scaled product reads them: 512-byte blocks of 128
 * rows x 128 K, inside a block the scale of row r and group g at byte (r % 32) * 16 + (r / 32) * 4 + g; the left operand's
 * blocks ordered [row / 128][k / 128], the right operand's by the product's 224-row tiles, [row / 224][k / 128][2] (rows
 * 0..127 and 128..223 of the tile).  Entries no element maps to are set to 127 (scale 1). */
size_t gpurs_mx_scale_bytes(uint64_t rows, uint64_t k, int right_operand);
int gpurs_quantize_mx_e4m3(gpurs_stream *stream, uint64_t rows, uint64_t k, gpurs_device_ptr source, uint64_t ld, int right_operand,
                           gpurs_device_ptr codes, gpurs_device_ptr scales);

/* ---- 2:4 structured sparsity (no counterpart in the reference, which has no sparse path) ---------- */

/* Bytes of metadata gpurs_compress_24 writes for an m x k matrix: one 2048-byte block per 128 rows x 128 K. */
size_t gpurs_metadata_bytes(uint64_t m, uint64_t k);

/* Compresses a row-major m x k matrix of GPURS_F16 / GPURS_BF16 with at most two non-zeros in every aligned
 * group of four along k (pitch `ld` elements, 0 = k; k a multiple of 128): `values` receives the m x k/2 kept
 * elements, `metadata` their positions in the layout the sparse kernels read.  `violations`, if not 0, points
 * to a u32 on the device that is incremented by the number of groups holding more than two non-zeros. */
int gpurs_compress_24(gpurs_stream *stream, int element_type, uint64_t m, uint64_t k, gpurs_device_ptr dense, uint64_t ld,
                      gpurs_device_ptr values, gpurs_device_ptr metadata, gpurs_device_ptr violations);

/* Size of the fixed device array behind gpurs_matmul_f32_static.  Every GPU that loads this library
 * holds this much memory for it until the process exits. */
#define GPURS_STATIC_SCRATCH_BYTES (32u << 20)

/* No counterpart in the reference.  The fp32 product C[m, n] = sum_k A[m, k] * B[n, k] (contiguous
 * row-major fp32 A m x k, B n x k, C m x n; same arithmetic as gpurs_matmul with GPURS_F32 operands and
 * GPURS_PRECISION_DEFAULT) for hosts that must not allocate device memory when they call: ones whose
 * whole device is owned by their own pool, and ones that cannot take the device-wide synchronisation an
 * allocation or a free implies.  The scratch for the split operands is a fixed array inside the library
 * image instead of an allocation, so (m + n) * 3 * k * 4 bytes (the A part rounded up to 256) must fit
 * GPURS_STATIC_SCRATCH_BYTES, else GPURS_E_SIZE_OVERFLOW.  All calls on a device share that array: calls
 * ordered by one stream are safe, calls that may overlap on the GPU race.  Every call looks the array's
 * device address up afresh (a host-side lookup, nothing is allocated), so closing and reopening a handle
 * is safe; the first call on a device also loads the kernels: make it before starting any stream capture. */
int gpurs_matmul_f32_static(gpurs_stream *stream, uint64_t m, uint64_t n, uint64_t k, gpurs_device_ptr a,
                            gpurs_device_ptr b, gpurs_device_ptr c);

/* ---- grouped (mixture-of-experts) product ----------------------------------------------------------- */

/* output[r, :] = input[routes[r], :] * weight[e]^T for offsets[e] <= r < offsets[e + 1]: the reference's `experts`
 * example (examples/ada/examples/grouped_matrix.rs:30-60).  input is tokens x k, weight [experts][n][k] (k contiguous),
 * output rows x n, all row-major; routes (u32 [rows]) and offsets (u32 [experts + 1], ascending, offsets[experts] <= rows)
 * live on the device.  Route values beyond tokens - 1 are clamped. */
typedef struct gpurs_grouped_desc {
    int32_t a_type;       /* GPURS_F16 or GPURS_BF16 (input and weight) */
    int32_t c_type;       /* the same 16-bit type, or GPURS_F32 */
    uint64_t rows, tokens, n, k, experts;
    uint64_t lda, ldc;    /* row pitches of input and output in elements; 0 = contiguous */
} gpurs_grouped_desc;

int gpurs_matmul_grouped(gpurs_stream *stream, const gpurs_grouped_desc *desc, gpurs_device_ptr input, gpurs_device_ptr routes,
                         gpurs_device_ptr offsets, gpurs_device_ptr weight, gpurs_device_ptr output);

/* ---- product whose result every GPU of the box receives ---------------------------------------------- */

/* No counterpart in the reference, which drives one GPU.  The M-sharded product of a box of GPUs followed by the
 * all-gather of C, as one kernel per GPU instead of a kernel and a collective.  Each GPU multiplies its block of rows of A by the replicated B and stores every finished 32-row box of C into the
 * block's place in the copy of the whole matrix that EVERY GPU keeps: the local copy through L2, the remote ones as
 * plain stores over NVLink, while the tensor cores work on the next tile.  No kernel waits on another GPU; when the
 * calls of all ranks have completed (each rank synchronises its stream, then the ranks meet at a host barrier), every
 * copy holds the whole matrix.
 *   full[t]  the gathered matrix (total_rows x n, pitch ld_full) on GPU t as an address valid in THIS process: the
 *            rank's own allocation for t == rank, gpurs_ipc_open of the owner's handle otherwise (peers of one box).
 * `desc` describes the local product as for gpurs_matmul (m = rows of this block; ldc 0 or ld_full; c_len ignored).
 * Supported: dense bf16->bf16, f16->f32, i8->i32, unscaled e4m3->bf16, and 2:4-sparse bf16->bf16 (desc.metadata set); bases and pitches of the gathered matrices
 * multiples of 16 bytes; every block but the last a multiple of 32 rows. */
typedef struct gpurs_gather_desc {
    uint32_t world;              /* GPUs that receive the result, 1..8 */
    uint32_t rank;               /* the one this call runs on */
    uint64_t row_offset;         /* first row of this call's block within the gathered matrix */
    uint64_t total_rows;         /* rows of the gathered matrix */
    uint64_t ld_full;            /* its row pitch in elements; 0 = n */
    gpurs_device_ptr full[8];
} gpurs_gather_desc;

int gpurs_matmul_allgather(gpurs_stream *stream, const gpurs_matmul_desc *desc, const gpurs_gather_desc *gather,
                           gpurs_device_ptr a, gpurs_device_ptr b);

/* ---- the optional all-gather of C as a plain collective ------------------------------------------------ */

/* No counterpart in the reference (one device, no collective: crates/gpurs/src/lib.rs:7-9).  After an M-sharded product
 * every GPU of the box holds its block of rows of C; these three calls make every GPU hold all of C with one NCCL
 * all-gather over NVLink, the baseline that gpurs_matmul_allgather (above) fuses into the product.  One communicator per
 * GPU and process (or thread).  How the 128-byte id travels from the rank that made it to the others is the host's
 * business (a file, a socket, any process group): gpurs_comm_unique_id on one rank, the same bytes to gpurs_comm_init on
 * all `world` ranks, which meet inside that call.
 * gpurs_comm_allgather is in place and stream-ordered: `full` is this rank's buffer of world * block_bytes bytes whose
 * block [rank * block_bytes, (rank + 1) * block_bytes) already holds this rank's rows (the product was written there);
 * when the call has completed on `stream`, block r holds rank r's rows.  Every rank must make the call, with the same
 * block_bytes.  Free the communicator on every rank after the last collective has completed. */
#define GPURS_COMM_ID_BYTES 128
typedef struct gpurs_comm gpurs_comm;
int gpurs_comm_unique_id(uint8_t id[GPURS_COMM_ID_BYTES]);
int gpurs_comm_init(gpurs_gpu *gpu, const uint8_t id[GPURS_COMM_ID_BYTES], uint32_t world, uint32_t rank, gpurs_comm **out);
int gpurs_comm_allgather(gpurs_comm *comm, gpurs_stream *stream, gpurs_device_ptr full, uint64_t block_bytes);
void gpurs_comm_free(gpurs_comm *comm);

/* Reads and clears the device status word: [0] code (0 = none), [1] block, [2] tile, [3] K-block of the
 * first bounded wait that gave up.  Synchronises the device. */
int gpurs_status_read(gpurs_gpu *gpu, uint32_t status[4]);

/* Self-test of the bounded device waits (no counterpart in the reference, whose device waits are unbounded): enqueues a
 * one-warp kernel whose wait can never be satisfied.  After about 1.5 s the wait gives up, the kernel records status code 4
 * and returns; the next gpurs_stream_synchronize reports GPURS_E_DEVICE_TIMEOUT and the context stays usable. */
int gpurs_self_test_timeout(gpurs_stream *stream);

/* Number of kernels this library has launched through `gpu` so far. */
uint64_t gpurs_launch_count(gpurs_gpu *gpu);

/* Detail of the calling thread's most recent failure: the operation, the CUDA error name and its
 * description (`driver::Error`, crates/driver/src/error.rs:8-16).  Pointers stay valid until the
 * thread's next failing call. */
int gpurs_last_error(const char **operation, const char **name, const char **description);

#if defined(__GNUC__)
#pragma GCC visibility pop
#endif
#ifdef __cplusplus
}
#endif
#endif /* GPURS_B200_H */
