"""gpurs_b200: the dense matrix-multiply path of gpurs, rebuilt for NVIDIA B200 (sm_100a).

The product is the C-ABI library `libgpurs_b200.so` (declared in include/gpurs_b200.h) and the CUDA
kernels embedded in it; this package is the Python mirror of the reference's host surface over that
ABI, used by the tests and the benchmark.
"""
from ._ffi import ALGO_AUTO, ALGO_CTA_PAIR, ALGO_SINGLE_CTA, ALGO_SKINNY, ALGO_SPLIT_LAST_ROUND, ALGO_WHOLE_TILES, ALGO_WIDE_TILES, ALGO_SQUARE_TILES, ALGO_GATHER_BY_COPIES, PRECISION_DEFAULT, PRECISION_TF32, SCALES_FP32_BLOCKS, SCALES_MX
from .host import (BF16, E4M3, F16, F32, I8, I32, DeviceBuffer, Event, Gpu, GpursError, Kernel, LaunchConfig,
                   MatmulOptions, Module, Stream, Communicator, comm_unique_id, GatheredMatrix, Graph, GraphExec, compress_24, matmul, matmul_allgather, matmul_host, matmul_grouped, quantize_e4m3, quantize_mx_e4m3)

__all__ = [
    "ALGO_AUTO", "ALGO_CTA_PAIR", "ALGO_SINGLE_CTA", "ALGO_SKINNY", "ALGO_SPLIT_LAST_ROUND", "ALGO_WHOLE_TILES", "ALGO_WIDE_TILES", "ALGO_SQUARE_TILES", "ALGO_GATHER_BY_COPIES", "PRECISION_DEFAULT", "PRECISION_TF32", "SCALES_FP32_BLOCKS", "SCALES_MX", "quantize_mx_e4m3", "BF16", "E4M3", "F16", "F32", "I8", "I32", "DeviceBuffer", "Event",
    "Gpu", "GpursError", "Communicator", "comm_unique_id", "GatheredMatrix", "Graph", "GraphExec", "compress_24", "matmul_allgather", "matmul_host", "matmul_grouped", "quantize_e4m3", "Kernel", "LaunchConfig", "MatmulOptions", "Module", "Stream", "matmul",
]
