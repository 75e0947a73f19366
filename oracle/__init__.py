"""numpy front end of the CPU oracle (oracle/gpurs_oracle.c).  TEST INFRASTRUCTURE ONLY.

Only the test-suite, the smoke check and the CPU-baseline / reference legs of the benchmark may import
this package; the shipped library never does.  `make -C oracle` builds the shared object.
"""
from __future__ import annotations

import ctypes as C
import subprocess
from pathlib import Path

import numpy as np

HERE = Path(__file__).resolve().parent
LIBRARY_PATH = HERE / "libgpurs_oracle.so"

FMT_F16, FMT_BF16, FMT_F32, FMT_I8, FMT_E4M3 = 0, 1, 2, 3, 4
_STORAGE = {FMT_F16: np.uint16, FMT_BF16: np.uint16, FMT_F32: np.float32, FMT_I8: np.int8, FMT_E4M3: np.uint8}

_library = None


def build() -> Path:
    subprocess.run(["make", "-C", str(HERE)], check=True, capture_output=True)
    return LIBRARY_PATH


def lib() -> C.CDLL:
    global _library
    if _library is None:
        if not LIBRARY_PATH.exists():
            build()
        L = C.CDLL(str(LIBRARY_PATH))
        L.gpurs_oracle_f16_from_f32.restype = C.c_uint16
        L.gpurs_oracle_f16_from_f32.argtypes = [C.c_float]
        L.gpurs_oracle_f16_to_f32.restype = C.c_float
        L.gpurs_oracle_f16_to_f32.argtypes = [C.c_uint16]
        L.gpurs_oracle_bf16_from_f32.restype = C.c_uint16
        L.gpurs_oracle_bf16_from_f32.argtypes = [C.c_float]
        L.gpurs_oracle_bf16_to_f32.restype = C.c_float
        L.gpurs_oracle_bf16_to_f32.argtypes = [C.c_uint16]
        L.gpurs_oracle_e4m3_from_f32.restype = C.c_uint8
        L.gpurs_oracle_e4m3_from_f32.argtypes = [C.c_float]
        L.gpurs_oracle_e4m3_to_f32.restype = C.c_float
        L.gpurs_oracle_e4m3_to_f32.argtypes = [C.c_uint8]
        L.gpurs_oracle_tf32_from_f32.restype = C.c_uint32
        L.gpurs_oracle_tf32_from_f32.argtypes = [C.c_float]
        L.gpurs_oracle_compress_24.restype = C.c_size_t
        L.gpurs_oracle_threads.restype = C.c_int
        _library = L
    return _library


def _p(array: np.ndarray):
    return C.c_void_p(array.ctypes.data)


def _convert(name: str, source: np.ndarray, out_dtype) -> np.ndarray:
    source = np.ascontiguousarray(source)
    out = np.empty(source.shape, dtype=out_dtype)
    getattr(lib(), name)(_p(source), _p(out), C.c_size_t(source.size))
    return out


def f16_from_f32(x): return _convert("gpurs_oracle_f16_from_f32_n", np.asarray(x, np.float32), np.uint16)
def f16_to_f32(x): return _convert("gpurs_oracle_f16_to_f32_n", np.asarray(x, np.uint16), np.float32)
def bf16_from_f32(x): return _convert("gpurs_oracle_bf16_from_f32_n", np.asarray(x, np.float32), np.uint16)
def bf16_to_f32(x): return _convert("gpurs_oracle_bf16_to_f32_n", np.asarray(x, np.uint16), np.float32)
def e4m3_from_f32(x): return _convert("gpurs_oracle_e4m3_from_f32_n", np.asarray(x, np.float32), np.uint8)
def e4m3_to_f32(x): return _convert("gpurs_oracle_e4m3_to_f32_n", np.asarray(x, np.uint8), np.float32)
def tf32_from_f32(x): return _convert("gpurs_oracle_tf32_from_f32_n", np.asarray(x, np.float32), np.uint32)


def decode(fmt: int, bits: np.ndarray) -> np.ndarray:
    """Values of a stored array as float64."""
    if fmt == FMT_F16: return f16_to_f32(bits).astype(np.float64)
    if fmt == FMT_BF16: return bf16_to_f32(bits).astype(np.float64)
    if fmt == FMT_E4M3: return e4m3_to_f32(bits).astype(np.float64)
    return np.asarray(bits).astype(np.float64)


def example_inputs(fmt: int, count: int):
    """The reference example's two operands (examples/matrix_benchmark.rs:5-14) as bit patterns."""
    left, right = np.empty(count, np.uint16), np.empty(count, np.uint16)
    lib().gpurs_oracle_example_inputs(C.c_int(fmt), C.c_size_t(count), _p(left), _p(right))
    return left, right


def fill_uniform_f32(count: int, seed: int) -> np.ndarray:
    out = np.empty(count, np.float32)
    lib().gpurs_oracle_fill_uniform_f32(_p(out), C.c_size_t(count), C.c_uint64(seed))
    return out


def fill_normal_f32(count: int, seed: int) -> np.ndarray:
    out = np.empty(count, np.float32)
    lib().gpurs_oracle_fill_normal_f32(_p(out), C.c_size_t(count), C.c_uint64(seed))
    return out


def fill_normal_16(fmt: int, count: int, seed: int) -> np.ndarray:
    out = np.empty(count, np.uint16)
    lib().gpurs_oracle_fill_normal_16(C.c_int(fmt), _p(out), C.c_size_t(count), C.c_uint64(seed))
    return out


def fill_int8(count: int, seed: int) -> np.ndarray:
    out = np.empty(count, np.int8)
    lib().gpurs_oracle_fill_int8(_p(out), C.c_size_t(count), C.c_uint64(seed))
    return out


def fill_sparse24_bf16(rows: int, columns: int, seed: int) -> np.ndarray:
    out = np.empty(rows * columns, np.uint16)
    lib().gpurs_oracle_fill_sparse24_bf16(_p(out), C.c_size_t(rows), C.c_size_t(columns), C.c_uint64(seed))
    return out


def quantize_e4m3(source: np.ndarray, rows: int, depth: int, block_rows: int):
    """(codes, scales) of a rows x depth fp32 matrix, one scale per block_rows x 128 block."""
    source = np.ascontiguousarray(source, np.float32)
    codes = np.empty(rows * depth, np.uint8)
    scales = np.empty(((rows + block_rows - 1) // block_rows) * ((depth + 127) // 128), np.float32)
    lib().gpurs_oracle_quantize_e4m3(_p(source), C.c_size_t(rows), C.c_size_t(depth), C.c_size_t(block_rows), _p(codes), _p(scales))
    return codes, scales


MX_TILE_ROWS = 224     # rows of the right operand per tile of the MX-scaled product


def quantize_mx_e4m3(source: np.ndarray, rows: int, depth: int):
    """MX quantisation (numpy restatement of the definition the library's header gives; the reference has no block
    quantiser, its E4M3 conversion is crates/gpurs/src/gpu/float8.rs:20-52): per 32 elements of a row the smallest
    power of two 2^e with absmax / 2^e <= 448 (e = 0 for an all-zero group), codes = E4M3(x / 2^e).  Returns (codes
    uint8 [rows * depth], exponents int [rows, depth / 32])."""
    x = np.asarray(source, np.float32).reshape(rows, depth // 32, 32)
    absmax = np.abs(x).max(axis=2).astype(np.float64)
    with np.errstate(divide="ignore"):
        exponents = np.where(absmax > 0, np.ceil(np.log2(absmax / 448.0)), 0.0).astype(np.int64)
    # log2 in floating point can be off by one ulp at exact powers of two: settle by the definition itself
    exponents = np.where((absmax > 0) & (absmax / np.exp2(exponents - 1.0) <= 448.0), exponents - 1, exponents)
    exponents = np.where((absmax > 0) & (absmax / np.exp2(exponents.astype(np.float64)) > 448.0), exponents + 1, exponents)
    exponents = np.clip(exponents, -127, 127)
    scaled = (x.astype(np.float64) / np.exp2(exponents.astype(np.float64))[:, :, None]).astype(np.float32)   # exact: a power of two
    return e4m3_from_f32(scaled.reshape(-1)), exponents


def mx_scale_index(right_operand: bool, row, k, k_blocks: int):
    """Byte index of the scale of element (row, k) in the tiled scale array of the left or right operand."""
    row, k = np.asarray(row, np.int64), np.asarray(k, np.int64)
    inside_block = lambda r: (r % 32) * 16 + ((r // 32) % 4) * 4 + (k // 32) % 4
    if not right_operand:
        return ((row // 128) * k_blocks + k // 128) * 512 + inside_block(row % 128)
    inside = row % MX_TILE_ROWS
    return (((row // MX_TILE_ROWS) * k_blocks + k // 128) * 2 + inside // 128) * 512 + inside_block(inside % 128)


def mx_tile_scales(exponents: np.ndarray, right_operand: bool) -> np.ndarray:
    """The exponents [rows, depth / 32] as the tiled array of UE8M0 bytes (unused entries 127)."""
    rows, groups = exponents.shape
    k_blocks = -(-groups // 4)
    size = (-(-rows // MX_TILE_ROWS) * k_blocks * 1024) if right_operand else (-(-rows // 128) * k_blocks * 512)
    tiled = np.full(size, 127, np.uint8)
    r, g = np.meshgrid(np.arange(rows), np.arange(groups), indexing="ij")
    tiled[mx_scale_index(right_operand, r, g * 32, k_blocks)] = (exponents + 127).astype(np.uint8)
    return tiled


def mx_dequantize(codes: np.ndarray, exponents: np.ndarray, rows: int, depth: int) -> np.ndarray:
    """codes * 2^e as fp64 [rows, depth]."""
    values = e4m3_to_f32(codes).astype(np.float64).reshape(rows, depth // 32, 32)
    return (values * np.exp2(exponents.astype(np.float64))[:, :, None]).reshape(rows, depth)


def compress_24(dense: np.ndarray, rows: int, depth: int):
    dense = np.ascontiguousarray(dense, np.uint16)
    values = np.empty(rows * depth // 2, np.uint16)
    indices = np.empty(rows * depth // 4, np.uint8)
    violations = lib().gpurs_oracle_compress_24(_p(dense), C.c_size_t(rows), C.c_size_t(depth), _p(values), _p(indices))
    return values, indices, int(violations)


def _scales(left_scales, right_scales):
    if left_scales is None:
        return None, None, C.c_void_p(0), C.c_void_p(0)
    ls = np.ascontiguousarray(left_scales, np.float32)
    rs = np.ascontiguousarray(right_scales, np.float32)
    return ls, rs, _p(ls), _p(rs)


def matmul_rows(fmt: int, left, right, columns: int, depth: int, rows, left_scales=None, right_scales=None) -> np.ndarray:
    """fp64 C[r, :] for the listed rows: the reference's check loop (examples/matrix_benchmark.rs:40-45)."""
    left = np.ascontiguousarray(left, _STORAGE[fmt])
    right = np.ascontiguousarray(right, _STORAGE[fmt])
    rows = np.ascontiguousarray(rows, np.int64)
    out = np.empty((rows.size, columns), np.float64)
    ls, rs, lsp, rsp = _scales(left_scales, right_scales)
    lib().gpurs_oracle_matmul_rows(C.c_int(fmt), _p(left), _p(right), C.c_size_t(columns), C.c_size_t(depth), _p(rows),
                                   C.c_size_t(rows.size), lsp, rsp, _p(out))
    return out


def matmul_samples(fmt: int, left, right, columns: int, depth: int, indices, left_scales=None, right_scales=None) -> np.ndarray:
    """fp64 C.flat[i] for the listed flat indices (the sampled check, examples/matrix_benchmark.rs:36-39)."""
    left = np.ascontiguousarray(left, _STORAGE[fmt])
    right = np.ascontiguousarray(right, _STORAGE[fmt])
    indices = np.ascontiguousarray(indices, np.int64)
    out = np.empty(indices.size, np.float64)
    ls, rs, lsp, rsp = _scales(left_scales, right_scales)
    lib().gpurs_oracle_matmul_samples(C.c_int(fmt), _p(left), _p(right), C.c_size_t(columns), C.c_size_t(depth), _p(indices),
                                      C.c_size_t(indices.size), lsp, rsp, _p(out))
    return out


def matmul_rows_i8(left, right, columns: int, depth: int, rows) -> np.ndarray:
    left = np.ascontiguousarray(left, np.int8)
    right = np.ascontiguousarray(right, np.int8)
    rows = np.ascontiguousarray(rows, np.int64)
    out = np.empty((rows.size, columns), np.int64)
    lib().gpurs_oracle_matmul_rows_i8(_p(left), _p(right), C.c_size_t(columns), C.c_size_t(depth), _p(rows), C.c_size_t(rows.size), _p(out))
    return out


def reference_sample_indices(rows: int, columns: int) -> np.ndarray:
    """The output indices the reference's report samples: every (size^2 / 4093)-th, at least every one
    (examples/matrix_benchmark.rs:36-37)."""
    step = max(rows * columns // 4093, 1)
    return np.arange(0, rows * columns, step, dtype=np.int64)


def threads() -> int:
    return int(lib().gpurs_oracle_threads())


def set_threads(count: int) -> int:
    """Run the loops on `count` threads from now on (whatever OMP_NUM_THREADS said at start-up); returns the new count."""
    lib().gpurs_oracle_set_threads(C.c_int(int(count)))
    return threads()


def usable_cores() -> int:
    """Cores this process may run on (its affinity mask), which is what a timed CPU baseline should use."""
    import os

    try:
        return len(os.sched_getaffinity(0))
    except AttributeError:
        return os.cpu_count() or 1
