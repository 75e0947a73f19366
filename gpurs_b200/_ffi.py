"""ctypes binding of the C ABI declared in include/gpurs_b200.h.

The library is built in-tree by `python -m gpurs_b200.build`; importing this module never builds and
never falls back to anything else: without the library, `load()` raises.
"""
from __future__ import annotations

import ctypes as C
from pathlib import Path

LIBRARY_PATH = Path(__file__).resolve().parent / "libgpurs_b200.so"

# Result codes and element types of include/gpurs_b200.h.
OK = 0
E_CONTEXT_MISMATCH = 100001
E_SIZE_OVERFLOW = 100002
E_LENGTH_MISMATCH = 100003
E_OVERLAP = 100004
E_INVALID_VIEW = 100005
E_ALIASING = 100006
E_UNKNOWN_KERNEL = 100007
E_INCOMPATIBLE_DEVICE = 100008
E_INVALID_ARGUMENT = 100009
E_DEVICE_TIMEOUT = 100010
E_DRIVER_UNAVAILABLE = 100011
E_COLLECTIVE = 100012
COMM_ID_BYTES = 128

F16, F32, BF16, I8, I32, E4M3 = 6, 7, 9, 100, 101, 102
ALGO_AUTO, ALGO_SINGLE_CTA, ALGO_CTA_PAIR, ALGO_SKINNY = 0, 1, 2, 3
ALGO_WHOLE_TILES = 0x100   # flag: never split the last round's tiles along K
ALGO_SPLIT_LAST_ROUND = 0x200   # flag: split it whenever it is not full
ALGO_WIDE_TILES = 0x400   # flag: 256 x 512 pair tiles (2:4 sparse: 512 x 224) wherever possible
ALGO_GATHER_BY_COPIES = 0x1000   # flag, matmul_allgather only: bands of rows sent by the copy engines
ALGO_SQUARE_TILES = 0x800   # flag: never 256 x 512 (2:4 sparse: 512 x 224) tiles
PRECISION_DEFAULT, PRECISION_TF32 = 0, 1
SCALES_FP32_BLOCKS, SCALES_MX = 0, 1
STATIC_SCRATCH_BYTES = 32 << 20


class LaunchConfigStruct(C.Structure):
    _fields_ = [("grid", C.c_uint32 * 3), ("block", C.c_uint32 * 3), ("shared_bytes", C.c_uint32), ("cluster", C.c_uint32 * 3)]


class MatmulDesc(C.Structure):
    _fields_ = [
        ("a_type", C.c_int32), ("c_type", C.c_int32),
        ("m", C.c_uint64), ("n", C.c_uint64), ("k", C.c_uint64),
        ("lda", C.c_uint64), ("ldb", C.c_uint64), ("ldc", C.c_uint64),
        ("a_len", C.c_uint64), ("b_len", C.c_uint64), ("c_len", C.c_uint64),
        ("algorithm", C.c_int32), ("max_ctas", C.c_int32), ("precision", C.c_int32), ("raster_rows", C.c_int32),
        ("scale_a", C.c_uint64), ("scale_b", C.c_uint64), ("metadata", C.c_uint64),
        ("l2_policy", C.c_int32), ("b_row_major", C.c_int32), ("bias", C.c_uint64),
        ("row_scale", C.c_uint64), ("column_scale", C.c_uint64), ("alpha", C.c_float), ("batches", C.c_int32),
        ("stride_a", C.c_uint64), ("stride_b", C.c_uint64), ("stride_c", C.c_uint64), ("row_absmax", C.c_uint64),
        ("scale_kind", C.c_int32), ("accumulate", C.c_int32),
        ("row_bias", C.c_uint64), ("residual", C.c_uint64), ("ldr", C.c_uint64), ("beta", C.c_float), ("reserved", C.c_int32),
        ("row_sum", C.c_uint64), ("launch", C.POINTER(LaunchConfigStruct)),
    ]


class GroupedDesc(C.Structure):
    _fields_ = [("a_type", C.c_int32), ("c_type", C.c_int32), ("rows", C.c_uint64), ("tokens", C.c_uint64), ("n", C.c_uint64),
                ("k", C.c_uint64), ("experts", C.c_uint64), ("lda", C.c_uint64), ("ldc", C.c_uint64)]


class GatherDesc(C.Structure):
    _fields_ = [("world", C.c_uint32), ("rank", C.c_uint32), ("row_offset", C.c_uint64), ("total_rows", C.c_uint64),
                ("ld_full", C.c_uint64), ("full", C.c_uint64 * 8)]


_P = C.c_void_p
_PP = C.POINTER(C.c_void_p)
_U64P = C.POINTER(C.c_uint64)

# name -> (restype, argtypes): every function the header declares.
SIGNATURES = {
    "gpurs_gpu_new": (C.c_int, [C.c_int, _PP]),
    "gpurs_gpu_free": (None, [_P]),
    "gpurs_gpu_properties": (C.c_int, [_P, C.POINTER(C.c_int), C.POINTER(C.c_int), C.POINTER(C.c_int), C.POINTER(C.c_size_t)]),
    "gpurs_stream_new": (C.c_int, [_P, _PP]),
    "gpurs_stream_borrow": (C.c_int, [_P, _P, _PP]),
    "gpurs_stream_free": (None, [_P]),
    "gpurs_stream_raw": (_P, [_P]),
    "gpurs_stream_synchronize": (C.c_int, [_P]),
    "gpurs_event_record_timed": (C.c_int, [_P, _PP]),
    "gpurs_event_synchronize": (C.c_int, [_P]),
    "gpurs_event_elapsed_ms": (C.c_int, [_P, _P, C.POINTER(C.c_float)]),
    "gpurs_event_free": (None, [_P]),
    "gpurs_alloc": (C.c_int, [_P, C.c_size_t, _U64P]),
    "gpurs_free": (C.c_int, [_P, C.c_uint64]),
    "gpurs_upload": (C.c_int, [_P, _P, C.c_size_t, _U64P]),
    "gpurs_zeros": (C.c_int, [_P, C.c_size_t, _U64P]),
    "gpurs_download": (C.c_int, [_P, C.c_uint64, _P, C.c_size_t]),
    "gpurs_copy_to_device": (C.c_int, [_P, C.c_uint64, _P, C.c_size_t]),
    "gpurs_copy_to_host": (C.c_int, [_P, _P, C.c_uint64, C.c_size_t]),
    "gpurs_fill_u8": (C.c_int, [_P, C.c_uint64, C.c_uint8, C.c_size_t]),
    "gpurs_memory_info": (C.c_int, [_P, C.POINTER(C.c_size_t), C.POINTER(C.c_size_t)]),
    "gpurs_host_alloc": (C.c_int, [_P, C.c_size_t, _PP]),
    "gpurs_host_free": (C.c_int, [_P, _P]),
    "gpurs_stream_capture_begin": (C.c_int, [_P]),
    "gpurs_stream_capture_end": (C.c_int, [_P, _PP]),
    "gpurs_graph_launch": (C.c_int, [_P, _P]),
    "gpurs_graph_free": (None, [_P]),
    "gpurs_ipc_export": (C.c_int, [_P, C.c_uint64, C.POINTER(C.c_uint8)]),
    "gpurs_ipc_open": (C.c_int, [_P, C.POINTER(C.c_uint8), _U64P]),
    "gpurs_ipc_close": (C.c_int, [_P, C.c_uint64]),
    "gpurs_tensor_map_encode": (C.c_int, [_P, _P, C.c_int, C.c_uint32, C.c_uint64, _U64P, _U64P, C.POINTER(C.c_uint32), C.c_int, C.c_int]),
    "gpurs_module_load": (C.c_int, [_P, _P, C.c_size_t, _PP]),
    "gpurs_module_free": (None, [_P]),
    "gpurs_module_kernel": (C.c_int, [_P, C.c_char_p, _PP]),
    "gpurs_kernel_reserve_shared": (C.c_int, [_P, C.c_uint32]),
    "gpurs_kernel_registers": (C.c_int, [_P, C.POINTER(C.c_int)]),
    "gpurs_kernel_launch": (C.c_int, [_P, _P, C.POINTER(LaunchConfigStruct), _PP]),
    "gpurs_kernel_image": (_P, [C.POINTER(C.c_size_t)]),
    "gpurs_matmul": (C.c_int, [_P, C.POINTER(MatmulDesc), C.c_uint64, C.c_uint64, C.c_uint64]),
    "gpurs_quantize_e4m3": (C.c_int, [_P, C.c_uint64, C.c_uint64, C.c_uint64, C.c_uint64, C.c_uint32, C.c_uint64, C.c_uint64]),
    "gpurs_mx_scale_bytes": (C.c_size_t, [C.c_uint64, C.c_uint64, C.c_int]),
    "gpurs_quantize_mx_e4m3": (C.c_int, [_P, C.c_uint64, C.c_uint64, C.c_uint64, C.c_uint64, C.c_int, C.c_uint64, C.c_uint64]),
    "gpurs_metadata_bytes": (C.c_size_t, [C.c_uint64, C.c_uint64]),
    "gpurs_compress_24": (C.c_int, [_P, C.c_int, C.c_uint64, C.c_uint64, C.c_uint64, C.c_uint64, C.c_uint64, C.c_uint64, C.c_uint64]),
    "gpurs_matmul_f32_static": (C.c_int, [_P, C.c_uint64, C.c_uint64, C.c_uint64, C.c_uint64, C.c_uint64, C.c_uint64]),
    "gpurs_matmul_grouped": (C.c_int, [_P, C.POINTER(GroupedDesc), C.c_uint64, C.c_uint64, C.c_uint64, C.c_uint64, C.c_uint64]),
    "gpurs_matmul_host": (C.c_int, [_P, C.POINTER(MatmulDesc), _P, _P, _P, C.c_uint64, C.c_uint64, C.c_uint64]),
    "gpurs_matmul_allgather": (C.c_int, [_P, C.POINTER(MatmulDesc), C.POINTER(GatherDesc), C.c_uint64, C.c_uint64]),
    "gpurs_comm_unique_id": (C.c_int, [C.POINTER(C.c_uint8)]),
    "gpurs_comm_init": (C.c_int, [_P, C.POINTER(C.c_uint8), C.c_uint32, C.c_uint32, _PP]),
    "gpurs_comm_allgather": (C.c_int, [_P, _P, C.c_uint64, C.c_uint64]),
    "gpurs_comm_free": (None, [_P]),
    "gpurs_self_test_timeout": (C.c_int, [_P]),
    "gpurs_status_read": (C.c_int, [_P, C.POINTER(C.c_uint32)]),
    "gpurs_launch_count": (C.c_uint64, [_P]),
    "gpurs_last_error": (C.c_int, [C.POINTER(C.c_char_p), C.POINTER(C.c_char_p), C.POINTER(C.c_char_p)]),
}

_library = None


def load() -> C.CDLL:
    """The loaded C-ABI library.  Raises if it has not been built: there is no other code path."""
    global _library
    if _library is None:
        if not LIBRARY_PATH.exists():
            raise ImportError(f"{LIBRARY_PATH} is missing: run `python -m gpurs_b200.build` first")
        library = C.CDLL(str(LIBRARY_PATH))
        for name, (restype, argtypes) in SIGNATURES.items():
            function = getattr(library, name)
            function.restype = restype
            function.argtypes = argtypes
        _library = library
    return _library
