"""Argument checking of the launcher and the drop-in door (external module launch), on a B200."""
import ctypes as C

import numpy as np
import pytest

import gpurs_b200 as G
from gpurs_b200 import _ffi
import oracle as O
from helpers import make_operands

pytestmark = pytest.mark.gpu


def code_of(call):
    with pytest.raises(G.GpursError) as raised:
        call()
    return raised.value.code


def test_rejections_happen_before_any_launch(gpu, stream):
    a = gpu.zeros(G.F16, 128 * 64)
    b = gpu.zeros(G.F16, 256 * 64)
    c = gpu.zeros(G.F32, 128 * 256)
    before = gpu.launches
    assert code_of(lambda: G.matmul(stream, a, b, c, [128, 256, 128])) == _ffi.E_LENGTH_MISMATCH      # A too short
    assert code_of(lambda: G.matmul(stream, a, b, c, [128, 512, 64])) == _ffi.E_LENGTH_MISMATCH      # B and C too short
    assert code_of(lambda: G.matmul(stream, a, b, c, [128, 256, 64], G.MatmulOptions(lda=32))) == _ffi.E_INVALID_VIEW
    assert code_of(lambda: G.matmul(stream, a, b, c, [128, 256, 60], G.MatmulOptions(lda=60, ldb=60))) == _ffi.E_INVALID_VIEW  # 120-byte rows
    assert code_of(lambda: G.matmul(stream, a.slice(1, a.len), b, c, [64, 256, 64])) == _ffi.E_INVALID_VIEW  # base not 16-byte aligned
    wrong = gpu.zeros(G.I32, 128 * 256)
    assert code_of(lambda: G.matmul(stream, a, b, wrong, [128, 256, 64])) == _ffi.E_INVALID_ARGUMENT  # f16 -> i32 does not exist
    assert code_of(lambda: G.matmul(stream, a, b, c, [1 << 31, 1, 64])) == _ffi.E_SIZE_OVERFLOW
    assert code_of(lambda: G.matmul(stream, a, b, c, [128, 256, 64], G.MatmulOptions(algorithm=9))) == _ffi.E_INVALID_ARGUMENT
    alias = gpu.import_allocation(a.pointer, 128 * 16, G.F32)  # the output lies over A
    assert code_of(lambda: G.matmul(stream, a, b, alias, [16, 128, 64], G.MatmulOptions(lda=64))) == _ffi.E_ALIASING
    # fp32 operands at full precision are multiplied over a depth of 3k, which the kernels index with 32 bits: refused
    # before the split kernels are enqueued (slice lengths left unchecked, so the depth check is what answers)
    deep = _ffi.MatmulDesc()
    deep.a_type, deep.c_type, deep.m, deep.n, deep.k = G.F32, G.F32, 1, 1, (0x7FFFFFFF // 3 // 4 + 1) * 4
    assert gpu._lib.gpurs_matmul(stream._handle, C.byref(deep), 1 << 40, 2 << 40, 3 << 40) == _ffi.E_SIZE_OVERFLOW
    # a k x n right operand of a kernel that reads B K-major is copied transposed first: not before the product has been checked
    scales = gpu.zeros(G.F32, 256)
    codes_a, codes_b, out = gpu.zeros(G.E4M3, 128 * 128), gpu.zeros(G.E4M3, 128 * 256), gpu.zeros(G.BF16, 128 * 256)
    refused = G.MatmulOptions(b_row_major=True, scale_a=scales, scale_b=scales, l2_policy=7)
    assert code_of(lambda: G.matmul(stream, codes_a, codes_b, out, [128, 256, 128], refused)) == _ffi.E_INVALID_ARGUMENT
    refused = G.MatmulOptions(b_row_major=True, precision=G.PRECISION_TF32, algorithm=G.ALGO_WHOLE_TILES | G.ALGO_WIDE_TILES | G.ALGO_SQUARE_TILES)
    single = gpu.zeros(G.F32, 128 * 256)
    assert code_of(lambda: G.matmul(stream, single, single, c, [128, 256, 128], refused)) == _ffi.E_INVALID_ARGUMENT
    assert gpu.launches == before
    error = pytest.raises(G.GpursError, lambda: G.matmul(stream, a, b, alias, [16, 128, 64])).value
    assert error.operation == "gpurs_matmul" and "overlaps" in error.description


def test_mixed_gpu_handles_are_a_context_mismatch(gpu, stream):
    other = G.Gpu(gpu.ordinal)
    try:
        a = other.zeros(G.F16, 64 * 64)
        b = gpu.zeros(G.F16, 64 * 64)
        c = gpu.zeros(G.F32, 64 * 64)
        assert code_of(lambda: G.matmul(stream, a, b, c, [64, 64, 64])) == _ffi.E_CONTEXT_MISMATCH
        del a
    finally:
        other.close()


def test_driver_errors_keep_their_cuda_code(gpu):
    with pytest.raises(G.GpursError) as raised:
        gpu.allocate(G.F32, 1 << 46)    # 256 TiB
    assert raised.value.code == 2 and raised.value.name == "CUDA_ERROR_OUT_OF_MEMORY"  # `is_out_of_memory`, crates/driver/src/error.rs:23-25


def test_tensor_map_encode_checks(gpu):
    buffer = gpu.zeros(G.F16, 256 * 256)
    descriptor = (C.c_uint8 * 192)()
    base = (C.addressof(descriptor) + 63) & ~63
    dims, strides, box = (C.c_uint64 * 2)(256, 256), (C.c_uint64 * 1)(512), (C.c_uint32 * 2)(64, 128)
    encode = gpu._lib.gpurs_tensor_map_encode
    assert encode(gpu._handle, base, G.F16, 2, buffer.pointer, dims, strides, box, 3, 3) == 0
    assert any(bytes(descriptor))
    assert encode(gpu._handle, base + 8, G.F16, 2, buffer.pointer, dims, strides, box, 3, 3) == _ffi.E_INVALID_VIEW
    assert encode(gpu._handle, base, G.F16, 2, buffer.pointer + 2, dims, strides, box, 3, 3) == _ffi.E_INVALID_VIEW
    wide = (C.c_uint32 * 2)(128, 128)   # 256-byte rows do not fit the 128-byte swizzle span
    assert encode(gpu._handle, base, G.F16, 2, buffer.pointer, dims, strides, wide, 3, 3) == _ffi.E_INVALID_VIEW
    tall = (C.c_uint32 * 2)(64, 512)
    assert encode(gpu._handle, base, G.F16, 2, buffer.pointer, dims, strides, tall, 3, 3) == _ffi.E_INVALID_VIEW
    assert encode(gpu._handle, base, 12345, 2, buffer.pointer, dims, strides, box, 3, 3) == _ffi.E_INVALID_ARGUMENT


class _Params(C.Structure):
    # gemm::Params of gpurs_b200/csrc/kernels/gemm_params.hpp (192 bytes)
    _fields_ = [("c", C.c_uint64), ("ldc", C.c_longlong), ("m", C.c_int), ("n", C.c_int), ("k", C.c_int), ("tiles_m", C.c_int),
                ("tiles_n", C.c_int), ("raster_rows", C.c_int), ("vector_stores", C.c_int), ("b_row_major", C.c_int), ("status", C.c_uint64),
                ("scale_a", C.c_uint64), ("scale_b", C.c_uint64), ("bias", C.c_uint64), ("l2_policy", C.c_int), ("batches", C.c_int),
                ("row_scale", C.c_uint64), ("column_scale", C.c_uint64), ("alpha", C.c_float), ("scaled_by_alpha", C.c_int),
                ("batch_stride_c", C.c_longlong), ("row_absmax", C.c_uint64), ("partials", C.c_uint64), ("split_counters", C.c_uint64),
                ("max_contributors", C.c_int), ("split_tiles", C.c_int), ("row_bias", C.c_uint64), ("residual", C.c_uint64),
                ("ldr", C.c_longlong), ("beta", C.c_float), ("accumulate", C.c_int), ("row_sum", C.c_uint64)]


assert C.sizeof(_Params) == 192


class _TensorMap(C.Structure):
    _fields_ = [("opaque", C.c_uint64 * 16)]


def _aligned_tensor_map():
    """A CUtensorMap-sized structure on a 64-byte boundary (ctypes aligns to 8 on its own)."""
    backing = (C.c_uint8 * 256)()
    offset = (-C.addressof(backing)) % 64
    tensor_map = _TensorMap.from_buffer(backing, offset)
    tensor_map._backing = backing
    return tensor_map


def test_external_module_door(gpu, stream):
    """A host that keeps its own launcher can load the kernel image and launch an entry itself:
    Gpu::load_module -> Module::kernel -> Kernel::reserve_shared -> Kernel::launch
    (crates/gpurs/src/raw/module.rs:64-207), with descriptors from gpurs_tensor_map_encode."""
    m, n, k = 256, 512, 192
    a_bits, b_bits = make_operands("bf16", m, n, k)
    a, b = gpu.upload(a_bits, G.BF16), gpu.upload(b_bits, G.BF16)
    c = gpu.zeros(G.F32, m * n)
    status = gpu.zeros(G.I32, 4)
    module = gpu.load_module(gpu.kernel_image())
    assert code_of(lambda: module.kernel("no_such_kernel")) == _ffi.E_UNKNOWN_KERNEL
    kernel = module.kernel("gpurs_gemm_bf16_f32_cg1")
    assert 0 < kernel.registers <= 255
    shared = 230400 + 1024   # 4 stages of 48 KiB, barriers, 32 KiB of epilogue staging, alignment slack
    kernel.reserve_shared(shared)
    map_a, map_b = _aligned_tensor_map(), _aligned_tensor_map()
    for tensor_map, buffer, rows, box_rows in ((map_a, a, m, 128), (map_b, b, n, 256)):
        dims, strides, box = (C.c_uint64 * 2)(k, rows), (C.c_uint64 * 1)(k * 2), (C.c_uint32 * 2)(64, box_rows)
        assert gpu._lib.gpurs_tensor_map_encode(gpu._handle, C.addressof(tensor_map), G.BF16, 2, buffer.pointer, dims, strides, box, 3, 3) == 0
    params = _Params(c=c.pointer, ldc=n, m=m, n=n, k=k, tiles_m=m // 128, tiles_n=n // 256, raster_rows=16, vector_stores=1, status=status.pointer)
    # the dense entries also take a descriptor of C for their TMA-store epilogue: 32 rows x 128 bytes per box
    map_c = _aligned_tensor_map()
    dims, strides, box = (C.c_uint64 * 2)(n, m), (C.c_uint64 * 1)(n * 4), (C.c_uint32 * 2)(32, 32)
    assert gpu._lib.gpurs_tensor_map_encode(gpu._handle, C.addressof(map_c), G.F32, 2, c.pointer, dims, strides, box, 3, 3) == 0
    kernel.launch(stream, G.LaunchConfig(grid=(4, 1, 1), block=(192, 1, 1), shared_bytes=shared), [map_a, map_b, map_c, params])
    stream.synchronize()
    got = c.download().reshape(m, n).astype(np.float64)
    expected = O.matmul_rows(O.FMT_BF16, a_bits, b_bits, n, k, np.arange(m))
    assert np.abs(got - expected).max() / np.abs(expected).max() < 1e-5
    assert (status.download() == 0).all()
    assert code_of(lambda: kernel.launch(stream, G.LaunchConfig(grid=(0, 1, 1), block=(192, 1, 1)), [map_a, map_b, map_c, params])) == _ffi.E_INVALID_VIEW


def test_streams_events_and_copies(gpu):
    s = gpu.stream()
    assert s.raw != 0
    host = np.arange(1 << 20, dtype=np.float32)
    device = gpu.allocate(G.F32, host.size)
    start = s.record_timed()
    s.copy_to_device(device, host.ctypes.data, host.nbytes)
    back = np.zeros_like(host)
    s.copy_to_host(back.ctypes.data, device, host.nbytes)
    end = s.record_timed()
    s.synchronize()
    assert np.array_equal(back, host) and start.elapsed_ms(end) > 0.0
    part = device.slice(1024, 2048)
    assert np.array_equal(part.download(), host[1024:2048])
    with pytest.raises(ValueError):
        device.slice(10, host.size + 1)
    borrowed = gpu.borrow_stream(s.raw)
    borrowed.synchronize()
