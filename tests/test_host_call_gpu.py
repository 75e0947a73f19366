"""The product with operands and result in host memory (gpurs_matmul_host): the reference example's upload / upload /
launch / download (examples/blackwell/examples/blackwell_matrix.rs:58-83) as one overlapped call."""
import ctypes as C

import numpy as np
import pytest

import gpurs_b200 as G
from gpurs_b200 import _ffi
import oracle as O
from helpers import KINDS, OUTPUTS, make_operands, run_matmul

pytestmark = pytest.mark.gpu


class Pinned:
    """A page-locked host array of `nbytes` bytes."""

    def __init__(self, gpu, nbytes):
        self.gpu, self.pointer, self.nbytes = gpu, C.c_void_p(), nbytes
        assert gpu._lib.gpurs_host_alloc(gpu._handle, max(nbytes, 1), C.byref(self.pointer)) == 0

    def fill(self, array):
        C.memmove(self.pointer, array.ctypes.data, array.nbytes)

    def read(self, dtype):
        return np.frombuffer(C.string_at(self.pointer, self.nbytes), dtype).copy()

    def __del__(self):
        self.gpu._lib.gpurs_host_free(self.gpu._handle, self.pointer)


def host_product(gpu, stream, kind, out, a_bits, b_bits, m, n, k, **options):
    element, out_element = KINDS[kind][0], OUTPUTS[out]
    out_dtype = {"bf16": np.uint16, "f16": np.uint16, "f32": np.float32, "i32": np.int32}[out]
    ldc = options.get("ldc", 0) or n
    c_elements = (m - 1) * ldc + n
    host_a, host_b = Pinned(gpu, a_bits.nbytes), Pinned(gpu, b_bits.nbytes)
    host_c = Pinned(gpu, c_elements * np.dtype(out_dtype).itemsize)
    host_a.fill(a_bits)
    host_b.fill(b_bits)
    host_c.fill(np.full(host_c.nbytes, 0x7F, np.uint8))
    a, b = gpu.allocate(element, a_bits.size), gpu.allocate(element, b_bits.size)
    c = gpu.allocate(out_element, c_elements)
    G.matmul_host(stream, host_a.pointer.value, host_b.pointer.value, host_c.pointer.value, a, b, c, [m, n, k], G.MatmulOptions(**options))
    stream.synchronize()
    return host_c.read(out_dtype)


@pytest.mark.parametrize("kind,out", [("bf16", "bf16"), ("f16", "f32"), ("i8", "i32"), ("e4m3", "bf16"), ("f32", "f32")])
@pytest.mark.parametrize("m,n,k", [(2048, 512, 256), (1000, 264, 144), (64, 256, 512), (3000, 128, 64)])
def test_host_call_equals_the_device_call(gpu, stream, kind, out, m, n, k):
    """Blocks of rows (eight of 256 for m = 2048, a ragged last one for m = 1000 and 3000, one piece for m = 64 and for
    fp32) give bit for bit what one call on resident operands gives: every output element is the same sum in the same
    order whichever block or tile it falls in."""
    a_bits, b_bits = make_operands(kind, m, n, k)
    expected = run_matmul(gpu, stream, kind, out, a_bits, b_bits, m, n, k)
    got = host_product(gpu, stream, kind, out, a_bits, b_bits, m, n, k)
    assert np.array_equal(got.view(np.uint8), expected.view(np.uint8))


@pytest.mark.parametrize("m,n,k", [(2048, 512, 256), (512, 2048, 128)])
def test_row_and_column_algebra_follows_the_blocks(gpu, stream, m, n, k):
    """Blocks of rows (m = 2048) and blocks of columns (n = 2048): the per-row and per-column vectors, the residual matrix and the
    row reductions are addressed block by block; same bits as one call on resident operands."""
    a_bits, b_bits = make_operands("bf16", m, n, k)
    rng = np.random.default_rng(5)
    bias, row_bias = gpu.upload(rng.standard_normal(n).astype(np.float32)), gpu.upload(rng.standard_normal(m).astype(np.float32))
    row_scale, column_scale = gpu.upload((1 + rng.random(m)).astype(np.float32)), gpu.upload((1 + rng.random(n)).astype(np.float32))
    residual = gpu.upload(rng.standard_normal(m * n).astype(np.float32))
    sums = [gpu.zeros(G.F32, m), gpu.zeros(G.F32, m)]
    peaks = [gpu.zeros(G.F32, m), gpu.zeros(G.F32, m)]
    options = dict(bias=bias, row_bias=row_bias, row_scale=row_scale, column_scale=column_scale, residual=residual, beta=0.5, alpha=1.5)
    expected = run_matmul(gpu, stream, "bf16", "f32", a_bits, b_bits, m, n, k, row_sum=sums[0], row_absmax=peaks[0], **options)
    got = host_product(gpu, stream, "bf16", "f32", a_bits, b_bits, m, n, k, row_sum=sums[1], row_absmax=peaks[1], **options)
    assert np.array_equal(got, expected)
    assert np.array_equal(peaks[0].download(), peaks[1].download())
    assert np.allclose(sums[0].download(), sums[1].download(), rtol=1e-5, atol=1e-3)       # atomic adds of the tiles' parts: any order


@pytest.mark.parametrize("m,n,k", [(2048, 512, 384), (256, 2048, 256), (640, 1536, 128)])
def test_block_scales_follow_their_blocks(gpu, stream, m, n, k):
    """Block-scaled FP8 by blocks of rows (m > n: A's scale rows move with the block) and by blocks of columns (n > m:
    B's scale rows do), with per-row, per-column and bias vectors on top."""
    a_bits, b_bits = make_operands("e4m3", m, n, k)
    rng = np.random.default_rng(4)
    k_blocks = (k + 127) // 128
    options = dict(scale_a=gpu.upload(rng.uniform(0.5, 2.0, m * k_blocks).astype(np.float32)),
                   scale_b=gpu.upload(rng.uniform(0.5, 2.0, ((n + 127) // 128) * k_blocks).astype(np.float32)),
                   row_scale=gpu.upload(rng.uniform(0.5, 2.0, m).astype(np.float32)),
                   column_scale=gpu.upload(rng.uniform(0.5, 2.0, n).astype(np.float32)),
                   bias=gpu.upload(rng.normal(0, 3, n).astype(np.float32)))
    expected = run_matmul(gpu, stream, "e4m3", "bf16", a_bits, b_bits, m, n, k, **options)
    got = host_product(gpu, stream, "e4m3", "bf16", a_bits, b_bits, m, n, k, **options)
    assert np.array_equal(got, expected)


@pytest.mark.parametrize("kind,out,m,n,k", [("f16", "f32", 16, 4096, 1024), ("bf16", "bf16", 300, 3000, 192), ("i8", "i32", 128, 1280, 256)])
def test_wide_products_go_by_blocks_of_columns(gpu, stream, kind, out, m, n, k):
    """n > m: A goes up whole and B in blocks of its rows; the decode shape (m = 16) runs the split-K kernel per block."""
    a_bits, b_bits = make_operands(kind, m, n, k)
    options = {} if out == "i32" else {"bias": gpu.upload((np.arange(n) / 16.0).astype(np.float32))}
    expected = run_matmul(gpu, stream, kind, out, a_bits, b_bits, m, n, k, **options)
    got = host_product(gpu, stream, kind, out, a_bits, b_bits, m, n, k, **options)
    if kind == "f16" and m == 16:
        # split-K sums depend on how many splits a launch uses, which depends on the block's width: compare with tolerance
        assert np.abs(got.astype(np.float64) - expected.astype(np.float64)).max() <= 1e-3 * np.abs(expected).max()
    else:
        assert np.array_equal(got.view(np.uint8), expected.view(np.uint8))


def test_int8_host_call_matches_the_oracle(gpu, stream):
    m, n, k = 1536, 384, 512
    a_bits, b_bits = make_operands("i8", m, n, k)
    rows = np.arange(0, m, 5)
    got = host_product(gpu, stream, "i8", "i32", a_bits, b_bits, m, n, k)
    assert np.array_equal(got.reshape(m, n)[rows].astype(np.int64), O.matmul_rows(O.FMT_I8, a_bits, b_bits, n, k, rows).astype(np.int64))


def test_pitched_output_and_repeated_calls(gpu, stream):
    """A pitched C keeps the bytes between rows; two calls in a row on the same buffers (the second with other inputs)
    do not overtake each other."""
    m, n, k, ldc = 1024, 200, 128, 256
    first = make_operands("bf16", m, n, k, seed=2)
    second = make_operands("bf16", m, n, k, seed=9)
    got = host_product(gpu, stream, "bf16", "bf16", first[0], first[1], m, n, k, ldc=ldc)
    expected = run_matmul(gpu, stream, "bf16", "bf16", first[0], first[1], m, n, k, ldc=ldc)
    padded = np.full(m * ldc, 0x7F7F, np.uint16)
    padded[: got.size] = got
    reference = np.full(m * ldc, 0x7F7F, np.uint16)
    reference[: expected.size] = expected
    assert np.array_equal(padded.reshape(m, ldc)[:, :n], reference.reshape(m, ldc)[:, :n])
    assert (padded.reshape(m, ldc)[:-1, n:] == 0x7F7F).all()

    host_a, host_b, host_c = Pinned(gpu, first[0].nbytes), Pinned(gpu, first[1].nbytes), Pinned(gpu, m * n * 2)
    a, b, c = gpu.allocate(G.BF16, m * k), gpu.allocate(G.BF16, n * k), gpu.allocate(G.BF16, m * n)
    results = []
    for operands in (first, second):
        host_a.fill(operands[0])
        host_b.fill(operands[1])
        G.matmul_host(stream, host_a.pointer.value, host_b.pointer.value, host_c.pointer.value, a, b, c, [m, n, k])
        stream.synchronize()
        results.append(host_c.read(np.uint16))
    assert np.array_equal(results[0], run_matmul(gpu, stream, "bf16", "bf16", first[0], first[1], m, n, k))
    assert np.array_equal(results[1], run_matmul(gpu, stream, "bf16", "bf16", second[0], second[1], m, n, k))


def test_host_call_rejects_bad_arguments(gpu, stream):
    lib = gpu._lib
    desc = _ffi.MatmulDesc()
    desc.a_type, desc.c_type, desc.m, desc.n, desc.k = G.BF16, G.BF16, 256, 256, 64
    buffer = gpu.zeros(G.BF16, 256 * 256)
    host = Pinned(gpu, 256 * 256 * 2)
    pointer = host.pointer.value
    assert lib.gpurs_matmul_host(None, C.byref(desc), pointer, pointer, pointer, buffer.pointer, buffer.pointer, buffer.pointer) == _ffi.E_INVALID_ARGUMENT
    assert lib.gpurs_matmul_host(stream._handle, C.byref(desc), None, pointer, pointer, buffer.pointer, buffer.pointer, buffer.pointer) == _ffi.E_INVALID_ARGUMENT
    assert lib.gpurs_matmul_host(stream._handle, C.byref(desc), pointer, pointer, pointer, buffer.pointer, buffer.pointer, buffer.pointer) == _ffi.E_ALIASING
    desc.metadata = buffer.pointer
    assert lib.gpurs_matmul_host(stream._handle, C.byref(desc), pointer, pointer, pointer, buffer.pointer, buffer.pointer, buffer.pointer) == _ffi.E_INVALID_ARGUMENT
    desc.metadata, desc.c_type = 0, G.I32
    assert lib.gpurs_matmul_host(stream._handle, C.byref(desc), pointer, pointer, pointer, buffer.pointer, buffer.pointer, buffer.pointer) == _ffi.E_INVALID_ARGUMENT
    stream.synchronize()
