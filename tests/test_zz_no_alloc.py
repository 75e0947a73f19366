"""gpurs_matmul_f32_static: the fp32 product for hosts that may not allocate device memory at call time
(their pool owns the whole device, or they cannot take the device-wide synchronisation that an
allocation or a free implies).  Its scratch is a fixed array inside the library, shared by every call,
so the test calls it twice in a row, with different operands, and checks each result against the
regular entry point (gpurs_matmul, which allocates its scratch) on the same operands.

The file name keeps it last in collection order: a run that stops at the first failure has by then run
every other test.  It creates its own Gpu handle, so it behaves the same alone in a fresh process and
after the rest of the suite."""
import ctypes as C

import numpy as np
import pytest

import gpurs_b200 as G
from gpurs_b200 import _ffi
import oracle as O
from helpers import relative_error

pytestmark = pytest.mark.gpu

TOLERANCE = 1e-4   # the bound the fp32 tests use, on |d| / max(|ref|, 1)


def static_matmul(gpu, stream, a, b, c, m, n, k):
    return gpu._lib.gpurs_matmul_f32_static(stream._handle, m, n, k, a.pointer, b.pointer, c.pointer)


def test_static_entry_matches_the_allocating_entry_twice_in_a_row():
    gpu = G.Gpu(0)
    try:
        stream = gpu.stream()
        for call, (m, n, k, seed) in enumerate([(1024, 1024, 1024, 11), (333, 520, 772, 23)]):
            a_host, b_host = O.fill_uniform_f32(m * k, seed), O.fill_uniform_f32(n * k, seed + 1)
            a, b = gpu.upload(a_host), gpu.upload(b_host)
            c_static = gpu.allocate(G.F32, m * n)
            c_regular = gpu.allocate(G.F32, m * n)
            gpu._lib.gpurs_fill_u8(stream._handle, c_static.pointer, 0x7F, c_static.nbytes)   # unwritten outputs would show
            assert static_matmul(gpu, stream, a, b, c_static, m, n, k) == 0, f"call {call}"
            G.matmul(stream, a, b, c_regular, [m, n, k])
            stream.synchronize()
            got = c_static.download().reshape(m, n).astype(np.float64)
            regular = c_regular.download().reshape(m, n).astype(np.float64)
            assert relative_error(got, regular) <= TOLERANCE, f"call {call}: differs from gpurs_matmul"
            rows = np.arange(0, m, max(1, m // 64))
            assert relative_error(got[rows], O.matmul_rows(O.FMT_F32, a_host, b_host, n, k, rows)) <= TOLERANCE, f"call {call}: differs from the oracle"
        assert gpu.status() == [0, 0, 0, 0]
    finally:
        gpu.close()


def free_bytes(gpu):
    free, total = C.c_size_t(), C.c_size_t()
    assert gpu._lib.gpurs_memory_info(gpu._handle, C.byref(free), C.byref(total)) == 0
    return free.value


def test_static_entry_allocates_nothing():
    """What the entry exists for: on a handle that has never run the allocating fp32 product, calls through the static
    entry leave the device's free memory exactly where it was, and each call is two launches (split, product).  The
    first call is the warm-up that loads the kernel image; the measurement starts after it."""
    gpu = G.Gpu(0)
    try:
        stream = gpu.stream()
        m, n, k = 512, 384, 640
        a_host, b_host = O.fill_uniform_f32(m * k, 5), O.fill_uniform_f32(n * k, 6)
        a, b, c = gpu.upload(a_host), gpu.upload(b_host), gpu.zeros(G.F32, m * n)
        assert static_matmul(gpu, stream, a, b, c, m, n, k) == 0
        stream.synchronize()
        before, launches = free_bytes(gpu), gpu.launches
        for _ in range(3):
            assert static_matmul(gpu, stream, a, b, c, m, n, k) == 0
        stream.synchronize()
        assert free_bytes(gpu) == before, "a call through the static entry changed the device's free memory"
        assert gpu.launches - launches == 6
        rows = np.arange(0, m, 16)
        got = c.download().reshape(m, n).astype(np.float64)
        assert relative_error(got[rows], O.matmul_rows(O.FMT_F32, a_host, b_host, n, k, rows)) <= TOLERANCE
        # the allocating entry, for contrast, takes its scratch from the device on its first call
        regular = gpu.zeros(G.F32, m * n)
        before = free_bytes(gpu)
        G.matmul(stream, a, b, regular, [m, n, k])
        stream.synchronize()
        assert free_bytes(gpu) < before
        assert relative_error(got, regular.download().reshape(m, n).astype(np.float64)) <= TOLERANCE
    finally:
        gpu.close()


def test_static_entry_survives_closing_and_reopening_the_handle():
    """The array's address is looked up at every call, under the handle that makes the call: a second handle opened after
    the first was closed computes the same product."""
    m, n, k = 256, 320, 512
    a_host, b_host = O.fill_uniform_f32(m * k, 31), O.fill_uniform_f32(n * k, 32)
    results = []
    for _ in range(2):
        gpu = G.Gpu(0)
        try:
            stream = gpu.stream()
            a, b = gpu.upload(a_host), gpu.upload(b_host)
            c_static, c_regular = gpu.zeros(G.F32, m * n), gpu.zeros(G.F32, m * n)
            assert static_matmul(gpu, stream, a, b, c_static, m, n, k) == 0
            G.matmul(stream, a, b, c_regular, [m, n, k])
            stream.synchronize()
            got = c_static.download()
            assert relative_error(got.astype(np.float64), c_regular.download().astype(np.float64)) <= TOLERANCE
            assert gpu.status() == [0, 0, 0, 0]
            results.append(got)
            del a, b, c_static, c_regular
        finally:
            gpu.close()
    assert np.array_equal(results[0], results[1])


def test_static_entry_rejects_what_does_not_fit():
    gpu = G.Gpu(0)
    try:
        stream = gpu.stream()
        small = gpu.zeros(G.F32, 64 * 64)
        before = gpu.launches
        # (m + n) * 3k * 4 bytes = 48 MiB > 32 MiB
        assert static_matmul(gpu, stream, small, small, small, 2048, 2048, 1024) == _ffi.E_SIZE_OVERFLOW
        operation, name, description = C.c_char_p(), C.c_char_p(), C.c_char_p()
        gpu._lib.gpurs_last_error(C.byref(operation), C.byref(name), C.byref(description))
        assert operation.value == b"gpurs_matmul_f32_static" and b"static scratch holds" in description.value
        assert static_matmul(gpu, stream, small, small, small, 64, 64, 62) == _ffi.E_INVALID_VIEW      # rows are not 16-byte multiples
        assert static_matmul(gpu, stream, small, small, small, 32, 32, 64) == _ffi.E_ALIASING          # output over an operand
        assert gpu._lib.gpurs_matmul_f32_static(None, 1, 1, 4, 0, 0, 0) == _ffi.E_INVALID_ARGUMENT
        # sizes at the edge of what 64-bit arithmetic on the split sizes holds are size errors, not wrapped sums
        assert static_matmul(gpu, stream, small, small, small, 0x7fffffff, 0x7fffffff, 0x7fffffff // 3 // 4 * 4) == _ffi.E_SIZE_OVERFLOW
        assert static_matmul(gpu, stream, small, small, small, 64, 64, 0x7fffffff // 3 + 1) == _ffi.E_SIZE_OVERFLOW
        assert gpu.launches == before
        assert _ffi.STATIC_SCRATCH_BYTES == 32 << 20
    finally:
        gpu.close()
