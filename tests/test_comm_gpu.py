"""The NCCL all-gather behind the C ABI on one GPU: a communicator of one rank is the whole lifecycle (id, init, the
in-place collective on a stream, free) without a second GPU; the bench drives the same calls with 2, 4 and 8 ranks and
compares every rank's gathered matrix with the fused product's."""
import ctypes as C

import numpy as np
import pytest

import gpurs_b200 as G
from gpurs_b200 import _ffi
from helpers import make_operands

pytestmark = pytest.mark.gpu


def test_one_rank_communicator_gathers_in_place(gpu, stream):
    m, n, k = 256, 512, 128
    a_bits, b_bits = make_operands("bf16", m, n, k)
    a, b = gpu.upload(a_bits, G.BF16), gpu.upload(b_bits, G.BF16)
    full = gpu.zeros(G.BF16, m * n)
    comm = G.Communicator(gpu, 0, 1, lambda unique: unique)
    try:
        G.matmul(stream, a, b, full, [m, n, k])
        comm.allgather(stream, full, m * n * 2)          # stream-ordered after the product, in place
        stream.synchronize()
        expected = gpu.zeros(G.BF16, m * n)
        G.matmul(stream, a, b, expected, [m, n, k])
        stream.synchronize()
        assert np.array_equal(full.download(), expected.download())
        comm.allgather(stream, full, 0)                  # nothing to gather is not an error
        with pytest.raises(G.GpursError) as raised:
            comm.allgather(stream, full, m * n * 2 + 2)
        assert raised.value.code == _ffi.E_LENGTH_MISMATCH
    finally:
        comm.close()


def test_communicator_arguments_are_checked(gpu, stream):
    raw = (C.c_uint8 * _ffi.COMM_ID_BYTES).from_buffer_copy(G.comm_unique_id())
    handle = C.c_void_p()
    assert gpu._lib.gpurs_comm_init(gpu._handle, raw, 0, 0, C.byref(handle)) == _ffi.E_INVALID_ARGUMENT
    assert gpu._lib.gpurs_comm_init(gpu._handle, raw, 2, 2, C.byref(handle)) == _ffi.E_INVALID_ARGUMENT
    assert gpu._lib.gpurs_comm_init(gpu._handle, None, 1, 0, C.byref(handle)) == _ffi.E_INVALID_ARGUMENT
    assert gpu._lib.gpurs_comm_unique_id(None) == _ffi.E_INVALID_ARGUMENT
    gpu._lib.gpurs_comm_free(None)
