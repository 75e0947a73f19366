"""Failure detection without a GPU fault: a kernel whose wait can never complete gives up after its time limit,
records the failure in the status word and returns, the host reports GPURS_E_DEVICE_TIMEOUT, and the same context
goes on computing correctly."""
import time

import numpy as np
import pytest

import gpurs_b200 as G
from gpurs_b200 import _ffi
import oracle as O
from helpers import make_operands, run_matmul

pytestmark = pytest.mark.gpu


def test_bounded_wait_gives_up_and_the_context_survives():
    gpu = G.Gpu(0)
    try:
        stream = gpu.stream()
        started = time.perf_counter()
        assert gpu._lib.gpurs_self_test_timeout(stream._handle) == 0
        with pytest.raises(G.GpursError) as raised:
            stream.synchronize()
        elapsed = time.perf_counter() - started
        assert raised.value.code == _ffi.E_DEVICE_TIMEOUT
        assert 1.0 < elapsed < 10.0            # the limit is 1.5 s; nothing hangs
        assert gpu.status() == [0, 0, 0, 0]    # synchronize collected and cleared the word
        # the context is still good: a product right after it is correct
        m, n, k = 256, 256, 256
        a, b = make_operands("bf16", m, n, k)
        got = run_matmul(gpu, stream, "bf16", "f32", a, b, m, n, k).reshape(m, n).astype(np.float64)
        expected = O.matmul_rows(O.FMT_BF16, a, b, n, k, np.arange(m))
        assert np.abs(got - expected).max() / np.abs(expected).max() < 1e-5
        # and the raw status word names the probe when read before a synchronize
        assert gpu._lib.gpurs_self_test_timeout(stream._handle) == 0
        assert gpu.status()[0] == 4
    finally:
        gpu.close()
