"""The device FP8 block quantiser against the oracle's and the golden fixture, and the quantise -> multiply
round trip of the block-scaled configuration."""
from pathlib import Path

import numpy as np
import pytest

import gpurs_b200 as G
from gpurs_b200 import _ffi
import oracle as O
from helpers import decode_output, relative_error

pytestmark = pytest.mark.gpu
GOLDEN = Path(__file__).resolve().parent / "golden"


@pytest.mark.parametrize("block_rows", [1, 128])
@pytest.mark.parametrize("shape", [(136, 300), (128, 128), (1, 4), (517, 1024), (300, 7168)])
def test_quantiser_matches_oracle_bit_for_bit(gpu, stream, shape, block_rows):
    rows, k = shape
    source = O.fill_normal_f32(rows * k, 21) * np.float32(3.0)
    source[: min(k, 128)] = 0.0   # an all-zero 1 x 128 block
    codes, scales = G.quantize_e4m3(stream, gpu.upload(source), rows, k, block_rows)
    stream.synchronize()
    expected_codes, expected_scales = O.quantize_e4m3(source, rows, k, block_rows)
    assert np.array_equal(scales.download(), expected_scales)
    assert np.array_equal(codes.download(), expected_codes)


@pytest.mark.parametrize("name,block_rows", [("row", 1), ("tile", 128)])
def test_quantiser_matches_golden(gpu, stream, name, block_rows):
    g = np.load(GOLDEN / "fp8_quantisation.npz")
    source = g["source"]
    rows, k = source.shape
    codes, scales = G.quantize_e4m3(stream, gpu.upload(source.reshape(-1)), rows, k, block_rows)
    stream.synchronize()
    assert np.array_equal(scales.download().reshape(g[f"{name}_scales"].shape), g[f"{name}_scales"])
    assert np.array_equal(codes.download().reshape(source.shape), g[f"{name}_codes"])


def test_quantise_then_multiply(gpu, stream):
    """fp32 sources -> device quantiser -> block-scaled product, against the oracle doing the same on the host and
    against the unquantised fp64 product (FP8 quantisation noise only)."""
    m, n, k = 256, 384, 1024
    a_source, b_source = O.fill_normal_f32(m * k, 31), O.fill_normal_f32(n * k, 32)
    a_codes, a_scales = G.quantize_e4m3(stream, gpu.upload(a_source), m, k, 1)
    b_codes, b_scales = G.quantize_e4m3(stream, gpu.upload(b_source), n, k, 128)
    c = gpu.zeros(G.BF16, m * n)
    G.matmul(stream, a_codes, b_codes, c, [m, n, k], G.MatmulOptions(scale_a=a_scales, scale_b=b_scales))
    stream.synchronize()
    got = decode_output(c.download(), "bf16").reshape(m, n)
    qa, sa = O.quantize_e4m3(a_source, m, k, 1)
    qb, sb = O.quantize_e4m3(b_source, n, k, 128)
    assert relative_error(got, O.matmul_rows(O.FMT_E4M3, qa, qb, n, k, np.arange(m), sa, sb)) <= 2e-2
    exact = a_source.reshape(m, k).astype(np.float64) @ b_source.reshape(n, k).astype(np.float64).T
    assert np.abs(got - exact).max() / np.abs(exact).max() < 0.05


def test_quantiser_rejections(gpu, stream):
    source, codes, scales = gpu.zeros(G.F32, 128 * 128), gpu.zeros(G.E4M3, 128 * 128), gpu.zeros(G.F32, 128)
    q = gpu._lib.gpurs_quantize_e4m3
    before = gpu.launches
    assert q(stream._handle, 128, 128, source.pointer, 0, 64, codes.pointer, scales.pointer) == _ffi.E_INVALID_ARGUMENT
    assert q(stream._handle, 128, 126, source.pointer, 0, 1, codes.pointer, scales.pointer) == _ffi.E_INVALID_VIEW
    assert q(stream._handle, 128, 128, source.pointer, 64, 1, codes.pointer, scales.pointer) == _ffi.E_INVALID_VIEW
    assert q(stream._handle, 128, 128, source.pointer, 0, 1, source.pointer, scales.pointer) == _ffi.E_ALIASING
    assert q(stream._handle, 0, 128, source.pointer, 0, 1, codes.pointer, scales.pointer) == 0
    assert gpu.launches == before
