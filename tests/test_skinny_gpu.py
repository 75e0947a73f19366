"""The decode-shaped ("skinny") product with bias: few rows of A against a large B, K split among CTAs and
reduced in split order (examples/ada/examples/skinny_matrix.rs in the reference), on a B200."""
import numpy as np
import pytest

import gpurs_b200 as G
from gpurs_b200 import _ffi
import oracle as O
from helpers import KINDS, decode_output, make_operands, relative_error

pytestmark = pytest.mark.gpu


def product(gpu, stream, kind, a, b, bias, m, n, k, out="f32", algorithm=G.ALGO_AUTO):
    c = gpu.allocate({"f32": G.F32, "bf16": G.BF16}[out], m * n)
    gpu._lib.gpurs_fill_u8(stream._handle, c.pointer, 0x7F, c.nbytes)
    options = G.MatmulOptions(algorithm=algorithm, bias=gpu.upload(bias) if bias is not None else None)
    G.matmul(stream, gpu.upload(a, KINDS[kind][0]), gpu.upload(b, KINDS[kind][0]), c, [m, n, k], options)
    stream.synchronize()
    return decode_output(c.download(), out).reshape(m, n)


def test_reference_skinny_example_is_reproduced_bit_for_bit(gpu, stream):
    """The reference's own run: 16 tokens x a 4096 x 4096 f16 weight + bias, inputs from its formulas
    (skinny_matrix.rs:74-81).  Every partial sum is exact in fp32, so the result must equal the fp64 check
    (skinny_matrix.rs:102-115) exactly, in whatever order the splits add."""
    tokens, columns, depth = 16, 4096, 4096
    index = np.arange(tokens * depth)
    inputs = O.f16_from_f32(((index * 13 % 31) / 16.0 - 1.0).astype(np.float32))
    index = np.arange(columns * depth)
    weight = O.f16_from_f32(((index * 7 % 29) / 16.0 - 1.0).astype(np.float32))
    bias = (np.arange(columns) / 64.0).astype(np.float32)
    got = product(gpu, stream, "f16", inputs, weight, bias, tokens, columns, depth)
    expected = O.matmul_rows(O.FMT_F16, inputs, weight, columns, depth, np.arange(tokens)) + bias.astype(np.float64)[None, :]
    assert np.array_equal(got, expected)
    sampled = np.arange(0, tokens * columns, 97)      # the indices the reference's check samples
    assert np.abs(got.reshape(-1)[sampled] - expected.reshape(-1)[sampled]).max() < 1e-2


@pytest.mark.parametrize("kind", ["f16", "bf16"])
@pytest.mark.parametrize("shape", [(1, 128, 64), (16, 4096, 4096), (7, 300, 136), (33, 1000, 2048), (64, 512, 8192), (48, 129, 72)])
def test_skinny_product_matches_oracle(gpu, stream, kind, shape):
    m, n, k = shape
    a, b = make_operands(kind, m, n, k)
    bias = O.fill_normal_f32(n, 77)
    got = product(gpu, stream, kind, a, b, bias, m, n, k)
    expected = O.matmul_rows(KINDS[kind][1], a, b, n, k, np.arange(m)) + bias.astype(np.float64)[None, :]
    assert relative_error(got, expected) <= 1e-3
    without = product(gpu, stream, kind, a, b, None, m, n, k)
    assert relative_error(without, expected - bias.astype(np.float64)[None, :]) <= 1e-3


def test_split_reduction_is_ordered(gpu, stream):
    """The splits add in split order, so two runs give the same bits; and the split kernel agrees with the
    unsplit tile kernel to fp32 summation accuracy."""
    m, n, k = 16, 2048, 8192
    a, b = make_operands("bf16", m, n, k)
    first = product(gpu, stream, "bf16", a, b, None, m, n, k, algorithm=G.ALGO_SKINNY)
    launches = gpu.launches
    second = product(gpu, stream, "bf16", a, b, None, m, n, k, algorithm=G.ALGO_SKINNY)
    assert gpu.launches == launches + 1           # one launch: no separate reduction kernel
    assert np.array_equal(first, second)
    tiled = product(gpu, stream, "bf16", a, b, None, m, n, k, algorithm=G.ALGO_SINGLE_CTA)
    # the unsplit kernel sums 8192 terms in the tensor core, whose fp32 accumulator truncates; the split sums are shorter
    assert relative_error(first, tiled) <= 3e-3


@pytest.mark.parametrize("algorithm", [G.ALGO_SINGLE_CTA, G.ALGO_CTA_PAIR])
@pytest.mark.parametrize("kind,out,tolerance", [("bf16", "bf16", 1e-2), ("f16", "f32", 1e-3)])
def test_bias_in_the_tile_kernels(gpu, stream, kind, out, tolerance, algorithm):
    m, n, k = 300, 520, 256
    a, b = make_operands(kind, m, n, k)
    bias = O.fill_normal_f32(n, 5) * np.float32(10.0)
    got = product(gpu, stream, kind, a, b, bias, m, n, k, out=out, algorithm=algorithm)
    expected = O.matmul_rows(KINDS[kind][1], a, b, n, k, np.arange(m)) + bias.astype(np.float64)[None, :]
    assert relative_error(got, expected) <= tolerance


def test_skinny_rejections(gpu, stream):
    a, b, c = gpu.zeros(G.F16, 128 * 64), gpu.zeros(G.F16, 128 * 64), gpu.zeros(G.F32, 128 * 128)
    with pytest.raises(G.GpursError) as raised:
        G.matmul(stream, a, b, c, [128, 128, 64], G.MatmulOptions(algorithm=G.ALGO_SKINNY))   # too many rows
    assert raised.value.code == _ffi.E_INVALID_ARGUMENT
    i8, out = gpu.zeros(G.I8, 64 * 64), gpu.zeros(G.I32, 64 * 64)
    with pytest.raises(G.GpursError) as raised:
        G.matmul(stream, i8, i8, out, [64, 64, 64], G.MatmulOptions(bias=gpu.zeros(G.F32, 64)))  # no bias on integer outputs
    assert raised.value.code == _ffi.E_INVALID_ARGUMENT
