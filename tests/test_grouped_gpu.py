"""The grouped (mixture-of-experts) product on a B200: rows gathered by index, one weight per expert
(examples/ada/examples/grouped_matrix.rs in the reference)."""
import numpy as np
import pytest

import gpurs_b200 as G
from gpurs_b200 import _ffi
import oracle as O
from helpers import decode_output, relative_error

pytestmark = pytest.mark.gpu

FORMATS = {"f16": (G.F16, O.FMT_F16, O.f16_from_f32), "bf16": (G.BF16, O.FMT_BF16, O.bf16_from_f32)}


def expected_product(fmt, inputs, weight, routes, offsets, n, k):
    """fp64 reference: per expert, the gathered rows against that expert's weight (the example's check,
    grouped_matrix.rs:101-115, on every output instead of every 61st)."""
    rows = int(offsets[-1])
    out = np.zeros((rows, n))
    gathered = inputs.reshape(-1, k)[routes[:rows]].reshape(-1)
    for e in range(len(offsets) - 1):
        begin, end = int(offsets[e]), int(offsets[e + 1])
        if end > begin:
            out[begin:end] = O.matmul_rows(fmt, gathered, weight.reshape(len(offsets) - 1, n * k)[e], n, k, np.arange(begin, end))
    return out


def run_grouped(gpu, stream, kind, out, inputs, weight, routes, offsets, rows, tokens, n, k):
    element = FORMATS[kind][0]
    output = gpu.allocate({"f32": G.F32, "f16": G.F16, "bf16": G.BF16}[out], rows * n)
    gpu._lib.gpurs_fill_u8(stream._handle, output.pointer, 0x7F, output.nbytes)
    G.matmul_grouped(stream, gpu.upload(inputs, element), gpu.upload(routes.astype(np.int32)), gpu.upload(offsets.astype(np.int32)),
                     gpu.upload(weight, element), output, rows, tokens, n, k, len(offsets) - 1)
    stream.synchronize()
    return output.download()


def test_reference_grouped_example_is_reproduced_bit_for_bit(gpu, stream):
    """The reference's own run: 1000 tokens over 8 experts (one of them empty, one with a single row), f16 in and
    out, its input formulas and routing (grouped_matrix.rs:66-82).  Inputs are multiples of 1/64, so the fp32 sums are
    exact and the f16 output is the correctly rounded exact product: bit for bit."""
    tokens, experts, columns, depth = 1000, 8, 1024, 512
    index = np.arange(tokens * depth)
    inputs = O.f16_from_f32(((index * 13 % 31) / 64.0 - 0.25).astype(np.float32))
    index = np.arange(experts * columns * depth)
    weight = O.f16_from_f32(((index * 7 % 29) / 64.0 - 0.25).astype(np.float32))
    routes = (np.arange(tokens) * 37 % tokens).astype(np.uint32)
    offsets = np.concatenate([[0], np.cumsum([100, 0, 237, 64, 1, 300, 150, 148])]).astype(np.uint32)
    bits = run_grouped(gpu, stream, "f16", "f16", inputs, weight, routes, offsets, tokens, tokens, columns, depth)
    expected = expected_product(O.FMT_F16, inputs, weight, routes, offsets, columns, depth)
    assert np.array_equal(bits, O.f16_from_f32(expected.astype(np.float32).reshape(-1)))
    got = decode_output(bits, "f16").reshape(tokens, columns)
    sampled = np.arange(0, tokens * columns, 61)     # the outputs the reference's check samples, its error measure
    error = np.abs(got.reshape(-1)[sampled] - expected.reshape(-1)[sampled]) / np.maximum(np.abs(expected.reshape(-1)[sampled]), 1.0)
    assert error.max() < 1e-2


@pytest.mark.parametrize("kind,out,tolerance", [("f16", "f32", 1e-3), ("bf16", "bf16", 1e-2), ("bf16", "f32", 1e-3)])
@pytest.mark.parametrize("counts,n,k", [([5], 64, 64), ([128, 128], 256, 128), ([0, 300, 1, 129, 0], 520, 200), ([700, 33, 512], 1032, 1024)])
def test_grouped_product_matches_oracle(gpu, stream, kind, out, tolerance, counts, n, k):
    element, fmt, encode = FORMATS[kind]
    experts, rows = len(counts), sum(counts)
    tokens = rows + 37                      # more activations than routed rows; some never used
    rng = np.random.default_rng(3)
    inputs = O.fill_normal_16(fmt, tokens * k, 1)
    weight = O.fill_normal_16(fmt, experts * n * k, 2)
    routes = rng.integers(0, tokens, rows).astype(np.uint32)
    offsets = np.concatenate([[0], np.cumsum(counts)]).astype(np.uint32)
    got = decode_output(run_grouped(gpu, stream, kind, out, inputs, weight, routes, offsets, rows, tokens, n, k), out).reshape(rows, n)
    assert relative_error(got, expected_product(fmt, inputs, weight, routes, offsets, n, k)) <= tolerance


def test_rows_past_the_last_offset_are_left_alone(gpu, stream):
    rows, tokens, n, k = 200, 64, 128, 64
    inputs, weight = O.fill_normal_16(O.FMT_F16, tokens * k, 1), O.fill_normal_16(O.FMT_F16, 2 * n * k, 2)
    routes = (np.arange(rows) % tokens).astype(np.uint32)
    offsets = np.array([0, 90, 150], np.uint32)        # rows 150..199 belong to no expert
    got = run_grouped(gpu, stream, "f16", "f32", inputs, weight, routes, offsets, rows, tokens, n, k).reshape(rows, n)
    poison = np.frombuffer(bytes([0x7F] * 4), np.float32)[0]
    assert (got[150:].view(np.uint32) == np.float32(poison).view(np.uint32)).all()
    assert relative_error(got[:150].astype(np.float64), expected_product(O.FMT_F16, inputs, weight, routes, offsets, n, k)) <= 1e-3


def test_grouped_rejections(gpu, stream):
    buffers = gpu.zeros(G.F16, 64 * 64), gpu.zeros(G.I32, 64), gpu.zeros(G.I32, 2), gpu.zeros(G.F16, 64 * 64), gpu.zeros(G.F16, 64 * 64)
    inputs, routes, offsets, weight, output = buffers

    def code(**changes):
        fields = dict(a_type=G.F16, c_type=G.F16, rows=64, tokens=64, n=64, k=64, experts=1, lda=0, ldc=0)
        fields.update(changes)
        desc = _ffi.GroupedDesc(*[fields[name] for name, _ in _ffi.GroupedDesc._fields_])
        return gpu._lib.gpurs_matmul_grouped(stream._handle, desc, inputs.pointer, routes.pointer, offsets.pointer, weight.pointer, output.pointer)

    before = gpu.launches
    assert code(a_type=G.F32) == _ffi.E_INVALID_ARGUMENT
    assert code(c_type=G.BF16) == _ffi.E_INVALID_ARGUMENT
    assert code(k=60) == _ffi.E_INVALID_VIEW
    assert code(lda=32) == _ffi.E_INVALID_VIEW
    assert code(rows=0) == 0
    assert gpu.launches == before
