"""The FP8 product with the tensor core's own block scaling (MX: a power-of-two scale per 32 elements of K) and its
quantiser.  The oracle is the fp64 product of the dequantised operands (codes times 2^e), the quantiser is compared
with the numpy restatement of its definition bit for bit."""
import numpy as np
import pytest

import gpurs_b200 as G
from gpurs_b200 import _ffi
import oracle as O
from helpers import decode_output, relative_error

pytestmark = pytest.mark.gpu


def quantized(gpu, stream, rows, k, right, seed, spread=True):
    """Device-quantised operand and its numpy twin."""
    source = O.fill_normal_f32(rows * k, seed)
    if spread:      # groups of very different magnitude, so that the scales matter
        rng = np.random.default_rng(seed)
        source = (source.reshape(rows, k // 32, 32) * np.exp2(rng.integers(-6, 7, (rows, k // 32, 1)).astype(np.float32))).reshape(-1).astype(np.float32)
    codes, scales = G.quantize_mx_e4m3(stream, gpu.upload(source), rows, k, right)
    stream.synchronize()
    expected_codes, exponents = O.quantize_mx_e4m3(source, rows, k)
    return codes, scales, expected_codes, exponents


@pytest.mark.parametrize("rows,k,right", [(128, 128, False), (300, 384, False), (224, 128, True), (500, 640, True), (1000, 256, True)])
def test_quantiser_matches_its_definition_bit_for_bit(gpu, stream, rows, k, right):
    codes, scales, expected_codes, exponents = quantized(gpu, stream, rows, k, right, seed=3)
    assert np.array_equal(codes.download(), expected_codes)
    assert np.array_equal(scales.download().view(np.uint8), O.mx_tile_scales(exponents, right))


def test_quantiser_edge_values(gpu, stream):
    """All-zero groups (scale 1), exact powers of two at the 448 boundary, tiny and huge magnitudes."""
    rows, k = 128, 128
    source = np.zeros((rows, k), np.float32)
    source[1, :32] = 448.0                  # exactly representable at scale 1
    source[2, :32] = 448.0001               # needs scale 2
    source[3, 32:64] = 2.0 ** -140          # subnormal input
    source[4, 64:96] = 3.0e38
    source[5, 96:] = -1.75 * 2.0 ** 20
    codes, scales = G.quantize_mx_e4m3(stream, gpu.upload(source.reshape(-1)), rows, k, False)
    stream.synchronize()
    expected_codes, exponents = O.quantize_mx_e4m3(source.reshape(-1), rows, k)
    assert exponents[1, 0] == 0 and exponents[2, 0] == 1 and exponents[0, 0] == 0 and exponents[5, 3] == 12
    assert np.array_equal(scales.download().view(np.uint8), O.mx_tile_scales(exponents, False))
    assert np.array_equal(codes.download(), expected_codes)


@pytest.mark.parametrize("algorithm", [G.ALGO_SINGLE_CTA, G.ALGO_CTA_PAIR])
@pytest.mark.parametrize("out,tolerance", [("f32", 1e-5), ("bf16", 1e-2)])
@pytest.mark.parametrize("m,n,k", [(128, 224, 128), (128, 128, 256), (200, 300, 384), (384, 672, 1024), (129, 449, 2048), (1024, 1000, 512)])
def test_product_matches_the_dequantised_fp64_product(gpu, stream, m, n, k, out, tolerance, algorithm):
    """Ragged rows and columns, several tiles in both directions, tiles whose second scale block is partly or wholly
    outside the matrix."""
    a, sa, a_codes, a_exp = quantized(gpu, stream, m, k, False, seed=11)
    b, sb, b_codes, b_exp = quantized(gpu, stream, n, k, True, seed=12)
    c = gpu.allocate(G.F32 if out == "f32" else G.BF16, m * n)
    gpu._lib.gpurs_fill_u8(stream._handle, c.pointer, 0x7F, c.nbytes)
    G.matmul(stream, a, b, c, [m, n, k], G.MatmulOptions(scale_a=sa, scale_b=sb, scale_kind=G.SCALES_MX, algorithm=algorithm))
    stream.synchronize()
    got = decode_output(c.download(), out).reshape(m, n)
    expected = O.mx_dequantize(a_codes, a_exp, m, k) @ O.mx_dequantize(b_codes, b_exp, n, k).T
    # the groups' magnitudes spread over 2^12, so small outputs are differences of large terms: the bound is relative to the
    # element plus a millionth of the largest output (fp32 accumulation)
    assert (np.abs(got - expected) <= tolerance * np.abs(expected) + 1e-6 * np.abs(expected).max()).all()
    assert gpu.status()[0] == 0


@pytest.mark.parametrize("algorithm,max_ctas,m,n,k", [(G.ALGO_CTA_PAIR | G.ALGO_SPLIT_LAST_ROUND, 8, 512, 1120, 1024),
                                                       (G.ALGO_SINGLE_CTA | G.ALGO_SPLIT_LAST_ROUND, 6, 640, 672, 512),
                                                       (G.ALGO_CTA_PAIR, 0, 256, 448, 8192), (G.ALGO_SINGLE_CTA, 0, 200, 300, 6144)])
def test_tiles_split_along_k(gpu, stream, algorithm, max_ctas, m, n, k):
    """The stream-K schedule on the MX kernel: a last round split by force on a small grid, and few tiles with a deep K split
    among idle groups by default; against the dequantised fp64 product, close to the whole-tile product, same bits on every run."""
    a, sa, a_codes, a_exp = quantized(gpu, stream, m, k, False, seed=31)
    b, sb, b_codes, b_exp = quantized(gpu, stream, n, k, True, seed=32)
    expected = O.mx_dequantize(a_codes, a_exp, m, k) @ O.mx_dequantize(b_codes, b_exp, n, k).T

    def product(flags):
        c = gpu.allocate(G.F32, m * n)
        gpu._lib.gpurs_fill_u8(stream._handle, c.pointer, 0x7F, c.nbytes)
        G.matmul(stream, a, b, c, [m, n, k], G.MatmulOptions(algorithm=flags, max_ctas=max_ctas, scale_a=sa, scale_b=sb, scale_kind=G.SCALES_MX))
        stream.synchronize()
        return c.download().reshape(m, n)

    got = product(algorithm)
    assert (np.abs(got - expected) <= 1e-5 * np.abs(expected) + 1e-5 * np.abs(expected).max()).all()
    whole = product((algorithm & ~G.ALGO_SPLIT_LAST_ROUND) | G.ALGO_WHOLE_TILES)
    assert (np.abs(got - whole) <= 1e-5 * np.abs(expected).max()).all()
    assert np.array_equal(got, product(algorithm))
    assert gpu.status() == [0, 0, 0, 0]


def test_doubling_a_scale_doubles_its_share_exactly(gpu, stream):
    """Raising every exponent of A by one doubles the fp32 result exactly; bias and a row scale ride on top."""
    m, n, k = 256, 448, 512
    a, sa, a_codes, a_exp = quantized(gpu, stream, m, k, False, seed=21, spread=False)
    b, sb, b_codes, b_exp = quantized(gpu, stream, n, k, True, seed=22, spread=False)
    doubled = gpu.upload(O.mx_tile_scales(a_exp + 1, False).view(np.int8), G.I8)
    results = []
    for scales in (sa, doubled):
        c = gpu.zeros(G.F32, m * n)
        G.matmul(stream, a, b, c, [m, n, k], G.MatmulOptions(scale_a=scales, scale_b=sb, scale_kind=G.SCALES_MX))
        stream.synchronize()
        results.append(c.download())
    assert np.array_equal(results[1], 2.0 * results[0])
    bias = (np.arange(n) / 8.0).astype(np.float32)
    rows = (1.0 + np.arange(m) % 3).astype(np.float32)
    c = gpu.zeros(G.F32, m * n)
    G.matmul(stream, a, b, c, [m, n, k], G.MatmulOptions(scale_a=sa, scale_b=sb, scale_kind=G.SCALES_MX, bias=gpu.upload(bias), row_scale=gpu.upload(rows)))
    stream.synchronize()
    assert np.array_equal(c.download().reshape(m, n), (results[0].reshape(m, n) * rows[:, None]) + bias[None, :])


def test_what_the_mx_product_rejects(gpu, stream):
    m, n, k = 128, 224, 128
    a, sa, _, _ = quantized(gpu, stream, m, k, False, seed=1)
    b, sb, _, _ = quantized(gpu, stream, n, k, True, seed=2)
    c = gpu.zeros(G.BF16, m * n)

    def code(shape=(m, n, k), **options):
        try:
            G.matmul(stream, a, b, c, list(shape), G.MatmulOptions(scale_kind=G.SCALES_MX, **options))
        except G.GpursError as error:
            return error.code
        return 0

    assert code(scale_a=sa, scale_b=sb) == 0
    assert code() == _ffi.E_INVALID_ARGUMENT                                    # no scales
    assert code(scale_a=sa, scale_b=sb, algorithm=G.ALGO_SKINNY) == _ffi.E_INVALID_ARGUMENT
    assert code(scale_a=sa, scale_b=sb, b_row_major=True) == 0                  # k x n right operand: copied transposed first
    assert code(shape=(m, n, 96), scale_a=sa, scale_b=sb) == _ffi.E_INVALID_VIEW  # depth not a multiple of 128
    assert code(scale_a=sa, scale_b=sb, batches=2) in (_ffi.E_INVALID_ARGUMENT, _ffi.E_LENGTH_MISMATCH)
    with pytest.raises(G.GpursError):
        G.matmul(stream, a, b, c, [m, n, k], G.MatmulOptions(scale_a=sa, scale_b=sb, scale_kind=7))
    stream.synchronize()
