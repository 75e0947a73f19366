"""The CPU oracle against the golden fixtures and against the properties the parity argument rests on.
No GPU needed."""
from pathlib import Path

import numpy as np
import pytest

import oracle as O

GOLDEN = Path(__file__).resolve().parent / "golden"


@pytest.fixture(scope="module")
def formats():
    return np.load(GOLDEN / "formats.npz")


def test_f16_from_f32_matches_golden(formats):
    assert np.array_equal(O.f16_from_f32(formats["x"]), formats["f16"])


def test_bf16_from_f32_matches_golden(formats):
    x, expected = formats["x"], formats["bf16"]
    got = O.bf16_from_f32(x)
    finite = ~np.isnan(x)
    assert np.array_equal(got[finite], expected[finite])
    # NaN: the reference keeps the payload's top bits and sets the quiet bit (float16.rs:74-76)
    assert ((got[~finite] & 0x7fc0) == 0x7fc0).all()


def test_e4m3_from_f32_matches_golden(formats):
    x, expected = formats["x"], formats["e4m3"]
    got = O.e4m3_from_f32(x)
    finite = ~np.isnan(x)
    assert np.array_equal(got[finite], expected[finite])
    assert (got[~finite] == 127).all()  # canonical NaN, sign dropped (float8.rs:25-27)


def test_tf32_from_f32_matches_golden(formats):
    assert np.array_equal(O.tf32_from_f32(formats["x"]), formats["tf32"])


def test_f16_decode_every_code(formats):
    codes = np.arange(65536, dtype=np.uint16)
    got = O.f16_to_f32(codes).view(np.uint32)
    expected = formats["f16_decoded"]
    nan = np.isnan(expected.view(np.float32))
    assert np.array_equal(got[~nan], expected[~nan])
    assert np.isnan(got.view(np.float32)[nan]).all()


def test_e4m3_decode_every_code(formats):
    codes = np.arange(256, dtype=np.uint8)
    got = O.e4m3_to_f32(codes).view(np.uint32)
    expected = formats["e4m3_decoded"]
    nan = np.isnan(expected.view(np.float32))
    assert np.array_equal(got[~nan], expected[~nan])
    assert np.isnan(got.view(np.float32)[nan]).all()


def test_e4m3_round_trip_and_saturation():
    codes = np.arange(256, dtype=np.uint8)
    values = O.e4m3_to_f32(codes)
    keep = ~np.isnan(values)
    assert np.array_equal(O.e4m3_from_f32(values[keep]), codes[keep])
    assert np.array_equal(O.e4m3_from_f32(np.array([1e9, -1e9, np.inf, -np.inf], np.float32)), np.array([0x7e, 0xfe, 0x7e, 0xfe], np.uint8))


def test_bf16_round_trip():
    codes = np.arange(65536, dtype=np.uint16)
    values = O.bf16_to_f32(codes)
    keep = ~np.isnan(values)
    assert np.array_equal(O.bf16_from_f32(values[keep]), codes[keep])


@pytest.mark.parametrize("fmt", [O.FMT_F16, O.FMT_BF16])
def test_example_inputs_closed_form(fmt):
    count = 5000
    left, right = O.example_inputs(fmt, count)
    i = np.arange(count)
    assert np.array_equal(O.decode(fmt, left), (i * 13 % 31) / 16.0 - 1.0)
    assert np.array_equal(O.decode(fmt, right), (i * 7 % 29) / 16.0 - 1.0)


@pytest.mark.parametrize("fmt", [O.FMT_F16, O.FMT_BF16])
def test_example_product_matches_golden_and_is_exact_in_fp32(fmt):
    g = np.load(GOLDEN / "example_product_320.npz")
    size = int(g["size"])
    left, right = O.example_inputs(fmt, size * size)
    rows = np.arange(size)
    expected = O.matmul_rows(fmt, left, right, size, size, rows)
    assert np.array_equal(expected, g["product"].astype(np.float64))
    # the property the bit-exact parity claim rests on: the fp64 sums are representable in fp32
    assert np.array_equal(expected.astype(np.float32).astype(np.float64), expected)
    # and so is every prefix sum, in any order: all terms are multiples of 2^-8 bounded by 1
    assert size * 1.0 < 2 ** 16


def test_sampled_check_agrees_with_row_check():
    m, n, k = 37, 53, 200
    a, b = O.fill_normal_16(O.FMT_BF16, m * k, 1), O.fill_normal_16(O.FMT_BF16, n * k, 2)
    full = O.matmul_rows(O.FMT_BF16, a, b, n, k, np.arange(m))
    indices = O.reference_sample_indices(m, n)
    assert indices[1] - indices[0] == max(m * n // 4093, 1)
    sampled = O.matmul_samples(O.FMT_BF16, a, b, n, k, indices)
    assert np.array_equal(sampled, full.reshape(-1)[indices])
    # against numpy on the decoded operands (different summation order: tolerance, not equality)
    dense = O.decode(O.FMT_BF16, a).reshape(m, k) @ O.decode(O.FMT_BF16, b).reshape(n, k).T
    assert np.allclose(full, dense, rtol=1e-12, atol=1e-9)


def test_int8_product_matches_golden():
    g = np.load(GOLDEN / "int8_product.npz")
    a, b = g["a"], g["b"]
    got = O.matmul_rows_i8(a.reshape(-1), b.reshape(-1), b.shape[0], a.shape[1], np.arange(a.shape[0]))
    assert np.array_equal(got, g["product"])
    as_float = O.matmul_rows(O.FMT_I8, a.reshape(-1), b.reshape(-1), b.shape[0], a.shape[1], np.arange(a.shape[0]))
    assert np.array_equal(as_float, g["product"].astype(np.float64))


def test_int8_generator_range_and_determinism():
    x = O.fill_int8(1 << 16, 5)
    assert x.min() == -128 and x.max() == 127
    assert np.array_equal(x, O.fill_int8(1 << 16, 5))
    assert not np.array_equal(x, O.fill_int8(1 << 16, 6))


def test_generators_distribution():
    u = O.fill_uniform_f32(1 << 18, 1)
    assert u.min() >= -1.0 and u.max() < 1.0 and abs(u.mean()) < 0.01
    z = O.fill_normal_f32(1 << 18, 2)
    assert abs(z.mean()) < 0.01 and abs(z.std() - 1.0) < 0.01


@pytest.mark.parametrize("name,block_rows", [("row", 1), ("tile", 128)])
def test_fp8_block_quantisation_matches_golden(name, block_rows):
    g = np.load(GOLDEN / "fp8_quantisation.npz")
    source = g["source"]
    codes, scales = O.quantize_e4m3(source.reshape(-1), source.shape[0], source.shape[1], block_rows)
    assert np.array_equal(scales.reshape(g[f"{name}_scales"].shape), g[f"{name}_scales"])
    assert np.array_equal(codes.reshape(source.shape), g[f"{name}_codes"])


def test_block_scaled_product_is_the_dequantised_product():
    m, n, k = 9, 130, 300
    a_src, b_src = O.fill_normal_f32(m * k, 1), O.fill_normal_f32(n * k, 2)
    qa, sa = O.quantize_e4m3(a_src, m, k, 1)
    qb, sb = O.quantize_e4m3(b_src, n, k, 128)
    got = O.matmul_rows(O.FMT_E4M3, qa, qb, n, k, np.arange(m), sa, sb)
    kb = (k + 127) // 128
    da = O.decode(O.FMT_E4M3, qa).reshape(m, k) * np.repeat(sa.reshape(m, kb).astype(np.float64), 128, axis=1)[:, :k]
    sb_full = np.repeat(np.repeat(sb.reshape(-1, kb).astype(np.float64), 128, axis=0)[:n], 128, axis=1)[:, :k]
    db = O.decode(O.FMT_E4M3, qb).reshape(n, k) * sb_full
    assert np.allclose(got, da @ db.T, rtol=1e-12, atol=1e-12)
    # quantisation error against the unquantised product stays within the FP8 tolerance of the config
    exact = a_src.reshape(m, k).astype(np.float64) @ b_src.reshape(n, k).astype(np.float64).T
    assert np.abs(got - exact).max() / np.abs(exact).max() < 0.05


def test_sparse24_generator_and_compression_round_trip():
    rows, depth = 24, 256
    dense = O.fill_sparse24_bf16(rows, depth, 3)
    groups = (dense.reshape(-1, 4) & 0x7fff) != 0
    assert (groups.sum(axis=1) == 2).all()
    values, indices, violations = O.compress_24(dense, rows, depth)
    assert violations == 0
    first, second = indices & 3, (indices >> 2) & 3
    assert (first < second).all()
    rebuilt = np.zeros((rows * depth // 4, 4), np.uint16)
    v = values.reshape(-1, 2)
    rebuilt[np.arange(len(v)), first] = v[:, 0]
    rebuilt[np.arange(len(v)), second] = v[:, 1]
    assert np.array_equal(rebuilt.reshape(-1), dense)
    # all six position pairs occur
    assert len(np.unique(indices)) == 6
    # a matrix that is not 2:4 is reported
    bad = dense.copy()
    bad[:4] = 0x3f80
    assert O.compress_24(bad, rows, depth)[2] == 1


def test_mx_quantiser_restatement_follows_its_definition():
    """The numpy restatement of the MX quantiser (test infrastructure for the MX-scaled product): per 32 elements the
    smallest power of two that brings the largest magnitude to 448 or below, codes = E4M3(x / 2^e), and the tiled scale
    layouts put every (row, group) at a distinct byte."""
    rows, depth = 96, 256
    rng = np.random.default_rng(5)
    source = (rng.normal(0, 1, (rows, depth // 32, 32)) * np.exp2(rng.integers(-20, 20, (rows, depth // 32, 1)))).astype(np.float32)
    source[0, 0] = 0.0                          # all-zero group
    source[1, 0] = 448.0                        # exactly at the boundary: scale 1
    source[2, 0, :] = 0.0
    source[2, 0, 3] = 449.0                     # just above: scale 2
    codes, exponents = O.quantize_mx_e4m3(source.reshape(-1), rows, depth)
    assert exponents[0, 0] == 0 and exponents[1, 0] == 0 and exponents[2, 0] == 1
    absmax = np.abs(source).max(axis=2).astype(np.float64)
    nonzero = absmax > 0
    assert (absmax[nonzero] / np.exp2(exponents[nonzero].astype(np.float64)) <= 448.0).all()
    assert (absmax[nonzero] / np.exp2(exponents[nonzero] - 1.0) > 448.0).all()           # and no smaller power would do
    back = O.mx_dequantize(codes, exponents, rows, depth).reshape(rows, depth // 32, 32)
    # E4M3 keeps 3 mantissa bits: relative error at most 2^-4 for values in the normal range of the scaled group
    scaled = np.abs(source.astype(np.float64)) / np.exp2(exponents.astype(np.float64))[:, :, None]
    normal = scaled >= 2.0 ** -6
    assert (np.abs(back - source)[normal] <= np.abs(source.astype(np.float64))[normal] * 2.0 ** -4).all()
    for right in (False, True):
        tiled = O.mx_tile_scales(exponents, right)
        r, g = np.meshgrid(np.arange(rows), np.arange(depth // 32), indexing="ij")
        index = O.mx_scale_index(right, r, g * 32, depth // 128)
        assert len(np.unique(index)) == index.size and index.max() < tiled.size
        assert np.array_equal(tiled[index], (exponents + 127).astype(np.uint8))
