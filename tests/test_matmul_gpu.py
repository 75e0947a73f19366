"""Parity of the CUDA GEMM path with the oracle, through the C ABI, on a B200."""
import numpy as np
import pytest

import gpurs_b200 as G
import oracle as O
from helpers import KINDS, decode_output, make_operands, relative_error, run_matmul, spread_rows

pytestmark = pytest.mark.gpu

ALGORITHMS = [G.ALGO_SINGLE_CTA, G.ALGO_CTA_PAIR]

# operand kind, output, tolerance on |d| / max(|ref|, 1) against the fp64 oracle (0 = bit-exact)
FLOAT_CASES = [
    ("f16", "f32", 1e-3),    # fp32 accumulation of exactly representable products: only summation-order error
    ("f16", "f16", 2e-3),    # + one rounding to binary16 (2^-11)
    ("bf16", "f32", 1e-3),
    ("bf16", "bf16", 1e-2),  # the tolerance the bf16 configuration states
    ("e4m3", "f32", 1e-3),
    ("e4m3", "bf16", 1e-2),
]
SMALL_SHAPES = [(128, 256, 64), (1, 8, 16), (200, 300, 144), (384, 768, 1024), (129, 257, 4096), (640, 512, 80)]


@pytest.mark.parametrize("algorithm", ALGORITHMS)
@pytest.mark.parametrize("shape", SMALL_SHAPES)
@pytest.mark.parametrize("kind,out,tolerance", FLOAT_CASES)
def test_float_product_matches_oracle(gpu, stream, kind, out, tolerance, shape, algorithm):
    m, n, k = shape
    a, b = make_operands(kind, m, n, k)
    got = decode_output(run_matmul(gpu, stream, kind, out, a, b, m, n, k, algorithm), out).reshape(m, n)
    expected = O.matmul_rows(KINDS[kind][1], a, b, n, k, np.arange(m))
    assert relative_error(got, expected) <= tolerance


@pytest.mark.parametrize("algorithm", ALGORITHMS)
@pytest.mark.parametrize("shape", SMALL_SHAPES + [(1024, 1024, 1024)])
def test_f32_product_meets_1e_4(gpu, stream, shape, algorithm):
    """fp32 operands, uniform[-1, 1): the default precision (three TF32 passes over a hi/lo split) stays
    within 1e-4 of the fp64 loop; (1024, 1024, 1024) is the f32 configuration."""
    m, n, k = shape
    a, b = make_operands("f32", m, n, k)
    got = run_matmul(gpu, stream, "f32", "f32", a, b, m, n, k, algorithm).reshape(m, n).astype(np.float64)
    assert relative_error(got, O.matmul_rows(O.FMT_F32, a, b, n, k, np.arange(m))) <= 1e-4


@pytest.mark.parametrize("algorithm", ALGORITHMS)
def test_f32_single_tf32_pass(gpu, stream, algorithm):
    """One TF32 pass is what the reference's `f32` tensor element computes (element.rs:75-110): inputs keep
    10 mantissa bits, so the bound is loose and grows with K."""
    m, n, k = 384, 768, 1024
    a, b = make_operands("f32", m, n, k)
    got = run_matmul(gpu, stream, "f32", "f32", a, b, m, n, k, algorithm, precision=G.PRECISION_TF32).reshape(m, n).astype(np.float64)
    expected = O.matmul_rows(O.FMT_F32, a, b, n, k, np.arange(m))
    error = relative_error(got, expected)
    assert 1e-5 < error <= 2e-2   # visibly TF32, not fp32


def scaled_operands(m, n, k, seed=1):
    a_source, b_source = O.fill_normal_f32(m * k, seed), O.fill_normal_f32(n * k, seed + 1)
    a_codes, a_scales = O.quantize_e4m3(a_source, m, k, 1)
    b_codes, b_scales = O.quantize_e4m3(b_source, n, k, 128)
    return a_codes, a_scales, b_codes, b_scales


@pytest.mark.parametrize("algorithm", ALGORITHMS)
@pytest.mark.parametrize("out,tolerance", [("f32", 1e-4), ("bf16", 2e-2)])
@pytest.mark.parametrize("shape", [(128, 256, 128), (200, 300, 400), (384, 768, 1024), (129, 257, 2048), (640, 512, 144)])
def test_block_scaled_fp8_matches_dequantised_product(gpu, stream, shape, out, tolerance, algorithm):
    """E4M3 operands with fp32 scales per 1 x 128 (A) and 128 x 128 (B) block against the fp64 product of
    the dequantised operands; 2e-2 is the tolerance the FP8 configuration states for bf16 output."""
    m, n, k = shape
    a, sa, b, sb = scaled_operands(m, n, k)
    scale_a, scale_b = gpu.upload(sa), gpu.upload(sb)
    bits = run_matmul(gpu, stream, "e4m3", out, a, b, m, n, k, algorithm, scale_a=scale_a, scale_b=scale_b)
    got = decode_output(bits, out).reshape(m, n)
    expected = O.matmul_rows(O.FMT_E4M3, a, b, n, k, np.arange(m), sa, sb)
    assert relative_error(got, expected) <= tolerance


def test_block_scaled_fp8_configuration(gpu, stream):
    """M=4096, N=7168, K=7168, bf16 out, tolerance 2e-2 against the dequantised fp64 product."""
    m, n, k = 4096, 7168, 7168
    a, sa, b, sb = scaled_operands(m, n, k)
    scale_a, scale_b = gpu.upload(sa), gpu.upload(sb)
    got = decode_output(run_matmul(gpu, stream, "e4m3", "bf16", a, b, m, n, k, scale_a=scale_a, scale_b=scale_b), "bf16")
    indices = O.reference_sample_indices(m, n)
    assert relative_error(got[indices], O.matmul_samples(O.FMT_E4M3, a, b, n, k, indices, sa, sb)) <= 2e-2
    rows = spread_rows(m, 16)
    assert relative_error(got.reshape(m, n)[rows], O.matmul_rows(O.FMT_E4M3, a, b, n, k, rows, sa, sb)) <= 2e-2
    # scaling every A scale by 2 doubles the product exactly
    doubled = gpu.upload(sa * np.float32(2.0))
    again = decode_output(run_matmul(gpu, stream, "e4m3", "bf16", a, b, m, n, k, scale_a=doubled, scale_b=scale_b), "bf16")
    assert np.array_equal(again, 2.0 * got)


@pytest.mark.parametrize("algorithm", ALGORITHMS)
@pytest.mark.parametrize("shape", SMALL_SHAPES + [(512, 512, 2048)])
def test_int8_product_is_bit_exact(gpu, stream, shape, algorithm):
    m, n, k = shape
    a, b = make_operands("i8", m, n, k)
    got = run_matmul(gpu, stream, "i8", "i32", a, b, m, n, k, algorithm).reshape(m, n)
    assert np.array_equal(got.astype(np.int64), O.matmul_rows_i8(a, b, n, k, np.arange(m)))


@pytest.mark.parametrize("algorithm", ALGORITHMS)
@pytest.mark.parametrize("kind", ["f16", "bf16"])
@pytest.mark.parametrize("size", [320, 1024])
def test_reference_example_inputs_are_reproduced_bit_for_bit(gpu, stream, kind, size, algorithm):
    """On the reference's own inputs every partial sum is exact in fp32, so the fp32 result is unique:
    any correct kernel, the reference's included, must equal the fp64 check loop bit for bit."""
    a, b = make_operands(kind, size, size, size, "example")
    got = run_matmul(gpu, stream, kind, "f32", a, b, size, size, size, algorithm).reshape(size, size)
    expected = O.matmul_rows(KINDS[kind][1], a, b, size, size, np.arange(size))
    assert np.array_equal(got.astype(np.float64), expected)


def test_golden_example_product(gpu, stream):
    from pathlib import Path

    g = np.load(Path(__file__).resolve().parent / "golden" / "example_product_320.npz")
    size = int(g["size"])
    a, b = make_operands("f16", size, size, size, "example")
    got = run_matmul(gpu, stream, "f16", "f32", a, b, size, size, size).reshape(size, size)
    assert np.array_equal(got, g["product"])


@pytest.mark.parametrize("algorithm", ALGORITHMS)
def test_reference_configuration_4096(gpu, stream, algorithm):
    """The reference example's own run: f16 4096^3, fp32 out, checked at the indices its report samples
    (examples/matrix_benchmark.rs:36-51) and on whole rows; bit-exact, well inside its 1e-2 bound."""
    size = 4096
    a, b = make_operands("f16", size, size, size, "example")
    got = run_matmul(gpu, stream, "f16", "f32", a, b, size, size, size, algorithm)
    indices = O.reference_sample_indices(size, size)
    assert np.array_equal(got[indices].astype(np.float64), O.matmul_samples(O.FMT_F16, a, b, size, size, indices))
    rows = spread_rows(size, 24)
    assert np.array_equal(got.reshape(size, size)[rows].astype(np.float64), O.matmul_rows(O.FMT_F16, a, b, size, size, rows))


@pytest.mark.parametrize("algorithm", ALGORITHMS)
def test_bf16_8192_configuration(gpu, stream, algorithm):
    """bf16 8192^3, N(0,1) operands, fp32 accumulate, bf16 out; max rel err 1e-2 against fp64."""
    size = 8192
    a, b = make_operands("bf16", size, size, size)
    bits = run_matmul(gpu, stream, "bf16", "bf16", a, b, size, size, size, algorithm)
    got = decode_output(bits, "bf16")
    indices = O.reference_sample_indices(size, size)
    assert relative_error(got[indices], O.matmul_samples(O.FMT_BF16, a, b, size, size, indices)) <= 1e-2
    rows = spread_rows(size, 32)
    assert relative_error(got.reshape(size, size)[rows], O.matmul_rows(O.FMT_BF16, a, b, size, size, rows)) <= 1e-2
    # size-independent property over the whole output: doubling A doubles every output exactly
    doubled = (a + np.uint16(0x0080)).astype(np.uint16)  # exponent + 1; no operand is near overflow
    bits2 = run_matmul(gpu, stream, "bf16", "bf16", doubled, b, size, size, size, algorithm)
    assert np.array_equal(decode_output(bits2, "bf16"), 2.0 * got)


def test_int8_8192_configuration_and_whole_matrix_checksum(gpu, stream):
    """int8 8192^3 -> int32, bit-exact on sampled rows, and the sum of ALL outputs equals
    sum_k (sum_m A[m,k]) * (sum_n B[n,k]) computed in int64 on the host."""
    size = 8192
    a, b = make_operands("i8", size, size, size)
    got = run_matmul(gpu, stream, "i8", "i32", a, b, size, size, size).reshape(size, size)
    rows = spread_rows(size, 32)
    assert np.array_equal(got[rows].astype(np.int64), O.matmul_rows_i8(a, b, size, size, rows))
    column_sums_a = a.reshape(size, size).astype(np.int64).sum(axis=0)
    column_sums_b = b.reshape(size, size).astype(np.int64).sum(axis=0)
    assert int(got.astype(np.int64).sum()) == int((column_sums_a * column_sums_b).sum())


@pytest.mark.parametrize("algorithm", ALGORITHMS)
def test_row_permutation_commutes(gpu, stream, algorithm):
    """Permuting the rows of A permutes the rows of C bit for bit: no output depends on where its tile lies."""
    m, n, k = 1024, 768, 512
    a, b = make_operands("bf16", m, n, k)
    base = run_matmul(gpu, stream, "bf16", "f32", a, b, m, n, k, algorithm).reshape(m, n)
    order = np.random.default_rng(0).permutation(m)
    permuted = run_matmul(gpu, stream, "bf16", "f32", a.reshape(m, k)[order].reshape(-1), b, m, n, k, algorithm).reshape(m, n)
    assert np.array_equal(permuted, base[order])


@pytest.mark.parametrize("algorithm", ALGORITHMS)
def test_row_pitches_and_untouched_padding(gpu, stream, algorithm):
    m, n, k, lda, ldb, ldc = 200, 264, 136, 144, 160, 272
    a_dense, b_dense = make_operands("f16", m, n, k)
    a = np.full(m * lda, 0x7E00, np.uint16)  # NaN in the padding: it must never be read into the product
    b = np.full(n * ldb, 0x7E00, np.uint16)
    a.reshape(m, lda)[:, :k] = a_dense.reshape(m, k)
    b.reshape(n, ldb)[:, :k] = b_dense.reshape(n, k)
    raw = run_matmul(gpu, stream, "f16", "f32", a, b, m, n, k, algorithm, lda=lda, ldb=ldb, ldc=ldc)
    padded = np.full(m * ldc, np.nan, np.float32)
    padded[: raw.size] = raw
    padded = padded.reshape(m, ldc)
    expected = O.matmul_rows(O.FMT_F16, a_dense, b_dense, n, k, np.arange(m))
    assert relative_error(padded[:, :n].astype(np.float64), expected) <= 1e-3
    poison = np.frombuffer(bytes([0x7F] * 4), np.float32)[0]
    tail = padded[:-1, n:]
    assert (tail.view(np.uint32) == np.float32(poison).view(np.uint32)).all(), "the kernel wrote outside its rows"


def test_unaligned_output_falls_back_to_scalar_stores(gpu, stream):
    m, n, k = 130, 77, 64   # n * 2 bytes is not a multiple of 16
    a, b = make_operands("bf16", m, n, k)
    got = decode_output(run_matmul(gpu, stream, "bf16", "bf16", a, b, m, n, k), "bf16").reshape(m, n)
    assert relative_error(got, O.matmul_rows(O.FMT_BF16, a, b, n, k, np.arange(m))) <= 1e-2


def test_empty_shapes(gpu, stream):
    a = gpu.upload(np.zeros(64, np.uint16), G.F16)
    b = gpu.upload(np.zeros(64, np.uint16), G.F16)
    c = gpu.upload(np.full(64, 7.0, np.float32))
    G.matmul(stream, a, b, c, [0, 8, 8])
    G.matmul(stream, a, b, c, [8, 0, 8])
    stream.synchronize()
    assert (c.download() == 7.0).all()      # nothing to write
    G.matmul(stream, a, b, c, [8, 8, 0])     # an empty sum is zero
    stream.synchronize()
    assert (c.download() == 0.0).all()


def test_launches_are_counted_and_status_is_clean(gpu, stream):
    before = gpu.launches
    a, b = make_operands("bf16", 256, 256, 256)
    run_matmul(gpu, stream, "bf16", "bf16", a, b, 256, 256, 256)
    assert gpu.launches == before + 1
    assert gpu.status() == [0, 0, 0, 0]


@pytest.mark.parametrize("algorithm", ALGORITHMS)
@pytest.mark.parametrize("kind,out,tolerance", [("f16", "f32", 1e-3), ("bf16", "bf16", 1e-2), ("e4m3", "f32", 1e-3), ("i8", "i32", 0.0)])
@pytest.mark.parametrize("shape", [(128, 256, 128), (200, 304, 144), (384, 768, 1024), (129, 272, 2048)])
def test_row_major_right_operand(gpu, stream, kind, out, tolerance, shape, algorithm):
    """C = A * B with B stored k x n (n contiguous), the ordinary row-major product, instead of the reference's
    n x k "right_transposed" operand: same numbers, the tensor core reads B N-major."""
    m, n, k = shape
    a, b = make_operands(kind, m, n, k)
    b_row_major = np.ascontiguousarray(b.reshape(n, k).T).reshape(-1)
    got = decode_output(run_matmul(gpu, stream, kind, out, a, b_row_major, m, n, k, algorithm, b_row_major=True), out).reshape(m, n)
    if kind == "i8":
        assert np.array_equal(got.astype(np.int64), O.matmul_rows_i8(a, b, n, k, np.arange(m)))
    else:
        assert relative_error(got, O.matmul_rows(KINDS[kind][1], a, b, n, k, np.arange(m))) <= tolerance


def test_row_major_right_operand_with_pitch(gpu, stream):
    m, n, k, ldb = 256, 264, 192, 272
    a, b = make_operands("bf16", m, n, k)
    padded = np.full(k * ldb, 0x7FC0, np.uint16)        # NaN in the padding columns: never read
    padded.reshape(k, ldb)[:, :n] = b.reshape(n, k).T
    got = decode_output(run_matmul(gpu, stream, "bf16", "f32", a, padded, m, n, k, G.ALGO_AUTO, b_row_major=True, ldb=ldb), "f32")
    assert relative_error(got.reshape(m, n), O.matmul_rows(O.FMT_BF16, a, b, n, k, np.arange(m))) <= 1e-3


@pytest.mark.parametrize("shape", [(256, 264, 192), (129, 300, 1024), (520, 1100, 384)])
def test_row_major_right_operand_of_the_k_major_only_kernels(gpu, stream, shape):
    """One-pass TF32 and block-scaled FP8 read B K-major only: a k x n operand (with a pitch) is copied transposed into the
    handle's workspace first, and the product equals the n x k call bit for bit."""
    m, n, k = shape
    ldb = n + 8
    fa, fb = make_operands("f32", m, n, k)
    padded = np.full(k * ldb, np.nan, np.float32)
    padded.reshape(k, ldb)[:, :n] = fb.reshape(n, k).T
    expected = run_matmul(gpu, stream, "f32", "f32", fa, fb, m, n, k, G.ALGO_AUTO, precision=G.PRECISION_TF32)
    got = run_matmul(gpu, stream, "f32", "f32", fa, padded, m, n, k, G.ALGO_AUTO, b_row_major=True, ldb=ldb, precision=G.PRECISION_TF32)
    assert np.array_equal(got, expected)
    if k % 128 == 0:
        a, sa, b, sb = scaled_operands(m, n, k, seed=9)
        scales = dict(scale_a=gpu.upload(sa), scale_b=gpu.upload(sb))
        ldb = (n + 15) // 16 * 16 + 16              # row pitches stay multiples of 16 bytes
        wide = np.full(k * ldb, 0x7F, np.uint8)
        wide.reshape(k, ldb)[:, :n] = b.reshape(n, k).T
        for algorithm in ALGORITHMS:
            expected = run_matmul(gpu, stream, "e4m3", "bf16", a, b, m, n, k, algorithm, **scales)
            assert np.array_equal(run_matmul(gpu, stream, "e4m3", "bf16", a, wide, m, n, k, algorithm, b_row_major=True, ldb=ldb, **scales), expected)
    assert gpu.status() == [0, 0, 0, 0]


@pytest.mark.parametrize("shape", [(1024, 1024, 1024), (200, 301, 132), (129, 64, 2048)])
def test_f32_row_major_right_operand(gpu, stream, shape):
    """The f32 configuration as it is stated, row-major C = A * B: B is k x n.  The full-precision path copies (splits) its
    operands anyway, and writes the copy of a k x n operand transposed; same bits as the n x k call, 1e-4 against fp64."""
    m, n, k = shape
    a, b = make_operands("f32", m, n, k)
    ldb = (n + 3) // 4 * 4                                # 16-byte row pitch
    row_major = np.full(k * ldb, np.nan, np.float32)      # NaN in the padding columns: never read
    row_major.reshape(k, ldb)[:, :n] = b.reshape(n, k).T
    got = run_matmul(gpu, stream, "f32", "f32", a, row_major, m, n, k, G.ALGO_AUTO, b_row_major=True, ldb=ldb)
    assert np.array_equal(got, run_matmul(gpu, stream, "f32", "f32", a, b, m, n, k))
    rows = spread_rows(m)
    assert relative_error(got.reshape(m, n)[rows].astype(np.float64), O.matmul_rows(O.FMT_F32, a, b, n, k, rows)) <= 1e-4


@pytest.mark.parametrize("kind,out", [("bf16", "bf16"), ("f16", "f32"), ("i8", "i32"), ("e4m3", "bf16"), ("f16", "f16"), ("bf16", "f32"), ("e4m3", "f32")])
@pytest.mark.parametrize("m,n,k", [(512, 1024, 256), (300, 1100, 192), (256, 520, 64), (1024, 2048, 1100 // 16 * 16), (2304, 1536, 512)])
def test_wide_tiles_give_the_same_product(gpu, stream, kind, out, m, n, k):
    """256 x 512 CTA-pair tiles (one 512-column accumulator, handed over in halves) against 256 x 256 ones: the sums and their
    order do not depend on the tile shape, so the results are equal bit for bit; sampled rows are checked against the oracle.
    Ragged m and n clip the last boxes; 2304 x 1536 gives one pair several tiles, so halves are reused across tile borders."""
    a, b = make_operands(kind, m, n, k)
    before = gpu.launches
    got = run_matmul(gpu, stream, kind, out, a, b, m, n, k, G.ALGO_CTA_PAIR | G.ALGO_WIDE_TILES, max_ctas=8 if m == 2304 else 0)
    assert gpu.launches == before + 1
    assert np.array_equal(got, run_matmul(gpu, stream, kind, out, a, b, m, n, k, G.ALGO_CTA_PAIR | G.ALGO_SQUARE_TILES | G.ALGO_WHOLE_TILES))
    rows = spread_rows(m, 12)
    values = decode_output(got, out).reshape(m, n)[rows]
    if kind == "i8":
        assert np.array_equal(values.astype(np.int64), O.matmul_rows_i8(a, b, n, k, rows))
    else:
        assert relative_error(values, O.matmul_rows(KINDS[kind][1], a, b, n, k, rows)) <= (1e-2 if out in ("bf16", "f16") else 1e-3)


@pytest.mark.parametrize("kind,out", [("bf16", "bf16"), ("f16", "f32"), ("e4m3", "bf16"), ("bf16", "f32"), ("f16", "f16")])
@pytest.mark.parametrize("m,n,k", [(512, 1024, 256), (700, 1100, 192)])
def test_wide_tiles_apply_the_output_algebra(gpu, stream, kind, out, m, n, k):
    """The wide tiles' `_ep` entries: alpha, row and column scales, bias, row bias and a residual matrix (C itself the second
    time) give the same bits as on the 256 x 256 tiles; products with row reductions stay on those whatever the flag says."""
    a, b = make_operands(kind, m, n, k)
    rng = np.random.default_rng(11)
    vectors = dict(bias=gpu.upload(rng.standard_normal(n).astype(np.float32)), row_bias=gpu.upload(rng.standard_normal(m).astype(np.float32)),
                   row_scale=gpu.upload((1 + rng.random(m)).astype(np.float32)), column_scale=gpu.upload((1 + rng.random(n)).astype(np.float32)), alpha=0.75)
    wide, square = G.ALGO_CTA_PAIR | G.ALGO_WIDE_TILES, G.ALGO_CTA_PAIR | G.ALGO_SQUARE_TILES | G.ALGO_WHOLE_TILES
    got = run_matmul(gpu, stream, kind, out, a, b, m, n, k, wide, **vectors)
    assert np.array_equal(got, run_matmul(gpu, stream, kind, out, a, b, m, n, k, square, **vectors))
    residual = gpu.upload(got.copy(), {"bf16": G.BF16, "f16": G.F16, "f32": G.F32}[out])
    with_residual = run_matmul(gpu, stream, kind, out, a, b, m, n, k, wide, residual=residual, beta=0.5, **vectors)
    assert np.array_equal(with_residual, run_matmul(gpu, stream, kind, out, a, b, m, n, k, square, residual=residual, beta=0.5, **vectors))
    assert not np.array_equal(with_residual, got)
    sums = [gpu.zeros(G.F32, m), gpu.zeros(G.F32, m)]
    reduced = run_matmul(gpu, stream, kind, out, a, b, m, n, k, wide, row_absmax=sums[0], **vectors)
    assert np.array_equal(reduced, got)
    assert np.array_equal(sums[0].download(), (lambda s: (run_matmul(gpu, stream, kind, out, a, b, m, n, k, square, row_absmax=s, **vectors), s.download())[1])(sums[1]))


@pytest.mark.parametrize("kind,out", [("i8", "i32"), ("f16", "f32"), ("bf16", "f32"), ("e4m3", "f32")])
@pytest.mark.parametrize("m,n,k,max_ctas", [(256, 960, 256, 0), (700, 1000, 192, 0), (1024, 8192, 128, 0), (1536, 1440, 256, 4)])
def test_480_column_tiles_give_the_same_product(gpu, stream, kind, out, m, n, k, max_ctas):
    """32-bit outputs whose 480-column tiles (256 + 224) need fewer rounds x columns than 512-wide ones get those by default:
    the same sums in the same order as on 256 x 256 tiles, ragged edges and several tiles per pair included."""
    a, b = make_operands(kind, m, n, k)
    got = run_matmul(gpu, stream, kind, out, a, b, m, n, k, G.ALGO_CTA_PAIR, max_ctas=max_ctas)
    assert np.array_equal(got, run_matmul(gpu, stream, kind, out, a, b, m, n, k, G.ALGO_CTA_PAIR | G.ALGO_SQUARE_TILES | G.ALGO_WHOLE_TILES, max_ctas=max_ctas))
    assert np.array_equal(got, run_matmul(gpu, stream, kind, out, a, b, m, n, k, G.ALGO_CTA_PAIR | G.ALGO_WIDE_TILES, max_ctas=max_ctas))
    assert gpu.status() == [0, 0, 0, 0]


def test_wide_and_square_tiles_exclude_each_other(gpu, stream):
    a, b = make_operands("bf16", 256, 512, 64)
    with pytest.raises(G.GpursError) as raised:
        run_matmul(gpu, stream, "bf16", "bf16", a, b, 256, 512, 64, G.ALGO_WIDE_TILES | G.ALGO_SQUARE_TILES)
    assert raised.value.code == 100009
