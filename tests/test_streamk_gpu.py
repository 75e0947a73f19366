"""Stream-K: when the tile count leaves the last round of the persistent grid mostly empty, the K-blocks of that round's
tiles are spread over the whole grid and the parts are added up, in a fixed order, by whoever arrives last
(crates/gpurs/src/gpu/tensor/schedule/stream.rs in the reference).  `max_ctas` shrinks the grid and ALGO_SPLIT_LAST_ROUND
splits whether or not it pays, so that small shapes exercise it."""
import numpy as np
import pytest

import gpurs_b200 as G
import oracle as O
from helpers import KINDS, decode_output, make_operands, relative_error, run_matmul

pytestmark = pytest.mark.gpu

# (algorithm, max_ctas, m, n): tiles % groups leaves a mostly empty last round
GEOMETRIES = [
    (G.ALGO_CTA_PAIR, 8, 512, 1536),      # 2 x 6 = 12 pair tiles on 4 pairs?  12 % 4 == 0: whole rounds only (control)
    (G.ALGO_CTA_PAIR, 8, 512, 1280),      # 10 tiles on 4 pairs: 2 split over 4
    (G.ALGO_CTA_PAIR, 16, 768, 768),      # 9 tiles on 8 pairs: 1 split over 8
    (G.ALGO_SINGLE_CTA, 6, 640, 768),     # 15 tiles on 6 CTAs: 3 split over 6
    (G.ALGO_SINGLE_CTA, 7, 1000, 700),    # 8 x 3 = 24 tiles on 7 CTAs: 3 split, ragged edges
]


@pytest.mark.parametrize("algorithm,max_ctas,m,n", GEOMETRIES)
@pytest.mark.parametrize("k", [128, 1024, 1104])
def test_int8_parts_add_up_exactly(gpu, stream, algorithm, max_ctas, m, n, k):
    """Integer sums do not depend on how K was divided: bit-equal to the whole-tile product and to the oracle."""
    a_bits, b_bits = make_operands("i8", m, n, k)
    whole = run_matmul(gpu, stream, "i8", "i32", a_bits, b_bits, m, n, k, algorithm=algorithm | G.ALGO_WHOLE_TILES, max_ctas=max_ctas)
    for _ in range(2):                      # twice: the arrival counters must be back at zero after a launch
        got = run_matmul(gpu, stream, "i8", "i32", a_bits, b_bits, m, n, k, algorithm=algorithm | G.ALGO_SPLIT_LAST_ROUND, max_ctas=max_ctas)
        assert np.array_equal(got, whole)
    rows = np.arange(0, m, 37)
    assert np.array_equal(got.reshape(m, n)[rows].astype(np.int64), O.matmul_rows(O.FMT_I8, a_bits, b_bits, n, k, rows).astype(np.int64))


@pytest.mark.parametrize("algorithm,max_ctas,m,n", GEOMETRIES[1:])
def test_exact_inputs_give_the_same_bits(gpu, stream, algorithm, max_ctas, m, n):
    """The reference example's inputs (multiples of 1/16): every partial sum is exact in fp32, so the split product equals
    the whole-tile one bit for bit."""
    k = 2048
    a_bits, b_bits = make_operands("f16", m, n, k, pattern="example")
    whole = run_matmul(gpu, stream, "f16", "f32", a_bits, b_bits, m, n, k, algorithm=algorithm | G.ALGO_WHOLE_TILES, max_ctas=max_ctas)
    got = run_matmul(gpu, stream, "f16", "f32", a_bits, b_bits, m, n, k, algorithm=algorithm | G.ALGO_SPLIT_LAST_ROUND, max_ctas=max_ctas)
    assert np.array_equal(got, whole)


@pytest.mark.parametrize("kind,out,tolerance", [("bf16", "bf16", 1e-2), ("f16", "f32", 1e-3), ("e4m3", "bf16", 2e-2), ("f16", "f16", 1e-2)])
@pytest.mark.parametrize("algorithm,max_ctas,m,n", GEOMETRIES[1:])
def test_float_products_stay_within_tolerance_with_epilogue(gpu, stream, kind, out, tolerance, algorithm, max_ctas, m, n):
    k = 1024
    a_bits, b_bits = make_operands(kind, m, n, k)
    bias = (np.arange(n) % 13 - 6).astype(np.float32)
    rows_scale = (1.0 + (np.arange(m) % 5) / 4.0).astype(np.float32)
    got = run_matmul(gpu, stream, kind, out, a_bits, b_bits, m, n, k, algorithm=algorithm | G.ALGO_SPLIT_LAST_ROUND, max_ctas=max_ctas, bias=gpu.upload(bias),
                     row_scale=gpu.upload(rows_scale))
    rows = np.arange(0, m, 29)
    expected = O.matmul_rows(KINDS[kind][1], a_bits, b_bits, n, k, rows) * rows_scale[rows, None] + bias[None, :]
    assert relative_error(decode_output(got, out).reshape(m, n)[rows], expected) <= tolerance
    # deterministic: the parts are added in the contributors' order whoever arrives last
    again = run_matmul(gpu, stream, kind, out, a_bits, b_bits, m, n, k, algorithm=algorithm | G.ALGO_SPLIT_LAST_ROUND, max_ctas=max_ctas, bias=gpu.upload(bias),
                       row_scale=gpu.upload(rows_scale))
    assert np.array_equal(got, again)


def test_full_grid_shape_that_splits(gpu, stream):
    """The reference example's own size on the full grid: 256 pair tiles on 74 pairs (3.46 rounds): 34 tiles are split."""
    size = 4096
    a_bits, b_bits = make_operands("f16", size, size, size, pattern="example")
    got = run_matmul(gpu, stream, "f16", "f32", a_bits, b_bits, size, size, size)
    whole = run_matmul(gpu, stream, "f16", "f32", a_bits, b_bits, size, size, size, algorithm=G.ALGO_WHOLE_TILES)
    assert np.array_equal(got, whole)
    rows = np.arange(0, size, 131)
    assert np.array_equal(got.reshape(size, size)[rows].astype(np.float64), O.matmul_rows(O.FMT_F16, a_bits, b_bits, size, size, rows))


@pytest.mark.parametrize("algorithm", [G.ALGO_CTA_PAIR, G.ALGO_SINGLE_CTA])
@pytest.mark.parametrize("m,n,k", [(256, 512, 16384), (520, 300, 8192), (128, 256, 12288)])
def test_few_tiles_and_a_deep_k_are_split_among_idle_groups(gpu, stream, algorithm, m, n, k):
    """Fewer tiles than CTA groups, K thousands deep (the reference's SplitDepth case): every tile's K-blocks go to up to four
    groups.  Integers: bit-equal to the whole-tile product and the oracle; the example's exact inputs: bit-equal; floats: within
    tolerance and the same bits on every run."""
    a_bits, b_bits = make_operands("i8", m, n, k)
    whole = run_matmul(gpu, stream, "i8", "i32", a_bits, b_bits, m, n, k, algorithm=algorithm | G.ALGO_WHOLE_TILES)
    for _ in range(2):
        got = run_matmul(gpu, stream, "i8", "i32", a_bits, b_bits, m, n, k, algorithm=algorithm)
        assert np.array_equal(got, whole)
    rows = np.arange(0, m, 37)
    assert np.array_equal(got.reshape(m, n)[rows].astype(np.int64), O.matmul_rows(O.FMT_I8, a_bits, b_bits, n, k, rows).astype(np.int64))
    a_bits, b_bits = make_operands("f16", m, n, k, pattern="example")
    assert np.array_equal(run_matmul(gpu, stream, "f16", "f32", a_bits, b_bits, m, n, k, algorithm=algorithm),
                          run_matmul(gpu, stream, "f16", "f32", a_bits, b_bits, m, n, k, algorithm=algorithm | G.ALGO_WHOLE_TILES))
    a_bits, b_bits = make_operands("bf16", m, n, k)
    got = run_matmul(gpu, stream, "bf16", "bf16", a_bits, b_bits, m, n, k, algorithm=algorithm)
    assert relative_error(decode_output(got, "bf16").reshape(m, n)[rows], O.matmul_rows(O.FMT_BF16, a_bits, b_bits, n, k, rows)) <= 1e-2
    assert np.array_equal(got, run_matmul(gpu, stream, "bf16", "bf16", a_bits, b_bits, m, n, k, algorithm=algorithm))
    assert gpu.status() == [0, 0, 0, 0]


@pytest.mark.parametrize("algorithm,max_ctas,m,n", GEOMETRIES[1:])
def test_promoted_products_split_the_same_way(gpu, stream, algorithm, max_ctas, m, n):
    """The kernels that promote every K-block to registers (fp32 as three TF32 passes, block-scaled FP8) take part in the same
    schedule: a group's share of a tile goes to scratch and the last promotion warp adds the parts in order.  fp32: within 1e-4
    of fp64 and within 1e-5 of the whole-tile product; FP8: within the configuration's 2e-2 / 1e-4; the same bits on every run."""
    k = 1024
    a_bits, b_bits = make_operands("f32", m, n, k)
    split = dict(algorithm=algorithm | G.ALGO_SPLIT_LAST_ROUND, max_ctas=max_ctas)
    got = run_matmul(gpu, stream, "f32", "f32", a_bits, b_bits, m, n, k, **split)
    whole = run_matmul(gpu, stream, "f32", "f32", a_bits, b_bits, m, n, k, algorithm=algorithm | G.ALGO_WHOLE_TILES, max_ctas=max_ctas)
    rows = np.arange(0, m, 29)
    assert relative_error(got.reshape(m, n)[rows].astype(np.float64), O.matmul_rows(O.FMT_F32, a_bits, b_bits, n, k, rows)) <= 1e-4
    assert relative_error(got.astype(np.float64), whole.astype(np.float64)) <= 1e-5
    assert np.array_equal(got, run_matmul(gpu, stream, "f32", "f32", a_bits, b_bits, m, n, k, **split))
    a_source, b_source = O.fill_normal_f32(m * k, 3), O.fill_normal_f32(n * k, 4)
    a_codes, sa = O.quantize_e4m3(a_source, m, k, 1)
    b_codes, sb = O.quantize_e4m3(b_source, n, k, 128)
    scales = dict(scale_a=gpu.upload(sa), scale_b=gpu.upload(sb))
    expected = O.matmul_rows(O.FMT_E4M3, a_codes, b_codes, n, k, rows, sa, sb)
    for out, tolerance in (("f32", 1e-4), ("bf16", 2e-2)):
        got = run_matmul(gpu, stream, "e4m3", out, a_codes, b_codes, m, n, k, **split, **scales)
        assert relative_error(decode_output(got, out).reshape(m, n)[rows], expected) <= tolerance
        assert np.array_equal(got, run_matmul(gpu, stream, "e4m3", out, a_codes, b_codes, m, n, k, **split, **scales))
    assert gpu.status() == [0, 0, 0, 0]


@pytest.mark.parametrize("m,n,k,flags,max_ctas", [(256, 512, 4096, 0, 0), (512, 1280, 512, G.ALGO_CTA_PAIR | G.ALGO_SPLIT_LAST_ROUND, 8)])
def test_one_pass_tf32_splits_too(gpu, stream, m, n, k, flags, max_ctas):
    """fp32 operands in one TF32 pass run the dense kernel: few tiles with a deep K, or a forced split of the last round."""
    a_bits, b_bits = make_operands("f32", m, n, k)
    got = run_matmul(gpu, stream, "f32", "f32", a_bits, b_bits, m, n, k, algorithm=flags, max_ctas=max_ctas, precision=G.PRECISION_TF32)
    whole = run_matmul(gpu, stream, "f32", "f32", a_bits, b_bits, m, n, k, algorithm=(flags & 0xff) | G.ALGO_WHOLE_TILES, max_ctas=max_ctas,
                       precision=G.PRECISION_TF32)
    rows = np.arange(0, m, 17)
    assert relative_error(got.reshape(m, n)[rows].astype(np.float64), O.matmul_rows(O.FMT_F32, a_bits, b_bits, n, k, rows)) <= 5e-2      # one TF32 pass: the operands keep 10 mantissa bits
    assert relative_error(got.astype(np.float64), whole.astype(np.float64)) <= 1e-3
    assert gpu.status() == [0, 0, 0, 0]


def test_fp32_split_depth(gpu, stream):
    """The fp32 configuration's shape class: few one-CTA tiles, 3k deep: split among idle CTAs by default."""
    m, n, k = 256, 512, 4096
    a_bits, b_bits = make_operands("f32", m, n, k)
    got = run_matmul(gpu, stream, "f32", "f32", a_bits, b_bits, m, n, k)
    whole = run_matmul(gpu, stream, "f32", "f32", a_bits, b_bits, m, n, k, algorithm=G.ALGO_WHOLE_TILES)
    rows = np.arange(0, m, 7)
    assert relative_error(got.reshape(m, n)[rows].astype(np.float64), O.matmul_rows(O.FMT_F32, a_bits, b_bits, n, k, rows)) <= 1e-4
    assert relative_error(got.astype(np.float64), whole.astype(np.float64)) <= 1e-5
    assert gpu.status() == [0, 0, 0, 0]


def test_unknown_algorithm_bits_are_refused(gpu, stream):
    a_bits, b_bits = make_operands("bf16", 128, 128, 64)
    for algorithm in (0x1000, G.ALGO_WHOLE_TILES | G.ALGO_SPLIT_LAST_ROUND, G.ALGO_WIDE_TILES | G.ALGO_SQUARE_TILES):
        with pytest.raises(G.GpursError):
            run_matmul(gpu, stream, "bf16", "bf16", a_bits, b_bits, 128, 128, 64, algorithm=algorithm)


@pytest.mark.parametrize("algorithm,max_ctas,m,n,k", [(G.ALGO_CTA_PAIR, 8, 1280, 256, 256), (G.ALGO_SINGLE_CTA, 16, 2176, 256, 256),
                                                      (G.ALGO_SINGLE_CTA, 16, 2176, 256, 384)])
def test_fewer_k_blocks_than_groups(gpu, stream, algorithm, max_ctas, m, n, k):
    """One tile left over and only two or three K-blocks to deal out: only as many groups take part as there are K-blocks
    (a group with nothing to do must not be counted among the tile's contributors)."""
    a_bits, b_bits = make_operands("i8", m, n, k)
    whole = run_matmul(gpu, stream, "i8", "i32", a_bits, b_bits, m, n, k, algorithm=algorithm | G.ALGO_WHOLE_TILES, max_ctas=max_ctas)
    got = run_matmul(gpu, stream, "i8", "i32", a_bits, b_bits, m, n, k, algorithm=algorithm | G.ALGO_SPLIT_LAST_ROUND, max_ctas=max_ctas)
    assert np.array_equal(got, whole)
    rows = np.arange(0, m, 41)
    assert np.array_equal(got.reshape(m, n)[rows].astype(np.int64), O.matmul_rows(O.FMT_I8, a_bits, b_bits, n, k, rows).astype(np.int64))
