"""Epilogue algebra of the tile kernels: C = acc * (alpha * row_scale[row]) * column_scale[column] + bias[column], the
`scale` / `scale_rows` / `scale_columns` / `add_columns` steps of the reference's accumulator tiles
(crates/gpurs/src/gpu/tensor/warp/accumulators.rs:86-110).  Every step is rounded to fp32 on its own, so the expected
values are computed here from the plain product with the same four fp32 operations and must match bit for bit."""
import numpy as np
import pytest

import gpurs_b200 as G
from gpurs_b200 import _ffi
import oracle as O
from helpers import make_operands, run_matmul

pytestmark = pytest.mark.gpu


def expected_from(acc, m, n, alpha, row_scale, column_scale, bias):
    value = acc.astype(np.float32).reshape(m, n)
    if alpha is not None or row_scale is not None:
        factor = np.full(m, np.float32(1.0 if alpha is None else alpha), np.float32)
        if row_scale is not None:
            factor = factor * row_scale
        value = value * factor[:, None]
    if column_scale is not None:
        value = value * column_scale[None, :]
    if bias is not None:
        value = value + bias[None, :]
    return value.astype(np.float32).reshape(-1)


def vectors(m, n, seed=3):
    rng = np.random.default_rng(seed)
    return (rng.uniform(0.5, 2.0, m).astype(np.float32), rng.uniform(0.25, 1.5, n).astype(np.float32), rng.normal(0, 4, n).astype(np.float32))


@pytest.mark.parametrize("algorithm", [G.ALGO_SINGLE_CTA, G.ALGO_CTA_PAIR])
@pytest.mark.parametrize("m,n,k", [(256, 512, 128), (300, 260, 96), (129, 77, 64), (1024, 1024, 256)])
@pytest.mark.parametrize("parts", ["all", "rows", "columns", "alpha", "alpha+bias"])
def test_f32_output_matches_the_four_steps_exactly(gpu, stream, algorithm, m, n, k, parts):
    """n = 77 and 260 exercise the per-lane store path and clipped boxes, 1024^2 the TMA-store path over several tiles."""
    a_bits, b_bits = make_operands("f16", m, n, k)
    acc = run_matmul(gpu, stream, "f16", "f32", a_bits, b_bits, m, n, k, algorithm=algorithm)
    rows, columns, bias = vectors(m, n)
    alpha = 0.375
    use = {"all": (alpha, rows, columns, bias), "rows": (None, rows, None, None), "columns": (None, None, columns, None),
           "alpha": (alpha, None, None, None), "alpha+bias": (alpha, None, None, bias)}[parts]
    options = {}
    if use[0] is not None:
        options["alpha"] = use[0]
    if use[1] is not None:
        options["row_scale"] = gpu.upload(use[1])
    if use[2] is not None:
        options["column_scale"] = gpu.upload(use[2])
    if use[3] is not None:
        options["bias"] = gpu.upload(use[3])
    got = run_matmul(gpu, stream, "f16", "f32", a_bits, b_bits, m, n, k, algorithm=algorithm, **options)
    assert np.array_equal(got, expected_from(acc, m, n, *use))


@pytest.mark.parametrize("kind,out", [("bf16", "bf16"), ("f16", "f16"), ("e4m3", "bf16"), ("bf16", "f32")])
def test_sixteen_bit_outputs_round_once_after_the_algebra(gpu, stream, kind, out):
    m, n, k = 384, 520, 144
    a_bits, b_bits = make_operands(kind, m, n, k)
    acc = run_matmul(gpu, stream, kind, "f32", a_bits, b_bits, m, n, k)          # the fp32 sums before any rounding
    rows, columns, bias = vectors(m, n, seed=8)
    got = run_matmul(gpu, stream, kind, out, a_bits, b_bits, m, n, k, alpha=1.5, row_scale=gpu.upload(rows), column_scale=gpu.upload(columns),
                     bias=gpu.upload(bias))
    expected = expected_from(acc, m, n, 1.5, rows, columns, bias)
    if out == "bf16":
        assert np.array_equal(got, O.bf16_from_f32(expected))
    elif out == "f16":
        assert np.array_equal(got, O.f16_from_f32(expected))
    else:
        assert np.array_equal(got, expected)


def test_block_scaled_and_sparse_products_take_the_same_epilogue(gpu, stream):
    """The promoted (block-scaled FP8) and the 2:4-sparse kernels share the store path."""
    m, n, k = 256, 256, 256
    rows, columns, bias = vectors(m, n, seed=5)
    a_bits, b_bits = make_operands("e4m3", m, n, k)
    k_blocks = k // 128
    scale_a = gpu.upload(np.full(m * k_blocks, 0.5, np.float32))
    scale_b = gpu.upload(np.full((n // 128) * k_blocks, 2.0, np.float32))
    acc = run_matmul(gpu, stream, "e4m3", "f32", a_bits, b_bits, m, n, k, scale_a=scale_a, scale_b=scale_b)
    got = run_matmul(gpu, stream, "e4m3", "f32", a_bits, b_bits, m, n, k, scale_a=scale_a, scale_b=scale_b, alpha=2.0,
                     row_scale=gpu.upload(rows), column_scale=gpu.upload(columns), bias=gpu.upload(bias))
    assert np.array_equal(got, expected_from(acc, m, n, 2.0, rows, columns, bias))

    dense_bits, b16 = make_operands("bf16", m, n, k)
    groups = dense_bits.reshape(-1, 4).copy()
    groups[:, 1] = 0
    groups[:, 3] = 0
    dense = gpu.upload(groups.reshape(-1), G.BF16)
    values, metadata, violations = G.compress_24(stream, dense, m, k)
    stream.synchronize()
    assert violations.download()[0] == 0
    b = gpu.upload(b16, G.BF16)
    outputs = []
    for extra in ({}, {"row_scale": gpu.upload(rows), "bias": gpu.upload(bias)}):
        c = gpu.zeros(G.F32, m * n)
        G.matmul(stream, values, b, c, [m, n, k], G.MatmulOptions(metadata=metadata, **extra))
        stream.synchronize()
        outputs.append(c.download())
    assert np.array_equal(outputs[1], expected_from(outputs[0], m, n, None, rows, None, bias))


def test_decode_shapes_with_scales_leave_the_split_k_path(gpu, stream):
    """m = 16 with a row scale: AUTO must not pick the split-K kernel (which only adds a bias), and asking for it is refused."""
    m, n, k = 16, 512, 1024
    a_bits, b_bits = make_operands("f16", m, n, k)
    acc = run_matmul(gpu, stream, "f16", "f32", a_bits, b_bits, m, n, k, algorithm=G.ALGO_SINGLE_CTA)
    rows, columns, bias = vectors(m, n)
    got = run_matmul(gpu, stream, "f16", "f32", a_bits, b_bits, m, n, k, row_scale=gpu.upload(rows), bias=gpu.upload(bias))
    assert np.array_equal(got, expected_from(acc, m, n, None, rows, None, bias))
    with pytest.raises(G.GpursError) as raised:
        run_matmul(gpu, stream, "f16", "f32", a_bits, b_bits, m, n, k, algorithm=G.ALGO_SKINNY, row_scale=gpu.upload(rows))
    assert raised.value.code == _ffi.E_INVALID_ARGUMENT


def test_integer_outputs_take_no_scales(gpu, stream):
    m = n = k = 128
    a_bits, b_bits = make_operands("i8", m, n, k)
    scale = gpu.upload(np.ones(m, np.float32))
    for extra in ({"row_scale": scale}, {"column_scale": scale}, {"alpha": 2.0}):
        with pytest.raises(G.GpursError) as raised:
            run_matmul(gpu, stream, "i8", "i32", a_bits, b_bits, m, n, k, **extra)
        assert raised.value.code == _ffi.E_INVALID_ARGUMENT
    assert np.array_equal(run_matmul(gpu, stream, "i8", "i32", a_bits, b_bits, m, n, k, alpha=1.0),
                          run_matmul(gpu, stream, "i8", "i32", a_bits, b_bits, m, n, k))


@pytest.mark.parametrize("kind,out", [("f16", "f32"), ("bf16", "bf16")])
@pytest.mark.parametrize("m,n,k", [(512, 1024, 128), (300, 260, 96), (129, 77, 64)])
def test_row_absmax_is_the_maximum_of_what_was_stored(gpu, stream, kind, out, m, n, k):
    """max |.| per output row over all column tiles, taken from the fp32 values before the output rounding (so for a
    bf16 output it is at least the stored maximum and within one rounding of it); folding a second product in keeps
    the larger of the two."""
    a_bits, b_bits = make_operands(kind, m, n, k)
    rows, columns, bias = vectors(m, n, seed=13)
    scales = dict(row_scale=gpu.upload(rows), column_scale=gpu.upload(columns), bias=gpu.upload(bias))
    exact = expected_from(run_matmul(gpu, stream, kind, "f32", a_bits, b_bits, m, n, k), m, n, None, rows, columns, bias).reshape(m, n)
    absmax = gpu.zeros(G.F32, m)
    run_matmul(gpu, stream, kind, out, a_bits, b_bits, m, n, k, row_absmax=absmax, **scales)
    assert np.array_equal(absmax.download(), np.abs(exact).max(axis=1))
    run_matmul(gpu, stream, kind, out, a_bits, b_bits, m, n, k, row_absmax=absmax, alpha=0.5, **scales)     # smaller values: no change
    assert np.array_equal(absmax.download(), np.abs(exact).max(axis=1))


def test_row_absmax_is_refused_where_it_is_not_computed(gpu, stream):
    m = n = k = 128
    absmax = gpu.zeros(G.F32, m)
    a_bits, b_bits = make_operands("i8", m, n, k)
    with pytest.raises(G.GpursError) as raised:
        run_matmul(gpu, stream, "i8", "i32", a_bits, b_bits, m, n, k, row_absmax=absmax)
    assert raised.value.code == _ffi.E_INVALID_ARGUMENT
    a_bits, b_bits = make_operands("f32", m, n, k)
    with pytest.raises(G.GpursError) as raised:
        run_matmul(gpu, stream, "f32", "f32", a_bits, b_bits, m, n, k, row_absmax=absmax)
    assert raised.value.code == _ffi.E_INVALID_ARGUMENT
    a_bits, b_bits = make_operands("f16", 16, n, k)
    got = run_matmul(gpu, stream, "f16", "f32", a_bits, b_bits, 16, n, k, row_absmax=absmax)      # AUTO leaves the split-K path
    assert np.array_equal(absmax.download()[:16], np.abs(got.reshape(16, n)).max(axis=1))
