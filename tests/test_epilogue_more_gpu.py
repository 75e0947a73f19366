"""The rest of the accumulator-tile algebra and the explicit launch geometry of the matmul launcher:

    C = acc * alpha * row_scale[row] * column_scale[column] + bias[column] + row_bias[row] + beta * residual[row, column]

`add_rows` and `add` of another tile (crates/gpurs/src/gpu/tensor/warp/accumulators.rs:82-105), `reduce_rows` with +
(accumulators.rs:112-128), the atomic `accumulate` of the f32 output matrix (output/reduction.rs:157-202) and
`stream.launch(LaunchConfig)` (host/stream.rs:28-52,142-148).  Each algebra step is rounded to fp32 on its own, so the
expected values are rebuilt here from the plain product with the same fp32 operations and must match bit for bit."""
import numpy as np
import pytest

import gpurs_b200 as G
from gpurs_b200 import _ffi
import oracle as O
from helpers import KINDS, OUTPUTS, make_operands, run_matmul

pytestmark = pytest.mark.gpu


def product(gpu, stream, kind, out, a_bits, b_bits, m, n, k, c=None, **options):
    """Like helpers.run_matmul, but into a caller's C (kept as it is before the call)."""
    a, b = gpu.upload(a_bits, KINDS[kind][0]), gpu.upload(b_bits, KINDS[kind][0])
    if c is None:
        c = gpu.allocate(OUTPUTS[out], m * n)
        gpu._lib.gpurs_fill_u8(stream._handle, c.pointer, 0x7F, c.nbytes)
    G.matmul(stream, a, b, c, [m, n, k], G.MatmulOptions(**options))
    stream.synchronize()
    return c


def widen(bits, out):
    return {"bf16": O.bf16_to_f32, "f16": O.f16_to_f32}.get(out, lambda x: x)(bits).astype(np.float32)


def narrow(values, out):
    return {"bf16": O.bf16_from_f32, "f16": O.f16_from_f32}.get(out, lambda x: x)(values.astype(np.float32))


@pytest.mark.parametrize("algorithm", [G.ALGO_SINGLE_CTA, G.ALGO_CTA_PAIR, G.ALGO_CTA_PAIR | G.ALGO_SPLIT_LAST_ROUND])
@pytest.mark.parametrize("m,n,k", [(256, 512, 256), (300, 260, 192), (129, 77, 64), (1024, 1024, 256)])
@pytest.mark.parametrize("out", ["f32", "bf16"])
def test_row_bias_and_residual_are_added_step_by_step(gpu, stream, algorithm, m, n, k, out):
    """n = 77 takes the per-lane stores, the others the staged TMA stores; the third algorithm also splits the last round's
    tiles along K, whose parts are added up by the warp that finishes the rows."""
    a_bits, b_bits = make_operands("f16" if out == "f32" else "bf16", m, n, k)
    kind = "f16" if out == "f32" else "bf16"
    acc = run_matmul(gpu, stream, kind, "f32", a_bits, b_bits, m, n, k, algorithm=algorithm).reshape(m, n)
    rng = np.random.default_rng(21)
    bias, row_bias = rng.normal(0, 2, n).astype(np.float32), rng.normal(0, 3, m).astype(np.float32)
    residual = narrow(rng.normal(0, 5, m * n), out)
    beta = np.float32(0.75)
    got = product(gpu, stream, kind, out, a_bits, b_bits, m, n, k, algorithm=algorithm, bias=gpu.upload(bias), row_bias=gpu.upload(row_bias),
                  residual=gpu.upload(residual, OUTPUTS[out]), beta=float(beta)).download()
    expected = (acc + bias[None, :]).astype(np.float32)
    expected = (expected + row_bias[:, None]).astype(np.float32)
    expected = (expected + (beta * widen(residual, out).reshape(m, n)).astype(np.float32)).astype(np.float32)
    assert np.array_equal(got, narrow(expected.reshape(-1), out))


@pytest.mark.parametrize("m,n,k", [(384, 512, 128), (200, 77, 64)])
def test_a_residual_may_be_the_output_itself(gpu, stream, m, n, k):
    """C = A B^T + beta * C, in place: every element is read by the thread that then writes it."""
    a_bits, b_bits = make_operands("bf16", m, n, k)
    acc = run_matmul(gpu, stream, "bf16", "f32", a_bits, b_bits, m, n, k).reshape(-1)
    start = O.bf16_from_f32(np.random.default_rng(4).normal(0, 3, m * n).astype(np.float32))
    c = gpu.upload(start, G.BF16)
    product(gpu, stream, "bf16", "bf16", a_bits, b_bits, m, n, k, c=c, residual=c, beta=0.5)
    expected = (acc + (np.float32(0.5) * O.bf16_to_f32(start)).astype(np.float32)).astype(np.float32)
    assert np.array_equal(c.download(), O.bf16_from_f32(expected))
    # a residual that overlaps C without being C is refused before anything is enqueued
    with pytest.raises(G.GpursError) as raised:
        product(gpu, stream, "bf16", "bf16", a_bits, b_bits, m - 1, n, k, c=c.slice(n, m * n), residual=c.slice(0, (m - 1) * n))
    assert raised.value.code == _ffi.E_ALIASING


@pytest.mark.parametrize("algorithm", [G.ALGO_SINGLE_CTA, G.ALGO_CTA_PAIR])
@pytest.mark.parametrize("m,n,k", [(256, 256, 64), (300, 260, 64), (129, 77, 64)])
def test_row_sum_adds_each_rows_values(gpu, stream, algorithm, m, n, k):
    """With the reference example's inputs every product and every partial sum is exact in fp32, so the row sums are
    exact whatever order the tiles' atomic adds arrive in; a second product folds in on top."""
    a_bits, b_bits = make_operands("f16", m, n, k, pattern="example")
    plain = run_matmul(gpu, stream, "f16", "f32", a_bits, b_bits, m, n, k, algorithm=algorithm).reshape(m, n)
    row_sum = gpu.zeros(G.F32, m)
    got = run_matmul(gpu, stream, "f16", "f32", a_bits, b_bits, m, n, k, algorithm=algorithm, row_sum=row_sum)
    assert np.array_equal(got.reshape(m, n), plain)
    assert np.array_equal(row_sum.download().astype(np.float64), plain.astype(np.float64).sum(axis=1))
    run_matmul(gpu, stream, "f16", "f16", a_bits, b_bits, m, n, k, algorithm=algorithm, row_sum=row_sum, alpha=0.5)   # taken before the rounding
    assert np.array_equal(row_sum.download().astype(np.float64), 1.5 * plain.astype(np.float64).sum(axis=1))


def test_row_sum_of_random_values_is_within_rounding(gpu, stream):
    m, n, k = 512, 2048, 256
    a_bits, b_bits = make_operands("bf16", m, n, k)
    plain = run_matmul(gpu, stream, "bf16", "f32", a_bits, b_bits, m, n, k).reshape(m, n).astype(np.float64)
    row_sum = gpu.zeros(G.F32, m)
    run_matmul(gpu, stream, "bf16", "bf16", a_bits, b_bits, m, n, k, row_sum=row_sum)
    assert np.abs(row_sum.download() - plain.sum(axis=1)).max() <= 1e-5 * np.abs(plain).sum(axis=1).max()


@pytest.mark.parametrize("algorithm", [G.ALGO_SINGLE_CTA, G.ALGO_CTA_PAIR, G.ALGO_CTA_PAIR | G.ALGO_SPLIT_LAST_ROUND])
@pytest.mark.parametrize("m,n,k", [(256, 512, 64), (300, 260, 64), (129, 77, 64)])
def test_accumulate_adds_into_what_the_output_holds(gpu, stream, algorithm, m, n, k):
    """Two products added into a C that starts at a known (exactly representable) value: with the reference example's
    inputs the result is exact, whichever way the adds reach memory (the TMA unit's reduction for aligned rows, per-element
    atomics otherwise)."""
    a_bits, b_bits = make_operands("f16", m, n, k, pattern="example")
    plain = run_matmul(gpu, stream, "f16", "f32", a_bits, b_bits, m, n, k, algorithm=algorithm)
    start = (np.arange(m * n) % 17 - 8).astype(np.float32) / 4
    c = gpu.upload(start)
    for _ in range(2):
        product(gpu, stream, "f16", "f32", a_bits, b_bits, m, n, k, c=c, algorithm=algorithm, accumulate=True)
    assert np.array_equal(c.download(), start + 2 * plain)
    # a depth split over two launches lands in one C: columns [0, k/2) and [k/2, k) of both operands
    half = k // 2
    a, b = gpu.upload(a_bits, G.F16), gpu.upload(b_bits, G.F16)
    total = gpu.zeros(G.F32, m * n)
    for part in range(2):
        G.matmul(stream, a.slice(part * half, m * k), b.slice(part * half, n * k), total, [m, n, half],
                 G.MatmulOptions(lda=k, ldb=k, algorithm=algorithm, accumulate=True))
    stream.synchronize()
    assert np.array_equal(total.download(), plain)


def test_the_promoted_and_sparse_kernels_take_the_new_steps_too(gpu, stream):
    m, n, k = 256, 256, 256
    rng = np.random.default_rng(9)
    row_bias, residual = rng.normal(0, 2, m).astype(np.float32), rng.normal(0, 2, m * n).astype(np.float32)
    a_bits, b_bits = make_operands("f32", m, n, k)
    plain = run_matmul(gpu, stream, "f32", "f32", a_bits, b_bits, m, n, k).reshape(m, n)
    got = product(gpu, stream, "f32", "f32", a_bits, b_bits, m, n, k, row_bias=gpu.upload(row_bias), residual=gpu.upload(residual), beta=2.0).download()
    expected = ((plain + row_bias[:, None]).astype(np.float32) + (np.float32(2.0) * residual.reshape(m, n)).astype(np.float32)).astype(np.float32)
    assert np.array_equal(got, expected.reshape(-1))
    start = np.full(m * n, 3.0, np.float32)
    c = gpu.upload(start)
    a_bits, b_bits = make_operands("f16", m, n, k, pattern="example")
    exact = run_matmul(gpu, stream, "f16", "f32", a_bits, b_bits, m, n, k)
    groups = a_bits.reshape(-1, 4).copy()
    groups[:, 0] = 0
    groups[:, 2] = 0
    values, metadata, violations = G.compress_24(stream, gpu.upload(groups.reshape(-1), G.F16), m, k)
    sparse_plain = gpu.zeros(G.F32, m * n)
    b = gpu.upload(b_bits, G.F16)
    G.matmul(stream, values, b, sparse_plain, [m, n, k], G.MatmulOptions(metadata=metadata))
    G.matmul(stream, values, b, c, [m, n, k], G.MatmulOptions(metadata=metadata, accumulate=True))
    stream.synchronize()
    assert violations.download()[0] == 0 and exact.size == m * n
    assert np.array_equal(c.download(), start + sparse_plain.download())


def test_new_steps_are_refused_where_they_do_not_apply(gpu, stream):
    m = n = k = 128
    vector, matrix = gpu.zeros(G.F32, m), gpu.zeros(G.F32, m * n)
    a_bits, b_bits = make_operands("i8", m, n, k)
    for extra in ({"row_bias": vector}, {"row_sum": vector}, {"accumulate": True}, {"residual": gpu.zeros(G.I32, m * n)}):
        with pytest.raises(G.GpursError) as raised:
            run_matmul(gpu, stream, "i8", "i32", a_bits, b_bits, m, n, k, **extra)
        assert raised.value.code == _ffi.E_INVALID_ARGUMENT
    a_bits, b_bits = make_operands("bf16", m, n, k)
    with pytest.raises(G.GpursError) as raised:           # atomic adds need an fp32 output
        run_matmul(gpu, stream, "bf16", "bf16", a_bits, b_bits, m, n, k, accumulate=True)
    assert raised.value.code == _ffi.E_INVALID_ARGUMENT
    with pytest.raises(G.GpursError) as raised:           # the split-K decode kernel adds a bias only
        run_matmul(gpu, stream, "bf16", "f32", a_bits[: 16 * k], b_bits, 16, n, k, algorithm=G.ALGO_SKINNY, row_bias=vector)
    assert raised.value.code == _ffi.E_INVALID_ARGUMENT
    with pytest.raises(G.GpursError) as raised:
        run_matmul(gpu, stream, "bf16", "f32", a_bits, b_bits, m, n, k, residual=matrix, ldr=n - 1)
    assert raised.value.code == _ffi.E_INVALID_VIEW
    got = run_matmul(gpu, stream, "bf16", "f32", a_bits[: 16 * k], b_bits, 16, n, k, row_bias=vector)      # AUTO leaves the split-K path
    assert np.array_equal(got, run_matmul(gpu, stream, "bf16", "f32", a_bits[: 16 * k], b_bits, 16, n, k, algorithm=G.ALGO_SINGLE_CTA))


@pytest.mark.parametrize("kind,out", [("bf16", "bf16"), ("i8", "i32"), ("f32", "f32")])
def test_an_explicit_launch_config_sets_the_persistent_grid(gpu, stream, kind, out):
    """A grid of one cluster walks all tiles alone and gives the same bits as the library's own geometry; the cluster
    size picks the tile algorithm when the caller left it open."""
    m, n, k = 520, 1100, 192
    a_bits, b_bits = make_operands(kind, m, n, k)
    whole = dict(algorithm=G.ALGO_WHOLE_TILES)
    for cluster in (1, 2):
        threads = 384 if kind == "f32" else 192
        reference = run_matmul(gpu, stream, kind, out, a_bits, b_bits, m, n, k,
                               algorithm=(G.ALGO_CTA_PAIR if cluster == 2 else G.ALGO_SINGLE_CTA) | G.ALGO_WHOLE_TILES)
        if kind == "f32" and cluster == 2:
            continue      # AUTO keeps the promoted kernels on one-CTA tiles whatever the cluster says
        before = gpu.launches
        got = run_matmul(gpu, stream, kind, out, a_bits, b_bits, m, n, k, launch=G.LaunchConfig(grid=(cluster, 1, 1), block=(threads, 1, 1), cluster=(cluster, 1, 1)), **whole)
        assert np.array_equal(got, reference)
        assert gpu.launches - before == (2 if kind == "f32" else 1)      # fp32: one split of both operands, one product
        got = run_matmul(gpu, stream, kind, out, a_bits, b_bits, m, n, k, launch=G.LaunchConfig(grid=(2, 3, 1), block=(0, 0, 0), cluster=(cluster, 1, 1)), **whole)
        assert np.array_equal(got, reference)


def test_a_launch_config_that_does_not_fit_the_kernel_is_refused(gpu, stream):
    m, n, k = 256, 256, 128
    a_bits, b_bits = make_operands("bf16", m, n, k)
    before = gpu.launches
    bad = [G.LaunchConfig(grid=(4, 1, 1), block=(128, 1, 1), cluster=(0, 0, 0)),                       # not the kernel's thread count
           G.LaunchConfig(grid=(3, 1, 1), block=(192, 1, 1), cluster=(2, 1, 1)),                       # not a whole number of pairs
           G.LaunchConfig(grid=(4, 1, 1), block=(192, 1, 1), shared_bytes=4096, cluster=(0, 0, 0)),    # less than the kernel needs
           G.LaunchConfig(grid=(4, 1, 1), block=(192, 1, 1), cluster=(1, 2, 1))]
    for config in bad:
        with pytest.raises(G.GpursError) as raised:
            run_matmul(gpu, stream, "bf16", "bf16", a_bits, b_bits, m, n, k, launch=config)
        assert raised.value.code == _ffi.E_INVALID_VIEW
    with pytest.raises(G.GpursError) as raised:     # an explicit algorithm and a cluster size that contradicts it
        run_matmul(gpu, stream, "bf16", "bf16", a_bits, b_bits, m, n, k, algorithm=G.ALGO_SINGLE_CTA, launch=G.LaunchConfig(grid=(4, 1, 1), block=(192, 1, 1), cluster=(2, 1, 1)))
    assert raised.value.code == _ffi.E_INVALID_VIEW
    a32, b32 = make_operands("f32", m, n, k)
    with pytest.raises(G.GpursError) as raised:     # fp32 operands: refused before the split kernels are enqueued
        run_matmul(gpu, stream, "f32", "f32", a32, b32, m, n, k, launch=G.LaunchConfig(grid=(4, 1, 1), block=(192, 1, 1), cluster=(0, 0, 0)))
    assert raised.value.code == _ffi.E_INVALID_VIEW
    with pytest.raises(G.GpursError) as raised:
        run_matmul(gpu, stream, "bf16", "f32", a_bits[: 16 * k], b_bits, 16, n, k, algorithm=G.ALGO_SKINNY, launch=G.LaunchConfig(grid=(4, 1, 1), block=(192, 1, 1)))
    assert raised.value.code == _ffi.E_INVALID_ARGUMENT
    assert gpu.launches == before
