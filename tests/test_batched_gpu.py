"""A batch of products of one shape in one launch (`OutputMatrix::batched` / `Tile::batch` in the reference,
crates/gpurs/src/gpu/tensor/output/matrix.rs:94-99, schedule/grid.rs:57-66): rank-3 descriptors, tiles of all matrices on
one persistent grid.  Every matrix of the batch must equal the single product of its operands bit for bit."""
import numpy as np
import pytest

import gpurs_b200 as G
from gpurs_b200 import _ffi
from helpers import KINDS, OUTPUTS, make_operands, run_matmul

pytestmark = pytest.mark.gpu


def run_batch(gpu, stream, kind, out, a_list, b_list, m, n, k, stride_a=0, stride_b=0, stride_c=0, **options):
    """Lays the operands out at the given strides (0 = packed), runs the batch, returns the list of outputs."""
    batches = len(a_list)
    sa, sb, sc = stride_a or m * k, stride_b or n * k, stride_c or m * n
    a_all = np.zeros((batches - 1) * sa + m * k, a_list[0].dtype)
    b_all = np.zeros((batches - 1) * sb + n * k, b_list[0].dtype)
    for i in range(batches):
        a_all[i * sa:i * sa + m * k] = a_list[i]
        b_all[i * sb:i * sb + n * k] = b_list[i]
    a, b = gpu.upload(a_all, KINDS[kind][0]), gpu.upload(b_all, KINDS[kind][0])
    c = gpu.allocate(OUTPUTS[out], (batches - 1) * sc + m * n)
    gpu._lib.gpurs_fill_u8(stream._handle, c.pointer, 0x7F, c.nbytes)
    G.matmul(stream, a, b, c, [m, n, k], G.MatmulOptions(batches=batches, stride_a=stride_a, stride_b=stride_b, stride_c=stride_c, **options))
    stream.synchronize()
    whole = c.download()
    return [whole[i * sc:i * sc + m * n] for i in range(batches)], whole


@pytest.mark.parametrize("algorithm", [G.ALGO_SINGLE_CTA, G.ALGO_CTA_PAIR])
@pytest.mark.parametrize("kind,out", [("bf16", "bf16"), ("f16", "f32"), ("f16", "f16"), ("bf16", "f32")])
@pytest.mark.parametrize("batches,m,n,k", [(3, 200, 136, 96), (2, 512, 512, 256), (5, 64, 77, 64), (16, 128, 256, 128)])
def test_every_matrix_of_the_batch_equals_its_single_product(gpu, stream, algorithm, kind, out, batches, m, n, k):
    """Ragged tiles inside every matrix (m = 200: rows past a matrix's end are zero, not the next matrix's), n = 77 on the
    per-lane store path, 16 matrices over more tiles than CTAs."""
    pairs = [make_operands(kind, m, n, k, seed=10 + 2 * i) for i in range(batches)]
    outputs, _ = run_batch(gpu, stream, kind, out, [p[0] for p in pairs], [p[1] for p in pairs], m, n, k, algorithm=algorithm)
    for (a_bits, b_bits), got in zip(pairs, outputs):
        assert np.array_equal(got, run_matmul(gpu, stream, kind, out, a_bits, b_bits, m, n, k, algorithm=algorithm))


def test_strided_batches_leave_the_gaps_alone(gpu, stream):
    m, n, k, batches = 130, 264, 72, 3
    strides = dict(stride_a=m * k + 64, stride_b=n * k + 128, stride_c=m * n + 40)
    pairs = [make_operands("bf16", m, n, k, seed=40 + i) for i in range(batches)]
    outputs, whole = run_batch(gpu, stream, "bf16", "bf16", [p[0] for p in pairs], [p[1] for p in pairs], m, n, k, **strides)
    for (a_bits, b_bits), got in zip(pairs, outputs):
        assert np.array_equal(got, run_matmul(gpu, stream, "bf16", "bf16", a_bits, b_bits, m, n, k))
    for i in range(batches - 1):
        gap = whole[i * strides["stride_c"] + m * n:(i + 1) * strides["stride_c"]]
        assert (gap == 0x7F7F).all()


def test_bias_applies_to_every_matrix(gpu, stream):
    m, n, k, batches = 256, 256, 64, 4
    bias = (np.arange(n) / 4.0).astype(np.float32)
    pairs = [make_operands("f16", m, n, k, seed=70 + i) for i in range(batches)]
    outputs, _ = run_batch(gpu, stream, "f16", "f32", [p[0] for p in pairs], [p[1] for p in pairs], m, n, k, bias=gpu.upload(bias))
    for (a_bits, b_bits), got in zip(pairs, outputs):
        assert np.array_equal(got, run_matmul(gpu, stream, "f16", "f32", a_bits, b_bits, m, n, k, bias=gpu.upload(bias), algorithm=G.ALGO_CTA_PAIR))


def test_what_a_batch_rejects(gpu, stream):
    m = n = k = 128
    a, b = gpu.zeros(G.BF16, 4 * m * k), gpu.zeros(G.BF16, 4 * n * k)
    c = gpu.zeros(G.BF16, 4 * m * n)

    def code(**options):
        try:
            G.matmul(stream, a, b, c, [m, n, k], G.MatmulOptions(**options))
        except G.GpursError as error:
            return error.code
        return 0

    assert code(batches=4) == 0
    assert code(batches=5) == _ffi.E_LENGTH_MISMATCH                       # the slices hold four matrices
    assert code(batches=4, stride_a=m * k - 8) == _ffi.E_INVALID_VIEW       # matrices of A would overlap
    assert code(batches=4, stride_a=m * k + 4) == _ffi.E_LENGTH_MISMATCH    # ... and a larger stride no longer fits the slice
    assert code(batches=2, stride_a=m * k + 4) == _ffi.E_INVALID_VIEW       # 8 bytes off a 16-byte boundary
    assert code(batches=4, b_row_major=True) == _ffi.E_INVALID_ARGUMENT
    assert code(batches=4, algorithm=G.ALGO_SKINNY) == _ffi.E_INVALID_ARGUMENT
    assert code(batches=-1) == _ffi.E_INVALID_ARGUMENT
    i8a, i8b, i32c = gpu.zeros(G.I8, 2 * m * k), gpu.zeros(G.I8, 2 * n * k), gpu.zeros(G.I32, 2 * m * n)
    with pytest.raises(G.GpursError) as raised:
        G.matmul(stream, i8a, i8b, i32c, [m, n, k], G.MatmulOptions(batches=2))
    assert raised.value.code == _ffi.E_INVALID_ARGUMENT
    stream.synchronize()
    assert gpu.status()[0] == 0
