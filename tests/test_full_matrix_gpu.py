"""Whole-matrix comparisons at the configurations' full sizes against an independent GPU implementation (the vendor
library through torch), which is itself checked against the CPU oracle on sampled rows in the same test.  The oracle
alone cannot cover 67 million outputs of depth 8192 in test time; the sampled-row and property tests elsewhere do not
look at every element.  torch is test infrastructure here, never part of the product path."""
import numpy as np
import pytest

import gpurs_b200 as G
import oracle as O
from helpers import make_operands, relative_error, run_matmul

pytestmark = pytest.mark.gpu
torch = pytest.importorskip("torch")


def as_tensor(bits: np.ndarray, rows: int, columns: int, dtype):
    """Bit patterns (uint16 / int8 arrays from the oracle) as a CUDA tensor of `dtype`."""
    host = torch.from_numpy(bits.reshape(rows, columns).copy())
    return host.view(dtype).cuda() if dtype in (torch.float16, torch.bfloat16) else host.cuda()


def test_reference_example_whole_matrix_is_exact(gpu, stream):
    """R0, f16 4096^3 -> f32 on the reference example's inputs: every partial sum is exact in fp32, so an fp32 product on
    the CUDA cores (TF32 off) must give the same 16.7 million bit patterns; that product matches the oracle's fp64 loop
    exactly on the sampled rows."""
    size = 4096
    a_bits, b_bits = make_operands("f16", size, size, size, pattern="example")
    ours = run_matmul(gpu, stream, "f16", "f32", a_bits, b_bits, size, size, size)
    previous = torch.backends.cuda.matmul.allow_tf32
    torch.backends.cuda.matmul.allow_tf32 = False
    try:
        a = as_tensor(a_bits.view(np.int16), size, size, torch.float16).float()
        b = as_tensor(b_bits.view(np.int16), size, size, torch.float16).float()
        theirs = torch.matmul(a, b.T).cpu().numpy()
    finally:
        torch.backends.cuda.matmul.allow_tf32 = previous
    rows = np.arange(0, size, 97)
    assert np.array_equal(theirs[rows].astype(np.float64), O.matmul_rows(O.FMT_F16, a_bits, b_bits, size, size, rows))
    assert np.array_equal(ours.reshape(size, size), theirs)


def test_bf16_8192_whole_matrix_against_the_vendor_library(gpu, stream):
    """C2: all 67 million bf16 outputs within 1e-2 of the library's (both round an fp32 sum of the same products to bf16,
    in different orders); the library's output is within 1e-2 of the oracle on sampled rows."""
    size = 8192
    a_bits, b_bits = make_operands("bf16", size, size, size)
    ours = O.bf16_to_f32(run_matmul(gpu, stream, "bf16", "bf16", a_bits, b_bits, size, size, size)).reshape(size, size)
    a = as_tensor(a_bits.view(np.int16), size, size, torch.bfloat16)
    b = as_tensor(b_bits.view(np.int16), size, size, torch.bfloat16)
    theirs = torch.matmul(a, b.T).float().cpu().numpy()
    del a, b
    rows = np.arange(0, size, 521)
    expected = O.matmul_rows(O.FMT_BF16, a_bits, b_bits, size, size, rows)
    assert relative_error(theirs[rows].astype(np.float64), expected) <= 1e-2
    assert relative_error(ours[rows].astype(np.float64), expected) <= 1e-2
    error = np.abs(ours - theirs) / np.maximum(np.abs(theirs), 1.0)
    assert float(error.max()) <= 1e-2
    assert not np.isnan(ours).any()


def test_int8_8192_whole_matrix_is_exact(gpu, stream):
    """C4: all 67 million int32 outputs equal the library's integer product (exact on both sides), which equals the
    oracle's int64 loop on sampled rows."""
    size = 8192
    a_bits, b_bits = make_operands("i8", size, size, size)
    ours = run_matmul(gpu, stream, "i8", "i32", a_bits, b_bits, size, size, size).reshape(size, size)
    a = as_tensor(a_bits.view(np.int8), size, size, torch.int8)
    b = as_tensor(b_bits.view(np.int8), size, size, torch.int8)
    try:
        theirs = torch._int_mm(a, b.T).cpu().numpy()
    except (RuntimeError, AttributeError) as error:      # pragma: no cover - depends on the torch build
        pytest.skip(f"no integer matrix product in this torch build: {error}")
    rows = np.arange(0, size, 521)
    assert np.array_equal(theirs[rows].astype(np.int64), O.matmul_rows(O.FMT_I8, a_bits, b_bits, size, size, rows).astype(np.int64))
    assert np.array_equal(ours, theirs)
