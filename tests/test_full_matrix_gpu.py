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


def test_block_scaled_fp8_whole_matrix(gpu, stream):
    """C3, 4096 x 7168 x 7168 block-scaled E4M3 -> bf16: all 29 million outputs within 2e-2 of an fp32 CUDA-core product of the
    dequantised operands (codes times their block scales, which is exact in fp32), itself within 1e-3 of the oracle's fp64
    product on sampled rows (fp32 summation over K = 7168; measured 3e-4)."""
    m, n, k = 4096, 7168, 7168
    a_source, b_source = O.fill_normal_f32(m * k, 1), O.fill_normal_f32(n * k, 2)
    a_codes, a_scales = O.quantize_e4m3(a_source, m, k, 1)
    b_codes, b_scales = O.quantize_e4m3(b_source, n, k, 128)
    del a_source, b_source
    ours = O.bf16_to_f32(run_matmul(gpu, stream, "e4m3", "bf16", a_codes, b_codes, m, n, k, scale_a=gpu.upload(a_scales),
                                    scale_b=gpu.upload(b_scales))).reshape(m, n)
    k_blocks = k // 128
    a = torch.from_numpy(a_codes.reshape(m, k).copy()).cuda().view(torch.float8_e4m3fn).float()
    a = (a.view(m, k_blocks, 128) * torch.from_numpy(a_scales.reshape(m, k_blocks, 1)).cuda()).view(m, k)
    b = torch.from_numpy(b_codes.reshape(n, k).copy()).cuda().view(torch.float8_e4m3fn).float()
    b = (b.view(n // 128, 128, k_blocks, 128) * torch.from_numpy(b_scales.reshape(n // 128, 1, k_blocks, 1)).cuda()).view(n, k)
    previous = torch.backends.cuda.matmul.allow_tf32
    torch.backends.cuda.matmul.allow_tf32 = False
    try:
        theirs = torch.matmul(a, b.T).cpu().numpy()
    finally:
        torch.backends.cuda.matmul.allow_tf32 = previous
    del a, b
    rows = np.arange(0, m, 331)
    expected = O.matmul_rows(O.FMT_E4M3, a_codes, b_codes, n, k, rows, a_scales, b_scales)
    assert relative_error(theirs[rows].astype(np.float64), expected) <= 1e-3
    error = np.abs(ours - theirs) / np.maximum(np.abs(theirs), 1.0)
    assert float(error.max()) <= 2e-2
    assert not np.isnan(ours).any()


def test_sparse_shard_whole_matrix(gpu, stream):
    """C5, one GPU's shard 2048 x 8192 (2:4) x 8192 -> bf16: all 16.8 million outputs within 1e-2 of the library's dense
    product of the densified operand (the definition of the sparse product), which is within 1e-2 of the oracle on
    sampled rows."""
    m, n, k = 2048, 8192, 8192
    dense = O.fill_sparse24_bf16(m, k, 3)
    b_bits = O.fill_normal_16(O.FMT_BF16, n * k, 4)
    values, metadata, violations = G.compress_24(stream, gpu.upload(dense, G.BF16), m, k)
    c = gpu.zeros(G.BF16, m * n)
    G.matmul(stream, values, gpu.upload(b_bits, G.BF16), c, [m, n, k], G.MatmulOptions(metadata=metadata))
    stream.synchronize()
    assert violations.download()[0] == 0
    ours = O.bf16_to_f32(c.download()).reshape(m, n)
    a = as_tensor(dense.view(np.int16), m, k, torch.bfloat16)
    b = as_tensor(b_bits.view(np.int16), n, k, torch.bfloat16)
    theirs = torch.matmul(a, b.T).float().cpu().numpy()
    del a, b
    rows = np.arange(0, m, 131)
    expected = O.matmul_rows(O.FMT_BF16, dense, b_bits, n, k, rows)
    assert relative_error(theirs[rows].astype(np.float64), expected) <= 1e-2
    error = np.abs(ours - theirs) / np.maximum(np.abs(theirs), 1.0)
    assert float(error.max()) <= 1e-2
