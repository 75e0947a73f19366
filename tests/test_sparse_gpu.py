"""2:4 structured-sparse products on a B200: the device compressor against the oracle's, and the sparse
GEMM against the fp64 product of the densified operand.  The reference has no sparse path, so parity here is
against the oracle alone (unpinned by the reference)."""
import numpy as np
import pytest

import gpurs_b200 as G
from gpurs_b200 import _ffi
import oracle as O
from helpers import decode_output, relative_error, spread_rows

pytestmark = pytest.mark.gpu


def metadata_offset(row, k):
    """gemm::metadata_offset of gpurs_b200/csrc/kernels/gemm_sparse_tcgen05.cuh."""
    return 16 * (row % 8) + 2 * ((row // 8) % 2) + 256 * (row // 16) + 128 * ((k // 16) % 2) + 4 * (k // 32) + (k % 16) // 8


def decode_metadata(raw, m, k):
    """The 4-bit position pair of every group of four, row-major, from the block layout."""
    raw = raw.view(np.uint8)
    rows, starts = np.arange(m)[:, None], (np.arange(k // 4) * 4)[None, :]
    block = (rows // 128) * (k // 128) + starts // 128
    byte = raw[block * 2048 + metadata_offset(rows % 128, starts % 128)]
    return ((byte >> (4 * ((starts % 8) // 4))) & 0xF).reshape(-1)


def sparse_product(gpu, stream, dense, b, m, n, k, out, algorithm, fmt=G.BF16, **options):
    values, metadata, violations = G.compress_24(stream, gpu.upload(dense, fmt), m, k)
    c = gpu.allocate({"f32": G.F32, "bf16": G.BF16}[out], m * n)
    gpu._lib.gpurs_fill_u8(stream._handle, c.pointer, 0x7F, c.nbytes)
    G.matmul(stream, values, gpu.upload(b, fmt), c, [m, n, k], G.MatmulOptions(algorithm=algorithm, metadata=metadata, **options))
    stream.synchronize()
    assert violations.download()[0] == 0
    return decode_output(c.download(), out).reshape(m, n)


@pytest.mark.parametrize("shape", [(128, 128), (200, 256), (384, 1024)])
def test_compressor_matches_oracle(gpu, stream, shape):
    m, k = shape
    dense = O.fill_sparse24_bf16(m, k, 5)
    values, metadata, violations = G.compress_24(stream, gpu.upload(dense, G.BF16), m, k)
    stream.synchronize()
    expected_values, expected_positions, _ = O.compress_24(dense, m, k)
    assert np.array_equal(values.download(), expected_values)
    assert np.array_equal(decode_metadata(metadata.download(), m, k), expected_positions)
    assert violations.download()[0] == 0
    assert metadata.len == gpu._lib.gpurs_metadata_bytes(m, k) == -(-m // 128) * (k // 128) * 2048


def test_compressor_pads_sparse_groups_and_counts_violations(gpu, stream):
    m, k = 128, 128
    dense = O.fill_sparse24_bf16(m, k, 6)
    dense[0:4] = 0                      # an empty group: keeps positions 0 and 1
    dense[4:8] = [0, 0, 0, 0x3F80]      # one non-zero at position 3: keeps 0 and 3
    dense[8:12] = 0x3F80                # four non-zeros: not 2:4
    values, metadata, violations = G.compress_24(stream, gpu.upload(dense, G.BF16), m, k)
    stream.synchronize()
    expected_values, expected_positions, expected_violations = O.compress_24(dense, m, k)
    assert expected_violations == 1 and violations.download()[0] == 1
    positions = decode_metadata(metadata.download(), m, k)
    assert list(positions[:2]) == [0b0100, 0b1100]
    assert np.array_equal(positions, expected_positions) and np.array_equal(values.download(), expected_values)


@pytest.mark.parametrize("algorithm", [G.ALGO_SINGLE_CTA, G.ALGO_CTA_PAIR])
@pytest.mark.parametrize("out,tolerance", [("f32", 1e-3), ("bf16", 1e-2)])
@pytest.mark.parametrize("shape", [(128, 256, 128), (200, 300, 256), (384, 768, 1024), (129, 257, 2048)])
def test_sparse_product_matches_densified_oracle(gpu, stream, shape, out, tolerance, algorithm):
    m, n, k = shape
    dense, b = O.fill_sparse24_bf16(m, k, 3), O.fill_normal_16(O.FMT_BF16, n * k, 4)
    got = sparse_product(gpu, stream, dense, b, m, n, k, out, algorithm)
    assert relative_error(got, O.matmul_rows(O.FMT_BF16, dense, b, n, k, np.arange(m))) <= tolerance


def test_sparse_f16(gpu, stream):
    m, n, k = 256, 256, 512
    dense_bf16 = O.fill_sparse24_bf16(m, k, 7)
    dense = O.f16_from_f32(O.bf16_to_f32(dense_bf16))          # same pattern and values, stored as binary16
    b = O.fill_normal_16(O.FMT_F16, n * k, 8)
    got = sparse_product(gpu, stream, dense, b, m, n, k, "f32", G.ALGO_AUTO, fmt=G.F16)
    assert relative_error(got, O.matmul_rows(O.FMT_F16, dense, b, n, k, np.arange(m))) <= 1e-3


def test_sparse_equals_dense_kernel_on_the_same_matrix(gpu, stream):
    """The sparse kernel on compressed A and the dense kernel on the densified A compute the same sums."""
    m, n, k = 512, 512, 1024
    dense, b = O.fill_sparse24_bf16(m, k, 9), O.fill_normal_16(O.FMT_BF16, n * k, 10)
    sparse = sparse_product(gpu, stream, dense, b, m, n, k, "f32", G.ALGO_CTA_PAIR)
    c = gpu.zeros(G.F32, m * n)
    G.matmul(stream, gpu.upload(dense, G.BF16), gpu.upload(b, G.BF16), c, [m, n, k])
    stream.synchronize()
    # not bit for bit: a sparse instruction sums 32 logical K at a time, a dense one 16, and the fp32
    # accumulator of the tensor core truncates after each
    assert relative_error(sparse, c.download().reshape(m, n).astype(np.float64)) <= 1e-4


@pytest.mark.parametrize("out", ["f32", "bf16"])
@pytest.mark.parametrize("shape,max_ctas", [((512, 224, 128), 0), ((512, 448, 1024), 0), ((700, 500, 1024), 0), ((129, 257, 2048), 0), ((1536, 1000, 512), 4),
                                            ((2048, 2240, 256), 0)])
def test_tall_tiles_equal_the_256_row_tiles(gpu, stream, shape, max_ctas, out):
    """512 x 224 pair tiles sum every output in the same order as the 256 x 224 ones: bit-equal, ragged edges, several tiles
    per pair (max_ctas 4); both agree with the densified oracle product.  With output algebra the flag changes nothing (that
    product stays on the 256-row tiles)."""
    m, n, k = shape
    dense, b = O.fill_sparse24_bf16(m, k, 21), O.fill_normal_16(O.FMT_BF16, n * k, 22)
    tall = sparse_product(gpu, stream, dense, b, m, n, k, out, G.ALGO_CTA_PAIR | G.ALGO_WIDE_TILES, max_ctas=max_ctas)
    short = sparse_product(gpu, stream, dense, b, m, n, k, out, G.ALGO_CTA_PAIR | G.ALGO_SQUARE_TILES, max_ctas=max_ctas)
    assert np.array_equal(tall, short)
    rows = spread_rows(m, 16)
    assert relative_error(tall[rows], O.matmul_rows(O.FMT_BF16, dense, b, n, k, rows)) <= (1e-3 if out == "f32" else 1e-2)
    bias = gpu.upload(np.linspace(-2, 2, n, dtype=np.float32), G.F32)
    assert np.array_equal(sparse_product(gpu, stream, dense, b, m, n, k, out, G.ALGO_CTA_PAIR | G.ALGO_WIDE_TILES, max_ctas=max_ctas, bias=bias),
                          sparse_product(gpu, stream, dense, b, m, n, k, out, G.ALGO_CTA_PAIR | G.ALGO_SQUARE_TILES, max_ctas=max_ctas, bias=bias))


def test_tall_tiles_f16(gpu, stream):
    m, n, k = 1024, 448, 512
    dense = O.f16_from_f32(O.bf16_to_f32(O.fill_sparse24_bf16(m, k, 23)))
    b = O.fill_normal_16(O.FMT_F16, n * k, 24)
    tall = sparse_product(gpu, stream, dense, b, m, n, k, "f32", G.ALGO_CTA_PAIR | G.ALGO_WIDE_TILES, fmt=G.F16)
    assert np.array_equal(tall, sparse_product(gpu, stream, dense, b, m, n, k, "f32", G.ALGO_CTA_PAIR | G.ALGO_SQUARE_TILES, fmt=G.F16))
    assert relative_error(tall, O.matmul_rows(O.FMT_F16, dense, b, n, k, np.arange(m))) <= 1e-3


@pytest.mark.parametrize("algorithm,max_ctas,shape", [(G.ALGO_CTA_PAIR | G.ALGO_SPLIT_LAST_ROUND | G.ALGO_SQUARE_TILES, 8, (512, 1120, 1024)),
                                                       (G.ALGO_SINGLE_CTA | G.ALGO_SPLIT_LAST_ROUND, 6, (640, 672, 512)),
                                                       (G.ALGO_CTA_PAIR | G.ALGO_SQUARE_TILES, 0, (256, 448, 8192)),
                                                       (G.ALGO_SINGLE_CTA, 0, (200, 300, 6144))])
@pytest.mark.parametrize("out", ["f32", "bf16"])
def test_sparse_tiles_split_along_k(gpu, stream, algorithm, max_ctas, shape, out):
    """The stream-K schedule on the sparse kernel: a last round split by force on a small grid (10 pair tiles on 4 pairs, 15
    tiles on 6 CTAs), and few tiles with a deep K split among idle groups by default.  Against the densified oracle product,
    close to the whole-tile product, and the same bits on every run."""
    m, n, k = shape
    dense, b = O.fill_sparse24_bf16(m, k, 41), O.fill_normal_16(O.FMT_BF16, n * k, 42)
    got = sparse_product(gpu, stream, dense, b, m, n, k, out, algorithm, max_ctas=max_ctas)
    rows = spread_rows(m, 12)
    assert relative_error(got[rows], O.matmul_rows(O.FMT_BF16, dense, b, n, k, rows)) <= (1e-3 if out == "f32" else 1e-2)
    whole = sparse_product(gpu, stream, dense, b, m, n, k, out, (algorithm & ~G.ALGO_SPLIT_LAST_ROUND) | G.ALGO_WHOLE_TILES, max_ctas=max_ctas)
    assert relative_error(got, whole) <= (1e-3 if out == "f32" else 1e-2)      # another order of the tensor core's truncating adds (8192 deep: 5e-4)
    assert np.array_equal(got, sparse_product(gpu, stream, dense, b, m, n, k, out, algorithm, max_ctas=max_ctas))
    assert gpu.status() == [0, 0, 0, 0]


def test_sparse_with_a_row_major_right_operand(gpu, stream):
    """B stored k x n, as the sparse configuration states C = A * B: copied transposed into the workspace, same bits as n x k."""
    m, n, k = 512, 448, 1024
    dense, b = O.fill_sparse24_bf16(m, k, 31), O.fill_normal_16(O.FMT_BF16, n * k, 32)
    expected = sparse_product(gpu, stream, dense, b, m, n, k, "bf16", G.ALGO_AUTO)
    row_major = np.ascontiguousarray(b.reshape(n, k).T).reshape(-1)
    assert np.array_equal(sparse_product(gpu, stream, dense, row_major, m, n, k, "bf16", G.ALGO_AUTO, b_row_major=True), expected)


def test_sparse_configuration_shard(gpu, stream):
    """One GPU's share of the sparse configuration: A 2048 x 8192 (of 16384 x 8192, 2:4), B 8192 x 8192,
    bf16 out, max rel err 1e-2 against the densified fp64 product."""
    m, n, k = 2048, 8192, 8192
    dense, b = O.fill_sparse24_bf16(m, k, 11), O.fill_normal_16(O.FMT_BF16, n * k, 12)
    got = sparse_product(gpu, stream, dense, b, m, n, k, "bf16", G.ALGO_AUTO)
    rows = spread_rows(m, 24)
    assert relative_error(got[rows], O.matmul_rows(O.FMT_BF16, dense, b, n, k, rows)) <= 1e-2
    indices = O.reference_sample_indices(m, n)
    assert relative_error(got.reshape(-1)[indices], O.matmul_samples(O.FMT_BF16, dense, b, n, k, indices)) <= 1e-2


def test_sparse_rejections(gpu, stream):
    values, b, c = gpu.zeros(G.BF16, 128 * 64), gpu.zeros(G.BF16, 256 * 128), gpu.zeros(G.F32, 128 * 256)
    metadata = gpu.zeros(G.I8, 2048)

    def code(call):
        with pytest.raises(G.GpursError) as raised:
            call()
        return raised.value.code

    before = gpu.launches
    assert code(lambda: G.matmul(stream, values, b, c, [128, 256, 64], G.MatmulOptions(metadata=metadata))) == _ffi.E_INVALID_VIEW   # depth not a multiple of 128
    assert code(lambda: G.matmul(stream, values, b, c, [256, 256, 128], G.MatmulOptions(metadata=metadata))) == _ffi.E_LENGTH_MISMATCH
    i8 = gpu.zeros(G.I8, 128 * 128)
    assert code(lambda: G.matmul(stream, i8, i8, gpu.zeros(G.I32, 128 * 128), [128, 128, 128], G.MatmulOptions(metadata=metadata))) == _ffi.E_INVALID_ARGUMENT
    assert gpu._lib.gpurs_compress_24(stream._handle, G.BF16, 128, 100, b.pointer, 0, values.pointer, metadata.pointer, 0) == _ffi.E_INVALID_VIEW
    assert gpu._lib.gpurs_compress_24(stream._handle, G.F32, 128, 128, b.pointer, 0, values.pointer, metadata.pointer, 0) == _ffi.E_INVALID_ARGUMENT
    assert gpu.launches == before
