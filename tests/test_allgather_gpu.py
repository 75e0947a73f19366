"""The M-sharded product whose epilogue stores every block of C into all ranks' copies of the gathered matrix.

The kernels of different ranks never wait on one another, so the ranks of these tests can share one GPU: first as
successive calls of one process (the "peers" are further allocations of the same device), then as two processes that map
each other's copy through CUDA IPC, which is the form a box of GPUs uses."""
import ctypes as C
import multiprocessing

import numpy as np
import pytest

import gpurs_b200 as G
from gpurs_b200 import _ffi
from gpurs_b200.sharding import shard_table
import oracle as O
from helpers import KINDS, OUTPUTS, make_operands, run_matmul

pytestmark = pytest.mark.gpu


def gather_in_one_process(gpu, stream, kind, out, a_bits, b_bits, m, n, k, world, **options):
    """All ranks' calls from this process; returns every rank's copy of the gathered matrix."""
    element = KINDS[kind][0]
    b = gpu.upload(b_bits, element)
    copies = [gpu.allocate(OUTPUTS[out], m * n) for _ in range(world)]
    for copy in copies:
        gpu._lib.gpurs_fill_u8(stream._handle, copy.pointer, 0x7F, copy.nbytes)
    for rank, (first, rows) in enumerate(shard_table(m, world)):
        a = gpu.upload(a_bits[first * k:(first + rows) * k], element) if rows else gpu.allocate(element, 16)
        desc = _ffi.MatmulDesc()
        desc.a_type, desc.c_type, desc.m, desc.n, desc.k = element, OUTPUTS[out], rows, n, k
        desc.bias = options["bias"].pointer if "bias" in options else 0
        desc.algorithm = options.get("algorithm", 0)
        if "row_bias" in options:
            desc.row_bias = options["row_bias"].pointer + 4 * first      # the local product's rows start at the block's first row
        if "scale_a" in options:
            # block-scaled E4M3: one fp32 scale per row of A and 128 of K, or (MX) a tile of 512 bytes per 128 rows and 128 of K
            desc.scale_kind = options.get("scale_kind", _ffi.SCALES_FP32_BLOCKS)
            per_row_block = 512 * ((k + 127) // 128)
            desc.scale_a = options["scale_a"].pointer + (first // 128 * per_row_block if desc.scale_kind == _ffi.SCALES_MX else 4 * first * ((k + 127) // 128))
            desc.scale_b = options["scale_b"].pointer
        gather = _ffi.GatherDesc()
        gather.world, gather.rank, gather.row_offset, gather.total_rows = world, rank, first, m
        for peer, copy in enumerate(copies):
            gather.full[peer] = copy.pointer
        code = gpu._lib.gpurs_matmul_allgather(stream._handle, C.byref(desc), C.byref(gather), a.pointer, b.pointer)
        assert code == 0, str(G.GpursError(code))
    stream.synchronize()
    return [copy.download() for copy in copies]


@pytest.mark.parametrize("kind,out", [("bf16", "bf16"), ("f16", "f32"), ("i8", "i32"), ("e4m3", "bf16")])
@pytest.mark.parametrize("m,n,k,world", [(512, 512, 256, 2), (1000, 520, 144, 3), (2048, 1024, 512, 8), (300, 264, 64, 4)])
def test_every_copy_holds_the_whole_product(gpu, stream, kind, out, m, n, k, world):
    """Every rank's copy equals the single-GPU product of the whole matrices bit for bit (same tiles, same order of
    accumulation); ragged last blocks, ranks without rows (m = 300 over 4 ranks) and partial tiles included."""
    a_bits, b_bits = make_operands(kind, m, n, k)
    whole = run_matmul(gpu, stream, kind, out, a_bits, b_bits, m, n, k, algorithm=G.ALGO_CTA_PAIR)
    for copy in gather_in_one_process(gpu, stream, kind, out, a_bits, b_bits, m, n, k, world):
        assert np.array_equal(copy, whole)


def test_int8_gather_matches_the_oracle_exactly(gpu, stream):
    m, n, k, world = 1024, 512, 512, 4
    a_bits, b_bits = make_operands("i8", m, n, k)
    rows = np.arange(0, m, 7)
    expected = O.matmul_rows(O.FMT_I8, a_bits, b_bits, n, k, rows)
    for copy in gather_in_one_process(gpu, stream, "i8", "i32", a_bits, b_bits, m, n, k, world):
        assert np.array_equal(copy.reshape(m, n)[rows].astype(np.int64), expected.astype(np.int64))


def test_bias_is_added_before_the_push(gpu, stream):
    m, n, k = 512, 384, 128
    a_bits, b_bits = make_operands("f16", m, n, k)
    bias = gpu.upload((np.arange(n) / 8.0).astype(np.float32))
    whole = run_matmul(gpu, stream, "f16", "f32", a_bits, b_bits, m, n, k, algorithm=G.ALGO_CTA_PAIR, bias=bias)
    for copy in gather_in_one_process(gpu, stream, "f16", "f32", a_bits, b_bits, m, n, k, 2, bias=bias):
        assert np.array_equal(copy, whole)


@pytest.mark.parametrize("kind,out", [("bf16", "bf16"), ("bf16", "f32"), ("i8", "i32"), ("f32", "f32")])
@pytest.mark.parametrize("m,n,k,world", [(512, 512, 256, 2), (1000, 520, 144, 3), (4096, 1024, 128, 2), (8192, 512, 64, 8), (300, 264, 64, 4)])
def test_copy_engine_form_fills_every_copy(gpu, stream, kind, out, m, n, k, world):
    """GPURS_ALGO_GATHER_BY_COPIES: the block in bands of rows (four bands of 512 rows for the 2048-row blocks here), every band
    sent to the other copies by copy streams: each copy equals the single-GPU product bit for bit, for output types the push
    kernels do not have as well (the bands are plain products)."""
    a_bits, b_bits = make_operands(kind, m, n, k)
    whole = run_matmul(gpu, stream, kind, out, a_bits, b_bits, m, n, k)
    for copy in gather_in_one_process(gpu, stream, kind, out, a_bits, b_bits, m, n, k, world, algorithm=G.ALGO_GATHER_BY_COPIES):
        assert np.array_equal(copy, whole)


def test_copy_engine_form_offsets_the_row_vectors(gpu, stream):
    m, n, k, world = 4096, 384, 128, 2
    a_bits, b_bits = make_operands("f16", m, n, k)
    bias = gpu.upload((np.arange(n) / 8.0).astype(np.float32))
    row_bias = gpu.upload((np.arange(m) % 97).astype(np.float32))
    whole = run_matmul(gpu, stream, "f16", "f32", a_bits, b_bits, m, n, k, bias=bias, row_bias=row_bias)
    for copy in gather_in_one_process(gpu, stream, "f16", "f32", a_bits, b_bits, m, n, k, world, bias=bias, row_bias=row_bias,
                                      algorithm=G.ALGO_GATHER_BY_COPIES):
        assert np.array_equal(copy, whole)


def test_copy_engine_form_offsets_the_scales_of_a_block_scaled_product(gpu, stream):
    """Bands of a block-scaled E4M3 product take their own rows of the A scales: every copy equals the product made in one piece."""
    m, n, k, world = 4096, 384, 512, 2
    a_source, b_source = O.fill_normal_f32(m * k, 5), O.fill_normal_f32(n * k, 6)
    a_bits, sa = O.quantize_e4m3(a_source, m, k, 1)
    b_bits, sb = O.quantize_e4m3(b_source, n, k, 128)
    scale_a, scale_b = gpu.upload(sa), gpu.upload(sb)
    whole = run_matmul(gpu, stream, "e4m3", "f32", a_bits, b_bits, m, n, k, scale_a=scale_a, scale_b=scale_b)
    for copy in gather_in_one_process(gpu, stream, "e4m3", "f32", a_bits, b_bits, m, n, k, world, scale_a=scale_a, scale_b=scale_b,
                                      algorithm=G.ALGO_GATHER_BY_COPIES):
        assert np.array_equal(copy, whole)


def test_copy_engine_form_offsets_the_tiled_scales_of_an_mx_product(gpu, stream):
    m, n, k, world = 2048, 448, 256, 2
    a_codes, scale_a = G.quantize_mx_e4m3(stream, gpu.upload(O.fill_normal_f32(m * k, 7)), m, k, False)
    b_codes, scale_b = G.quantize_mx_e4m3(stream, gpu.upload(O.fill_normal_f32(n * k, 8)), n, k, True)
    stream.synchronize()
    a_bits, b_bits = a_codes.download(), b_codes.download()
    scales = dict(scale_a=scale_a, scale_b=scale_b, scale_kind=_ffi.SCALES_MX)
    whole = run_matmul(gpu, stream, "e4m3", "bf16", a_bits, b_bits, m, n, k, **scales)
    for copy in gather_in_one_process(gpu, stream, "e4m3", "bf16", a_bits, b_bits, m, n, k, world, algorithm=G.ALGO_GATHER_BY_COPIES, **scales):
        assert np.array_equal(copy, whole)


def test_arguments_the_gathering_product_rejects(gpu, stream):
    lib = gpu._lib
    a, b, full = gpu.zeros(G.BF16, 256 * 64), gpu.zeros(G.BF16, 256 * 64), gpu.zeros(G.BF16, 512 * 256)

    def call(m=256, total=512, offset=0, world=2, rank=0, a_type=G.BF16, c_type=G.BF16, pointer=None, algorithm=0, n=256):
        desc = _ffi.MatmulDesc()
        desc.a_type, desc.c_type, desc.m, desc.n, desc.k, desc.algorithm = a_type, c_type, m, n, 64, algorithm
        gather = _ffi.GatherDesc()
        gather.world, gather.rank, gather.row_offset, gather.total_rows = world, rank, offset, total
        for peer in range(min(world, 8)):
            gather.full[peer] = full.pointer if pointer is None else pointer
        return lib.gpurs_matmul_allgather(stream._handle, C.byref(desc), C.byref(gather), a.pointer, b.pointer)

    assert call() == 0
    assert call(world=9) == _ffi.E_INVALID_ARGUMENT
    assert call(world=0) == _ffi.E_INVALID_ARGUMENT
    assert call(rank=2) == _ffi.E_INVALID_ARGUMENT
    assert call(offset=384) == _ffi.E_LENGTH_MISMATCH                 # 384 + 256 > 512
    assert call(m=100, offset=0) == _ffi.E_INVALID_VIEW               # a block that is not the last must be whole boxes of 32 rows
    assert call(m=100, offset=412) == 0                               # ... the last one may be ragged
    assert call(c_type=G.F32) == _ffi.E_INVALID_ARGUMENT              # bf16 -> f32 has no push kernel
    assert call(a_type=G.E4M3, c_type=G.F32) == _ffi.E_INVALID_ARGUMENT   # nor has e4m3 -> f32
    assert call(pointer=a.pointer) == _ffi.E_ALIASING                  # a copy of the result over an operand
    assert call(pointer=full.pointer + 2) == _ffi.E_INVALID_VIEW      # base not on a 16-byte boundary
    assert call(n=250) == _ffi.E_INVALID_VIEW                         # pitch of 500 bytes
    assert call(algorithm=G.ALGO_SINGLE_CTA) == _ffi.E_INVALID_ARGUMENT
    assert call(pointer=0) == _ffi.E_INVALID_ARGUMENT
    stream.synchronize()
    assert gpu.status()[0] == 0


def _rank_process(rank, world, m, n, k, inbox, outboxes, results):
    """One rank of the two-process test: own Gpu handle on device 0, own copy, peers mapped through IPC."""
    try:
        gpu = G.Gpu(0)
        stream = gpu.stream()
        a_bits, b_bits = make_operands("bf16", m, n, k)

        def exchange(handle):
            for peer, box in enumerate(outboxes):
                if peer != rank:
                    box.put((rank, handle))
            handles = {rank: handle}
            while len(handles) < world:
                sender, raw = inbox.get(timeout=120)
                handles[sender] = raw
            return [handles[r] for r in range(world)]

        gathered = G.GatheredMatrix(gpu, G.BF16, m, n, rank, world, exchange)
        first, rows = shard_table(m, world)[rank]
        a = gpu.upload(a_bits[first * k:(first + rows) * k], G.BF16)
        b = gpu.upload(b_bits, G.BF16)
        G.matmul_allgather(stream, a, b, gathered, [rows, n, k], first)
        stream.synchronize()
        exchange(b"done")                       # host barrier: every rank's kernel has completed
        results.put((rank, gathered.local.download().tobytes(), gpu.status()[0]))
        exchange(b"read")                       # nobody unmaps while a peer may still be reading
        gathered.close()
    except Exception as error:                  # pragma: no cover - reported to the parent
        results.put((rank, repr(error), -1))


def test_two_processes_exchange_blocks_through_ipc(gpu, stream):
    """Two processes, each with its own copy of the gathered matrix and an IPC mapping of the other's: after both have
    run their kernel and met, both copies hold the whole product."""
    m, n, k, world = 1024, 512, 256, 2
    a_bits, b_bits = make_operands("bf16", m, n, k)
    whole = run_matmul(gpu, stream, "bf16", "bf16", a_bits, b_bits, m, n, k, algorithm=G.ALGO_CTA_PAIR)
    context = multiprocessing.get_context("spawn")
    inboxes = [context.Queue() for _ in range(world)]
    results = context.Queue()
    workers = [context.Process(target=_rank_process, args=(rank, world, m, n, k, inboxes[rank], inboxes, results)) for rank in range(world)]
    for worker in workers:
        worker.start()
    try:
        outcomes = [results.get(timeout=300) for _ in range(world)]
    finally:
        for worker in workers:
            worker.join(timeout=60)
            if worker.is_alive():
                worker.kill()
    for rank, payload, status in outcomes:
        assert status == 0, payload
        assert np.array_equal(np.frombuffer(payload, np.uint16), whole), f"rank {rank}"


@pytest.mark.parametrize("m,n,k,world", [(512, 448, 256, 2), (1024, 1000, 512, 4), (768, 224, 128, 3)])
def test_sparse_product_pushes_its_blocks_too(gpu, stream, m, n, k, world):
    """The 2:4-sparse bf16 kernel has the same push epilogue (its 224-column tiles end in a half box): every copy equals the
    single-GPU sparse product bit for bit."""
    dense = O.fill_sparse24_bf16(m, k, 7)
    b_bits = O.fill_normal_16(O.FMT_BF16, n * k, 8)
    b = gpu.upload(b_bits, G.BF16)
    values, metadata, _ = G.compress_24(stream, gpu.upload(dense, G.BF16), m, k)
    whole = gpu.zeros(G.BF16, m * n)
    G.matmul(stream, values, b, whole, [m, n, k], G.MatmulOptions(metadata=metadata, algorithm=G.ALGO_CTA_PAIR))
    stream.synchronize()
    expected = whole.download()
    copies = [gpu.allocate(G.BF16, m * n) for _ in range(world)]
    for copy in copies:
        gpu._lib.gpurs_fill_u8(stream._handle, copy.pointer, 0x7F, copy.nbytes)
    for rank, (first, rows) in enumerate(shard_table(m, world)):
        if rows == 0:
            continue
        shard_values, shard_metadata, _ = G.compress_24(stream, gpu.upload(dense[first * k:(first + rows) * k], G.BF16), rows, k)
        desc = _ffi.MatmulDesc()
        desc.a_type, desc.c_type, desc.m, desc.n, desc.k, desc.metadata = G.BF16, G.BF16, rows, n, k, shard_metadata.pointer
        gather = _ffi.GatherDesc()
        gather.world, gather.rank, gather.row_offset, gather.total_rows = world, rank, first, m
        for peer, copy in enumerate(copies):
            gather.full[peer] = copy.pointer
        code = gpu._lib.gpurs_matmul_allgather(stream._handle, C.byref(desc), C.byref(gather), shard_values.pointer, b.pointer)
        assert code == 0
        stream.synchronize()
    for copy in copies:
        assert np.array_equal(copy.download(), expected)
