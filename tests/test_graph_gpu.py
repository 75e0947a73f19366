"""Recording products into a graph and replaying them (`Stream::capture` / `GraphExec::launch` in the reference,
crates/gpurs/src/host/graph/capture.rs:112-149 and graph/exec.rs:48-72)."""
import numpy as np
import pytest

import gpurs_b200 as G
from gpurs_b200 import _ffi
from helpers import KINDS, make_operands, run_matmul

pytestmark = pytest.mark.gpu


def test_replays_follow_the_buffers_contents(gpu, stream):
    """A recorded bf16 product reads its operands at replay time: new contents in the same buffers give the new product,
    bit-equal to a direct call, and nothing runs while recording."""
    m, n, k = 384, 520, 256
    first = make_operands("bf16", m, n, k, seed=1)
    second = make_operands("bf16", m, n, k, seed=7)
    a, b = gpu.upload(first[0], G.BF16), gpu.upload(first[1], G.BF16)
    c = gpu.zeros(G.BF16, m * n)
    before = gpu.launches
    graph = stream.capture(lambda s: G.matmul(s, a, b, c, [m, n, k]))
    stream.synchronize()
    assert not c.download().any()                      # recorded, not run
    executable = graph.instantiate()
    executable.launch(stream)
    stream.synchronize()
    assert np.array_equal(c.download(), run_matmul(gpu, stream, "bf16", "bf16", first[0], first[1], m, n, k))
    for buffer, bits in ((a, second[0]), (b, second[1])):
        assert gpu._lib.gpurs_copy_to_device(stream._handle, buffer.pointer, bits.ctypes.data, bits.nbytes) == 0
    launches = gpu.launches
    executable.launch(stream)
    executable.launch(stream)
    stream.synchronize()
    assert gpu.launches - launches == 2                # one kernel per replay
    assert np.array_equal(c.download(), run_matmul(gpu, stream, "bf16", "bf16", second[0], second[1], m, n, k))
    assert gpu.launches > before


def test_a_chain_of_products_is_one_submission(gpu, stream):
    """Two dependent products and a fill recorded together: y = (x W1^T) W2^T with an int8 -> int32 product beside them."""
    m, d = 256, 256
    x_bits, w1_bits = make_operands("f16", m, d, d, seed=3)
    _, w2_bits = make_operands("f16", m, d, d, seed=5)
    x, w1, w2 = (gpu.upload(bits, G.F16) for bits in (x_bits, w1_bits, w2_bits))
    hidden, y = gpu.zeros(G.F16, m * d), gpu.zeros(G.F32, m * d)
    p_bits, q_bits = make_operands("i8", m, d, d)
    p, q, r = gpu.upload(p_bits, G.I8), gpu.upload(q_bits, G.I8), gpu.zeros(G.I32, m * d)

    def record(s):
        assert gpu._lib.gpurs_fill_u8(s._handle, y.pointer, 0x7F, y.nbytes) == 0
        G.matmul(s, x, w1, hidden, [m, d, d])
        G.matmul(s, hidden, w2, y, [m, d, d])
        G.matmul(s, p, q, r, [m, d, d])

    executable = stream.capture(record).instantiate()
    executable.launch(stream)
    stream.synchronize()
    expected_hidden = run_matmul(gpu, stream, "f16", "f16", x_bits, w1_bits, m, d, d)
    assert np.array_equal(hidden.download(), expected_hidden)
    assert np.array_equal(y.download(), run_matmul(gpu, stream, "f16", "f32", expected_hidden, w2_bits, m, d, d))
    assert np.array_equal(r.download(), run_matmul(gpu, stream, "i8", "i32", p_bits, q_bits, m, d, d))


@pytest.mark.parametrize("kind,m,n,k", [("f32", 200, 136, 260), ("f16", 16, 1024, 2048)])
def test_products_that_borrow_scratch_replay_after_a_warm_up(gpu, stream, kind, m, n, k):
    """fp32 operands (split copies in scratch) and the split-K kernel (turn counters, partial sums): once the scratch
    exists a recording borrows it, and replays interleave correctly with direct calls on another stream."""
    a_bits, b_bits = make_operands(kind, m, n, k)
    expected = run_matmul(gpu, stream, kind, "f32", a_bits, b_bits, m, n, k)       # also the warm-up
    a, b = gpu.upload(a_bits, KINDS[kind][0]), gpu.upload(b_bits, KINDS[kind][0])
    c = gpu.zeros(G.F32, m * n)
    executable = stream.capture(lambda s: G.matmul(s, a, b, c, [m, n, k])).instantiate()
    other = gpu.stream()
    for _ in range(3):
        executable.launch(stream)
        assert np.array_equal(run_matmul(gpu, other, kind, "f32", a_bits, b_bits, m, n, k), expected)
    stream.synchronize()
    assert np.array_equal(c.download(), expected)
    assert gpu.status()[0] == 0


def test_scratch_cannot_grow_inside_a_capture():
    """On a fresh handle (no scratch yet) recording an fp32 product is refused, the capture still ends cleanly, and the
    handle keeps working."""
    gpu = G.Gpu(0)
    stream = gpu.stream()
    m = n = k = 128
    a_bits, b_bits = make_operands("f32", m, n, k)
    a, b, c = gpu.upload(a_bits, G.F32), gpu.upload(b_bits, G.F32), gpu.zeros(G.F32, m * n)
    with pytest.raises(G.GpursError) as raised:
        stream.capture(lambda s: G.matmul(s, a, b, c, [m, n, k]))
    assert raised.value.code == _ffi.E_INVALID_ARGUMENT
    G.matmul(stream, a, b, c, [m, n, k])
    stream.synchronize()
    assert c.download().any()


def test_a_graph_keeps_its_scratch_when_the_handle_outgrows_it():
    """A recording holds the address of the scratch block it was made with.  A later, larger product makes the handle
    take a bigger block; the old one must stay allocated for the graph, whose replays still compute the recorded product,
    and is released with the graph."""
    gpu = G.Gpu(0)
    try:
        stream = gpu.stream()
        m, n, k = 136, 200, 132
        a_bits, b_bits = make_operands("f32", m, n, k)
        expected = run_matmul(gpu, stream, "f32", "f32", a_bits, b_bits, m, n, k)        # warm-up: the first, small scratch block
        a, b = gpu.upload(a_bits, G.F32), gpu.upload(b_bits, G.F32)
        c = gpu.zeros(G.F32, m * n)
        graph = stream.capture(lambda s: G.matmul(s, a, b, c, [m, n, k]))
        executable = graph.instantiate()
        big = 1024                                                                       # 24 MiB of split copies: the block grows
        big_a, big_b = make_operands("f32", big, big, big, seed=9)
        big_expected = run_matmul(gpu, stream, "f32", "f32", big_a, big_b, big, big, big)
        for _ in range(2):
            gpu._lib.gpurs_fill_u8(stream._handle, c.pointer, 0x7F, c.nbytes)
            executable.launch(stream)
            stream.synchronize()
            assert np.array_equal(c.download(), expected)
            assert np.array_equal(run_matmul(gpu, stream, "f32", "f32", big_a, big_b, big, big, big), big_expected)
        del executable, graph            # the old block goes with the graph
        assert np.array_equal(run_matmul(gpu, stream, "f32", "f32", a_bits, b_bits, m, n, k), expected)
        assert gpu.status() == [0, 0, 0, 0]
        del a, b, c
    finally:
        gpu.close()


def test_graph_of_another_handle_is_rejected(gpu, stream):
    other = G.Gpu(0)
    c = gpu.zeros(G.F32, 64)
    graph = stream.capture(lambda s: gpu._lib.gpurs_fill_u8(s._handle, c.pointer, 1, c.nbytes))
    assert other._lib.gpurs_graph_launch(graph._handle, other.stream()._handle) == _ffi.E_CONTEXT_MISMATCH
    assert gpu._lib.gpurs_graph_launch(None, stream._handle) == _ffi.E_INVALID_ARGUMENT
    assert gpu._lib.gpurs_stream_capture_begin(None) == _ffi.E_INVALID_ARGUMENT
