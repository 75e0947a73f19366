"""The CUDA restatement of the reference kernel's design (oracle/reference_design.cu: one CTA per 128 x 256 tile, one thread
issuing the tile copies and the products, one accumulator) is the baseline the benchmark times beside the product's f16
kernel.  Here it is checked like the product: bit-exact against the CPU oracle on the reference example's inputs, whose
partial sums are all exact in fp32 (examples/matrix_benchmark.rs:5-14,36-51), and equal to the product's own result."""
import numpy as np
import pytest

import gpurs_b200 as G
import oracle as O
from oracle.reference_design import ReferenceDesign
from helpers import make_operands, run_matmul

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("m,n,k", [(512, 768, 320), (300, 520, 192), (128, 256, 64), (1024, 1024, 4096)])
def test_reference_design_reproduces_the_example_product(gpu, stream, m, n, k):
    a_bits, b_bits = make_operands("f16", m, n, k, pattern="example")
    a, b = gpu.upload(a_bits, G.F16), gpu.upload(b_bits, G.F16)
    c = gpu.allocate(G.F32, m * n)
    gpu._lib.gpurs_fill_u8(stream._handle, c.pointer, 0x7F, c.nbytes)
    design = ReferenceDesign(gpu)
    design.launch(stream, design.prepare(a, b, c, m, n, k))
    stream.synchronize()
    assert not design.status.download().any(), "a bounded wait in the baseline kernel gave up"
    got = c.download()
    rows = np.arange(m)
    assert np.array_equal(got.reshape(m, n).astype(np.float64), O.matmul_rows(O.FMT_F16, a_bits, b_bits, n, k, rows))
    assert np.array_equal(got, run_matmul(gpu, stream, "f16", "f32", a_bits, b_bits, m, n, k))
