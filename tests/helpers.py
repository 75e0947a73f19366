"""Shared pieces of the GPU parity tests: seeded inputs from the oracle, the launch through the public
host surface (which goes through the C ABI), and the comparison against the oracle."""
from __future__ import annotations

import numpy as np

import gpurs_b200 as G
import oracle as O

# operand kind -> (library element type, oracle format)
KINDS = {"f16": (G.F16, O.FMT_F16), "bf16": (G.BF16, O.FMT_BF16), "f32": (G.F32, O.FMT_F32), "i8": (G.I8, O.FMT_I8), "e4m3": (G.E4M3, O.FMT_E4M3)}
OUTPUTS = {"f32": G.F32, "bf16": G.BF16, "f16": G.F16, "i32": G.I32}


def make_operands(kind: str, m: int, n: int, k: int, pattern: str = "random", seed: int = 1):
    """(A bits, B bits) for an m x k left and n x k right operand."""
    fmt = KINDS[kind][1]
    if pattern == "example":  # the reference example's formula, examples/matrix_benchmark.rs:5-14
        left, right = O.example_inputs(fmt, max(m, n) * k)
        return left[: m * k].copy(), right[: n * k].copy()
    if kind in ("f16", "bf16"):
        return O.fill_normal_16(fmt, m * k, seed), O.fill_normal_16(fmt, n * k, seed + 1)
    if kind == "f32":
        return O.fill_uniform_f32(m * k, seed), O.fill_uniform_f32(n * k, seed + 1)
    if kind == "i8":
        return O.fill_int8(m * k, seed), O.fill_int8(n * k, seed + 1)
    if kind == "e4m3":
        return O.e4m3_from_f32(O.fill_normal_f32(m * k, seed)), O.e4m3_from_f32(O.fill_normal_f32(n * k, seed + 1))
    raise ValueError(kind)


def decode_output(bits: np.ndarray, out: str) -> np.ndarray:
    if out == "bf16":
        return O.bf16_to_f32(bits).astype(np.float64)
    if out == "f16":
        return O.f16_to_f32(bits).astype(np.float64)
    return bits.astype(np.float64)


def run_matmul(gpu, stream, kind, out, a_bits, b_bits, m, n, k, algorithm=G.ALGO_AUTO, **options) -> np.ndarray:
    """Upload, multiply on the GPU through the public API, download; returns the raw output array.
    The output is pre-filled with 0x7f bytes so that an element the kernel fails to write shows up."""
    a = gpu.upload(a_bits, KINDS[kind][0])
    b = gpu.upload(b_bits, KINDS[kind][0])
    ldc = options.get("ldc", 0) or n
    c = gpu.allocate(OUTPUTS[out], (m - 1) * ldc + n if m else 0)
    if c.len:
        gpu._lib.gpurs_fill_u8(stream._handle, c.pointer, 0x7F, c.nbytes)
    G.matmul(stream, a, b, c, [m, n, k], G.MatmulOptions(algorithm=algorithm, **options))
    stream.synchronize()
    return c.download()


def relative_error(got: np.ndarray, expected: np.ndarray) -> float:
    """max |got - expected| / max(|expected|, 1): the floor keeps entries near zero meaningful, as in the
    reference's grouped example (examples/ada/examples/grouped_matrix.rs:113).  NaN counts as infinite."""
    error = np.abs(got - expected) / np.maximum(np.abs(expected), 1.0)
    return float(np.where(np.isnan(error), np.inf, error).max()) if error.size else 0.0


def spread_rows(m: int, count: int = 48) -> np.ndarray:
    """Rows spread over the matrix plus the first and last few and the tile-boundary neighbours."""
    picks = [np.arange(0, m, max(1, m // count)), np.arange(min(m, 4)), np.arange(max(0, m - 4), m), np.array([127, 128, 255, 256]) % m]
    return np.unique(np.concatenate(picks))
