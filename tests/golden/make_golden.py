"""Regenerates the golden fixtures in this directory.  Run from the repository root:

    python tests/golden/make_golden.py

Nothing here uses the oracle or the library under test.  The expected values come from independent
implementations: numpy's float16, torch's bfloat16 / float8_e4m3fn casts, exact integer and float64
arithmetic in numpy.  The reference project itself (Rust) cannot be built where these were made and
holds no fixtures of its own, so these files pin the oracle to the published definitions of the
formats and to the closed form of the reference's example inputs
(examples/matrix_benchmark.rs:5-14: left[i] = (i*13 mod 31)/16 - 1, right[i] = (i*7 mod 29)/16 - 1).
"""
from pathlib import Path

import numpy as np
import torch

HERE = Path(__file__).resolve().parent


def format_vectors():
    rng = np.random.default_rng(20251125)
    pieces = [rng.standard_normal(4000).astype(np.float32) * np.float32(s) for s in (1e-9, 1e-6, 1e-4, 1e-2, 1, 30, 500, 7e4, 3e38)]
    # every binary16 / E4M3 rounding boundary region: midpoints between neighbours and their float32 neighbours
    e4 = torch.arange(0, 127, dtype=torch.uint8).view(torch.float8_e4m3fn).to(torch.float32).numpy()
    mids = ((e4[:-1].astype(np.float64) + e4[1:].astype(np.float64)) / 2).astype(np.float32)
    around = np.concatenate([mids, np.nextafter(mids, np.float32(np.inf)), np.nextafter(mids, np.float32(-np.inf)), e4])
    h = np.arange(0, 0x7c00, 37, dtype=np.uint16).view(np.float16).astype(np.float32)
    hm = ((h[:-1].astype(np.float64) + h[1:].astype(np.float64)) / 2).astype(np.float32)
    special = np.array([0.0, -0.0, np.inf, -np.inf, np.nan, 65504, 65519.996, 65520, 65536, 448, 464, 465, 1e-45, 6e-8, 5.96e-8, 2.98e-8,
                        2.9802322e-8, 2.0 ** -24, 2.0 ** -25, 1.0, 1.0009766, 1.00048828125, 1.00146484375, 2.0 ** -9, 2.0 ** -10, 3 * 2.0 ** -11],
                       dtype=np.float32)
    x = np.concatenate(pieces + [around, -around, hm, -hm, special]).astype(np.float32)
    t = torch.from_numpy(x)
    f16 = x.astype(np.float16).view(np.uint16)
    bf16 = t.to(torch.bfloat16).view(torch.int16).numpy().view(np.uint16)
    # torch's e4m3fn cast does not saturate (overflow becomes NaN); the reference saturates to +-448
    clamped = torch.where(torch.isnan(t), t, t.clamp(-448.0, 448.0))
    e4m3 = clamped.to(torch.float8_e4m3fn).view(torch.uint8).numpy()
    bits = x.view(np.uint32)
    finite = (bits & 0x7f800000) != 0x7f800000
    tf32 = np.where(finite, (bits + np.uint32(0x1000)) & np.uint32(0xffffe000), bits | np.where(np.isnan(x), 0x400000, 0).astype(np.uint32))
    all16 = np.arange(65536, dtype=np.uint16)
    np.savez_compressed(HERE / "formats.npz", x=x, f16=f16, bf16=bf16, e4m3=e4m3, tf32=tf32.astype(np.uint32),
                        f16_decoded=all16.view(np.float16).astype(np.float32).view(np.uint32),
                        e4m3_decoded=torch.arange(256, dtype=torch.int32).to(torch.uint8).view(torch.float8_e4m3fn).to(torch.float32).numpy().view(np.uint32))


def example_product():
    """The reference example's own configuration, scaled down: size 320 (not a tile multiple)."""
    size = 320
    i = np.arange(size * size, dtype=np.int64)
    left = ((i * 13 % 31) / 16.0 - 1.0).reshape(size, size)
    right = ((i * 7 % 29) / 16.0 - 1.0).reshape(size, size)
    product = left @ right.T  # exact: every term is a multiple of 1/256 and the sums stay far below 2^53
    assert (product.astype(np.float32).astype(np.float64) == product).all()
    np.savez_compressed(HERE / "example_product_320.npz", size=size, product=product.astype(np.float32))


def int8_product():
    rng = np.random.default_rng(7)
    a = rng.integers(-128, 128, size=(96, 200), dtype=np.int8)
    b = rng.integers(-128, 128, size=(72, 200), dtype=np.int8)
    np.savez_compressed(HERE / "int8_product.npz", a=a, b=b, product=a.astype(np.int64) @ b.astype(np.int64).T)


def fp8_block_quantisation():
    rng = np.random.default_rng(11)
    source = rng.standard_normal((136, 300)).astype(np.float32)
    source[5, 128:256] = 0.0  # an all-zero 1x128 block: scale 1
    out = {}
    for name, block_rows in (("row", 1), ("tile", 128)):
        rows, depth = source.shape
        rb, kb = -(-rows // block_rows), -(-depth // 128)
        scales = np.ones((rb, kb), np.float32)
        codes = np.zeros_like(source, dtype=np.uint8)
        for r in range(rb):
            for k in range(kb):
                block = source[r * block_rows:(r + 1) * block_rows, k * 128:(k + 1) * 128]
                absmax = np.abs(block).max()
                scale = np.float32(absmax) / np.float32(448.0) if absmax > 0 else np.float32(1.0)
                scales[r, k] = scale
                q = torch.from_numpy((block / scale).astype(np.float32)).clamp(-448, 448).to(torch.float8_e4m3fn).view(torch.uint8).numpy()
                codes[r * block_rows:(r + 1) * block_rows, k * 128:(k + 1) * 128] = q
        out[f"{name}_codes"], out[f"{name}_scales"] = codes, scales
    np.savez_compressed(HERE / "fp8_quantisation.npz", source=source, **out)


if __name__ == "__main__":
    format_vectors()
    example_product()
    int8_product()
    fp8_block_quantisation()
    for f in sorted(HERE.glob("*.npz")):
        print(f.name, f.stat().st_size)
