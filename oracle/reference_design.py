"""Launcher of the CUDA restatement of the reference kernel's design (oracle/reference_design.cu).  TEST INFRASTRUCTURE:
used by the tests and by the benchmark's `reference_design` figure, never by the product.  It goes through the product's
external-module door (load an image, take a kernel, launch it with a LaunchConfig), the way a gpurs host would launch a
kernel of its own (crates/gpurs/src/raw/module.rs:64-207)."""
from __future__ import annotations

import ctypes as C
from pathlib import Path

IMAGE_PATH = Path(__file__).resolve().parent / "reference_design.fatbin"
TILE_ROWS, TILE_COLUMNS, DEPTH, STAGES, THREADS = 128, 256, 64, 4, 128
SHARED_BYTES = STAGES * (TILE_ROWS + TILE_COLUMNS) * DEPTH * 2 + 128 + 1024


class _TensorMap(C.Structure):
    _fields_ = [("opaque", C.c_uint64 * 16)]


def _aligned_tensor_map():
    backing = (C.c_uint8 * 256)()
    tensor_map = _TensorMap.from_buffer(backing, (-C.addressof(backing)) % 64)
    tensor_map._backing = backing
    return tensor_map


class ReferenceDesign:
    """The f16 -> f32 kernel of the reference's Blackwell example, restated: 128 x 256 x 64 tiles, one CTA per tile."""

    def __init__(self, gpu):
        import gpurs_b200 as G

        if not IMAGE_PATH.exists():
            raise FileNotFoundError(f"{IMAGE_PATH} is missing: run `make -C oracle` where nvcc is installed")
        self.G, self.gpu = G, gpu
        self.module = gpu.load_module(IMAGE_PATH.read_bytes())
        self.kernel = self.module.kernel("gpurs_reference_design_f16_f32")
        self.kernel.reserve_shared(SHARED_BYTES)
        self.status = gpu.zeros(G.I32, 4)

    def prepare(self, a, b, c, m: int, n: int, k: int):
        """Encodes the two operand descriptors (boxes of 64 x 128 and 64 x 256 elements, as the reference's) and returns the
        argument list of a launch."""
        G, gpu = self.G, self.gpu
        map_a, map_b = _aligned_tensor_map(), _aligned_tensor_map()
        for tensor_map, buffer, rows, box_rows in ((map_a, a, m, TILE_ROWS), (map_b, b, n, TILE_COLUMNS)):
            dims, strides, box = (C.c_uint64 * 2)(k, rows), (C.c_uint64 * 1)(k * 2), (C.c_uint32 * 2)(DEPTH, box_rows)
            code = gpu._lib.gpurs_tensor_map_encode(gpu._handle, C.addressof(tensor_map), G.F16, 2, buffer.pointer, dims, strides, box, 3, 3)
            if code != 0:
                raise G.GpursError(code)
        tiles = -(-m // TILE_ROWS) * -(-n // TILE_COLUMNS)
        config = G.LaunchConfig(grid=(tiles, 1, 1), block=(THREADS, 1, 1), shared_bytes=SHARED_BYTES)
        arguments = [map_a, map_b, C.c_uint64(c.pointer), C.c_int(m), C.c_int(n), C.c_int(k), C.c_uint64(self.status.pointer)]
        return config, arguments

    def launch(self, stream, prepared) -> None:
        config, arguments = prepared
        self.kernel.launch(stream, config, arguments)
