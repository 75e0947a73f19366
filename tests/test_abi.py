"""The C-ABI library without a GPU: it loads, exports what the header declares, lays its structs out
as the header says, and refuses to work without a CUDA driver instead of falling back to anything."""
import ctypes as C
import re
import subprocess
from pathlib import Path

import pytest

from gpurs_b200 import _ffi

ROOT = Path(__file__).resolve().parents[1]
HEADER = (ROOT / "include" / "gpurs_b200.h").read_text()


def declared_functions():
    return sorted(set(re.findall(r"^\s*(?:const\s+)?[A-Za-z_0-9]+\s*\*?\s*(gpurs_[a-z0-9_]+)\(", HEADER, flags=re.M)))


def test_header_declares_the_expected_surface():
    names = declared_functions()
    for needed in ("gpurs_gpu_new", "gpurs_stream_new", "gpurs_upload", "gpurs_zeros", "gpurs_download", "gpurs_tensor_map_encode",
                   "gpurs_module_load", "gpurs_kernel_launch", "gpurs_matmul", "gpurs_last_error"):
        assert needed in names


def test_library_exports_every_declared_symbol():
    library = _ffi.load()
    for name in declared_functions():
        assert hasattr(library, name), f"{name} is declared in the header but not exported"


def test_binding_covers_every_declared_symbol():
    assert sorted(_ffi.SIGNATURES) == declared_functions()


def test_struct_layouts_match_a_c_compiler(tmp_path):
    source = tmp_path / "layout.c"
    source.write_text(
        '#include "gpurs_b200.h"\n#include <stdio.h>\n#include <stddef.h>\n'
        "int main(void){printf(\"%zu %zu %zu %zu %zu %zu %zu %zu %zu %zu %zu\\n\", sizeof(gpurs_matmul_desc), offsetof(gpurs_matmul_desc, m),"
        " offsetof(gpurs_matmul_desc, lda), offsetof(gpurs_matmul_desc, algorithm), offsetof(gpurs_matmul_desc, scale_a),"
        " sizeof(gpurs_launch_config), offsetof(gpurs_launch_config, cluster), offsetof(gpurs_matmul_desc, accumulate),"
        " offsetof(gpurs_matmul_desc, beta), offsetof(gpurs_matmul_desc, row_sum), offsetof(gpurs_matmul_desc, launch));return 0;}\n")
    binary = tmp_path / "layout"
    subprocess.run(["gcc", "-std=c99", "-pedantic", "-Wall", "-Werror", "-I", str(ROOT / "include"), str(source), "-o", str(binary)], check=True)
    sizes = [int(x) for x in subprocess.run([str(binary)], capture_output=True, text=True, check=True).stdout.split()]
    D, L = _ffi.MatmulDesc, _ffi.LaunchConfigStruct
    assert sizes == [C.sizeof(D), D.m.offset, D.lda.offset, D.algorithm.offset, D.scale_a.offset, C.sizeof(L), L.cluster.offset,
                     D.accumulate.offset, D.beta.offset, D.row_sum.offset, D.launch.offset]


def test_kernel_image_is_embedded():
    library = _ffi.load()
    size = C.c_size_t()
    pointer = library.gpurs_kernel_image(C.byref(size))
    assert pointer and size.value > 10000
    image = C.string_at(pointer, size.value)
    assert image == (ROOT / "gpurs_b200" / "kernels.fatbin").read_bytes()
    for entry in (b"gpurs_gemm_bf16_bf16_cg2", b"gpurs_gemm_f16_f32_cg1", b"gpurs_gemm_i8_i32_cg2"):
        assert entry in image


def test_null_arguments_are_rejected_without_a_driver():
    library = _ffi.load()
    assert library.gpurs_gpu_new(0, None) == _ffi.E_INVALID_ARGUMENT
    assert library.gpurs_stream_new(None, None) == _ffi.E_INVALID_ARGUMENT
    assert library.gpurs_matmul(None, None, 0, 0, 0) == _ffi.E_INVALID_ARGUMENT
    operation, name, description = C.c_char_p(), C.c_char_p(), C.c_char_p()
    assert library.gpurs_last_error(C.byref(operation), C.byref(name), C.byref(description)) == _ffi.E_INVALID_ARGUMENT
    assert operation.value == b"gpurs_matmul"


def test_no_cuda_driver_means_an_error_not_a_fallback():
    import torch

    if torch.cuda.is_available():
        pytest.skip("a CUDA driver is present")
    import gpurs_b200

    with pytest.raises(gpurs_b200.GpursError) as raised:
        gpurs_b200.Gpu(0)
    assert raised.value.code in (_ffi.E_DRIVER_UNAVAILABLE, 100, 3)  # no libcuda, or a stub / no device


def test_product_code_does_not_touch_the_oracle():
    """The shipped package must not import, link or read anything under oracle/."""
    for path in list((ROOT / "gpurs_b200").rglob("*.py")) + list((ROOT / "gpurs_b200" / "csrc").rglob("*.*")):
        text = path.read_text(errors="ignore")
        assert "oracle" not in text.lower() or path.name == "build.py", f"{path} mentions the oracle"


def test_kernel_sources_hold_no_multicast_loads():
    """TMA loads are never multicast across a cluster: each CTA fetches its own tiles."""
    for path in (ROOT / "gpurs_b200" / "csrc").rglob("*.cu*"):
        for line in path.read_text().splitlines():
            if "cp.async.bulk" in line:
                assert "multicast" not in line, f"{path}: {line.strip()}"
