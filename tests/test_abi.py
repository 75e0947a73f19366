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


def test_every_kernel_the_launchers_can_name_is_in_the_image():
    """The launchers build entry names from a stem and the chosen form; a name without an entry would only fail on a GPU, for
    the shapes that choose it.  Every combination the host code can produce (csrc/host/matmul.cpp) is looked up here."""
    image = (ROOT / "gpurs_b200" / "kernels.fatbin").read_bytes()
    dense = ["f16_f32", "f16_f16", "bf16_f32", "bf16_bf16", "e4m3_f32", "e4m3_bf16", "tf32_f32", "i8_i32"]
    names = []
    for stem in dense:
        algebra = stem != "i8_i32"                      # output algebra is for float outputs
        for group in (1, 2):
            names += [f"gpurs_gemm_{stem}_cg{group}", f"gpurs_gemm_{stem}_sk_cg{group}"]
            if algebra:
                names += [f"gpurs_gemm_{stem}_ep_cg{group}", f"gpurs_gemm_{stem}_sk_ep_cg{group}"]
        if stem != "tf32_f32":                          # wide tiles: 16-bit and 8-bit operands
            names.append(f"gpurs_gemm_{stem}_w512_cg2")
            if algebra:
                names.append(f"gpurs_gemm_{stem}_w512_ep_cg2")
            if stem.endswith("32"):                     # 480-column tiles: 32-bit outputs
                names.append(f"gpurs_gemm_{stem}_w480_cg2")
    names += [f"gpurs_gemm_{stem}_push_cg2" for stem in ("bf16_bf16", "f16_f32", "i8_i32", "e4m3_bf16")]
    names += [f"gpurs_gemm_{stem}_batched_cg{group}" for stem in ("bf16_bf16", "bf16_f32", "f16_f16", "f16_f32") for group in (1, 2)]
    for stem in ("sparse_bf16_bf16", "sparse_bf16_f32", "sparse_f16_f32"):
        names += [f"gpurs_gemm_{stem}_cg1", f"gpurs_gemm_{stem}_cg2", f"gpurs_gemm_{stem}_sk_cg1", f"gpurs_gemm_{stem}_sk_cg2", f"gpurs_gemm_{stem}_t512_cg2"]
    names.append("gpurs_gemm_sparse_bf16_bf16_push_cg2")
    for stem in ("e4m3_scaled_bf16", "e4m3_scaled_f32", "tf32_promoted_f32", "e4m3_mx_bf16", "e4m3_mx_f32"):
        names += [f"gpurs_gemm_{stem}_cg{group}" for group in (1, 2)] + [f"gpurs_gemm_{stem}_sk_cg{group}" for group in (1, 2)]
    names += ["gpurs_gemm_e4m3_blockscaled_bf16_cg2", "gpurs_gemm_e4m3_blockscaled_f32_cg2"]
    names += [f"gpurs_gemm_skinny_{kind}_f32_t{tokens}" for kind in ("f16", "bf16") for tokens in (16, 32, 64)]
    names += [f"gpurs_gemm_grouped_{stem}" for stem in ("f16_f16", "f16_f32", "bf16_bf16", "bf16_f32")]
    names += ["gpurs_split_tf32", "gpurs_split_tf32_pair", "gpurs_split_tf32_transposed", "gpurs_transpose_b8", "gpurs_transpose_b16", "gpurs_transpose_b32",
              "gpurs_quantize_e4m3_rows", "gpurs_quantize_e4m3_tiles", "gpurs_quantize_mx_e4m3", "gpurs_compress_24", "gpurs_wait_probe"]
    missing = [name for name in names if (name.encode() + b"\x00") not in image]
    assert not missing, missing
