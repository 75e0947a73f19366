"""The C++ mirror of the host surface (gpurs_b200/cpp/gpurs.hpp) and the reference's Blackwell example ported
onto it (gpurs_b200/cpp/blackwell_matrix.cpp)."""
import re
import subprocess
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parents[1]
PACKAGE = ROOT / "gpurs_b200"


@pytest.fixture(scope="module")
def example(tmp_path_factory):
    binary = tmp_path_factory.mktemp("cpp") / "blackwell_matrix"
    subprocess.run(["g++", "-std=c++17", "-O2", "-Wall", "-Wextra", "-Werror", str(PACKAGE / "cpp" / "blackwell_matrix.cpp"), "-o", str(binary),
                    "-L", str(PACKAGE), "-lgpurs_b200", f"-Wl,-rpath,{PACKAGE}"], check=True)
    return binary


def test_example_builds_and_refuses_to_run_without_a_driver(example):
    import torch

    if torch.cuda.is_available():
        pytest.skip("a CUDA driver is present")
    done = subprocess.run([str(example), "128"], capture_output=True, text=True)
    assert done.returncode == 2 and "gpurs_gpu_new" in done.stderr


@pytest.mark.gpu
@pytest.mark.parametrize("size", [320, 4096])
def test_example_reproduces_the_reference_check(example, size):
    """The reference's own self-check (sampled fp64 loop, bound 1e-2) passes, with error exactly zero."""
    done = subprocess.run([str(example), str(size)], capture_output=True, text=True, timeout=600)
    assert done.returncode == 0, done.stderr
    line = re.fullmatch(rf"{size}x{size}x{size}: ([0-9.]+) ms, ([0-9.]+) TFLOP/s, max abs error ([0-9.e+-]+)\n", done.stdout)
    assert line, done.stdout
    assert float(line.group(3)) == 0.0
