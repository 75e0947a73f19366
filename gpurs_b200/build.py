"""Builds the native half of gpurs_b200 in-tree.

Two artefacts, both next to this file:
  libgpurs_b200.so   the C-ABI library (host code over the CUDA driver API) with the sm_100a kernel
                     image embedded in it
  kernels.fatbin     the same kernel image on its own, for hosts that load it through their own
                     module path (the reference's `Gpu::load_module`, crates/gpurs/src/raw/module.rs:64-67)

Run as `python -m gpurs_b200.build`.  nvcc cross-compiles for sm_100a without a GPU.
"""
from __future__ import annotations

import os
import subprocess
import sys
from pathlib import Path

PACKAGE = Path(__file__).resolve().parent
CSRC = PACKAGE / "csrc"
LIBRARY = PACKAGE / "libgpurs_b200.so"
IMAGE = PACKAGE / "kernels.fatbin"
CUDA_HOME = Path(os.environ.get("CUDA_HOME", "/usr/local/cuda"))

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "--expt-relaxed-constexpr", "-Xptxas", "-v",
]


def _run(command: list[str], log: list[str]) -> None:
    done = subprocess.run(command, capture_output=True, text=True)
    log.append("$ " + " ".join(command))
    log.append(done.stdout + done.stderr)
    if done.returncode != 0:
        sys.stderr.write("\n".join(log[-2:]))
        raise RuntimeError(f"build step failed: {' '.join(command[:3])} ...")


def _newest(paths) -> float:
    return max(p.stat().st_mtime for p in paths)


def build(force: bool = False, verbose: bool = False) -> Path:
    kernels = sorted((CSRC / "kernels").glob("*.cu"))
    kernel_deps = kernels + sorted((CSRC / "kernels").glob("*.cuh")) + sorted((CSRC / "kernels").glob("*.hpp"))
    host = sorted((CSRC / "host").glob("*.cpp"))
    host_cuda = sorted((CSRC / "host").glob("*.cu"))   # host code that needs the CUDA runtime (static device data)
    host_deps = host + host_cuda + sorted((CSRC / "kernels").glob("*.hpp")) + sorted((CSRC / "host").glob("*.hpp")) + [CSRC / "host" / "image.S", PACKAGE.parent / "include" / "gpurs_b200.h"]
    log: list[str] = []
    nvcc = str(CUDA_HOME / "bin" / "nvcc")
    if force or not IMAGE.exists() or IMAGE.stat().st_mtime < _newest(kernel_deps):
        objects = []
        scratch = PACKAGE / "build"
        scratch.mkdir(exist_ok=True)
        # One relocatable-free fatbin per source would need several modules at run time; compile all
        # kernels as one translation unit list into a single image instead.
        unit = scratch / "all_kernels.cu"
        unit.write_text("".join(f'#include "{k}"\n' for k in kernels))
        # --no-compress: the entry names stay readable in the image (a host, or a test without a GPU, can list them)
        _run([nvcc, *NVCC_FLAGS, "--no-compress", "-I", str(CSRC / "kernels"), "-fatbin", "-o", str(IMAGE), str(unit)], log)
        (scratch / "ptxas.log").write_text(log[-1])
        del objects
    if force or not LIBRARY.exists() or LIBRARY.stat().st_mtime < max(_newest(host_deps), IMAGE.stat().st_mtime):
        scratch = PACKAGE / "build"
        scratch.mkdir(exist_ok=True)
        objects = []
        for source in host_cuda:
            target = scratch / (source.stem + ".o")
            _run([nvcc, *NVCC_FLAGS, "-Xcompiler", "-fPIC,-fvisibility=hidden", "-c", str(source), "-o", str(target)], log)
            objects.append(str(target))
        _run(["g++", "-std=c++17", "-O2", "-fPIC", "-shared", "-fvisibility=hidden", "-Wall", "-Wextra",
              "-I", str(CUDA_HOME / "include"), f'-DGPURS_IMAGE_PATH="{IMAGE}"',
              *[str(h) for h in host], str(CSRC / "host" / "image.S"), *objects,
              "-o", str(LIBRARY), "-L", str(CUDA_HOME / "lib64"), "-lcudart_static", "-lrt", "-ldl", "-lpthread",
              # keep the statically linked CUDA runtime private to this library: another copy (torch's) may
              # live in the same process
              "-Wl,--exclude-libs,ALL", "-Wl,-Bsymbolic"], log)
    if verbose:
        print("\n".join(log))
    return LIBRARY


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv))
