"""In-tree build of the CUDA library (nvcc, sm_100a only).

``python -m nectarml_b200.build`` compiles ``csrc/nml_api.cu`` (which includes the contraction
kernels) and ``csrc/nml_layers.cu`` (normalisation / optimizer kernels of the training step) into ``nectarml_b200/libnectarml_b200.so``.  nvcc cross-compiles without a GPU.
"""
from __future__ import annotations

import os
import subprocess
import sys

_HERE = os.path.dirname(os.path.abspath(__file__))
SOURCES = [os.path.join(_HERE, "csrc", "nml_api.cu"), os.path.join(_HERE, "csrc", "nml_layers.cu")]
HEADERS = [os.path.join(_HERE, "csrc", n) for n in ("nml_ptx.cuh", "nml_umma.cuh", "nml_prepass.cuh")] + [
    os.path.join(os.path.dirname(_HERE), "include", "nectarml_b200.h")]
OUTPUT = os.path.join(_HERE, "libnectarml_b200.so")

NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
              "-shared", "-Xcompiler", "-fPIC"]


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), "/usr/local/cuda/bin/nvcc", "nvcc"):
        if cand and (os.path.sep not in cand or os.path.exists(cand)):
            return cand
    raise RuntimeError("nvcc not found")


def up_to_date() -> bool:
    if not os.path.exists(OUTPUT):
        return False
    t = os.path.getmtime(OUTPUT)
    return all(os.path.getmtime(p) <= t for p in SOURCES + HEADERS)


def build(force: bool = False, verbose: bool = False) -> str:
    """Builds the library if sources are newer than it; returns its path."""
    if not force and up_to_date():
        return OUTPUT
    cmd = [_nvcc()] + NVCC_FLAGS + (["-Xptxas", "-v"] if verbose else []) + ["-o", OUTPUT] + SOURCES
    res = subprocess.run(cmd, capture_output=True, text=True)
    if verbose or res.returncode != 0:
        sys.stderr.write(res.stdout + res.stderr)
    if res.returncode != 0:
        raise RuntimeError("nvcc failed: " + " ".join(cmd))
    return OUTPUT


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv))
