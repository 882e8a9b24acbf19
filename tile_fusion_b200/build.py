"""Builds libtilefusion_b200.so in-tree with nvcc for sm_100a."""
from __future__ import annotations

import os
import subprocess

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)
LIB = os.path.join(HERE, "libtilefusion_b200.so")
SOURCES = ["kernels.cu", "api.cu", "inspector.cpp", "planner.cpp", "tiling.cpp", "noalloc.cu", "gemm_tc.cu", "tile_pipeline.cu", "lattice.cpp", "lattice_march.cu", "multi.cu", "io.cpp", "reorder.cpp"]
HEADERS = ["kernels.cuh", "launch.h", "tf_internal.h", "gemm_tc.cuh", "gemm_tc_host.h", "lattice_march.h", "host_stage.h"]


def _stale() -> bool:
    if not os.path.exists(LIB):
        return True
    t = os.path.getmtime(LIB)
    deps = [os.path.join(HERE, "csrc", f) for f in SOURCES + HEADERS]
    deps.append(os.path.join(ROOT, "include", "tile_fusion_b200.h"))
    return any(os.path.getmtime(d) > t for d in deps)


def build(force: bool = False, verbose: bool = False) -> str:
    if not force and not _stale():
        return LIB
    nvcc = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
    cmd = [nvcc, "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
           "-Xcompiler", "-fPIC", "-shared", "-I" + os.path.join(ROOT, "include"),
           "-I" + os.path.join(HERE, "csrc")]
    if verbose:
        cmd += ["-Xptxas", "-v"]
    cmd += [os.path.join(HERE, "csrc", f) for f in SOURCES] + ["-ldl", "-o", LIB]
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode != 0:
        raise RuntimeError("nvcc failed:\n" + res.stdout + res.stderr)
    if verbose:
        print(res.stderr)
    return LIB


if __name__ == "__main__":
    print(build(force=True, verbose=True))
