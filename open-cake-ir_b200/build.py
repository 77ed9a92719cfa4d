"""Builds ``libcake_b200.so`` (every CUDA kernel of the package plus the C ABI) for sm_100a.

``nvcc`` cross-compiles without a GPU.  Flags follow the reference's rule for native code --
exact architecture, never the ``-arch`` shorthand (docs/NATIVE_CUDA_DESIGN.md:92-96).  The
library links the CUDA runtime statically and resolves the one driver entry point it needs at
run time, so it can be loaded (not run) on a machine without a driver.
"""
from __future__ import annotations

import os
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

HERE = Path(__file__).resolve().parent
CSRC = HERE / "csrc"
LIBRARY = HERE / "libcake_b200.so"
SOURCES = ("rmsnorm.cu", "gemm_fp8.cu", "moe.cu", "routing_v4.cu", "decode_gqa.cu", "decode_mla.cu", "ep.cu", "misc.cu")
# The architecture selectors are the two the target document (targets/sm_100a_native.json) declares and the
# only ones: the long form of `-gencode arch=compute_100a,code=sm_100a`.
ARCH_FLAGS = ("--gpu-architecture=compute_100a", "--gpu-code=sm_100a")
NVCC_FLAGS = (*ARCH_FLAGS, "-lineinfo", "-O3", "-std=c++17", "-Xcompiler", "-fPIC", "-Xptxas", "-v")


def _nvcc() -> str:
    for candidate in (os.environ.get("NVCC"), "/usr/local/cuda/bin/nvcc", "nvcc"):
        if candidate and (os.path.sep not in candidate or os.path.exists(candidate)):
            return candidate
    raise RuntimeError("nvcc not found")


def is_stale() -> bool:
    if not LIBRARY.exists():
        return True
    built = LIBRARY.stat().st_mtime
    deps = list(CSRC.glob("*.cu")) + list(CSRC.glob("*.cuh")) + [HERE.parent / "include" / "cake_b200.h"]
    return any(p.stat().st_mtime > built for p in deps)


def build_library(force: bool = False, verbose: bool = False) -> Path:
    if not force and not is_stale():
        return LIBRARY
    out = HERE / "build"
    out.mkdir(exist_ok=True)
    nvcc = _nvcc()

    def compile_one(name: str):
        obj = out / (name + ".o")
        cmd = [nvcc, *NVCC_FLAGS, "-c", str(CSRC / name), "-o", str(obj)]
        done = subprocess.run(cmd, capture_output=True, text=True)
        if done.returncode != 0:
            raise RuntimeError(f"nvcc failed on {name}:\n{done.stderr}")
        (out / (name + ".ptxas.txt")).write_text(done.stderr)
        return obj

    with ThreadPoolExecutor(max_workers=len(SOURCES)) as pool:
        objects = list(pool.map(compile_one, SOURCES))
    link = [nvcc, "-shared", "-o", str(LIBRARY), *map(str, objects), "-cudart", "static"]
    done = subprocess.run(link, capture_output=True, text=True)
    if done.returncode != 0:
        raise RuntimeError(f"link failed:\n{done.stderr}")
    if verbose:
        print(f"built {LIBRARY}", file=sys.stderr)
    return LIBRARY


if __name__ == "__main__":
    build_library(force="--force" in sys.argv, verbose=True)
