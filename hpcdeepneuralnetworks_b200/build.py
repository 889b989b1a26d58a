"""In-tree build of libb2blas.so (sm_100a only) with nvcc.

``python -m hpcdeepneuralnetworks_b200.build`` compiles every ``csrc/*.cu`` into objects under
``csrc/build/`` (skipping files whose object is newer than all sources/headers) and links
``hpcdeepneuralnetworks_b200/libb2blas.so``.  nvcc cross-compiles without a GPU.
"""
from __future__ import annotations

import glob
import os
import shutil
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor

PKG = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(PKG, "csrc")
OBJ = os.path.join(CSRC, "build")
LIB = os.path.join(PKG, "libb2blas.so")

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC", "--expt-relaxed-constexpr", "-cudart", "shared",
]


def nvcc() -> str:
    exe = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(exe):
        raise RuntimeError("nvcc not found: the CUDA kernels cannot be built")
    return exe


def _stale(target: str, deps: list[str]) -> bool:
    if not os.path.exists(target):
        return True
    t = os.path.getmtime(target)
    return any(os.path.getmtime(d) > t for d in deps)


def build(verbose: bool = False, force: bool = False, ptxas_info: bool = False) -> str:
    os.makedirs(OBJ, exist_ok=True)
    sources = sorted(glob.glob(os.path.join(CSRC, "*.cu")))
    headers = sorted(glob.glob(os.path.join(CSRC, "*.cuh"))) + sorted(glob.glob(os.path.join(CSRC, "*.inc"))) + [os.path.join(PKG, "..", "include", "b2blas.h")]
    jobs = []
    objs = []
    for src in sources:
        obj = os.path.join(OBJ, os.path.basename(src)[:-3] + ".o")
        objs.append(obj)
        if force or _stale(obj, [src] + headers):
            cmd = [nvcc()] + NVCC_FLAGS + (["-Xptxas", "-v"] if ptxas_info else []) + ["-c", src, "-o", obj]
            jobs.append(cmd)

    def run(cmd):
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError("nvcc failed:\n" + " ".join(cmd) + "\n" + r.stdout + r.stderr)
        return r.stdout + r.stderr

    if jobs:
        with ThreadPoolExecutor(max_workers=min(8, len(jobs))) as ex:
            for out in ex.map(run, jobs):
                if verbose or ptxas_info:
                    sys.stderr.write(out)
    if jobs or force or _stale(LIB, objs):
        cmd = [nvcc(), "-shared", "-cudart", "shared", "-o", LIB] + objs + \
              ["-Xlinker", "-rpath,/usr/local/cuda/lib64", "-ldl"]
        run(cmd)
    build_driver()
    return LIB


DRIVER_SRC = os.path.join(PKG, "drivers", "b2_driver.cpp")
DRIVER_BIN = os.path.join(PKG, "drivers", "b2_driver")


def build_driver() -> str:
    """The C++ command-line driver (reference-shaped main() over the C ABI), linked against libb2blas.so."""
    if _stale(DRIVER_BIN, [DRIVER_SRC, LIB, os.path.join(PKG, "..", "include", "b2blas.h")]):
        cmd = [nvcc(), "-O2", "-std=c++17", "-I" + os.path.join(PKG, "..", "include"), DRIVER_SRC, "-o", DRIVER_BIN,
               "-L" + PKG, "-lb2blas", "-cudart", "shared", "-Xlinker", "-rpath," + PKG, "-Xlinker", "-rpath,/usr/local/cuda/lib64"]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError("driver build failed:\n" + " ".join(cmd) + "\n" + r.stdout + r.stderr)
    return DRIVER_BIN


if __name__ == "__main__":
    path = build(verbose=True, force="--force" in sys.argv, ptxas_info="--ptxas" in sys.argv)
    print(path)
