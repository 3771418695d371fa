"""Builds libb200q.so (the C-ABI CUDA library) in-tree with nvcc for sm_100a.

Run as ``python -m full_inference_engine_b200.build`` or call :func:`build_library`.
The shared object lands in ``full_inference_engine_b200/lib/``; it is rebuilt only
when a source or header is newer than it.
"""

from __future__ import annotations

import concurrent.futures
import os
import shutil
import subprocess
import sys

PACKAGE_DIR = os.path.dirname(os.path.abspath(__file__))
REPO_ROOT = os.path.dirname(PACKAGE_DIR)
CSRC = os.path.join(PACKAGE_DIR, "csrc")
INCLUDE = os.path.join(REPO_ROOT, "include")
LIB_DIR = os.path.join(PACKAGE_DIR, "lib")
LIB_PATH = os.path.join(LIB_DIR, "libb200q.so")
SOURCES = ("api.cu", "quantize.cu", "gemv_simt.cu", "gemm_tc.cu", "gemm_sk.cu", "gemm_i8.cu", "static_scratch.cu")

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-O3", "-std=c++17", "-lineinfo",
    "-Xcompiler", "-fPIC",
    "-Xptxas", "-v",
    "-I", INCLUDE, "-I", CSRC,
]


def _nvcc() -> str:
    found = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(found):
        raise RuntimeError("nvcc not found: libb200q.so cannot be built on this machine")
    return found


def _stale() -> bool:
    if not os.path.exists(LIB_PATH):
        return True
    built = os.path.getmtime(LIB_PATH)
    deps = [os.path.join(CSRC, name) for name in os.listdir(CSRC)]
    deps += [os.path.join(INCLUDE, name) for name in os.listdir(INCLUDE)]
    return any(os.path.getmtime(path) > built for path in deps)


def _compile(source: str, obj_dir: str, verbose: bool) -> str:
    out = os.path.join(obj_dir, source.replace(".cu", ".o"))
    cmd = [_nvcc(), *NVCC_FLAGS, "-c", os.path.join(CSRC, source), "-o", out]
    done = subprocess.run(cmd, capture_output=True, text=True)
    if verbose or done.returncode:
        sys.stderr.write(done.stdout + done.stderr)
    if done.returncode:
        raise RuntimeError(f"nvcc failed on {source}")
    with open(out + ".ptxas.log", "w") as log:
        log.write(done.stderr)
    return out


def build_library(force: bool = False, verbose: bool = False) -> str:
    """Compile and link the library if needed; returns its path."""
    if not force and not _stale():
        return LIB_PATH
    obj_dir = os.path.join(REPO_ROOT, "build", "b200q")
    os.makedirs(obj_dir, exist_ok=True)
    os.makedirs(LIB_DIR, exist_ok=True)
    with concurrent.futures.ThreadPoolExecutor(max_workers=len(SOURCES)) as pool:
        objects = list(pool.map(lambda s: _compile(s, obj_dir, verbose), SOURCES))
    link = [_nvcc(), "-shared", "-o", LIB_PATH, *objects,
            "-gencode", "arch=compute_100a,code=sm_100a", "-cudart", "static"]
    done = subprocess.run(link, capture_output=True, text=True)
    if done.returncode:
        sys.stderr.write(done.stdout + done.stderr)
        raise RuntimeError("linking libb200q.so failed")
    return LIB_PATH


if __name__ == "__main__":
    print(build_library(force="--force" in sys.argv, verbose="-v" in sys.argv))
