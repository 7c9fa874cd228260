"""Ahead-of-time build of ``libvelox_b200.so`` (sm_100a only) with plain nvcc.

The reference JIT-compiles one TVM-FFI module per kernel at first use
(``veloxvoice/kernels/utils.py:38-86``); this library is one shared object with a C ABI,
built once and loaded with ctypes.  ``python -m velox_voice_b200.build`` rebuilds it.
"""

from __future__ import annotations

import hashlib
import os
import shutil
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
LIB_DIR = os.path.join(HERE, "lib")
LIB_PATH = os.path.join(LIB_DIR, "libvelox_b200.so")
STAMP = os.path.join(LIB_DIR, "libvelox_b200.stamp")
SOURCES = ("vx_api.cu", "vx_quant.cu", "vx_gemm.cu", "vx_noalloc.cu", "vx_pack.cu")
NVCC_FLAGS = (
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-lineinfo", "-O3", "-std=c++17", "--threads", "4",
    "-Xcompiler", "-fPIC", "-shared", "-cudart", "static",
)


def _source_digest() -> str:
    h = hashlib.sha256()
    names = sorted(os.listdir(CSRC)) + [os.path.join("..", "..", "include", "velox_b200.h")]
    for n in names:
        path = os.path.join(CSRC, n)
        if os.path.isfile(path):
            h.update(n.encode())
            with open(path, "rb") as f:
                h.update(f.read())
    h.update(" ".join(NVCC_FLAGS).encode())
    return h.hexdigest()


def is_current() -> bool:
    if not (os.path.exists(LIB_PATH) and os.path.exists(STAMP)):
        return False
    with open(STAMP) as f:
        return f.read().strip() == _source_digest()


def build(force: bool = False, verbose: bool = False) -> str:
    """Compile the library if the sources changed; returns the path of the shared object."""
    if not force and is_current():
        return LIB_PATH
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(nvcc):
        raise RuntimeError("nvcc not found: cannot build libvelox_b200.so")
    os.makedirs(LIB_DIR, exist_ok=True)
    cmd = [nvcc, *NVCC_FLAGS, "-o", LIB_PATH] + [os.path.join(CSRC, s) for s in SOURCES]
    if verbose:
        cmd.insert(1, "-Xptxas=-v")
        print(" ".join(cmd), file=sys.stderr)
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode != 0:
        raise RuntimeError(f"nvcc failed ({res.returncode}):\n{res.stdout}\n{res.stderr}")
    if verbose:
        print(res.stderr, file=sys.stderr)
    with open(STAMP, "w") as f:
        f.write(_source_digest())
    return LIB_PATH


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv))
