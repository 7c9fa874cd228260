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
SOURCES = ("vx_api.cu", "vx_quant.cu", "vx_gemm.cu", "vx_noalloc.cu", "vx_pack.cu", "vx_mel.cu", "vx_attn.cu", "vx_gemm_ln.cu")
NVCC_FLAGS = (
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC",
)
LINK_FLAGS = ("-gencode", "arch=compute_100a,code=sm_100a", "-shared", "-cudart", "static")
OBJ_DIR = os.path.join(LIB_DIR, "obj")


def _headers_digest() -> str:
    h = hashlib.sha256()
    names = sorted(n for n in os.listdir(CSRC) if n.endswith((".cuh", ".h")))
    paths = [os.path.join(CSRC, n) for n in names] + [os.path.join(HERE, "..", "include", "velox_b200.h")]
    for path in paths:
        if os.path.isfile(path):
            h.update(os.path.basename(path).encode())
            with open(path, "rb") as f:
                h.update(f.read())
    h.update(" ".join(NVCC_FLAGS).encode())
    return h.hexdigest()


def _file_digest(name: str, extra: str) -> str:
    h = hashlib.sha256(extra.encode())
    with open(os.path.join(CSRC, name), "rb") as f:
        h.update(f.read())
    return h.hexdigest()


def _source_digest() -> str:
    hd = _headers_digest()
    h = hashlib.sha256(" ".join(LINK_FLAGS).encode())
    for n in SOURCES:
        h.update(_file_digest(n, hd).encode())
    return h.hexdigest()


def is_current() -> bool:
    if not (os.path.exists(LIB_PATH) and os.path.exists(STAMP)):
        return False
    with open(STAMP) as f:
        return f.read().strip() == _source_digest()


def compile_objects(defines=(), obj_dir: str = OBJ_DIR, sources=SOURCES, force: bool = False, verbose: bool = False):
    """Compile each source to an object (only those whose text, headers or flags changed), in
    parallel; returns the object paths.  ``defines``: extra ``-DNAME=VALUE`` strings."""
    from concurrent.futures import ThreadPoolExecutor

    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(nvcc):
        raise RuntimeError("nvcc not found: cannot build libvelox_b200.so")
    os.makedirs(obj_dir, exist_ok=True)
    hd = _headers_digest() + " ".join(defines)

    def one(name):
        obj = os.path.join(obj_dir, name[:-3] + ".o")
        stamp = obj + ".stamp"
        dig = _file_digest(name, hd)
        if not force and os.path.exists(obj) and os.path.exists(stamp) and open(stamp).read().strip() == dig:
            return obj
        cmd = [nvcc, *NVCC_FLAGS, *defines, "-c", os.path.join(CSRC, name), "-o", obj]
        if verbose:
            cmd.insert(1, "-Xptxas=-v")
            print(" ".join(cmd), file=sys.stderr)
        res = subprocess.run(cmd, capture_output=True, text=True)
        if res.returncode != 0:
            raise RuntimeError(f"nvcc failed on {name} ({res.returncode}):\n{res.stdout}\n{res.stderr}")
        if verbose:
            print(res.stderr, file=sys.stderr)
        with open(stamp, "w") as f:
            f.write(dig)
        return obj

    with ThreadPoolExecutor(max_workers=min(len(sources), os.cpu_count() or 1)) as ex:
        return list(ex.map(one, sources))


def link(objects, out_path: str) -> str:
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    os.makedirs(os.path.dirname(out_path), exist_ok=True)
    res = subprocess.run([nvcc, *LINK_FLAGS, "-o", out_path, *objects], capture_output=True, text=True)
    if res.returncode != 0:
        raise RuntimeError(f"link failed ({res.returncode}):\n{res.stdout}\n{res.stderr}")
    return out_path


def build(force: bool = False, verbose: bool = False) -> str:
    """Compile the library if the sources changed; returns the path of the shared object."""
    if not force and is_current():
        return LIB_PATH
    objects = compile_objects(force=force, verbose=verbose)
    link(objects, LIB_PATH)
    with open(STAMP, "w") as f:
        f.write(_source_digest())
    return LIB_PATH


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv))
