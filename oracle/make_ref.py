"""Fill ``oracle/_ref/`` with the reference project's own Python package and kernel tests.

TEST INFRASTRUCTURE.  ``oracle/_ref/`` is git-ignored: nothing of the reference is committed to
this repository.  The copy exists so that, on a machine that has no checkout of the reference,

* the GPU tests can run the reference's REAL quantizers (its Triton kernels,
  ``veloxvoice/kernels/ops/triton_ops.py``) next to this library's and compare bytes,
* the reference's own kernel test bodies (``tests/kernels/test_dgx_mxfp4_gemm.py``) and its own
  model classes (``veloxvoice/models/wenet/torch_conformer.py``) can be executed against the
  operators this library installs,
* the CPU arm of the benchmark can time the reference's own ``DenseLinear`` (fp32 ``F.linear``).

    python oracle/make_ref.py [path to a checkout of the reference]

The source tree is only read.  Re-running replaces the copy.  Only Python files are copied: the
reference's kernel sources stay where they are.
"""

from __future__ import annotations

import os
import shutil
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
DEST = os.path.join(HERE, "_ref")
DEFAULT_SRC = os.environ.get("VELOX_REFERENCE_DIR", "/root/reference")
WANTED = (
    ("veloxvoice", "veloxvoice"),
    (os.path.join("tests", "kernels", "test_dgx_mxfp4_gemm.py"), os.path.join("ref_tests", "test_dgx_mxfp4_gemm.py")),
    (os.path.join("tests", "kernels", "test_power_mel_log.py"), os.path.join("ref_tests", "test_power_mel_log.py")),
    (os.path.join("tests", "kernels", "test_cuda_ops.py"), os.path.join("ref_tests", "test_cuda_ops.py")),
)


def available() -> bool:
    return os.path.isdir(os.path.join(DEST, "veloxvoice"))


def make(src: str = DEFAULT_SRC, quiet: bool = False) -> bool:
    """Copy the wanted parts of ``src`` into ``oracle/_ref``; False when ``src`` does not exist."""
    if not os.path.isdir(os.path.join(src, "veloxvoice")):
        if not quiet:
            print(f"no reference checkout at {src}: oracle/_ref left as it is", file=sys.stderr)
        return False
    tmp = DEST + ".tmp"
    shutil.rmtree(tmp, ignore_errors=True)
    os.makedirs(tmp)
    for rel_src, rel_dst in WANTED:
        s, d = os.path.join(src, rel_src), os.path.join(tmp, rel_dst)
        if os.path.isdir(s):
            # Python only: the reference's CUDA / C++ kernel sources (veloxvoice/kernels/csrc) are never
            # compiled or run by anything here -- its operators are replaced before they would be built
            shutil.copytree(s, d, ignore=shutil.ignore_patterns("__pycache__", "*.pyc", "csrc", "*.cu", "*.cuh", "*.h", "*.cpp"))
        elif os.path.isfile(s):
            os.makedirs(os.path.dirname(d), exist_ok=True)
            shutil.copy2(s, d)
    shutil.rmtree(DEST, ignore_errors=True)
    os.replace(tmp, DEST)
    if not quiet:
        print(DEST)
    return True


def add_to_path() -> bool:
    """Make ``import veloxvoice`` resolve to the copy (no-op when it is absent)."""
    if not available():
        return False
    if DEST not in sys.path:
        sys.path.insert(0, DEST)
    return True


if __name__ == "__main__":
    ok = make(sys.argv[1] if len(sys.argv) > 1 else DEFAULT_SRC)
    sys.exit(0 if ok else 1)
