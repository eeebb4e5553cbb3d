"""Build recipe for the test oracle (never for the product).

* ``liboracle.so``             - the C restatement in ``oracle.c`` (gcc).
* ``_ref/libglmssd_ref.so``    - the reference engine's own CUDA kernels, compiled unmodified from
  where they lie in the mounted reference tree (``crates/cuda/kernels/*.cu``) with the flags of
  ``crates/cuda/build.rs:39-46`` and ``-arch=sm_100a``.  Built only when that tree is present; the
  output is git-ignored and travels to the GPU machine as a prebuilt file.  No reference source
  is copied into this repository.
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
ORACLE_SO = os.path.join(HERE, "liboracle.so")
REF_DIR = os.path.join(HERE, "_ref")
REF_SO = os.path.join(REF_DIR, "libglmssd_ref.so")
# where the reference project is mounted (its crates/cuda/kernels directory); absent on a machine without it
REF_KERNELS = os.environ.get("GLMSSD_REFERENCE_KERNELS",
                             os.path.join(os.sep, "root", "reference", "crates", "cuda", "kernels"))


def _newer(target: str, sources: list[str]) -> bool:
    if not os.path.exists(target):
        return False
    t = os.path.getmtime(target)
    return all(os.path.getmtime(s) <= t for s in sources)


def build_oracle(force: bool = False) -> str:
    srcs = [os.path.join(HERE, "oracle.c"), os.path.join(HERE, "oracle.h")]
    if not force and _newer(ORACLE_SO, srcs):
        return ORACLE_SO
    gcc = shutil.which("gcc")
    if gcc is None:
        if os.path.exists(ORACLE_SO):
            return ORACLE_SO
        raise RuntimeError("gcc not found and no prebuilt liboracle.so")
    # -mavx2/-mfma/-mf16c rather than -march=native: the library is built on one machine and run on another.
    cmd = [gcc, "-O3", "-mavx2", "-mfma", "-mf16c", "-fPIC", "-shared", "-std=c11", "-Wall", "-o", ORACLE_SO,
           srcs[0], "-lm", "-lpthread"]
    subprocess.check_call(cmd)
    return ORACLE_SO


def build_reference(force: bool = False) -> str | None:
    """Compile the reference's CUDA kernels into oracle/_ref/. Returns None if the tree is absent."""
    names = ["ops.cu", "gemm.cu", "quants.cu", "runtime.cu"]
    srcs = [os.path.join(REF_KERNELS, n) for n in names]
    if not all(os.path.exists(s) for s in srcs):
        return REF_SO if os.path.exists(REF_SO) else None
    if not force and _newer(REF_SO, srcs):
        return REF_SO
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(nvcc):
        return REF_SO if os.path.exists(REF_SO) else None
    os.makedirs(REF_DIR, exist_ok=True)
    cmd = [nvcc, "-O3", "--use_fast_math", "-std=c++20", "-lineinfo", "-arch=sm_100a", "-I", REF_KERNELS,
           "-Xcompiler", "-fPIC", "-shared", "-o", REF_SO] + srcs
    subprocess.check_call(cmd)
    return REF_SO


if __name__ == "__main__":
    print(build_oracle(force="--force" in sys.argv))
    print(build_reference(force="--force" in sys.argv))
