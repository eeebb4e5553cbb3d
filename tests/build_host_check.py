"""Builds tests/host_check from tests/host_check.cpp: the test driver of the C++ host mirror
(glm-ssd_b200/host/glmssd_host.hpp), linked against the attention library and, as its checker, the CPU oracle.
Test infrastructure: it lives here, beside the test that runs it, so that nothing in the product package
names the oracle."""
from __future__ import annotations

import importlib
import os
import shutil
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def build_host_check(force: bool = False) -> str:
    pkg_build = importlib.import_module("glm-ssd_b200.build")
    from oracle import build as obuild
    pkg_dir = pkg_build.HERE
    exe = os.path.join(ROOT, "tests", "host_check")
    src = os.path.join(ROOT, "tests", "host_check.cpp")
    deps = [src, os.path.join(pkg_dir, "host", "glmssd_host.hpp"), os.path.join(ROOT, "include", "glmssd_attn.h")]
    if not force and os.path.exists(exe) and all(os.path.getmtime(d) <= os.path.getmtime(exe) for d in deps):
        return exe
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(nvcc):
        if os.path.exists(exe):
            return exe
        raise RuntimeError("nvcc not found; cannot build tests/host_check")
    pkg_build.build()
    obuild.build_oracle()
    cmd = [nvcc, "-O2", "-std=c++17", "-x", "cu", "-o", exe, src, "-L" + pkg_dir, "-lglmssd_attn",
           "-L" + os.path.join(ROOT, "oracle"), "-loracle",
           "-Xlinker", "-rpath," + pkg_dir, "-Xlinker", "-rpath," + os.path.join(ROOT, "oracle")]
    subprocess.check_call(cmd)
    return exe


if __name__ == "__main__":
    print(build_host_check(force="--force" in sys.argv))
