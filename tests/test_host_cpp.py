"""The C++ host mirror (glm-ssd_b200/host/glmssd_host.hpp) through its test driver tests/host_check.cpp."""
import os
import subprocess

import pytest

from conftest import ROOT

BIN = os.path.join(ROOT, "tests", "host_check")


def _build():
    from build_host_check import build_host_check
    return build_host_check()


def test_host_mirror_compiles_and_checks_arguments():
    exe = _build()
    out = subprocess.run([exe, "--no-gpu"], capture_output=True, text=True, timeout=120)
    assert out.returncode == 0, out.stdout + out.stderr
    assert "no-gpu checks: ok" in out.stdout


@pytest.mark.gpu
def test_host_mirror_decode_session_matches_oracle():
    exe = BIN if os.path.exists(BIN) else _build()
    out = subprocess.run([exe], capture_output=True, text=True, timeout=300)
    assert out.returncode == 0, out.stdout + out.stderr
    assert "host session" in out.stdout and "FAILED" not in out.stdout
