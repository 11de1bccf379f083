"""Compiles tests/native/device_scope_test.cpp against csrc/rt/device_scope.hpp with the host
compiler and runs it: the runtime plugin's current-device bookkeeping, cross-device copy
ordering and pending-upload tracking, exercised with a recording stand-in for the CUDA calls."""
import os
import shutil
import subprocess

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.mark.skipif(shutil.which("g++") is None, reason="no host C++ compiler")
def test_device_scope_restores_the_callers_device_and_orders_copies(tmp_path):
    exe = str(tmp_path / "device_scope_test")
    subprocess.run(["g++", "-std=c++17", "-O1", "-Wall", "-I", os.path.join(ROOT, "polarai-framework_b200", "csrc"),
                    "-o", exe, os.path.join(ROOT, "tests", "native", "device_scope_test.cpp")], check=True)
    out = subprocess.run([exe], capture_output=True, text=True, timeout=60)
    assert out.returncode == 0, out.stdout + out.stderr
    assert "device_scope: 0 failures" in out.stdout
