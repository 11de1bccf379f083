"""Compiles tests/native/tc_plan_test.cpp against csrc/tc_plan.hpp with the host compiler and
runs it: the work planning the tensor-core kernels execute on the device, checked on the CPU."""
import os
import shutil
import subprocess

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.mark.skipif(shutil.which("g++") is None, reason="no host C++ compiler")
def test_every_slab_once_and_slots_distinct(tmp_path):
    exe = str(tmp_path / "tc_plan_test")
    subprocess.run(["g++", "-std=c++17", "-O1", "-Wall", "-I", os.path.join(ROOT, "polarai-framework_b200", "csrc"),
                    "-o", exe, os.path.join(ROOT, "tests", "native", "tc_plan_test.cpp")], check=True)
    out = subprocess.run([exe], capture_output=True, text=True, timeout=300)
    assert out.returncode == 0, out.stdout + out.stderr
    assert " 0 failures" in out.stdout
