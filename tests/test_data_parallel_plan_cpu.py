"""Compiles tests/native/data_parallel_plan_test.cpp against csrc/executor/data_parallel_plan.hpp
with the host compiler and runs it: which tensors of a recorded builtin program are split by
rows over the devices, which are replicated, and where a sum over devices is due."""
import os
import shutil
import subprocess

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.mark.skipif(shutil.which("g++") is None, reason="no host C++ compiler")
def test_batch_sharding_plan_rules(tmp_path):
    exe = str(tmp_path / "data_parallel_plan_test")
    subprocess.run(["g++", "-std=c++17", "-O1", "-Wall", "-I", os.path.join(ROOT, "polarai-framework_b200", "csrc"),
                    "-o", exe, os.path.join(ROOT, "tests", "native", "data_parallel_plan_test.cpp")], check=True)
    out = subprocess.run([exe], capture_output=True, text=True, timeout=60)
    assert out.returncode == 0, out.stdout + out.stderr
    assert "data_parallel_plan: 0 failures" in out.stdout
