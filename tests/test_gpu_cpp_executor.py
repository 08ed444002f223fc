"""Builds and runs the C++ host mirror's executor test (tests/cpp/executor_test.cpp) on a B200:
pinned threads, every thread calls run(), spin barrier per operator, chunked prompt then
decode steps, checked against the CPU oracle inside the binary."""
import os
import shutil
import subprocess

import pytest

import ellm_b200
import oracle

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_cpp_executor_spmd_generation(tmp_path):
    ellm_b200.load()
    oracle.load()
    cuda = os.environ.get("CUDA_HOME", "/usr/local/cuda")
    exe = str(tmp_path / "executor_test")
    cmd = [shutil.which("g++") or "g++", "-std=c++17", "-O2", "-pthread", os.path.join(ROOT, "tests", "cpp", "executor_test.cpp"),
           "-I", os.path.join(ROOT, "include"), "-I", os.path.join(ROOT, "oracle"), "-I", os.path.join(cuda, "include"),
           "-L", os.path.join(ROOT, "ellm_b200"), "-lellm_attn", "-L", os.path.join(ROOT, "oracle", "_build"), "-lellm_oracle",
           "-L", os.path.join(cuda, "lib64"), "-lcudart",
           "-Wl,-rpath," + os.path.join(ROOT, "ellm_b200"), "-Wl,-rpath," + os.path.join(ROOT, "oracle", "_build"),
           "-Wl,-rpath," + os.path.join(cuda, "lib64"), "-o", exe]
    subprocess.run(cmd, check=True, capture_output=True, text=True)
    for threads in ("1", "7"):
        res = subprocess.run([exe, threads], capture_output=True, text=True, timeout=300)
        assert res.returncode == 0, res.stdout + res.stderr
        assert "cache mismatches 0" in res.stdout
