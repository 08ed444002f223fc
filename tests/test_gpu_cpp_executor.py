"""Builds and runs the C++ host mirror's executor tests (tests/cpp/) on a B200: pinned threads,
every thread calls run(), spin barrier per operator, chunked prompt then decode steps, checked
against the CPU oracle inside the binaries - the attention operator alone, and a whole
attention-only layer (projection operators either side of it)."""
import os
import shutil
import subprocess

import pytest

import ellm_b200
import oracle

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _build(tmp_path, name, with_oracle=True):
    ellm_b200.load()
    oracle.load()
    cuda = os.environ.get("CUDA_HOME", "/usr/local/cuda")
    exe = str(tmp_path / name)
    cmd = [shutil.which("g++") or "g++", "-std=c++17", "-O2", "-pthread", os.path.join(ROOT, "tests", "cpp", name + ".cpp"),
           "-I", os.path.join(ROOT, "include"), "-I", os.path.join(ROOT, "oracle"), "-I", os.path.join(cuda, "include"),
           "-L", os.path.join(ROOT, "ellm_b200"), "-lellm_attn", "-L", os.path.join(ROOT, "oracle", "_build"), "-lellm_oracle",
           "-L", os.path.join(cuda, "lib64"), "-lcudart",
           "-Wl,-rpath," + os.path.join(ROOT, "ellm_b200"), "-Wl,-rpath," + os.path.join(ROOT, "oracle", "_build"),
           "-Wl,-rpath," + os.path.join(cuda, "lib64"), "-o", exe]
    subprocess.run(cmd, check=True, capture_output=True, text=True)
    return exe


def test_cpp_layer_through_operator_queue(tmp_path):
    exe = _build(tmp_path, "layer_test")
    for threads in ("1", "5"):
        res = subprocess.run([exe, threads], capture_output=True, text=True, timeout=300)
        assert res.returncode == 0, res.stdout + res.stderr
        assert "V rows off 0" in res.stdout


def test_cpp_async_executor_eight_layers_graph_decode(tmp_path):
    """8 layers x 32 decode steps through start_generation_async: one wait per step instead of a
    barrier per operator, decode steps operator by operator and as a replayed CUDA graph - same
    bits both ways, and within the stack's tolerance of the oracle."""
    exe = _build(tmp_path, "async_layers_test")
    for threads in ("1", "4"):
        res = subprocess.run([exe, threads, "8", "32"], capture_output=True, text=True, timeout=600)
        assert res.returncode == 0, res.stdout + res.stderr
        assert "same bits" in res.stdout


def test_cpp_stack_decode_bench_runs(tmp_path):
    """The C++ timing program of the stack's decode step (the benchmark runs it at 48 layers and a
    32768-token context) on a small geometry, both as a replayed graph and operator by operator."""
    import json
    exe = _build(tmp_path, "stack_decode_bench")
    for graph in ("1", "0"):
        res = subprocess.run([exe, "4", "2048", "12", graph], capture_output=True, text=True, timeout=300)
        assert res.returncode == 0, res.stdout + res.stderr
        line = json.loads(res.stdout.strip().splitlines()[-1])
        assert line["finite"] and line["timed_steps"] == 10 and 0 < line["tpot_ms"] < 50


def test_cpp_executor_spmd_generation(tmp_path):
    exe = _build(tmp_path, "executor_test")
    for threads in ("1", "7"):
        res = subprocess.run([exe, threads], capture_output=True, text=True, timeout=300)
        assert res.returncode == 0, res.stdout + res.stderr
        assert "cache mismatches 0" in res.stdout
