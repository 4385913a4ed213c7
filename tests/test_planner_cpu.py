"""Builds and runs the host-only planner test (split-K units of decode attention, tile pairs of prefill attention)."""
import os
import shutil
import subprocess

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
PKG = os.path.join(ROOT, "yet-another-halo-engine_b200")


def _cuda_include():
    for d in (os.environ.get("CUDA_HOME"), "/usr/local/cuda"):
        if d and os.path.isfile(os.path.join(d, "include", "cuda_runtime.h")):
            return os.path.join(d, "include")
    nvcc = shutil.which("nvcc")
    if nvcc:
        d = os.path.join(os.path.dirname(os.path.dirname(os.path.realpath(nvcc))), "include")
        if os.path.isfile(os.path.join(d, "cuda_runtime.h")):
            return d
    return None


def test_planners_on_the_host(tmp_path):
    inc = _cuda_include()
    if inc is None:
        pytest.skip("the planner header includes the CUDA runtime's type definitions; no CUDA include directory found")
    exe = tmp_path / "planner_test"
    cmd = ["g++", "-std=c++20", "-O1", "-Wall", "-Wextra", "-I", os.path.join(ROOT, "include"), "-I", PKG, "-I", inc,
           os.path.join(ROOT, "tests", "cpp", "planner_test.cc"), "-o", str(exe)]
    r = subprocess.run(cmd, capture_output=True, text=True)
    assert r.returncode == 0, r.stderr[-3000:]
    r = subprocess.run([str(exe)], capture_output=True, text=True, timeout=120)
    assert r.returncode == 0 and "planner_test: ok" in r.stdout, r.stdout + r.stderr
