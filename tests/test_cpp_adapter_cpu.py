"""Builds and runs the C++ adapter test (engine/model/kv_cache.hpp over the C ABI) against a host-only context."""
import os
import subprocess

import yahkv

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
PKG = os.path.join(ROOT, "yet-another-halo-engine_b200")


def test_cpp_adapter_on_a_host_only_context(tmp_path):
    exe = tmp_path / "kv_cache_test"
    cmd = ["g++", "-std=c++20", "-O1", "-Wall", "-Wextra", "-I", os.path.join(ROOT, "include"), "-I", PKG,
           os.path.join(ROOT, "tests", "cpp", "kv_cache_test.cc"), yahkv.LIB_PATH, "-Wl,-rpath," + PKG, "-o", str(exe)]
    r = subprocess.run(cmd, capture_output=True, text=True)
    assert r.returncode == 0, r.stderr[-3000:]
    r = subprocess.run([str(exe)], capture_output=True, text=True, timeout=120)
    assert r.returncode == 0 and "kv_cache_test: ok" in r.stdout, r.stdout + r.stderr
