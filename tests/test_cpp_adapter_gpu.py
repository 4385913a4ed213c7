"""The C++ adapter (engine/model/kv_cache.hpp) on the GPU: a compiled program appends a prompt, runs chunked-prefill
attention, decode steps (eager and as a device-resident batch) and a snapshot round trip through the adapter with its
own device buffers, and this test compares what it wrote with the float64 oracle."""
import os
import subprocess

import numpy as np
import pytest

import oracle as O
import yahkv

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
PKG = os.path.join(ROOT, "yet-another-halo-engine_b200")
CUDA = os.environ.get("CUDA_HOME", "/usr/local/cuda")


@pytest.mark.parametrize("fmt", [yahkv.FMT_Q8_0, yahkv.FMT_Q4_0])
def test_cpp_adapter_prefill_and_decode_against_the_oracle(tmp_path, fmt):
    exe = tmp_path / "kv_cache_gpu_test"
    cmd = ["g++", "-std=c++20", "-O1", "-Wall", "-Wextra", "-I", os.path.join(ROOT, "include"), "-I", PKG,
           "-I", os.path.join(CUDA, "include"), os.path.join(ROOT, "tests", "cpp", "kv_cache_gpu_test.cc"),
           yahkv.LIB_PATH, "-L" + os.path.join(CUDA, "lib64"), "-lcudart", "-Wl,-rpath," + PKG,
           "-Wl,-rpath," + os.path.join(CUDA, "lib64"), "-o", str(exe)]
    r = subprocess.run(cmd, capture_output=True, text=True)
    assert r.returncode == 0, r.stderr[-3000:]
    n_prompt, n_decode = 200, 5
    n = n_prompt + n_decode
    rng = np.random.default_rng(23)
    K = rng.standard_normal((n, 4, 256)).astype(np.float16)
    V = rng.standard_normal((n, 4, 256)).astype(np.float16)
    q = rng.standard_normal((n, 24, 256)).astype(np.float16)
    table = rng.permutation(64)[:4].astype(np.int32)
    for name, a in (("k.f16", K), ("v.f16", V), ("q.f16", q), ("table.i32", table)):
        a.tofile(tmp_path / name)
    r = subprocess.run([str(exe), str(tmp_path), str(n_prompt), str(n_decode), str(fmt)], capture_output=True, text=True,
                       timeout=300)
    assert r.returncode == 0 and "kv_cache_gpu_test: ok" in r.stdout, r.stdout + r.stderr
    pool = O.PagedPool(fmt, 64)
    pool.append(table, 0, K, V)
    pre = np.fromfile(tmp_path / "prefill.f32", np.float32).reshape(n_prompt, 24, 256)
    dec = np.fromfile(tmp_path / "decode.f32", np.float32).reshape(n_decode, 24, 256)
    want = pool.attend_prefill_f64(table, 0, q[:n_prompt])
    assert np.abs(pre - want).max() <= 2e-3
    for s in range(n_decode):
        p = n_prompt + s
        assert np.abs(dec[s] - pool.attend_decode_f64(table, p + 1, q[p])).max() <= 2e-3, s
    loaded = np.fromfile(tmp_path / "loaded.f32", np.float32).reshape(24, 256)
    assert np.abs(loaded - pool.attend_decode_f64(table, n, q[n - 1])).max() <= 2e-3
    assert np.abs(loaded - dec[-1]).max() <= 1e-5   # the same bytes on other pages (the split may differ)
