"""Helpers of the GPU parity tests: run the same appends through the library and the CPU oracle and compare."""
import numpy as np
import torch

import oracle as O
import yahkv


def dev(a):
    """numpy array -> CUDA tensor with the same bytes (float16 arrays stay float16)."""
    t = torch.from_numpy(np.ascontiguousarray(a)).cuda()
    torch.cuda.synchronize()   # the library runs on its own stream, not on torch's
    return t


def pool_pages(cache, layer, num_pages):
    """Whole pools of one layer read back through the C ABI, in the oracle's array shapes."""
    out = []
    for side in (yahkv.SIDE_K, yahkv.SIDE_V):
        pages = [cache.read_page(layer, side, p) for p in range(num_pages)]
        out.append(np.stack([c for c, _ in pages]))
        out.append(np.stack([s for _, s in pages]))
    kc, ks, vc, vs = out
    return kc, ks, vc, vs


def assert_pools_equal(cache, layer, pool):
    kc, ks, vc, vs = pool_pages(cache, layer, pool.num_pages)
    assert np.array_equal(kc, pool.kcodes), f"K codes differ in {(kc != pool.kcodes).sum()} bytes"
    assert np.array_equal(ks, pool.kscales), f"K scales differ in {(ks != pool.kscales).sum()} values"
    assert np.array_equal(vc, pool.vcodes), f"V codes differ in {(vc != pool.vcodes).sum()} bytes"
    assert np.array_equal(vs, pool.vscales), f"V scales differ in {(vs != pool.vscales).sum()} values"


def fill_both(cache, pool, layer, seq, table, K, V, chunk=4096):
    """Append K, V [n][4][256] fp16 at positions 0..n-1 of `seq` on the GPU (in chunks) and in the oracle pool."""
    n = K.shape[0]
    cache.seq_set_table(seq, table)
    for s in range(0, n, chunk):
        e = min(n, s + chunk)
        cache.append(layer, np.full(e - s, seq, np.int32), np.arange(s, e, dtype=np.int64), dev(K[s:e]), dev(V[s:e]))
    cache.sync()
    if pool is not None:
        pool.append(table, 0, K, V)
