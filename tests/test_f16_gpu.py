"""Unquantized fp16 pages (YAHKV_FMT_F16), the reference's fp16 cache mode: appends byte for byte (the rows as they
came, through shuffled tables), decode attention against the float64 model to the reference checker's bar
(max|err| / max|ref| < 1e-4, engine/gpu/loom/tools/dattn_check.py:92-94), chunked prefill at 2e-3 / 1e-3 (fp16 operands
on the tensor cores), the fused RoPE append, and what the format refuses."""
import numpy as np
import pytest
import torch

import oracle as O
import yahkv
from gpu_util import assert_pools_equal, dev

pytestmark = pytest.mark.gpu


def run_decode(cache, layer, seqs, q, gate=None, n_splits=0):
    out = torch.full((len(seqs), 24, 256), float("nan"), device="cuda")
    torch.cuda.synchronize()
    cache.attend_decode(layer, seqs, dev(q), out, gate=None if gate is None else dev(gate), out_dtype=yahkv.OUT_F32,
                        n_splits=n_splits)
    cache.sync()
    return out.cpu().numpy().astype(np.float64)


def test_ragged_batch_appends_and_decode_steps():
    rng = np.random.default_rng(17)
    lens = [1, 63, 64, 65, 100, 1000, 24 * 64 + 5, 2049]
    pages = [(n + 8 + 63) // 64 for n in lens]
    num_pages = sum(pages) + 3
    cache = yahkv.KvCache(n_layers=2, num_pages=num_pages, fmt=yahkv.FMT_F16, max_seqs=len(lens),
                          max_pages_per_seq=max(pages), max_batch_tokens=4096)
    pool = O.PagedPool(O.FMT_F16, num_pages)
    perm = rng.permutation(num_pages).astype(np.int32)
    seqs, tables, off = [], [], 0
    for i, n in enumerate(lens):
        s = cache.seq_create()
        table = perm[off:off + pages[i]].copy()
        off += pages[i]
        cache.seq_set_table(s, table)
        K = rng.standard_normal((n, 4, 256)).astype(np.float16)
        V = rng.standard_normal((n, 4, 256)).astype(np.float16)
        V[:, :, ::31] *= 15.0                      # outlier channels
        K[0, 0, :4] = [0.0, -0.0, 6.1e-5, 65504.0] if n > 1 else K[0, 0, :4]   # zeros, a subnormal neighbour, the largest
        for c0 in range(0, n, 4096):
            c1 = min(n, c0 + 4096)
            cache.append(1, np.full(c1 - c0, s, np.int32), np.arange(c0, c1, dtype=np.int64), dev(K[c0:c1]), dev(V[c0:c1]))
        pool.append(table, 0, K, V)
        seqs.append(s), tables.append(table)
    cache.sync()
    assert_pools_equal(cache, 1, pool)
    assert_pools_equal(cache, 0, O.PagedPool(O.FMT_F16, num_pages))     # the other layer is untouched
    cur = list(lens)
    for step in range(3):
        k = rng.standard_normal((len(lens), 4, 256)).astype(np.float16)
        v = rng.standard_normal((len(lens), 4, 256)).astype(np.float16)
        q = (0.5 * rng.standard_normal((len(lens), 24, 256))).astype(np.float16)
        gate = rng.standard_normal((len(lens), 24, 256)).astype(np.float32)
        cache.append(1, seqs, cur, dev(k), dev(v))
        for i in range(len(lens)):
            pool.append(tables[i], cur[i], k[i:i + 1], v[i:i + 1])
        cur = [n + 1 for n in cur]
        want = np.stack([pool.attend_decode_f64(tables[i], cur[i], q[i], gate[i]) for i in range(len(lens))])
        for n_splits in (0, 1, 5, 64):
            got = run_decode(cache, 1, seqs, q, gate, n_splits)
            err = np.abs(got - want).reshape(len(lens), -1).max(1)
            assert err.max() <= 2e-3 and err.max() / np.abs(want).max() < 1e-4, (step, n_splits, err)
    assert_pools_equal(cache, 1, pool)
    with pytest.raises(yahkv.YahkvError):
        cache.export_token(1, seqs[0], 0)
    cache.close()


def test_chunked_prefill_and_rope_append():
    rng = np.random.default_rng(19)
    chunks = [300, 212, 128, 1, 391]
    total = sum(chunks)
    pages = (total + 63) // 64
    num_pages, eps = pages + 4, 1e-6
    cache = yahkv.KvCache(n_layers=1, num_pages=num_pages, fmt=yahkv.FMT_F16, max_seqs=2, max_pages_per_seq=pages,
                          max_batch_tokens=512, max_prefill_keys=pages * 64)
    pool = O.PagedPool(O.FMT_F16, num_pages)
    table = rng.permutation(num_pages)[:pages].astype(np.int32)
    seq = cache.seq_create()
    cache.seq_set_table(seq, table)
    qw = (1.0 + 0.2 * rng.standard_normal(256)).astype(np.float32)
    kw = (1.0 + 0.2 * rng.standard_normal(256)).astype(np.float32)
    start = 0
    for c in chunks:                               # every chunk enters through the fused norm + RoPE + append
        q32 = rng.standard_normal((c, 24, 256)).astype(np.float32)
        k32 = rng.standard_normal((c, 4, 256)).astype(np.float32)
        v32 = rng.standard_normal((c, 4, 256)).astype(np.float32)
        gate = rng.standard_normal((c, 24, 256)).astype(np.float32)
        pos = np.arange(start, start + c, dtype=np.int64)
        q16 = torch.zeros((c, 24, 256), dtype=torch.float16, device="cuda")
        cache.rope_append(0, np.full(c, seq, np.int32), pos, dev(q32), dev(k32), dev(v32), dev(qw), dev(kw), eps, q16)
        out = torch.full((c, 24, 256), float("nan"), device="cuda")
        cache.attend_prefill(0, [seq], [c], q16, out, gate=dev(gate), out_dtype=yahkv.OUT_F32)
        cache.sync()
        want_q = O.rope_rows(q32, qw, eps, np.repeat(pos, 24)).reshape(c, 24, 256)
        assert np.array_equal(q16.cpu().numpy().view(np.uint16), want_q.view(np.uint16))
        pool.append(table, start, O.rope_rows(k32, kw, eps, np.repeat(pos, 4)).reshape(c, 4, 256), v32.astype(np.float16))
        got = out.cpu().numpy().astype(np.float64)
        for r in sorted({0, c - 1, c // 2, min(c - 1, 127), min(c - 1, 128)}):
            want = pool.attend_prefill_f64(table, start, want_q, r, r + 1, gate)[0]
            err = np.abs(got[r] - want).max()
            assert err <= 2e-3 and err <= 1e-3 * np.abs(want).max(), (start, c, r, err)
        start += c
    assert_pools_equal(cache, 0, pool)
    cache.close()
