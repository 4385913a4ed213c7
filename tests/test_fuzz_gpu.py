"""Seeded random configurations of the whole path against the float64 oracle: ragged batches of sequences with random
lengths around page and tile boundaries, random split counts, both formats, with and without the gate, both output
types; appends in random chunkings; a prefill chunk followed by decode steps on the same cache."""
import numpy as np
import pytest
import torch

import oracle as O
import yahkv
from gpu_util import assert_pools_equal, dev

pytestmark = pytest.mark.gpu
ABS_TOL = 2e-3


def _random_case(rng, fmt, n_seqs, max_len, max_chunk):
    cached = [int(rng.integers(0, max_len)) for _ in range(n_seqs)]
    chunks = [int(rng.integers(1, max_chunk)) for _ in range(n_seqs)]
    totals = [a + b for a, b in zip(cached, chunks)]
    pages = [(n + 1 + 63) // 64 for n in totals]                     # room for one decode token
    num_pages = sum(pages) + 2
    cache = yahkv.KvCache(n_layers=1, num_pages=num_pages, fmt=fmt, max_seqs=n_seqs, max_pages_per_seq=max(pages),
                          max_batch_tokens=2048)
    pool = O.PagedPool(fmt, num_pages)
    free = list(rng.permutation(num_pages))
    seqs, tables, kv = [], [], []
    for n, p in zip(totals, pages):
        s = cache.seq_create()
        t = np.array([free.pop() for _ in range(p)], np.int32)
        cache.seq_set_table(s, t)
        seqs.append(s), tables.append(t)
        kv.append((rng.standard_normal((n + 1, 4, 256)).astype(np.float16),
                   rng.standard_normal((n + 1, 4, 256)).astype(np.float16)))
    return cache, pool, seqs, tables, kv, cached, chunks, totals


@pytest.mark.parametrize("seed", range(6))
def test_random_prefill_then_decode(seed):
    rng = np.random.default_rng(1000 + seed)
    fmt = yahkv.FMT_Q8_0 if seed % 2 == 0 else yahkv.FMT_Q4_0
    n_seqs = int(rng.integers(1, 5))
    cache, pool, seqs, tables, kv, cached, chunks, totals = _random_case(rng, fmt, n_seqs, 700, 260)
    # cached part: appended in random pieces, interleaved across sequences in one call per round
    done = [0] * n_seqs
    while any(d < c for d, c in zip(done, cached)):
        ids, pos, ks, vs = [], [], [], []
        for i in range(n_seqs):
            step = min(cached[i] - done[i], int(rng.integers(1, 200)))
            if step <= 0:
                continue
            ids += [seqs[i]] * step
            pos += list(range(done[i], done[i] + step))
            ks.append(kv[i][0][done[i]:done[i] + step]), vs.append(kv[i][1][done[i]:done[i] + step])
            done[i] += step
        cache.append(0, np.array(ids, np.int32), np.array(pos, np.int64), dev(np.concatenate(ks)), dev(np.concatenate(vs)))
    # the chunk, then chunked-prefill attention over cache + chunk
    ids = np.concatenate([np.full(c, s, np.int32) for s, c in zip(seqs, chunks)])
    pos = np.concatenate([np.arange(a, a + c) for a, c in zip(cached, chunks)])
    cache.append(0, ids, pos, dev(np.concatenate([kv[i][0][cached[i]:totals[i]] for i in range(n_seqs)])),
                 dev(np.concatenate([kv[i][1][cached[i]:totals[i]] for i in range(n_seqs)])))
    for i in range(n_seqs):
        pool.append(tables[i], 0, kv[i][0][:totals[i]], kv[i][1][:totals[i]])
    cache.sync()
    assert_pools_equal(cache, 0, pool)
    use_gate, f32 = bool(rng.integers(0, 2)), bool(rng.integers(0, 2))
    rows = sum(chunks)
    q = rng.standard_normal((rows, 24, 256)).astype(np.float16)
    gate = rng.standard_normal((rows, 24, 256)).astype(np.float32) if use_gate else None
    out = torch.full((rows, 24, 256), float("nan"), device="cuda", dtype=torch.float32 if f32 else torch.float16)
    torch.cuda.synchronize()
    cache.attend_prefill(0, seqs, chunks, dev(q), out, gate=None if gate is None else dev(gate),
                         out_dtype=yahkv.OUT_F32 if f32 else yahkv.OUT_F16)
    cache.sync()
    got = out.float().cpu().numpy().astype(np.float64)
    r0 = 0
    for i in range(n_seqs):
        want = pool.attend_prefill_f64(tables[i], cached[i], q[r0:r0 + chunks[i]],
                                       gate=None if gate is None else gate[r0:r0 + chunks[i]])
        tol = ABS_TOL + (0 if f32 else np.abs(want).max() * 2.0 ** -11)
        assert np.abs(got[r0:r0 + chunks[i]] - want).max() <= tol, (seed, i, cached[i], chunks[i])
        r0 += chunks[i]
    # one decode step on top, random split count
    k1 = np.stack([kv[i][0][totals[i]] for i in range(n_seqs)])
    v1 = np.stack([kv[i][1][totals[i]] for i in range(n_seqs)])
    cache.append(0, np.array(seqs, np.int32), np.array(totals, np.int64), dev(k1), dev(v1))
    qd = rng.standard_normal((n_seqs, 24, 256)).astype(np.float16)
    outd = torch.full((n_seqs, 24, 256), float("nan"), device="cuda")
    torch.cuda.synchronize()
    cache.attend_decode(0, seqs, dev(qd), outd, out_dtype=yahkv.OUT_F32, n_splits=int(rng.integers(0, 5)))
    cache.sync()
    gotd = outd.cpu().numpy().astype(np.float64)
    for i in range(n_seqs):
        pool.append(tables[i], totals[i], kv[i][0][totals[i]:totals[i] + 1], kv[i][1][totals[i]:totals[i] + 1])
        want = pool.attend_decode_f64(tables[i], totals[i] + 1, qd[i])
        assert np.abs(gotd[i] - want).max() <= ABS_TOL, (seed, i, totals[i])
    cache.close()
