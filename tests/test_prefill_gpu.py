"""Chunked-prefill attention on the GPU (fp16 dequantize pass + tcgen05 kernel) against the float64 oracle.
Tolerance: 2e-3 max-abs with fp32 softmax accumulation, on fp16 Q/K/V ~ N(0,1) as the benchmark configuration has."""
import numpy as np
import pytest
import torch

import oracle as O
import yahkv
from gpu_util import dev

pytestmark = pytest.mark.gpu
ABS_TOL = 2e-3


def build(fmt, cached, chunks, seed, n_layers=1, layer=0):
    """Sequences with `cached[i]` tokens appended earlier and a chunk of `chunks[i]` tokens appended now."""
    rng = np.random.default_rng(seed)
    totals = [a + b for a, b in zip(cached, chunks)]
    num_pages = sum((n + 63) // 64 for n in totals) + 3
    cache = yahkv.KvCache(n_layers=n_layers, num_pages=num_pages, fmt=fmt, max_seqs=len(totals),
                          max_pages_per_seq=max((n + 63) // 64 for n in totals), max_batch_tokens=4096)
    pool = O.PagedPool(fmt, num_pages)
    free = list(rng.permutation(num_pages))
    seqs, tables = [], []
    for n, c0 in zip(totals, cached):
        s = cache.seq_create()
        table = np.array([free.pop() for _ in range((n + 63) // 64)], np.int32)
        cache.seq_set_table(s, table)
        K = rng.standard_normal((n, 4, 256)).astype(np.float16)
        V = rng.standard_normal((n, 4, 256)).astype(np.float16)
        if c0:
            cache.append(layer, np.full(c0, s, np.int32), np.arange(c0), dev(K[:c0]), dev(V[:c0]))
        cache.append(layer, np.full(n - c0, s, np.int32), np.arange(c0, n), dev(K[c0:]), dev(V[c0:]))   # the chunk
        pool.append(table, 0, K, V)
        seqs.append(s); tables.append(table)
    return cache, pool, seqs, tables, rng


def run_prefill(cache, layer, seqs, chunks, q, gate, out_dtype):
    rows = sum(chunks)
    out = torch.full((rows, 24, 256), float("nan"), device="cuda",
                     dtype=torch.float32 if out_dtype == yahkv.OUT_F32 else torch.float16)
    torch.cuda.synchronize()   # the fill runs on torch's stream, the library on its own
    cache.attend_prefill(layer, seqs, chunks, dev(q), out, gate=None if gate is None else dev(gate), out_dtype=out_dtype)
    cache.sync()
    return out.float().cpu().numpy().astype(np.float64)


@pytest.mark.parametrize("fmt", [yahkv.FMT_Q8_0, yahkv.FMT_Q4_0])
def test_one_sequence_cache_plus_chunk(fmt):
    cached, chunk = 200, 130
    cache, pool, seqs, tables, rng = build(fmt, [cached], [chunk], seed=41)
    q = rng.standard_normal((chunk, 24, 256)).astype(np.float16)
    gate = rng.standard_normal((chunk, 24, 256)).astype(np.float32)
    want = pool.attend_prefill_f64(tables[0], cached, q, gate=gate)
    got = run_prefill(cache, 0, seqs, [chunk], q, gate, yahkv.OUT_F32)
    err = np.abs(got - want).reshape(chunk, -1).max(1)
    assert err.max() <= ABS_TOL, (int(err.argmax()), err.max())
    got16 = run_prefill(cache, 0, seqs, [chunk], q, None, yahkv.OUT_F16)
    want_plain = pool.attend_prefill_f64(tables[0], cached, q)
    assert np.abs(got16 - want_plain).max() <= ABS_TOL + np.abs(want_plain).max() * 2.0 ** -11


def test_ragged_batch_of_chunks():
    cached = [0, 63, 500, 1000, 64]
    chunks = [100, 1, 129, 300, 128]
    cache, pool, seqs, tables, rng = build(yahkv.FMT_Q8_0, cached, chunks, seed=42, n_layers=2, layer=1)
    q = rng.standard_normal((sum(chunks), 24, 256)).astype(np.float16)
    got = run_prefill(cache, 1, seqs, chunks, q, None, yahkv.OUT_F32)
    row = 0
    for i, c in enumerate(chunks):
        want = pool.attend_prefill_f64(tables[i], cached[i], q[row:row + c])
        err = np.abs(got[row:row + c] - want).max()
        assert err <= ABS_TOL, (i, err)
        row += c


def test_prefill_rows_equal_decode_of_the_same_position():
    # the last row of a chunk is exactly a decode step over the whole sequence
    cached, chunk = 300, 70
    cache, pool, seqs, tables, rng = build(yahkv.FMT_Q8_0, [cached], [chunk], seed=43)
    q = rng.standard_normal((chunk, 24, 256)).astype(np.float16)
    got = run_prefill(cache, 0, seqs, [chunk], q, None, yahkv.OUT_F32)
    dec = torch.zeros(1, 24, 256, device="cuda")
    cache.attend_decode(0, seqs, dev(q[-1:]), dec, out_dtype=yahkv.OUT_F32)
    cache.sync()
    assert np.abs(got[-1] - dec.cpu().numpy()[0]).max() <= ABS_TOL


def test_full_size_chunk_properties():
    """At the benchmark configuration's size (30,720 cached + a 2,048-token chunk, 512 key tiles per query tile), where
    the float64 oracle would take minutes: size-independent properties.
    (1) the softmax weights sum to one: with every cached V row equal, every output row is that row dequantized;
    (2) a chunk row is the decode step of the same position (two different kernels, split-K vs tensor-core tiles)."""
    cached, chunk, n = 30720, 2048, 32768
    rng = np.random.default_rng(45)
    cache = yahkv.KvCache(n_layers=1, num_pages=n // 64 + 2, fmt=yahkv.FMT_Q8_0, max_seqs=1, max_pages_per_seq=n // 64,
                          max_batch_tokens=4096)
    s = cache.seq_create()
    cache.seq_set_table(s, rng.permutation(n // 64 + 2)[: n // 64].astype(np.int32))
    vrow = rng.standard_normal((1, 4, 256)).astype(np.float16)
    for p0 in range(0, n, 4096):
        K = torch.randn((4096, 4, 256), device="cuda", dtype=torch.float16)
        V = dev(np.broadcast_to(vrow, (4096, 4, 256)).copy())
        torch.cuda.synchronize()
        cache.append(0, np.full(4096, s, np.int32), np.arange(p0, p0 + 4096), K, V)
    cache.sync()
    q = rng.standard_normal((chunk, 24, 256)).astype(np.float16)
    got = run_prefill(cache, 0, [s], [chunk], q, None, yahkv.OUT_F32)
    _, vb = cache.export_token(0, s, 0)
    want = O.dequantize(vb, yahkv.FMT_Q8_0).reshape(4, 256).astype(np.float64)
    assert np.abs(got - np.repeat(want, 6, axis=0)[None]).max() <= ABS_TOL   # fp16(code x scale) rounds V by <= 2^-11
    # (2): random V in the last 70 positions breaks the symmetry, then compare rows with decode steps
    K2 = rng.standard_normal((70, 4, 256)).astype(np.float16)
    V2 = rng.standard_normal((70, 4, 256)).astype(np.float16)
    cache.seq_set_len(s, n - 70)
    cache.append(0, np.full(70, s, np.int32), np.arange(n - 70, n), dev(K2), dev(V2))
    got = run_prefill(cache, 0, [s], [chunk], q, None, yahkv.OUT_F32)
    for row in (chunk - 1, chunk - 40):
        cache.seq_set_len(s, n - (chunk - 1 - row))
        dec = torch.zeros(1, 24, 256, device="cuda")
        torch.cuda.synchronize()
        cache.attend_decode(0, [s], dev(q[row:row + 1]), dec, out_dtype=yahkv.OUT_F32)
        cache.sync()
        assert np.abs(got[row] - dec.cpu().numpy()[0]).max() <= ABS_TOL
    cache.close()


def test_tail_tiles_split_along_the_keys():
    """With 20 SMs (10 SM pairs) to fill, the 24 tile pairs of this call leave a last wave of 4: those are split into
    two key ranges each and joined by the merge kernel (three launches instead of two). Results against the oracle, gate and fp16 output
    included, and against the unsplit run."""
    cached, chunk = 500, 129
    runs = []
    for sms in (0, 20):
        cache, pool, seqs, tables, rng = build(yahkv.FMT_Q8_0, [cached], [chunk], seed=46)
        cache.debug_set_prefill_sms(sms)
        q = rng.standard_normal((chunk, 24, 256)).astype(np.float16)
        gate = rng.standard_normal((chunk, 24, 256)).astype(np.float32)
        before = cache.launch_count()
        got = run_prefill(cache, 0, seqs, [chunk], q, gate, yahkv.OUT_F32)
        launches = cache.launch_count() - before
        got16 = run_prefill(cache, 0, seqs, [chunk], q, None, yahkv.OUT_F16)
        want = pool.attend_prefill_f64(tables[0], cached, q, gate=gate)
        want_plain = pool.attend_prefill_f64(tables[0], cached, q)
        assert np.abs(got - want).max() <= ABS_TOL
        assert np.abs(got16 - want_plain).max() <= ABS_TOL + np.abs(want_plain).max() * 2.0 ** -11
        runs.append((got, launches))
        cache.close()
    assert runs[0][1] == 2 and runs[1][1] == 3
    assert np.abs(runs[0][0] - runs[1][0]).max() <= 5e-4


def test_prefill_errors_launch_nothing():
    cache, pool, seqs, tables, rng = build(yahkv.FMT_Q8_0, [10], [5], seed=44)
    q = torch.zeros(20, 24, 256, dtype=torch.float16, device="cuda")
    out = torch.zeros(20, 24, 256, dtype=torch.float16, device="cuda")
    before = cache.launch_count()
    for seq_ids, chunks, code in (([seqs[0]], [16], yahkv.ERR_ORDER), ([seqs[0]], [0], yahkv.ERR_INVALID),
                                  ([3], [1], yahkv.ERR_INVALID)):
        with pytest.raises(yahkv.YahkvError) as e:
            cache.attend_prefill(0, seq_ids, chunks, q, out)
        assert e.value.code == code
    assert cache.launch_count() == before


@pytest.mark.parametrize("fmt", [yahkv.FMT_Q8_0, yahkv.FMT_KV8A16])
def test_raw_query_prologue_is_rope_then_attend(fmt):
    """yahkv_attend_prefill_qraw (norm + RoPE of the raw f32 q rows inside the attention kernel's prologue, the
    reference's QNORM option, gen_attn_fa.py:56-61) against the two-step path: the oracle's normed, rotated fp16 q rows
    (the bits yahkv_rope_append's q_out holds) through the float64 attention model, and bit for bit against
    yahkv_rope_append's q_out followed by yahkv_attend_prefill. A ragged batch of chunks, a 127 / 128 tile edge, rows past
    the last tile's end, chunk positions up to 1299."""
    rng = np.random.default_rng(45)
    eps = 1e-6
    cached, chunks = [0, 1000, 70], [129, 300, 58]
    totals = [a + b for a, b in zip(cached, chunks)]
    num_pages = sum((n + 63) // 64 for n in totals) + 2
    cache = yahkv.KvCache(n_layers=1, num_pages=num_pages, fmt=fmt, max_seqs=3, max_pages_per_seq=24, max_batch_tokens=1024)
    qw = (1.0 + 0.2 * rng.standard_normal(256)).astype(np.float32)
    kw = (1.0 + 0.2 * rng.standard_normal(256)).astype(np.float32)
    pool = O.PagedPool(yahkv.FMT_Q8_0, num_pages)   # followed for q8_0 only (the tile formats have their own tests)
    seqs = []
    for n, c0 in zip(totals, cached):
        s = cache.seq_create()
        cache.seq_reserve(s, n)
        if c0:   # the cached part: plain fp16 rows
            K = rng.standard_normal((c0, 4, 256)).astype(np.float16)
            V = rng.standard_normal((c0, 4, 256)).astype(np.float16)
            cache.append(0, np.full(c0, s, np.int32), np.arange(c0), dev(K), dev(V))
            pool.append(cache.seq_table(s), 0, K, V)
        seqs.append(s)
    ids = np.concatenate([np.full(c, s, np.int32) for s, c in zip(seqs, chunks)])
    pos = np.concatenate([np.arange(c0, c0 + c) for c0, c in zip(cached, chunks)])
    n = len(ids)
    q = (rng.standard_normal((n, 24, 256)) * 2).astype(np.float32)
    k = rng.standard_normal((n, 4, 256)).astype(np.float32)
    v = rng.standard_normal((n, 4, 256)).astype(np.float32)
    q_dev, qw_dev = dev(q), dev(qw)
    q_out = torch.zeros((n, 24, 256), dtype=torch.float16, device="cuda")
    torch.cuda.synchronize()
    cache.rope_append(0, ids, pos, q_dev, dev(k), dev(v), qw_dev, dev(kw), eps, q_out)   # K, V into the cache; q_out to compare
    cache.sync()
    want_q = O.rope_rows(q, qw, eps, np.repeat(pos, 24)).reshape(n, 24, 256)
    assert np.array_equal(q_out.cpu().numpy().view(np.uint16), want_q.view(np.uint16))
    two_step = torch.full((n, 24, 256), float("nan"), device="cuda", dtype=torch.float32)
    fused = torch.full((n, 24, 256), float("nan"), device="cuda", dtype=torch.float32)
    torch.cuda.synchronize()
    cache.attend_prefill(0, seqs, chunks, q_out, two_step, out_dtype=yahkv.OUT_F32)
    cache.attend_prefill_qraw(0, seqs, chunks, q_dev, qw_dev, eps, fused, out_dtype=yahkv.OUT_F32)
    cache.sync()
    a, b = two_step.cpu().numpy(), fused.cpu().numpy()
    assert np.isfinite(b).all()
    assert np.array_equal(a.view(np.uint32), b.view(np.uint32))   # the same q bits into the same kernel
    if fmt == yahkv.FMT_Q8_0:   # and against the float64 model
        k16 = O.rope_rows(k, kw, eps, np.repeat(pos, 4)).reshape(n, 4, 256)
        v16 = v.astype(np.float16)
        row = 0
        for s_, c0, c in zip(seqs, cached, chunks):
            pool.append(cache.seq_table(s_), c0, k16[row:row + c], v16[row:row + c])
            want = pool.attend_prefill_f64(cache.seq_table(s_), c0, want_q[row:row + c])
            assert np.abs(b[row:row + c] - want).max() <= ABS_TOL
            row += c
    cache.close()
