"""The CUDA path against the float64 oracle at the sizes the benchmark configurations run, through the C ABI.

Every expected value here comes from `oracle.PagedPool` (the CPU restatement), never from another library call:
  * the single-sequence parity fixture done literally: 4096 appends of one token each through a permuted table, pools
    byte-exact, then one decode step at position 4095;
  * the batch-decode configuration: sequences of the seed-0 batch, the longest (32,7xx tokens) included, in one
    shuffled pool, with automatic splits, fixed splits and the captured-graph batch path;
  * the long-context configuration: one 131,072-token q4_0 sequence merged from 64 splits;
  * the chunked-prefill configuration: 4 x (30,720 cached + a 2,048-token chunk), query rows chosen to cover the first
    and last row, the 127 / 128 tile edge, tiles that the planner splits along the keys and tiles it does not.
Tolerances: appends byte-exact (engine/gpu/loom/tools/dattn_q_check.py:223-225); decode attention 2e-3 max-abs and
the reference checker's own bar max|err| / max|ref| < 1e-4 (dattn_q_check.py:205-208). Prefill attention: 2e-3
max-abs and 1e-3 relative: it multiplies fp16 operands (dequantized K/V rounded to fp16, fp16 weights), each of which
carries 2^-11 = 4.9e-4 of relative rounding, and the reference does not hold its own prefill kernel to a bit-level or
1e-4 bar either (docs/architecture.md:88: judged by KL gates).
"""
import numpy as np
import pytest
import torch

import oracle as O
import yahkv
from gpu_util import assert_pools_equal, dev
from recipes import outlier_kv

pytestmark = pytest.mark.gpu
ABS_TOL, REL_TOL = 2e-3, 1e-4


def check(got, want, what, rel_tol=REL_TOL):
    err = float(np.abs(got - want).max())
    ref = float(np.abs(want).max())
    assert err <= ABS_TOL and err < rel_tol * ref, (what, err, err / ref)
    return err


def fill_sequence(cache, pool, layer, seq, table, n, rng, chunk=8192):
    """n tokens of fp16 N(0,1) K/V into `seq` on the GPU and into the oracle pool, chunk by chunk (host memory holds
    one chunk at a time)."""
    cache.seq_set_table(seq, table)
    for c0 in range(0, n, chunk):
        c1 = min(n, c0 + chunk)
        K = rng.standard_normal((c1 - c0, 4, 256), dtype=np.float32).astype(np.float16)
        V = rng.standard_normal((c1 - c0, 4, 256), dtype=np.float32).astype(np.float16)
        cache.append(layer, np.full(c1 - c0, seq, np.int32), np.arange(c0, c1, dtype=np.int64), dev(K), dev(V))
        pool.append(table, c0, K, V)
    cache.sync()


@pytest.mark.parametrize("fmt", [yahkv.FMT_Q8_0, yahkv.FMT_Q4_0])
def test_parity_fixture_one_token_per_call(fmt):
    n, num_pages = 4096, 64
    K, V, rng = outlier_kv(n, seed=0)
    table = rng.permutation(num_pages).astype(np.int32)
    q = rng.standard_normal((1, 24, 256)).astype(np.float16)
    cache = yahkv.KvCache(num_pages=num_pages, fmt=fmt, max_seqs=1, max_pages_per_seq=num_pages)
    seq = cache.seq_create()
    cache.seq_set_table(seq, table)
    Kd, Vd = dev(K), dev(V)
    one = np.zeros(1, np.int32) + seq
    for p in range(n):
        cache.append(0, one, np.array([p], np.int64), Kd[p:p + 1], Vd[p:p + 1])
    cache.sync()
    pool = O.PagedPool(fmt, num_pages)
    pool.append(table, 0, K, V)
    assert_pools_equal(cache, 0, pool)
    out = torch.zeros(1, 24, 256, device="cuda")
    cache.attend_decode(0, [seq], dev(q), out, out_dtype=yahkv.OUT_F32)
    cache.sync()
    want = pool.attend_decode_f64(table, n, q[0])
    assert np.abs(out.cpu().numpy()[0] - want).max() <= ABS_TOL
    cache.close()


def test_batch_decode_configuration_against_the_oracle():
    lens_all = np.random.default_rng(0).integers(1024, 32768 + 1, 32)        # the benchmark's seed-0 batch
    order = np.argsort(lens_all)
    picks = [int(order[-1]), int(order[0]), int(order[16]), int(order[-2]), int(order[7])]   # longest, shortest, ...
    lens = [int(lens_all[i]) for i in picks] + [32768]        # and the configuration's longest possible context
    assert lens[0] == int(lens_all.max())
    steps = 2
    pages = [(n + steps + 63) // 64 for n in lens]
    num_pages = sum(pages) + 17
    rng = np.random.default_rng(1234)
    cache = yahkv.KvCache(n_layers=1, num_pages=num_pages, fmt=yahkv.FMT_Q8_0, max_seqs=len(lens),
                          max_pages_per_seq=max(pages) + 1)
    pool = O.PagedPool(yahkv.FMT_Q8_0, num_pages)
    perm = rng.permutation(num_pages).astype(np.int32)
    seqs, tables, off = [], [], 0
    for i, n in enumerate(lens):
        s = cache.seq_create()
        table = perm[off:off + pages[i]].copy()
        off += pages[i]
        fill_sequence(cache, pool, 0, s, table, n, rng)
        seqs.append(s), tables.append(table)
    b = len(lens)
    q = rng.standard_normal((b, 24, 256)).astype(np.float16)
    gate = rng.standard_normal((b, 24, 256)).astype(np.float32)
    want = np.stack([pool.attend_decode_f64(tables[i], lens[i], q[i], gate[i]) for i in range(b)])
    worst = 0.0
    for n_splits in (0, 1, 64):
        out = torch.full((b, 24, 256), float("nan"), device="cuda")
        torch.cuda.synchronize()
        cache.attend_decode(0, seqs, dev(q), out, gate=dev(gate), out_dtype=yahkv.OUT_F32, n_splits=n_splits)
        cache.sync()
        worst = max(worst, check(out.cpu().numpy(), want, ("eager", n_splits)))
    # the device-resident batch replayed from a captured graph: each replay appends one token and attends
    batch = yahkv.DecodeBatch(cache, seqs)
    batch.prepare(steps)
    side = torch.cuda.Stream()
    k_s = torch.zeros(b, 4, 256, device="cuda", dtype=torch.float16)
    v_s, q_s = torch.zeros_like(k_s), torch.zeros(b, 24, 256, device="cuda", dtype=torch.float16)
    o_s = torch.zeros(b, 24, 256, device="cuda", dtype=torch.float32)
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph, stream=side):
        sp = torch.cuda.current_stream().cuda_stream
        batch.plan(stream=sp)
        batch.decode_layer(0, k_s, v_s, q_s, o_s, out_dtype=yahkv.OUT_F32, stream=sp)
        batch.advance(stream=sp)
    cur = list(lens)
    for step in range(steps):
        k = rng.standard_normal((b, 4, 256)).astype(np.float16)
        v = rng.standard_normal((b, 4, 256)).astype(np.float16)
        qq = rng.standard_normal((b, 24, 256)).astype(np.float16)
        k_s.copy_(torch.from_numpy(k)), v_s.copy_(torch.from_numpy(v)), q_s.copy_(torch.from_numpy(qq))
        torch.cuda.synchronize()
        graph.replay()
        torch.cuda.synchronize()
        for i in range(b):
            pool.append(tables[i], cur[i], k[i:i + 1], v[i:i + 1])
        cur = [n + 1 for n in cur]
        want = np.stack([pool.attend_decode_f64(tables[i], cur[i], qq[i]) for i in range(b)])
        worst = max(worst, check(o_s.cpu().numpy(), want, ("graph", step)))
    batch.commit(steps)
    cache.sync()
    for i, s in enumerate(seqs):      # the graph's appends are the oracle's bytes
        kb, vb = cache.export_token(0, s, cur[i] - 1)
        slot = O.slot(tables[i], cur[i] - 1, num_pages)
        assert np.array_equal(kb, pool.export_row(0, slot)) and np.array_equal(vb, pool.export_row(1, slot))
    batch.close()
    cache.close()
    print(f"batch-decode configuration: worst max-abs error {worst:.2e}")


def test_long_context_q4_0_with_64_splits_against_the_oracle():
    n, fmt = 131072, yahkv.FMT_Q4_0
    pages = n // 64
    rng = np.random.default_rng(77)
    cache = yahkv.KvCache(n_layers=1, num_pages=pages + 5, fmt=fmt, max_seqs=1, max_pages_per_seq=pages)
    pool = O.PagedPool(fmt, pages + 5)
    table = rng.permutation(pages + 5)[:pages].astype(np.int32)
    s = cache.seq_create()
    fill_sequence(cache, pool, 0, s, table, n, rng)
    q = rng.standard_normal((1, 24, 256)).astype(np.float16)
    want = pool.attend_decode_f64(table, n, q[0])
    for n_splits in (64, 0):
        out = torch.full((1, 24, 256), float("nan"), device="cuda")
        torch.cuda.synchronize()
        cache.attend_decode(0, [s], dev(q), out, out_dtype=yahkv.OUT_F32, n_splits=n_splits)
        cache.sync()
        check(out.cpu().numpy()[0], want, ("q4_0 131072", n_splits))
    cache.close()


def test_chunked_prefill_configuration_against_the_oracle():
    n_seq, cached, chunk = 4, 30720, 2048
    n = cached + chunk
    pages = n // 64
    rng = np.random.default_rng(4)
    num_pages = n_seq * pages + 8
    cache = yahkv.KvCache(n_layers=1, num_pages=num_pages, fmt=yahkv.FMT_Q8_0, max_seqs=n_seq, max_pages_per_seq=pages,
                          max_batch_tokens=n_seq * chunk)
    pool = O.PagedPool(yahkv.FMT_Q8_0, num_pages)
    perm = rng.permutation(num_pages).astype(np.int32)
    seqs, tables = [], []
    for i in range(n_seq):
        s = cache.seq_create()
        table = perm[i * pages:(i + 1) * pages].copy()
        fill_sequence(cache, pool, 0, s, table, n, rng)       # cached part and the chunk's own keys
        seqs.append(s), tables.append(table)
    q = rng.standard_normal((n_seq * chunk, 24, 256), dtype=np.float32).astype(np.float16)
    gate = rng.standard_normal((n_seq * chunk, 24, 256), dtype=np.float32)
    out = torch.full((n_seq * chunk, 24, 256), float("nan"), device="cuda")
    torch.cuda.synchronize()
    cache.attend_prefill(0, seqs, [chunk] * n_seq, dev(q), out, gate=dev(gate), out_dtype=yahkv.OUT_F32)
    cache.sync()
    got = out.cpu().numpy()
    assert np.isfinite(got).all()
    # Rows per sequence: the chunk's first and last row, both sides of the first tile edge, and two interior rows. The
    # planner sorts tiles by their key count and splits the ones of the last partly filled wave along the keys: those
    # are the chunk's first row tiles, so rows 0 .. 128 sit in split tiles and the late rows in whole ones.
    rows = {0: [0, 127, 128, 2047], 1: [1, 1000, 1407, 2046], 2: [64, 129, 1920, 2047], 3: [0, 255, 256, 1024]}
    worst, checked = 0.0, 0
    for i in range(n_seq):
        qi, gi = q[i * chunk:(i + 1) * chunk], gate[i * chunk:(i + 1) * chunk]
        for r in rows[i]:
            want = pool.attend_prefill_f64(tables[i], cached, qi, q_begin=r, q_end=r + 1, gate=gi)[0]
            worst = max(worst, check(got[i * chunk + r], want, ("prefill", i, r), rel_tol=1e-3))
            checked += 1
    assert checked >= 16
    cache.close()
    print(f"chunked-prefill configuration: {checked} rows, worst max-abs error {worst:.2e}")


@pytest.mark.parametrize("fmt", [yahkv.FMT_KV8A16, yahkv.FMT_KV4A16])
def test_batch_decode_configuration_in_the_reference_formats(fmt):
    """The benchmark batch's longest and shortest contexts and the configuration's maximum (32768) in the reference's
    own cache formats: chunked fill with a per-sequence K mean, then two decode steps (append one token, attend) with
    automatic, single and 64-way splits, every row against the float64 model over the oracle's own pools."""
    lens_all = np.random.default_rng(0).integers(1024, 32768 + 1, 32)
    lens = [int(lens_all.max()), int(lens_all.min()), 32768 - 2]
    steps = 2
    pages = [(n + steps + 63) // 64 for n in lens]
    num_pages = sum(pages) + 9
    rng = np.random.default_rng(4321 + fmt)
    cache = yahkv.KvCache(n_layers=1, num_pages=num_pages, fmt=fmt, max_seqs=len(lens), max_pages_per_seq=max(pages) + 1)
    pool = (O.Kv8Pool if fmt == yahkv.FMT_KV8A16 else O.Kv4Pool)(num_pages)
    perm = rng.permutation(num_pages).astype(np.int32)
    seqs, tables, states, off = [], [], [], 0
    for i, n in enumerate(lens):
        s = cache.seq_create()
        table = perm[off:off + pages[i]].copy()
        off += pages[i]
        cache.seq_set_table(s, table)
        m = (0.5 * rng.standard_normal((4, 256))).astype(np.float32)
        cache.seq_set_kmean(s, m)
        st = pool.new_sequence(m)
        for c0 in range(0, n, 8192):
            c1 = min(n, c0 + 8192)
            K = (rng.standard_normal((c1 - c0, 4, 256), dtype=np.float32) + m).astype(np.float16)
            V = rng.standard_normal((c1 - c0, 4, 256), dtype=np.float32).astype(np.float16)
            cache.append(0, np.full(c1 - c0, s, np.int32), np.arange(c0, c1, dtype=np.int64), dev(K), dev(V))
            pool.append(table, c0, K, V, *st)
        seqs.append(s), tables.append(table), states.append(st)
    cache.sync()
    b = len(lens)
    cur = list(lens)
    for step in range(steps):
        k = rng.standard_normal((b, 4, 256)).astype(np.float16)
        v = rng.standard_normal((b, 4, 256)).astype(np.float16)
        q = rng.standard_normal((b, 24, 256)).astype(np.float16)
        gate = rng.standard_normal((b, 24, 256)).astype(np.float32)
        cache.append(0, seqs, cur, dev(k), dev(v))
        for i in range(b):
            pool.append(tables[i], cur[i], k[i:i + 1], v[i:i + 1], *states[i])
        cur = [n + 1 for n in cur]
        want = np.stack([pool.attend_decode_f64(tables[i], cur[i], q[i], states[i][0], gate[i]) for i in range(b)])
        for n_splits in (0, 1, 64):
            out = torch.full((b, 24, 256), float("nan"), device="cuda")
            torch.cuda.synchronize()
            cache.attend_decode(0, seqs, dev(q), out, gate=dev(gate), out_dtype=yahkv.OUT_F32, n_splits=n_splits)
            cache.sync()
            check(out.cpu().numpy(), want, (fmt, step, n_splits))
    # the last page of every sequence, byte for byte (K rows of the decode steps, the V tiles they completed)
    for i in range(b):
        p = int(tables[i][(cur[i] - 1) // 64])
        for side, codes, pairs in ((yahkv.SIDE_K, pool.kcodes, pool.kscales), (yahkv.SIDE_V, pool.vcodes, pool.vstats)):
            got_c, got_p = cache.read_page(0, side, p)
            if side == yahkv.SIDE_K:
                n_tok = (cur[i] - 1) % 64 + 1
                assert np.array_equal(got_c[:, :n_tok], codes[p][:, :n_tok]) and np.array_equal(got_p[:, :n_tok], pairs[p][:, :n_tok])
            else:
                n_tiles = ((cur[i] - 1) % 64 + 1) // 16       # complete tiles of the page
                assert np.array_equal(got_c[:, :n_tiles], codes[p][:, :n_tiles]) and np.array_equal(got_p[:, :n_tiles], pairs[p][:, :n_tiles])
    cache.close()
