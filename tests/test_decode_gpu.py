"""Paged split-K decode attention on the GPU against the float64 oracle and the golden vectors.
Tolerance: 2e-3 max-abs (fp32 softmax accumulation), and the reference's own bar for its kernels,
max|err| / max|ref| < 1e-4 (dattn_q_check.py:205-208), on N(0,1) data."""
import numpy as np
import pytest
import torch

import oracle as O
import yahkv
from gpu_util import dev, fill_both
from recipes import checker_recipe, outlier_kv

pytestmark = pytest.mark.gpu
ABS_TOL = 2e-3


def run_decode(cache, layer, seqs, q, gate=None, out_dtype=yahkv.OUT_F32, n_splits=0):
    n = len(seqs)
    out = torch.full((n, 24, 256), float("nan"), device="cuda",
                     dtype=torch.float32 if out_dtype == yahkv.OUT_F32 else torch.float16)
    torch.cuda.synchronize()   # the fill runs on torch's stream, the library on its own
    cache.attend_decode(layer, seqs, dev(q), out, gate=None if gate is None else dev(gate), out_dtype=out_dtype,
                        n_splits=n_splits)
    cache.sync()
    return out.float().cpu().numpy().astype(np.float64)


@pytest.mark.parametrize("name,fmt", [("q8_0", yahkv.FMT_Q8_0), ("q4_0", yahkv.FMT_Q4_0)])
def test_checker_recipe_against_golden(golden, name, fmt):
    r = checker_recipe()
    cache = yahkv.KvCache(num_pages=r["T"] // 64, fmt=fmt, max_seqs=1, max_pages_per_seq=r["T"] // 64)
    seq = cache.seq_create()
    n = r["pos"] + 1
    fill_both(cache, None, 0, seq, r["ptab"], r["K"][:n], r["V"][:n])
    for gate, key in ((r["gate"], "gated"), (None, "plain")):
        want = golden[f"attn_{name}_{key}"]
        for n_splits in (0, 1, 3):
            got = run_decode(cache, 0, [seq], r["q"][None], None if gate is None else gate[None], n_splits=n_splits)[0]
            err = np.abs(got - want).max()
            assert err <= ABS_TOL and err / np.abs(want).max() < 1e-4, (key, n_splits, err)


@pytest.mark.parametrize("fmt", [yahkv.FMT_Q8_0, yahkv.FMT_Q4_0])
def test_parity_fixture_with_outlier_channels(fmt):
    # one sequence, 4096 tokens, four x20 outlier channels per head, permuted 64-page table, q ~ N(0,1)
    n = 4096
    K, V, rng = outlier_kv(n, seed=0)
    table = rng.permutation(64).astype(np.int32)
    q = rng.standard_normal((1, 24, 256)).astype(np.float16)
    cache = yahkv.KvCache(num_pages=64, fmt=fmt, max_seqs=1, max_pages_per_seq=64)
    pool = O.PagedPool(fmt, 64)
    seq = cache.seq_create()
    fill_both(cache, pool, 0, seq, table, K, V)
    want = pool.attend_decode_f64(table, n, q[0])
    for n_splits in (0, 1, 64):
        got = run_decode(cache, 0, [seq], q, n_splits=n_splits)[0]
        assert np.abs(got - want).max() <= ABS_TOL, (n_splits, np.abs(got - want).max())
    got16 = run_decode(cache, 0, [seq], q, out_dtype=yahkv.OUT_F16)[0]
    assert np.abs(got16 - want).max() <= ABS_TOL + np.abs(want).max() * 2.0 ** -11


@pytest.mark.parametrize("fmt", [yahkv.FMT_Q8_0, yahkv.FMT_Q4_0])
def test_ragged_batch_edge_lengths(fmt):
    # lengths around every boundary: 1 key, a page minus one, exactly a page, a page plus one, many pages
    lens = [1, 2, 15, 16, 17, 63, 64, 65, 127, 128, 129, 1000, 1024, 2500]
    rng = np.random.default_rng(5)
    num_pages = sum((n + 63) // 64 for n in lens) + 5
    cache = yahkv.KvCache(n_layers=2, num_pages=num_pages, fmt=fmt, max_seqs=len(lens), max_pages_per_seq=40)
    pool = O.PagedPool(fmt, num_pages)
    free = list(rng.permutation(num_pages))
    seqs, tables = [], []
    for n in lens:
        s = cache.seq_create()
        table = np.array([free.pop() for _ in range((n + 63) // 64)], np.int32)
        K = rng.standard_normal((n, 4, 256)).astype(np.float16)
        V = rng.standard_normal((n, 4, 256)).astype(np.float16)
        fill_both(cache, pool, 1, s, table, K, V)
        seqs.append(s); tables.append(table)
    q = (0.5 * rng.standard_normal((len(lens), 24, 256))).astype(np.float16)
    gate = rng.standard_normal((len(lens), 24, 256)).astype(np.float32)
    want = np.stack([pool.attend_decode_f64(tables[i], lens[i], q[i], gate[i]) for i in range(len(lens))])
    for n_splits in (0, 1, 7):
        got = run_decode(cache, 1, seqs, q, gate, n_splits=n_splits)
        err = np.abs(got - want).reshape(len(lens), -1).max(1)
        assert err.max() <= ABS_TOL, (n_splits, err)
        assert err.max() / np.abs(want).max() < 1e-4
    # a sub-batch in another order reads the right rows
    order = [13, 0, 7]
    got = run_decode(cache, 1, [seqs[i] for i in order], q[order], gate[order])
    assert np.abs(got - want[order]).max() <= ABS_TOL


def test_recycled_pages_do_not_leak_into_the_next_sequence():
    rng = np.random.default_rng(8)
    cache = yahkv.KvCache(num_pages=4, max_seqs=2, max_pages_per_seq=4)
    a = cache.seq_create()
    big = (100 * rng.standard_normal((256, 4, 256))).astype(np.float16)
    fill_both(cache, None, 0, a, [0, 1, 2, 3], big, big)
    cache.seq_free(a)
    b = cache.seq_create()
    pool = O.PagedPool(yahkv.FMT_Q8_0, 4)
    K = rng.standard_normal((70, 4, 256)).astype(np.float16)
    V = rng.standard_normal((70, 4, 256)).astype(np.float16)
    cache.seq_reserve(b, 70)
    table = cache.seq_table(b)
    fill_both(cache, pool, 0, b, table, K, V)
    q = rng.standard_normal((1, 24, 256)).astype(np.float16)
    got = run_decode(cache, 0, [b], q)[0]
    want = pool.attend_decode_f64(table, 70, q[0])
    assert np.abs(got - want).max() <= ABS_TOL


def test_append_then_attend_sees_the_new_key_and_errors_are_caught():
    rng = np.random.default_rng(10)
    cache = yahkv.KvCache(num_pages=8, max_seqs=2, max_pages_per_seq=4)
    pool = O.PagedPool(yahkv.FMT_Q8_0, 8)
    s = cache.seq_create()
    q = rng.standard_normal((1, 24, 256)).astype(np.float16)
    out = torch.zeros(1, 24, 256, device="cuda")
    with pytest.raises(yahkv.YahkvError) as e:
        cache.attend_decode(0, [s], dev(q), out, out_dtype=yahkv.OUT_F32)      # nothing appended yet
    assert e.value.code == yahkv.ERR_ORDER
    cache.seq_reserve(s, 200)
    table = cache.seq_table(s)
    K = rng.standard_normal((130, 4, 256)).astype(np.float16)
    V = rng.standard_normal((130, 4, 256)).astype(np.float16)
    for p in range(130):      # decode loop: append position p, then attend over 0..p
        cache.append(0, [s], [p], dev(K[p:p + 1]), dev(V[p:p + 1]))
        if p in (0, 1, 63, 64, 129):
            pool_p = O.PagedPool(yahkv.FMT_Q8_0, 8)
            pool_p.append(table, 0, K[:p + 1], V[:p + 1])
            got = run_decode(cache, 0, [s], q)[0]
            assert np.abs(got - pool_p.attend_decode_f64(table, p + 1, q[0])).max() <= ABS_TOL, p
    with pytest.raises(yahkv.YahkvError):
        cache.attend_decode(0, [s], dev(q), out, out_dtype=5)
    with pytest.raises(yahkv.YahkvError):
        cache.attend_decode(0, [s], dev(q), out, out_dtype=yahkv.OUT_F32, n_splits=65)
    with pytest.raises(yahkv.YahkvError):
        cache.attend_decode(1, [s], dev(q), out, out_dtype=yahkv.OUT_F32)


def test_host_buffer_step_matches_device_calls():
    rng = np.random.default_rng(12)
    cache = yahkv.KvCache(n_layers=2, num_pages=16, max_seqs=3, max_pages_per_seq=4)
    pool = O.PagedPool(yahkv.FMT_Q8_0, 16)
    seqs = [cache.seq_create() for _ in range(3)]
    lens = [5, 64, 100]
    hist = []
    for s, n in zip(seqs, lens):
        cache.seq_reserve(s, n + 2)
        K = rng.standard_normal((n + 2, 4, 256)).astype(np.float16)
        V = rng.standard_normal((n + 2, 4, 256)).astype(np.float16)
        fill_both(cache, None, 1, s, cache.seq_table(s), K[:n], V[:n])
        hist.append((K, V))
    for step in range(2):
        k = np.stack([hist[i][0][lens[i] + step] for i in range(3)])
        v = np.stack([hist[i][1][lens[i] + step] for i in range(3)])
        q = rng.standard_normal((3, 24, 256)).astype(np.float16)
        gate = rng.standard_normal((3, 24, 256)).astype(np.float32)
        out = np.zeros((3, 24, 256), np.float32)
        cache.decode_step_host(1, seqs, k, v, q, out, gate=gate, out_dtype=yahkv.OUT_F32)
        for i, s in enumerate(seqs):
            p = O.PagedPool(yahkv.FMT_Q8_0, 16)
            n = lens[i] + step + 1
            p.append(cache.seq_table(s), 0, hist[i][0][:n], hist[i][1][:n])
            want = p.attend_decode_f64(cache.seq_table(s), n, q[i], gate[i])
            assert np.abs(out[i] - want).max() <= ABS_TOL


def test_pipelined_host_steps_match_the_blocking_ones():
    """Six layer-steps queued back to back with page-locked host buffers (two staging sets in turn, copies on their own
    streams) give bit-identical outputs to the same steps made one at a time on a second cache."""
    rng = np.random.default_rng(77)
    lens, n_layers = [70, 200, 129], 3
    caches = [yahkv.KvCache(n_layers=n_layers, num_pages=16, fmt=yahkv.FMT_Q8_0, max_seqs=3, max_pages_per_seq=5)
              for _ in range(2)]
    seqs = [[c.seq_create() for _ in lens] for c in caches]
    for i, n in enumerate(lens):
        K = rng.standard_normal((n, 4, 256)).astype(np.float16)
        V = rng.standard_normal((n, 4, 256)).astype(np.float16)
        for c, ss in zip(caches, seqs):
            c.seq_reserve(ss[i], n + 2)
            for layer in range(n_layers):
                c.append(layer, np.full(n, ss[i], np.int32), np.arange(n), dev(K), dev(V))
    pin = lambda shape, dt: torch.empty(shape, dtype=dt).pin_memory()
    steps = [(step, layer) for step in range(2) for layer in range(n_layers)]
    k = [pin((3, 4, 256), torch.float16).copy_(torch.from_numpy(rng.standard_normal((3, 4, 256)).astype(np.float16))) for _ in steps]
    v = [pin((3, 4, 256), torch.float16).copy_(torch.from_numpy(rng.standard_normal((3, 4, 256)).astype(np.float16))) for _ in steps]
    q = [pin((3, 24, 256), torch.float16).copy_(torch.from_numpy(rng.standard_normal((3, 24, 256)).astype(np.float16))) for _ in steps]
    out_a = [pin((3, 24, 256), torch.float32).zero_() for _ in steps]
    out_b = [pin((3, 24, 256), torch.float32).zero_() for _ in steps]
    for i, (_, layer) in enumerate(steps):
        caches[0].decode_step_host_async(layer, seqs[0], k[i], v[i], q[i], out_a[i], out_dtype=yahkv.OUT_F32)
    caches[0].decode_step_host_wait()
    for i, (_, layer) in enumerate(steps):
        caches[1].decode_step_host(layer, seqs[1], k[i], v[i], q[i], out_b[i], out_dtype=yahkv.OUT_F32)
    for a, b in zip(out_a, out_b):
        assert torch.equal(a, b) and float(a.abs().max()) > 0
    assert [caches[0].seq_len(s, 0) for s in seqs[0]] == [n + 2 for n in lens]
    for c in caches:
        c.close()


@pytest.mark.parametrize("fmt,ctx_len,batch", [(yahkv.FMT_Q8_0, 32768, 4), (yahkv.FMT_Q4_0, 131072, 1)])
def test_full_length_properties(fmt, ctx_len, batch):
    """At the benchmark's context lengths, where the float64 oracle would take minutes: size-independent properties.
    (1) softmax weights sum to one: with every cached V row equal, the output is that row dequantized, for any K and q.
    (2) split invariance: 1, 64 and automatic splits agree."""
    pages = ctx_len // 64
    cache = yahkv.KvCache(num_pages=batch * pages, fmt=fmt, max_seqs=batch, max_pages_per_seq=pages)
    g = torch.Generator(device="cuda").manual_seed(1)
    v_row = torch.randn(1, 4, 256, device="cuda", generator=g).half()
    seqs = []
    perm = torch.randperm(batch * pages, generator=torch.Generator().manual_seed(2)).numpy().astype(np.int32)
    for b in range(batch):
        s = cache.seq_create()
        cache.seq_set_table(s, perm[b * pages:(b + 1) * pages])
        for c0 in range(0, ctx_len, 8192):
            K = torch.randn(8192, 4, 256, device="cuda", generator=g).half()
            cache.append(0, np.full(8192, s, np.int32), np.arange(c0, c0 + 8192), K, v_row.expand(8192, 4, 256).contiguous())
        seqs.append(s)
    q = torch.randn(batch, 24, 256, device="cuda", generator=g).half()
    outs = {}
    for n_splits in (0, 1, 64):
        out = torch.zeros(batch, 24, 256, device="cuda")
        cache.attend_decode(0, seqs, q, out, out_dtype=yahkv.OUT_F32, n_splits=n_splits)
        cache.sync()
        outs[n_splits] = out.cpu().numpy()
    kb, vb = cache.export_token(0, seqs[0], ctx_len - 1)
    v_deq = O.dequantize(vb, fmt).reshape(4, 256)
    want = np.repeat(v_deq, 6, axis=0)[None].repeat(batch, 0)
    for n_splits, got in outs.items():
        assert np.abs(got - want).max() <= ABS_TOL, n_splits
    # The tensor-core MMA truncates its fp32 accumulate, so one unit summing all 512+ pages drifts by up to
    # ~1e-4 relative against 64 short units; still far inside the tolerance.
    assert np.abs(outs[1] - outs[64]).max() <= 5e-4 and np.abs(outs[0] - outs[64]).max() <= 5e-4


def test_head_sharded_contexts_produce_disjoint_slices_of_the_same_output():
    """Contexts that hold KV heads {0,1} and {2,3} of the same sequences (the head-sharded layout) write exactly the
    rows of their own query heads, bit-identical to a context that holds all four, and leave the other rows alone;
    the same for chunked prefill."""
    rng = np.random.default_rng(91)
    n, chunk = 333, 70
    K = rng.standard_normal((n, 4, 256)).astype(np.float16)
    V = rng.standard_normal((n, 4, 256)).astype(np.float16)
    q = rng.standard_normal((1, 24, 256)).astype(np.float16)
    qc = rng.standard_normal((chunk, 24, 256)).astype(np.float16)
    table = rng.permutation(8)[:6].astype(np.int32)
    outs = []
    for begin, count in ((0, 0), (0, 2), (2, 2)):
        c = yahkv.KvCache(n_layers=1, num_pages=8, fmt=yahkv.FMT_Q8_0, max_seqs=1, max_pages_per_seq=6,
                          kv_head_begin=begin, kv_head_count=count)
        s = c.seq_create()
        c.seq_set_table(s, table)
        c.append(0, np.full(n, s, np.int32), np.arange(n), dev(K), dev(V))
        dec = torch.full((1, 24, 256), float("nan"), device="cuda")
        pre = torch.full((chunk, 24, 256), float("nan"), device="cuda")
        torch.cuda.synchronize()
        c.attend_decode(0, [s], dev(q), dec, out_dtype=yahkv.OUT_F32, n_splits=3)
        c.attend_prefill(0, [s], [chunk], dev(qc), pre, out_dtype=yahkv.OUT_F32)
        c.sync()
        outs.append((dec.cpu().numpy(), pre.cpu().numpy()))
        if count:
            with pytest.raises(yahkv.YahkvError):
                yahkv.DecodeBatch(c, [s])
        c.close()
    (dec_all, pre_all), lo, hi = outs
    assert not np.isnan(dec_all).any() and not np.isnan(pre_all).any()
    for (dec, pre), heads in ((lo, slice(0, 12)), (hi, slice(12, 24))):
        other = slice(12, 24) if heads.start == 0 else slice(0, 12)
        assert np.array_equal(dec[:, heads], dec_all[:, heads]) and np.isnan(dec[:, other]).all()
        assert np.array_equal(pre[:, heads], pre_all[:, heads]) and np.isnan(pre[:, other]).all()
