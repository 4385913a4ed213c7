"""The reference's own kv8a16 cache format on the GPU (YAHKV_FMT_KV8A16): appends byte-exact against the CPU restatement
(itself pinned bit for bit to the reference's numpy models, tests/test_kv8a16_oracle_cpu.py) and against the golden
vectors made with those models; decode attention against the float64 model to the reference checker's own bar,
max|err| / max|ref| < 1e-4 (engine/gpu/loom/tools/dattn_q_check.py:205-208). Pages hold 64 tokens = four 16-key tiles
here (256 tokens in the reference)."""
import hashlib
import os

import numpy as np
import pytest
import torch

import oracle as O
import yahkv
from gpu_util import dev
from recipes import kv8a16_recipe

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def read_pools(cache, layer, num_pages):
    k = [cache.read_page(layer, yahkv.SIDE_K, p) for p in range(num_pages)]
    v = [cache.read_page(layer, yahkv.SIDE_V, p) for p in range(num_pages)]
    return (np.stack([a for a, _ in k]), np.stack([b for _, b in k]), np.stack([a for a, _ in v]), np.stack([b for _, b in v]))


def assert_pools(cache, layer, pool):
    kc, ks, vc, vs = read_pools(cache, layer, pool.num_pages)
    assert np.array_equal(kc, pool.kcodes), f"K codes differ in {(kc != pool.kcodes).sum()} bytes"
    assert np.array_equal(ks, pool.kscales), f"K scale pairs differ in {(ks != pool.kscales).sum()} values"
    assert np.array_equal(vc, pool.vcodes), f"V codes differ in {(vc != pool.vcodes).sum()} bytes"
    assert np.array_equal(vs, pool.vstats), f"V statistic pairs differ in {(vs != pool.vstats).sum()} values"


def run_decode(cache, layer, seqs, q, gate=None, n_splits=0):
    out = torch.full((len(seqs), 24, 256), float("nan"), device="cuda")
    torch.cuda.synchronize()
    cache.attend_decode(layer, seqs, dev(q), out, gate=None if gate is None else dev(gate), out_dtype=yahkv.OUT_F32,
                        n_splits=n_splits)
    cache.sync()
    return out.cpu().numpy().astype(np.float64)


def test_checker_recipe_against_the_reference_models():
    g8 = np.load(os.path.join(ROOT, "tests", "golden", "kv8a16.npz"))
    r = kv8a16_recipe()
    n = int(g8["n_keys"])
    rng = np.random.default_rng(3)
    num_pages = 7
    table = rng.permutation(num_pages)[:5].astype(np.int32)
    cache = yahkv.KvCache(n_layers=2, num_pages=num_pages, fmt=yahkv.FMT_KV8A16, max_seqs=2, max_pages_per_seq=5)
    pool = O.Kv8Pool(num_pages)
    open_tile, mean = pool.new_sequence(r["m"])
    seq = cache.seq_create()
    cache.seq_set_table(seq, table)
    cache.seq_set_kmean(seq, r["m"])
    K, V = r["K"].reshape(-1, 4, 256), r["V"].reshape(-1, 4, 256)
    Kd, Vd = dev(K), dev(V)

    def append(p0, p1):
        cache.append(1, np.full(p1 - p0, seq, np.int32), np.arange(p0, p1, dtype=np.int64), Kd[p0:p1], Vd[p0:p1])
        pool.append(table, p0, K[p0:p1], V[p0:p1], open_tile, mean)
    append(0, 100)                       # a chunk that ends inside a tile
    for p in range(100, 130):            # single tokens across tile boundaries (the decode path)
        append(p, p + 1)
    append(130, n)
    cache.sync()
    assert_pools(cache, 1, pool)
    assert_pools(cache, 0, O.Kv8Pool(num_pages))        # the other layer is untouched
    got_open = cache.read_open_tile(seq, 1)
    used = n - 16 * ((n - 1) // 16)
    assert np.array_equal(got_open.view(np.uint16)[:, :, :used], open_tile[:, :, :used])
    # the reference's own arrays: the first two tiles' dwords and pairs as its numpy models made them
    kc, ks, vc, vs = read_pools(cache, 1, num_pages)
    for t in range(2):
        want_c = g8["vq_head"][t].view(np.uint8).reshape(4, 256, 16)
        want_s = g8["vs_head"][t].view(np.uint16).reshape(4, 256, 2)
        assert np.array_equal(vc[table[0], :, t], want_c) and np.array_equal(vs[table[0], :, t], want_s)
    for p in range(32):
        assert np.array_equal(kc[table[0], :, p].reshape(-1), g8["kq_head"][p].view(np.uint8))
        assert np.array_equal(ks[table[0], :, p].reshape(-1), g8["ks_head"][p].view(np.uint16))
    for name, gate in (("gated", r["gate"]), ("plain", None)):
        want = g8[f"attn_{name}"]
        for n_splits in (0, 1, 3):
            got = run_decode(cache, 1, [seq], r["q"][None], None if gate is None else gate[None], n_splits)[0]
            err = np.abs(got - want).max()
            assert err <= 2e-3 and err / np.abs(want).max() < 1e-4, (name, n_splits, err, err / np.abs(want).max())
    cache.close()


def test_ragged_batch_with_means_and_decode_steps():
    rng = np.random.default_rng(11)
    lens = [1, 15, 16, 17, 64, 100, 1000, 2049]
    pages = [(n + 8 + 63) // 64 for n in lens]
    num_pages = sum(pages) + 3
    cache = yahkv.KvCache(n_layers=1, num_pages=num_pages, fmt=yahkv.FMT_KV8A16, max_seqs=len(lens),
                          max_pages_per_seq=max(pages), max_batch_tokens=4096)
    pool = O.Kv8Pool(num_pages)
    perm = rng.permutation(num_pages).astype(np.int32)
    seqs, tables, states, off = [], [], [], 0
    for i, n in enumerate(lens):
        s = cache.seq_create()
        table = perm[off:off + pages[i]].copy()
        off += pages[i]
        cache.seq_set_table(s, table)
        m = (0.5 * rng.standard_normal((4, 256))).astype(np.float32) if i % 2 else np.zeros((4, 256), np.float32)
        cache.seq_set_kmean(s, m)
        st = pool.new_sequence(m)
        K = (rng.standard_normal((n, 4, 256)) + m).astype(np.float16)
        V = rng.standard_normal((n, 4, 256)).astype(np.float16)
        for c0 in range(0, n, 4096):
            c1 = min(n, c0 + 4096)
            cache.append(0, np.full(c1 - c0, s, np.int32), np.arange(c0, c1, dtype=np.int64), dev(K[c0:c1]), dev(V[c0:c1]))
        pool.append(table, 0, K, V, *st)
        seqs.append(s), tables.append(table), states.append(st)
    cache.sync()
    assert_pools(cache, 0, pool)
    cur = list(lens)
    for step in range(3):                # batched decode steps: one token per sequence, then attend
        k = rng.standard_normal((len(lens), 4, 256)).astype(np.float16)
        v = rng.standard_normal((len(lens), 4, 256)).astype(np.float16)
        q = (0.5 * rng.standard_normal((len(lens), 24, 256))).astype(np.float16)
        gate = rng.standard_normal((len(lens), 24, 256)).astype(np.float32)
        cache.append(0, seqs, cur, dev(k), dev(v))
        for i in range(len(lens)):
            pool.append(tables[i], cur[i], k[i:i + 1], v[i:i + 1], *states[i])
        cur = [n + 1 for n in cur]
        want = np.stack([pool.attend_decode_f64(tables[i], cur[i], q[i], states[i][0], gate[i]) for i in range(len(lens))])
        for n_splits in (0, 5):
            got = run_decode(cache, 0, seqs, q, gate, n_splits)
            err = np.abs(got - want).reshape(len(lens), -1).max(1)
            assert err.max() <= 2e-3 and err.max() / np.abs(want).max() < 1e-4, (step, n_splits, err)
    assert_pools(cache, 0, pool)
    # what the format does not support is refused before anything is launched
    x = torch.zeros(4, 24, 256, dtype=torch.float16, device="cuda")
    for call in (lambda: cache.export_token(0, seqs[0], 0),
                 lambda: cache.seq_set_len(seqs[0], 1),
                 lambda: cache.seq_set_kmean(seqs[0], np.zeros((4, 256), np.float32))):
        with pytest.raises(yahkv.YahkvError):
            call()
    cache.close()


def test_chunked_prefill_attention():
    """A prompt goes in as chunks (append, then attend_prefill over the cache, the chunk included), with lengths that
    end inside a tile, on a tile edge and on a page edge; sampled rows of every chunk against the float64 model over the
    dequantized cache. The operands are fp16 on the tensor cores: 2e-3 absolute, 1e-3 of the largest output."""
    rng = np.random.default_rng(23)
    chunks = [300, 212, 128, 1, 391]           # ends: inside a tile, 512 (page edge), 640, 641, 1032
    total = sum(chunks)
    pages = (total + 63) // 64
    num_pages = pages + 4
    cache = yahkv.KvCache(n_layers=2, num_pages=num_pages, fmt=yahkv.FMT_KV8A16, max_seqs=2, max_pages_per_seq=pages,
                          max_batch_tokens=512, max_prefill_keys=pages * 64)
    pool = O.Kv8Pool(num_pages)
    table = rng.permutation(num_pages)[:pages].astype(np.int32)
    m = (0.5 * rng.standard_normal((4, 256))).astype(np.float32)
    seq = cache.seq_create()
    cache.seq_set_table(seq, table)
    cache.seq_set_kmean(seq, m)
    open_tile, mean = pool.new_sequence(m)
    K = (rng.standard_normal((total, 4, 256)) + m).astype(np.float16)
    V = rng.standard_normal((total, 4, 256)).astype(np.float16)
    start = 0
    for c in chunks:
        q = (0.5 * rng.standard_normal((c, 24, 256))).astype(np.float16)
        gate = rng.standard_normal((c, 24, 256)).astype(np.float32)
        cache.append(1, np.full(c, seq, np.int32), np.arange(start, start + c, dtype=np.int64), dev(K[start:start + c]),
                     dev(V[start:start + c]))
        pool.append(table, start, K[start:start + c], V[start:start + c], open_tile, mean)
        out = torch.full((c, 24, 256), float("nan"), device="cuda")
        cache.attend_prefill(1, [seq], [c], dev(q), out, gate=dev(gate), out_dtype=yahkv.OUT_F32)
        cache.sync()
        got = out.cpu().numpy().astype(np.float64)
        assert np.isfinite(got).all()
        rows = sorted({0, c - 1, c // 2, min(c - 1, 127), min(c - 1, 128)})
        for r in rows:
            want = pool.attend_prefill_f64(table, start, q, open_tile, r, r + 1, gate)[0]
            err = np.abs(got[r] - want).max()
            assert err <= 2e-3 and err <= 1e-3 * np.abs(want).max(), (start, c, r, err, np.abs(want).max())
        start += c
    assert_pools(cache, 1, pool)
    # decode continues from the prefilled cache
    k1 = rng.standard_normal((1, 4, 256)).astype(np.float16)
    v1 = rng.standard_normal((1, 4, 256)).astype(np.float16)
    q1 = (0.5 * rng.standard_normal((1, 24, 256))).astype(np.float16)
    cache.append(1, [seq], [start], dev(k1), dev(v1))
    pool.append(table, start, k1, v1, open_tile, mean)
    got = run_decode(cache, 1, [seq], q1)[0]
    want = pool.attend_decode_f64(table, start + 1, q1[0], open_tile)
    err = np.abs(got - want).max()
    assert err <= 2e-3 and err / np.abs(want).max() < 1e-4, err
    cache.close()



@pytest.mark.parametrize("fmt", [yahkv.FMT_KV8A16, yahkv.FMT_KV4A16])
def test_fused_rope_append_is_rope_then_append(fmt):
    """yahkv_rope_append on the tile formats == the oracle's RMSNorm + RoPE (rounded to fp16) followed by the format's
    own append, bit for bit: q_out halves, pool codes, pairs, the open tile. Two sequences, a chunk then single tokens."""
    rng = np.random.default_rng(13)
    num_pages, eps = 12, 1e-6
    Pool = O.Kv8Pool if fmt == yahkv.FMT_KV8A16 else O.Kv4Pool
    cache = yahkv.KvCache(n_layers=2, num_pages=num_pages, fmt=fmt, max_seqs=2, max_pages_per_seq=5, max_batch_tokens=512)
    pool = Pool(num_pages)
    qw = (1.0 + 0.2 * rng.standard_normal(256)).astype(np.float32)
    kw = (1.0 + 0.2 * rng.standard_normal(256)).astype(np.float32)
    seqs = [cache.seq_create(), cache.seq_create()]
    states = []
    for s in seqs:
        cache.seq_reserve(s, 300)
        m = (0.5 * rng.standard_normal((4, 256))).astype(np.float32)
        cache.seq_set_kmean(s, m)
        states.append(pool.new_sequence(m))
    calls = [(np.array([seqs[0]] * 130 + [seqs[1]] * 77, np.int32), np.concatenate([np.arange(130), np.arange(77)]))]
    calls += [(np.array(seqs, np.int32), np.array([130 + i, 77 + i])) for i in range(5)]
    for ids, pos in calls:
        n = len(ids)
        q = (rng.standard_normal((n, 24, 256)) * 2).astype(np.float32)
        k = (rng.standard_normal((n, 4, 256)) * 3).astype(np.float32)
        v = rng.standard_normal((n, 4, 256)).astype(np.float32)
        q_out = torch.zeros((n, 24, 256), dtype=torch.float16, device="cuda")
        torch.cuda.synchronize()
        cache.rope_append(1, ids, pos, dev(q), dev(k), dev(v), dev(qw), dev(kw), eps, q_out)
        cache.sync()
        want_q = O.rope_rows(q, qw, eps, np.repeat(pos, 24))
        assert np.array_equal(q_out.cpu().numpy().view(np.uint16).reshape(-1, 256), want_q.view(np.uint16))
        k16 = O.rope_rows(k, kw, eps, np.repeat(pos, 4)).reshape(n, 4, 256)
        v16 = v.astype(np.float16)
        for s, st in zip(seqs, states):
            sel = ids == s
            pool.append(cache.seq_table(s), int(pos[sel][0]), k16[sel], v16[sel], *st)
    assert_pools(cache, 1, pool)
    for s, st, n in zip(seqs, states, (135, 82)):
        used = n - 16 * ((n - 1) // 16)
        assert np.array_equal(cache.read_open_tile(s, 1).view(np.uint16)[:, :, :used], st[0][:, :, :used])
        assert cache.seq_len(s, 1) == n
    cache.close()
