"""The reference's 4-bit cache format kv4a16 on the GPU (YAHKV_FMT_KV4A16): appends byte-exact against the CPU
restatement (tests/test_kv4a16_oracle_cpu.py pins that one to the reference's numpy models: V bit for bit, K under the
reference checker's own bar, the f32 rotation being the kernel's and not the model's float64 one); decode attention
against the float64 model over the cache's own bytes to the checker's bar, max|err| / max|ref| < 1e-4
(engine/gpu/loom/tools/dattn_q_check.py:205-208); prefill attention with fp16 operands to 2e-3 / 1e-3. Pages hold 64
tokens = four 16-key tiles here (256 tokens in the reference)."""
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
    g4 = np.load(os.path.join(ROOT, "tests", "golden", "kv4a16.npz"))
    r = kv8a16_recipe()
    n = int(g4["n_keys"])
    rng = np.random.default_rng(3)
    num_pages = 7
    table = rng.permutation(num_pages)[:5].astype(np.int32)
    cache = yahkv.KvCache(n_layers=2, num_pages=num_pages, fmt=yahkv.FMT_KV4A16, max_seqs=2, max_pages_per_seq=5)
    pool = O.Kv4Pool(num_pages)
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
    assert_pools(cache, 0, O.Kv4Pool(num_pages))        # the other layer is untouched
    got_open = cache.read_open_tile(seq, 1)
    used = n - 16 * ((n - 1) // 16)
    assert np.array_equal(got_open.view(np.uint16)[:, :, :used], open_tile[:, :, :used])
    # the reference's own arrays: the first two V tiles as its numpy model made them, and its K rows where they agree
    kc, ks, vc, vs = read_pools(cache, 1, num_pages)
    for t in range(2):
        want_c = g4["vq_head"][t].view(np.uint8).reshape(4, 256, 8)
        want_s = g4["vs_head"][t].view(np.uint16).reshape(4, 256, 2)
        assert np.array_equal(vc[table[0], :, t], want_c) and np.array_equal(vs[table[0], :, t], want_s)
    same = sum(np.array_equal(kc[table[p // 64], :, p % 64].reshape(-1), g4["kq"][p].view(np.uint8)) for p in range(n))
    assert same >= n - 3, same           # a code may sit one level off the float64 model's on a rounding boundary
    for name, gate in (("gated", r["gate"]), ("plain", None)):
        want = pool.attend_decode_f64(table, n, r["q"], open_tile, gate)
        for n_splits in (0, 1, 3):
            got = run_decode(cache, 1, [seq], r["q"][None], None if gate is None else gate[None], n_splits)[0]
            err = np.abs(got - want).max()
            assert err <= 2e-3 and err / np.abs(want).max() < 1e-4, (name, n_splits, err, err / np.abs(want).max())
        if same == n:                    # then the reference model's own answer applies too
            assert np.abs(got - g4[f"attn_{name}"]).max() / np.abs(want).max() < 1e-4
    cache.close()


def test_ragged_batch_with_means_and_decode_steps():
    rng = np.random.default_rng(11)
    lens = [1, 15, 16, 17, 64, 100, 1000, 2049]
    pages = [(n + 8 + 63) // 64 for n in lens]
    num_pages = sum(pages) + 3
    cache = yahkv.KvCache(n_layers=1, num_pages=num_pages, fmt=yahkv.FMT_KV4A16, max_seqs=len(lens),
                          max_pages_per_seq=max(pages), max_batch_tokens=4096)
    pool = O.Kv4Pool(num_pages)
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
        V[:, :, ::41] *= 9.0             # outlier channels
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
    x = torch.zeros(4, 24, 256, dtype=torch.float16, device="cuda")
    for call in (lambda: cache.export_token(0, seqs[0], 0),
                 lambda: cache.seq_set_len(seqs[0], 1), lambda: cache.seq_set_kmean(seqs[0], np.zeros((4, 256), np.float32))):
        with pytest.raises(yahkv.YahkvError):
            call()
    del x
    cache.close()


def test_chunked_prefill_attention():
    rng = np.random.default_rng(29)
    chunks = [300, 212, 128, 1, 391]           # ends: inside a tile, 512 (page edge), 640, 641, 1032
    total = sum(chunks)
    pages = (total + 63) // 64
    num_pages = pages + 4
    cache = yahkv.KvCache(n_layers=2, num_pages=num_pages, fmt=yahkv.FMT_KV4A16, max_seqs=2, max_pages_per_seq=pages,
                          max_batch_tokens=512, max_prefill_keys=pages * 64)
    pool = O.Kv4Pool(num_pages)
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
        for r in sorted({0, c - 1, c // 2, min(c - 1, 127), min(c - 1, 128)}):
            want = pool.attend_prefill_f64(table, start, q, open_tile, r, r + 1, gate)[0]
            err = np.abs(got[r] - want).max()
            assert err <= 2e-3 and err <= 1e-3 * np.abs(want).max(), (start, c, r, err, np.abs(want).max())
        start += c
    assert_pools(cache, 1, pool)
    cache.close()
