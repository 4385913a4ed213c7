"""The CPU restatement of the reference's kv8a16 cache format (oracle/kv8a16_oracle.cpp) against golden vectors made
with the reference's own numpy models (tests/golden/make_golden_kv8a16.py): K code dwords and scale pairs per token, V
code dwords and statistic pairs per 16-key tile, the dequantized values, all bit for bit; decode attention with an
open fp16 tile to 1e-12."""
import hashlib
import os

import numpy as np
import pytest

import oracle as O
from recipes import kv8a16_recipe

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def g8():
    return np.load(os.path.join(ROOT, "tests", "golden", "kv8a16.npz"))


def sha(a):
    return hashlib.sha256(np.ascontiguousarray(a).tobytes()).hexdigest()


def reference_layout_k(r):
    """Our per-token quantizer output in the reference's array layouts: kq [T][256] u32, ks [T][16] f16, K - m f32."""
    T = r["T"]
    kq, ks, kd = np.zeros((T, 256), np.uint32), np.zeros((T, 16), np.float16), np.zeros((T, 1024), np.float32)
    mean = r["m"].reshape(4, 256)
    for p in range(T):
        codes, scales = O.kv8_quant_k(r["K"][p].reshape(4, 256), mean)
        kq[p] = codes.reshape(-1).view(np.uint32)        # a head's 256 bytes are its 64 dwords, heads in order
        ks[p] = scales.reshape(-1).view(np.float16)
        kd[p] = O.kv8_deq_k(codes, scales).reshape(-1)
    return kq, ks, kd


def reference_layout_v(r):
    T = r["T"]
    tiles = T // 16
    vq, vs = np.zeros((tiles, 1024, 4), np.uint32), np.zeros((tiles, 1024, 2), np.float16)
    vd = np.zeros((T, 1024), np.float32)
    for t in range(tiles):
        codes, stats = O.kv8_quant_vtile(r["V"][16 * t:16 * t + 16].reshape(16, 4, 256))
        vq[t] = codes.reshape(1024, 16).view(np.uint32)
        vs[t] = stats.reshape(1024, 2).view(np.float16)
        vd[16 * t:16 * t + 16] = O.kv8_deq_vtile(codes, stats).reshape(16, 1024)
    return vq, vs, vd


def test_quantizers_and_decoders_match_the_reference_models_bit_for_bit(g8):
    r = kv8a16_recipe()
    kq, ks, kd = reference_layout_k(r)
    assert np.array_equal(kq[:32], g8["kq_head"]) and np.array_equal(ks[:32].view(np.uint16), g8["ks_head"].view(np.uint16))
    assert sha(kq) == str(g8["kq_sha"]) and sha(ks) == str(g8["ks_sha"]) and sha(kd) == str(g8["kd_sha"])
    vq, vs, vd = reference_layout_v(r)
    assert np.array_equal(vq[:2], g8["vq_head"]) and np.array_equal(vs[:2].view(np.uint16), g8["vs_head"].view(np.uint16))
    assert sha(vq) == str(g8["vq_sha"]) and sha(vs) == str(g8["vs_sha"]) and sha(vd) == str(g8["vd_sha"])


def test_paged_append_and_attention_with_an_open_tile(g8):
    r = kv8a16_recipe()
    n = int(g8["n_keys"])
    rng = np.random.default_rng(3)
    num_pages = 7
    table = rng.permutation(num_pages)[:5].astype(np.int32)
    pool = O.Kv8Pool(num_pages)
    open_tile, mean = pool.new_sequence(r["m"])
    K, V = r["K"].reshape(-1, 4, 256), r["V"].reshape(-1, 4, 256)
    pool.append(table, 0, K[:100], V[:100], open_tile, mean)          # a chunk that ends inside a tile
    for p in range(100, 130):                                          # single tokens across tile boundaries
        pool.append(table, p, K[p:p + 1], V[p:p + 1], open_tile, mean)
    pool.append(table, 130, K[130:n], V[130:n], open_tile, mean)
    # placement: tile t of the sequence sits in page table[t // 4], slot t % 4; token p in page table[p // 64]
    codes, stats = O.kv8_quant_vtile(V[16 * 9:16 * 10])
    assert np.array_equal(pool.vcodes[table[9 // 4], :, 9 % 4], codes) and np.array_equal(pool.vstats[table[9 // 4], :, 9 % 4], stats)
    kc, ks = O.kv8_quant_k(K[77], mean)
    assert np.array_equal(pool.kcodes[table[1], :, 77 - 64], kc) and np.array_equal(pool.kscales[table[1], :, 77 - 64], ks)
    assert np.array_equal(open_tile.view(np.float16)[:, :, :n - 288], V[288:n].transpose(1, 2, 0))   # keys 288 .. 299
    for name, gate in (("gated", r["gate"]), ("plain", None)):
        got = pool.attend_decode_f64(table, n, r["q"], open_tile, gate)
        assert np.abs(got - g8[f"attn_{name}"]).max() < 1e-12, name
    # the prefill model (numpy over the same dequantizers): its last row is the decode model's answer, and an earlier
    # row sees only the keys up to its own position
    for gate in (r["gate"], None):
        want = pool.attend_decode_f64(table, n, r["q"], open_tile, gate)
        got = pool.attend_prefill_f64(table, n - 1, r["q"][None], open_tile, gate=None if gate is None else gate[None])[0]
        assert np.abs(got - want).max() < 1e-12
    q2 = np.stack([r["q"], r["q"]])
    two = pool.attend_prefill_f64(table, n - 2, q2, open_tile)
    Kd, Vd = pool.dequantized(table, n, open_tile)
    s = (Kd[:n - 1, 0].astype(np.float64) @ q2[0, 0].astype(np.float64)) / 16.0
    w = np.exp(s - s.max())
    assert np.abs(two[0, 0] - (w @ Vd[:n - 1, 0].astype(np.float64)) / w.sum()).max() < 1e-12
