"""The CPU restatement of the reference's kv4a16 format against golden vectors made with the reference's own numpy
models (tests/golden/make_golden_kv4a16.py). The V side is bit for bit. The K side rotates in f32 (as the reference's
kernel does) where the model rotates in float64, so a code may sit one level off where a rotated value lands on a
rounding boundary: the bar is the reference checker's own, dequantized values within 1e-2
(engine/gpu/loom/tools/dattn_q_check.py:231-236), plus: at most a level apart, and rarely. The attention model is
pinned exactly by handing it the MODEL's codes."""
import hashlib
import os

import numpy as np
import pytest

import oracle as O
from recipes import kv8a16_recipe

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def g4():
    return np.load(os.path.join(ROOT, "tests", "golden", "kv4a16.npz"))


def sha(a):
    return hashlib.sha256(np.ascontiguousarray(a).tobytes()).hexdigest()


def nibbles(kq_row):
    """[128] u32 -> the 1024 codes of a token in dim order (dim 2j of a dword's 8 at bits 4j, 2j + 1 at 16 + 4j)."""
    out = np.zeros((128, 8), np.int32)
    for i in range(8):
        out[:, i] = (kq_row >> (4 * (i // 2) + (16 if i % 2 else 0))) & 15
    return out.reshape(-1)


def test_k_quantizer_within_the_checkers_bar_and_v_bit_for_bit(g4):
    r = kv8a16_recipe()
    T, mean = r["T"], r["m"].reshape(4, 256)
    off, worst, worst_s = 0, 0.0, 0.0
    for p in range(T):
        codes, scales = O.kv4_quant_k(r["K"][p].reshape(4, 256), mean)
        kq = codes.reshape(-1).view(np.uint32)                       # a head's 128 bytes are its 32 dwords
        d = np.abs(nibbles(kq) - nibbles(g4["kq"][p]))
        assert d.max() <= 1
        off += int(d.sum())
        want = O.kv4_deq_k(g4["kq"][p].view(np.uint8).reshape(4, 128), g4["ks"][p].view(np.uint16).reshape(4, 8, 2))
        worst = max(worst, float(np.abs(O.kv4_deq_k(codes, scales) - want).max()))
        worst_s = max(worst_s, float(np.abs(scales.reshape(-1).view(np.float16).astype(np.float32) - g4["ks"][p].astype(np.float32)).max()))
    assert worst < 1e-2, worst                       # the checker's bar (typical step of a group: 0.4)
    assert off <= T * 1024 // 2000, off              # a code in a few thousand at most
    assert worst_s <= 2e-3, worst_s                  # an f16 ulp of a pair value where lo or hi moved by an f32 ulp
    # the decoder itself, on the model's codes, is exact
    kd = np.stack([O.kv4_deq_k(g4["kq"][p].view(np.uint8).reshape(4, 128), g4["ks"][p].view(np.uint16).reshape(4, 8, 2)).reshape(-1)
                   for p in range(T)])
    assert sha(kd) == str(g4["kd_sha"])
    tiles = T // 16
    vq, vs = np.zeros((tiles, 1024, 2), np.uint32), np.zeros((tiles, 1024, 2), np.float16)
    vd = np.zeros((T, 1024), np.float32)
    for t in range(tiles):
        codes, stats = O.kv4_quant_vtile(r["V"][16 * t:16 * t + 16].reshape(16, 4, 256))
        vq[t] = codes.reshape(1024, 8).view(np.uint32)
        vs[t] = stats.reshape(1024, 2).view(np.float16)
        vd[16 * t:16 * t + 16] = O.kv4_deq_vtile(codes, stats).reshape(16, 1024)
    assert np.array_equal(vq[:2], g4["vq_head"]) and np.array_equal(vs[:2].view(np.uint16), g4["vs_head"].view(np.uint16))
    assert sha(vq) == str(g4["vq_sha"]) and sha(vs) == str(g4["vs_sha"]) and sha(vd) == str(g4["vd_sha"])


def test_hadamard_is_the_reference_matrix_and_self_inverse():
    i = np.arange(256)
    H = np.where(np.array([[bin(a & b).count("1") % 2 for b in i] for a in i]), -1.0, 1.0)   # dattn_q_check.py:50-55
    x = np.random.default_rng(0).standard_normal((3, 256))
    assert np.abs(O.hadamard256_f64(x) - x @ H.T / 16.0).max() < 1e-12
    assert np.abs(O.hadamard256_f64(O.hadamard256_f64(x)) - x).max() < 1e-12


def test_paged_append_and_attention_with_an_open_tile(g4):
    r = kv8a16_recipe()
    n = int(g4["n_keys"])
    rng = np.random.default_rng(3)
    num_pages = 7
    table = rng.permutation(num_pages)[:5].astype(np.int32)
    pool = O.Kv4Pool(num_pages)
    open_tile, mean = pool.new_sequence(r["m"])
    K, V = r["K"].reshape(-1, 4, 256), r["V"].reshape(-1, 4, 256)
    pool.append(table, 0, K[:100], V[:100], open_tile, mean)          # a chunk that ends inside a tile
    for p in range(100, 130):                                          # single tokens across tile boundaries
        pool.append(table, p, K[p:p + 1], V[p:p + 1], open_tile, mean)
    pool.append(table, 130, K[130:n], V[130:n], open_tile, mean)
    codes, stats = O.kv4_quant_vtile(V[16 * 9:16 * 10])
    assert np.array_equal(pool.vcodes[table[9 // 4], :, 9 % 4], codes) and np.array_equal(pool.vstats[table[9 // 4], :, 9 % 4], stats)
    kc, ks = O.kv4_quant_k(K[77], mean)
    assert np.array_equal(pool.kcodes[table[1], :, 77 - 64], kc) and np.array_equal(pool.kscales[table[1], :, 77 - 64], ks)
    assert np.array_equal(open_tile.view(np.float16)[:, :, :n - 288], V[288:n].transpose(1, 2, 0))   # keys 288 .. 299
    # with our own K codes the answer is the model's to within what a few one-level differences move it
    for name, gate in (("gated", r["gate"]), ("plain", None)):
        got = pool.attend_decode_f64(table, n, r["q"], open_tile, gate)
        assert np.abs(got - g4[f"attn_{name}"]).max() < 2e-4 * np.abs(g4[f"attn_{name}"]).max() + 1e-5, name
    # with the MODEL's K codes in the pool it is the model's exactly
    for p in range(n):
        pool.kcodes[table[p // 64], :, p % 64] = g4["kq"][p].view(np.uint8).reshape(4, 128)
        pool.kscales[table[p // 64], :, p % 64] = g4["ks"][p].view(np.uint16).reshape(4, 8, 2)
    for name, gate in (("gated", r["gate"]), ("plain", None)):
        got = pool.attend_decode_f64(table, n, r["q"], open_tile, gate)
        assert np.abs(got - g4[f"attn_{name}"]).max() < 1e-12, name
        # the prefill model's last row is the decode model's answer
        pre = pool.attend_prefill_f64(table, n - 1, r["q"][None], open_tile, gate=None if gate is None else gate[None])[0]
        assert np.abs(pre - got).max() < 1e-12
