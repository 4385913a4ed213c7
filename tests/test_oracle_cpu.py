"""The CPU oracle against the reference's own code and the committed golden vectors (no GPU)."""
import hashlib

import numpy as np
import pytest

import oracle as O
from recipes import checker_recipe, codec_input, outlier_kv


def sha(a):
    return hashlib.sha256(np.ascontiguousarray(a).tobytes()).hexdigest()


@pytest.mark.parametrize("name,fmt", [("q8_0", O.FMT_Q8_0), ("q4_0", O.FMT_Q4_0)])
def test_codec_matches_golden(golden, name, fmt):
    x = codec_input()
    blocks = O.quantize(x, fmt)
    assert sha(blocks) == str(golden[f"codec_{name}_sha256"])
    head = golden[f"codec_{name}_head"]
    assert np.array_equal(blocks[: head.size], head)
    deq = O.dequantize(blocks, fmt)
    assert sha(deq) == str(golden[f"codec_{name}_deq_sha256"])
    assert np.array_equal(deq[:2048], golden[f"codec_{name}_deq_head"])


@pytest.mark.skipif(not O.have_ref(), reason="oracle/_ref (the reference's compiled codecs) is not built")
def test_codec_matches_reference_build():
    rng = np.random.default_rng(11)
    x = (rng.standard_normal(32 * 50000) * rng.choice([0.01, 1.0, 30.0], 32 * 50000)).astype(np.float16).astype(np.float32)
    assert np.array_equal(O.quantize(x, O.FMT_Q8_0), O.ref_quantize_q8_0(x))
    for fmt in (O.FMT_Q8_0, O.FMT_Q4_0):
        raw = rng.integers(0, 256, 20000 * O.block_bytes(fmt), dtype=np.uint8).reshape(-1, O.block_bytes(fmt))
        raw[:, :2] = rng.uniform(0.001, 0.05, 20000).astype(np.float16).view(np.uint8).reshape(-1, 2)
        assert np.array_equal(O.dequantize(raw, fmt), O.ref_dequantize(raw, fmt))


def test_q4_0_quantizer_matches_gguf_package():
    gguf = pytest.importorskip("gguf")
    from gguf.quants import quantize
    rng = np.random.default_rng(12)
    x = (rng.standard_normal(32 * 100000) * rng.choice([0.05, 1.0, 20.0], 32 * 100000)).astype(np.float16).astype(np.float32)
    want = quantize(x.reshape(-1, 32), gguf.GGMLQuantizationType.Q4_0).reshape(-1)
    assert np.array_equal(O.quantize(x, O.FMT_Q4_0), want)


def test_q8_0_round_trip_within_half_a_step():
    # the reference's own check of QuantizeQ8_0 (engine/tests/gguf_check.py:70-83)
    rng = np.random.default_rng(13)
    x = rng.standard_normal(32 * 256).astype(np.float32) * 0.02
    x[rng.integers(0, x.size, 40)] *= 25
    back = O.dequantize(O.quantize(x, O.FMT_Q8_0), O.FMT_Q8_0)
    step = np.repeat(np.abs(x.reshape(-1, 32)).max(1) / 127, 32)
    assert np.all(np.abs(back - x) <= step * (0.5 + 1e-3) + np.abs(x) * 2.0 ** -10)


def test_slot_rule_and_clamps():
    table = np.array([5, 2, 7], np.int32)
    assert O.slot(table, 0, 8) == 5 * 64
    assert O.slot(table, 63, 8) == 5 * 64 + 63
    assert O.slot(table, 64, 8) == 2 * 64
    assert O.slot(table, 191, 8) == 7 * 64 + 63
    assert O.slot(table, -3, 8) == 5 * 64            # position clamped to 0
    assert O.slot(table, 10_000, 8) == 7 * 64 + 63   # position clamped to the table's span
    assert O.slot(np.array([9, -1], np.int32), 70, 8) == 0 * 64 + 6   # page id clamped into the pool
    assert O.slot(np.array([9, -1], np.int32), 3, 8) == 7 * 64 + 3
    assert O.validate_table(table, 8) == -1
    assert O.validate_table(np.array([0, 8], np.int32), 8) == 1
    assert O.validate_table(np.array([-1, 3], np.int32), 8) == 0


@pytest.mark.parametrize("fmt", [O.FMT_Q8_0, O.FMT_Q4_0])
def test_append_places_rows_and_leaves_the_rest(fmt):
    rng = np.random.default_rng(3)
    num_pages = 6
    table = rng.permutation(num_pages)[:4].astype(np.int32)
    K, V, _ = outlier_kv(130, seed=4)
    pool = O.PagedPool(fmt, num_pages)
    pool.append(table, 0, K[:70], V[:70])
    pool.append(table, 70, K[70:], V[70:])
    for pos in (0, 63, 64, 129):
        s = table[pos // 64] * 64 + pos % 64
        assert np.array_equal(pool.export_row(0, s), O.quantize(K[pos].astype(np.float32), fmt))
        assert np.array_equal(pool.export_row(1, s), O.quantize(V[pos].astype(np.float32), fmt))
    used = np.zeros(num_pages * 64, bool)
    for pos in range(130):
        used[table[pos // 64] * 64 + pos % 64] = True
    kc = pool.kcodes.transpose(0, 2, 1, 3).reshape(num_pages * 64, -1)
    assert not kc[~used].any() and kc[used].any(1).all()


@pytest.mark.parametrize("name,fmt", [("q8_0", O.FMT_Q8_0), ("q4_0", O.FMT_Q4_0)])
def test_decode_attention_matches_golden(golden, name, fmt):
    r = checker_recipe()
    pool = O.PagedPool(fmt, r["T"] // 64)
    pool.append(r["ptab"], 0, r["K"], r["V"])
    n = r["pos"] + 1
    # pool bytes equal the reference's blocks
    kb = np.concatenate([pool.export_row(0, r["ptab"][p // 64] * 64 + p % 64) for p in range(r["T"])])
    assert sha(kb) == str(golden[f"attn_{name}_kblocks_sha256"])
    for gate, key in ((r["gate"], "gated"), (None, "plain")):
        want = golden[f"attn_{name}_{key}"]
        got = pool.attend_decode_f64(r["ptab"], n, r["q"], gate)
        assert np.abs(got - want).max() <= 1e-12 * max(1.0, np.abs(want).max())
        got32 = pool.attend_decode_f32(r["ptab"][None, :], [n], r["q"][None], None if gate is None else gate[None])[0]
        # the reference's tolerance for its f32 kernels against this float64 model (dattn_q_check.py:205-208)
        assert np.abs(got32 - want).max() / np.abs(want).max() < 1e-4


def test_prefill_oracle_agrees_with_decode_oracle():
    rng = np.random.default_rng(21)
    K, V, _ = outlier_kv(200, seed=5)
    table = rng.permutation(8)[:4].astype(np.int32)
    pool = O.PagedPool(O.FMT_Q8_0, 8)
    pool.append(table, 0, K, V)
    q = rng.standard_normal((72, 24, 256)).astype(np.float16)
    gate = rng.standard_normal((72, 24, 256)).astype(np.float32)
    start = 200 - 72
    out = pool.attend_prefill_f64(table, start, q, gate=gate)
    for i in (0, 1, 35, 71):
        want = pool.attend_decode_f64(table, start + i + 1, q[i], gate[i])
        assert np.abs(out[i] - want).max() < 1e-12
    part = pool.attend_prefill_f64(table, start, q, q_begin=30, q_end=40, gate=gate)
    assert np.array_equal(part, out[30:40])


def test_rope_rows_follow_the_formula():
    # inv_rms = 1/sqrt(mean(x^2) + eps); normed = x * inv_rms * w; NeoX rotation of dims (p, p + 32), p < 32, by
    # pos / 1e7^(2p/64); dims 64.. pass through (yah_fused_qk_rope_f32.loom:4-6, :32). Result rounded to fp16.
    rng = np.random.default_rng(3)
    x = (rng.standard_normal((6, 256)) * 2).astype(np.float32)
    w = (1 + 0.1 * rng.standard_normal(256)).astype(np.float32)
    pos = np.array([0, 1, 63, 64, 4095, 131071], np.int32)
    got = O.rope_rows(x, w, 1e-6, pos).astype(np.float64)
    for i, p0 in enumerate(pos):
        xd, wd = x[i].astype(np.float64), w.astype(np.float64)
        n = xd / np.sqrt((xd ** 2).mean() + 1e-6) * wd
        ang = p0 / 1e7 ** (2 * np.arange(32) / 64)
        want = n.copy()
        want[:32] = n[:32] * np.cos(ang) - n[32:64] * np.sin(ang)
        want[32:64] = n[:32] * np.sin(ang) + n[32:64] * np.cos(ang)
        assert np.abs(got[i] - want).max() <= np.abs(want).max() * 2.0 ** -11 + 1e-6
