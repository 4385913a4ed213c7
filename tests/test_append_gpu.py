"""KV append on the GPU against the oracle and the reference's codecs: quantized bytes, fp16 scales and page placement
must be bit-exact (the reference's own append checks are byte-exact too: dattn_check.py:108-109, dattn_q_check.py:223-225)."""
import numpy as np
import pytest
import torch

import oracle as O
import yahkv
from gpu_util import assert_pools_equal, dev, fill_both
from recipes import codec_input, outlier_kv

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("fmt", [yahkv.FMT_Q8_0, yahkv.FMT_Q4_0])
def test_single_token_appends_fill_a_shuffled_table(fmt):
    # The parity fixture in small: one sequence, tokens appended one call at a time through a permuted table,
    # K/V ~ N(0,1) with four x20 outlier channels per head.
    n, num_pages = 300, 8
    K, V, rng = outlier_kv(n, seed=0)
    table = rng.permutation(num_pages)[:5].astype(np.int32)
    cache = yahkv.KvCache(n_layers=2, num_pages=num_pages, fmt=fmt, max_seqs=2, max_pages_per_seq=8)
    seq = cache.seq_create()
    cache.seq_set_table(seq, table)
    Kd, Vd = dev(K), dev(V)
    for p in range(n):
        cache.append(1, [seq], [p], Kd[p:p + 1], Vd[p:p + 1])
    cache.sync()
    pool = O.PagedPool(fmt, num_pages)
    pool.append(table, 0, K, V)
    assert_pools_equal(cache, 1, pool)
    assert_pools_equal(cache, 0, O.PagedPool(fmt, num_pages))      # the other layer is untouched
    for p in (0, 63, 64, 299):
        kb, vb = cache.export_token(1, seq, p)
        assert np.array_equal(kb, O.quantize(K[p].astype(np.float32), fmt))
        assert np.array_equal(vb, O.quantize(V[p].astype(np.float32), fmt))
    if fmt == yahkv.FMT_Q8_0 and O.have_ref():
        kb, _ = cache.export_token(1, seq, 137)
        assert np.array_equal(kb, O.ref_quantize_q8_0(K[137].astype(np.float32)))   # the reference's QuantizeQ8_0 itself
    assert cache.seq_len(seq, 1) == n and cache.seq_len(seq, 0) == 0


@pytest.mark.parametrize("name,fmt", [("q8_0", yahkv.FMT_Q8_0), ("q4_0", yahkv.FMT_Q4_0)])
def test_codec_known_answers(golden, name, fmt):
    # The codec golden vector (all-zero block, constant block, sign-mirrored ties, outliers) pushed through append.
    x = codec_input().reshape(-1, 4, 256).astype(np.float16)     # 128 tokens
    n = x.shape[0]
    cache = yahkv.KvCache(num_pages=2, fmt=fmt, max_seqs=1, max_pages_per_seq=2)
    seq = cache.seq_create()
    cache.seq_set_table(seq, [1, 0])
    cache.append(0, np.zeros(n, np.int32), np.arange(n), dev(x), dev(x[::-1].copy()))
    blocks = np.concatenate([cache.export_token(0, seq, p)[0] for p in range(n)])
    head = golden[f"codec_{name}_head"]
    assert np.array_equal(blocks[: head.size], head)
    import hashlib
    assert hashlib.sha256(blocks.tobytes()).hexdigest() == str(golden[f"codec_{name}_sha256"])
    vblocks = np.concatenate([cache.export_token(0, seq, p)[1] for p in range(n)])
    assert np.array_equal(vblocks, O.quantize(x[::-1].astype(np.float32), fmt))


@pytest.mark.parametrize("fmt", [yahkv.FMT_Q8_0, yahkv.FMT_Q4_0])
def test_batched_ragged_appends(fmt):
    rng = np.random.default_rng(7)
    num_pages = 40
    cache = yahkv.KvCache(n_layers=1, num_pages=num_pages, fmt=fmt, max_seqs=5, max_pages_per_seq=12)
    pool = O.PagedPool(fmt, num_pages)
    lens = [1, 64, 65, 200, 130]
    seqs = [cache.seq_create() for _ in lens]
    data = []
    for s, n in zip(seqs, lens):
        cache.seq_reserve(s, n + 3)
        K = (rng.standard_normal((n + 3, 4, 256)) * rng.choice([0.02, 1, 15], (n + 3, 4, 1))).astype(np.float16)
        V = rng.standard_normal((n + 3, 4, 256)).astype(np.float16)
        data.append((K, V))
    # a prefill-style call mixing all sequences, tokens interleaved
    ids, pos, ks, vs = [], [], [], []
    for t in range(max(lens)):
        for i, n in enumerate(lens):
            if t < n:
                ids.append(seqs[i]); pos.append(t); ks.append(data[i][0][t]); vs.append(data[i][1][t])
    cache.append(0, ids, pos, dev(np.stack(ks)), dev(np.stack(vs)))
    # then three decode-style steps, one token per sequence
    for step in range(3):
        cache.append(0, seqs, [n + step for n in lens], dev(np.stack([data[i][0][lens[i] + step] for i in range(5)])),
                     dev(np.stack([data[i][1][lens[i] + step] for i in range(5)])))
    cache.sync()
    for i, s in enumerate(seqs):
        pool.append(cache.seq_table(s), 0, data[i][0], data[i][1])
        assert cache.seq_len(s, 0) == lens[i] + 3
    assert_pools_equal(cache, 0, pool)


def test_slot_mapping_variant_and_padding_tokens():
    rng = np.random.default_rng(9)
    cache = yahkv.KvCache(num_pages=4, max_seqs=1, max_pages_per_seq=4)
    pool = O.PagedPool(yahkv.FMT_Q8_0, 4)
    K = rng.standard_normal((6, 4, 256)).astype(np.float16)
    V = rng.standard_normal((6, 4, 256)).astype(np.float16)
    slots = np.array([3 * 64 + 5, -1, 0, 2 * 64 + 63, -1, 64], np.int64)
    cache.append_slots(0, 6, dev(slots), dev(K), dev(V))
    cache.sync()
    pool.append_slots(slots, K, V)
    assert_pools_equal(cache, 0, pool)


def test_order_and_range_errors_launch_nothing():
    cache = yahkv.KvCache(num_pages=4, max_seqs=2, max_pages_per_seq=2)
    s = cache.seq_create()
    cache.seq_reserve(s, 64)
    x = torch.zeros(2, 4, 256, dtype=torch.float16, device="cuda")
    before = cache.launch_count()
    for ids, pos, code in (([s], [1], yahkv.ERR_ORDER), ([s, s], [0, 2], yahkv.ERR_ORDER), ([1], [0], yahkv.ERR_INVALID)):
        with pytest.raises(yahkv.YahkvError) as e:
            cache.append(0, ids, pos, x, x)
        assert e.value.code == code
    with pytest.raises(yahkv.YahkvError) as e:
        cache.append(0, [s] * 2, [0, 1], None, x)
    assert cache.launch_count() == before
    cache.append(0, [s] * 2, [0, 1], x, x)
    cache.seq_set_len(s, 64)
    with pytest.raises(yahkv.YahkvError) as e:
        cache.append(0, [s], [64], x, x)      # past the reserved pages
    assert e.value.code == yahkv.ERR_INVALID
    assert cache.launch_count() == before + 1


@pytest.mark.parametrize("fmt", [yahkv.FMT_Q8_0, yahkv.FMT_Q4_0])
def test_fused_rope_append_is_rope_then_append(fmt):
    """yahkv_rope_append == the oracle's RMSNorm + RoPE (rounded to fp16) followed by the plain append, bit for bit:
    q_out halves, pool codes, scales and placement. Two sequences, a chunk then single tokens, positions up to 4999."""
    rng = np.random.default_rng(11)
    num_pages, eps = 96, 1e-6
    cache = yahkv.KvCache(n_layers=2, num_pages=num_pages, fmt=fmt, max_seqs=2, max_pages_per_seq=80, max_batch_tokens=512)
    pool = O.PagedPool(fmt, num_pages)
    qw = (1.0 + 0.2 * rng.standard_normal(256)).astype(np.float32)
    kw = (1.0 + 0.2 * rng.standard_normal(256)).astype(np.float32)
    seqs = [cache.seq_create(), cache.seq_create()]
    starts = [0, 4700]
    for s, n0 in zip(seqs, starts):
        cache.seq_reserve(s, n0 + 300)
        cache.seq_set_len(s, n0)          # earlier positions stand in as already cached
    calls = [(np.array([seqs[0]] * 130 + [seqs[1]] * 129, np.int32),
              np.concatenate([np.arange(130), 4700 + np.arange(129)]))]
    calls += [(np.array(seqs, np.int32), np.array([130 + i, 4829 + i])) for i in range(3)]
    for ids, pos in calls:
        n = len(ids)
        q = (rng.standard_normal((n, 24, 256)) * 2).astype(np.float32)
        k = (rng.standard_normal((n, 4, 256)) * 3).astype(np.float32)
        k[:, :, 5] *= 20.0                                             # an outlier channel inside the rotated dims
        v = rng.standard_normal((n, 4, 256)).astype(np.float32)
        q_out = torch.zeros((n, 24, 256), dtype=torch.float16, device="cuda")
        torch.cuda.synchronize()
        cache.rope_append(1, ids, pos, dev(q), dev(k), dev(v), dev(qw), dev(kw), eps, q_out)
        cache.sync()
        want_q = O.rope_rows(q, qw, eps, np.repeat(pos, 24))
        assert np.array_equal(q_out.cpu().numpy().view(np.uint16).reshape(-1, 256), want_q.view(np.uint16))
        k16 = O.rope_rows(k, kw, eps, np.repeat(pos, 4)).reshape(n, 4, 256)
        v16 = v.astype(np.float16)
        for s in seqs:
            m = ids == s
            pool.append(cache.seq_table(s), int(pos[m][0]), k16[m], v16[m])
    assert_pools_equal(cache, 1, pool)
    assert [cache.seq_len(s, 1) for s in seqs] == [133, 4832]
    cache.close()


def test_empty_calls_are_accepted_and_launch_nothing():
    """Zero tokens / zero sequences: every hot call returns success without a launch (the engine queues whatever a
    scheduling step produced, which may be nothing)."""
    cache = yahkv.KvCache(n_layers=1, num_pages=4, fmt=yahkv.FMT_Q8_0, max_seqs=2, max_pages_per_seq=2)
    s = cache.seq_create()
    cache.seq_reserve(s, 10)
    x = torch.zeros((1, 24, 256), dtype=torch.float16, device="cuda")
    xf = torch.zeros((1, 24, 256), dtype=torch.float32, device="cuda")
    empty_i32, empty_i64 = np.zeros(0, np.int32), np.zeros(0, np.int64)
    before = cache.launch_count()
    cache.append(0, empty_i32, empty_i64, x, x)
    cache.rope_append(0, empty_i32, empty_i64, xf, xf, xf, xf, xf, 1e-6, x)
    cache.append_slots(0, 0, torch.zeros(1, dtype=torch.int64, device="cuda"), x, x)
    cache.attend_decode(0, empty_i32, x, x)
    cache.attend_prefill(0, empty_i32, empty_i32, x, x)
    cache.sync()
    assert cache.launch_count() == before and cache.seq_len(s, 0) == 0
    # and a sequence with no keys yet cannot be attended
    with pytest.raises(yahkv.YahkvError) as e:
        cache.attend_decode(0, [s], x, x)
    assert e.value.code == yahkv.ERR_ORDER
    cache.close()
