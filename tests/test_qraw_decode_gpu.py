"""yahkv_attend_decode_qraw (the attention kernel's prologue norms and rotates the raw f32 query rows: the attend-side
half of the reference's norm + RoPE fusion, engine/gpu/loom/yah_fused_qk_rope_f32.loom:1-9) for every cache format:
bit for bit the result of yahkv_rope_append's q output followed by yahkv_attend_decode, whose q bits are pinned to the
oracle's; and for q8_0 the float64 attention model on top."""
import numpy as np
import pytest
import torch

import oracle as O
import yahkv
from gpu_util import dev

pytestmark = pytest.mark.gpu
FORMATS = [yahkv.FMT_Q8_0, yahkv.FMT_Q4_0, yahkv.FMT_KV8A16, yahkv.FMT_KV4A16, yahkv.FMT_F16]


@pytest.mark.parametrize("fmt", FORMATS)
def test_raw_query_decode_is_rope_then_attend(fmt):
    rng = np.random.default_rng(300 + fmt)
    eps = 1e-6
    lens = [1, 64, 333, 1500]                 # keys per sequence after this step's append
    pages = [(n + 63) // 64 for n in lens]
    num_pages = sum(pages) + 2
    cache = yahkv.KvCache(n_layers=2, num_pages=num_pages, fmt=fmt, max_seqs=len(lens), max_pages_per_seq=max(pages),
                          max_batch_tokens=2048, max_splits=16)
    qw = (1.0 + 0.2 * rng.standard_normal(256)).astype(np.float32)
    kw = (1.0 + 0.2 * rng.standard_normal(256)).astype(np.float32)
    pool = O.PagedPool(yahkv.FMT_Q8_0, num_pages)   # followed for q8_0 only
    seqs = []
    for n in lens:
        s = cache.seq_create()
        cache.seq_reserve(s, n)
        if fmt in (yahkv.FMT_KV8A16, yahkv.FMT_KV4A16):
            cache.seq_set_kmean(s, (0.3 * rng.standard_normal((4, 256))).astype(np.float32))
        if n > 1:   # the context before this step, plain fp16 rows
            K = rng.standard_normal((n - 1, 4, 256)).astype(np.float16)
            V = rng.standard_normal((n - 1, 4, 256)).astype(np.float16)
            cache.append(1, np.full(n - 1, s, np.int32), np.arange(n - 1), dev(K), dev(V))
            if fmt == yahkv.FMT_Q8_0:
                pool.append(cache.seq_table(s), 0, K, V)
        seqs.append(s)
    b = len(seqs)
    pos = np.array([n - 1 for n in lens], np.int64)
    q = (rng.standard_normal((b, 24, 256)) * 2).astype(np.float32)
    k = rng.standard_normal((b, 4, 256)).astype(np.float32)
    v = rng.standard_normal((b, 4, 256)).astype(np.float32)
    gate = rng.standard_normal((b, 24, 256)).astype(np.float32)
    q_dev, qw_dev = dev(q), dev(qw)
    q_out = torch.zeros((b, 24, 256), dtype=torch.float16, device="cuda")
    torch.cuda.synchronize()
    cache.rope_append(1, seqs, pos, q_dev, dev(k), dev(v), qw_dev, dev(kw), eps, q_out)   # this step's token
    cache.sync()
    want_q = O.rope_rows(q, qw, eps, np.repeat(pos, 24)).reshape(b, 24, 256)
    assert np.array_equal(q_out.cpu().numpy().view(np.uint16), want_q.view(np.uint16))
    for n_splits, use_gate in ((0, False), (1, True), (5, False), (16, True)):
        two_step = torch.full((b, 24, 256), float("nan"), device="cuda")
        fused = torch.full((b, 24, 256), float("nan"), device="cuda")
        g = dev(gate) if use_gate else None
        torch.cuda.synchronize()
        cache.attend_decode(1, seqs, q_out, two_step, gate=g, out_dtype=yahkv.OUT_F32, n_splits=n_splits)
        cache.attend_decode_qraw(1, seqs, q_dev, qw_dev, eps, fused, gate=g, out_dtype=yahkv.OUT_F32, n_splits=n_splits)
        cache.sync()
        a, f = two_step.cpu().numpy(), fused.cpu().numpy()
        assert np.isfinite(f).all()
        assert np.array_equal(a.view(np.uint32), f.view(np.uint32)), (fmt, n_splits)
    if fmt == yahkv.FMT_Q8_0:   # and the float64 model over the oracle's own pool
        k16 = O.rope_rows(k, kw, eps, np.repeat(pos, 4)).reshape(b, 4, 256)
        v16 = v.astype(np.float16)
        for i, s in enumerate(seqs):
            pool.append(cache.seq_table(s), int(pos[i]), k16[i:i + 1], v16[i:i + 1])
            want = pool.attend_decode_f64(cache.seq_table(s), lens[i], want_q[i], gate[i])
            err = np.abs(f[i] - want).max()
            assert err <= 2e-3 and err < 1e-4 * np.abs(want).max()
    cache.close()
