"""Device-resident decode batches (plan / decode_layer / advance from device-side lengths), eagerly and replayed from
a captured CUDA graph, against the ordinary host-planned calls on a twin cache with the same contents."""
import numpy as np
import pytest
import torch

import yahkv
from gpu_util import assert_pools_equal, dev, pool_pages

pytestmark = pytest.mark.gpu
LAYERS = 2


FORMATS = [yahkv.FMT_Q8_0, yahkv.FMT_KV8A16, yahkv.FMT_KV4A16, yahkv.FMT_F16]


def twin_caches(lens, seed, extra_tokens, fmt=yahkv.FMT_Q8_0, **config):
    rng = np.random.default_rng(seed)
    pages = [(n + extra_tokens + 63) // 64 for n in lens]
    num_pages = sum(pages) + 2
    caches = [yahkv.KvCache(n_layers=LAYERS, num_pages=num_pages, max_seqs=len(lens), max_pages_per_seq=max(pages), fmt=fmt,
                            **config)
              for _ in range(2)]
    perm = rng.permutation(num_pages).astype(np.int32)
    seqs, off = [], 0
    for i, n in enumerate(lens):
        K = rng.standard_normal((LAYERS, n, 4, 256)).astype(np.float16)
        V = rng.standard_normal((LAYERS, n, 4, 256)).astype(np.float16)
        for c in caches:
            s = c.seq_create()
            c.seq_set_table(s, perm[off:off + pages[i]])
            for layer in range(LAYERS):
                c.append(layer, np.full(n, s, np.int32), np.arange(n), dev(K[layer]), dev(V[layer]))
        seqs.append(s)
        off += pages[i]
    return caches[0], caches[1], seqs, num_pages, rng


def host_step(cache, seqs, lens, k, v, q, gate):
    outs = []
    for layer in range(LAYERS):
        cache.append(layer, seqs, lens, dev(k[layer]), dev(v[layer]))
        out = torch.zeros(len(seqs), 24, 256, device="cuda")
        torch.cuda.synchronize()
        cache.attend_decode(layer, seqs, dev(q[layer]), out, gate=dev(gate[layer]), out_dtype=yahkv.OUT_F32)
        cache.sync()
        outs.append(out.cpu().numpy())
    return outs


def step_inputs(rng, n):
    return (rng.standard_normal((LAYERS, n, 4, 256)).astype(np.float16),
            rng.standard_normal((LAYERS, n, 4, 256)).astype(np.float16),
            rng.standard_normal((LAYERS, n, 24, 256)).astype(np.float16),
            rng.standard_normal((LAYERS, n, 24, 256)).astype(np.float32))


@pytest.mark.parametrize("fmt", FORMATS)
def test_eager_batch_steps_match_host_planned_steps(fmt):
    # page boundaries, a unit boundary (24 pages) and, for the tile formats, 16-key tile boundaries get crossed
    lens = [5, 63, 64, 1535, 24 * 64 - 2, 700, 13]
    ref, cache, seqs, num_pages, rng = twin_caches(lens, 61, extra_tokens=8, fmt=fmt)
    batch = yahkv.DecodeBatch(cache, seqs)
    assert batch.prepare(6) is True
    cur = list(lens)
    for step in range(6):
        k, v, q, gate = step_inputs(rng, len(seqs))
        want = host_step(ref, seqs, cur, k, v, q, gate)
        batch.plan()
        for layer in range(LAYERS):
            out = torch.zeros(len(seqs), 24, 256, device="cuda")
            torch.cuda.synchronize()
            batch.decode_layer(layer, dev(k[layer]), dev(v[layer]), dev(q[layer]), out, gate=dev(gate[layer]),
                               out_dtype=yahkv.OUT_F32)
            cache.sync()
            assert np.abs(out.cpu().numpy() - want[layer]).max() <= 1e-4, (step, layer)
        batch.advance()
        batch.commit(1)
        cur = [n + 1 for n in cur]
        assert [cache.seq_len(s, 1) for s in seqs] == cur
    for layer in range(LAYERS):      # the appends landed in the same places with the same bytes
        a, b = pool_pages(ref, layer, num_pages), pool_pages(cache, layer, num_pages)
        assert all(np.array_equal(x, y) for x, y in zip(a, b))
    with pytest.raises(yahkv.YahkvError) as e:
        batch.commit(1)                  # nothing prepared beyond the six steps
    assert e.value.code == yahkv.ERR_ORDER
    assert batch.prepare(3) is False     # same unit layout: a captured graph stays valid
    batch.close()


@pytest.mark.parametrize("fmt", FORMATS)
def test_replayed_cuda_graph_matches_host_planned_steps(fmt):
    lens = [300, 64 * 24 - 3, 2000, 1, 30]
    ref, cache, seqs, num_pages, rng = twin_caches(lens, 62, extra_tokens=8, fmt=fmt)
    n = len(seqs)
    batch = yahkv.DecodeBatch(cache, seqs)
    batch.prepare(6)
    side = torch.cuda.Stream()
    k_s = torch.zeros(LAYERS, n, 4, 256, device="cuda", dtype=torch.float16)
    v_s = torch.zeros_like(k_s)
    q_s = torch.zeros(LAYERS, n, 24, 256, device="cuda", dtype=torch.float16)
    g_s = torch.zeros(LAYERS, n, 24, 256, device="cuda", dtype=torch.float32)
    o_s = torch.zeros(LAYERS, n, 24, 256, device="cuda", dtype=torch.float32)
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph, stream=side):
        sp = torch.cuda.current_stream().cuda_stream
        batch.plan(stream=sp)
        for layer in range(LAYERS):
            batch.decode_layer(layer, k_s[layer], v_s[layer], q_s[layer], o_s[layer], gate=g_s[layer],
                               out_dtype=yahkv.OUT_F32, stream=sp)
        batch.advance(stream=sp)
    cur = list(lens)
    for step in range(5):
        k, v, q, gate = step_inputs(rng, n)
        want = host_step(ref, seqs, cur, k, v, q, gate)
        k_s.copy_(torch.from_numpy(k)); v_s.copy_(torch.from_numpy(v))
        q_s.copy_(torch.from_numpy(q)); g_s.copy_(torch.from_numpy(gate))
        graph.replay()
        torch.cuda.synchronize()
        got = o_s.cpu().numpy()
        for layer in range(LAYERS):
            assert np.abs(got[layer] - want[layer]).max() <= 1e-4, (step, layer)
        cur = [x + 1 for x in cur]
    batch.commit(5)
    cache.sync()
    assert [cache.seq_len(s, 0) for s in seqs] == cur
    for layer in range(LAYERS):
        a, b = pool_pages(ref, layer, num_pages), pool_pages(cache, layer, num_pages)
        assert all(np.array_equal(x, y) for x, y in zip(a, b))
    # after the batch, the ordinary calls continue from the committed lengths
    k, v, q, gate = step_inputs(rng, n)
    want = host_step(ref, seqs, cur, k, v, q, gate)
    got = host_step(cache, seqs, cur, k, v, q, gate)
    assert all(np.abs(a - b).max() <= 1e-4 for a, b in zip(got, want))
    batch.close()


def test_batch_refuses_what_it_cannot_hold():
    cache = yahkv.KvCache(n_layers=2, num_pages=4, max_seqs=2, max_pages_per_seq=2)
    s = cache.seq_create()
    cache.seq_reserve(s, 10)
    x = torch.zeros(10, 4, 256, dtype=torch.float16, device="cuda")
    cache.append(0, np.full(10, s, np.int32), np.arange(10), x, x)     # layer 1 stays empty
    with pytest.raises(yahkv.YahkvError) as e:
        yahkv.DecodeBatch(cache, [s])
    assert e.value.code == yahkv.ERR_ORDER
    cache.append(1, np.full(10, s, np.int32), np.arange(10), x, x)
    batch = yahkv.DecodeBatch(cache, [s])
    with pytest.raises(yahkv.YahkvError) as e:
        batch.plan()                                                   # not prepared
    assert e.value.code == yahkv.ERR_ORDER
    with pytest.raises(yahkv.YahkvError) as e:
        batch.prepare(64 * 2)                                          # past max_pages_per_seq
    assert e.value.code == yahkv.ERR_CAPACITY
    batch.prepare(5)
    batch.close()


@pytest.mark.parametrize("fmt", FORMATS)
def test_raw_projection_steps_eager_and_replayed(fmt):
    """batch_decode_layer_raw (norm + RoPE + append of K / V at the device-resident positions, the query side in the
    part kernel's prologue) against yahkv_rope_append + yahkv_attend_decode on a twin cache: one eager step (which
    also builds the RoPE table), then steps replayed from a captured graph; the pools end up byte for byte equal."""
    lens = [300, 64 * 24 - 3, 1000, 1, 15]
    ref, cache, seqs, num_pages, rng = twin_caches(lens, 63, extra_tokens=8, fmt=fmt)
    n, eps = len(seqs), 1e-6
    qw = dev((1.0 + 0.2 * rng.standard_normal(256)).astype(np.float32))
    kw = dev((1.0 + 0.2 * rng.standard_normal(256)).astype(np.float32))
    batch = yahkv.DecodeBatch(cache, seqs)
    batch.prepare(6)

    def raw_inputs():
        return ((rng.standard_normal((LAYERS, n, 24, 256)) * 2).astype(np.float32),
                rng.standard_normal((LAYERS, n, 4, 256)).astype(np.float32),
                rng.standard_normal((LAYERS, n, 4, 256)).astype(np.float32),
                rng.standard_normal((LAYERS, n, 24, 256)).astype(np.float32))

    def ref_step(cur, q, k, v, gate):
        outs = []
        for layer in range(LAYERS):
            q16 = torch.zeros(n, 24, 256, dtype=torch.float16, device="cuda")
            out = torch.zeros(n, 24, 256, device="cuda")
            torch.cuda.synchronize()
            ref.rope_append(layer, seqs, np.array(cur, np.int64), dev(q[layer]), dev(k[layer]), dev(v[layer]), qw, kw, eps, q16)
            ref.attend_decode(layer, seqs, q16, out, gate=dev(gate[layer]), out_dtype=yahkv.OUT_F32)
            ref.sync()
            outs.append(out.cpu().numpy())
        return outs

    cur = list(lens)
    q, k, v, gate = raw_inputs()                      # one eager step
    want = ref_step(cur, q, k, v, gate)
    batch.plan()
    for layer in range(LAYERS):
        out = torch.zeros(n, 24, 256, device="cuda")
        torch.cuda.synchronize()
        batch.decode_layer_raw(layer, dev(q[layer]), dev(k[layer]), dev(v[layer]), qw, kw, eps, out, gate=dev(gate[layer]),
                               out_dtype=yahkv.OUT_F32)
        cache.sync()
        assert np.abs(out.cpu().numpy() - want[layer]).max() <= 1e-4, layer
    batch.advance()
    cur = [x + 1 for x in cur]
    side = torch.cuda.Stream()
    q_s = torch.zeros(LAYERS, n, 24, 256, device="cuda")
    k_s = torch.zeros(LAYERS, n, 4, 256, device="cuda")
    v_s = torch.zeros_like(k_s)
    g_s = torch.zeros(LAYERS, n, 24, 256, device="cuda")
    o_s = torch.zeros(LAYERS, n, 24, 256, device="cuda")
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph, stream=side):
        sp = torch.cuda.current_stream().cuda_stream
        batch.plan(stream=sp)
        for layer in range(LAYERS):
            batch.decode_layer_raw(layer, q_s[layer], k_s[layer], v_s[layer], qw, kw, eps, o_s[layer], gate=g_s[layer],
                                   out_dtype=yahkv.OUT_F32, stream=sp)
        batch.advance(stream=sp)
    for step in range(4):
        q, k, v, gate = raw_inputs()
        want = ref_step(cur, q, k, v, gate)
        q_s.copy_(torch.from_numpy(q)); k_s.copy_(torch.from_numpy(k))
        v_s.copy_(torch.from_numpy(v)); g_s.copy_(torch.from_numpy(gate))
        graph.replay()
        torch.cuda.synchronize()
        got = o_s.cpu().numpy()
        for layer in range(LAYERS):
            assert np.abs(got[layer] - want[layer]).max() <= 1e-4, (step, layer)
        cur = [x + 1 for x in cur]
    batch.commit(5)
    cache.sync()
    assert [cache.seq_len(s, 1) for s in seqs] == cur
    for layer in range(LAYERS):
        a, b = pool_pages(ref, layer, num_pages), pool_pages(cache, layer, num_pages)
        assert all(np.array_equal(x, y) for x, y in zip(a, b))
    batch.close()


@pytest.mark.parametrize("n_splits", [0, 3])
def test_long_sequences_get_longer_units_not_a_long_tail(n_splits):
    """A sequence that needs more than max_splits units of the automatic size gets longer units (the same page count
    for every sequence of the batch) instead of one last unit that takes all the rest; yahkv_batch_set_splits asks for
    a unit count outright. Outputs against the host-planned calls; a change of the unit size reports a changed layout."""
    lens = [64 * 130 + 5, 500, 64 * 40]
    ref, cache, seqs, num_pages, rng = twin_caches(lens, 64, extra_tokens=8, fmt=yahkv.FMT_Q8_0, max_splits=4,
                                                   max_batch_tokens=16384)
    batch = yahkv.DecodeBatch(cache, seqs)
    if n_splits:
        batch.set_splits(n_splits)
    assert batch.prepare(4) is True
    assert batch.prepare(4) is False
    cur = list(lens)
    for step in range(3):
        k, v, q, gate = step_inputs(rng, len(seqs))
        want = host_step(ref, seqs, cur, k, v, q, gate)
        batch.plan()
        for layer in range(LAYERS):
            out = torch.zeros(len(seqs), 24, 256, device="cuda")
            torch.cuda.synchronize()
            batch.decode_layer(layer, dev(k[layer]), dev(v[layer]), dev(q[layer]), out, gate=dev(gate[layer]),
                               out_dtype=yahkv.OUT_F32)
            cache.sync()
            assert np.abs(out.cpu().numpy() - want[layer]).max() <= 1e-4, (step, layer)
        batch.advance()
        batch.commit(1)
        cur = [n + 1 for n in cur]
    batch.set_splits(2 if n_splits else 1)       # other units: a captured graph would have to be captured again
    assert batch.prepare(2) is True
    with pytest.raises(yahkv.YahkvError) as e:
        batch.set_splits(5)                      # above max_splits
    assert e.value.code == yahkv.ERR_CAPACITY
    batch.close()
