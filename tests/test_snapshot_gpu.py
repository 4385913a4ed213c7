"""Cache snapshots: save sequences, load them into another context where they land on different pages, and get the
same attention; refuse mismatched contexts and broken files without leaving anything behind."""
import numpy as np
import pytest
import torch

import yahkv
from gpu_util import dev

pytestmark = pytest.mark.gpu


def attend(cache, layer, seqs, q):
    out = torch.zeros(len(seqs), 24, 256, device="cuda")
    torch.cuda.synchronize()
    cache.attend_decode(layer, seqs, dev(q), out, out_dtype=yahkv.OUT_F32)
    cache.sync()
    return out.cpu().numpy()


@pytest.mark.parametrize("fmt", [yahkv.FMT_Q8_0, yahkv.FMT_Q4_0, yahkv.FMT_KV8A16, yahkv.FMT_KV4A16, yahkv.FMT_F16])
def test_snapshot_round_trip_onto_other_pages(tmp_path, fmt):
    rng = np.random.default_rng(51)
    a = yahkv.KvCache(n_layers=2, num_pages=12, fmt=fmt, max_seqs=3, max_pages_per_seq=6)
    lens = [130, 64]
    seqs = []
    tile_fmt = fmt in (yahkv.FMT_KV8A16, yahkv.FMT_KV4A16)
    for n in lens:
        s = a.seq_create()
        a.seq_reserve(s, n + 1)
        if tile_fmt:                    # these formats carry a K mean and an open fp16 tile per (sequence, layer)
            a.seq_set_kmean(s, (0.5 * rng.standard_normal((4, 256))).astype(np.float32))
        for layer in range(2):
            K = rng.standard_normal((n, 4, 256)).astype(np.float16)
            V = rng.standard_normal((n, 4, 256)).astype(np.float16)
            a.append(layer, np.full(n, s, np.int32), np.arange(n), dev(K), dev(V))
        seqs.append(s)
    q = rng.standard_normal((2, 24, 256)).astype(np.float16)
    want = [attend(a, layer, seqs, q) for layer in range(2)]
    path = tmp_path / "kv.snap"
    a.snapshot_save(seqs, path)
    # one more decode step in the original context: the loaded copy must continue the same way
    k1 = rng.standard_normal((2, 4, 256)).astype(np.float16)
    v1 = rng.standard_normal((2, 4, 256)).astype(np.float16)
    a.append(1, seqs, lens, dev(k1), dev(v1))
    want_next = attend(a, 1, seqs, q)
    a.close()

    b = yahkv.KvCache(n_layers=2, num_pages=20, fmt=fmt, max_seqs=4, max_pages_per_seq=6)
    other = b.seq_create()
    b.seq_reserve(other, 64 * 3)                  # shifts where the loaded pages land
    loaded = b.snapshot_load(path)
    assert len(loaded) == 2 and other not in loaded
    assert [b.seq_len(s, 1) for s in loaded] == lens
    assert b.seq_table(loaded[0]).tolist() == [3, 4, 5] and b.pages_free() == 20 - 3 - 3 - 2
    for layer in range(2):
        assert np.array_equal(attend(b, layer, loaded, q), want[layer])     # same bytes, same kernel: identical
    b.append(1, loaded, lens, dev(k1), dev(v1))
    assert np.array_equal(attend(b, 1, loaded, q), want_next)

    # a context of another format or layer count refuses the file and stays untouched
    other_fmt = yahkv.FMT_Q4_0 if fmt != yahkv.FMT_Q4_0 else yahkv.FMT_Q8_0
    for kw in (dict(n_layers=2, fmt=other_fmt), dict(n_layers=3, fmt=fmt)):
        c = yahkv.KvCache(num_pages=20, max_seqs=4, max_pages_per_seq=6, **kw)
        with pytest.raises(yahkv.YahkvError) as e:
            c.snapshot_load(path)
        assert e.value.code == yahkv.ERR_INVALID and c.pages_free() == 20
    # a pool too small for the snapshot fails cleanly: no sequence, no page left behind
    d = yahkv.KvCache(n_layers=2, num_pages=3, fmt=fmt, max_seqs=4, max_pages_per_seq=6)
    with pytest.raises(yahkv.YahkvError) as e:
        d.snapshot_load(path)
    assert e.value.code == yahkv.ERR_NO_PAGES and d.pages_free() == 3
    assert d.seq_create() == 0
    # a truncated file
    raw = path.read_bytes()
    (tmp_path / "cut.snap").write_bytes(raw[: len(raw) // 2])
    with pytest.raises(yahkv.YahkvError):
        b.snapshot_load(tmp_path / "cut.snap")
    assert b.pages_free() == 20 - 3 - 3 - 2
