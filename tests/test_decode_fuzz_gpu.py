"""Randomised decode attention over all five cache formats: many small batches with ragged lengths (1 token up to a
dozen pages, lengths on and around tile and page edges), shuffled tables, every split count from one unit per sequence
to more units than pages, with and without the gate, each output row against the float64 oracle over the pools the
oracle itself filled (appends byte-exact). Bars: 2e-3 max-abs and 1e-4 of the largest output
(engine/gpu/loom/tools/dattn_q_check.py:205-208)."""
import numpy as np
import pytest
import torch

import oracle as O
import yahkv
from gpu_util import dev

pytestmark = pytest.mark.gpu
FORMATS = [yahkv.FMT_Q8_0, yahkv.FMT_Q4_0, yahkv.FMT_KV8A16, yahkv.FMT_KV4A16, yahkv.FMT_F16]
EDGES = [1, 2, 15, 16, 17, 31, 32, 33, 63, 64, 65, 127, 128, 129, 191, 192, 193, 255, 256, 257]


@pytest.mark.parametrize("fmt", FORMATS)
def test_random_batches_against_the_oracle(fmt):
    rng = np.random.default_rng(1000 + fmt)
    tile_fmt = fmt in (yahkv.FMT_KV8A16, yahkv.FMT_KV4A16)
    worst = 0.0
    for case in range(6):
        n_seqs = int(rng.integers(1, 5))
        lens = [int(rng.choice(EDGES)) if rng.random() < 0.5 else int(rng.integers(1, 800)) for _ in range(n_seqs)]
        pages = [(n + 63) // 64 for n in lens]
        num_pages = sum(pages) + 3
        cache = yahkv.KvCache(n_layers=1, num_pages=num_pages, fmt=fmt, max_seqs=n_seqs, max_pages_per_seq=max(pages),
                              max_batch_tokens=1024, max_splits=64)
        pool = (O.Kv8Pool if fmt == yahkv.FMT_KV8A16 else O.Kv4Pool)(num_pages) if tile_fmt else O.PagedPool(fmt, num_pages)
        perm = rng.permutation(num_pages).astype(np.int32)
        seqs, tables, states, off = [], [], [], 0
        for i, n in enumerate(lens):
            s = cache.seq_create()
            table = perm[off:off + pages[i]].copy()
            off += pages[i]
            cache.seq_set_table(s, table)
            K = rng.standard_normal((n, 4, 256)).astype(np.float16)
            V = rng.standard_normal((n, 4, 256)).astype(np.float16)
            if rng.random() < 0.5:
                V[:, :, ::29] *= 10.0
            st = None
            if tile_fmt:
                m = (0.5 * rng.standard_normal((4, 256))).astype(np.float32)
                cache.seq_set_kmean(s, m)
                st = pool.new_sequence(m)
                K = (K.astype(np.float32) + m).astype(np.float16)
            cut = int(rng.integers(0, n + 1))                  # two append calls with a random boundary
            for c0, c1 in ((0, cut), (cut, n)):
                if c1 > c0:
                    cache.append(0, np.full(c1 - c0, s, np.int32), np.arange(c0, c1, dtype=np.int64), dev(K[c0:c1]), dev(V[c0:c1]))
                    if tile_fmt:
                        pool.append(table, c0, K[c0:c1], V[c0:c1], *st)
                    else:
                        pool.append(table, c0, K[c0:c1], V[c0:c1])
            seqs.append(s), tables.append(table), states.append(st)
        q = (0.5 * rng.standard_normal((n_seqs, 24, 256))).astype(np.float16)
        gate = rng.standard_normal((n_seqs, 24, 256)).astype(np.float32)
        for use_gate in (False, True):
            g = gate if use_gate else None
            if tile_fmt:
                want = np.stack([pool.attend_decode_f64(tables[i], lens[i], q[i], states[i][0], None if g is None else g[i])
                                 for i in range(n_seqs)])
            else:
                want = np.stack([pool.attend_decode_f64(tables[i], lens[i], q[i], None if g is None else g[i])
                                 for i in range(n_seqs)])
            for n_splits in (0, 1, 2, 3, 7, 64):
                out = torch.full((n_seqs, 24, 256), float("nan"), device="cuda")
                torch.cuda.synchronize()
                cache.attend_decode(0, seqs, dev(q), out, gate=None if g is None else dev(g), out_dtype=yahkv.OUT_F32,
                                    n_splits=n_splits)
                cache.sync()
                got = out.cpu().numpy().astype(np.float64)
                err = np.abs(got - want).max()
                assert err <= 2e-3 and err < 1e-4 * np.abs(want).max(), (fmt, case, lens, n_splits, use_gate, err)
                worst = max(worst, err / np.abs(want).max())
        cache.close()
    assert worst < 1e-4
