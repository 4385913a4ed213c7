"""Randomised chunked-prefill attention: ragged batches of chunks (1 row up to several query tiles, cached lengths on
and around tile and page edges), shuffled tables, the wave size of the tile planner varied so that tiles get split
along the keys into 2..4 parts, with and without the gate, fp16 and f32 outputs, every output row against the float64
oracle over pools the oracle itself filled. Bar: 2e-3 max-abs (fp16 operands, fp32 softmax)."""
import numpy as np
import pytest
import torch

import oracle as O
import yahkv
from gpu_util import dev

pytestmark = pytest.mark.gpu
EDGES = [0, 1, 63, 64, 65, 127, 128, 129, 191, 255, 256, 257, 511, 512]
ABS_TOL = 2e-3


@pytest.mark.parametrize("fmt", [yahkv.FMT_Q8_0, yahkv.FMT_Q4_0, yahkv.FMT_F16])
def test_random_chunk_batches_against_the_oracle(fmt):
    rng = np.random.default_rng(2000 + fmt)
    for case in range(5):
        n_seqs = int(rng.integers(1, 5))
        cached = [int(rng.choice(EDGES)) if rng.random() < 0.5 else int(rng.integers(0, 2500)) for _ in range(n_seqs)]
        chunks = [int(rng.choice([1, 2, 127, 128, 129, 300])) if rng.random() < 0.5 else int(rng.integers(1, 400))
                  for _ in range(n_seqs)]
        totals = [a + b for a, b in zip(cached, chunks)]
        pages = [(n + 63) // 64 for n in totals]
        num_pages = sum(pages) + 3
        cache = yahkv.KvCache(n_layers=1, num_pages=num_pages, fmt=fmt, max_seqs=n_seqs, max_pages_per_seq=max(pages),
                              max_batch_tokens=4096)
        pool = O.PagedPool(fmt, num_pages)
        perm = rng.permutation(num_pages).astype(np.int32)
        seqs, tables, off = [], [], 0
        for i, n in enumerate(totals):
            s = cache.seq_create()
            table = perm[off:off + pages[i]].copy()
            off += pages[i]
            cache.seq_set_table(s, table)
            K = rng.standard_normal((n, 4, 256)).astype(np.float16)
            V = rng.standard_normal((n, 4, 256)).astype(np.float16)
            for c0, c1 in ((0, cached[i]), (cached[i], n)):
                if c1 > c0:
                    cache.append(0, np.full(c1 - c0, s, np.int32), np.arange(c0, c1, dtype=np.int64), dev(K[c0:c1]), dev(V[c0:c1]))
            pool.append(table, 0, K, V)
            seqs.append(s), tables.append(table)
        rows = sum(chunks)
        q = rng.standard_normal((rows, 24, 256)).astype(np.float16)
        gate = rng.standard_normal((rows, 24, 256)).astype(np.float32)
        want, want_gated, row = [], [], 0
        for i, c in enumerate(chunks):
            want.append(pool.attend_prefill_f64(tables[i], cached[i], q[row:row + c]))
            want_gated.append(pool.attend_prefill_f64(tables[i], cached[i], q[row:row + c], gate=gate[row:row + c]))
            row += c
        want, want_gated = np.concatenate(want), np.concatenate(want_gated)
        for sms in (0, int(rng.choice([2, 4, 6, 10, 14, 22, 40]))):   # 0: no splitting; else the planner's wave in SMs
            cache.debug_set_prefill_sms(sms)
            for use_gate, f32 in ((False, True), (True, False)):
                out = torch.full((rows, 24, 256), float("nan"), device="cuda", dtype=torch.float32 if f32 else torch.float16)
                torch.cuda.synchronize()
                cache.attend_prefill(0, seqs, chunks, dev(q), out, gate=dev(gate) if use_gate else None,
                                     out_dtype=yahkv.OUT_F32 if f32 else yahkv.OUT_F16)
                cache.sync()
                got = out.float().cpu().numpy().astype(np.float64)
                ref = want_gated if use_gate else want
                tol = ABS_TOL + (0.0 if f32 else np.abs(ref).max() * 2.0 ** -11)
                err = np.abs(got - ref).max()
                assert np.isfinite(got).all() and err <= tol, (fmt, case, cached, chunks, sms, use_gate, err)
        cache.close()
