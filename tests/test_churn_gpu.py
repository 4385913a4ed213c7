"""The serving-churn driver on the GPU with a parity probe: sequences are admitted over recycled pages, retired and
regrown for a number of steps; at every step one decode slot and the prefill slot hold real K/V on one layer and their
outputs are compared with float64 attention over the bytes the cache holds (read back through the C ABI)."""
import numpy as np
import pytest
import torch

import yahkv
from gpu_util import dev
from parity_probe import ABS_TOL, ChurnProbe, check_decode_row, check_prefill_rows
from yahkv.churn import ChurnRunner, ChurnSchedule, pages_needed

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("fmt", [yahkv.FMT_Q8_0, yahkv.FMT_Q4_0])
def test_churn_steps_with_parity_probe(fmt):
    layers, probe_layer = 2, 1
    sched = ChurnSchedule(n_slots=12, ctx_lo=40, ctx_hi=3000, n_decode=8, chunk=256, finish_frac=0.2, seed=5)
    cap_pages = (sched.ctx_hi + sched.chunk + 64 + 63) // 64 + 1
    cache = yahkv.KvCache(n_layers=layers, num_pages=pages_needed(sched, 0, 1), fmt=fmt, max_seqs=sched.n_slots,
                          max_pages_per_seq=cap_pages, max_batch_tokens=1024)
    runner = ChurnRunner(cache, sched, 0, 1, n_layers=layers)
    probe = ChurnProbe(runner, probe_layer, seed=9)
    rng = np.random.default_rng(17)
    nd = sched.n_decode

    def gpu(kind, sids, pos):
        n = len(pos)
        if kind == "decode":
            k, v = rng.standard_normal((2, n, 4, 256)).astype(np.float16)
            q = rng.standard_normal((n, 24, 256)).astype(np.float16)
            for layer in range(layers):
                out = torch.full((n, 24, 256), float("nan"), device="cuda")
                cache.append(layer, sids, pos, dev(k), dev(v))
                torch.cuda.synchronize()
                cache.attend_decode(layer, sids, dev(q), out, out_dtype=yahkv.OUT_F32)
                cache.sync()
                if layer == probe_layer and probe.decode_slot is not None:
                    i = sids.index(runner.seq[probe.decode_slot])
                    probe.record(*check_decode_row(cache, layer, sids[i], int(pos[i]) + 1, q[i], out[i].cpu().numpy()))
        else:
            k, v = rng.standard_normal((2, n, 4, 256)).astype(np.float16)
            q = rng.standard_normal((n, 24, 256)).astype(np.float16)
            for layer in range(layers):
                out = torch.full((n, 24, 256), float("nan"), device="cuda")
                cache.append(layer, np.full(n, sids[0], np.int32), pos, dev(k), dev(v))
                torch.cuda.synchronize()
                cache.attend_prefill(layer, sids, [n], dev(q), out, out_dtype=yahkv.OUT_F32)
                cache.sync()
                if layer == probe_layer and probe.prefill_slot is not None:
                    probe.record(*check_prefill_rows(cache, layer, sids[0], int(pos[0]), q, out.cpu().numpy(),
                                                     [0, 127, 128, n - 1]))

    total = pages_needed(sched, 0, 1)
    for k in range(8):
        probe.arm(k, dev)
        rec = runner.step(k, gpu)
        assert rec["pages_free"] + runner.pages_in_use() == total
    assert probe.checks >= 12, probe.checks
    # prefill rows multiply fp16 operands (2^-11 relative rounding each), so the relative bar here is 1e-3
    assert probe.worst <= ABS_TOL and probe.worst_rel < 1e-3, (probe.worst, probe.worst_rel)
    assert nd == 8
    cache.close()
