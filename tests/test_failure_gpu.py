"""The give-up path of the library's bounded device waits, exercised without faulting anything: a kernel waits a few
milliseconds on a barrier nobody arrives at, stops waiting, records the sticky status word and returns; the host sees
it at the next sync as an error with a message, the word is cleared, and the context keeps working.
The reference's model is the same: bounded polls and a sticky status (engine/gpu/loom/tools/gen_chain.py:12-19)."""
import time

import numpy as np
import pytest
import torch

import oracle as O
import yahkv
from gpu_util import dev, fill_both

pytestmark = pytest.mark.gpu


def test_a_wait_that_runs_out_is_reported_and_the_context_survives():
    rng = np.random.default_rng(3)
    cache = yahkv.KvCache(num_pages=4, max_seqs=1, max_pages_per_seq=4)
    pool = O.PagedPool(yahkv.FMT_Q8_0, 4)
    s = cache.seq_create()
    K = rng.standard_normal((100, 4, 256)).astype(np.float16)
    V = rng.standard_normal((100, 4, 256)).astype(np.float16)
    fill_both(cache, pool, 0, s, [2, 0], K, V)
    cache.sync()                                    # clean so far
    t0 = time.perf_counter()
    cache.debug_wait_timeout(5000)                  # 5 ms limit
    with pytest.raises(yahkv.YahkvError) as e:
        cache.sync()
    waited = time.perf_counter() - t0
    assert e.value.code == yahkv.ERR_CUDA and "gave up a bounded wait" in e.value.message
    assert 0.004 <= waited < 1.0, waited            # it did wait, and only for about the limit
    cache.sync()                                    # the word is sticky until read, then cleared
    q = rng.standard_normal((1, 24, 256)).astype(np.float16)
    out = torch.zeros(1, 24, 256, device="cuda")
    cache.attend_decode(0, [s], dev(q), out, out_dtype=yahkv.OUT_F32)
    cache.sync()
    assert np.abs(out.cpu().numpy()[0] - pool.attend_decode_f64([2, 0], 100, q[0])).max() <= 2e-3
    # the host-buffer step reports it too (blocking and pipelined forms)
    cache.seq_reserve(s, 102)
    k1 = rng.standard_normal((1, 4, 256)).astype(np.float16)
    hout = np.zeros((1, 24, 256), np.float32)
    cache.debug_wait_timeout(2000)
    with pytest.raises(yahkv.YahkvError) as e:
        cache.decode_step_host(0, [s], k1, k1, q, hout, out_dtype=yahkv.OUT_F32)
    assert e.value.code == yahkv.ERR_CUDA
    cache.decode_step_host(0, [s], k1, k1, q, hout, out_dtype=yahkv.OUT_F32)     # and works again
    assert np.isfinite(hout).all() and cache.seq_len(s, 0) == 102
    with pytest.raises(yahkv.YahkvError):
        cache.debug_wait_timeout(0)
    cache.close()
