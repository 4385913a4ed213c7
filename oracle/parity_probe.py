"""Checks of a live GPU cache against the CPU oracle.

TEST INFRASTRUCTURE ONLY, like the rest of this directory: imported by tests/ and by bench.py, which verifies a sampled
output of every workload against the oracle before its timed region. Nothing here is on a product path.

The cache is read back through the library's inspection calls (yahkv_read_page, yahkv_export_token), so what the
oracle attends over is exactly the bytes the GPU kernels read. A sequence's pages are copied into a compact oracle
pool (page i of the copy = the sequence's i-th logical page): attention depends on the table only through which
bytes each position maps to, so the compact copy gives the same result without holding the whole pool on the host.
"""
import numpy as np

import oracle as O

ABS_TOL = 2e-3     # the path's stated bar on attention outputs
REL_TOL = 1e-4     # the reference checker's own bar (engine/gpu/loom/tools/dattn_q_check.py:205-208)


def compact_pool(cache, layer, seq, n_tokens=None):
    """(oracle pool, identity table) holding the pages of `seq` in logical order, read back from the GPU."""
    table = cache.seq_table(seq)
    if n_tokens is not None:
        table = table[: (int(n_tokens) + O.PAGE_TOKENS - 1) // O.PAGE_TOKENS]
    if cache.fmt in (O.FMT_KV8A16, O.FMT_KV4A16):
        pool = (O.Kv8Pool if cache.fmt == O.FMT_KV8A16 else O.Kv4Pool)(max(len(table), 1))
        for i, p in enumerate(table):
            pool.kcodes[i], pool.kscales[i] = cache.read_page(layer, 0, int(p))
            pool.vcodes[i], pool.vstats[i] = cache.read_page(layer, 1, int(p))
        return pool, np.arange(len(table), dtype=np.int32)
    pool = O.PagedPool(cache.fmt, max(len(table), 1))
    for i, p in enumerate(table):
        pool.kcodes[i], pool.kscales[i] = cache.read_page(layer, 0, int(p))
        pool.vcodes[i], pool.vscales[i] = cache.read_page(layer, 1, int(p))
    return pool, np.arange(len(table), dtype=np.int32)


def errors(got, want):
    err = float(np.abs(np.asarray(got, np.float64) - want).max())
    return err, err / max(float(np.abs(want).max()), 1e-30)


def check_decode_row(cache, layer, seq, n_keys, q_row, out_row, gate_row=None, out_is_f16=False):
    """Max-abs and relative error of one decode output row [24][256] against float64 attention over the cache's own
    bytes. fp16 outputs carry their rounding (2^-11 relative) on top."""
    pool, table = compact_pool(cache, layer, seq, n_keys)
    if cache.fmt in (O.FMT_KV8A16, O.FMT_KV4A16):     # the newest tile is read from the sequence's open fp16 tile
        open_tile = cache.read_open_tile(seq, layer).view(np.uint16)
        want = pool.attend_decode_f64(table, int(n_keys), np.asarray(q_row, np.float16), open_tile, gate_row)
    else:
        want = pool.attend_decode_f64(table, int(n_keys), np.asarray(q_row, np.float16), gate_row)
    err, rel = errors(out_row, want)
    slack = float(np.abs(want).max()) * 2.0 ** -11 if out_is_f16 else 0.0
    return err, rel, slack


def check_prefill_rows(cache, layer, seq, start, q_chunk, out_chunk, rows, gate_chunk=None, out_is_f16=False):
    """Worst error over the given rows of one sequence's chunk (q_chunk, out_chunk: [chunk][24][256])."""
    n_total = int(start) + len(q_chunk)
    pool, table = compact_pool(cache, layer, seq, n_total)
    worst, worst_rel, slack = 0.0, 0.0, 0.0
    for r in rows:
        want = pool.attend_prefill_f64(table, int(start), np.asarray(q_chunk, np.float16), q_begin=int(r),
                                       q_end=int(r) + 1, gate=gate_chunk)[0]
        err, rel = errors(out_chunk[r], want)
        worst, worst_rel = max(worst, err), max(worst_rel, rel)
        if out_is_f16:
            slack = max(slack, float(np.abs(want).max()) * 2.0 ** -11)
    return worst, worst_rel, slack


def check_appended_token(cache, layer, seq, pos, k_row, v_row):
    """True when the blocks the cache holds for one position are the oracle's quantization of the fp16 rows."""
    if cache.fmt in (O.FMT_KV8A16, O.FMT_KV4A16):   # K row against the oracle's quantizer (zero mean); V tiles are covered by the tests
        page = int(cache.seq_table(seq)[int(pos) // O.PAGE_TOKENS])
        codes, scales = cache.read_page(layer, 0, page)
        quant = O.kv8_quant_k if cache.fmt == O.FMT_KV8A16 else O.kv4_quant_k
        want_c, want_s = quant(np.asarray(k_row, np.float16), np.zeros((4, 256), np.float32))
        tok = int(pos) % O.PAGE_TOKENS
        return bool(np.array_equal(codes[:, tok], want_c) and np.array_equal(scales[:, tok], want_s))
    if cache.fmt == O.FMT_F16:        # fp16 pages hold the rows as they came
        page, tok = int(cache.seq_table(seq)[int(pos) // O.PAGE_TOKENS]), int(pos) % O.PAGE_TOKENS
        kc, _ = cache.read_page(layer, 0, page)
        vc, _ = cache.read_page(layer, 1, page)
        return bool(np.array_equal(kc[:, tok].view(np.float16), np.asarray(k_row, np.float16)) and
                    np.array_equal(vc[:, tok].view(np.float16), np.asarray(v_row, np.float16)))
    kb, vb = cache.export_token(layer, seq, int(pos))
    k32 = np.asarray(k_row, np.float16).astype(np.float32)
    v32 = np.asarray(v_row, np.float16).astype(np.float32)
    return bool(np.array_equal(kb, O.quantize(k32, cache.fmt)) and np.array_equal(vb, O.quantize(v32, cache.fmt)))


class ChurnProbe:
    """Parity probe for the serving-churn driver: before a step, one of the step's decode slots and its prefill slot
    are refilled with real K/V on one layer (the churn itself admits sequences over recycled pages without writing
    them), and after the step's calls their outputs are compared with float64 attention over the cache's bytes."""

    def __init__(self, runner, layer, seed=0, fill_chunk=1024):
        self.runner, self.layer, self.fill_chunk = runner, layer, fill_chunk
        self.rng = np.random.default_rng([seed, runner.rank])
        self.worst, self.worst_rel, self.checks = 0.0, 0.0, 0

    def arm(self, k, to_device):
        """Picks this rank's probe slots of step k and refills them; returns the picked (decode slot, prefill slot),
        either of which may be None. `to_device` turns a numpy fp16 array into a device tensor."""
        r = self.runner
        finished, _, prefill_slot, decode = r.sched.step(k)
        gone = {int(s) for s in finished}
        mine = [int(s) for s in decode if int(s) % r.world == r.rank and int(s) not in gone
                and r.length[int(s)] + 1 <= r.ctx_cap]
        self.decode_slot = min(mine, key=lambda s: r.length[s]) if mine else None
        own_prefill = prefill_slot % r.world == r.rank and r.length[prefill_slot] + r.sched.chunk <= r.ctx_cap
        self.prefill_slot = int(prefill_slot) if own_prefill else None
        for slot in (self.decode_slot, self.prefill_slot):
            if slot is not None:
                self._refill(slot, to_device)
        return self.decode_slot, self.prefill_slot

    def _refill(self, slot, to_device):
        cache, sid, n = self.runner.cache, self.runner.seq[slot], self.runner.length[slot]
        cache.seq_set_len(sid, 0, layer=self.layer)
        for c0 in range(0, n, self.fill_chunk):
            c1 = min(n, c0 + self.fill_chunk)
            K = self.rng.standard_normal((c1 - c0, 4, 256), dtype=np.float32).astype(np.float16)
            V = self.rng.standard_normal((c1 - c0, 4, 256), dtype=np.float32).astype(np.float16)
            cache.append(self.layer, np.full(c1 - c0, sid, np.int32), np.arange(c0, c1, dtype=np.int64), to_device(K),
                         to_device(V))
        cache.sync()

    def record(self, err, rel, slack=0.0):
        self.worst, self.worst_rel, self.checks = max(self.worst, err - slack), max(self.worst_rel, rel), self.checks + 1
