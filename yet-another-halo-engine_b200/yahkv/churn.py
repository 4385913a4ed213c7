"""Seed-driven serving churn over a sharded set of sequences (the whole-box configuration).

A fixed population of sequence slots (256 in the configuration) is partitioned by slot across the GPUs of a box:
slot s belongs to rank s % world. Every rank derives the SAME global schedule from the seed and applies only its own
slots, so there is no exchange on the data path; what a rank does depends on the seed, the step and its rank alone.

Per step of the schedule:
  * a tenth of the slots finish: their pages go back to the free list and a new sequence takes the slot, with a
    context length drawn uniformly from [ctx_lo, ctx_hi]; its pages come from the recycled pool (LIFO, so they are
    scattered and hold the previous owner's blocks, which the new owner's keys simply overwrite as it is filled);
  * one slot (round robin) is in prefill: it appends a chunk of `chunk` tokens and runs chunked-prefill attention;
  * `n_decode` other slots append one token each and run decode attention.
The reference engine serves one sequence at a time (engine/serve/yah_server.cc:229-236) and has no allocator; this
driver exists to exercise the page allocator, the block tables and the kernels under allocation churn.

`ChurnRunner` applies the schedule to a `KvCache`. With a host-only cache (device = -1) it drives the allocator and
tables alone, which is what the CPU tests and the multi-rank gloo test use; with a GPU cache it also launches the
appends and attentions (inputs are synthetic device tensors supplied by the caller).
"""
import numpy as np


class ChurnSchedule:
    def __init__(self, n_slots=256, ctx_lo=512, ctx_hi=65536, n_decode=240, chunk=1024, finish_frac=0.1, seed=0):
        self.n_slots, self.ctx_lo, self.ctx_hi = n_slots, ctx_lo, ctx_hi
        self.n_decode, self.chunk, self.finish_frac, self.seed = min(n_decode, n_slots - 1), chunk, finish_frac, seed
        rng = np.random.default_rng(seed)
        self.initial_lens = rng.integers(ctx_lo, ctx_hi + 1, n_slots)

    def step(self, k):
        """Events of step k, identical on every rank: (finished slots, their new lengths, prefill slot, decode slots)."""
        rng = np.random.default_rng([self.seed, k + 1])
        n_fin = max(1, int(round(self.n_slots * self.finish_frac)))
        prefill_slot = k % self.n_slots
        others = np.array([s for s in range(self.n_slots) if s != prefill_slot])
        finished = np.sort(rng.choice(others, n_fin, replace=False))
        new_lens = rng.integers(self.ctx_lo, self.ctx_hi + 1, n_fin)
        decode = np.sort(rng.choice(others, self.n_decode, replace=False))
        return finished, new_lens, prefill_slot, decode


def owner(slot, world):
    return slot % world


class ChurnRunner:
    """Applies a ChurnSchedule to one rank's KvCache. Lengths are capped at ctx_cap tokens so a slot never outgrows
    its block table; a slot that would, finishes instead (it is replaced by a fresh sequence of the drawn length)."""

    def __init__(self, cache, schedule, rank=0, world=1, n_layers=1, ctx_cap=None):
        self.cache, self.sched, self.rank, self.world, self.n_layers = cache, schedule, rank, world, n_layers
        self.ctx_cap = ctx_cap or schedule.ctx_hi + schedule.chunk + 64
        self.slots = [s for s in range(schedule.n_slots) if owner(s, world) == rank]
        self.seq = {}       # slot -> sequence id of the cache
        self.length = {}    # slot -> tokens
        for s in self.slots:
            self._admit(s, int(schedule.initial_lens[s]))
        self.stats = []

    def _admit(self, slot, n_tokens):
        sid = self.cache.seq_create()
        self.cache.seq_reserve(sid, n_tokens)
        self.cache.seq_set_len(sid, n_tokens)      # the recycled pages' contents stand in for the prompt's cache
        self.seq[slot], self.length[slot] = sid, n_tokens

    def _retire(self, slot):
        self.cache.seq_free(self.seq[slot])

    def step(self, k, gpu=None):
        """gpu: None (allocator only) or a callable gpu(kind, seq_ids, positions) that launches the step's device
        work for this rank: kind is "decode" (one token per sequence) or "prefill" (positions = the chunk's)."""
        finished, new_lens, prefill_slot, decode = self.sched.step(k)
        freed = admitted = 0
        for slot, n in zip(finished, new_lens):
            if owner(int(slot), self.world) != self.rank:
                continue
            freed += (self.length[int(slot)] + 63) // 64
            self._retire(int(slot))
            self._admit(int(slot), int(n))
            admitted += (int(n) + 63) // 64
        mine_decode = [int(s) for s in decode if owner(int(s), self.world) == self.rank]
        # a slot whose table is full restarts as a fresh short sequence instead of growing
        for s in list(mine_decode) + ([prefill_slot] if owner(prefill_slot, self.world) == self.rank else []):
            grow = self.sched.chunk if s == prefill_slot else 1
            if self.length[s] + grow > self.ctx_cap:
                self._retire(s)
                self._admit(s, self.sched.ctx_lo)
        tokens = 0
        if owner(prefill_slot, self.world) == self.rank:
            sid, n = self.seq[prefill_slot], self.length[prefill_slot]
            self.cache.seq_reserve(sid, n + self.sched.chunk)
            if gpu is not None:
                gpu("prefill", [sid], np.arange(n, n + self.sched.chunk, dtype=np.int64))
            else:
                self.cache.seq_set_len(sid, n + self.sched.chunk)
            self.length[prefill_slot] = n + self.sched.chunk
            tokens += self.sched.chunk
        if mine_decode:
            sids = [self.seq[s] for s in mine_decode]
            pos = np.array([self.length[s] for s in mine_decode], np.int64)
            for sid, p in zip(sids, pos):
                self.cache.seq_reserve(sid, int(p) + 1)
            if gpu is not None:
                gpu("decode", sids, pos)
            else:
                for sid, p in zip(sids, pos):
                    self.cache.seq_set_len(sid, int(p) + 1)
            for s in mine_decode:
                self.length[s] += 1
            tokens += len(mine_decode)
        rec = {"step": k, "rank": self.rank, "pages_free": self.cache.pages_free(), "freed": freed,
               "admitted": admitted, "tokens": tokens, "decode": len(mine_decode),
               "cached_tokens": int(sum(self.length.values())),
               "attended_keys": int(sum(self.length[s] for s in mine_decode))}
        self.stats.append(rec)
        return rec

    def pages_in_use(self):
        return sum((n + 63) // 64 for n in self.length.values())


def pages_needed(schedule, rank, world):
    """Pages that always suffice for a rank's slots (every slot at its cap): the pool size for tests and benches."""
    mine = sum(1 for s in range(schedule.n_slots) if owner(s, world) == rank)
    return mine * ((schedule.ctx_hi + schedule.chunk + 64 + 63) // 64 + 1)
