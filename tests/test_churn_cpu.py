"""The serving-churn driver on host-only contexts: allocator invariants under free/allocate churn, and the multi-rank
path (sequences partitioned by slot, no exchange on the data path) as two gloo ranks on the CPU."""
import os
import subprocess
import sys

import numpy as np

import yahkv
from yahkv.churn import ChurnRunner, ChurnSchedule, owner, pages_needed

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
SMALL = dict(n_slots=24, ctx_lo=40, ctx_hi=2000, n_decode=20, chunk=128, finish_frac=0.1, seed=3)


def host_cache(sched, rank, world, n_layers=2):
    cap_pages = (sched.ctx_hi + sched.chunk + 64 + 63) // 64 + 1
    return yahkv.KvCache(device=-1, n_layers=n_layers, num_pages=pages_needed(sched, rank, world),
                         max_seqs=sched.n_slots, max_pages_per_seq=cap_pages)


def run_rank(rank, world, steps):
    sched = ChurnSchedule(**SMALL)
    cache = host_cache(sched, rank, world)
    runner = ChurnRunner(cache, sched, rank, world, n_layers=2)
    total = pages_needed(sched, rank, world)
    recs = []
    for k in range(steps):
        rec = runner.step(k)
        assert rec["pages_free"] + runner.pages_in_use() == total      # no page lost or double-counted
        recs.append(rec)
    tables = {s: cache.seq_table(runner.seq[s]).tolist() for s in runner.slots}
    flat = [p for t in tables.values() for p in t]
    assert len(flat) == len(set(flat))                                 # no page owned twice
    for s in runner.slots:
        assert cache.seq_len(runner.seq[s], 0) == runner.length[s] == cache.seq_len(runner.seq[s], 1)
    return recs, {s: runner.length[s] for s in runner.slots}


def test_schedule_is_deterministic_and_well_formed():
    a, b = ChurnSchedule(**SMALL), ChurnSchedule(**SMALL)
    assert np.array_equal(a.initial_lens, b.initial_lens)
    for k in range(5):
        fa, la, pa, da = a.step(k)
        fb, lb, pb, db = b.step(k)
        assert np.array_equal(fa, fb) and np.array_equal(la, lb) and pa == pb and np.array_equal(da, db)
        assert pa not in fa and pa not in da and len(set(da)) == len(da) == SMALL["n_decode"]
        assert len(fa) == round(SMALL["n_slots"] * SMALL["finish_frac"])


def test_single_rank_churn_keeps_allocator_consistent():
    recs, lengths = run_rank(0, 1, 60)
    assert sum(r["freed"] for r in recs) > 0 and sum(r["admitted"] for r in recs) > 0
    assert all(r["tokens"] == SMALL["n_decode"] + SMALL["chunk"] for r in recs)


def test_partition_covers_every_slot_once_and_matches_the_single_rank_run():
    recs1, len1 = run_rank(0, 1, 30)
    merged = {}
    tokens = np.zeros(30, int)
    for rank in range(3):
        recs, lens = run_rank(rank, 3, 30)
        assert all(owner(s, 3) == rank for s in lens)
        assert not set(lens) & set(merged)
        merged.update(lens)
        tokens += np.array([r["tokens"] for r in recs])
    assert merged == len1                                              # same final state, however it is sharded
    assert np.array_equal(tokens, [r["tokens"] for r in recs1])


WORKER = r"""
import os, sys, json
sys.path.insert(0, os.path.join({root!r}, "tests")); sys.path.insert(0, os.path.join({root!r}, "yet-another-halo-engine_b200"))
import torch.distributed as dist
from test_churn_cpu import run_rank
dist.init_process_group("gloo")
rank, world = dist.get_rank(), dist.get_world_size()
recs, lens = run_rank(rank, world, 25)
out = [None] * world
dist.all_gather_object(out, {{"tokens": [r["tokens"] for r in recs], "keys": [r["attended_keys"] for r in recs], "lens": lens}})
if rank == 0:
    print("RESULT " + json.dumps(out))
dist.barrier()
dist.destroy_process_group()
"""


def test_two_gloo_ranks_shard_the_schedule(tmp_path):
    script = tmp_path / "worker.py"
    script.write_text(WORKER.format(root=ROOT))
    env = dict(os.environ, MASTER_ADDR="127.0.0.1", PYTHONDONTWRITEBYTECODE="1")
    r = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2",
                        "--master-addr", "127.0.0.1", "--master-port", "29531", str(script)],
                       capture_output=True, text=True, env=env, timeout=300)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-2000:]
    import json
    line = [l for l in r.stdout.splitlines() if l.startswith("RESULT ")][-1]
    out = json.loads(line[len("RESULT "):])
    recs1, len1 = run_rank(0, 1, 25)
    merged = {}
    for part in out:
        merged.update({int(k): v for k, v in part["lens"].items()})
    assert merged == len1
    tokens = np.sum([p["tokens"] for p in out], axis=0)
    keys = np.sum([p["keys"] for p in out], axis=0)
    assert np.array_equal(tokens, [r["tokens"] for r in recs1])
    assert np.array_equal(keys, [r["attended_keys"] for r in recs1])
