#!/usr/bin/env python3
"""Benchmark of the paged quantized KV-cache hot path on B200.

Workload (the batch-decode configuration): 32 sequences per GPU, 16 full-attention layers, 24 query / 4 KV heads of
dim 256, q8_0 cache in 64-token pages, per-sequence context lengths uniform in [1024, 32768] (seed 0), pages drawn from
one shuffled pool so block tables are non-contiguous, fp16 K/V/q ~ N(0,1). One step = for each layer: append one new
token per sequence, then decode-attend over the whole context. Data is synthetic.

  value        KV GB/s: algorithmic cache bytes attended (sum of context lengths x 2176 B x layers) / device time of
               the K timed steps, inputs resident in HBM, whole job over all GPUs (weak scaling: 32 sequences per GPU).
  e2e          the same metric through yahkv_decode_step_host_async / _wait: per layer the step's K/V/q come from
               pinned HOST memory and every layer's attention output is back in host memory before the step ends,
               all inside the timed region.
  roofline     the split-K attention kernel alone: algorithmic bytes per launch / its mean device time, from CUDA
               event pairs the library records around every launch inside the timed region.
  cpu_baseline the CPU oracle (a port: the reference has no CPU attention) on a bounded sample of the same workload.

`--impl reference` times the CPU arm alone: the reference project's CPU code for this path is its block codec
(QuantizeQ8_0, compiled from its sources into oracle/_ref when available) plus, for attention, the oracle port that
restates its numpy checker; all host threads, bounded sample.
"""
import argparse
import json
import os
import subprocess
import sys
import tempfile
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
for p in (os.path.join(ROOT, "yet-another-halo-engine_b200"), os.path.join(ROOT, "oracle")):
    if p not in sys.path:
        sys.path.insert(0, p)

LAYERS, BATCH, CTX_LO, CTX_HI = 16, 32, 1024, 32768
N_SPLITS = 0          # split-K units per (sequence, kv head); 0 = the library's automatic choice
METRIC, UNIT = "q8_0_paged_decode_attn_kv_gbps", "GB/s"
# DRAM bytes per algorithmic byte of the split-K attention kernel, from an ncu capture of one full-size launch of this
# workload (1.238827 GB read + 11.76 MB written for 1.236479 GB of cache): profiles/decode_part_q8_0_batch32.md.
NCU_DRAM_PER_ALGORITHMIC_BYTE = {"q8_0": 1.0114}


def workload(rank, layers):
    rng = np.random.default_rng(rank)          # rank 0 = seed 0, the single-GPU configuration
    lens = rng.integers(CTX_LO, CTX_HI + 1, BATCH)
    return {"rng": rng, "lens": lens, "layers": layers}


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        d = json.load(open(path))
        return float(d["hbm_gbs"]), "measured"
    return 6650.0, "fallback"


class ClockSampler:
    """nvidia-smi clocks and throttle reasons sampled every 50 ms; started ahead of the warm-up (the tool takes a
    moment to come up) and cut to the timed region by its own timestamps."""
    Q = ("timestamp,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index):
        self.f = tempfile.NamedTemporaryFile("w+", suffix=".csv", delete=False)
        try:
            self.p = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-lms",
                                       "50", "-i", str(gpu_index)], stdout=self.f, stderr=subprocess.DEVNULL)
        except OSError:
            self.p = None

    def stop(self, t_begin=None, t_end=None):
        """t_begin / t_end: time.time() bounds of the timed region (None = keep every sample)."""
        if self.p is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.p.terminate()
        self.p.wait()
        self.f.flush()
        import datetime
        rows = []
        for r in open(self.f.name).read().strip().splitlines():
            r = r.split(", ")
            if len(r) < 9:
                continue
            try:
                ts = datetime.datetime.strptime(r[0].strip(), "%Y/%m/%d %H:%M:%S.%f").timestamp()
            except ValueError:
                ts = None
            if ts is None or t_begin is None or (t_begin - 0.05 <= ts <= t_end + 0.05):
                rows.append(r)
        os.unlink(self.f.name)
        sm = [float(r[1]) for r in rows if len(r) >= 9]
        reasons = set()
        for r in rows:
            if len(r) < 9:
                continue
            for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), r[5:9]):
                if v.strip().lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": float(np.median(sm)) if sm else None,
                "sm_max_mhz": float(rows[0][2]) if rows and len(rows[0]) >= 3 else None,
                "reasons": sorted(reasons), "samples": len(sm)}


def cpu_arm(layers_sample=1, seqs_sample=8, reps=2):
    """CPU timing of the same workload on a bounded sample: `seqs_sample` sequences of the seed-0 batch, one layer.
    Returns (attention GB/s, append Mtok/s, threads, description)."""
    import oracle as O
    w = workload(0, 1)
    rng, lens = w["rng"], w["lens"][:seqs_sample]
    pages = [(int(n) + 64) // 64 + 1 for n in lens]
    num_pages = sum(pages)
    perm = rng.permutation(num_pages).astype(np.int32)
    pool = O.PagedPool(O.FMT_Q8_0, num_pages)
    stride = max(pages)
    tables = np.zeros((len(lens), stride), np.int32)
    off = 0
    t_append, n_append = 0.0, 0
    for i, n in enumerate(lens):
        tables[i, :pages[i]] = perm[off:off + pages[i]]
        off += pages[i]
        K = rng.standard_normal((int(n), 4, 256), dtype=np.float32).astype(np.float16)
        V = rng.standard_normal((int(n), 4, 256), dtype=np.float32).astype(np.float16)
        t0 = time.perf_counter()
        pool.append(tables[i, :pages[i]], 0, K, V)      # the reference's QuantizeQ8_0 arithmetic + paged scatter
        t_append += time.perf_counter() - t0
        n_append += int(n)
    q = rng.standard_normal((len(lens), 24, 256), dtype=np.float32).astype(np.float16)
    best = float("inf")
    for _ in range(reps):
        t0 = time.perf_counter()
        pool.attend_decode_f32(tables, lens.astype(np.int32), q)
        best = min(best, time.perf_counter() - t0)
    gbs = float(lens.sum()) * 2176 / best / 1e9
    return gbs, n_append / t_append / 1e6, O.THREADS, (
        f"{seqs_sample} of {BATCH} sequences ({int(lens.sum())} cached tokens), 1 of {LAYERS} layers, best of {reps}")


def reference_arm(args, rank):
    if rank != 0:
        return
    t0 = time.perf_counter()
    vals = []
    t_steps = []
    for _ in range(max(1, min(args.steps, 3))):
        ts = time.perf_counter()
        gbs, mtok, threads, sample = cpu_arm(reps=1)
        t_steps.append(time.perf_counter() - ts)
        vals.append(gbs)
    gbs = float(np.median(vals))
    import oracle as O
    line = {
        "impl": "reference", "metric": METRIC, "value": gbs, "unit": UNIT, "n_gpus": args.gpus, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": float(np.median(t_steps)) * 1e3, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "u8", "data": "synthetic",
        "config": {"workload": "batch32_decode_16layers_q8_0_ctx1024-32768_page64", "note":
                   "CPU arm; the reference has no CPU attention, so attention is the oracle port of its numpy checker "
                   "and append is its QuantizeQ8_0 arithmetic"},
        "cpu_baseline": {"value": gbs, "unit": UNIT, "cores": threads, "kind": "port", "sample": sample,
                         "append_mtok_s": mtok, "ref_codec_built": O.have_ref()},
        "e2e": {"value": gbs, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "wall_s": time.perf_counter() - t0,
    }
    print(json.dumps(line))


def prefill_arm(args, local_rank):
    """The chunked-prefill configuration: 4 sequences with 30720 cached tokens (q8_0) each append a 2048-token chunk
    (quantize + scatter) and run causal attention of the chunk over cache + chunk; one layer per step, single GPU."""
    import torch
    import yahkv
    torch.cuda.set_device(local_rank)
    n_seq, cached, chunk = 4, 30720, 2048
    pages = (cached + chunk) // 64
    rng = np.random.default_rng(0)
    cache = yahkv.KvCache(device=local_rank, n_layers=1, num_pages=n_seq * pages + 8, fmt=yahkv.FMT_Q8_0, max_seqs=n_seq,
                          max_pages_per_seq=pages, max_batch_tokens=n_seq * chunk)
    perm = rng.permutation(n_seq * pages + 8).astype(np.int32)
    # An explicit stream: the legacy default stream's handle is 0, which the library reads as "use the context's own
    # stream", and events recorded on one stream say nothing about kernels on another.
    stream = torch.cuda.Stream()
    torch.cuda.set_stream(stream)
    sptr = stream.cuda_stream
    assert sptr != 0
    gen = torch.Generator(device="cuda").manual_seed(7)
    seqs = []
    for i in range(n_seq):
        s = cache.seq_create()
        cache.seq_set_table(s, perm[i * pages:(i + 1) * pages])
        for c0 in range(0, cached, 8192):
            n = min(8192, cached - c0)
            K = torch.randn(n, 4, 256, device="cuda", generator=gen).half()
            V = torch.randn(n, 4, 256, device="cuda", generator=gen).half()
            cache.append(0, np.full(n, s, np.int32), np.arange(c0, c0 + n), K, V, stream=sptr)
        seqs.append(s)
    kc = torch.randn(n_seq * chunk, 4, 256, device="cuda", generator=gen).half()
    vc = torch.randn(n_seq * chunk, 4, 256, device="cuda", generator=gen).half()
    q = torch.randn(n_seq * chunk, 24, 256, device="cuda", generator=gen).half()
    out = torch.zeros(n_seq * chunk, 24, 256, device="cuda", dtype=torch.float16)
    ids = np.repeat(np.array(seqs, np.int32), chunk)
    pos = np.tile(np.arange(cached, cached + chunk, dtype=np.int64), n_seq)

    def step():
        for s in seqs:
            cache.seq_set_len(s, cached)        # the same chunk is appended again each step
        cache.append(0, ids, pos, kc, vc, stream=sptr)
        cache.attend_prefill(0, seqs, [chunk] * n_seq, q, out, stream=sptr)

    for _ in range(max(args.warmup, 3)):
        step()
    torch.cuda.synchronize()
    cache.kernel_timing(True)
    sampler = ClockSampler(local_rank)
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t_begin = time.time()
    ev0.record(stream)
    for _ in range(args.steps):
        step()
    ev1.record(stream)
    torch.cuda.synchronize()
    t_end = time.time()
    ms = ev0.elapsed_time(ev1)
    clocks = sampler.stop(t_begin, t_end)
    att_ms, att_n = cache.kernel_timing_read(yahkv.KERNEL_PREFILL)
    deq_ms, deq_n = cache.kernel_timing_read(yahkv.KERNEL_PREFILL_DEQUANT)
    app_ms, app_n = cache.kernel_timing_read(yahkv.KERNEL_APPEND)
    flops = n_seq * 4 * 24 * 256 * sum(cached + i + 1 for i in range(chunk))
    peaks = json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json"))) if os.path.exists(
        os.path.join(ROOT, "MEASURED_PEAKS.json")) else {"bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}
    achieved = flops / (att_ms / max(att_n, 1) * 1e-3) / 1e12
    line = {
        "metric": "q8_0_chunked_prefill_attn_tflops", "value": flops * args.steps / (ms * 1e-3) / 1e12,
        "unit": "TFLOP/s", "n_gpus": 1, "steps": args.steps, "warmup": max(args.warmup, 3),
        "ms_per_step": ms / args.steps, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "f16", "data": "synthetic",
        "config": {"workload": "chunked_prefill_4seq_30720cached_2048chunk_q8_0_1layer",
                   "l2": "inputs larger than L2 (285 MB of cache + 537 MB fp16 scratch per step)"},
        "extra": {"attention_ms": att_ms / max(att_n, 1), "dequant_ms": deq_ms / max(deq_n, 1),
                  "append_ms": app_ms / max(app_n, 1),
                  "append_mtok_s": n_seq * chunk / (app_ms / max(app_n, 1) * 1e-3) / 1e6},
        "roofline": {"kernel": "PrefillKernel (tcgen05)", "bound": "tensor", "achieved": achieved,
                     "peak": peaks["bf16_tflops_sustained"], "unit": "TFLOP/s",
                     "frac": achieved / peaks["bf16_tflops_sustained"], "peak_kind": "of measured (sustained)",
                     "frac_of_burst": achieved / peaks["bf16_tflops"], "traffic": None},
        "gpu_launches": 3 * args.steps, "clocks": clocks,
    }
    print(json.dumps(line))
    cache.close()


def churn_arm(args, rank, local_rank, world):
    """The whole-box serving-churn configuration, scaled with the GPU count (weak scaling): 32 sequence slots per GPU
    (256 on 8 GPUs, the configuration), contexts uniform in [512, 65536], per step 30 decode tokens per GPU plus one
    1024-token prefill chunk per box, a tenth of the slots finishing and being re-admitted from the recycled page
    pool; q8_0, 64-token pages, `--layers` layers (16 = the configuration). Sequences are partitioned by slot; the only
    communication is the barrier and the max-over-ranks of the device time."""
    import torch
    import torch.distributed as dist
    import yahkv
    from yahkv.churn import ChurnRunner, ChurnSchedule, pages_needed

    torch.cuda.set_device(local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    layers = args.layers
    sched = ChurnSchedule(n_slots=32 * world, ctx_lo=512, ctx_hi=65536, n_decode=30 * world, chunk=1024,
                          finish_frac=0.1, seed=0)
    cap_pages = (sched.ctx_hi + sched.chunk + 64 + 63) // 64 + 1
    cache = yahkv.KvCache(device=local_rank, n_layers=layers, num_pages=pages_needed(sched, rank, world),
                          fmt=yahkv.FMT_Q8_0, max_seqs=40, max_pages_per_seq=cap_pages, max_batch_tokens=2048)
    runner = ChurnRunner(cache, sched, rank, world, n_layers=layers)
    stream = torch.cuda.Stream()
    torch.cuda.set_stream(stream)
    sptr = stream.cuda_stream
    gen = torch.Generator(device="cuda").manual_seed(99 + rank)
    nd = 40
    k1 = torch.randn(nd, 4, 256, device="cuda", generator=gen).half()
    v1 = torch.randn(nd, 4, 256, device="cuda", generator=gen).half()
    q1 = torch.randn(nd, 24, 256, device="cuda", generator=gen).half()
    o1 = torch.zeros(nd, 24, 256, device="cuda", dtype=torch.float16)
    kc = torch.randn(sched.chunk, 4, 256, device="cuda", generator=gen).half()
    vc = torch.randn(sched.chunk, 4, 256, device="cuda", generator=gen).half()
    qc = torch.randn(sched.chunk, 24, 256, device="cuda", generator=gen).half()
    oc = torch.zeros(sched.chunk, 24, 256, device="cuda", dtype=torch.float16)
    work = {"decode_keys": 0, "prefill_flops": 0.0}

    def gpu(kind, sids, pos):
        n = len(pos)
        if kind == "decode":
            for layer in range(layers):
                cache.append(layer, sids, pos, k1[:n], v1[:n], stream=sptr)
                cache.attend_decode(layer, sids, q1[:n], o1[:n], stream=sptr)
            work["decode_keys"] += int(pos.sum()) + n
        else:
            ids = np.full(n, sids[0], np.int32)
            for layer in range(layers):
                cache.append(layer, ids, pos, kc, vc, stream=sptr)
                cache.attend_prefill(layer, sids, [n], qc, oc, stream=sptr)
            work["prefill_flops"] += 4.0 * 24 * 256 * float((pos + 1).sum())

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    step_no = 0
    for _ in range(max(args.warmup, 3)):
        runner.step(step_no, gpu)
        step_no += 1
    barrier()
    work["decode_keys"], work["prefill_flops"] = 0, 0.0
    launches0 = cache.launch_count()
    sampler = ClockSampler(local_rank) if rank == 0 else None
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    t_begin = time.time()
    ev0.record(stream)
    tokens = 0
    for _ in range(args.steps):
        tokens += runner.step(step_no, gpu)["tokens"]
        step_no += 1
    ev1.record(stream)
    barrier()
    t_end = time.time()
    cache.sync()                       # raises if a kernel recorded an error status
    ms = ev0.elapsed_time(ev1)
    clocks = sampler.stop(t_begin, t_end) if sampler else None
    stats = torch.tensor([ms, tokens, work["decode_keys"], work["prefill_flops"], cache.launch_count() - launches0],
                         dtype=torch.float64, device="cuda")
    if world > 1:
        mx, sm = stats.clone(), stats.clone()
        dist.all_reduce(mx, op=dist.ReduceOp.MAX)
        dist.all_reduce(sm, op=dist.ReduceOp.SUM)
        ms, tokens, dkeys, pflops, launches = mx[0].item(), sm[1].item(), sm[2].item(), sm[3].item(), sm[4].item()
    else:
        tokens, dkeys, pflops, launches = stats[1].item(), stats[2].item(), stats[3].item(), stats[4].item()
    if rank == 0:
        line = {
            "metric": "serving_churn_tokens_per_s", "value": tokens / (ms * 1e-3), "unit": "tok/s", "n_gpus": world,
            "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": ms / args.steps,
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "u8", "data": "synthetic",
            "config": {"workload": f"churn_{sched.n_slots}slots_{layers}layers_q8_0_ctx512-65536_page64",
                       "slots_per_gpu": 32, "decode_tokens_per_step": sched.n_decode, "prefill_chunk": sched.chunk,
                       "finish_frac": 0.1, "note": "attention + append only; new sequences take recycled pages as "
                       "their prompt cache; sequences partitioned by slot, no collective on the data path"},
            "extra": {"decode_kv_gbps": dkeys * layers * 2176 / (ms * 1e-3) / 1e9,
                      "prefill_tflops_averaged_over_the_run": pflops * layers / (ms * 1e-3) / 1e12,
                      "pages_free_rank0": cache.pages_free(), "device_bytes_rank0": cache.device_bytes()},
            "gpu_launches": int(launches), "clocks": clocks,
        }
        print(json.dumps(line))
    cache.close()
    if world > 1:
        dist.destroy_process_group()


def headshard_arm(args, rank, local_rank, world):
    """The head-sharded layout (benchmark only): every GPU holds all 32 sequences but only 4 / world of the KV heads
    (and their query heads); after each layer's attention the ranks' output slices are joined by one NCCL all-gather.
    Strong scaling: the total work is one batch-32 step whatever the number of GPUs (1, 2 or 4)."""
    import torch
    import torch.distributed as dist
    import yahkv

    if world not in (1, 2, 4):
        if rank == 0:
            print(json.dumps({"metric": METRIC, "workload": "head_sharded", "n_gpus": world,
                              "unavailable": "4 KV heads shard at most 4 ways"}))
        return
    torch.cuda.set_device(local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    w = workload(0, args.layers)                      # the same sequences on every rank
    rng, lens, layers = w["rng"], w["lens"].copy(), w["layers"]
    hc = 4 // world
    grow = 2 * (args.warmup + args.steps) + 2
    pages = [(int(n) + grow + 63) // 64 for n in lens]
    num_pages = sum(pages) + 64
    cache = yahkv.KvCache(device=local_rank, n_layers=layers, num_pages=num_pages, fmt=yahkv.FMT_Q8_0, max_seqs=BATCH,
                          max_pages_per_seq=max(pages) + 1, max_batch_tokens=8192, kv_head_begin=rank * hc,
                          kv_head_count=hc)
    perm = rng.permutation(num_pages).astype(np.int32)
    stream = torch.cuda.Stream()
    torch.cuda.set_stream(stream)
    sptr = stream.cuda_stream
    gen = torch.Generator(device="cuda").manual_seed(1234)
    seqs, off = [], 0
    for i, n in enumerate(lens):
        s = cache.seq_create()
        cache.seq_set_table(s, perm[off:off + pages[i]])
        off += pages[i]
        seqs.append(s)
        for c0 in range(0, int(n), 8192):
            c1 = min(int(n), c0 + 8192)
            K = torch.randn(c1 - c0, 4, 256, device="cuda", generator=gen).half()
            V = torch.randn(c1 - c0, 4, 256, device="cuda", generator=gen).half()
            ids, pos = np.full(c1 - c0, s, np.int32), np.arange(c0, c1, dtype=np.int64)
            for layer in range(layers):
                cache.append(layer, ids, pos, K, V, stream=sptr)
    cache.sync()
    seq_ids = np.array(seqs, np.int32)
    k_new = torch.randn(layers, BATCH, 4, 256, device="cuda", generator=gen).half()
    v_new = torch.randn(layers, BATCH, 4, 256, device="cuda", generator=gen).half()
    q = torch.randn(layers, BATCH, 24, 256, device="cuda", generator=gen).half()
    out = torch.zeros(layers, BATCH, 24, 256, device="cuda", dtype=torch.float16)
    mine = slice(rank * hc * 6, (rank + 1) * hc * 6)
    joined = torch.zeros(world, BATCH, hc * 6, 256, device="cuda", dtype=torch.float16)

    def step(gather):
        pos = np.array([cache.seq_len(s, 0) for s in seqs], np.int64)
        for layer in range(layers):
            cache.append(layer, seq_ids, pos, k_new[layer], v_new[layer], stream=sptr)
            cache.attend_decode(layer, seq_ids, q[layer], out[layer], stream=sptr)
            if gather and world > 1:
                dist.all_gather_into_tensor(joined, out[layer][:, mine].contiguous())
        return int(pos.sum()) + BATCH

    def timed(gather):
        for _ in range(args.warmup):
            step(gather)
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(stream)
        keys = sum(step(gather) for _ in range(args.steps))
        e1.record(stream)
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1), keys

    ms_c, _ = timed(False)
    ms_g, keys = timed(True)
    stats = torch.tensor([ms_c, ms_g], dtype=torch.float64, device="cuda")
    if world > 1:
        dist.all_reduce(stats, op=dist.ReduceOp.MAX)
    ms_c, ms_g = stats[0].item(), stats[1].item()
    if rank == 0:
        bytes_all = keys * layers * yahkv.bytes_per_token(yahkv.FMT_Q8_0)     # all four KV heads, once
        peak, peak_kind = measured_peaks()
        print(json.dumps({
            "metric": METRIC, "value": bytes_all / (ms_g * 1e-3) / 1e9, "unit": UNIT, "n_gpus": world,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms_g / args.steps, "higher_is_better": True,
            "scaling": "strong", "vs_baseline": None, "dtype": "u8", "data": "synthetic",
            "config": {"workload": "batch32_decode_%dlayers_q8_0_head_sharded" % layers, "kv_heads_per_gpu": hc,
                       "sharding": "KV heads partitioned across GPUs; one NCCL all-gather of the output slices per layer"},
            "extra": {"ms_per_step_without_gather": ms_c / args.steps,
                      "gather_ms_per_step": (ms_g - ms_c) / args.steps,
                      "gathered_bytes_per_step": layers * BATCH * 24 * 256 * 2,
                      "frac_of_measured_hbm_per_gpu": bytes_all / (ms_g * 1e-3) / 1e9 / world / peak},
            "gpu_launches": 2 * 3 * layers * args.steps}))
    cache.close()
    if world > 1:
        dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=100)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="yahkv", choices=["yahkv", "reference"])
    ap.add_argument("--layers", type=int, default=LAYERS, help="layers per step (16 = the configuration)")
    ap.add_argument("--fmt", default="q8_0", choices=["q8_0", "q4_0"], help="cache format (q8_0 = the configuration)")
    ap.add_argument("--workload", default="decode", choices=["decode", "prefill", "longctx", "churn", "headshard"],
                    help="decode = the batch-32 configuration (default, the headline metric); prefill = chunked "
                         "prefill; longctx = batch 8 x 131072 tokens, q4_0, 64 splits, one layer")
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline leg")
    ap.add_argument("--no-e2e", action="store_true", help="skip the host-buffer leg")
    ap.add_argument("--no-graph", action="store_true", help="skip the captured-graph leg (value = eager calls)")
    args = ap.parse_args()
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if args.impl == "reference":
        reference_arm(args, rank)
        return
    if args.warmup < 3:
        args.warmup = 3
    if args.workload == "prefill":
        if rank == 0:
            prefill_arm(args, local_rank)
        return
    if args.workload == "churn":
        churn_arm(args, rank, local_rank, world)
        return
    if args.workload == "headshard":
        headshard_arm(args, rank, local_rank, world)
        return
    if args.workload == "longctx":
        global BATCH, CTX_LO, CTX_HI, N_SPLITS
        BATCH, CTX_LO, CTX_HI, N_SPLITS = 8, 131072, 131072, 64
        args.fmt = "q4_0"
        if args.layers == LAYERS:
            args.layers = 1

    import torch
    import torch.distributed as dist
    import yahkv

    torch.cuda.set_device(local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    w = workload(rank, args.layers)
    rng, lens, layers = w["rng"], w["lens"].copy(), w["layers"]
    total_steps = args.warmup + args.steps
    e2e_steps = 0 if args.no_e2e else min(args.steps, 4) + 1
    graph_steps = 0 if (args.no_graph or N_SPLITS) else args.steps + 3
    grow = total_steps + graph_steps + e2e_steps + 2
    pages = [(int(n) + grow + 63) // 64 for n in lens]
    num_pages = sum(pages) + 64
    fmt = yahkv.FMT_Q8_0 if args.fmt == "q8_0" else yahkv.FMT_Q4_0
    cache = yahkv.KvCache(device=local_rank, n_layers=layers, num_pages=num_pages, fmt=fmt,
                          max_seqs=BATCH, max_pages_per_seq=max(pages) + 1, max_batch_tokens=8192)
    perm = rng.permutation(num_pages).astype(np.int32)
    seqs, off = [], 0
    # An explicit stream: the legacy default stream's handle is 0, which the library reads as "use the context's own
    # stream", and events recorded on one stream say nothing about kernels on another.
    stream = torch.cuda.Stream()
    torch.cuda.set_stream(stream)
    sptr = stream.cuda_stream
    assert sptr != 0
    gen = torch.Generator(device="cuda").manual_seed(1234 + rank)
    for i, n in enumerate(lens):
        s = cache.seq_create()
        cache.seq_set_table(s, perm[off:off + pages[i]])
        off += pages[i]
        seqs.append(s)
        for c0 in range(0, int(n), 8192):
            c1 = min(int(n), c0 + 8192)
            K = torch.randn(c1 - c0, 4, 256, device="cuda", generator=gen).half()
            V = torch.randn(c1 - c0, 4, 256, device="cuda", generator=gen).half()
            ids, pos = np.full(c1 - c0, s, np.int32), np.arange(c0, c1, dtype=np.int64)
            for layer in range(layers):
                cache.append(layer, ids, pos, K, V, stream=sptr)
    cache.sync()

    seq_ids = np.array(seqs, np.int32)
    k_new = torch.randn(layers, BATCH, 4, 256, device="cuda", generator=gen).half()
    v_new = torch.randn(layers, BATCH, 4, 256, device="cuda", generator=gen).half()
    q = torch.randn(layers, BATCH, 24, 256, device="cuda", generator=gen).half()
    out = torch.zeros(layers, BATCH, 24, 256, device="cuda", dtype=torch.float16)

    def step():
        pos = np.array([cache.seq_len(s, 0) for s in seqs], np.int64)
        for layer in range(layers):
            cache.append(layer, seq_ids, pos, k_new[layer], v_new[layer], stream=sptr)
            cache.attend_decode(layer, seq_ids, q[layer], out[layer], n_splits=N_SPLITS, stream=sptr)
        return int(pos.sum()) + BATCH            # keys attended per layer in this step

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    sampler = ClockSampler(local_rank) if rank == 0 else None
    for _ in range(args.warmup):
        step()
    barrier()
    cache.kernel_timing(True)
    launches0 = cache.launch_count()
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    t_begin = time.time()
    ev0.record(stream)
    keys = 0
    for _ in range(args.steps):
        keys += step()
    ev1.record(stream)
    barrier()
    t_end = time.time()
    ms = ev0.elapsed_time(ev1)
    clocks = sampler.stop(t_begin, t_end) if sampler else None
    launches = cache.launch_count() - launches0
    part_ms, part_n = cache.kernel_timing_read(yahkv.KERNEL_DECODE_PART)
    comb_ms, comb_n = cache.kernel_timing_read(yahkv.KERNEL_DECODE_COMBINE)
    app_ms, app_n = cache.kernel_timing_read(yahkv.KERNEL_APPEND)
    cache.kernel_timing(False)
    bytes_attended = keys * layers * yahkv.bytes_per_token(fmt)

    # ---- the same steps as one captured CUDA graph per step (device-resident lengths, no host planning) ----
    g_ms = g_bytes = None
    if graph_steps:
        batch = yahkv.DecodeBatch(cache, seq_ids)
        batch.prepare(graph_steps, stream=sptr)
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=stream):
            cs = torch.cuda.current_stream().cuda_stream
            batch.plan(stream=cs)
            for layer in range(layers):
                batch.decode_layer(layer, k_new[layer], v_new[layer], q[layer], out[layer], stream=cs)
            batch.advance(stream=cs)
        lens_now = sum(cache.seq_len(s, 0) for s in seqs)
        for _ in range(3):
            graph.replay()
        barrier()
        g0, g1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        g0.record(stream)
        for _ in range(args.steps):
            graph.replay()
        g1.record(stream)
        barrier()
        g_ms = g0.elapsed_time(g1)
        g_keys = sum(lens_now + BATCH * (3 + i) + BATCH for i in range(args.steps))
        g_bytes = g_keys * layers * yahkv.bytes_per_token(fmt)
        batch.commit(graph_steps)
        cache.sync()
        batch.close()

    # ---- end to end through the host-buffer entry point ----
    e2e = None
    if not args.no_e2e:
        hk = k_new.cpu().pin_memory()
        hv = v_new.cpu().pin_memory()
        hq = q.cpu().pin_memory()
        hout = torch.zeros(layers, BATCH, 24, 256, dtype=torch.float16).pin_memory()

        def host_step():
            n = sum(cache.seq_len(s, 0) for s in seqs) + BATCH
            for layer in range(layers):   # queued back to back; the copies overlap the previous layer's kernels
                cache.decode_step_host_async(layer, seq_ids, hk[layer], hv[layer], hq[layer], hout[layer])
            cache.decode_step_host_wait()   # the step's outputs are in host memory
            return n
        host_step()
        barrier()
        t0 = time.perf_counter()
        e_keys = 0
        for _ in range(e2e_steps - 1):
            e_keys += host_step()
        torch.cuda.synchronize()
        e_s = time.perf_counter() - t0
        e_bytes = e_keys * layers * yahkv.bytes_per_token(fmt)
        e2e = {"bytes": e_bytes, "s": e_s,
               "h2d": layers * BATCH * (2 * 4 * 256 * 2 + 24 * 256 * 2), "d2h": layers * BATCH * 24 * 256 * 2}

    # ---- aggregate over ranks: bytes summed, time = max ----
    stats = torch.tensor([ms, bytes_attended, e2e["s"] if e2e else 0.0, e2e["bytes"] if e2e else 0.0,
                          part_ms / max(part_n, 1), g_ms or 0.0, g_bytes or 0.0], dtype=torch.float64, device="cuda")
    if world > 1:
        mx = stats.clone()
        dist.all_reduce(mx, op=dist.ReduceOp.MAX)
        sm = stats.clone()
        dist.all_reduce(sm, op=dist.ReduceOp.SUM)
        ms, bytes_all, e_s, e_bytes_all = mx[0].item(), sm[1].item(), mx[2].item(), sm[3].item()
        g_ms_all, g_bytes_all = mx[5].item(), sm[6].item()
    else:
        bytes_all, e_s, e_bytes_all = bytes_attended, stats[2].item(), stats[3].item()
        g_ms_all, g_bytes_all = stats[5].item(), stats[6].item()
    # headline: the captured-graph steps when they ran (the fastest way the public API offers), else the eager calls
    eager_value, eager_ms_per_step = bytes_all / (ms * 1e-3) / 1e9, ms / args.steps
    use_graph = g_ms_all > 0
    if use_graph:
        ms, bytes_all = g_ms_all, g_bytes_all
    if rank == 0:
        peak, peak_kind = measured_peaks()
        part_bytes = bytes_attended / max(part_n, 1)
        part_mean_ms = part_ms / max(part_n, 1)
        achieved = part_bytes / (part_mean_ms * 1e-3) / 1e9 if part_n else 0.0
        line = {
            "metric": METRIC if args.fmt == "q8_0" else METRIC.replace("q8_0", args.fmt),
            "value": bytes_all / (ms * 1e-3) / 1e9, "unit": UNIT, "n_gpus": world,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms / args.steps, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "u8", "data": "synthetic",
            "config": {"workload": f"batch{BATCH}_decode_{layers}layers_{args.fmt}_ctx{CTX_LO}-{CTX_HI}_page64",
                       "seqs_per_gpu": BATCH, "n_splits": N_SPLITS,
                       "layers": layers, "mean_ctx": float(lens.mean()), "pages_shuffled": True,
                       "l2": "inputs larger than L2: each layer reads its own ~1.2 GB of cache per step",
                       "sharding": "sequences partitioned across GPUs, no collective on the data path"},
            "extra": {"step_mode": "one captured CUDA graph per 16-layer step (yahkv_batch_*)" if use_graph
                      else "eager per-layer calls (yahkv_append + yahkv_attend_decode)",
                      "eager_value": eager_value, "eager_ms_per_step": eager_ms_per_step,
                      "append_mtok_s": (app_n * BATCH) / (app_ms * 1e-3) / 1e6 if app_n else None,
                      "append_us_per_launch": app_ms / max(app_n, 1) * 1e3,
                      "batch_decode_tok_s": world * BATCH * args.steps / (ms * 1e-3),
                      "batch_decode_note": "attention + append of 16 layers only; the rest of the model is out of scope",
                      "combine_us_per_launch": comb_ms / max(comb_n, 1) * 1e3,
                      "frac_of_nominal_8000": bytes_all / (ms * 1e-3) / 1e9 / world / 8000.0,
                      "device_bytes": cache.device_bytes()},
            "roofline": {"kernel": f"DecodePartKernel<{args.fmt}>", "bound": "hbm", "achieved": achieved, "peak": peak,
                         "unit": "GB/s", "frac": achieved / peak, "peak_kind": f"of {peak_kind}",
                         "launches": part_n, "mean_us": part_mean_ms * 1e3, "traffic": None},
            "gpu_launches": (2 + 3 * layers) * args.steps if use_graph else launches, "clocks": clocks,
        }
        if e2e:
            line["e2e"] = {"value": e_bytes_all / e_s / 1e9, "unit": UNIT, "h2d_bytes_per_step": e2e["h2d"],
                           "d2h_bytes_per_step": e2e["d2h"], "steps": e2e_steps - 1,
                           "api": "yahkv_decode_step_host_async per layer + yahkv_decode_step_host_wait per step (pinned host K/V/q in, outputs back in host memory before the step ends)"}
        if args.fmt in NCU_DRAM_PER_ALGORITHMIC_BYTE:
            line["roofline"]["traffic"] = NCU_DRAM_PER_ALGORITHMIC_BYTE[args.fmt] * part_bytes
            line["roofline"]["traffic_note"] = ("(dram__bytes_read.sum + dram__bytes_write.sum) / algorithmic bytes of "
                                                "one ncu-captured launch of this workload, times this run's bytes "
                                                "per launch")
        if world == 1 and not args.no_cpu:
            gbs, mtok, threads, sample = cpu_arm()
            line["cpu_baseline"] = {"value": gbs, "unit": UNIT, "cores": threads, "kind": "port", "sample": sample,
                                    "append_mtok_s": mtok}
        print(json.dumps(line))
    cache.close()
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
