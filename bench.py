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
  parity       before anything is timed, sampled outputs of the workload are compared with the float64 oracle over the
               bytes the cache holds (read back through the C ABI), and the step's appended tokens with the oracle's
               quantizer; the line carries "parity_checked" and the errors, and a run whose check fails prints no number.

With N GPUs the N x 32 contexts are drawn from one seed-0 stream (the first 32 are the single-GPU batch) and dealt to
the ranks longest first, each to the rank with the least tokens so far, 32 per rank, so the ranks' work is balanced
and the aggregate measures the library rather than the draw.

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
# q4_0: the long-context launch (1.2094 GB + 22.8 MB for 1.2080 GB), profiles/decode_longctx_q4_0.md; kv8a16: the
# batch-32 launch (1.3311 GB + 14.8 MB for 1.3271 GB), profiles/decode_part_kv8a16_batch32.md.
NCU_DRAM_PER_ALGORITHMIC_BYTE = {"q8_0": 1.0114, "q4_0": 1.0200, "kv8a16": 1.0142}
# kv4a16: the batch-32 launch (803.0 MB + 14.9 MB for 0.800 GB), profiles/decode_part_kv4a16_batch32.md.
NCU_DRAM_PER_ALGORITHMIC_BYTE["kv4a16"] = 1.0224
# The prefill kernel's DRAM bytes per launch of the chunked-prefill workload (5.920 GB read + 0.101 GB written: the fp16
# scratch is streamed once per wave of query tiles), profiles/prefill_q8_0_chunk2048.md.
NCU_DRAM_BYTES_PREFILL_LAUNCH = 6.021e9


def workload(rank, world, layers):
    """Context lengths of this rank: world x BATCH draws from the seed-0 stream (its first BATCH values are the
    single-GPU batch), dealt longest first to the rank with the fewest tokens so far, BATCH per rank."""
    rng = np.random.default_rng(0)
    all_lens = rng.integers(CTX_LO, CTX_HI + 1, BATCH * world)
    if world == 1:
        return {"rng": rng, "lens": all_lens, "layers": layers, "all_rank_tokens": [int(all_lens.sum())]}
    load, count, mine = [0] * world, [0] * world, [[] for _ in range(world)]
    for n in sorted((int(x) for x in all_lens), reverse=True):
        r = min((i for i in range(world) if count[i] < BATCH), key=lambda i: (load[i], i))
        load[r] += n
        count[r] += 1
        mine[r].append(n)
    return {"rng": np.random.default_rng([0, rank]), "lens": np.array(mine[rank], dtype=np.int64), "layers": layers,
            "all_rank_tokens": load}


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        d = json.load(open(path))
        return float(d["hbm_gbs"]), "measured"
    return 6650.0, "fallback"


class ClockSampler:
    """SM clock and throttle reasons of one GPU during the timed region. Read in-process through NVML (the library
    nvidia-smi itself reads) every 5 ms by a thread, so that even a region of a few tens of milliseconds holds samples;
    where the NVML binding is missing, `nvidia-smi -lms 50` in a child process stands in. Reading only: nothing is
    set. Samples are cut to the timed region by their own time stamps."""
    Q = ("timestamp,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")
    REASON_BITS = (("hw_slowdown", 0x8), ("hw_thermal_slowdown", 0x40), ("sw_thermal_slowdown", 0x20), ("sw_power_cap", 0x4))

    def __init__(self, gpu_index):
        self.samples, self.max_mhz, self.thread, self.p, self.halt = [], None, None, None, False
        try:
            import threading
            import pynvml
            pynvml.nvmlInit()
            try:     # the device this process computes on, whatever CUDA_VISIBLE_DEVICES did to the numbering
                uuid = str(torch.cuda.get_device_properties(gpu_index).uuid)
                handle = pynvml.nvmlDeviceGetHandleByUUID(("GPU-" + uuid) if not uuid.startswith("GPU-") else uuid)
            except Exception:
                handle = pynvml.nvmlDeviceGetHandleByIndex(gpu_index)
            self.max_mhz = float(pynvml.nvmlDeviceGetMaxClockInfo(handle, pynvml.NVML_CLOCK_SM))

            def loop():
                while not self.halt:
                    try:
                        mhz = pynvml.nvmlDeviceGetClockInfo(handle, pynvml.NVML_CLOCK_SM)
                        bits = pynvml.nvmlDeviceGetCurrentClocksEventReasons(handle)
                        self.samples.append((time.time(), float(mhz), int(bits)))
                    except Exception:
                        pass
                    time.sleep(0.005)
            self.thread = threading.Thread(target=loop, daemon=True)
            self.thread.start()
            return
        except Exception:
            self.thread = None
        self.f = tempfile.NamedTemporaryFile("w+", suffix=".csv", delete=False)
        try:
            self.p = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-lms",
                                       "50", "-i", str(gpu_index)], stdout=self.f, stderr=subprocess.DEVNULL)
        except OSError:
            self.p = None

    def stop(self, t_begin=None, t_end=None):
        """t_begin / t_end: time.time() bounds of the timed region (None = keep every sample)."""
        if self.thread is not None:
            self.halt = True
            self.thread.join(timeout=1.0)
            rows, widened = [], None
            for pad in (0.0, 0.1, 0.5):      # a very short region may fall between two samples: then its surroundings
                rows = [r for r in self.samples if t_begin is None or t_begin - pad <= r[0] <= t_end + pad]
                if rows or t_begin is None:
                    widened = pad if pad > 0 else None
                    break
            reasons = sorted({name for _, _, bits in rows for name, bit in self.REASON_BITS if bits & bit})
            return {"sm_mhz": float(np.median([r[1] for r in rows])) if rows else None, "sm_max_mhz": self.max_mhz,
                    "reasons": reasons, "samples": len(rows), "source": "nvml, every 5 ms",
                    **({"window": f"timed region widened by {widened} s on both sides to catch samples"} if widened else {})}
        if self.p is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.p.terminate()
        self.p.wait()
        self.f.flush()
        import datetime
        stamped = []
        for r in open(self.f.name).read().strip().splitlines():
            r = r.split(", ")
            if len(r) < 9:
                continue
            try:
                ts = datetime.datetime.strptime(r[0].strip(), "%Y/%m/%d %H:%M:%S.%f").timestamp()
            except ValueError:
                ts = None
            stamped.append((ts, r))
        # A timed region shorter than a few sampling periods may catch no sample: then the samples just around it
        # (the warm-up before, the end-to-end leg after: the same kernels under the same load) stand in, and the
        # line says so.
        pad = 0.05
        for pad in (0.05, 0.3, 1.0):
            rows = [r for ts, r in stamped if ts is None or t_begin is None or (t_begin - pad <= ts <= t_end + pad)]
            if len(rows) >= 2 or t_begin is None:
                break
        widened = pad if (t_begin is not None and pad > 0.05) else None
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
                "reasons": sorted(reasons), "samples": len(sm), "source": "nvidia-smi -lms 50",
                **({"window": f"timed region widened by {widened} s on both sides to catch samples"} if widened else {})}


def cpu_pool(lens, fmt, rng):
    """Oracle pool holding `lens` tokens per sequence of N(0,1) fp16 K/V behind shuffled tables. Returns (pool,
    tables, seconds spent quantizing, tokens, K rows of the first sequence for the codec timing)."""
    import oracle as O
    pages = [(int(n) + 64) // 64 + 1 for n in lens]
    num_pages = sum(pages)
    perm = rng.permutation(num_pages).astype(np.int32)
    pool = O.PagedPool(fmt, num_pages)
    tables = np.zeros((len(lens), max(pages)), np.int32)
    off, t_append, n_append, first = 0, 0.0, 0, None
    for i, n in enumerate(lens):
        tables[i, :pages[i]] = perm[off:off + pages[i]]
        off += pages[i]
        for c0 in range(0, int(n), 16384):
            c1 = min(int(n), c0 + 16384)
            K = rng.standard_normal((c1 - c0, 4, 256), dtype=np.float32).astype(np.float16)
            V = rng.standard_normal((c1 - c0, 4, 256), dtype=np.float32).astype(np.float16)
            t0 = time.perf_counter()
            pool.append(tables[i, :pages[i]], c0, K, V)      # the reference's QuantizeQ8_0 arithmetic + paged scatter
            t_append += time.perf_counter() - t0
            n_append += c1 - c0
            if first is None:
                first = K
    return pool, tables, t_append, n_append, first


def cpu_arm(fmt_name="q8_0", lens=None, reps=2, pool_cache=None):
    """CPU timing of a bounded sample of the decode workload: by default 8 sequences of the seed-0 batch, one layer.
    Returns a dict: attention GB/s, append Mtok/s (oracle port and, when built, the reference's own QuantizeQ8_0),
    threads, the sample's description, seconds of the best attention pass."""
    import oracle as O
    fmt = O.FMT_Q8_0 if fmt_name == "q8_0" else O.FMT_Q4_0
    if lens is None:
        lens = workload(0, 1, 1)["lens"][:8]
        what = f"8 of {BATCH} sequences"
    else:
        what = f"{len(lens)} sequence(s)"
    lens = np.asarray(lens)
    if pool_cache is not None and "pool" in pool_cache:
        pool, tables, t_app, n_app, first = pool_cache["pool"]
    else:
        pool, tables, t_app, n_app, first = cpu_pool(lens, fmt, np.random.default_rng(5))
        if pool_cache is not None:
            pool_cache["pool"] = (pool, tables, t_app, n_app, first)
    q = np.random.default_rng(6).standard_normal((len(lens), 24, 256), dtype=np.float32).astype(np.float16)
    best = float("inf")
    for _ in range(reps):
        t0 = time.perf_counter()
        pool.attend_decode_f32(tables, lens.astype(np.int32), q)
        best = min(best, time.perf_counter() - t0)
    bpt = 2176 if fmt_name == "q8_0" else 1152
    res = {"gbs": float(lens.sum()) * bpt / best / 1e9, "append_mtok_s_port": n_app / t_app / 1e6,
           "threads": O.THREADS, "pass_s": best,
           "sample": f"{what} ({int(lens.sum())} cached tokens, {fmt_name}), 1 layer, best of {reps}"}
    if fmt_name == "q8_0" and O.have_ref():   # the reference's own codec, compiled from its sources, single thread
        x = first.astype(np.float32)
        t0 = time.perf_counter()
        O.ref_quantize_q8_0(x)
        res["append_mtok_s_reference_codec_1thread"] = x.shape[0] / 2 / (time.perf_counter() - t0) / 1e6
    return res


def cpu_parity_fixture():
    """The single-sequence parity fixture timed on the CPU in full: 4096 single-token appends through a permuted
    table, then one decode step at position 4095 (oracle port)."""
    import oracle as O
    rng = np.random.default_rng(0)
    n, num_pages = 4096, 64
    K = rng.standard_normal((n, 4, 256), dtype=np.float32).astype(np.float16)
    V = rng.standard_normal((n, 4, 256), dtype=np.float32).astype(np.float16)
    table = rng.permutation(num_pages).astype(np.int32)
    q = rng.standard_normal((1, 24, 256), dtype=np.float32).astype(np.float16)
    pool = O.PagedPool(O.FMT_Q8_0, num_pages)
    t0 = time.perf_counter()
    for p in range(n):
        pool.append(table, p, K[p:p + 1], V[p:p + 1], threads=1)
    t_app = time.perf_counter() - t0
    t0 = time.perf_counter()
    pool.attend_decode_f32(table[None], np.array([n], np.int32), q)
    t_att = time.perf_counter() - t0
    return {"workload": "parity fixture: 1 sequence, 4096 single-token appends + 1 decode step, q8_0",
            "append_ms_4096_calls": t_app * 1e3, "attend_ms": t_att * 1e3, "attend_gbs": n * 2176 / t_att / 1e9}


def reference_arm(args, rank):
    """The CPU arm alone. A step is one attention pass over the sample (its pool is built once, outside the steps)."""
    if rank != 0:
        return
    import oracle as O
    t0 = time.perf_counter()
    steps = max(1, min(args.steps, 20))
    warm = max(1, min(args.warmup, 2))
    cache = {}
    cpu_arm(reps=warm, pool_cache=cache)
    passes = [cpu_arm(reps=1, pool_cache=cache) for _ in range(steps)]
    res = passes[0]
    pass_s = float(np.median([p["pass_s"] for p in passes]))
    gbs = res["gbs"] * res["pass_s"] / pass_s
    line = {
        "impl": "reference", "metric": METRIC, "value": gbs, "unit": UNIT, "n_gpus": args.gpus, "steps": steps,
        "warmup": warm, "ms_per_step": pass_s * 1e3, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "u8", "data": "synthetic",
        "config": {"workload": "batch32_decode_16layers_q8_0_ctx1024-32768_page64", "note":
                   "CPU arm; the reference has no CPU attention, so attention is the oracle port of its numpy checker "
                   "and append is its QuantizeQ8_0 arithmetic; a step is one attention pass over the stated sample, "
                   "steps and warmup are what ran (at most 20 and 2)"},
        "cpu_baseline": {"value": gbs, "unit": UNIT, "cores": res["threads"], "kind": "port", "sample": res["sample"],
                         "append_mtok_s": res["append_mtok_s_port"],
                         "append_mtok_s_reference_codec_1thread": res.get("append_mtok_s_reference_codec_1thread"),
                         "ref_codec_built": O.have_ref(), "parity_fixture": cpu_parity_fixture()},
        "e2e": {"value": gbs, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "wall_s": time.perf_counter() - t0,
    }
    print(json.dumps(line))


def prefill_arm(args, local_rank):
    """The chunked-prefill configuration: 4 sequences with 30720 cached tokens (q8_0) each append a 2048-token chunk
    (quantize + scatter) and run causal attention of the chunk over cache + chunk; one layer per step, single GPU.
    value: attention TFLOP/s of the whole step with the chunk resident in HBM; e2e: the same step with the chunk's
    K/V/q coming from pinned host memory and the attention output copied back to it, inside the timed region."""
    import torch
    import yahkv
    torch.cuda.set_device(local_rank)
    n_seq, cached, chunk = 4, 30720, 2048
    pages = (cached + chunk) // 64
    rng = np.random.default_rng(0)
    cache = yahkv.KvCache(device=local_rank, n_layers=1, num_pages=n_seq * pages + 8, fmt=yahkv.FMT_Q8_0, max_seqs=n_seq,
                          max_pages_per_seq=pages, max_batch_tokens=n_seq * chunk, max_prefill_keys=n_seq * pages * 64)
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

    def step(k=kc, v=vc, qq=q):
        for s in seqs:
            cache.seq_set_len(s, cached)        # the same chunk is appended again each step
        cache.append(0, ids, pos, k, v, stream=sptr)
        cache.attend_prefill(0, seqs, [chunk] * n_seq, qq, out, stream=sptr)

    sampler = ClockSampler(local_rank)   # ahead of the warm-up: the timed region is only tens of milliseconds long
    warm = max(args.warmup, 3)
    for _ in range(warm):
        step()
    torch.cuda.synchronize()
    parity = None
    if not args.no_parity:
        import parity_probe as P
        i = 1                                   # rows of the second sequence: first, tile edge, interior, last
        rows = [0, 127, 128, 1333, 2047]
        e, r, slack = P.check_prefill_rows(cache, 0, seqs[i], cached, q[i * chunk:(i + 1) * chunk].cpu().numpy(),
                                           out[i * chunk:(i + 1) * chunk].cpu().numpy(), rows, out_is_f16=True)
        ok = e <= P.ABS_TOL + slack and P.check_appended_token(cache, 0, seqs[i], cached + 5,
                                                               kc[i * chunk + 5].cpu().numpy(), vc[i * chunk + 5].cpu().numpy())
        parity = {"ok": bool(ok), "max_abs_err": e, "max_rel_err": r, "rows": len(rows),
                  "against": "float64 oracle over the cache bytes read back through the C ABI; outputs are fp16"}
        if not ok:
            raise SystemExit(f"parity check failed before timing: {parity}")
    cache.kernel_timing(True)
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
    cache.kernel_timing(False)
    flops = n_seq * 4 * 24 * 256 * sum(cached + i + 1 for i in range(chunk))

    # ---- end to end: the chunk comes from pinned host memory, the output goes back to it ----
    hk, hv, hq = kc.cpu().pin_memory(), vc.cpu().pin_memory(), q.cpu().pin_memory()
    hout = torch.zeros(n_seq * chunk, 24, 256, dtype=torch.float16).pin_memory()
    dk, dv, dq = torch.empty_like(kc), torch.empty_like(vc), torch.empty_like(q)

    # One sequence at a time, three streams: while sequence i is appended and attended, the chunk of sequence i + 1
    # comes in and the output of sequence i - 1 goes out. Events order every buffer slice between the streams, also
    # across steps (a slice is not overwritten before its last reader is done).
    s_in, s_out = torch.cuda.Stream(), torch.cuda.Stream()
    ev_in = [torch.cuda.Event() for _ in range(n_seq)]
    ev_done = [torch.cuda.Event() for _ in range(n_seq)]
    ev_back = [torch.cuda.Event() for _ in range(n_seq)]
    ids_1, pos_1 = ids[:chunk].copy(), pos[:chunk].copy()

    def host_step(first):
        for i, sq in enumerate(seqs):
            sl = slice(i * chunk, (i + 1) * chunk)
            with torch.cuda.stream(s_in):
                if not first:
                    s_in.wait_event(ev_done[i])        # the previous step's kernels have read this slice
                dk[sl].copy_(hk[sl], non_blocking=True), dv[sl].copy_(hv[sl], non_blocking=True)
                dq[sl].copy_(hq[sl], non_blocking=True)
                ev_in[i].record(s_in)
            stream.wait_event(ev_in[i])
            if not first:
                stream.wait_event(ev_back[i])          # the previous step's output slice is back on the host
            cache.seq_set_len(sq, cached)
            ids_1[:] = sq
            cache.append(0, ids_1, pos_1, dk[sl], dv[sl], stream=sptr)
            cache.attend_prefill(0, [sq], [chunk], dq[sl], out[sl], stream=sptr)
            ev_done[i].record(stream)
            with torch.cuda.stream(s_out):
                s_out.wait_event(ev_done[i])
                hout[sl].copy_(out[sl], non_blocking=True)
                ev_back[i].record(s_out)
    out_device_leg = out.float().cpu()
    host_step(True)
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    for _ in range(args.steps):
        host_step(False)
    torch.cuda.synchronize()
    e_s = time.perf_counter() - t0

    peaks = json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json"))) if os.path.exists(
        os.path.join(ROOT, "MEASURED_PEAKS.json")) else {"bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0,
                                                         "sm_max_mhz": 1965.0}
    peak_kind = "measured" if os.path.exists(os.path.join(ROOT, "MEASURED_PEAKS.json")) else "fallback"
    achieved = flops / (att_ms / max(att_n, 1) * 1e-3) / 1e12
    # The burst peak was taken at the top SM clock; inside this seconds-long tensor-bound step the part runs power
    # capped, so the peak the kernel could reach is the burst figure scaled by the clock sampled during the run.
    sm_mhz = clocks.get("sm_mhz") or peaks.get("sm_max_mhz", 1965.0)
    peak_at_clock = peaks["bf16_tflops"] * sm_mhz / peaks.get("sm_max_mhz", 1965.0)
    line = {
        "metric": "q8_0_chunked_prefill_attn_tflops", "value": flops * args.steps / (ms * 1e-3) / 1e12,
        "unit": "TFLOP/s", "n_gpus": 1, "steps": args.steps, "warmup": warm,
        "ms_per_step": ms / args.steps, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "f16", "data": "synthetic",
        "config": {"workload": "chunked_prefill_4seq_30720cached_2048chunk_q8_0_1layer",
                   "l2": "inputs larger than L2 (285 MB of cache + 537 MB fp16 scratch per step)"},
        "extra": {"attention_ms": att_ms / max(att_n, 1), "dequant_ms": deq_ms / max(deq_n, 1),
                  "append_ms": app_ms / max(app_n, 1),
                  "append_mtok_s": n_seq * chunk / (app_ms / max(app_n, 1) * 1e-3) / 1e6},
        "roofline": {"kernel": "PrefillKernel (tcgen05)", "bound": "tensor", "achieved": achieved,
                     "peak": peak_at_clock, "unit": "TFLOP/s", "frac": achieved / peak_at_clock,
                     "peak_kind": f"of {peak_kind}: burst bf16 peak x (median SM MHz in the run / max SM MHz)",
                     "frac_of_burst": achieved / peaks["bf16_tflops"],
                     "frac_of_sustained": achieved / peaks["bf16_tflops_sustained"],
                     "traffic": NCU_DRAM_BYTES_PREFILL_LAUNCH,
                     "traffic_note": "dram__bytes_read.sum + dram__bytes_write.sum of one ncu-captured launch of this "
                                     "workload; the kernel is tensor-bound, its algorithmic unit is the flop"},
        "e2e": {"value": flops * args.steps / e_s / 1e12, "unit": "TFLOP/s",
                "h2d_bytes_per_step": n_seq * chunk * (2 * 4 * 256 + 24 * 256) * 2,
                "d2h_bytes_per_step": n_seq * chunk * 24 * 256 * 2, "steps": args.steps,
                "api": "per sequence: pinned host chunk -> cudaMemcpyAsync -> yahkv_append + yahkv_attend_prefill -> "
                       "output back to pinned host memory; copies in, kernels and copies out on three streams "
                       "ordered by events, all inside the timed region",
                "max_abs_diff_to_device_leg": float((hout.float() - out_device_leg).abs().max())},
        "gpu_launches": 3 * args.steps, "clocks": clocks,
    }
    if parity is not None:
        line["parity_checked"], line["parity"] = parity["ok"], parity
    if not args.no_cpu:
        # CPU port on a bounded sample: the float64 oracle over 16 query rows of one sequence
        import parity_probe as P
        pool, table = P.compact_pool(cache, 0, seqs[0], cached + chunk)
        rows = list(range(0, chunk, chunk // 16))[:16]
        qh = q[:chunk].cpu().numpy()
        t0 = time.perf_counter()
        for r in rows:
            pool.attend_prefill_f64(table, cached, qh, q_begin=r, q_end=r + 1)
        dt = time.perf_counter() - t0
        cf = 4 * 24 * 256 * sum(cached + r + 1 for r in rows)
        import oracle as O
        line["cpu_baseline"] = {"value": cf / dt / 1e12, "unit": "TFLOP/s", "cores": O.THREADS, "kind": "port",
                                "sample": "16 of 8192 query rows of the chunk (one sequence), float64 oracle, each "
                                          "call dequantizes the sequence's 32768 keys first"}
    print(json.dumps(line))
    cache.close()


def churn_arm(args, rank, local_rank, world):
    """The whole-box serving-churn configuration, scaled with the GPU count (weak scaling): 32 sequence slots per GPU
    (256 on 8 GPUs, the configuration), contexts uniform in [512, 65536], per step 30 decode tokens per GPU plus one
    1024-token prefill chunk per box, a tenth of the slots finishing and being re-admitted from the recycled page
    pool; q8_0, 64-token pages, `--layers` layers (16 = the configuration). Sequences are partitioned by slot; the only
    communication is the barrier and the max-over-ranks of the device time. Before the timed steps, two probed steps
    refill one decode slot and the prefill slot with real K/V on one layer and compare their outputs with the float64
    oracle."""
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
                          fmt=yahkv.FMT_Q8_0, max_seqs=40, max_pages_per_seq=cap_pages, max_batch_tokens=2048,
                          max_prefill_keys=cap_pages * 64)      # the prefill scratch is allocated once, up front
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
    host = {}                                 # pinned host copies for the end-to-end leg
    work = {"decode_keys": 0, "prefill_flops": 0.0, "h2d": 0, "d2h": 0}
    probe, probe_layer = None, min(1, layers - 1)

    def gpu(kind, sids, pos):
        n = len(pos)
        if kind == "decode":
            for layer in range(layers):
                if host:
                    k1[:n].copy_(host["k1"][:n], non_blocking=True), v1[:n].copy_(host["v1"][:n], non_blocking=True)
                    q1[:n].copy_(host["q1"][:n], non_blocking=True)
                cache.append(layer, sids, pos, k1[:n], v1[:n], stream=sptr)
                cache.attend_decode(layer, sids, q1[:n], o1[:n], stream=sptr)
                if host:
                    host["o1"][:n].copy_(o1[:n], non_blocking=True)
                    work["h2d"] += n * (2 * 4 + 24) * 256 * 2
                    work["d2h"] += n * 24 * 256 * 2
                if probe is not None and layer == probe_layer and probe.decode_slot is not None:
                    import parity_probe as P
                    cache.sync()
                    i = list(sids).index(runner.seq[probe.decode_slot])
                    probe.record(*P.check_decode_row(cache, layer, sids[i], int(pos[i]) + 1, q1[i].cpu().numpy(),
                                                     o1[i].cpu().numpy(), out_is_f16=True))
            work["decode_keys"] += int(pos.sum()) + n
        else:
            ids = np.full(n, sids[0], np.int32)
            for layer in range(layers):
                if host:
                    kc.copy_(host["kc"], non_blocking=True), vc.copy_(host["vc"], non_blocking=True)
                    qc.copy_(host["qc"], non_blocking=True)
                cache.append(layer, ids, pos, kc, vc, stream=sptr)
                cache.attend_prefill(layer, sids, [n], qc, oc, stream=sptr)
                if host:
                    host["oc"].copy_(oc, non_blocking=True)
                    work["h2d"] += n * (2 * 4 + 24) * 256 * 2
                    work["d2h"] += n * 24 * 256 * 2
                if probe is not None and layer == probe_layer and probe.prefill_slot is not None:
                    import parity_probe as P
                    cache.sync()
                    probe.record(*P.check_prefill_rows(cache, layer, sids[0], int(pos[0]), qc.cpu().numpy(),
                                                       oc.cpu().numpy(), [0, 127, 128, n - 1], out_is_f16=True))
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
    parity = None
    if not args.no_parity:
        import parity_probe as P
        probe = P.ChurnProbe(runner, probe_layer, seed=21, fill_chunk=2048)

        def to_dev(a):
            t = torch.from_numpy(a).cuda()
            torch.cuda.synchronize()
            return t
        for _ in range(2):
            probe.arm(step_no, to_dev)
            runner.step(step_no, gpu)
            step_no += 1
        cache.sync()
        pe = torch.tensor([probe.worst, probe.worst_rel, float(probe.checks)], dtype=torch.float64, device="cuda")
        if world > 1:
            mx = pe.clone()
            dist.all_reduce(mx, op=dist.ReduceOp.MAX)
            dist.all_reduce(pe, op=dist.ReduceOp.SUM)
            pe[0], pe[1] = mx[0], mx[1]
        parity = {"ok": bool(pe[0].item() <= P.ABS_TOL and pe[2].item() >= 1), "max_abs_err": pe[0].item(),
                  "max_rel_err": pe[1].item(), "rows": int(pe[2].item()),
                  "against": "float64 oracle over the cache bytes read back through the C ABI, on slots refilled with "
                             "real K/V before two probed churn steps"}
        probe = None
        if not parity["ok"]:
            raise SystemExit(f"parity check failed before timing: {parity}")
    barrier()
    work["decode_keys"], work["prefill_flops"] = 0, 0.0
    launches0 = cache.launch_count()
    cache.kernel_timing(True)
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
    kt = {k: cache.kernel_timing_read(getattr(yahkv, "KERNEL_" + k)) for k in
          ("APPEND", "DECODE_PART", "DECODE_COMBINE", "PREFILL", "PREFILL_DEQUANT")}
    cache.kernel_timing(False)
    launches = cache.launch_count() - launches0
    dkeys_mine, pflops_mine = work["decode_keys"], work["prefill_flops"]

    # ---- end to end: the same schedule continues with every call's K/V/q coming from pinned host memory and its
    # output copied back to it ----
    e_s = e_tokens = 0.0
    if not args.no_e2e:
        for name, t in (("k1", k1), ("v1", v1), ("q1", q1), ("o1", o1), ("kc", kc), ("vc", vc), ("qc", qc), ("oc", oc)):
            host[name] = t.cpu().pin_memory()
        runner.step(step_no, gpu)
        step_no += 1
        barrier()
        work["h2d"] = work["d2h"] = 0
        t0 = time.perf_counter()
        for _ in range(args.steps):
            e_tokens += runner.step(step_no, gpu)["tokens"]
            step_no += 1
        torch.cuda.synchronize()
        e_s = time.perf_counter() - t0
        host.clear()

    stats = torch.tensor([ms, tokens, dkeys_mine, pflops_mine, launches, kt["DECODE_PART"][0] + kt["DECODE_COMBINE"][0],
                          kt["PREFILL"][0] + kt["PREFILL_DEQUANT"][0], kt["APPEND"][0], e_s, e_tokens,
                          work["h2d"], work["d2h"], kt["DECODE_PART"][0], kt["DECODE_PART"][1]],
                         dtype=torch.float64, device="cuda")
    allr = [stats]
    if world > 1:
        allr = [torch.zeros_like(stats) for _ in range(world)]
        dist.all_gather(allr, stats)
    rows = [t.cpu().numpy() for t in allr]
    if rank == 0:
        ms_max = max(r[0] for r in rows)
        tokens_all, dkeys, pflops = sum(r[1] for r in rows), sum(r[2] for r in rows), sum(r[3] for r in rows)
        e_s_max, e_tok_all = max(r[8] for r in rows), sum(r[9] for r in rows)
        peak, peak_kind = measured_peaks()
        part_ms, part_n = rows[0][12], rows[0][13]
        part_achieved = rows[0][2] * layers * 2176 / (part_ms * 1e-3) / 1e9 if part_ms else 0.0
        per_rank = [{"rank": i, "device_ms": r[0], "idle_ms_waiting_for_the_slowest_rank": ms_max - r[0],
                     "decode_kernel_ms": r[5], "prefill_kernel_ms": r[6], "append_kernel_ms": r[7],
                     "decode_kv_gbps_in_kernel": r[2] * layers * 2176 / (r[5] * 1e-3) / 1e9 if r[5] else None,
                     "prefill_tflops_in_kernel": r[3] * layers / (r[6] * 1e-3) / 1e12 if r[6] else None}
                    for i, r in enumerate(rows)]
        line = {
            "metric": "serving_churn_tokens_per_s", "value": tokens_all / (ms_max * 1e-3), "unit": "tok/s",
            "n_gpus": world, "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": ms_max / args.steps,
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "u8", "data": "synthetic",
            "config": {"workload": f"churn_{sched.n_slots}slots_{layers}layers_q8_0_ctx512-65536_page64",
                       "slots_per_gpu": 32, "decode_tokens_per_step": sched.n_decode, "prefill_chunk": sched.chunk,
                       "finish_frac": 0.1, "note": "attention + append only; new sequences take recycled pages as "
                       "their prompt cache; sequences partitioned by slot, no collective on the data path",
                       "l2": "inputs larger than L2: every step reads gigabytes of cache per rank"},
            "extra": {"decode_kv_gbps": dkeys * layers * 2176 / (ms_max * 1e-3) / 1e9,
                      "prefill_tflops_averaged_over_the_run": pflops * layers / (ms_max * 1e-3) / 1e12,
                      "pages_free_rank0": cache.pages_free(), "device_bytes_rank0": cache.device_bytes(),
                      "per_rank": per_rank},
            "roofline": {"kernel": "DecodePartKernel<q8_0> (rank 0, inside the churn steps)", "bound": "hbm",
                         "achieved": part_achieved, "peak": peak, "unit": "GB/s", "frac": part_achieved / peak,
                         "peak_kind": f"of {peak_kind}", "launches": int(part_n), "traffic": None},
            "gpu_launches": int(sum(r[4] for r in rows)), "clocks": clocks,
        }
        if parity is not None:
            line["parity_checked"], line["parity"] = parity["ok"], parity
        if e_s_max > 0:
            line["e2e"] = {"value": e_tok_all / e_s_max, "unit": "tok/s", "steps": args.steps,
                           "h2d_bytes_per_step": sum(r[10] for r in rows) / args.steps,
                           "d2h_bytes_per_step": sum(r[11] for r in rows) / args.steps,
                           "api": "every append / attend call's K, V, q copied from pinned host memory ahead of it and "
                                  "its output copied back, on the calls' stream, inside the timed region"}
        if world == 1 and not args.no_cpu:
            lens4 = np.sort(sched.initial_lens)[::8][:4]
            res = cpu_arm("q8_0", lens=lens4, reps=1)
            line["cpu_baseline"] = {"value": 4.0 / (res["pass_s"] * layers), "unit": "tok/s", "cores": res["threads"],
                                    "kind": "port", "sample": "decode attention of 4 slots (" + res["sample"] +
                                    f"), scaled to {layers} layers; prefill and append not timed on the CPU"}
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
    w = workload(0, 1, args.layers)                   # the same sequences on every rank
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
    ap.add_argument("--fmt", default="q8_0", choices=["q8_0", "q4_0", "kv8a16", "kv4a16", "f16"],
                    help="cache format (q8_0 = the configuration; kv8a16 / kv4a16 = the reference's own formats)")
    ap.add_argument("--workload", default="decode", choices=["decode", "prefill", "longctx", "churn", "headshard"],
                    help="decode = the batch-32 configuration (default, the headline metric); prefill = chunked "
                         "prefill; longctx = batch 8 x 131072 tokens, q4_0, 64 splits, one layer")
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline leg")
    ap.add_argument("--no-e2e", action="store_true", help="skip the host-buffer leg")
    ap.add_argument("--no-graph", action="store_true", help="skip the captured-graph leg (value = eager calls)")
    ap.add_argument("--no-parity", action="store_true", help="skip the oracle check of sampled outputs before timing")
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
    w = workload(rank, world, args.layers)
    rng, lens, layers = w["rng"], w["lens"].copy(), w["layers"]
    total_steps = args.warmup + args.steps
    e2e_steps = 0 if args.no_e2e else args.steps + 1
    graph_steps = 0 if args.no_graph else args.steps + 3
    grow = total_steps + graph_steps + e2e_steps + 2
    pages = [(int(n) + grow + 63) // 64 for n in lens]
    num_pages = sum(pages) + 64
    fmt = {"q8_0": yahkv.FMT_Q8_0, "q4_0": yahkv.FMT_Q4_0, "kv8a16": yahkv.FMT_KV8A16, "kv4a16": yahkv.FMT_KV4A16, "f16": yahkv.FMT_F16}[args.fmt]
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
    parity = None
    if not args.no_parity:
        # The last warm-up step's layer-0 outputs of the shortest and of a middle sequence against the float64 oracle
        # over the cache's own bytes, and that step's appended tokens against the oracle's quantizer.
        import parity_probe as P
        order = np.argsort(lens)
        picks = [int(order[0])] if BATCH <= 8 else [int(order[0]), int(order[len(order) // 2])]
        q0, o0 = q[0].cpu().numpy(), out[0].cpu().numpy()
        k0, v0 = k_new[0].cpu().numpy(), v_new[0].cpu().numpy()
        err = rel = 0.0
        ok = True
        for i in picks:
            n_keys = cache.seq_len(seqs[i], 0)
            e, r, slack = P.check_decode_row(cache, 0, seqs[i], n_keys, q0[i], o0[i], out_is_f16=True)
            err, rel = max(err, e), max(rel, r)
            ok = ok and e <= P.ABS_TOL + slack and P.check_appended_token(cache, 0, seqs[i], n_keys - 1, k0[i], v0[i])
        parity = {"ok": bool(ok), "max_abs_err": err, "max_rel_err": rel, "rows": len(picks),
                  "against": "float64 oracle over the cache bytes read back through the C ABI; appended tokens "
                             "byte-exact against the oracle quantizer; outputs are fp16"}
        if not ok:
            raise SystemExit(f"parity check failed before timing: {parity}")
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
        if N_SPLITS:
            batch.set_splits(N_SPLITS)     # the configuration's split count, as the eager calls pass it
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
    per_rank = None
    if world > 1:
        mx = stats.clone()
        dist.all_reduce(mx, op=dist.ReduceOp.MAX)
        sm = stats.clone()
        dist.all_reduce(sm, op=dist.ReduceOp.SUM)
        allr = [torch.zeros_like(stats) for _ in range(world)]
        dist.all_gather(allr, stats)
        per_rank = {"eager_ms": [t[0].item() for t in allr], "eager_bytes": [t[1].item() for t in allr],
                    "graph_ms": [t[5].item() for t in allr], "graph_bytes": [t[6].item() for t in allr],
                    "part_kernel_us": [t[4].item() * 1e3 for t in allr], "cached_tokens": w["all_rank_tokens"]}
        if parity is not None:
            pe = torch.tensor([parity["max_abs_err"], parity["max_rel_err"]], dtype=torch.float64, device="cuda")
            dist.all_reduce(pe, op=dist.ReduceOp.MAX)
            parity["max_abs_err"], parity["max_rel_err"] = pe[0].item(), pe[1].item()
            parity["rows"] *= world
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
            "extra": {"step_mode": f"one captured CUDA graph per {layers}-layer step (yahkv_batch_*)" if use_graph
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
        if parity is not None:
            line["parity_checked"] = parity["ok"]
            line["parity"] = parity
        if per_rank is not None:
            line["extra"]["per_rank"] = per_rank
        if e2e:
            line["e2e"] = {"value": e_bytes_all / e_s / 1e9, "unit": UNIT, "h2d_bytes_per_step": e2e["h2d"],
                           "d2h_bytes_per_step": e2e["d2h"], "steps": e2e_steps - 1, "timed_by": "host clock around "
                           "the steps, device idle before and after (synchronize on both sides)",
                           "api": "yahkv_decode_step_host_async per layer + yahkv_decode_step_host_wait per step (pinned host K/V/q in, outputs back in host memory before the step ends)"}
        if args.fmt in NCU_DRAM_PER_ALGORITHMIC_BYTE:
            line["roofline"]["traffic"] = NCU_DRAM_PER_ALGORITHMIC_BYTE[args.fmt] * part_bytes
            line["roofline"]["traffic_note"] = ("(dram__bytes_read.sum + dram__bytes_write.sum) / algorithmic bytes of "
                                                "one ncu-captured launch of this workload, times this run's bytes "
                                                "per launch")
        if world == 1 and not args.no_cpu and args.fmt not in ("kv8a16", "kv4a16", "f16"):
            res = cpu_arm(args.fmt, lens=None if args.workload == "decode" else lens[:1])
            line["cpu_baseline"] = {"value": res["gbs"], "unit": UNIT, "cores": res["threads"], "kind": "port",
                                    "sample": res["sample"], "append_mtok_s": res["append_mtok_s_port"],
                                    "append_mtok_s_reference_codec_1thread":
                                        res.get("append_mtok_s_reference_codec_1thread")}
        print(json.dumps(line))
    cache.close()
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
