"""yahkv_attend_decode_noalloc against yahkv_attend_decode.

The no-allocation entry point exists for hosts that are not allowed to allocate GPU memory once running (their own
allocator owns the device, or an allocation's implicit synchronisation is unacceptable), and that therefore cannot
create a context either: they hand over their own pools, block tables and lengths, and the library keeps the split-K
scratch in a static device array. This test plays such a host: it copies a context's pools into plain torch tensors
(through the inspection calls), calls the context-free entry point on them twice in a row, with different queries and
lengths, so the second call runs on a scratch array that still holds the first call's units and partials, and
compares both results with the context's own attend call at the same split count and with the float64 oracle. The
status word of the static array is read back through yahkv_noalloc_status (an asynchronous copy into this host's own
memory, so no allocation there either) and must be clean; lengths of 0 and beyond the table are clamped as documented.
It also checks that requests beyond the static array's capacity are refused. The file name sorts last so a run that stops at the first failure has
already run every other test.
"""
import numpy as np
import pytest
import torch

import oracle as O
import yahkv

pytestmark = pytest.mark.gpu
TOL = 2e-3   # the tolerance of the other attention tests; the two entry points share kernels, so they agree far closer


def _pools_as_tensors(cache, num_pages):
    sides = []
    for side in (yahkv.SIDE_K, yahkv.SIDE_V):
        pages = [cache.read_page(0, side, p) for p in range(num_pages)]
        # read_page hands out GGUF codes; the call under test takes device pools, whose q8_0 V bytes are sign-flipped
        sides.append(torch.from_numpy(yahkv.device_codes(cache.fmt, np.stack([c for c, _ in pages]), side)).cuda())
        sides.append(torch.from_numpy(np.stack([s for _, s in pages]).view(np.int16)).cuda())
    return sides   # kcodes, kscales, vcodes, vscales


@pytest.mark.parametrize("fmt", [yahkv.FMT_Q8_0, yahkv.FMT_Q4_0])
def test_noalloc_matches_context_path_on_two_calls_in_a_row(fmt):
    rng = np.random.default_rng(31)
    lens = [700, 64, 1, 3000, 129]
    pages_per = [(n + 63) // 64 for n in lens]
    num_pages, stride = sum(pages_per) + 3, max(pages_per)
    cache = yahkv.KvCache(num_pages=num_pages, fmt=fmt, max_seqs=len(lens), max_pages_per_seq=stride)
    pool = O.PagedPool(fmt, num_pages)
    perm = rng.permutation(num_pages).astype(np.int32)
    seqs, off = [], 0
    tables = np.zeros((len(lens), stride), np.int32)
    for i, n in enumerate(lens):
        s = cache.seq_create()
        cache.seq_set_table(s, perm[off:off + pages_per[i]])
        tables[i, :pages_per[i]] = perm[off:off + pages_per[i]]
        off += pages_per[i]
        Kh = rng.standard_normal((n, 4, 256)).astype(np.float16)
        Vh = rng.standard_normal((n, 4, 256)).astype(np.float16)
        cache.append(0, np.full(n, s, np.int32), np.arange(n), torch.from_numpy(Kh).cuda(), torch.from_numpy(Vh).cuda())
        pool.append(tables[i, :pages_per[i]], 0, Kh, Vh)
        seqs.append(s)
    cache.sync()
    kcodes, kscales, vcodes, vscales = _pools_as_tensors(cache, num_pages)
    tables_dev = torch.from_numpy(tables).cuda()

    # second call: other queries, a gate, shorter visible lengths, another split count and output type
    calls = [
        dict(lens=lens, n_splits=4, gate=False, out_dtype=yahkv.OUT_F32),
        dict(lens=[650, 40, 1, 1500, 128], n_splits=2, gate=True, out_dtype=yahkv.OUT_F16),
    ]
    for call in calls:
        q = torch.from_numpy(rng.standard_normal((len(lens), 24, 256)).astype(np.float16)).cuda()
        gate = torch.from_numpy(rng.standard_normal((len(lens), 24, 256)).astype(np.float32)).cuda() if call["gate"] else None
        dt = torch.float32 if call["out_dtype"] == yahkv.OUT_F32 else torch.float16
        for s, n in zip(seqs, call["lens"]):
            cache.seq_set_len(s, n)
        want = torch.zeros(len(lens), 24, 256, device="cuda", dtype=dt)
        cache.attend_decode(0, seqs, q, want, gate=gate, out_dtype=call["out_dtype"], n_splits=call["n_splits"])
        cache.sync()
        got = torch.full((len(lens), 24, 256), float("nan"), device="cuda", dtype=dt)
        lens_dev = torch.tensor(call["lens"], dtype=torch.int32, device="cuda")
        yahkv.attend_decode_noalloc(fmt=fmt, n_layers=1, num_pages=num_pages, layer=0, kcodes=kcodes, vcodes=vcodes,
                                    kscales=kscales, vscales=vscales, tables=tables_dev, table_stride=stride,
                                    n_seqs=len(lens), lens=lens_dev, q=q, out=got, gate=gate,
                                    out_dtype=call["out_dtype"], n_splits=call["n_splits"],
                                    stream=torch.cuda.current_stream().cuda_stream)
        torch.cuda.synchronize()
        status = torch.full((1,), -1, dtype=torch.int32).pin_memory()
        yahkv.noalloc_status(status, stream=torch.cuda.current_stream().cuda_stream)
        torch.cuda.synchronize()
        assert int(status[0]) == 0, "a kernel of the no-allocation path gave up a wait"
        err = (got.float() - want.float()).abs().max().item()
        assert err <= TOL, (call, err)
        assert torch.isfinite(got.float()).all()
        # and against the float64 oracle, not only against the sibling entry point
        gate_h = None if gate is None else gate.cpu().numpy()
        for i, n in enumerate(call["lens"]):
            ref = pool.attend_decode_f64(tables[i], n, q[i].cpu().numpy(), None if gate_h is None else gate_h[i])
            slack = np.abs(ref).max() * 2.0 ** -11 if call["out_dtype"] == yahkv.OUT_F16 else 0.0
            assert np.abs(got[i].float().cpu().numpy() - ref).max() <= TOL + slack, (call, i)
    # lengths read from device memory are clamped to [1, table_stride * 64]: 0 behaves as 1, too large as the cap
    q = torch.from_numpy(rng.standard_normal((len(lens), 24, 256)).astype(np.float16)).cuda()
    outs = []
    for test_lens in ([0, 64, 1, 10 ** 6, 129], [1, 64, 1, stride * 64, 129]):
        got = torch.full((len(lens), 24, 256), float("nan"), device="cuda")
        yahkv.attend_decode_noalloc(fmt=fmt, n_layers=1, num_pages=num_pages, layer=0, kcodes=kcodes, vcodes=vcodes,
                                    kscales=kscales, vscales=vscales, tables=tables_dev, table_stride=stride,
                                    n_seqs=len(lens), lens=torch.tensor(test_lens, dtype=torch.int32, device="cuda"),
                                    q=q, out=got, out_dtype=yahkv.OUT_F32, n_splits=3,
                                    stream=torch.cuda.current_stream().cuda_stream)
        torch.cuda.synchronize()
        outs.append(got.cpu().numpy())
    assert np.isfinite(outs[0]).all() and np.array_equal(outs[0], outs[1])


def test_noalloc_refuses_what_the_static_scratch_cannot_hold():
    x = torch.zeros(16, dtype=torch.int32, device="cuda")
    base = dict(fmt=yahkv.FMT_Q8_0, n_layers=1, num_pages=4, layer=0, kcodes=x, vcodes=x, kscales=x, vscales=x,
                tables=x, table_stride=1, lens=x, q=x, out=x)
    for extra, code in ((dict(n_seqs=yahkv.NOALLOC_MAX_SEQS + 1, n_splits=1), yahkv.ERR_CAPACITY),
                        (dict(n_seqs=64, n_splits=5), yahkv.ERR_CAPACITY),       # 64 * 4 * 5 > 1024 units
                        (dict(n_seqs=1, n_splits=0), yahkv.ERR_INVALID),
                        (dict(n_seqs=1, n_splits=1, layer=1), yahkv.ERR_INVALID)):
        args = dict(base)
        args.update(extra)
        with pytest.raises(yahkv.YahkvError) as e:
            yahkv.attend_decode_noalloc(**args)
        assert e.value.code == code and e.value.message
    args = dict(base, n_seqs=1, n_splits=1)
    args["q"] = None
    with pytest.raises(yahkv.YahkvError):
        yahkv.attend_decode_noalloc(**args)
