"""The C ABI's host side without a GPU: exported symbols, the page allocator, block tables, validation, and that the
hot path refuses to run (there is no CPU fallback)."""
import ctypes
import os
import re

import numpy as np
import pytest

import yahkv


def host_ctx(**kw):
    args = dict(device=-1, n_layers=2, num_pages=10, max_seqs=4, max_pages_per_seq=6)
    args.update(kw)
    return yahkv.KvCache(**args)


def test_library_exports_every_declared_symbol():
    header = open(os.path.join(yahkv.INCLUDE_DIR, "yahkv.h")).read()
    declared = set(re.findall(r"\b(yahkv_[a-z0-9_]+)\s*\(", header))
    assert declared, "no declarations found in include/yahkv.h"
    lib = ctypes.CDLL(yahkv.LIB_PATH)
    for name in sorted(declared):
        assert hasattr(lib, name), f"{name} is declared but not exported"
    assert declared == set(yahkv.SIGNATURES), declared ^ set(yahkv.SIGNATURES)


def test_config_is_validated():
    for bad in (dict(n_q_heads=32), dict(head_dim=128), dict(page_tokens=256), dict(fmt=7), dict(num_pages=0),
                dict(n_layers=0), dict(max_seqs=0), dict(num_pages=1 << 24, n_layers=64), dict(max_splits=1025)):
        with pytest.raises(yahkv.YahkvError) as e:
            host_ctx(**bad)
        assert e.value.code == yahkv.ERR_INVALID
    host_ctx(max_splits=1024).close()        # the combine kernel's limit itself is accepted


def test_allocator_is_lifo_and_recycles():
    c = host_ctx()
    a, b = c.seq_create(), c.seq_create()
    assert (a, b) == (0, 1) and c.pages_free() == 10
    c.seq_reserve(a, 65)                     # two pages
    assert c.seq_table(a).tolist() == [0, 1] and c.pages_free() == 8
    c.seq_reserve(b, 1)
    assert c.seq_table(b).tolist() == [2]
    c.seq_reserve(a, 64 * 3)                 # grows by one, keeps the first two
    assert c.seq_table(a).tolist() == [0, 1, 3]
    c.seq_reserve(a, 10)                     # never shrinks
    assert c.seq_table(a).tolist() == [0, 1, 3]
    c.seq_free(a)
    assert c.pages_free() == 9
    d = c.seq_create()
    assert d == a                            # sequence slots recycle too
    c.seq_reserve(d, 64 * 2)
    assert c.seq_table(d).tolist() == [3, 1]  # last freed, first reused
    assert c.seq_len(d, 0) == 0 and c.seq_len(d, 1) == 0


def test_exhaustion_leaves_state_unchanged():
    c = host_ctx(num_pages=3)
    a, b = c.seq_create(), c.seq_create()
    c.seq_reserve(a, 128)
    with pytest.raises(yahkv.YahkvError) as e:
        c.seq_reserve(b, 129)                # needs 3, only 1 free
    assert e.value.code == yahkv.ERR_NO_PAGES
    assert c.pages_free() == 1 and c.seq_table(b).size == 0
    with pytest.raises(yahkv.YahkvError) as e:
        c.seq_reserve(a, 64 * 7)             # wider than the table
    assert e.value.code == yahkv.ERR_CAPACITY
    for _ in range(2):
        c.seq_create()
    with pytest.raises(yahkv.YahkvError) as e:
        c.seq_create()
    assert e.value.code == yahkv.ERR_CAPACITY


def test_set_table_is_validated_like_the_reference():
    c = host_ctx()
    a, b = c.seq_create(), c.seq_create()
    c.seq_set_table(a, [7, 2, 9])
    assert c.seq_table(a).tolist() == [7, 2, 9] and c.pages_free() == 7
    for pages, code in (([1, 10], yahkv.ERR_INVALID), ([-1], yahkv.ERR_INVALID), ([4, 4], yahkv.ERR_INVALID),
                        ([2], yahkv.ERR_INVALID), (list(range(7)), yahkv.ERR_CAPACITY)):
        with pytest.raises(yahkv.YahkvError) as e:
            c.seq_set_table(b, pages)
        assert e.value.code == code
        assert c.seq_table(b).size == 0 and c.pages_free() == 7
    c.seq_set_table(a, [2, 5])               # own pages may be reused; 7 and 9 go back
    assert c.pages_free() == 8
    c.seq_reserve(b, 64 * 8 // 8)
    assert c.seq_table(b)[0] not in (2, 5)


def test_lengths_and_ids_are_checked():
    c = host_ctx()
    a = c.seq_create()
    c.seq_reserve(a, 100)
    c.seq_set_len(a, 100)
    assert c.seq_len(a, 1) == 100
    c.seq_set_len(a, 40, layer=0)
    assert (c.seq_len(a, 0), c.seq_len(a, 1)) == (40, 100)
    with pytest.raises(yahkv.YahkvError):
        c.seq_set_len(a, 129)
    with pytest.raises(yahkv.YahkvError):
        c.seq_set_len(a, 1, layer=2)
    for bad in (-1, 3, 99):
        with pytest.raises(yahkv.YahkvError):
            c.seq_reserve(bad, 1)
        with pytest.raises(yahkv.YahkvError):
            c.seq_free(bad)
    c.seq_free(a)
    with pytest.raises(yahkv.YahkvError):
        c.seq_free(a)


def test_hot_path_has_no_cpu_fallback():
    c = host_ctx()
    a = c.seq_create()
    c.seq_reserve(a, 64)
    buf = np.zeros((1, 24, 256), np.float16)
    calls = [
        lambda: c.append(0, [a], [0], buf, buf),
        lambda: c.append_slots(0, 1, np.zeros(1, np.int64), buf, buf),
        lambda: c.attend_decode(0, [a], buf, buf),
        lambda: c.attend_prefill(0, [a], [1], buf, buf),
        lambda: c.decode_step_host(0, [a], buf, buf, buf, buf),
        lambda: c.read_page(0, 0, 0),
        lambda: c.export_token(0, a, 0),
        lambda: c.sync(),
    ]
    for call in calls:
        with pytest.raises(yahkv.YahkvError) as e:
            call()
        assert e.value.code == yahkv.ERR_NO_DEVICE
    assert c.seq_len(a, 0) == 0              # the refused append did not advance the length


def test_create_without_a_gpu_fails_loudly():
    import torch
    if torch.cuda.is_available():
        pytest.skip("a GPU is present")
    with pytest.raises(yahkv.YahkvError) as e:
        yahkv.KvCache(device=0)
    assert e.value.code in (yahkv.ERR_NO_DEVICE, yahkv.ERR_CUDA)


def test_kv_head_range_is_validated():
    ok = dict(device=-1, n_layers=1, num_pages=4, max_seqs=1, max_pages_per_seq=4)
    yahkv.KvCache(**ok, kv_head_begin=2, kv_head_count=2).close()
    for begin, count in ((3, 2), (-1, 1), (1, 0), (0, 5)):
        with pytest.raises(yahkv.YahkvError):
            yahkv.KvCache(**ok, kv_head_begin=begin, kv_head_count=count)
