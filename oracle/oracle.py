"""ctypes binding of the CPU oracle (oracle/yahkv_oracle.cpp) and of the reference's own codecs (oracle/_ref).

TEST INFRASTRUCTURE ONLY. Importers: tests/, the smoke check and the CPU-baseline / reference arm of bench.py. The
shipped library and its Python binding never import this module.

`PagedPool` models one layer's K and V pools in host memory in the library's layout, so a test can run the same
appends through the oracle and the GPU and compare the bytes.
"""
import ctypes
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
ORACLE_SO = os.path.join(_HERE, "libyahkv_oracle.so")
REF_SO = os.path.join(_HERE, "_ref", "libyah_ref_codec.so")

Q_HEADS, KV_HEADS, HEAD_DIM, PAGE_TOKENS, BLOCKS = 24, 4, 256, 64, 8
FMT_Q8_0, FMT_Q4_0, FMT_KV8A16, FMT_KV4A16, FMT_F16 = 0, 1, 2, 3, 4
GGML_Q4_0, GGML_Q8_0 = 2, 8  # ggml type ids the reference's Dequantize takes


def build():
    """Compile the oracle, and the reference's codecs when its checkout is present (oracle/Makefile)."""
    r = subprocess.run(["make", "-C", _HERE], capture_output=True, text=True)
    if r.returncode:
        raise RuntimeError("building the oracle failed:\n" + r.stdout[-2000:] + r.stderr[-2000:])


def _p(a):
    return None if a is None else a.ctypes.data_as(ctypes.c_void_p)


if not os.path.exists(ORACLE_SO):
    build()
_o = ctypes.CDLL(ORACLE_SO)
_o.yahkv_oracle_slot.restype = ctypes.c_int64
_ref = ctypes.CDLL(REF_SO) if os.path.exists(REF_SO) else None
THREADS = _o.yahkv_oracle_hardware_threads()


def have_ref():
    return _ref is not None


def code_bytes(fmt):
    return 512 if fmt == FMT_F16 else (256 if fmt == FMT_Q8_0 else 128)


def block_bytes(fmt):
    return 34 if fmt == FMT_Q8_0 else 18


def quantize(x, fmt):
    """f32 array (size a multiple of 32) -> GGUF blocks as uint8."""
    x = np.ascontiguousarray(x, np.float32).reshape(-1)
    out = np.zeros(x.size // 32 * block_bytes(fmt), np.uint8)
    fn = _o.yahkv_oracle_quantize_q8_0 if fmt == FMT_Q8_0 else _o.yahkv_oracle_quantize_q4_0
    fn(_p(x), ctypes.c_uint64(x.size), _p(out))
    return out


def dequantize(blocks, fmt):
    blocks = np.ascontiguousarray(blocks, np.uint8).reshape(-1)
    n = blocks.size // block_bytes(fmt) * 32
    y = np.zeros(n, np.float32)
    fn = _o.yahkv_oracle_dequantize_q8_0 if fmt == FMT_Q8_0 else _o.yahkv_oracle_dequantize_q4_0
    fn(_p(blocks), ctypes.c_uint64(n), _p(y))
    return y


def ref_quantize_q8_0(x):
    """The reference's QuantizeQ8_0 itself (engine/core/gguf_quant.cpp:310-320), compiled from its sources."""
    x = np.ascontiguousarray(x, np.float32).reshape(-1)
    out = np.zeros(x.size // 32 * 34, np.uint8)
    _ref.yah_ref_quantize_q8_0(_p(x), ctypes.c_uint64(x.size), _p(out))
    return out


def ref_dequantize(blocks, fmt):
    """The reference's Dequantize itself (engine/core/gguf_quant.cpp:291-308)."""
    blocks = np.ascontiguousarray(blocks, np.uint8).reshape(-1)
    n = blocks.size // block_bytes(fmt) * 32
    y = np.zeros(n, np.float32)
    rc = _ref.yah_ref_dequantize(GGML_Q8_0 if fmt == FMT_Q8_0 else GGML_Q4_0, _p(blocks), _p(y), ctypes.c_uint64(n))
    assert rc == 0
    return y


def rope_rows(x, weight, eps, pos):
    """Head rows [rows][256] f32 -> RMSNorm + NeoX RoPE (64 of 256 dims, theta 1e7) -> fp16; pos: one per row."""
    x = np.ascontiguousarray(x, np.float32).reshape(-1, 256)
    weight = np.ascontiguousarray(weight, np.float32)
    pos = np.ascontiguousarray(pos, np.int32)
    assert weight.size == 256 and pos.size == x.shape[0]
    out = np.zeros(x.shape, np.uint16)
    _o.yahkv_oracle_rope_rows(_p(x), ctypes.c_int64(x.shape[0]), _p(weight), ctypes.c_float(eps), _p(pos), _p(out))
    return out.view(np.float16)


def validate_table(table, num_pages):
    table = np.ascontiguousarray(table, np.int32)
    return _o.yahkv_oracle_validate_table(_p(table), len(table), num_pages)


def slot(table, pos, num_pages, page_tokens=PAGE_TOKENS):
    table = np.ascontiguousarray(table, np.int32)
    return _o.yahkv_oracle_slot(page_tokens, num_pages, _p(table), len(table), ctypes.c_int64(pos))


class PagedPool:
    """One layer's pools on the host: codes [P][4][64][cb] u8 and scales [P][4][64][8] u16, for K and for V."""

    def __init__(self, fmt, num_pages):
        self.fmt, self.num_pages = fmt, num_pages
        cb = code_bytes(fmt)
        self.kcodes = np.zeros((num_pages, KV_HEADS, PAGE_TOKENS, cb), np.uint8)
        self.vcodes = np.zeros_like(self.kcodes)
        self.kscales = np.zeros((num_pages, KV_HEADS, PAGE_TOKENS, 0 if fmt == FMT_F16 else BLOCKS), np.uint16)
        self.vscales = np.zeros_like(self.kscales)

    def append(self, table, pos0, k, v, threads=THREADS):
        """k, v: [n][4][256] float16 at logical positions pos0 .. pos0 + n - 1 of a sequence with this table."""
        table = np.ascontiguousarray(table, np.int32)
        for x, codes, scales in ((k, self.kcodes, self.kscales), (v, self.vcodes, self.vscales)):
            x = np.ascontiguousarray(x, np.float16)
            n = x.shape[0]
            _o.yahkv_oracle_append_seq(self.fmt, PAGE_TOKENS, self.num_pages, _p(codes), _p(scales), _p(table),
                                       len(table), ctypes.c_int64(pos0), n, _p(x.view(np.uint16)), threads)

    def append_slots(self, slots, k, v, threads=THREADS):
        slots = np.ascontiguousarray(slots, np.int64)
        for x, codes, scales in ((k, self.kcodes, self.kscales), (v, self.vcodes, self.vscales)):
            x = np.ascontiguousarray(x, np.float16)
            _o.yahkv_oracle_append_slots(self.fmt, PAGE_TOKENS, self.num_pages, _p(codes), _p(scales), _p(slots),
                                         len(slots), _p(x.view(np.uint16)), threads)

    def export_row(self, side, slot_):
        codes, scales = (self.kcodes, self.kscales) if side == 0 else (self.vcodes, self.vscales)
        out = np.zeros(KV_HEADS * BLOCKS * block_bytes(self.fmt), np.uint8)
        _o.yahkv_oracle_export_row(self.fmt, PAGE_TOKENS, self.num_pages, _p(codes), _p(scales),
                                   ctypes.c_int64(slot_), _p(out))
        return out

    def attend_decode_f64(self, table, n_keys, q, gate=None, scale=1.0 / 16.0, threads=THREADS):
        """q [24][256] float16, gate [24][256] float32 or None -> out [24][256] float64."""
        table = np.ascontiguousarray(table, np.int32)
        q = np.ascontiguousarray(q, np.float16)
        gate = None if gate is None else np.ascontiguousarray(gate, np.float32)
        out = np.zeros((Q_HEADS, HEAD_DIM), np.float64)
        _o.yahkv_oracle_attend_decode_f64(self.fmt, PAGE_TOKENS, self.num_pages, _p(self.kcodes), _p(self.kscales),
                                          _p(self.vcodes), _p(self.vscales), _p(table), len(table),
                                          ctypes.c_int64(n_keys), _p(q.view(np.uint16)), _p(gate),
                                          ctypes.c_double(scale), _p(out), threads)
        return out

    def attend_decode_f32(self, tables, n_keys, q, gate=None, scale=1.0 / 16.0, threads=THREADS):
        """Batched two-level f32 attention: tables [n][stride] int32, n_keys [n], q [n][24][256] float16."""
        tables = np.ascontiguousarray(tables, np.int32)
        n_keys = np.ascontiguousarray(n_keys, np.int32)
        q = np.ascontiguousarray(q, np.float16)
        gate = None if gate is None else np.ascontiguousarray(gate, np.float32)
        out = np.zeros((len(n_keys), Q_HEADS, HEAD_DIM), np.float32)
        _o.yahkv_oracle_attend_decode_f32(self.fmt, PAGE_TOKENS, self.num_pages, _p(self.kcodes), _p(self.kscales),
                                          _p(self.vcodes), _p(self.vscales), _p(tables), tables.shape[1], _p(n_keys),
                                          len(n_keys), _p(q.view(np.uint16)), _p(gate), ctypes.c_float(scale),
                                          _p(out), threads)
        return out

    def attend_prefill_f64(self, table, start, q, q_begin=0, q_end=None, gate=None, scale=1.0 / 16.0,
                           threads=THREADS):
        """q [n_q][24][256] float16 for a chunk at positions start .. start + n_q - 1 (already appended)."""
        table = np.ascontiguousarray(table, np.int32)
        q = np.ascontiguousarray(q, np.float16)
        n_q = q.shape[0]
        q_end = n_q if q_end is None else q_end
        gate = None if gate is None else np.ascontiguousarray(gate, np.float32)
        out = np.zeros((q_end - q_begin, Q_HEADS, HEAD_DIM), np.float64)
        _o.yahkv_oracle_attend_prefill_f64(self.fmt, PAGE_TOKENS, self.num_pages, _p(self.kcodes), _p(self.kscales),
                                           _p(self.vcodes), _p(self.vscales), _p(table), len(table),
                                           ctypes.c_int64(start), n_q, q_begin, q_end, _p(q.view(np.uint16)),
                                           _p(gate), ctypes.c_double(scale), _p(out), threads)
        return out


# ---- the reference's own kv8a16 format (oracle/kv8a16_oracle.cpp) ------------------------------------------------
def kv8_quant_k(k_row, mean):
    """One token's K [4][256] fp16 and the channel mean [4][256] f32 -> (codes [4][256] u8, scale pairs [4][2][2] u16)."""
    k_row = np.ascontiguousarray(k_row, np.float16).reshape(KV_HEADS, HEAD_DIM)
    mean = np.ascontiguousarray(mean, np.float32).reshape(KV_HEADS, HEAD_DIM)
    codes, scales = np.zeros((KV_HEADS, HEAD_DIM), np.uint8), np.zeros((KV_HEADS, 2, 2), np.uint16)
    _o.yahkv_oracle_kv8_quant_k(_p(k_row.view(np.uint16)), _p(mean), _p(codes), _p(scales))
    return codes, scales


def kv8_deq_k(codes, scales):
    out = np.zeros((KV_HEADS, HEAD_DIM), np.float32)
    _o.yahkv_oracle_kv8_deq_k(_p(np.ascontiguousarray(codes, np.uint8)), _p(np.ascontiguousarray(scales, np.uint16)), _p(out))
    return out


def kv8_quant_vtile(v_tile):
    """v [16 keys][4][256] fp16 -> (codes [4][256][16] u8, stat pairs [4][256][2] u16)."""
    v_tile = np.ascontiguousarray(v_tile, np.float16).reshape(16, KV_HEADS, HEAD_DIM)
    codes, stats = np.zeros((KV_HEADS, HEAD_DIM, 16), np.uint8), np.zeros((KV_HEADS, HEAD_DIM, 2), np.uint16)
    _o.yahkv_oracle_kv8_quant_vtile(_p(v_tile.view(np.uint16)), _p(codes), _p(stats))
    return codes, stats


def kv8_deq_vtile(codes, stats):
    out = np.zeros((16, KV_HEADS, HEAD_DIM), np.float32)
    _o.yahkv_oracle_kv8_deq_vtile(_p(np.ascontiguousarray(codes, np.uint8)), _p(np.ascontiguousarray(stats, np.uint16)), _p(out))
    return out


class Kv8Pool:
    """One layer's kv8a16 pools on the host in the library's layout (64-token pages of four 16-key tiles). Sequence
    state that the format needs beyond the pools (the open fp16 V tile, the K channel mean) is the caller's: see
    `new_sequence`."""

    def __init__(self, num_pages):
        self.num_pages = num_pages
        self.kcodes = np.zeros((num_pages, KV_HEADS, PAGE_TOKENS, HEAD_DIM), np.uint8)
        self.kscales = np.zeros((num_pages, KV_HEADS, PAGE_TOKENS, 2, 2), np.uint16)
        self.vcodes = np.zeros((num_pages, KV_HEADS, PAGE_TOKENS // 16, HEAD_DIM, 16), np.uint8)
        self.vstats = np.zeros((num_pages, KV_HEADS, PAGE_TOKENS // 16, HEAD_DIM, 2), np.uint16)

    @staticmethod
    def new_sequence(mean=None):
        """(open tile [4][256][16] fp16 as u16, mean [4][256] f32) of a fresh sequence."""
        m = np.zeros((KV_HEADS, HEAD_DIM), np.float32) if mean is None else np.ascontiguousarray(mean, np.float32).reshape(KV_HEADS, HEAD_DIM).copy()
        return np.zeros((KV_HEADS, HEAD_DIM, 16), np.uint16), m

    def append(self, table, pos0, k, v, open_tile, mean):
        table = np.ascontiguousarray(table, np.int32)
        k = np.ascontiguousarray(k, np.float16)
        v = np.ascontiguousarray(v, np.float16)
        _o.yahkv_oracle_kv8_append_seq(PAGE_TOKENS, self.num_pages, _p(self.kcodes), _p(self.kscales), _p(self.vcodes),
                                       _p(self.vstats), _p(open_tile), _p(mean), _p(table), len(table),
                                       ctypes.c_int64(pos0), k.shape[0], _p(k.view(np.uint16)), _p(v.view(np.uint16)))

    def attend_decode_f64(self, table, n_keys, q, open_tile, gate=None, scale=1.0 / 16.0, threads=THREADS):
        table = np.ascontiguousarray(table, np.int32)
        q = np.ascontiguousarray(q, np.float16)
        gate = None if gate is None else np.ascontiguousarray(gate, np.float32)
        out = np.zeros((Q_HEADS, HEAD_DIM), np.float64)
        _o.yahkv_oracle_kv8_attend_decode_f64(PAGE_TOKENS, self.num_pages, _p(self.kcodes), _p(self.kscales),
                                              _p(self.vcodes), _p(self.vstats), _p(open_tile), _p(table), len(table),
                                              ctypes.c_int64(n_keys), _p(q.view(np.uint16)), _p(gate),
                                              ctypes.c_double(scale), _p(out), threads)
        return out

    def dequantized(self, table, n_keys, open_tile):
        """(K, V) [n_keys][4][256] f32 of one sequence as attention sees them: K = (u - 128) s (mean not added back),
        V tiles dequantized except the tile of the newest key, which is the open fp16 tile."""
        table = np.ascontiguousarray(table, np.int32)
        validate_table(table, self.num_pages)
        K = np.zeros((n_keys, KV_HEADS, HEAD_DIM), np.float32)
        V = np.zeros((n_keys, KV_HEADS, HEAD_DIM), np.float32)
        for pos in range(n_keys):
            pg, tok = table[pos // PAGE_TOKENS], pos % PAGE_TOKENS
            K[pos] = kv8_deq_k(self.kcodes[pg, :, tok], self.kscales[pg, :, tok])
        newest = (n_keys - 1) // 16
        for t in range(newest + 1):
            k0, k1 = 16 * t, min(n_keys, 16 * t + 16)
            if t == newest:
                tile = np.ascontiguousarray(open_tile).view(np.float16).astype(np.float32)      # [4][256][16]
                V[k0:k1] = np.transpose(tile, (2, 0, 1))[:k1 - k0]
            else:
                pg, tl = table[k0 // PAGE_TOKENS], (k0 % PAGE_TOKENS) // 16
                V[k0:k1] = kv8_deq_vtile(self.vcodes[pg, :, tl], self.vstats[pg, :, tl])[:k1 - k0]
        return K, V

    def attend_prefill_f64(self, table, start, q, open_tile, q_begin=0, q_end=None, gate=None, scale=1.0 / 16.0):
        """Causal attention of chunk rows [q_begin, q_end) (row i sits at position start + i) over the cache as it is
        after the chunk's append, in float64: q [rows][24][256] fp16 -> out [q_end - q_begin][24][256]. The
        dequantize-then-attend form of the reference's prefill (gen_attn_fa.py:4648-4860, :3005-3042)."""
        q = np.ascontiguousarray(q, np.float16)
        q_end = q.shape[0] if q_end is None else q_end
        n_keys = start + q.shape[0]
        K, V = self.dequantized(table, n_keys, open_tile)
        K, V = K.astype(np.float64), V.astype(np.float64)
        out = np.zeros((q_end - q_begin, Q_HEADS, HEAD_DIM), np.float64)
        group = Q_HEADS // KV_HEADS
        for i in range(q_begin, q_end):
            vis = start + i + 1
            for h in range(Q_HEADS):
                kvh = h // group
                s_ = (K[:vis, kvh] @ q[i, h].astype(np.float64)) * scale
                w = np.exp(s_ - s_.max())
                o = (w @ V[:vis, kvh]) / w.sum()
                if gate is not None:
                    o = o / (1.0 + np.exp(-np.asarray(gate[i, h], np.float64)))
                out[i - q_begin, h] = o
        return out


# ---- the reference's own kv4a16 format (oracle/kv4a16_oracle.cpp) ------------------------------------------------
def hadamard256_f64(x):
    """H256 x / 16 over the last axis (length 256), float64; self-inverse."""
    x = np.ascontiguousarray(x, np.float64).copy()
    _o.yahkv_oracle_hadamard256_f64(_p(x), x.size // HEAD_DIM)
    return x


def kv4_quant_k(k_row, mean):
    """One token's K [4][256] fp16 and the channel mean [4][256] f32 -> (codes [4][128] u8, scale pairs [4][8][2] u16)."""
    k_row = np.ascontiguousarray(k_row, np.float16).reshape(KV_HEADS, HEAD_DIM)
    mean = np.ascontiguousarray(mean, np.float32).reshape(KV_HEADS, HEAD_DIM)
    codes, scales = np.zeros((KV_HEADS, 128), np.uint8), np.zeros((KV_HEADS, 8, 2), np.uint16)
    _o.yahkv_oracle_kv4_quant_k(_p(k_row.view(np.uint16)), _p(mean), _p(codes), _p(scales))
    return codes, scales


def kv4_deq_k(codes, scales):
    """-> the rotated (k - mean) [4][256] f32."""
    out = np.zeros((KV_HEADS, HEAD_DIM), np.float32)
    _o.yahkv_oracle_kv4_deq_k(_p(np.ascontiguousarray(codes, np.uint8)), _p(np.ascontiguousarray(scales, np.uint16)), _p(out))
    return out


def kv4_quant_vtile(v_tile):
    """v [16 keys][4][256] fp16 -> (codes [4][256][8] u8, stat pairs [4][256][2] u16)."""
    v_tile = np.ascontiguousarray(v_tile, np.float16).reshape(16, KV_HEADS, HEAD_DIM)
    codes, stats = np.zeros((KV_HEADS, HEAD_DIM, 8), np.uint8), np.zeros((KV_HEADS, HEAD_DIM, 2), np.uint16)
    _o.yahkv_oracle_kv4_quant_vtile(_p(v_tile.view(np.uint16)), _p(codes), _p(stats))
    return codes, stats


def kv4_deq_vtile(codes, stats):
    out = np.zeros((16, KV_HEADS, HEAD_DIM), np.float32)
    _o.yahkv_oracle_kv4_deq_vtile(_p(np.ascontiguousarray(codes, np.uint8)), _p(np.ascontiguousarray(stats, np.uint16)), _p(out))
    return out


class Kv4Pool:
    """One layer's kv4a16 pools on the host in the library's layout (64-token pages of four 16-key tiles); the
    counterpart of Kv8Pool."""

    def __init__(self, num_pages):
        self.num_pages = num_pages
        self.kcodes = np.zeros((num_pages, KV_HEADS, PAGE_TOKENS, 128), np.uint8)
        self.kscales = np.zeros((num_pages, KV_HEADS, PAGE_TOKENS, 8, 2), np.uint16)
        self.vcodes = np.zeros((num_pages, KV_HEADS, PAGE_TOKENS // 16, HEAD_DIM, 8), np.uint8)
        self.vstats = np.zeros((num_pages, KV_HEADS, PAGE_TOKENS // 16, HEAD_DIM, 2), np.uint16)

    new_sequence = staticmethod(Kv8Pool.new_sequence)

    def append(self, table, pos0, k, v, open_tile, mean):
        table = np.ascontiguousarray(table, np.int32)
        k = np.ascontiguousarray(k, np.float16)
        v = np.ascontiguousarray(v, np.float16)
        _o.yahkv_oracle_kv4_append_seq(PAGE_TOKENS, self.num_pages, _p(self.kcodes), _p(self.kscales), _p(self.vcodes),
                                       _p(self.vstats), _p(open_tile), _p(mean), _p(table), len(table),
                                       ctypes.c_int64(pos0), k.shape[0], _p(k.view(np.uint16)), _p(v.view(np.uint16)))

    def attend_decode_f64(self, table, n_keys, q, open_tile, gate=None, scale=1.0 / 16.0, threads=THREADS):
        table = np.ascontiguousarray(table, np.int32)
        q = np.ascontiguousarray(q, np.float16)
        gate = None if gate is None else np.ascontiguousarray(gate, np.float32)
        out = np.zeros((Q_HEADS, HEAD_DIM), np.float64)
        _o.yahkv_oracle_kv4_attend_decode_f64(PAGE_TOKENS, self.num_pages, _p(self.kcodes), _p(self.kscales),
                                              _p(self.vcodes), _p(self.vstats), _p(open_tile), _p(table), len(table),
                                              ctypes.c_int64(n_keys), _p(q.view(np.uint16)), _p(gate),
                                              ctypes.c_double(scale), _p(out), threads)
        return out

    def dequantized(self, table, n_keys, open_tile, threads=THREADS):
        """(K rotated by H256 / 16, V) [n_keys][4][256] f32 of one sequence as attention sees them."""
        table = np.ascontiguousarray(table, np.int32)
        validate_table(table, self.num_pages)
        K = np.zeros((n_keys, KV_HEADS, HEAD_DIM), np.float32)
        V = np.zeros((n_keys, KV_HEADS, HEAD_DIM), np.float32)
        _o.yahkv_oracle_kv4_dequantize(PAGE_TOKENS, self.num_pages, _p(self.kcodes), _p(self.kscales), _p(self.vcodes),
                                       _p(self.vstats), _p(open_tile), _p(table), len(table), ctypes.c_int64(n_keys),
                                       _p(K), _p(V), threads)
        return K, V

    def attend_prefill_f64(self, table, start, q, open_tile, q_begin=0, q_end=None, gate=None, scale=1.0 / 16.0):
        """Causal attention of chunk rows [q_begin, q_end) over the cache after the chunk's append, in float64, with q
        rotated like the cached K (dattn_q_check.py:203): the same numbers as attending over un-rotated rows."""
        q = np.ascontiguousarray(q, np.float16)
        q_end = q.shape[0] if q_end is None else q_end
        K, V = self.dequantized(table, start + q.shape[0], open_tile)
        K, V = K.astype(np.float64), V.astype(np.float64)
        out = np.zeros((q_end - q_begin, Q_HEADS, HEAD_DIM), np.float64)
        group = Q_HEADS // KV_HEADS
        for i in range(q_begin, q_end):
            vis = start + i + 1
            qr = hadamard256_f64(q[i].astype(np.float64))
            for h in range(Q_HEADS):
                kvh = h // group
                s_ = (K[:vis, kvh] @ qr[h]) * scale
                w = np.exp(s_ - s_.max())
                o = (w @ V[:vis, kvh]) / w.sum()
                if gate is not None:
                    o = o / (1.0 + np.exp(-np.asarray(gate[i, h], np.float64)))
                out[i - q_begin, h] = o
        return out

