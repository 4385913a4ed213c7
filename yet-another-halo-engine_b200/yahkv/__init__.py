"""ctypes binding of libyahkv.so, the C ABI declared in include/yahkv.h.

This is the Python face of the library for tests and benchmarks; the product is the shared library itself. There is
no fallback of any kind: if libyahkv.so has not been built, importing this module raises, and hot-path calls on a
context without a GPU return YAHKV_ERR_NO_DEVICE.

`KvCache` mirrors the calls the reference engine makes on this path (engine/model/loom_decoder.hpp:254-268: append,
then attend over keys 0..pos, then the merge with the sigmoid gate), batched over sequences.
"""
import ctypes
import os
import subprocess

import numpy as np

_PKG_DIR = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
LIB_PATH = os.path.join(_PKG_DIR, "libyahkv.so")
INCLUDE_DIR = os.path.join(os.path.dirname(_PKG_DIR), "include")

FMT_Q8_0, FMT_Q4_0, FMT_KV8A16, FMT_KV4A16, FMT_F16 = 0, 1, 2, 3, 4
SIDE_K, SIDE_V = 0, 1
OUT_F16, OUT_F32 = 0, 1
KERNEL_APPEND, KERNEL_DECODE_PART, KERNEL_DECODE_COMBINE, KERNEL_PREFILL, KERNEL_PREFILL_DEQUANT = 0, 1, 2, 3, 4
OK = 0
ERR_INVALID, ERR_NO_PAGES, ERR_CUDA, ERR_NO_DEVICE, ERR_ORDER, ERR_CAPACITY = -1, -2, -3, -4, -5, -6

Q_HEADS, KV_HEADS, HEAD_DIM, PAGE_TOKENS, BLOCKS = 24, 4, 256, 64, 8


def code_bytes(fmt):
    return 512 if fmt == FMT_F16 else (128 if fmt in (FMT_Q4_0, FMT_KV4A16) else 256)


def bytes_per_token(fmt):
    """K + V bytes one cached token takes in one layer (codes + fp16 scales, all 4 kv heads)."""
    if fmt == FMT_KV8A16:     # K: 256 B + 2 pairs per head; V: 256 B + a sixteenth of 256 pairs per head
        return KV_HEADS * (256 + 8) + KV_HEADS * (256 + 64)
    if fmt == FMT_KV4A16:     # K: 128 B + 8 pairs per head; V: 128 B + a sixteenth of 256 pairs per head
        return KV_HEADS * (128 + 32) + KV_HEADS * (128 + 64)
    if fmt == FMT_F16:        # fp16 rows, no scales
        return 2 * KV_HEADS * 512
    return 2 * KV_HEADS * (code_bytes(fmt) + BLOCKS * 2)


def page_shapes(fmt, side):
    """(codes shape, scales shape) of one page record as yahkv_read_page returns it."""
    if fmt == FMT_F16:
        return (KV_HEADS, PAGE_TOKENS, 512), (KV_HEADS, PAGE_TOKENS, 0)
    if fmt not in (FMT_KV8A16, FMT_KV4A16):
        return (KV_HEADS, PAGE_TOKENS, code_bytes(fmt)), (KV_HEADS, PAGE_TOKENS, BLOCKS)
    wide = fmt == FMT_KV8A16
    if side == SIDE_K:
        return (KV_HEADS, PAGE_TOKENS, 256 if wide else 128), (KV_HEADS, PAGE_TOKENS, 2 if wide else 8, 2)
    return (KV_HEADS, PAGE_TOKENS // 16, HEAD_DIM, 16 if wide else 8), (KV_HEADS, PAGE_TOKENS // 16, HEAD_DIM, 2)


class Config(ctypes.Structure):
    _fields_ = [
        ("device", ctypes.c_int32),
        ("n_layers", ctypes.c_int32),
        ("n_q_heads", ctypes.c_int32),
        ("n_kv_heads", ctypes.c_int32),
        ("head_dim", ctypes.c_int32),
        ("page_tokens", ctypes.c_int32),
        ("num_pages", ctypes.c_int32),
        ("fmt", ctypes.c_int32),
        ("max_seqs", ctypes.c_int32),
        ("max_pages_per_seq", ctypes.c_int32),
        ("max_splits", ctypes.c_int32),
        ("max_batch_tokens", ctypes.c_int32),
        ("softmax_scale", ctypes.c_float),
        ("kv_head_begin", ctypes.c_int32),
        ("kv_head_count", ctypes.c_int32),
        ("max_prefill_keys", ctypes.c_int32),
    ]


class NoAllocArgs(ctypes.Structure):
    """yahkv_noalloc_args: everything yahkv_attend_decode_noalloc reads; the caller owns all of it."""
    _fields_ = [
        ("fmt", ctypes.c_int32),
        ("n_layers", ctypes.c_int32),
        ("num_pages", ctypes.c_int32),
        ("layer", ctypes.c_int32),
        ("kcodes", ctypes.c_void_p),
        ("vcodes", ctypes.c_void_p),
        ("kscales", ctypes.c_void_p),
        ("vscales", ctypes.c_void_p),
        ("tables_dev", ctypes.c_void_p),
        ("table_stride", ctypes.c_int32),
        ("n_seqs", ctypes.c_int32),
        ("lens_dev", ctypes.c_void_p),
        ("q_dev", ctypes.c_void_p),
        ("gate_dev", ctypes.c_void_p),
        ("out_dev", ctypes.c_void_p),
        ("out_dtype", ctypes.c_int32),
        ("n_splits", ctypes.c_int32),
        ("softmax_scale", ctypes.c_float),
        ("stream", ctypes.c_void_p),
    ]


NOALLOC_MAX_SEQS, NOALLOC_MAX_UNITS = 256, 1024


class YahkvError(RuntimeError):
    def __init__(self, code, message):
        super().__init__(f"{code} ({_error_name(code)}): {message}")
        self.code = code
        self.message = message


def build(verbose=False):
    """Compile libyahkv.so for sm_100a in the package directory (nvcc cross-compiles without a GPU)."""
    r = subprocess.run(["make", "-C", _PKG_DIR, "-j4"], capture_output=True, text=True)
    if verbose or r.returncode:
        print(r.stdout[-4000:], r.stderr[-4000:])
    if r.returncode:
        raise RuntimeError("building libyahkv.so failed")


_c = ctypes
_VP, _I32, _I64 = _c.c_void_p, _c.c_int32, _c.c_int64
_PI32, _PI64 = _c.POINTER(_c.c_int32), _c.POINTER(_c.c_int64)

# name -> (restype, argtypes): every entry point include/yahkv.h declares.
SIGNATURES = {
    "yahkv_create": (_I32, [_c.POINTER(Config), _c.POINTER(_VP)]),
    "yahkv_destroy": (None, [_VP]),
    "yahkv_last_error": (_c.c_char_p, [_VP]),
    "yahkv_error_name": (_c.c_char_p, [_I32]),
    "yahkv_seq_create": (_I32, [_VP, _PI32]),
    "yahkv_seq_free": (_I32, [_VP, _I32]),
    "yahkv_seq_reserve": (_I32, [_VP, _I32, _I64]),
    "yahkv_seq_set_table": (_I32, [_VP, _I32, _VP, _I32]),
    "yahkv_seq_table": (_I32, [_VP, _I32, _c.POINTER(_PI32), _PI32]),
    "yahkv_seq_len": (_I32, [_VP, _I32, _I32, _PI64]),
    "yahkv_seq_set_len": (_I32, [_VP, _I32, _I32, _I64]),
    "yahkv_pages_free": (_I32, [_VP, _PI32]),
    "yahkv_seq_set_kmean": (_I32, [_VP, _I32, _I32, _VP]),
    "yahkv_read_open_tile": (_I32, [_VP, _I32, _I32, _VP]),
    "yahkv_append": (_I32, [_VP, _I32, _I32, _VP, _VP, _VP, _VP, _VP]),
    "yahkv_rope_append": (_I32, [_VP, _I32, _I32, _VP, _VP, _VP, _VP, _VP, _VP, _VP, ctypes.c_float, _VP, _VP]),
    "yahkv_append_slots": (_I32, [_VP, _I32, _I32, _VP, _VP, _VP, _VP]),
    "yahkv_attend_decode": (_I32, [_VP, _I32, _I32, _VP, _VP, _VP, _VP, _I32, _I32, _VP]),
    "yahkv_attend_decode_qraw": (_I32, [_VP, _I32, _I32, _VP, _VP, _VP, ctypes.c_float, _VP, _VP, _I32, _I32, _VP]),
    "yahkv_attend_prefill": (_I32, [_VP, _I32, _I32, _VP, _VP, _VP, _VP, _VP, _I32, _VP]),
    "yahkv_attend_prefill_qraw": (_I32, [_VP, _I32, _I32, _VP, _VP, _VP, _VP, ctypes.c_float, _VP, _VP, _I32, _VP]),
    "yahkv_decode_step_host": (_I32, [_VP, _I32, _I32, _VP, _VP, _VP, _VP, _VP, _VP, _I32]),
    "yahkv_decode_step_host_async": (_I32, [_VP, _I32, _I32, _VP, _VP, _VP, _VP, _VP, _VP, _I32]),
    "yahkv_decode_step_host_wait": (_I32, [_VP]),
    "yahkv_read_page": (_I32, [_VP, _I32, _I32, _I32, _VP, _VP]),
    "yahkv_write_page": (_I32, [_VP, _I32, _I32, _I32, _VP, _VP]),
    "yahkv_export_token": (_I32, [_VP, _I32, _I32, _I64, _VP, _VP]),
    "yahkv_sync": (_I32, [_VP]),
    "yahkv_batch_create": (_I32, [_VP, _I32, _VP, _c.POINTER(_VP)]),
    "yahkv_batch_destroy": (None, [_VP]),
    "yahkv_batch_prepare": (_I32, [_VP, _I32, _PI32, _VP]),
    "yahkv_batch_set_splits": (_I32, [_VP, _I32]),
    "yahkv_batch_plan": (_I32, [_VP, _VP]),
    "yahkv_batch_decode_layer": (_I32, [_VP, _I32, _VP, _VP, _VP, _VP, _VP, _I32, _VP]),
    "yahkv_batch_decode_layer_raw": (_I32, [_VP, _I32, _VP, _VP, _VP, _VP, _VP, ctypes.c_float, _VP, _VP, _I32, _VP]),
    "yahkv_batch_advance": (_I32, [_VP, _VP]),
    "yahkv_batch_commit": (_I32, [_VP, _I32]),
    "yahkv_snapshot_save": (_I32, [_VP, _I32, _VP, _c.c_char_p]),
    "yahkv_snapshot_load": (_I32, [_VP, _c.c_char_p, _VP, _PI32]),
    "yahkv_device_bytes": (_I32, [_VP, _PI64]),
    "yahkv_launch_count": (_I32, [_VP, _PI64]),
    "yahkv_attend_decode_noalloc": (_I32, [_c.POINTER(NoAllocArgs), _c.c_char_p, _I32]),
    "yahkv_noalloc_status": (_I32, [_PI32, _VP]),
    "yahkv_debug_wait_timeout": (_I32, [_VP, _I64, _VP]),
    "yahkv_debug_set_prefill_sms": (_I32, [_VP, _I32]),
    "yahkv_kernel_timing": (_I32, [_VP, _I32]),
    "yahkv_kernel_timing_read": (_I32, [_VP, _I32, _c.POINTER(_c.c_double), _PI64]),
}


def _load():
    if not os.path.exists(LIB_PATH):
        raise ImportError(f"{LIB_PATH} is missing: build it first (make -C {_PKG_DIR}); there is no fallback path")
    lib = ctypes.CDLL(LIB_PATH)
    for name, (res, args) in SIGNATURES.items():
        fn = getattr(lib, name)
        fn.restype, fn.argtypes = res, args
    return lib


lib = _load()


def _error_name(code):
    return lib.yahkv_error_name(code).decode()


def _ptr(x):
    """Device or host address of a tensor / array / int / None as a c_void_p."""
    if x is None:
        return None
    if isinstance(x, int):
        return ctypes.c_void_p(x)
    if isinstance(x, np.ndarray):
        return x.ctypes.data_as(ctypes.c_void_p)
    if hasattr(x, "data_ptr"):  # torch tensor
        return ctypes.c_void_p(x.data_ptr())
    raise TypeError(f"cannot take the address of {type(x)}")


def _i32(a):
    return np.ascontiguousarray(a, dtype=np.int32)


def device_codes(fmt, codes, side):
    """GGUF code bytes (as read_page returns them) -> the form the device pools hold: q8_0 V bytes with the sign bit
    flipped (u = code + 128); q8_0 K bytes and q4_0 unchanged. The same call converts back. For callers that build
    device pools themselves (attend_decode_noalloc)."""
    codes = np.ascontiguousarray(codes, np.uint8)
    return codes ^ np.uint8(0x80) if fmt == FMT_Q8_0 and side == SIDE_V else codes


def attend_decode_noalloc(*, fmt, n_layers, num_pages, layer, kcodes, vcodes, kscales, vscales, tables, table_stride,
                          n_seqs, lens, q, out, gate=None, out_dtype=OUT_F16, n_splits=1, softmax_scale=0.0,
                          stream=None):
    """Context-free decode attention for hosts that may not allocate on the GPU: every buffer is the caller's, the
    split-K scratch is a static array inside the library. Raises YahkvError when the request is refused."""
    def addr(x):
        p = _ptr(x)
        return None if p is None else p.value
    args = NoAllocArgs(fmt, n_layers, num_pages, layer, addr(kcodes), addr(vcodes), addr(kscales), addr(vscales),
                       addr(tables), table_stride, n_seqs, addr(lens), addr(q), addr(gate), addr(out), out_dtype,
                       n_splits, softmax_scale, addr(stream))
    err = ctypes.create_string_buffer(256)
    rc = lib.yahkv_attend_decode_noalloc(ctypes.byref(args), err, len(err))
    if rc != OK:
        raise YahkvError(rc, err.value.decode())


def noalloc_status(status_host, stream=None):
    """Queues the copy of the no-allocation path's status word into `status_host` (an int32 array or pinned tensor of
    one element) on `stream`; read it after synchronising the stream."""
    rc = lib.yahkv_noalloc_status(ctypes.cast(_ptr(status_host), _PI32), _ptr(stream))
    if rc != OK:
        raise YahkvError(rc, "noalloc_status: no yahkv_attend_decode_noalloc call has run on this device yet")


class DecodeBatch:
    """Device-resident decode stepping over a fixed set of sequences (yahkv_batch): plan / decode_layer / advance
    touch no host state and may be captured into a CUDA graph; prepare and commit are the host-side bookends."""

    def __init__(self, cache, seq_ids):
        self.cache = cache
        seq_ids = _i32(seq_ids)
        self.n = len(seq_ids)
        self._h = ctypes.c_void_p()
        cache._check(lib.yahkv_batch_create(cache._h, self.n, _ptr(seq_ids), ctypes.byref(self._h)))

    def close(self):
        if self._h:
            lib.yahkv_batch_destroy(self._h)
            self._h = ctypes.c_void_p()

    def prepare(self, horizon_steps, stream=None):
        """Returns True when the unit layout changed (a captured graph must then be captured again)."""
        changed = ctypes.c_int32()
        self.cache._check(lib.yahkv_batch_prepare(self._h, horizon_steps, ctypes.byref(changed), _ptr(stream)))
        return bool(changed.value)

    def plan(self, stream=None):
        self.cache._check(lib.yahkv_batch_plan(self._h, _ptr(stream)))

    def set_splits(self, n_splits):
        """Split-K units per (sequence, kv head) of the longest sequence from the next prepare() on; 0 = automatic."""
        self.cache._check(lib.yahkv_batch_set_splits(self._h, int(n_splits)))

    def decode_layer(self, layer, k, v, q, out, gate=None, out_dtype=OUT_F16, stream=None):
        self.cache._check(lib.yahkv_batch_decode_layer(self._h, layer, _ptr(k), _ptr(v), _ptr(q), _ptr(gate), _ptr(out),
                                                       out_dtype, _ptr(stream)))

    def decode_layer_raw(self, layer, q, k, v, q_weight, k_weight, eps, out, gate=None, out_dtype=OUT_F16, stream=None):
        """decode_layer on the raw f32 projections: norm + RoPE + append of K / V, the query side in the part kernel."""
        self.cache._check(lib.yahkv_batch_decode_layer_raw(self._h, layer, _ptr(q), _ptr(k), _ptr(v), _ptr(q_weight),
                                                           _ptr(k_weight), float(eps), _ptr(gate), _ptr(out), out_dtype,
                                                           _ptr(stream)))

    def advance(self, stream=None):
        self.cache._check(lib.yahkv_batch_advance(self._h, _ptr(stream)))

    def commit(self, steps):
        self.cache._check(lib.yahkv_batch_commit(self._h, steps))


class KvCache:
    """One context = one GPU's pools, block tables and allocator (yahkv_ctx)."""

    def __init__(self, *, device=0, n_layers=1, num_pages=64, fmt=FMT_Q8_0, max_seqs=8, max_pages_per_seq=64,
                 max_splits=0, max_batch_tokens=0, softmax_scale=0.0, n_q_heads=Q_HEADS, n_kv_heads=KV_HEADS,
                 head_dim=HEAD_DIM, page_tokens=PAGE_TOKENS, kv_head_begin=0, kv_head_count=0, max_prefill_keys=0):
        self.cfg = Config(device, n_layers, n_q_heads, n_kv_heads, head_dim, page_tokens, num_pages, fmt, max_seqs,
                          max_pages_per_seq, max_splits, max_batch_tokens, softmax_scale, kv_head_begin, kv_head_count,
                          max_prefill_keys)
        self.fmt = fmt
        self._h = ctypes.c_void_p()
        rc = lib.yahkv_create(ctypes.byref(self.cfg), ctypes.byref(self._h))
        if rc != OK:
            raise YahkvError(rc, lib.yahkv_last_error(None).decode())

    def close(self):
        if self._h:
            lib.yahkv_destroy(self._h)
            self._h = ctypes.c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def _check(self, rc):
        if rc != OK:
            raise YahkvError(rc, lib.yahkv_last_error(self._h).decode())

    # ---- allocator / tables ----
    def seq_create(self):
        s = ctypes.c_int32(-1)
        self._check(lib.yahkv_seq_create(self._h, ctypes.byref(s)))
        return s.value

    def seq_free(self, seq):
        self._check(lib.yahkv_seq_free(self._h, seq))

    def seq_reserve(self, seq, n_tokens):
        self._check(lib.yahkv_seq_reserve(self._h, seq, n_tokens))

    def seq_set_table(self, seq, pages):
        pages = _i32(pages)
        self._check(lib.yahkv_seq_set_table(self._h, seq, _ptr(pages), len(pages)))

    def seq_table(self, seq):
        p, n = _PI32(), ctypes.c_int32()
        self._check(lib.yahkv_seq_table(self._h, seq, ctypes.byref(p), ctypes.byref(n)))
        return np.ctypeslib.as_array(p, shape=(n.value,)).copy() if n.value else np.zeros(0, np.int32)

    def seq_len(self, seq, layer=0):
        n = ctypes.c_int64()
        self._check(lib.yahkv_seq_len(self._h, seq, layer, ctypes.byref(n)))
        return n.value

    def seq_set_len(self, seq, length, layer=-1):
        self._check(lib.yahkv_seq_set_len(self._h, seq, layer, length))

    def pages_free(self):
        n = ctypes.c_int32()
        self._check(lib.yahkv_pages_free(self._h, ctypes.byref(n)))
        return n.value

    # ---- hot path ----
    def append(self, layer, seq_ids, positions, k, v, stream=None):
        seq_ids = _i32(seq_ids)
        positions = np.ascontiguousarray(positions, dtype=np.int64)
        assert len(seq_ids) == len(positions)
        self._check(lib.yahkv_append(self._h, layer, len(seq_ids), _ptr(seq_ids), _ptr(positions), _ptr(k), _ptr(v),
                                     _ptr(stream)))

    def rope_append(self, layer, seq_ids, positions, q, k, v, q_weight, k_weight, eps, q_out, stream=None):
        """Fused QK RMSNorm + RoPE + append: f32 device q [n][24][256], k, v [n][4][256]; q_out fp16 [n][24][256]."""
        seq_ids = _i32(seq_ids)
        positions = np.ascontiguousarray(positions, dtype=np.int64)
        assert len(seq_ids) == len(positions)
        self._check(lib.yahkv_rope_append(self._h, layer, len(seq_ids), _ptr(seq_ids), _ptr(positions), _ptr(q), _ptr(k),
                                          _ptr(v), _ptr(q_weight), _ptr(k_weight), float(eps), _ptr(q_out), _ptr(stream)))

    def append_slots(self, layer, n_tokens, slot_mapping, k, v, stream=None):
        self._check(lib.yahkv_append_slots(self._h, layer, n_tokens, _ptr(slot_mapping), _ptr(k), _ptr(v),
                                           _ptr(stream)))

    def attend_decode(self, layer, seq_ids, q, out, gate=None, out_dtype=OUT_F16, n_splits=0, stream=None):
        seq_ids = _i32(seq_ids)
        self._check(lib.yahkv_attend_decode(self._h, layer, len(seq_ids), _ptr(seq_ids), _ptr(q), _ptr(gate),
                                            _ptr(out), out_dtype, n_splits, _ptr(stream)))

    def attend_decode_qraw(self, layer, seq_ids, q_raw, q_weight, eps, out, gate=None, out_dtype=OUT_F16, n_splits=0,
                           stream=None):
        """attend_decode on the raw f32 q projection: the kernel's prologue norms and rotates each head row."""
        seq_ids = _i32(seq_ids)
        self._check(lib.yahkv_attend_decode_qraw(self._h, layer, len(seq_ids), _ptr(seq_ids), _ptr(q_raw), _ptr(q_weight),
                                                 float(eps), _ptr(gate), _ptr(out), out_dtype, n_splits, _ptr(stream)))

    def attend_prefill(self, layer, seq_ids, chunk_lens, q, out, gate=None, out_dtype=OUT_F16, stream=None):
        seq_ids, chunk_lens = _i32(seq_ids), _i32(chunk_lens)
        self._check(lib.yahkv_attend_prefill(self._h, layer, len(seq_ids), _ptr(seq_ids), _ptr(chunk_lens), _ptr(q),
                                             _ptr(gate), _ptr(out), out_dtype, _ptr(stream)))

    def attend_prefill_qraw(self, layer, seq_ids, chunk_lens, q_raw, q_weight, eps, out, gate=None, out_dtype=OUT_F16,
                            stream=None):
        """attend_prefill on the raw f32 q projection: the kernel's prologue norms and rotates its rows."""
        seq_ids, chunk_lens = _i32(seq_ids), _i32(chunk_lens)
        self._check(lib.yahkv_attend_prefill_qraw(self._h, layer, len(seq_ids), _ptr(seq_ids), _ptr(chunk_lens),
                                                  _ptr(q_raw), _ptr(q_weight), float(eps), _ptr(gate), _ptr(out),
                                                  out_dtype, _ptr(stream)))

    def decode_step_host(self, layer, seq_ids, k, v, q, out, gate=None, out_dtype=OUT_F16):
        seq_ids = _i32(seq_ids)
        self._check(lib.yahkv_decode_step_host(self._h, layer, len(seq_ids), _ptr(seq_ids), _ptr(k), _ptr(v), _ptr(q),
                                               _ptr(gate), _ptr(out), out_dtype))

    def decode_step_host_async(self, layer, seq_ids, k, v, q, out, gate=None, out_dtype=OUT_F16):
        """Queues the step; the (page-locked) buffers must stay alive and untouched until decode_step_host_wait()."""
        seq_ids = _i32(seq_ids)
        self._check(lib.yahkv_decode_step_host_async(self._h, layer, len(seq_ids), _ptr(seq_ids), _ptr(k), _ptr(v),
                                                     _ptr(q), _ptr(gate), _ptr(out), out_dtype))

    def decode_step_host_wait(self):
        self._check(lib.yahkv_decode_step_host_wait(self._h))

    # ---- inspection ----
    def seq_set_kmean(self, seq, mean, layer=-1):
        """kv8a16 / kv4a16: the per-channel K mean [4][256] f32 of a sequence (before its first append)."""
        mean = np.ascontiguousarray(mean, np.float32).reshape(KV_HEADS, HEAD_DIM)
        self._check(lib.yahkv_seq_set_kmean(self._h, seq, layer, _ptr(mean)))

    def read_open_tile(self, seq, layer):
        """kv8a16 / kv4a16: the current open V tile [4][256][16] as float16."""
        tile = np.zeros((KV_HEADS, HEAD_DIM, 16), np.float16)
        self._check(lib.yahkv_read_open_tile(self._h, seq, layer, _ptr(tile)))
        return tile

    def read_page(self, layer, side, page):
        cs, ss = page_shapes(self.fmt, side)
        codes = np.zeros(cs, np.uint8)
        scales = np.zeros(ss, np.uint16)
        self._check(lib.yahkv_read_page(self._h, layer, side, page, _ptr(codes), _ptr(scales)))
        return codes, scales

    def write_page(self, layer, side, page, codes, scales):
        codes = np.ascontiguousarray(codes, dtype=np.uint8)
        scales = np.ascontiguousarray(scales, dtype=np.uint16)
        self._check(lib.yahkv_write_page(self._h, layer, side, page, _ptr(codes), _ptr(scales)))

    def export_token(self, layer, seq, pos):
        nb = KV_HEADS * BLOCKS * (2 + code_bytes(self.fmt) // BLOCKS)
        k, v = np.zeros(nb, np.uint8), np.zeros(nb, np.uint8)
        self._check(lib.yahkv_export_token(self._h, layer, seq, pos, _ptr(k), _ptr(v)))
        return k, v

    def snapshot_save(self, seq_ids, path):
        seq_ids = _i32(seq_ids)
        self._check(lib.yahkv_snapshot_save(self._h, len(seq_ids), _ptr(seq_ids), str(path).encode()))

    def snapshot_load(self, path, max_seqs=1024):
        """Loads every sequence of the snapshot; returns their new ids in the saved order."""
        ids = np.zeros(max_seqs, np.int32)
        n = ctypes.c_int32(max_seqs)
        self._check(lib.yahkv_snapshot_load(self._h, str(path).encode(), _ptr(ids), ctypes.byref(n)))
        return ids[:n.value].tolist()

    def sync(self):
        self._check(lib.yahkv_sync(self._h))

    def device_bytes(self):
        n = ctypes.c_int64()
        self._check(lib.yahkv_device_bytes(self._h, ctypes.byref(n)))
        return n.value

    def kernel_timing(self, enable):
        self._check(lib.yahkv_kernel_timing(self._h, 1 if enable else 0))

    def kernel_timing_read(self, kernel):
        """(total device milliseconds, launches) of one kernel since timing was enabled."""
        ms, n = ctypes.c_double(), ctypes.c_int64()
        self._check(lib.yahkv_kernel_timing_read(self._h, kernel, ctypes.byref(ms), ctypes.byref(n)))
        return ms.value, n.value

    def debug_wait_timeout(self, limit_us, stream=None):
        """Runs a device wait that cannot succeed for at most limit_us; the next sync() then reports it."""
        self._check(lib.yahkv_debug_wait_timeout(self._h, int(limit_us), _ptr(stream)))

    def debug_set_prefill_sms(self, n_sm):
        self._check(lib.yahkv_debug_set_prefill_sms(self._h, int(n_sm)))

    def launch_count(self):
        n = ctypes.c_int64()
        self._check(lib.yahkv_launch_count(self._h, ctypes.byref(n)))
        return n.value
