#!/usr/bin/env python3
"""Generates tests/golden/*.npz: known answers for the KV path made with the REFERENCE's own code, not with ours.

Run it where the reference checkout is present (the REF variable of oracle/Makefile points at it) and the `gguf`
package is installed:
    python tests/golden/make_golden.py
What produces each answer:
  * q8_0 blocks: the reference's QuantizeQ8_0 (engine/core/gguf_quant.cpp:310-320), compiled unchanged from its
    sources into oracle/_ref/libyah_ref_codec.so by oracle/Makefile.
  * q4_0 blocks: gguf.quants.quantize (the gguf package the reference's codec test pins, engine/tests/gguf_check.py:5;
    the reference has no q4_0 quantizer of its own).
  * dequantized values: the reference's Dequantize (engine/core/gguf_quant.cpp:291-308, Q8_0 :72-75, Q4_0 :48-51).
  * decode attention: the float64 numpy model of the reference's checker, engine/gpu/loom/tools/dattn_q_check.py:193-201
    (scores K.q/16, exp(s - max), normalise, @V, / (1 + exp(-gate))), over K/V dequantized by the reference decoder.
    That function is a closure inside the checker's main(), which needs an AMD GPU to run, so its six lines are
    evaluated here on the checker's own data recipe (seed 5: K, V ~ N(0,1) fp16, q = 0.3 N(0,1), gate ~ N(0,1),
    page table = rng.permutation(pages), T = 1024, pos = 700; dattn_q_check.py:147-157), with 64-token pages.
Inputs are not stored (they are re-derived from the seeds); outputs are stored as a SHA-256 of the full byte string
plus a readable prefix, and the attention outputs in full.
"""
import hashlib
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, os.path.join(ROOT, "oracle"))
sys.path.insert(0, HERE)
import oracle as O  # noqa: E402  (only for the ctypes handles of oracle/_ref; none of our restatement is called here)
from recipes import codec_input, checker_recipe  # noqa: E402

from gguf import GGMLQuantizationType as Q  # noqa: E402
from gguf.quants import quantize as gguf_quantize  # noqa: E402


def sha(a):
    return hashlib.sha256(np.ascontiguousarray(a).tobytes()).hexdigest()


def ref_blocks(x, fmt):
    if fmt == O.FMT_Q8_0:
        return O.ref_quantize_q8_0(x)
    return gguf_quantize(np.ascontiguousarray(x, np.float32).reshape(-1, 32), Q.Q4_0).reshape(-1)


def checker_attention(Kd, Vd, q, gate, n):
    """engine/gpu/loom/tools/dattn_q_check.py:193-201, with K/V already dequantized: [T][4][256] f32."""
    ref = np.zeros((24, 256))
    for hh in range(24):
        kv = hh // 6
        s = Kd[:n, kv].astype(np.float64) @ q[hh].astype(np.float64) / 16.0
        pr = np.exp(s - s.max())
        pr /= pr.sum()
        ref[hh] = (pr @ Vd[:n, kv].astype(np.float64)) / (1.0 + np.exp(-gate[hh].astype(np.float64)))
    return ref


def main():
    assert O.have_ref(), "oracle/_ref is not built: run `make -C oracle` with the reference checkout present"
    out = {}
    # ---- codec known answers ----
    x = codec_input()
    for name, fmt in (("q8_0", O.FMT_Q8_0), ("q4_0", O.FMT_Q4_0)):
        blocks = ref_blocks(x, fmt)
        out[f"codec_{name}_sha256"] = np.array(sha(blocks))
        out[f"codec_{name}_head"] = blocks[: 64 * O.block_bytes(fmt)].copy()
        deq = O.ref_dequantize(blocks, fmt)
        out[f"codec_{name}_deq_sha256"] = np.array(sha(deq))
        out[f"codec_{name}_deq_head"] = deq[:2048].copy()
    # ---- decode attention on the checker's recipe ----
    r = checker_recipe()
    n = r["pos"] + 1
    for name, fmt in (("q8_0", O.FMT_Q8_0), ("q4_0", O.FMT_Q4_0)):
        kb = ref_blocks(r["K"].astype(np.float32), fmt)
        vb = ref_blocks(r["V"].astype(np.float32), fmt)
        Kd = O.ref_dequantize(kb, fmt).reshape(r["T"], 4, 256)
        Vd = O.ref_dequantize(vb, fmt).reshape(r["T"], 4, 256)
        out[f"attn_{name}_kblocks_sha256"] = np.array(sha(kb))
        out[f"attn_{name}_vblocks_sha256"] = np.array(sha(vb))
        out[f"attn_{name}_gated"] = checker_attention(Kd, Vd, r["q"], r["gate"], n)
        out[f"attn_{name}_plain"] = checker_attention(Kd, Vd, r["q"], np.full_like(r["gate"], 1e9), n)
    np.savez_compressed(os.path.join(HERE, "kv_path.npz"), **out)
    print("wrote", os.path.join(HERE, "kv_path.npz"), {k: (v.shape if v.ndim else str(v)[:16]) for k, v in out.items()})


if __name__ == "__main__":
    main()
