#!/usr/bin/env python3
"""Quality of the cache formats on the parity fixture's distribution: GGUF q8_0 / q4_0 (this library) against the
reference's own kv8a16 / kv4a16, whose numpy models are IMPORTED from the reference checkout
(engine/gpu/loom/tools/dattn_q_check.py: quant_k / deq_k :61-98, quant_vtile / deq_vtile :101-137) and not restated.

Data: 4,096 tokens, 4 KV heads x 256, K and V ~ N(0,1) as fp16 with four fixed outlier channels per head scaled x20
(tests/golden/recipes.py), 24 queries ~ N(0,1), float64 attention (scores K.q / 16, softmax, @ V) over the exact fp16
K/V and over each format's dequantized K/V. kv8a16 / kv4a16 centre K on a per-channel mean taken over the first
2,048 tokens (yah_kmean works on the first chunk, engine/gpu/loom/tools/gen_kvq.py:99-163) and quantize V per
16-key tile and channel.

Usage (where the reference checkout is present): python tests/golden/make_format_study.py <reference root>
Prints a markdown table; the copy in tests/golden/format_study.md was made this way."""
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.abspath(os.path.join(HERE, "..", ".."))
sys.path.insert(0, os.path.join(ROOT, "oracle"))
sys.path.insert(0, HERE)
import oracle as O  # noqa: E402
from recipes import outlier_kv  # noqa: E402


def attend(K, V, q):
    """float64 attention of q [24][256] over K, V [n][4][256] (GQA 6)."""
    out = np.zeros((24, 256))
    for h in range(24):
        s = K[:, h // 6] @ q[h] / 16.0
        p = np.exp(s - s.max())
        out[h] = (p / p.sum()) @ V[:, h // 6]
    return out


def main():
    ref = sys.argv[1]
    sys.path.insert(0, os.path.join(ref, "engine", "gpu", "loom", "tools"))
    import dattn_q_check as C   # the reference's models

    n = 4096
    K16, V16, rng = outlier_kv(n, seed=0)
    q = rng.standard_normal((24, 256))
    K, V = K16.astype(np.float64), V16.astype(np.float64)
    want = attend(K, V, q)
    rows = []

    def report(name, bytes_per_token, Kd, Vd):
        got = attend(Kd, Vd, q)
        rows.append((name, bytes_per_token, np.sqrt(((Kd - K) ** 2).mean()), np.sqrt(((Vd - V) ** 2).mean()),
                     np.abs(got - want).max(), np.sqrt(((got - want) ** 2).mean())))

    for name, fmt, b in (("q8_0 (GGUF, this library)", O.FMT_Q8_0, 2176), ("q4_0 (GGUF, this library)", O.FMT_Q4_0, 1152)):
        Kd = O.dequantize(O.quantize(K16.astype(np.float32), fmt), fmt).reshape(n, 4, 256).astype(np.float64)
        Vd = O.dequantize(O.quantize(V16.astype(np.float32), fmt), fmt).reshape(n, 4, 256).astype(np.float64)
        report(name, b, Kd, Vd)

    mean = K16[:2048].astype(np.float32).reshape(2048, 1024).mean(0).astype(np.float32)
    for name, bits, b in (("kv8a16 (reference)", 8, 1056 + 1280), ("kv4a16 (reference)", 4, 640 + 768)):
        Kd = np.zeros((n, 1024))
        for t in range(n):
            dw, sc = C.quant_k(K16[t].reshape(1024).astype(np.float32), mean, bits)
            x = C.deq_k(dw, sc, bits).astype(np.float64)
            if bits == 4:   # the 4-bit K lives in the rotated basis: rotate back for the comparison
                x = (x.reshape(4, 256) @ C.H / 16.0).reshape(1024)
            Kd[t] = x + mean
        Vd = np.zeros((n, 1024))
        Vf = V16.reshape(n, 1024).astype(np.float32)
        for t0 in range(0, n, 16):
            dw, st = C.quant_vtile(Vf[t0:t0 + 16], bits)
            Vd[t0:t0 + 16] = C.deq_vtile(dw, st, bits)
        report(name, b, Kd.reshape(n, 4, 256), Vd.reshape(n, 4, 256))

    print("| format | bytes / token / layer | rms error of K | rms error of V | attention max-abs error | attention rms error |")
    print("|---|---:|---:|---:|---:|---:|")
    for r in rows:
        print("| %s | %d | %.4f | %.4f | %.2e | %.2e |" % r)


if __name__ == "__main__":
    main()
