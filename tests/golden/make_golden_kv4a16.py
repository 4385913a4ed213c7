#!/usr/bin/env python3
"""Generates tests/golden/kv4a16.npz: known answers for the reference's own kv4a16 cache format, made with the
REFERENCE's numpy models of its quantizers, imported from its checker (engine/gpu/loom/tools/dattn_q_check.py:61-137:
quant_k, deq_k, quant_vtile, deq_vtile with bits = 4), not with this repository's restatement.

    python tests/golden/make_golden_kv4a16.py <path of the reference checkout>

Inputs are re-derived from seeds (recipes.kv8a16_recipe, the checker's own data recipe); stored are
  * the K code dwords and scale pairs of all 320 tokens in the reference's array layouts (kq [T][128] u32, ks [T][64]
    f16). In full, not as hashes: the model rotates in float64 and a kernel in f32, so K codes are compared under the
    checker's own bar (dequantized values within 1e-2, dattn_q_check.py:231-236), and the attention answer below is
    checked by handing these codes to the oracle;
  * per 16-key tile the V code dwords and (S, C') pairs (vq [tiles][1024][2] u32, vs [tiles][1024][2] f16): the first
    two tiles in full, all of them as SHA-256 (the V side is bit-exact);
  * decode attention at n = 300 keys (18 quantized tiles + an open tile of 12 keys), float64, by the checker's model
    (dattn_q_check.py:193-204: q rotated by H256 / 16, scores K.q / 16 over the DEQUANTIZED rotated K - m, exp(s - max),
    normalise, @ V with the open tile's keys in fp16, / (1 + exp(-gate))). That function is a closure inside the
    checker's main(), which needs an AMD GPU, so its lines are evaluated here.
"""
import hashlib
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, HERE)
from recipes import kv8a16_recipe  # noqa: E402


def sha(a):
    return hashlib.sha256(np.ascontiguousarray(a).tobytes()).hexdigest()


def main():
    ref = sys.argv[1]
    sys.dont_write_bytecode = True          # the reference tree is read-only
    sys.path.insert(0, os.path.join(ref, "engine", "gpu", "loom", "tools"))
    import dattn_q_check as C
    r = kv8a16_recipe()
    T, m, K, V = r["T"], r["m"], r["K"], r["V"]
    kq = np.zeros((T, 128), np.uint32)
    ks = np.zeros((T, 64), np.float16)
    Kd = np.zeros((T, 1024), np.float32)
    for p in range(T):
        kq[p], ks[p] = C.quant_k(K[p].astype(np.float32), m, 4)
        Kd[p] = C.deq_k(kq[p], ks[p], 4)
    tiles = T // 16
    vq = np.zeros((tiles, 1024, 2), np.uint32)
    vs = np.zeros((tiles, 1024, 2), np.float16)
    Vq = np.zeros((T, 1024), np.float32)
    for t in range(tiles):
        vq[t], vs[t] = C.quant_vtile(V[16 * t:16 * t + 16], 4)
        Vq[16 * t:16 * t + 16] = C.deq_vtile(vq[t], vs[t], 4)
    n = 300
    cur = (n - 1) // 16                      # the open tile: its keys are read in fp16
    Vd = Vq.copy()
    Vd[16 * cur:] = V[16 * cur:].astype(np.float32)
    qr = r["q"].astype(np.float64) @ C.H.T / 16.0
    out = {}
    for name, gate in (("gated", r["gate"]), ("plain", None)):
        o = np.zeros((24, 256))
        for hh in range(24):
            kv = hh // 6
            s = Kd[:n, kv * 256:kv * 256 + 256].astype(np.float64) @ qr[hh] / 16.0
            pr = np.exp(s - s.max())
            pr /= pr.sum()
            o[hh] = pr @ Vd[:n, kv * 256:kv * 256 + 256].astype(np.float64)
            if gate is not None:
                o[hh] /= 1.0 + np.exp(-gate[hh].astype(np.float64))
        out[name] = o
    np.savez_compressed(os.path.join(HERE, "kv4a16.npz"), kq=kq, ks=ks, vq_head=vq[:2], vs_head=vs[:2],
                        vq_sha=sha(vq), vs_sha=sha(vs), vd_sha=sha(Vq), kd_sha=sha(Kd),
                        attn_gated=out["gated"], attn_plain=out["plain"], n_keys=n)
    print("wrote kv4a16.npz", sha(kq)[:12], sha(vq)[:12], float(np.abs(out["plain"]).max()))


if __name__ == "__main__":
    main()
