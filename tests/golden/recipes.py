"""Seeded input recipes shared by the golden-vector generator and the tests (inputs are re-derived, never stored)."""
import numpy as np


def codec_input(n_blocks=4096, seed=0):
    """fp16-representable values ~ N(0,1) with sparse x20 outliers, as f32 (what append widens its fp16 input to)."""
    rng = np.random.default_rng(seed)
    x = rng.standard_normal(n_blocks * 32).astype(np.float32)
    x[rng.integers(0, x.size, n_blocks // 4)] *= 20
    x[:32] = 0.0                      # an all-zero block (d = 0)
    x[32:64] = np.float32(0.5)        # a constant block
    x[64:96] = -x[96:128]             # sign-mirrored pair: q4_0's "first of the largest" rule
    return x.astype(np.float16).astype(np.float32)


def checker_recipe(T=1024, pos=700, seed=5):
    """The data recipe of the reference's quantized-decode checker (engine/gpu/loom/tools/dattn_q_check.py:147-157),
    with 64-token pages: K, V ~ N(0,1) fp16, q = 0.3 N(0,1), gate ~ N(0,1), a permuted page table."""
    rng = np.random.default_rng(seed)
    npg = T // 64
    ptab = rng.permutation(npg).astype(np.int32)
    K = rng.standard_normal((T, 4, 256)).astype(np.float16)
    V = rng.standard_normal((T, 4, 256)).astype(np.float16)
    q = (0.3 * rng.standard_normal((24, 256))).astype(np.float16)
    gate = rng.standard_normal((24, 256)).astype(np.float32)
    return {"T": T, "pos": pos, "ptab": ptab, "K": K, "V": V, "q": q, "gate": gate}


def outlier_kv(n_tokens, seed=0, n_outliers=4, factor=20.0):
    """K, V [n][4][256] fp16 ~ N(0,1) with `n_outliers` fixed channels per head scaled by `factor` (the parity
    fixture's distribution), and the rng for whatever the caller draws next."""
    rng = np.random.default_rng(seed)
    ch = np.stack([rng.choice(256, n_outliers, replace=False) for _ in range(8)])  # per (side, head)
    K = rng.standard_normal((n_tokens, 4, 256)).astype(np.float32)
    V = rng.standard_normal((n_tokens, 4, 256)).astype(np.float32)
    for h in range(4):
        K[:, h, ch[h]] *= factor
        V[:, h, ch[4 + h]] *= factor
    return K.astype(np.float16), V.astype(np.float16), rng


def kv8a16_recipe(T=320, seed=5):
    """Data recipe of the reference's quantized-decode checker for its own cache formats
    (engine/gpu/loom/tools/dattn_q_check.py:147-157): a per-channel K mean m = 0.5 N(0,1), K = N(0,1) + m and
    V = N(0,1) as fp16 [T][1024], q = 0.3 N(0,1) f32 rounded to fp16, gate ~ N(0,1)."""
    rng = np.random.default_rng(seed)
    m = (0.5 * rng.standard_normal(1024)).astype(np.float32)
    K = (rng.standard_normal((T, 1024)) + m).astype(np.float16)
    V = rng.standard_normal((T, 1024)).astype(np.float16)
    q = (0.3 * rng.standard_normal((24, 256))).astype(np.float16)
    gate = rng.standard_normal((24, 256)).astype(np.float32)
    return {"T": T, "m": m, "K": K, "V": V, "q": q, "gate": gate}
