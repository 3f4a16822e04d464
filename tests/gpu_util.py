"""Helpers shared by the GPU parity tests (seeded synthetic weights and activations)."""
import importlib

import numpy as np


def load_bt():
    mod = importlib.import_module("bit-ttt-engine_b200")
    mod.lib()
    return mod


def ternary_packed(rng, n, k, p_code3=0.0):
    """Uniform ternary weights (p = 1/3 each) as reference codes packed 4 per byte,
    row-major [n, k/4]; optionally sprinkles the unused code 11."""
    codes = rng.integers(0, 3, size=(n, k), dtype=np.uint8)  # 0 -> 0, 1 -> +1, 2 -> -1
    if p_code3 > 0:
        codes = np.where(rng.random((n, k)) < p_code3, 3, codes).astype(np.uint8)
    c = codes.reshape(n, k // 4, 4)
    return (c[..., 0] | (c[..., 1] << 2) | (c[..., 2] << 4) | (c[..., 3] << 6)).astype(np.uint8)


from oracle.staged import ATT_TOL, LOGIT_TOL, rel_err, staged_decode_step  # noqa: E402,F401


def seed_kv_caches(gpu, states, cfg, t0, rng):
    """Fills positions [0, t0) of every layer's Q8 KV cache with seeded random rows - the same
    bytes and scales on the GPU (bt_kv_import) and in the oracle's per-sequence states - and
    declares t0 positions consumed, so that the next decode step attends over a long context
    without t0 steps of prefill.  Scales are drawn around the magnitude real rows have."""
    n_kv, hd = cfg.n_kv_heads, cfg.hidden_dim // cfg.n_heads
    for li in range(cfg.num_layers):
        cache = gpu.kv_cache(li)
        for b, st in enumerate(states):
            kq = rng.integers(0, 256, size=(n_kv, t0, hd), dtype=np.uint8)
            vq = rng.integers(0, 256, size=(n_kv, t0, hd), dtype=np.uint8)
            ks = rng.uniform(0.005, 0.03, size=(n_kv, t0)).astype(np.float32)
            vs = rng.uniform(0.005, 0.03, size=(n_kv, t0)).astype(np.float32)
            cache.load(b, kq, ks, vq, vs)
            st.kq[li] = [np.ascontiguousarray(kq[:, t]) for t in range(t0)]
            st.vq[li] = [np.ascontiguousarray(vq[:, t]) for t in range(t0)]
            st.ks[li] = [np.ascontiguousarray(ks[:, t]) for t in range(t0)]
            st.vs[li] = [np.ascontiguousarray(vs[:, t]) for t in range(t0)]
    for st in states:
        st.pos = t0
    gpu.seek(t0)
