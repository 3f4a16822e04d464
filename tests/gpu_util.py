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
