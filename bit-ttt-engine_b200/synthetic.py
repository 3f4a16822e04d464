"""Seeded synthetic checkpoints with the shapes of the reference's model families.

No model weights ship with the reference, so tests and the benchmark build random-init
models of the right shape: ternary projections as packed 2-bit codes + one f32 scale,
dense embedding / lm_head (values representable in bf16), unit RMSNorm weights.
"""
from __future__ import annotations

from dataclasses import dataclass, field

import numpy as np

from .layers import pack_ternary
from .model import (BitLlama, BitLlamaConfig, T_EMBED, T_LM_HEAD, T_NORM1, T_NORM2, T_NORM_F, W_DOWN,
                    W_GATE, W_K, W_O, W_Q, W_TTT_DOWN, W_TTT_UP, W_UP, W_V)

TINY_TTT = BitLlamaConfig("ttt", 32000, 256, 4, 4, 4, 688, inner_lr=0.01)
TINY_LLAMA_TEST = BitLlamaConfig("llama", 1000, 256, 2, 8, 2, 512, max_position_embeddings=64)
TINYLLAMA_1B = BitLlamaConfig("llama", 32000, 2048, 22, 32, 4, 5632, max_position_embeddings=2048)
LLAMA3_8B = BitLlamaConfig("llama", 128256, 4096, 32, 32, 8, 14336, rope_theta=500000.0,
                           max_position_embeddings=4096)


@dataclass
class SyntheticWeights:
    cfg: BitLlamaConfig
    embed: np.ndarray
    lm_head: np.ndarray
    norm_f: np.ndarray
    layers: list = field(default_factory=list)  # dicts: norm1, norm2, kind -> (packed, scale, n, k)
    dense_f16: bool = False  # embedding and lm_head hold IEEE-half values (a converted checkpoint): keep them so


def _bf16_round(a: np.ndarray) -> np.ndarray:
    """Round f32 to the nearest bf16-representable value (ties to even), still f32."""
    u = np.ascontiguousarray(a, np.float32).view(np.uint32)
    r = ((u + 0x7FFF + ((u >> 16) & 1)) & 0xFFFF0000).astype(np.uint32)
    return r.view(np.float32)


def _ternary_codes(rng, n, k):
    codes = rng.integers(0, 3, size=(n, k // 4, 4), dtype=np.uint8)
    return (codes[..., 0] | (codes[..., 1] << 2) | (codes[..., 2] << 4) | (codes[..., 3] << 6)).astype(np.uint8)


def linear_shapes(cfg: BitLlamaConfig):
    """kind -> (n_out, k_in) for one block (model/block.rs:43-64, layers/ttt.rs:29-34,
    layers/attention.rs:121-129, layers/swiglu.rs:24-26)."""
    H, I = cfg.hidden_dim, cfg.intermediate_dim
    shapes = {W_GATE: (I, H), W_UP: (I, H), W_DOWN: (H, I)}
    if cfg.arch == "ttt":
        shapes.update({W_TTT_DOWN: (H // 4, H), W_TTT_UP: (H, H // 4)})
    else:
        hd = H // cfg.n_heads
        shapes.update({W_Q: (cfg.n_heads * hd, H), W_K: (cfg.n_kv_heads * hd, H),
                       W_V: (cfg.n_kv_heads * hd, H), W_O: (H, cfg.n_heads * hd)})
    return shapes


def _multi_basis_codes(rng, n, k, n_bases):
    """Random ternary bases in the converted layout [n, k/4, n_bases] with decreasing scales, the shape a
    greedy residual decomposition produces (tools/conversion/convert_llama_v2.py:28-72)."""
    planes = [_ternary_codes(rng, n, k) for _ in range(n_bases)]
    scales = np.array([0.016 / (2.6 ** b) for b in range(n_bases)], np.float32)
    return np.ascontiguousarray(np.stack(planes, axis=2)), scales


def make_weights(cfg: BitLlamaConfig, seed: int = 2000, from_latent: bool = True,
                 share_layers: bool = False, n_bases: int = 1) -> SyntheticWeights:
    """from_latent: draw N(0, 0.02) dense weights and run PackedTensor::pack on them (small
    models); otherwise draw the ternary codes uniformly (p = 1/3) with scale 0.016.
    n_bases > 1: every projection gets that many random ternary bases (converted-checkpoint layout).
    share_layers: reuse layer 0's host arrays for every layer (the device copies stay
    distinct) - keeps host-side generation of multi-GB models short."""
    rng = np.random.default_rng(seed)
    V, H = cfg.vocab_size, cfg.hidden_dim
    w = SyntheticWeights(cfg,
                         _bf16_round(rng.normal(0, 0.02, (V, H)).astype(np.float32)),
                         _bf16_round(rng.normal(0, 0.02, (V, H)).astype(np.float32)),
                         np.ones(H, np.float32))
    for li in range(cfg.num_layers):
        if share_layers and li > 0:
            w.layers.append(w.layers[0])
            continue
        layer = {"norm1": np.ones(H, np.float32), "norm2": np.ones(H, np.float32)}
        for kind, (n, k) in linear_shapes(cfg).items():
            if n_bases > 1:
                packed, scale = _multi_basis_codes(rng, n, k, n_bases)
            elif from_latent:
                dense = rng.normal(0, 0.02, (n, k)).astype(np.float32)
                packed, scale = pack_ternary(dense)
                packed = packed.reshape(n, k // 4)
            else:
                packed, scale = _ternary_codes(rng, n, k), 0.016
            layer[kind] = (packed, scale if n_bases > 1 else float(scale), n, k)
        w.layers.append(layer)
    return w


def shard_weights(w: SyntheticWeights, rank: int, size: int) -> SyntheticWeights:
    """This rank's tensor-parallel shard: q/k/v by heads and gate/up by rows (column-parallel),
    o_proj and down_proj by packed input columns (row-parallel); everything else replicated."""
    if size <= 1:
        return w
    cfg = w.cfg
    hd = cfg.hidden_dim // cfg.n_heads
    out = SyntheticWeights(cfg, w.embed, w.lm_head, w.norm_f, dense_f16=w.dense_f16)
    cache = {}
    for layer in w.layers:
        if id(layer) in cache:
            out.layers.append(cache[id(layer)])
            continue
        new = {"norm1": layer["norm1"], "norm2": layer["norm2"]}
        for kind, val in layer.items():
            if not isinstance(kind, int):
                continue
            packed, scale, n, k = val
            if np.ndim(packed) == 3:
                raise ValueError("tensor parallelism takes one basis per projection")
            packed = np.ascontiguousarray(packed).reshape(n, k // 4)
            if kind in (W_Q, W_K, W_V, W_GATE, W_UP):      # split output rows
                rows = n // size
                new[kind] = (np.ascontiguousarray(packed[rank * rows:(rank + 1) * rows]), scale, rows, k)
            elif kind in (W_O, W_DOWN):                     # split input columns (4 per byte)
                cols = k // size
                assert cols % 4 == 0
                new[kind] = (np.ascontiguousarray(packed[:, rank * cols // 4:(rank + 1) * cols // 4]), scale, n, cols)
            else:
                raise ValueError("tensor parallelism covers arch llama only")
        cache[id(layer)] = new
        out.layers.append(new)
    del hd
    return out


def build_model(w: SyntheticWeights, max_batch: int = 1, device: int = 0, tp_rank: int = 0,
                tp_size: int = 1) -> BitLlama:
    w = shard_weights(w, tp_rank, tp_size)
    m = BitLlama(w.cfg, max_batch=max_batch, device=device, tp_rank=tp_rank, tp_size=tp_size)
    m.set_tensor(T_EMBED, w.embed, f16=w.dense_f16)
    m.set_tensor(T_LM_HEAD, w.lm_head, f16=w.dense_f16)
    m.set_tensor(T_NORM_F, w.norm_f)
    for li, layer in enumerate(w.layers):
        m.set_tensor(T_NORM1, layer["norm1"], li)
        m.set_tensor(T_NORM2, layer["norm2"], li)
        for kind, val in layer.items():
            if isinstance(kind, int):
                packed, scale, n, k = val
                m.set_linear(li, kind, packed, scale, n, k)
    m.finalize()
    return m
