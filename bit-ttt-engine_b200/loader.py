"""Converted checkpoints on disk: safetensors reader / writer, config aliases, tensor names.

Mirrors what `BitLlama::load` and `Llama::load_auto` accept (model/llama.rs:37-158,
model/block.rs:27-64, layers/adaptive_linear.rs:40-84, model/config.rs:20-59):

* a directory with `config.json` and `model.safetensors` (or any `*.safetensors` files),
* HF tensor names (`model.embed_tokens`, `model.layers.N.self_attn.q_proj`, `model.norm`, ...)
  or the legacy ones (`embed`, `layers.N`, `norm_f`, `norm1` / `norm2`),
* every projection either as the converter writes it (`X.weight_packed` u8
  `[out, in/4, bases]` + `X.scales` `[bases]`, tools/conversion/convert_llama_v2.py:258-283) or as a
  dense `X.weight` `[out, in]`, which is packed on load like `BitLinear::precompute_packed`
  (layers/bit_linear.rs:44-50),
* norms, embedding and head in f32, f16 or bf16 (the engine loads everything as f32).

The safetensors container is read and written here directly (8-byte little-endian header
length, JSON header, raw little-endian tensor data); no third-party package is needed.
"""
from __future__ import annotations

import glob
import json
import os
import struct

import numpy as np

from .layers import pack_ternary
from .model import (BitLlamaConfig, W_DOWN, W_GATE, W_K, W_O, W_Q, W_TTT_DOWN, W_TTT_UP, W_UP, W_V)
from .synthetic import SyntheticWeights, linear_shapes

_DTYPES = {
    "F64": np.float64, "F32": np.float32, "F16": np.float16, "I64": np.int64, "I32": np.int32,
    "I16": np.int16, "I8": np.int8, "U8": np.uint8, "BOOL": np.bool_, "U16": np.uint16, "U32": np.uint32,
    "U64": np.uint64,
}
_NAMES = {np.dtype(v): k for k, v in _DTYPES.items()}


class CheckpointError(ValueError):
    pass


def _bf16_to_f32(raw: np.ndarray) -> np.ndarray:
    return (raw.astype(np.uint32) << 16).view(np.float32)


def read_safetensors(path: str) -> dict:
    """name -> numpy array (bf16 tensors come back as f32).  The file is memory-mapped; arrays
    of the other dtypes are views into the mapping."""
    size = os.path.getsize(path)
    if size < 8:
        raise CheckpointError(f"{path}: too short for a safetensors file")
    with open(path, "rb") as f:
        (hlen,) = struct.unpack("<Q", f.read(8))
        if hlen > size - 8 or hlen > 100 * 1024 * 1024:
            raise CheckpointError(f"{path}: header length {hlen} does not fit the file")
        try:
            header = json.loads(f.read(hlen).decode("utf-8"))
        except (UnicodeDecodeError, json.JSONDecodeError) as e:
            raise CheckpointError(f"{path}: header is not JSON ({e})") from None
    data = np.memmap(path, dtype=np.uint8, mode="r", offset=8 + hlen) if size > 8 + hlen else np.zeros(0, np.uint8)
    out = {}
    for name, info in header.items():
        if name == "__metadata__":
            continue
        dt, shape, (b0, b1) = info["dtype"], tuple(info["shape"]), info["data_offsets"]
        if not (0 <= b0 <= b1 <= data.size):
            raise CheckpointError(f"{path}: tensor {name} lies outside the file")
        raw = data[b0:b1]
        count = int(np.prod(shape, dtype=np.int64))
        if dt == "BF16":
            if raw.size != 2 * count:
                raise CheckpointError(f"{path}: tensor {name} has {raw.size} bytes, shape {shape} needs {2 * count}")
            out[name] = _bf16_to_f32(raw.view(np.uint16)).reshape(shape)
            continue
        if dt not in _DTYPES:
            raise CheckpointError(f"{path}: tensor {name} has unsupported dtype {dt}")
        npdt = np.dtype(_DTYPES[dt])
        if raw.size != npdt.itemsize * count:
            raise CheckpointError(f"{path}: tensor {name} has {raw.size} bytes, shape {shape} needs {npdt.itemsize * count}")
        out[name] = raw.view(npdt).reshape(shape)
    return out


def write_safetensors(path: str, tensors: dict, metadata: dict | None = None) -> None:
    """Writes name -> array in the order given (dtypes of `read_safetensors`, no bf16)."""
    header, offset, blobs = {}, 0, []
    if metadata:
        header["__metadata__"] = {str(k): str(v) for k, v in metadata.items()}
    for name, arr in tensors.items():
        arr = np.ascontiguousarray(arr)
        if arr.dtype not in _NAMES:
            raise CheckpointError(f"tensor {name}: dtype {arr.dtype} cannot be stored")
        blob = arr.tobytes()
        header[name] = {"dtype": _NAMES[arr.dtype], "shape": list(arr.shape), "data_offsets": [offset, offset + len(blob)]}
        offset += len(blob)
        blobs.append(blob)
    text = json.dumps(header, separators=(",", ":")).encode("utf-8")
    text += b" " * (-len(text) % 8)  # keeps the data 8-byte aligned, as the reference writers do
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(text)))
        f.write(text)
        for blob in blobs:
            f.write(blob)


def config_from_dict(d: dict) -> BitLlamaConfig:
    """config.json with either name set (model/config.rs:29-43: hidden_size, num_hidden_layers /
    n_layers, num_attention_heads, num_key_value_heads, intermediate_size) and the engine's
    defaults: arch ttt, rope_theta 10000, max_position_embeddings 2048, MLP width 4 * hidden."""
    def pick(*names, default=None):
        for n in names:
            if n in d and d[n] is not None:
                return d[n]
        if default is None:
            raise CheckpointError(f"config: none of {names} is present")
        return default

    hidden = int(pick("hidden_dim", "hidden_size"))
    return BitLlamaConfig(
        arch=str(d.get("arch", "ttt")),
        vocab_size=int(pick("vocab_size")),
        hidden_dim=hidden,
        num_layers=int(pick("num_layers", "num_hidden_layers", "n_layers")),
        n_heads=int(pick("n_heads", "num_attention_heads")),
        n_kv_heads=int(pick("n_kv_heads", "num_key_value_heads")),
        intermediate_dim=int(pick("intermediate_dim", "intermediate_size", default=4 * hidden)),
        inner_lr=float(d.get("inner_lr", 0.0)),
        rope_theta=float(d.get("rope_theta", 10000.0)),
        max_position_embeddings=int(d.get("max_position_embeddings", 2048)),
    )


def _f32(a) -> np.ndarray:
    return np.ascontiguousarray(a, dtype=np.float32)


def _first(tensors: dict, names, what: str):
    for n in names:
        if n in tensors:
            return tensors[n]
    raise CheckpointError(f"checkpoint: {what} not found (tried {', '.join(names)})")


def _linear(tensors: dict, prefix: str, n_out: int, k_in: int):
    """(packed, scale(s)) for one projection: BitLinear::load first (dense weight, packed here), then
    the converted format (layers/adaptive_linear.rs:42-84): `weight_packed` [n_out, k_in/4, n_bases] with
    `scales` [n_bases] - one basis comes back as [n_out, k_in/4] with a float scale, several as the 3-d
    array with an array of scales - or the legacy one-byte-per-weight layout [n_out, k_in/4, n_bases, 4]
    (tools/conversion/convert_adaptive.py:43-83), rewritten to 2 bits per weight."""
    if prefix + ".weight" in tensors:
        dense = _f32(tensors[prefix + ".weight"])
        if dense.shape != (n_out, k_in):
            raise CheckpointError(f"{prefix}.weight has shape {dense.shape}, expected {(n_out, k_in)}")
        packed, scale = pack_ternary(dense)
        return packed.reshape(n_out, k_in // 4), float(scale)
    if prefix + ".scales" not in tensors or prefix + ".weight_packed" not in tensors:
        raise CheckpointError(f"checkpoint: neither {prefix}.weight nor {prefix}.weight_packed / .scales is present")
    scales = _f32(tensors[prefix + ".scales"]).reshape(-1)
    packed = tensors[prefix + ".weight_packed"]
    if packed.dtype != np.uint8:  # older converters stored the byte values as f32 (adaptive_linear.rs:66-75)
        packed = np.asarray(packed).astype(np.uint8)
    if not 1 <= scales.size <= 8:
        raise CheckpointError(f"{prefix}.scales has {scales.size} entries, the format allows 1..8")
    if packed.ndim == 4:  # legacy layout: one signed byte per weight, 4 weights per block
        if packed.shape != (n_out, k_in // 4, scales.size, 4):
            raise CheckpointError(f"{prefix}.weight_packed has shape {packed.shape}, expected {(n_out, k_in // 4, scales.size, 4)}")
        from . import check, lib
        l3 = np.ascontiguousarray(packed).view(np.int8)
        packed = np.zeros((n_out, k_in // 4, scales.size), np.uint8)
        check(lib().bt_convert_l3_to_l2(l3.ctypes.data, n_out, k_in, scales.size, packed.ctypes.data))
    if packed.shape != (n_out, k_in // 4, scales.size):
        raise CheckpointError(f"{prefix}.weight_packed has shape {packed.shape}, expected {(n_out, k_in // 4, scales.size)}")
    if scales.size == 1:
        return np.ascontiguousarray(packed[:, :, 0]), float(scales[0])
    return np.ascontiguousarray(packed), scales


def weights_from_tensors(tensors: dict, cfg: BitLlamaConfig) -> SyntheticWeights:
    """Name resolution of BitLlama::load (model/llama.rs:84-141) and BitLlamaBlock::load
    (model/block.rs:33-64) over a name -> array mapping."""
    V, H = cfg.vocab_size, cfg.hidden_dim
    embed_raw = _first(tensors, ["model.embed_tokens.weight", "embed.weight"], "embedding")
    head_raw = _first(tensors, ["lm_head.weight"], "lm_head")
    embed, head = _f32(embed_raw), _f32(head_raw)
    norm_f = _f32(_first(tensors, ["model.norm.weight", "norm_f.weight"], "final norm"))
    for name, arr, shape in (("embedding", embed, (V, H)), ("lm_head", head, (V, H)), ("final norm", norm_f, (H,))):
        if arr.shape != shape:
            raise CheckpointError(f"checkpoint: {name} has shape {arr.shape}, expected {shape}")
    w = SyntheticWeights(cfg, embed, head, norm_f)
    # the converter stores embedding and head as IEEE halves; the device tables then keep exactly those values
    w.dense_f16 = np.asarray(embed_raw).dtype == np.float16 and np.asarray(head_raw).dtype == np.float16
    names = {W_Q: "self_attn.q_proj", W_K: "self_attn.k_proj", W_V: "self_attn.v_proj", W_O: "self_attn.o_proj",
             W_GATE: "mlp.gate_proj", W_UP: "mlp.up_proj", W_DOWN: "mlp.down_proj",
             W_TTT_DOWN: "ttt.down", W_TTT_UP: "ttt.up"}
    for li in range(cfg.num_layers):
        hf = (f"model.layers.{li}.self_attn.q_proj.weight" in tensors or
              f"model.layers.{li}.post_attention_layernorm.weight" in tensors)
        p = f"model.layers.{li}" if hf else f"layers.{li}"
        layer = {
            "norm1": _f32(_first(tensors, [f"{p}.norm1.model.norm.weight", f"{p}.norm1.weight",
                                           f"{p}.input_layernorm.weight"], f"layer {li} norm1")),
            "norm2": _f32(_first(tensors, [f"{p}.norm2.model.norm.weight", f"{p}.norm2.weight",
                                           f"{p}.post_attention_layernorm.weight"], f"layer {li} norm2")),
        }
        for key in ("norm1", "norm2"):
            if layer[key].shape != (H,):
                raise CheckpointError(f"checkpoint: layer {li} {key} has shape {layer[key].shape}, expected {(H,)}")
        for kind, (n, k) in linear_shapes(cfg).items():
            packed, scale = _linear(tensors, f"{p}.{names[kind]}", n, k)
            layer[kind] = (packed, scale, n, k)
        w.layers.append(layer)
    return w


def load_checkpoint(path: str):
    """(config, weights) from a model directory (config.json + *.safetensors) or from a single
    .safetensors file with config.json beside it."""
    directory = path if os.path.isdir(path) else os.path.dirname(os.path.abspath(path))
    cfg_path = os.path.join(directory, "config.json")
    if not os.path.exists(cfg_path):
        raise CheckpointError(f"{cfg_path} is missing")
    with open(cfg_path, "r", encoding="utf-8") as f:
        cfg = config_from_dict(json.load(f))
    files = [path] if os.path.isfile(path) else sorted(glob.glob(os.path.join(directory, "*.safetensors")))
    if not files:
        raise CheckpointError(f"no .safetensors file in {directory}")
    tensors = {}
    for fp in files:
        tensors.update(read_safetensors(fp))
    return cfg, weights_from_tensors(tensors, cfg)


def save_checkpoint(directory: str, w: SyntheticWeights, hf_names: bool = True, dense_dtype=np.float16) -> None:
    """Writes weights in the converter's layout (one basis): config.json + model.safetensors.
    Embedding, head and norms are stored as `dense_dtype` like the converter's `.half()`."""
    cfg = w.cfg
    os.makedirs(directory, exist_ok=True)
    names = {W_Q: "self_attn.q_proj", W_K: "self_attn.k_proj", W_V: "self_attn.v_proj", W_O: "self_attn.o_proj",
             W_GATE: "mlp.gate_proj", W_UP: "mlp.up_proj", W_DOWN: "mlp.down_proj",
             W_TTT_DOWN: "ttt.down", W_TTT_UP: "ttt.up"}
    t = {}
    t["model.embed_tokens.weight" if hf_names else "embed.weight"] = w.embed.astype(dense_dtype)
    for li, layer in enumerate(w.layers):
        p = f"model.layers.{li}" if hf_names else f"layers.{li}"
        t[f"{p}.input_layernorm.weight" if hf_names else f"{p}.norm1.weight"] = layer["norm1"].astype(dense_dtype)
        t[f"{p}.post_attention_layernorm.weight" if hf_names else f"{p}.norm2.weight"] = layer["norm2"].astype(dense_dtype)
        for kind, val in layer.items():
            if isinstance(kind, int):
                packed, scale, n, k = val
                scales = np.atleast_1d(np.asarray(scale, np.float32))
                t[f"{p}.{names[kind]}.weight_packed"] = np.ascontiguousarray(packed, np.uint8).reshape(n, k // 4, scales.size)
                t[f"{p}.{names[kind]}.scales"] = scales
    t["model.norm.weight" if hf_names else "norm_f.weight"] = w.norm_f.astype(dense_dtype)
    t["lm_head.weight"] = w.lm_head.astype(dense_dtype)
    write_safetensors(os.path.join(directory, "model.safetensors"), t)
    d = {"arch": cfg.arch, "vocab_size": cfg.vocab_size, "inner_lr": cfg.inner_lr, "rope_theta": cfg.rope_theta,
         "max_position_embeddings": cfg.max_position_embeddings}
    if hf_names:
        d.update(hidden_size=cfg.hidden_dim, num_hidden_layers=cfg.num_layers, num_attention_heads=cfg.n_heads,
                 num_key_value_heads=cfg.n_kv_heads, intermediate_size=cfg.intermediate_dim)
    else:
        d.update(hidden_dim=cfg.hidden_dim, num_layers=cfg.num_layers, n_heads=cfg.n_heads,
                 n_kv_heads=cfg.n_kv_heads, intermediate_dim=cfg.intermediate_dim)
    with open(os.path.join(directory, "config.json"), "w", encoding="utf-8") as f:
        json.dump(d, f, indent=1)


def load_model(path: str, max_batch: int = 1, device: int = 0):
    """`Llama::load_auto` for the decode path: read the checkpoint and build the device model."""
    from .synthetic import build_model
    cfg, w = load_checkpoint(path)
    return build_model(w, max_batch=max_batch, device=device)
