"""Generates tests/golden/converter_l2.npz and tests/golden/converted_tiny/ from the reference's own
Python converter.

Run once in a container that has the reference checked out (path given by
--reference); the GPU host has no copy of the reference, which is why the outputs are
committed.  What is pinned:

* quantize_adaptive_basis + pack_2bit of tools/conversion/convert_llama_v2.py:28-72,
  111-151 on seeded weights (NumBases 1 and 3): ternary bases, scales and the packed
  [Out, In/4, NumBases] bytes;
* pack_interleaved (the one-byte-per-weight legacy layout, :74-109).

* a whole converted checkpoint: the converter's own main() (tools/conversion/convert_llama_v2.py:163-283,
  default NumBases = 3) run on a seeded tiny Llama-shaped model directory (hidden 128, 2 layers,
  4 query / 2 KV heads of 32, MLP 256, vocabulary 96), so that tests/golden/converted_tiny/ holds a config.json and a
  model.safetensors written by the reference's code, byte for byte.

The four packing known-answer vectors of crates/rust_engine/src/kernels/packing.rs:
156-261 are short enough to be written out in tests/test_oracle_golden.py itself.
"""
import argparse
import importlib.util
import os
import sys
import types

import numpy as np
import torch


def load_converter(ref_root):
    path = os.path.join(ref_root, "tools", "conversion", "convert_llama_v2.py")
    # The converter imports huggingface_hub only for its download helper.
    if "huggingface_hub" not in sys.modules:
        try:
            import huggingface_hub  # noqa: F401
        except Exception:
            stub = types.ModuleType("huggingface_hub")
            stub.snapshot_download = lambda *a, **k: None
            sys.modules["huggingface_hub"] = stub
    spec = importlib.util.spec_from_file_location("ref_convert_llama_v2", path)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", required=True, help="checkout of the reference project")
    ap.add_argument("--out", default=os.path.join(os.path.dirname(os.path.abspath(__file__)),
                                                  "converter_l2.npz"))
    args = ap.parse_args()
    conv = load_converter(args.reference)
    out = {}
    for tag, (n_out, k_in, n_bases, seed) in {
        "a": (16, 32, 1, 101),
        "b": (24, 64, 3, 102),
        "c": (8, 16, 2, 103),
    }.items():
        g = torch.Generator().manual_seed(seed)
        w = torch.randn(n_out, k_in, generator=g) * 0.02
        bases, scales = conv.quantize_adaptive_basis(w, n_bases)
        packed = conv.pack_2bit(bases)
        out[f"{tag}_w"] = w.numpy().astype(np.float32)
        out[f"{tag}_bases"] = bases.numpy().astype(np.int8)
        out[f"{tag}_scales"] = scales.numpy().astype(np.float32)
        out[f"{tag}_packed"] = packed.numpy().astype(np.uint8)
        out[f"{tag}_legacy"] = conv.pack_interleaved(bases).numpy().astype(np.uint8)
    np.savez_compressed(args.out, **out)
    print("wrote", args.out, {k: v.shape for k, v in out.items()})
    convert_tiny_model(conv, os.path.join(os.path.dirname(os.path.abspath(args.out)), "converted_tiny"))


def convert_tiny_model(conv, out_dir):
    """A seeded HF-style Llama checkpoint in a temporary directory, converted by the reference's main()."""
    import json
    import tempfile
    from safetensors.torch import save_file
    H, L, NH, NKV, I, V = 128, 2, 4, 2, 256, 96
    hd = H // NH
    g = torch.Generator().manual_seed(2024)
    t = {"model.embed_tokens.weight": torch.randn(V, H, generator=g) * 0.02,
         "lm_head.weight": torch.randn(V, H, generator=g) * 0.02,
         "model.norm.weight": 1.0 + 0.1 * torch.randn(H, generator=g)}
    for li in range(L):
        p = f"model.layers.{li}"
        for name, shape in (("self_attn.q_proj", (NH * hd, H)), ("self_attn.k_proj", (NKV * hd, H)),
                            ("self_attn.v_proj", (NKV * hd, H)), ("self_attn.o_proj", (H, NH * hd)),
                            ("mlp.gate_proj", (I, H)), ("mlp.up_proj", (I, H)), ("mlp.down_proj", (H, I))):
            t[f"{p}.{name}.weight"] = torch.randn(*shape, generator=g) * 0.02
        t[f"{p}.input_layernorm.weight"] = 1.0 + 0.1 * torch.randn(H, generator=g)
        t[f"{p}.post_attention_layernorm.weight"] = 1.0 + 0.1 * torch.randn(H, generator=g)
    with tempfile.TemporaryDirectory() as src:
        save_file({k: v.contiguous() for k, v in t.items()}, os.path.join(src, "model.safetensors"))
        with open(os.path.join(src, "config.json"), "w") as f:
            json.dump({"hidden_size": H, "num_hidden_layers": L, "num_attention_heads": NH, "num_key_value_heads": NKV,
                       "intermediate_size": I, "vocab_size": V, "rope_theta": 10000.0, "max_position_embeddings": 64}, f)
        argv = sys.argv
        sys.argv = ["convert_llama_v2.py", "--model-id", src, "--output-dir", out_dir]
        try:
            conv.main()
        finally:
            sys.argv = argv
    print("wrote", out_dir, os.listdir(out_dir))


if __name__ == "__main__":
    main()
