"""Generates tests/golden/converter_l2.npz from the reference's own Python converter.

Run once in a container that has the reference checked out (path given by
--reference); the GPU host has no copy of the reference, which is why the outputs are
committed.  What is pinned:

* quantize_adaptive_basis + pack_2bit of tools/conversion/convert_llama_v2.py:28-72,
  111-151 on seeded weights (NumBases 1 and 3): ternary bases, scales and the packed
  [Out, In/4, NumBases] bytes;
* pack_interleaved (the one-byte-per-weight legacy layout, :74-109).

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


if __name__ == "__main__":
    main()
