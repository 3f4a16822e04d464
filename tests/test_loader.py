"""Checkpoint loader: safetensors container, config aliases and tensor-name resolution
(model/llama.rs:84-141, model/block.rs:33-64, layers/adaptive_linear.rs:40-84,
model/config.rs:29-43), then a loaded model against the same weights set directly."""
import importlib
import json
import os
import struct

import numpy as np
import pytest


@pytest.fixture(scope="module")
def mods():
    bt = importlib.import_module("bit-ttt-engine_b200")
    bt.lib()
    return (importlib.import_module("bit-ttt-engine_b200.loader"),
            importlib.import_module("bit-ttt-engine_b200.synthetic"),
            importlib.import_module("bit-ttt-engine_b200.model"))


def test_safetensors_round_trip_and_bf16(mods, tmp_path):
    loader, _, _ = mods
    rng = np.random.default_rng(0)
    t = {"a": rng.normal(size=(3, 5)).astype(np.float32), "b": rng.integers(0, 255, size=(4, 2, 1), dtype=np.uint8),
         "c": rng.normal(size=(7,)).astype(np.float16), "empty": np.zeros((0, 4), np.float32)}
    path = str(tmp_path / "x.safetensors")
    loader.write_safetensors(path, t, metadata={"format": "pt"})
    back = loader.read_safetensors(path)
    assert set(back) == set(t)
    for k in t:
        assert back[k].dtype == t[k].dtype and back[k].shape == t[k].shape and np.array_equal(back[k], t[k])
    # a bf16 tensor written by hand: 1.0 = 0x3F80, -2.5 = 0xC020
    header = json.dumps({"w": {"dtype": "BF16", "shape": [2], "data_offsets": [0, 4]}}).encode()
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(header)) + header + struct.pack("<HH", 0x3F80, 0xC020))
    w = loader.read_safetensors(path)["w"]
    assert w.dtype == np.float32 and w.tolist() == [1.0, -2.5]


def test_safetensors_rejects_broken_files(mods, tmp_path):
    loader, _, _ = mods
    path = str(tmp_path / "bad.safetensors")
    with open(path, "wb") as f:
        f.write(b"\x01\x02")
    with pytest.raises(loader.CheckpointError):
        loader.read_safetensors(path)
    header = json.dumps({"w": {"dtype": "F32", "shape": [4], "data_offsets": [0, 16]}}).encode()
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(header)) + header + b"\0" * 8)  # data shorter than the header says
    with pytest.raises(loader.CheckpointError):
        loader.read_safetensors(path)
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", 1 << 40) + b"{}")
    with pytest.raises(loader.CheckpointError):
        loader.read_safetensors(path)


def test_config_aliases_and_defaults(mods):
    loader, _, _ = mods
    hf = loader.config_from_dict({"arch": "llama", "vocab_size": 100, "hidden_size": 64, "num_hidden_layers": 2,
                                  "num_attention_heads": 4, "num_key_value_heads": 2, "intermediate_size": 128,
                                  "rope_theta": 500000.0})
    own = loader.config_from_dict({"arch": "llama", "vocab_size": 100, "hidden_dim": 64, "n_layers": 2, "n_heads": 4,
                                   "n_kv_heads": 2, "intermediate_dim": 128, "rope_theta": 500000.0})
    assert hf == own and hf.max_position_embeddings == 2048
    d = loader.config_from_dict({"vocab_size": 10, "hidden_dim": 32, "num_layers": 1, "n_heads": 1, "n_kv_heads": 1})
    assert d.arch == "ttt" and d.intermediate_dim == 128 and d.rope_theta == 10000.0  # model/config.rs defaults
    with pytest.raises(loader.CheckpointError):
        loader.config_from_dict({"vocab_size": 10})


@pytest.mark.parametrize("arch,hf_names", [("llama", True), ("llama", False), ("ttt", True)])
def test_name_resolution_matches_direct_weights(mods, tmp_path, arch, hf_names):
    loader, syn, _ = mods
    cfg = syn.TINY_LLAMA_TEST if arch == "llama" else syn.BitLlamaConfig("ttt", 500, 64, 2, 4, 4, 176, inner_lr=0.01)
    w = syn.make_weights(cfg, seed=11)
    d = str(tmp_path / "ckpt")
    loader.save_checkpoint(d, w, hf_names=hf_names, dense_dtype=np.float32)
    cfg2, w2 = loader.load_checkpoint(d)
    assert cfg2 == cfg
    assert np.array_equal(w2.embed, w.embed) and np.array_equal(w2.lm_head, w.lm_head)
    for a, b in zip(w.layers, w2.layers):
        assert set(a) == set(b)
        for k in a:
            if isinstance(k, int):
                assert np.array_equal(np.asarray(a[k][0]).reshape(a[k][2], -1), b[k][0]) and a[k][1] == pytest.approx(b[k][1])
                assert a[k][2:] == b[k][2:]
            else:
                assert np.array_equal(a[k], b[k])


def test_dense_weights_are_packed_on_load_and_errors(mods, tmp_path):
    loader, syn, _ = mods
    cfg = syn.BitLlamaConfig("ttt", 50, 32, 1, 1, 1, 64, inner_lr=0.01)
    rng = np.random.default_rng(3)
    H, I, d = 32, 64, 8
    dense = {"ttt.down": (d, H), "ttt.up": (H, d), "mlp.gate_proj": (I, H), "mlp.up_proj": (I, H), "mlp.down_proj": (H, I)}
    t = {"embed.weight": rng.normal(size=(50, H)).astype(np.float32), "lm_head.weight": rng.normal(size=(50, H)).astype(np.float32),
         "norm_f.weight": np.ones(H, np.float32), "layers.0.norm1.weight": np.ones(H, np.float32),
         "layers.0.norm2.weight": np.ones(H, np.float32)}
    for name, shape in dense.items():
        t[f"layers.0.{name}.weight"] = rng.normal(0, 0.02, size=shape).astype(np.float32)
    w = loader.weights_from_tensors(t, cfg)
    bt = importlib.import_module("bit-ttt-engine_b200")
    packed, scale = bt.pack_ternary(t["layers.0.mlp.gate_proj.weight"])
    model = importlib.import_module("bit-ttt-engine_b200.model")
    got = w.layers[0][model.W_GATE]
    assert np.array_equal(got[0].reshape(-1), packed.reshape(-1)) and got[1] == pytest.approx(float(scale))
    # a missing projection is reported by name; several bases come back in the converted layout
    t2 = dict(t)
    del t2["layers.0.mlp.up_proj.weight"]
    with pytest.raises(loader.CheckpointError, match="up_proj"):
        loader.weights_from_tensors(t2, cfg)
    t3 = dict(t)
    del t3["layers.0.mlp.up_proj.weight"]
    t3["layers.0.mlp.up_proj.weight_packed"] = np.zeros((I, H // 4, 3), np.uint8)
    t3["layers.0.mlp.up_proj.scales"] = np.ones(3, np.float32)
    w3 = loader.weights_from_tensors(t3, cfg).layers[0][model.W_UP]
    assert w3[0].shape == (I, H // 4, 3) and np.array_equal(w3[1], np.ones(3, np.float32))
    # the legacy one-byte-per-weight layout [out, in/4, bases, 4] is rewritten to 2 bits per weight
    bases = rng.integers(-1, 2, size=(3, I, H)).astype(np.int8)
    t4 = dict(t3)
    t4["layers.0.mlp.up_proj.weight_packed"] = np.ascontiguousarray(bases.reshape(3, I, H // 4, 4).transpose(1, 2, 0, 3)).view(np.uint8)
    w4 = loader.weights_from_tensors(t4, cfg).layers[0][model.W_UP]
    codes = np.where(bases > 0, 1, np.where(bases < 0, 2, 0)).astype(np.uint8).reshape(3, I, H // 4, 4)
    expect = (codes[..., 0] | (codes[..., 1] << 2) | (codes[..., 2] << 4) | (codes[..., 3] << 6)).transpose(1, 2, 0)
    assert np.array_equal(w4[0], expect)
    t5 = dict(t4)
    t5["layers.0.mlp.up_proj.weight_packed"] = np.zeros((I, H // 4, 2), np.uint8)
    with pytest.raises(loader.CheckpointError, match="up_proj"):
        loader.weights_from_tensors(t5, cfg)


@pytest.mark.gpu
def test_loaded_checkpoint_runs_like_direct_weights(mods, tmp_path):
    torch = pytest.importorskip("torch")
    if not torch.cuda.is_available():
        pytest.fail("GPU tests need a CUDA device")
    loader, syn, _ = mods
    cfg = syn.TINY_LLAMA_TEST
    w = syn.make_weights(cfg, seed=5)
    d = str(tmp_path / "ckpt")
    loader.save_checkpoint(d, w, hf_names=True, dense_dtype=np.float32)
    cfg2, w2 = loader.load_checkpoint(os.path.join(d, "model.safetensors"))
    a, b = syn.build_model(w), syn.build_model(w2)
    for tok in (3, 17, 256, 999):
        la, na = a.forward_one(np.array([tok], np.int32))
        lb, nb = b.forward_one(np.array([tok], np.int32))
        assert np.array_equal(la, lb) and np.array_equal(na, nb)


@pytest.mark.gpu
def test_ttt_memory_file_round_trip(mods, tmp_path):
    """Llama::save_memory / load_memory (model/llama.rs:575-611): the TTT states survive a
    trip through the file, and a model that loads them continues exactly like the original."""
    torch = pytest.importorskip("torch")
    if not torch.cuda.is_available():
        pytest.fail("GPU tests need a CUDA device")
    loader, syn, _ = mods
    cfg = syn.BitLlamaConfig("ttt", 500, 64, 2, 4, 4, 176, inner_lr=0.05)
    w = syn.make_weights(cfg, seed=9)
    a, b = syn.build_model(w), syn.build_model(w)
    for tok in (1, 2, 3, 4, 5):
        a.forward_one(np.array([tok], np.int32))
    path = str(tmp_path / "memory.soul")
    a.save_memory(path)
    saved = loader.read_safetensors(path)
    assert set(saved) == {"layer_0", "layer_1"} and saved["layer_0"].shape == (16, 16)
    assert np.abs(saved["layer_0"]).max() > 0
    b.load_memory(path)
    for li in range(2):
        assert np.array_equal(a.ttt_state(li).cpu().numpy(), b.ttt_state(li).cpu().numpy())
    la, _ = a.forward_one(np.array([7], np.int32))
    lb, _ = b.forward_one(np.array([7], np.int32))
    assert np.array_equal(la, lb)


@pytest.mark.gpu
def test_kv_cache_in_the_memory_file(mods, tmp_path):
    """Attention blocks: the Q8 cache rows and the position travel in the same file (an addition to the
    reference's format, which holds TTT states only); a model that loads them continues bit for bit."""
    torch = pytest.importorskip("torch")
    if not torch.cuda.is_available():
        pytest.fail("GPU tests need a CUDA device")
    loader, syn, _ = mods
    w = syn.make_weights(syn.TINY_LLAMA_TEST, seed=21)
    a, b = syn.build_model(w, max_batch=2), syn.build_model(w, max_batch=2)
    rng = np.random.default_rng(5)
    for _ in range(9):
        a.forward_one(rng.integers(0, 1000, size=2).astype(np.int32))
    path = str(tmp_path / "memory.soul")
    a.save_memory(path)
    saved = loader.read_safetensors(path)
    assert int(saved["kv_position"][0]) == 9 and saved["kv_0.k_q"].shape == (2, 2, 9, 32) and saved["kv_1.v_s"].shape == (2, 2, 9)
    b.load_memory(path)
    assert b.current_pos == 9
    tok = np.array([11, 12], np.int32)
    la, na = a.forward_one(tok)
    lb, nb = b.forward_one(tok)
    assert np.array_equal(la, lb) and np.array_equal(na, nb)


def test_reference_converted_checkpoint_is_read(mods, oracle):
    """tests/golden/converted_tiny was written by the reference's own converter (its main(), default
    NumBases = 3; regenerate with tests/golden/make_golden.py): the container parser, the HF tensor names,
    the fp16 norms / embeddings and the three-basis projections are read as the converter wrote them."""
    loader, syn, _ = mods
    here = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "converted_tiny")
    cfg, w = loader.load_checkpoint(here)
    assert (cfg.arch, cfg.hidden_dim, cfg.num_layers, cfg.n_heads, cfg.n_kv_heads, cfg.intermediate_dim, cfg.vocab_size) == \
        ("llama", 128, 2, 4, 2, 256, 96)
    model = importlib.import_module("bit-ttt-engine_b200.model")
    packed, scales, n, k = w.layers[1][model.W_DOWN]
    assert packed.shape == (128, 64, 3) and packed.dtype == np.uint8 and scales.shape == (3,) and (n, k) == (128, 256)
    assert scales[0] > scales[1] > scales[2] > 0  # greedy residual decomposition: shrinking scales
    # the dense reconstruction of the three bases (AdaptiveBitLinear::load, layers/adaptive_linear.rs:86-109)
    # approximates a N(0, 0.02) matrix: residual well below the weights themselves
    dense = oracle.decode_l2(packed, scales)
    assert 0.015 < dense.std() < 0.025


@pytest.mark.gpu
def test_reference_converted_checkpoint_decodes_and_prefills_like_the_oracle(mods, oracle):
    """The converter's default output (three bases per projection) loaded as a model: decode steps and a
    batched prefill checked stage by stage against the oracle built from the same file."""
    torch = pytest.importorskip("torch")
    if not torch.cuda.is_available():
        pytest.fail("GPU tests need a CUDA device")
    from oracle.staged import staged_decode_step, staged_prefill
    loader, syn, _ = mods
    here = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "converted_tiny")
    cfg, w = loader.load_checkpoint(here)
    ref = oracle.model_from_weights(w)
    rng = np.random.default_rng(12)
    for batch in (2, 11):  # streaming kernel, tensor-core kernel
        gpu = loader.load_model(here, max_batch=batch)
        states = [ref.new_state() for _ in range(batch)]
        staged_prefill(oracle, ref, gpu, cfg, rng.integers(0, cfg.vocab_size, size=(batch, 9)), states)
        for _ in range(3):
            staged_decode_step(oracle, ref, gpu, cfg, rng.integers(0, cfg.vocab_size, size=batch), states)
        assert gpu.current_pos == 12
