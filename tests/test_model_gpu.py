"""GPU parity of the whole decode step (BitLlama::forward_one) against the oracle:
teacher-forced logits and final TTT states / KV caches within 1e-3."""
import importlib

import numpy as np
import pytest

from gpu_util import load_bt, staged_decode_step

torch = pytest.importorskip("torch")
pytestmark = pytest.mark.gpu

REL_TOL = 1e-3


@pytest.fixture(scope="module")
def bt():
    if not torch.cuda.is_available():
        pytest.fail("GPU tests need a CUDA device")
    return load_bt()


def rel_err(a, b):
    return float(np.abs(a - b).max() / max(np.abs(b).max(), 1e-30))


def run_staged(bt, oracle, cfg, n_tokens, seed, batch):
    """Teacher-forced decode from an empty cache / zero TTT states, every step checked stage by stage
    against the oracle (see oracle/staged.py for why logits of free-running pipelines are not compared)."""
    syn = importlib.import_module("bit-ttt-engine_b200.synthetic")
    w = syn.make_weights(cfg, seed=seed)
    gpu = syn.build_model(w, max_batch=batch)
    ref = oracle.model_from_weights(w)
    states = [ref.new_state() for _ in range(batch)]
    tokens = np.random.default_rng(7).integers(0, cfg.vocab_size, size=(n_tokens, batch))
    for t in range(n_tokens):
        staged_decode_step(oracle, ref, gpu, cfg, tokens[t], states)
    assert gpu.current_pos == n_tokens
    return gpu, ref, states


def test_tiny_ttt_model_teacher_forced(bt, oracle):
    syn = importlib.import_module("bit-ttt-engine_b200.synthetic")
    cfg = syn.TINY_TTT  # 4 layers, hidden 256, MLP 688, vocab 32000, TTT layers
    gpu, ref, states = run_staged(bt, oracle, cfg, 12, 2000, batch=1)
    for li in range(cfg.num_layers):
        w_gpu = gpu.ttt_state(li)[0].cpu().numpy()
        assert rel_err(w_gpu, states[0].w[li]) <= REL_TOL
    # reset gives the same logits again
    l0, _ = gpu.forward_one([5])
    gpu.reset_kv_cache()
    assert gpu.current_pos == 0
    l1, _ = gpu.forward_one([5])
    assert not np.array_equal(l0, l1)
    gpu.reset_kv_cache()
    staged_decode_step(oracle, ref, gpu, cfg, [5], [ref.new_state()])  # from the fresh state: matches the oracle again


def test_tiny_llama_model_teacher_forced_batch2(bt, oracle):
    syn = importlib.import_module("bit-ttt-engine_b200.synthetic")
    cfg = syn.TINY_LLAMA_TEST  # 2 layers, hidden 256, 8 q heads / 2 kv heads, head_dim 32
    gpu, ref, states = run_staged(bt, oracle, cfg, 10, 3000, batch=2)
    # free-running comparison, for the record: the two pipelines may part by quantisation noise
    free = [ref.new_state() for _ in range(2)]
    gpu.reset_kv_cache()
    tokens = np.random.default_rng(8).integers(0, cfg.vocab_size, size=(6, 2))
    worst = 0.0
    for t in range(6):
        logits, _ = gpu.forward_one(tokens[t])
        for b in range(2):
            worst = max(worst, rel_err(logits[b], ref.forward_one(int(tokens[t, b]), free[b])))
    assert worst <= 5e-2, worst
    assert bt.lib().bt_device_check(0) == 0


@pytest.mark.parametrize("batch", [3, 5, 8])
def test_tiny_llama_model_teacher_forced_batch_3_to_8(bt, oracle, batch):
    # three to eight sequences: a quantiser kernel in front of every product instead of the fused prologue
    syn = importlib.import_module("bit-ttt-engine_b200.synthetic")
    run_staged(bt, oracle, syn.TINY_LLAMA_TEST, 6, 3300 + batch, batch=batch)
    assert bt.lib().bt_device_check(0) == 0


def test_position_limit(bt):
    syn = importlib.import_module("bit-ttt-engine_b200.synthetic")
    cfg = syn.BitLlamaConfig("llama", 64, 64, 1, 2, 1, 64, max_position_embeddings=3)
    gpu = syn.build_model(syn.make_weights(cfg, seed=1))
    for _ in range(3):
        gpu.forward_one([1])
    with pytest.raises(bt.BitTTTError) as ei:
        gpu.forward_one([1])
    assert ei.value.status == bt.BT_ERR_SHAPE


def test_models_batch_12_use_tensor_core_product(bt, oracle):
    # more than 8 sequences: projections run on the tcgen05 kernel, row transforms separately
    syn = importlib.import_module("bit-ttt-engine_b200.synthetic")
    run_staged(bt, oracle, syn.TINY_LLAMA_TEST, 4, 3100, batch=12)
    run_staged(bt, oracle, syn.BitLlamaConfig("ttt", 500, 256, 2, 4, 4, 688, inner_lr=0.01), 4, 3200, batch=12)
    assert bt.lib().bt_device_check(0) == 0


@pytest.mark.parametrize("arch,batch", [("llama", 1), ("llama", 6), ("llama", 12), ("ttt", 2), ("ttt", 10)])
def test_models_with_several_bases_per_projection(bt, oracle, arch, batch):
    # the converter's default is three bases per projection: q|k|v and gate|up are fused per basis, every
    # projection adds its per-basis products in basis order before the residual
    syn = importlib.import_module("bit-ttt-engine_b200.synthetic")
    cfg = syn.TINY_LLAMA_TEST if arch == "llama" else syn.BitLlamaConfig("ttt", 500, 256, 2, 4, 4, 688, inner_lr=0.01)
    w = syn.make_weights(cfg, seed=3400 + batch, n_bases=3)
    gpu = syn.build_model(w, max_batch=batch)
    ref = oracle.model_from_weights(w)
    states = [ref.new_state() for _ in range(batch)]
    tokens = np.random.default_rng(batch).integers(0, cfg.vocab_size, size=(4, batch))
    for t in range(4):
        staged_decode_step(oracle, ref, gpu, cfg, tokens[t], states)
    assert bt.lib().bt_device_check(0) == 0
