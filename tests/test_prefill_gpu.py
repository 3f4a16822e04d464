"""Batched prefill (bt_model_prefill): tensor-core products over all rows, one-pass K/V append, causal
attention over blocks of query positions, chunked TTT update - checked stage by stage against the
oracle (oracle/staged.py) and, where the arithmetic is reproducible bit for bit, against token-by-token
decode, whose semantics it must have (the reference CLI's prefill loop, model/llama.rs:495-498)."""
import importlib

import numpy as np
import pytest

from gpu_util import load_bt, rel_err, seed_kv_caches, staged_decode_step
from oracle.staged import staged_prefill

torch = pytest.importorskip("torch")
pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def bt():
    if not torch.cuda.is_available():
        pytest.fail("GPU tests need a CUDA device")
    return load_bt()


@pytest.fixture(scope="module")
def syn():
    return importlib.import_module("bit-ttt-engine_b200.synthetic")


@pytest.mark.parametrize("batch,n_first,n_second", [(1, 13, 7), (2, 37, 5), (5, 16, 1)])
def test_prefill_tiny_llama_then_decode_then_prefill_again(bt, oracle, syn, batch, n_first, n_second):
    cfg = syn.TINY_LLAMA_TEST  # 2 layers, hidden 256, 8 q heads / 2 kv heads (4 per group), head_dim 32
    w = syn.make_weights(cfg, seed=6000 + batch)
    gpu = syn.build_model(w, max_batch=batch)
    ref = oracle.model_from_weights(w)
    states = [ref.new_state() for _ in range(batch)]
    rng = np.random.default_rng(batch)
    staged_prefill(oracle, ref, gpu, cfg, rng.integers(0, cfg.vocab_size, size=(batch, n_first)), states)
    for _ in range(2):  # decode continues on the cache the prefill filled
        staged_decode_step(oracle, ref, gpu, cfg, rng.integers(0, cfg.vocab_size, size=batch), states)
    staged_prefill(oracle, ref, gpu, cfg, rng.integers(0, cfg.vocab_size, size=(batch, n_second)), states)  # past > 0
    assert gpu.current_pos == n_first + 2 + n_second
    assert bt.lib().bt_device_check(0) == 0


def test_prefill_first_layer_cache_equals_token_by_token(bt, oracle, syn):
    # layer 0's keys and values depend on the embeddings only, so they must be the same bytes whichever
    # way the tokens went in; the logits of the two ways agree up to the quantisers' rounding noise
    cfg = syn.TINY_LLAMA_TEST
    w = syn.make_weights(cfg, seed=6100)
    a, b = syn.build_model(w, max_batch=2), syn.build_model(w, max_batch=2)
    tokens = np.random.default_rng(3).integers(0, cfg.vocab_size, size=(2, 21))
    la, _ = a.prefill(tokens)
    for t in range(tokens.shape[1]):
        lb, _ = b.forward_one(tokens[:, t])
    for s in range(2):
        ea, eb = a.kv_cache(0).export(s, 21), b.kv_cache(0).export(s, 21)
        for x, y in zip(ea, eb):
            assert np.array_equal(x, y)
    assert rel_err(la, lb) <= 5e-2


@pytest.mark.parametrize("ttt_chunk", [1, 16])
def test_prefill_tiny_ttt(bt, oracle, syn, ttt_chunk):
    cfg = syn.BitLlamaConfig("ttt", 500, 256, 2, 4, 4, 688, inner_lr=0.01)
    w = syn.make_weights(cfg, seed=6200)
    gpu = syn.build_model(w, max_batch=3)
    ref = oracle.model_from_weights(w)
    states = [ref.new_state() for _ in range(3)]
    rng = np.random.default_rng(5)
    tokens = rng.integers(0, cfg.vocab_size, size=(3, 37))
    logits, _ = staged_prefill(oracle, ref, gpu, cfg, tokens, states, ttt_chunk=ttt_chunk)
    for li in range(cfg.num_layers):
        for s in range(3):
            assert rel_err(gpu.ttt_state(li)[s].cpu().numpy(), states[s].w[li]) <= 1e-6
    staged_decode_step(oracle, ref, gpu, cfg, rng.integers(0, cfg.vocab_size, size=3), states)
    if ttt_chunk == 1:
        # without attention every stage is reproducible: the batched prefill IS the token-by-token loop, bit for bit
        other = syn.build_model(w, max_batch=3)
        for t in range(tokens.shape[1]):
            lo, _ = other.forward_one(tokens[:, t])
        assert np.array_equal(lo, logits)
    assert bt.lib().bt_device_check(0) == 0


def test_prefill_llama8b_block_shape_long_context(bt, oracle, syn):
    # the 8B block shape (4 query heads per KV head, head_dim 128) with 2000 positions already cached:
    # every query block walks 16 tiles of keys; 1 sequence x 48 tokens and 3 sequences x 40 tokens
    cfg = syn.BitLlamaConfig("llama", 2048, 4096, 1, 32, 8, 14336, rope_theta=500000.0, max_position_embeddings=2112)
    w = syn.make_weights(cfg, seed=6300, from_latent=False)
    gpu = syn.build_model(w, max_batch=3)
    ref = oracle.model_from_weights(w)
    for batch, n in ((1, 48), (3, 40)):
        gpu.reset_kv_cache()
        states = [ref.new_state() for _ in range(batch)]
        rng = np.random.default_rng(n)
        seed_kv_caches(gpu, states, cfg, 2000, rng)
        staged_prefill(oracle, ref, gpu, cfg, rng.integers(0, cfg.vocab_size, size=(batch, n)), states)
        staged_decode_step(oracle, ref, gpu, cfg, rng.integers(0, cfg.vocab_size, size=batch), states)
    assert bt.lib().bt_device_check(0) == 0


def test_prefill_tinyllama_shape_and_chunking(bt, oracle, syn):
    # 8 query heads per KV head, head_dim 64 (two query positions per attention CTA); 2100 rows in all, so
    # the prefill is worked off in two chunks and the second one attends over the first one's cache rows
    cfg = syn.BitLlamaConfig("llama", 512, 2048, 1, 32, 4, 5632, max_position_embeddings=1100)
    w = syn.make_weights(cfg, seed=6400, from_latent=False)
    gpu = syn.build_model(w, max_batch=2)
    ref = oracle.model_from_weights(w)
    states = [ref.new_state() for _ in range(2)]
    rng = np.random.default_rng(9)
    tokens = rng.integers(0, cfg.vocab_size, size=(2, 1050))
    logits, nxt = gpu.prefill(tokens)
    assert gpu.current_pos == 1050
    # the stage-by-stage check on a short continuation (the long prefill itself would take the oracle minutes)
    for s, st in enumerate(states):
        for li in range(cfg.num_layers):
            kq, ks, vq, vs = gpu.kv_cache(li).export(s, 1050)
            st.kq[li] = [np.ascontiguousarray(kq[:, t]) for t in range(1050)]
            st.ks[li] = [np.ascontiguousarray(ks[:, t]) for t in range(1050)]
            st.vq[li] = [np.ascontiguousarray(vq[:, t]) for t in range(1050)]
            st.vs[li] = [np.ascontiguousarray(vs[:, t]) for t in range(1050)]
        st.pos = 1050
    staged_prefill(oracle, ref, gpu, cfg, rng.integers(0, cfg.vocab_size, size=(2, 9)), states)
    assert bt.lib().bt_device_check(0) == 0


def test_prefill_errors(bt, syn):
    cfg = syn.BitLlamaConfig("llama", 64, 64, 1, 2, 1, 64, max_position_embeddings=8)
    gpu = syn.build_model(syn.make_weights(cfg, seed=1))
    with pytest.raises(bt.BitTTTError) as ei:
        gpu.prefill(np.zeros((1, 9), np.int32))
    assert ei.value.status == bt.BT_ERR_SHAPE  # beyond max_position_embeddings
    with pytest.raises(bt.BitTTTError) as ei:
        gpu.prefill(np.zeros((2, 3), np.int32))
    assert ei.value.status == bt.BT_ERR_SHAPE  # more sequences than max_batch
    gpu.prefill(np.zeros((1, 8), np.int32))
    assert gpu.current_pos == 8
