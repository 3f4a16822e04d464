"""Parity at the shapes the benchmark times: the Llama-3-8B block (hidden 4096, MLP 14336,
32 query / 8 KV heads of 128), the TinyLlama block (2048 / 5632 / 32 query / 4 KV heads of 64),
a hidden size above 4096, the 128256-row lm_head and the tensor-core product at 512 and 4096
tokens.  Models are cut to one or two layers and (mostly) a small vocabulary so that the CPU
oracle finishes in seconds; the caches are seeded with a long random context so that decode
attention runs over many spans, as it does in the benchmark at context 2048.  Decode steps are
checked stage by stage (see gpu_util.staged_decode_step for why, and for the tolerances)."""
import importlib

import numpy as np
import pytest

from gpu_util import load_bt, rel_err, seed_kv_caches, staged_decode_step, ternary_packed

torch = pytest.importorskip("torch")
pytestmark = pytest.mark.gpu

REL_TOL = 1e-3  # stated tolerance for f32 outputs and logits


@pytest.fixture(scope="module")
def bt():
    if not torch.cuda.is_available():
        pytest.fail("GPU tests need a CUDA device")
    return load_bt()


@pytest.fixture(scope="module")
def syn():
    return importlib.import_module("bit-ttt-engine_b200.synthetic")


def teacher_forced_from_context(oracle, syn, gpu, ref, cfg, batch, t0, n_steps, seed):
    """Seeds `t0` positions of context, then decodes `n_steps` teacher-forced tokens, every step checked
    stage by stage against the oracle (gpu_util.staged_decode_step)."""
    gpu.reset_kv_cache()
    states = [ref.new_state() for _ in range(batch)]
    rng = np.random.default_rng(seed)
    seed_kv_caches(gpu, states, cfg, t0, rng)
    tokens = rng.integers(0, cfg.vocab_size, size=(n_steps, batch))
    for t in range(n_steps):
        staged_decode_step(oracle, ref, gpu, cfg, tokens[t], states)
    assert gpu.current_pos == t0 + n_steps


@pytest.fixture(scope="module")
def llama8b_two_layers(bt, oracle, syn):
    cfg = syn.BitLlamaConfig("llama", 2048, 4096, 2, 32, 8, 14336, rope_theta=500000.0,
                             max_position_embeddings=2112)
    w = syn.make_weights(cfg, seed=5100, from_latent=False)
    return cfg, syn.build_model(w, max_batch=64), oracle.model_from_weights(w)


@pytest.mark.parametrize("batch,steps", [(1, 10), (2, 4), (8, 3), (12, 2), (64, 2)])
def test_llama8b_block_shape_long_context(bt, oracle, syn, llama8b_two_layers, batch, steps):
    # batch 1 crosses position 2048 (t0 = 2040): the benchmark's attention configuration, 16 spans
    # of 128 positions and then a 17th position group; batches above 8 run the tensor-core products
    cfg, gpu, ref = llama8b_two_layers
    teacher_forced_from_context(oracle, syn, gpu, ref, cfg, batch, 2040 if batch == 1 else 2046, steps, 77 + batch)
    assert bt.lib().bt_device_check(0) == 0


@pytest.mark.parametrize("batch,steps", [(1, 6), (16, 2)])
def test_tinyllama_block_shape(bt, oracle, syn, batch, steps):
    # 4 KV heads of 64 dims, 8 query heads per KV head
    cfg = syn.BitLlamaConfig("llama", 2048, 2048, 2, 32, 4, 5632, max_position_embeddings=640)
    w = syn.make_weights(cfg, seed=5200, from_latent=False)
    gpu = syn.build_model(w, max_batch=batch)
    ref = oracle.model_from_weights(w)
    teacher_forced_from_context(oracle, syn, gpu, ref, cfg, batch, 509, steps, 99 + batch)
    assert bt.lib().bt_device_check(0) == 0


def test_hidden_above_4096(bt, oracle, syn):
    # hidden 8192: the RMSNorm prologue of the product kernel holds two groups of 16 inputs per thread
    cfg = syn.BitLlamaConfig("llama", 512, 8192, 1, 64, 8, 1024, max_position_embeddings=64)
    w = syn.make_weights(cfg, seed=5300, from_latent=False)
    gpu = syn.build_model(w, max_batch=2)
    ref = oracle.model_from_weights(w)
    for batch in (1, 2):
        teacher_forced_from_context(oracle, syn, gpu, ref, cfg, batch, 5, 4, 5 + batch)
    assert bt.lib().bt_device_check(0) == 0


def test_lm_head_full_vocabulary(bt, oracle, syn):
    # the 128256-row dense head: warp-per-row kernel (up to 8 sequences) and tensor-core kernel (more)
    cfg = syn.BitLlamaConfig("llama", 128256, 4096, 1, 32, 8, 512, rope_theta=500000.0, max_position_embeddings=32)
    rng = np.random.default_rng(5400)
    block = syn._bf16_round(rng.normal(0, 0.02, (8016, cfg.hidden_dim)).astype(np.float32))
    table = np.tile(block, (16, 1))[:cfg.vocab_size]
    w = syn.make_weights(syn.BitLlamaConfig("llama", 16, 4096, 1, 32, 8, 512, rope_theta=500000.0, max_position_embeddings=32),
                         seed=5401, from_latent=False)
    w.cfg, w.embed, w.lm_head = cfg, table, table
    gpu = syn.build_model(w, max_batch=12)
    ref = oracle.model_from_weights(w)
    for batch in (1, 12):
        teacher_forced_from_context(oracle, syn, gpu, ref, cfg, batch, 3, 2, 40 + batch)
    assert bt.lib().bt_device_check(0) == 0


@pytest.mark.parametrize("m,n,k", [(512, 4096, 14336), (4096, 4096, 14336), (512, 14336, 4096), (4096, 14336, 4096)])
def test_tensor_core_product_at_prefill_sizes(bt, oracle, m, n, k):
    # 512 and 4096 tokens through the tcgen05 kernel; the oracle runs on a sample of output rows
    rng = np.random.default_rng(m + n + k)
    packed = ternary_packed(rng, n, k, p_code3=0.01)
    x = rng.normal(0, 1, (m, k)).astype(np.float32)
    lin = bt.BitLinear.from_packed(packed, [0.016], n, k)
    ws = bt.Workspace(0, 768 << 20)
    y = lin.forward(torch.from_numpy(x).cuda(), workspace=ws).cpu().numpy()
    rows = np.unique(np.concatenate([rng.integers(0, n, 96), [0, n - 1]]))
    toks = np.unique(np.concatenate([rng.integers(0, m, 160), [0, m - 1]]))
    ref = oracle.bitlinear_q(x[toks], np.ascontiguousarray(packed[rows]), [0.016], rows.size)
    got = y[np.ix_(toks, rows)]
    assert rel_err(got, ref) <= REL_TOL
    assert np.array_equal(got, ref)
    assert bt.lib().bt_device_check(0) == 0


def test_tensor_core_product_bf16_and_multi_basis(bt, oracle):
    rng = np.random.default_rng(61)
    # bf16 activations in, bf16 out, 40 tokens
    n, k, m = 512, 1024, 40
    packed = ternary_packed(rng, n, k)
    lin = bt.BitLinear.from_packed(packed, [0.016], n, k)
    xb = torch.from_numpy(rng.normal(0, 1, (m, k)).astype(np.float32)).bfloat16()
    y = lin.forward(xb.cuda()).float().cpu().numpy()
    ref = oracle.bitlinear_q(xb.float().numpy(), packed, [0.016], n)
    assert np.array_equal(y, torch.from_numpy(ref).bfloat16().float().numpy())
    # three bases, 70 tokens (two token blocks of the tensor-core kernel)
    n, k, m = 272, 768, 70
    bases = rng.integers(-1, 2, size=(3, n, k)).astype(np.int8)
    packed3 = oracle.pack_l2(bases)
    scales = np.array([0.02, 0.007, 0.003], np.float32)
    x = rng.normal(0, 1, (m, k)).astype(np.float32)
    lin3 = bt.BitLinear.from_packed(packed3, scales, n, k)
    y3 = lin3.forward(torch.from_numpy(x).cuda()).cpu().numpy()
    ref3 = oracle.bitlinear_q(x, packed3, scales, n, n_bases=3)
    assert rel_err(y3, ref3) <= REL_TOL
    assert np.array_equal(y3, ref3)
    assert bt.lib().bt_device_check(0) == 0


@pytest.mark.parametrize("m,n,k,nb", [(512, 14336, 1024, 2), (500, 14328, 1024, 1), (500, 14328, 768, 3)])
def test_tensor_core_product_register_split_paths(bt, oracle, m, n, k, nb):
    # Tiles of 256 rows x 128 tokens (the kernel whose epilogue warps take a whole accumulator row into registers):
    # whole tiles with a second basis accumulated onto the first, and ragged edges (a last token block of 116 tokens,
    # a last warp with rows beyond the matrix), where a warp falls back to the batched epilogue.
    rng = np.random.default_rng(m + n + k + nb)
    bases = rng.integers(-1, 2, size=(nb, n, k)).astype(np.int8)
    packed = oracle.pack_l2(bases)
    scales = np.array([0.02, 0.007, 0.003][:nb], np.float32)
    x = rng.normal(0, 1, (m, k)).astype(np.float32)
    lin = bt.BitLinear.from_packed(packed, scales, n, k)
    ws = bt.Workspace(0, 768 << 20)
    y = lin.forward(torch.from_numpy(x).cuda(), workspace=ws).cpu().numpy()
    rows = np.unique(np.concatenate([rng.integers(0, n, 96), [0, 127, 128, 255, 256, n - 130, n - 9, n - 1]]))
    toks = np.unique(np.concatenate([rng.integers(0, m, 120), [0, 127, 128, 383, 384, m - 1]]))
    ref = oracle.bitlinear_q(x[toks], np.ascontiguousarray(packed[rows]), scales, rows.size, n_bases=nb)
    got = y[np.ix_(toks, rows)]
    assert rel_err(got, ref) <= REL_TOL
    assert np.array_equal(got, ref)
    assert bt.lib().bt_device_check(0) == 0
