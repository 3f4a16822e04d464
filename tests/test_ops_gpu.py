"""GPU parity of the TTT update, the Q8 KV cache + decode attention, against the oracle."""
import numpy as np
import pytest

from gpu_util import load_bt

torch = pytest.importorskip("torch")
pytestmark = pytest.mark.gpu

REL_TOL = 1e-3  # stated tolerance for f32 outputs / states


@pytest.fixture(scope="module")
def bt():
    if not torch.cuda.is_available():
        pytest.fail("GPU tests need a CUDA device")
    return load_bt()


def rel_err(a, b):
    return float(np.abs(a - b).max() / max(np.abs(b).max(), 1e-30))


@pytest.mark.parametrize("d", [4, 16, 64, 128, 512])
def test_ttt_step_sequence(bt, oracle, d):
    # recipe of bin/test_memory.rs:14-75: deterministic features, lr 0.1, A/B/A/B pattern
    rng = np.random.default_rng(d)
    batch, steps, lr = 3, 6, 0.1
    w_ref = rng.normal(0, 0.05, (batch, d, d)).astype(np.float32)
    w_gpu = torch.from_numpy(w_ref.copy()).cuda()
    pats = rng.normal(0, 1, (2, batch, d)).astype(np.float32)
    for s in range(steps):
        f = pats[s % 2]
        z = bt.ttt_update(w_gpu, torch.from_numpy(f).cuda(), lr).cpu().numpy()
        for b in range(batch):
            z_ref = oracle.ttt_step(w_ref[b], f[b], lr)
            assert rel_err(z[b], z_ref) <= REL_TOL
    assert rel_err(w_gpu.cpu().numpy(), w_ref) <= REL_TOL


@pytest.mark.parametrize("t_len,chunk", [(16, 16), (37, 16), (5, 32), (64, 1)])
def test_ttt_chunkwise(bt, oracle, t_len, chunk):
    rng = np.random.default_rng(t_len * 100 + chunk)
    batch, d, lr = 2, 64, 0.01
    w_ref = rng.normal(0, 0.05, (batch, d, d)).astype(np.float32)
    feats = rng.normal(0, 1, (batch, t_len, d)).astype(np.float32)
    w_gpu = torch.from_numpy(w_ref.copy()).cuda()
    z = bt.ttt_update(w_gpu, torch.from_numpy(feats).cuda(), lr, chunk).cpu().numpy()
    for b in range(batch):
        z_ref = oracle.ttt_chunk(w_ref[b], feats[b], lr, chunk)
        assert rel_err(z[b], z_ref) <= REL_TOL
    assert rel_err(w_gpu.cpu().numpy(), w_ref) <= REL_TOL


def test_ttt_zero_feature_is_safe(bt):
    w = torch.zeros(1, 16, 16, device="cuda")
    z = bt.ttt_update(w, torch.zeros(1, 16, device="cuda"), 0.1)
    assert torch.isfinite(z).all() and torch.isfinite(w).all()


@pytest.mark.parametrize("n_heads,n_kv,hd,steps,batch,max_seq,every", [
    (4, 2, 64, 9, 2, 128, 1), (32, 8, 128, 5, 2, 128, 1), (8, 1, 32, 70, 2, 128, 1), (4, 4, 64, 3, 2, 128, 1),
    # one span per (sequence, KV head) pair (80 pairs: two would not fit in one wave): the span grows past
    # one and two 128-position tiles, so the tile loop, the next-tile copies and the running maximum are used
    (16, 8, 128, 290, 10, 320, 41), (8, 8, 64, 150, 10, 160, 29)])
def test_attention_decode_matches_oracle(bt, oracle, n_heads, n_kv, hd, steps, batch, max_seq, every):
    rng = np.random.default_rng(n_heads * 1000 + hd)
    theta = 10000.0
    cache = bt.QuantizedKVCache(max_seq, batch, n_kv, hd)
    hist = [dict(kq=[], ks=[], vq=[], vs=[]) for _ in range(batch)]
    qkv_dim = (n_heads + 2 * n_kv) * hd
    for p in range(steps):
        qkv = rng.normal(0, 1, (batch, qkv_dim)).astype(np.float32)
        pos = torch.full((batch,), p, dtype=torch.int32, device="cuda")
        out = bt.attn_decode(cache, torch.from_numpy(qkv).cuda(), pos, n_heads, theta).cpu().numpy()
        for b in range(batch):
            q = oracle.rope(qkv[b, :n_heads * hd].reshape(n_heads, hd), p, theta)
            k = oracle.rope(qkv[b, n_heads * hd:(n_heads + n_kv) * hd].reshape(n_kv, hd), p, theta)
            v = qkv[b, (n_heads + n_kv) * hd:].reshape(n_kv, hd)
            kq, ks = oracle.kv_quant(k)
            vq, vs = oracle.kv_quant(v)
            h = hist[b]
            h["kq"].append(kq); h["ks"].append(ks); h["vq"].append(vq); h["vs"].append(vs)
            t = p + 1
            if p % every != 0 and p != steps - 1:
                continue  # long runs: the oracle checks every few steps and the last one
            kall = np.stack(h["kq"], 1); vall = np.stack(h["vq"], 1)
            ksc = np.stack(h["ks"], 1); vsc = np.stack(h["vs"], 1)
            kd = oracle.kv_dequant(kall.reshape(n_kv * t, hd), ksc.reshape(-1)).reshape(n_kv, t, hd)
            vd = oracle.kv_dequant(vall.reshape(n_kv * t, hd), vsc.reshape(-1)).reshape(n_kv, t, hd)
            ref = oracle.attn_decode(q, kd, vd).reshape(-1)
            assert rel_err(out[b], ref) <= REL_TOL, (p, b)
    # the stored cache bytes: equal to the oracle's up to rounding ties of the RoPE'd keys
    for b in range(batch):
        kq, ks, vq, vs = cache.export(b, steps)
        assert np.array_equal(vq, np.stack(hist[b]["vq"], 1))          # v is not rotated: exact
        assert np.array_equal(vs, np.stack(hist[b]["vs"], 1))
        assert np.abs(kq.astype(np.int32) - np.stack(hist[b]["kq"], 1).astype(np.int32)).max() <= 1
        assert rel_err(ks, np.stack(hist[b]["ks"], 1)) <= 1e-5


def test_kv_cache_reset_and_ones(bt):
    # tests/attention_test.rs:35-64 feeds ones of shape (1,2,1,64): q = 255, scale = 1/127
    cache = bt.QuantizedKVCache(8, 1, 2, 64)
    qkv = torch.ones(1, (2 + 4) * 64, device="cuda")
    pos = torch.zeros(1, dtype=torch.int32, device="cuda")
    out = bt.attn_decode(cache, qkv, pos, 2, 10000.0)
    kq, ks, vq, vs = cache.export(0, 1)
    assert (vq == 255).all() and np.allclose(vs, 1 / 127) and (kq == 255).all()
    assert np.allclose(out.cpu().numpy(), 1.0, atol=1e-6)  # one key: softmax = 1, out = v
    cache.reset()
    kq, ks, vq, vs = cache.export(0, 1)
    assert (kq == 128).all() and (ks == 0).all()
