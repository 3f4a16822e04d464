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
    (16, 8, 128, 290, 10, 320, 41), (8, 8, 64, 150, 10, 160, 29),
    # one (sequence, KV head) pair, as on a rank of eight-way tensor parallelism: the largest cluster the GPU
    # offers, most of its spans empty at first, more and more of them pushing partial columns as the context grows
    (4, 1, 128, 300, 1, 2112, 37)])
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


def test_kv_append_standalone_and_import_export(bt, oracle):
    # QuantizedKVCache::append on its own (layers/kv_cache.rs:50-92): stored bytes and scales equal
    # the oracle's quantize_q8; export -> import into a second cache -> same attention output
    rng = np.random.default_rng(123)
    batch, n_kv, hd, n_heads, steps = 3, 2, 64, 8, 5
    cache = bt.QuantizedKVCache(16, batch, n_kv, hd)
    ks_all, vs_all = [], []
    for p in range(steps):
        k = rng.normal(0, 1, (batch, n_kv, hd)).astype(np.float32)
        v = rng.normal(0, 1, (batch, n_kv, hd)).astype(np.float32)
        if p == 2:
            v[1] = 0  # an all-zero row: scale 0, bytes 128
        pos = torch.full((batch,), p, dtype=torch.int32, device="cuda")
        cache.append(torch.from_numpy(k).cuda(), torch.from_numpy(v).cuda(), pos)
        ks_all.append(k); vs_all.append(v)
    for b in range(batch):
        kq, ks, vq, vs = cache.export(b, steps)
        for p in range(steps):
            q0, s0 = oracle.kv_quant(ks_all[p][b])
            assert np.array_equal(kq[:, p], q0) and np.array_equal(ks[:, p], s0)
            q1, s1 = oracle.kv_quant(vs_all[p][b])
            assert np.array_equal(vq[:, p], q1) and np.array_equal(vs[:, p], s1)
    kq, ks, vq, vs = cache.export(1, steps)
    assert (vq[:, 2] == 128).all() and (vs[:, 2] == 0).all()
    # a second cache restored from the exported rows attends identically
    other = bt.QuantizedKVCache(16, batch, n_kv, hd)
    for b in range(batch):
        other.load(b, *cache.export(b, steps))
    qkv = torch.from_numpy(rng.normal(0, 1, (batch, (n_heads + 2 * n_kv) * hd)).astype(np.float32)).cuda()
    pos = torch.full((batch,), steps, dtype=torch.int32, device="cuda")
    a = bt.attn_decode(cache, qkv, pos, n_heads, 10000.0)
    b2 = bt.attn_decode(other, qkv, pos, n_heads, 10000.0)
    assert torch.equal(a, b2)


@pytest.mark.parametrize("n_heads,n_kv,hd,t0,batch", [(32, 8, 128, 2040, 1), (32, 4, 64, 700, 1), (8, 8, 96, 300, 2),
                                                         (32, 8, 128, 1500, 24)])
def test_attention_long_context_many_spans(bt, oracle, n_heads, n_kv, hd, t0, batch):
    # a long seeded context: with one sequence the positions are cut over a whole cluster of spans
    # (16 x 128 at 2048), with 24 sequences x 8 KV heads every CTA walks many tiles of its own
    rng = np.random.default_rng(t0 + hd)
    max_seq = t0 + 16
    cache = bt.QuantizedKVCache(max_seq, batch, n_kv, hd)
    seeds = []
    for b in range(batch):
        kq = rng.integers(0, 256, size=(n_kv, t0, hd), dtype=np.uint8)
        vq = rng.integers(0, 256, size=(n_kv, t0, hd), dtype=np.uint8)
        ks = rng.uniform(0.005, 0.03, size=(n_kv, t0)).astype(np.float32)
        vs = rng.uniform(0.005, 0.03, size=(n_kv, t0)).astype(np.float32)
        cache.load(b, kq, ks, vq, vs)
        seeds.append([kq, ks, vq, vs])
    theta = 500000.0
    qkv_dim = (n_heads + 2 * n_kv) * hd
    for step in range(10):
        p = t0 + step
        qkv = rng.normal(0, 1, (batch, qkv_dim)).astype(np.float32)
        pos = torch.full((batch,), p, dtype=torch.int32, device="cuda")
        out = bt.attn_decode(cache, torch.from_numpy(qkv).cuda(), pos, n_heads, theta).cpu().numpy()
        for b in range(batch):
            q = oracle.rope(qkv[b, :n_heads * hd].reshape(n_heads, hd), p, theta)
            k = oracle.rope(qkv[b, n_heads * hd:(n_heads + n_kv) * hd].reshape(n_kv, hd), p, theta)
            v = qkv[b, (n_heads + n_kv) * hd:].reshape(n_kv, hd)
            kq1, ks1 = oracle.kv_quant(k)
            vq1, vs1 = oracle.kv_quant(v)
            s = seeds[b]
            s[0] = np.concatenate([s[0], kq1[:, None]], 1); s[1] = np.concatenate([s[1], ks1[:, None]], 1)
            s[2] = np.concatenate([s[2], vq1[:, None]], 1); s[3] = np.concatenate([s[3], vs1[:, None]], 1)
            if batch > 4 and b % 5 != 0:
                continue  # the oracle checks every fifth sequence of the large batch
            t = p + 1
            kd = oracle.kv_dequant(s[0].reshape(n_kv * t, hd), s[1].reshape(-1)).reshape(n_kv, t, hd)
            vd = oracle.kv_dequant(s[2].reshape(n_kv * t, hd), s[3].reshape(-1)).reshape(n_kv, t, hd)
            ref = oracle.attn_decode(q, kd, vd).reshape(-1)
            assert rel_err(out[b], ref) <= REL_TOL, (step, b, rel_err(out[b], ref))
            assert rel_err(out[b], ref) <= 2e-5, (step, b, rel_err(out[b], ref))  # expected accuracy of the f32 path
    assert bt.lib().bt_device_check(0) == 0
