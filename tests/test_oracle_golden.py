"""Pins the CPU oracle: the reference's own known-answer vectors for packing
(crates/rust_engine/src/kernels/packing.rs:156-261), fixtures produced by the
reference's Python converter (tests/golden/make_golden.py), and the C code against an
independent numpy restatement."""
import os

import numpy as np
import pytest

GOLD = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "converter_l2.npz")


def test_pack_dense_cycle(oracle):
    # packing.rs:156-173: scale ~ 1.0, exact round-trip within 1e-4
    w = np.array([1, -1, 1, -1, -1, 1, 1, 1], np.float32)
    packed, scale = oracle.pack_l1(w)
    assert abs(scale - 1.0) < 1e-3
    assert np.allclose(oracle.unpack_l1(packed, 8, scale), w, atol=1e-4)


def test_pack_sparse_cycle(oracle):
    # packing.rs:176-202: scale 0.5, dequantises to +-0.5
    w = np.array([1, -1, 0, 0, 1, -1, 0, 0], np.float32)
    packed, scale = oracle.pack_l1(w)
    assert abs(scale - 0.5) < 1e-3
    assert np.allclose(oracle.unpack_l1(packed, 8, scale),
                       [0.5, -0.5, 0, 0, 0.5, -0.5, 0, 0], atol=1e-4)


def test_unpack_manual_byte_73(oracle):
    # packing.rs:205-232: byte 73 <-> [+1, -1, 0, +1] at scale 1.0, exact
    out = oracle.unpack_l1(np.array([73], np.uint8), 4, 1.0)
    assert out.tolist() == [1.0, -1.0, 0.0, 1.0]
    packed, _ = oracle.pack_l1(np.array([1, -1, 0, 1], np.float32))
    assert packed.tolist() == [73]


def test_pack_padding(oracle):
    # packing.rs:236-261: [1,1,1,1,-1] -> bytes [85, 2], length 2
    w = np.array([1, 1, 1, 1, -1], np.float32)
    packed, scale = oracle.pack_l1(w)
    assert packed.tolist() == [85, 2]
    assert np.allclose(oracle.unpack_l1(packed, 5, scale), w, atol=1e-4)


def test_code_11_decodes_to_zero(oracle):
    # kernels/cpu.rs:55-59 LUT [0,1,-1,0]; packing.rs:120-124 `_ => 0.0`
    assert oracle.unpack_l1(np.array([0xFF], np.uint8), 4, 2.0).tolist() == [0, 0, 0, 0]
    x = np.arange(1, 33, dtype=np.float32)[None, :]
    y = oracle.bitlinear_f32(x, np.full(8, 0xFF, np.uint8), 1, 1.0)
    assert y[0, 0] == 0.0


@pytest.mark.parametrize("tag", ["a", "b", "c"])
def test_converter_fixtures(oracle, tag):
    g = np.load(GOLD)
    bases, scales, packed = g[f"{tag}_bases"], g[f"{tag}_scales"], g[f"{tag}_packed"]
    # pack_2bit layout [Out, In/4, NumBases]: convert_llama_v2.py:111-151
    assert np.array_equal(oracle.pack_l2(bases), packed)
    # reader side (adaptive_linear.rs:86-109) inverts the writer
    w = oracle.decode_l2(packed, scales)
    expect = np.zeros_like(w)
    for b in range(bases.shape[0]):
        expect += bases[b].astype(np.float32) * scales[b]
    assert np.array_equal(w, expect)
    # single-basis L2 is byte-identical to L1 and the converter's scale is mean|w| (no eps)
    if bases.shape[0] == 1:
        l1, scale = oracle.pack_l1(g[f"{tag}_w"])
        assert np.array_equal(l1, packed.reshape(-1))
        assert abs(scale - (scales[0] + 1e-6)) < 1e-7
    # legacy one-byte-per-weight layout [Out, In/4, NumBases, 4] with -1 stored as 255
    legacy = g[f"{tag}_legacy"].astype(np.int8)
    n, kq, nb, _ = legacy.shape
    assert np.array_equal(legacy.transpose(2, 0, 1, 3).reshape(nb, n, kq * 4), bases)


def test_c_matches_numpy_twin(oracle):
    rng = np.random.default_rng(5)
    for (m, n, k) in [(1, 3, 4), (2, 5, 36), (3, 7, 688), (8, 16, 256)]:
        w = rng.normal(0, 0.02, (n, k)).astype(np.float32)
        p_c, s_c = oracle.pack_l1(w)
        p_np, s_np = oracle.np_pack_l1(w)
        assert np.array_equal(p_c, p_np) and abs(s_c - s_np) < 1e-9
        rows = p_c.reshape(n, k // 4)
        x = rng.normal(0, 1, (m, k)).astype(np.float32)
        q_c, sx_c, qs_c = oracle.act_quant(x)
        q_np, sx_np = oracle.np_act_quant(x)
        assert np.array_equal(q_c, q_np) and np.array_equal(sx_c, sx_np)
        assert np.array_equal(qs_c, q_np.astype(np.int32).sum(axis=1))
        acc = oracle.bitlinear_i32(q_c, p_c, n)
        assert np.array_equal(acc, oracle.np_bitlinear_i32(q_np, rows, k))
        # integer-valued f32 activations through the f32 kernel give the same integers
        # (every partial sum < 2^24): kernels/cpu.rs:73-124
        y = oracle.bitlinear_f32(q_c.astype(np.float32), p_c, n, 1.0)
        assert np.array_equal(y, acc.astype(np.float32))
        # the quantised pipeline = ((acc * s_w) * s_x)
        yq = oracle.bitlinear_q(x, p_c, [s_c], n)
        expect = (acc.astype(np.float32) * np.float32(s_c)) * sx_c[:, None]
        assert np.array_equal(yq, expect)


def test_act_quant_zero_row_and_saturation(oracle):
    x = np.zeros((2, 8), np.float32)
    x[1] = [1, -1, 0.5, -0.5, 0.25, 0, 1, -1]
    q, s, qs = oracle.act_quant(x)
    assert s[0] == 0 and not q[0].any()
    assert q[1].tolist() == [127, -127, 64, -64, 32, 0, 127, -127]  # .5 ties away from zero


def test_ttt_step_matches_formula(oracle):
    rng = np.random.default_rng(9)
    d = 16
    w = rng.normal(0, 0.1, (d, d)).astype(np.float32)
    f = rng.normal(0, 1, d).astype(np.float32)
    w0 = w.copy()
    z = oracle.ttt_step(w, f, 0.1)
    fh = f / (np.sqrt((f * f).sum()) + 1e-6)
    z_ref = w0 @ fh
    assert np.allclose(z, z_ref, rtol=1e-5, atol=1e-6)
    assert np.allclose(w, w0 - 0.1 * np.outer(z_ref - fh, fh), rtol=1e-5, atol=1e-6)
    # chunk of one token == single step (layers/ttt.rs:80-119 vs :48-74)
    w2 = w0.copy()
    z2 = oracle.ttt_chunk(w2, f[None, :], 0.1, 1)
    assert np.allclose(z2[0], z, rtol=1e-6, atol=1e-7) and np.allclose(w2, w, rtol=1e-6, atol=1e-7)


def test_kv_quant_roundtrip(oracle):
    # attention_test.rs:35-64 uses ones of shape (1,2,1,64): q = 255, s = 1/127
    q, s = oracle.kv_quant(np.ones((2, 64), np.float32))
    assert (q == 255).all() and np.allclose(s, 1 / 127)
    assert np.allclose(oracle.kv_dequant(q, s), 1.0, atol=1e-6)
    q0, s0 = oracle.kv_quant(np.zeros((1, 64), np.float32))
    assert (q0 == 128).all() and s0[0] == 0


def test_rope_and_attention_small(oracle):
    rng = np.random.default_rng(3)
    hd = 8
    x = rng.normal(0, 1, (2, hd)).astype(np.float32)
    assert np.array_equal(oracle.rope(x, 0, 10000.0), x)  # position 0 is the identity
    y = oracle.rope(x, 5, 10000.0)
    inv = (1.0 / 10000.0 ** (np.arange(0, hd, 2) / hd)).astype(np.float32)
    fr = np.float32(5) * inv
    c, s = np.cos(fr), np.sin(fr)
    ref = np.concatenate([x[:, :4] * c - x[:, 4:] * s, x[:, :4] * s + x[:, 4:] * c], axis=1)
    assert np.allclose(y, ref, atol=1e-6)
    q = rng.normal(0, 1, (4, hd)).astype(np.float32)
    k = rng.normal(0, 1, (2, 5, hd)).astype(np.float32)
    v = rng.normal(0, 1, (2, 5, hd)).astype(np.float32)
    out = oracle.attn_decode(q, k, v)
    for h in range(4):
        sc = (k[h // 2] @ q[h]) / np.sqrt(hd)
        p = np.exp(sc - sc.max()); p /= p.sum()
        assert np.allclose(out[h], p @ v[h // 2], atol=1e-5)
