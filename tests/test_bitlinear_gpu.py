"""GPU parity of the BitLinear path against the CPU oracle, through the C ABI.

Tiers: exact-int (int32 accumulators bitwise equal to the oracle's, which equals the
reference CPU kernel on integer-valued inputs, kernels/cpu.rs:73-124); f32 outputs of the
quantised pipeline within 1e-3 relative (they are expected to be bit-identical); bf16
outputs within one bf16 ulp of the rounded oracle."""
import numpy as np
import pytest

from gpu_util import load_bt, ternary_packed

torch = pytest.importorskip("torch")
pytestmark = pytest.mark.gpu

REL_TOL = 1e-3  # stated tolerance for floating-point outputs


@pytest.fixture(scope="module")
def bt():
    if not torch.cuda.is_available():
        pytest.fail("GPU tests need a CUDA device")
    return load_bt()


SHAPES = [  # (m, n, k)
    (1, 16, 256), (1, 64, 64), (1, 256, 688), (3, 100, 4), (1, 17, 36), (8, 2048, 2048),
    (2, 688, 256), (1, 4096, 4096), (5, 1024, 4096), (7, 48, 14336), (17, 64, 512), (33, 32, 256),
    # product kernel for up to 8 tokens: 16 KB ring stages (8 tokens of a long K leave no room for
    # 32 KB ones), an odd number of row tiles per CTA, and more row tiles per CTA than the ring has
    # slots and than there are accumulate buffers (slots and buffers are reused)
    (8, 160, 14336), (1, 7120, 4096), (1, 41000, 512), (3, 41000, 512),
    # one rank's slices of the 8B projections under 8-way tensor parallelism
    (1, 4096, 512), (1, 4096, 1792), (1, 768, 4096), (2, 3584, 4096),
]


@pytest.mark.parametrize("m,n,k", SHAPES)
def test_int32_accumulators_bit_exact(bt, oracle, m, n, k):
    rng = np.random.default_rng(1000 + m + n + k)
    packed = ternary_packed(rng, n, k, p_code3=0.02)
    q = rng.integers(-127, 128, size=(m, k), dtype=np.int8)
    lin = bt.BitLinear.from_packed(packed, [1.0], n, k)
    acc = lin.forward_q(torch.from_numpy(q).cuda()).cpu().numpy()
    ref = oracle.bitlinear_i32(q, packed, n)
    assert np.array_equal(acc, ref)
    # the reference f32 kernel on the same integer-valued inputs gives the same integers
    ref_f = oracle.bitlinear_f32(q.astype(np.float32), packed, n, 1.0)
    assert np.array_equal(acc.astype(np.float32), ref_f)


def test_saturation_rows(bt, oracle):
    # all +1 / all -1 weights against +-127 activations: the largest accumulators possible
    n, k = 32, 14336
    codes = np.zeros((n, k // 4), np.uint8)
    codes[0::2] = 0x55  # +1
    codes[1::2] = 0xAA  # -1
    q = np.full((2, k), 127, np.int8)
    q[1] = -127
    lin = bt.BitLinear.from_packed(codes, [1.0], n, k)
    acc = lin.forward_q(torch.from_numpy(q).cuda()).cpu().numpy()
    assert acc[0, 0] == 127 * k and acc[0, 1] == -127 * k and acc[1, 0] == -127 * k
    assert np.array_equal(acc, oracle.bitlinear_i32(q, codes, n))


def test_config1_forward_f32(bt, oracle):
    # 2048x2048 ternary weight, scale = mean|N(0,0.02)|, 8 tokens x 2048 ~ N(0,1)
    rng = np.random.default_rng(1234)
    n = k = 2048
    packed = ternary_packed(rng, n, k)
    scale = float(np.abs(np.random.default_rng(99).normal(0, 0.02, n * k)).mean() + 1e-6)
    x = np.random.default_rng(1235).normal(0, 1, (8, k)).astype(np.float32)
    lin = bt.BitLinear.from_packed(packed, [scale], n, k)
    y = lin.forward(torch.from_numpy(x).cuda()).cpu().numpy()
    ref = oracle.bitlinear_q(x, packed, [scale], n)
    assert np.abs(y - ref).max() <= REL_TOL * np.abs(ref).max()
    assert np.array_equal(y, ref)  # same operations in the same order
    # host-buffer entry point gives the same numbers
    assert np.array_equal(lin.forward_host(x), y)
    # informational: distance to the reference's un-quantised f32 kernel
    full = oracle.bitlinear_f32(x, packed, n, scale)
    assert np.abs(y - full).max() <= 0.05 * np.abs(full).max()


def test_act_quant_matches_oracle(bt, oracle):
    rng = np.random.default_rng(7)
    x = rng.normal(0, 1, (5, 688)).astype(np.float32)
    x[3] = 0
    q, s, qs = bt.act_quant(torch.from_numpy(x).cuda())
    q0, s0, qs0 = oracle.act_quant(x)
    assert np.array_equal(q.cpu().numpy(), q0)
    assert np.array_equal(s.cpu().numpy(), s0)
    assert np.array_equal(qs.cpu().numpy(), qs0)


def test_pack_then_forward_like_reference_layer(bt, oracle):
    # BitLinear::load + precompute_packed + forward on a rank-3 input
    rng = np.random.default_rng(21)
    n, k = 96, 128
    w = rng.normal(0, 0.02, (n, k)).astype(np.float32)
    lin = bt.BitLinear.load(k, n, w)
    lin.precompute_packed()
    x = rng.normal(0, 1, (2, 3, k)).astype(np.float32)
    y = lin.forward(torch.from_numpy(x).cuda()).cpu().numpy()
    assert y.shape == (2, 3, n)
    p, s = oracle.pack_l1(w)
    ref = oracle.bitlinear_q(x.reshape(6, k), p, [s], n).reshape(2, 3, n)
    assert np.array_equal(y, ref)


def test_multi_basis_converted_layout(bt, oracle):
    rng = np.random.default_rng(31)
    n, k, nb = 80, 320, 3
    bases = rng.integers(-1, 2, size=(nb, n, k)).astype(np.int8)
    packed = oracle.pack_l2(bases)
    scales = np.array([0.02, 0.007, 0.003], np.float32)
    x = rng.normal(0, 1, (4, k)).astype(np.float32)
    lin = bt.BitLinear.from_packed(packed, scales, n, k)
    y = lin.forward(torch.from_numpy(x).cuda()).cpu().numpy()
    ref = oracle.bitlinear_q(x, packed, scales, n, n_bases=nb)
    assert np.abs(y - ref).max() <= REL_TOL * np.abs(ref).max()
    assert np.array_equal(y, ref)
    # and against the reference's dense reconstruction on the quantised activations
    wd = oracle.decode_l2(packed, scales)
    qx, sx, _ = oracle.act_quant(x)
    dense = (qx.astype(np.float32) * sx[:, None]) @ wd.T
    assert np.abs(y - dense).max() <= REL_TOL * np.abs(dense).max()


def test_bf16_in_out(bt, oracle):
    rng = np.random.default_rng(41)
    n, k = 256, 1024
    packed = ternary_packed(rng, n, k)
    x = torch.from_numpy(rng.normal(0, 1, (3, k)).astype(np.float32)).bfloat16()
    lin = bt.BitLinear.from_packed(packed, [0.016], n, k)
    y = lin.forward(x.cuda()).float().cpu().numpy()
    ref = oracle.bitlinear_q(x.float().numpy(), packed, [0.016], n)
    ref_bf16 = torch.from_numpy(ref).bfloat16().float().numpy()
    assert np.array_equal(y, ref_bf16)


def test_shape_error_wording(bt):
    packed = np.zeros((16, 16), np.uint8)
    lin = bt.BitLinear.from_packed(packed, [1.0], 16, 64)
    with pytest.raises(bt.BitTTTError) as ei:
        lin.forward(torch.zeros(2, 32, device="cuda"))
    assert ei.value.status == bt.BT_ERR_SHAPE
    assert "Shape mismatch: Input [2, 32] vs Weight [16, 64]" in ei.value.message  # kernels/cpu.rs:22-30
    with pytest.raises(bt.BitTTTError) as ei:
        bt.BitLinear.from_packed(np.zeros(16 * 4, np.uint8), [1.0], 16, 18)
    assert ei.value.status == bt.BT_ERR_ALIGN
    assert lin.forward(torch.zeros(0, 64, device="cuda")).shape == (0, 16)  # empty input
    assert bt.lib().bt_device_check(0) == 0


@pytest.mark.parametrize("m,n,k", [(9, 128, 256), (64, 256, 1024), (100, 1000, 688), (300, 2048, 2048), (130, 48, 4096)])
def test_tensor_core_path_many_tokens(bt, oracle, m, n, k):
    # more than 8 tokens go through the tcgen05 kernel; same bits as the oracle pipeline
    rng = np.random.default_rng(m * 7 + n)
    packed = ternary_packed(rng, n, k, p_code3=0.01)
    x = rng.normal(0, 1, (m, k)).astype(np.float32)
    x[m // 2] = 0  # an all-zero token
    lin = bt.BitLinear.from_packed(packed, [0.016], n, k)
    y = lin.forward(torch.from_numpy(x).cuda()).cpu().numpy()
    ref = oracle.bitlinear_q(x, packed, [0.016], n)
    assert np.abs(y - ref).max() <= REL_TOL * np.abs(ref).max()
    assert np.array_equal(y, ref)
    assert bt.lib().bt_device_check(0) == 0
