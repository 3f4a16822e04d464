"""The reference's own CUDA kernels as a second opinion on the ternary product.

oracle/_ref/libref_kernels.so holds bit_linear_forward (kernels/bit_op.cu:4-45) and
adaptive_gemm_n3_kernel_f32 (kernels/adaptive_bit_op.cu:74-161), compiled unchanged from
the reference's source files (oracle/Makefile, target `ref`).  The reference itself never
launches them, but they are its statement of the arithmetic: on integer-valued inputs every
f32 sum is exact, so the reference kernel, the CPU oracle and this library's int32
accumulators must agree bit for bit."""
import numpy as np
import pytest

from gpu_util import load_bt, rel_err, ternary_packed

torch = pytest.importorskip("torch")
pytestmark = pytest.mark.gpu

REL_TOL = 1e-3


@pytest.fixture(scope="module")
def bt():
    if not torch.cuda.is_available():
        pytest.fail("GPU tests need a CUDA device")
    return load_bt()


@pytest.fixture(scope="module")
def ref(oracle):
    if oracle.ref_lib() is None:
        pytest.fail("oracle/_ref/libref_kernels.so is missing: run `make -C oracle ref REFERENCE=<reference checkout>`")
    return oracle


@pytest.mark.parametrize("m,n,k", [(1, 64, 64), (3, 100, 36), (8, 2048, 2048), (2, 688, 256), (1, 4096, 4096),
                                   (5, 48, 14336), (17, 64, 512)])
def test_bit_linear_forward_kernel_pins_oracle_and_library(bt, ref, m, n, k):
    rng = np.random.default_rng(500 + m + n + k)
    packed = ternary_packed(rng, n, k, p_code3=0.02)
    q = rng.integers(-127, 128, size=(m, k), dtype=np.int8)
    # the reference kernel on integer-valued f32 inputs, scale 1
    y_ref = ref.ref_bit_linear_forward(q.astype(np.float32), packed, n, 1.0)
    # the CPU restatement of BitLinearCpu::forward gives the same integers ...
    assert np.array_equal(ref.bitlinear_f32(q.astype(np.float32), packed, n, 1.0), y_ref)
    assert np.array_equal(ref.bitlinear_i32(q, packed, n).astype(np.float32), y_ref)
    # ... and so do this library's accumulators
    lin = bt.BitLinear.from_packed(packed, [1.0], n, k)
    acc = lin.forward_q(torch.from_numpy(q).cuda()).cpu().numpy()
    assert np.array_equal(acc.astype(np.float32), y_ref)


def test_bit_linear_forward_kernel_on_real_valued_inputs(bt, ref):
    # f32 inputs: the reference kernel adds sequentially over k, the CPU kernel in 8 lanes; both are
    # f32 evaluations of the same sum and agree to rounding, and the quantised pipeline of this
    # library stays within the activation-quantisation noise of them
    rng = np.random.default_rng(9)
    m, n, k = 4, 512, 2048
    packed = ternary_packed(rng, n, k)
    x = rng.normal(0, 1, (m, k)).astype(np.float32)
    y_ref = ref.ref_bit_linear_forward(x, packed, n, 0.016)
    assert rel_err(ref.bitlinear_f32(x, packed, n, 0.016), y_ref) <= 1e-5
    lin = bt.BitLinear.from_packed(packed, [0.016], n, k)
    y = lin.forward(torch.from_numpy(x).cuda()).cpu().numpy()
    assert rel_err(y, y_ref) <= 0.05


@pytest.mark.parametrize("m,n,k", [(1, 64, 64), (4, 80, 320), (11, 96, 1024)])
def test_adaptive_gemm_n3_kernel_pins_multi_basis_product(bt, ref, m, n, k):
    # legacy one-byte-per-weight layout, three bases.  Integer-valued activations with max |x| = 127
    # (quantisation scale exactly 1) and power-of-two basis scales make every operation exact on both
    # sides, so the results must be equal although the orders of summation differ.
    rng = np.random.default_rng(700 + m + n + k)
    bases = rng.integers(-1, 2, size=(3, n, k)).astype(np.int8)
    scales = np.array([0.5, 0.125, 0.03125], np.float32)
    x = rng.integers(-127, 128, size=(m, k)).astype(np.float32)
    x[:, 0] = 127.0
    l3 = ref.pack_l3(bases)
    assert l3.shape == (n, k // 4, 3, 4)
    y_ref = ref.ref_adaptive_gemm_n3(x, l3, scales)
    lin = bt.BitLinear.from_l3(l3, scales, n, k)
    y = lin.forward(torch.from_numpy(x).cuda()).cpu().numpy()
    assert np.array_equal(y, y_ref)
    # the same checkpoint in the 2-bit layout, through the oracle
    l2 = ref.pack_l2(bases)
    assert np.array_equal(ref.bitlinear_q(x, l2, scales, n, n_bases=3), y_ref)
    # and the reader refuses bytes that are not ternary
    bad = l3.copy()
    bad[0, 0, 0, 0] = 5
    with pytest.raises(bt.BitTTTError) as ei:
        bt.BitLinear.from_l3(bad, scales, n, k)
    assert ei.value.status == bt.BT_ERR_ARG
