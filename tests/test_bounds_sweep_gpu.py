"""Exhaustive small-shape sweep of the BitLinear product with canary words around every
output buffer.  Every token count 1..33 (the 8-token chunks of the streaming kernel, the
64-token blocks of the tensor-core kernel and their ragged ends) times odd output widths
times input widths around the 256-input tile boundary; outputs are compared bit for bit with
the oracle and the words before and after the output must be untouched: an out-of-bounds
store in a padded tile (n_out % 16 != 0, k_in % 256 != 0) shows up here."""
import ctypes as C

import numpy as np
import pytest

from gpu_util import load_bt, ternary_packed

torch = pytest.importorskip("torch")
pytestmark = pytest.mark.gpu

CANARY = 64                      # 32-bit words on each side of an output buffer
SENTINEL_I32 = -1412623820       # 0xABCD1234 as int32
N_VALUES = (1, 17, 33, 255)
K_VALUES = (4, 8, 36, 252, 256, 260, 688)


@pytest.fixture(scope="module")
def bt():
    if not torch.cuda.is_available():
        pytest.fail("GPU tests need a CUDA device")
    return load_bt()


def guarded(m, n, dtype):
    buf = torch.full((2 * CANARY + m * n,), SENTINEL_I32, dtype=torch.int32, device="cuda")
    return buf, buf[CANARY:CANARY + m * n].view(dtype).view(m, n)


def canaries_intact(buf, m, n):
    head = buf[:CANARY]
    tail = buf[CANARY + m * n:]
    return bool((head == SENTINEL_I32).all()) and bool((tail == SENTINEL_I32).all())


@pytest.mark.parametrize("k", K_VALUES)
def test_all_token_counts_with_canaries(bt, oracle, k):
    L = bt.lib()
    stream = C.c_void_p(torch.cuda.current_stream().cuda_stream)
    rng = np.random.default_rng(8000 + k)
    for n in N_VALUES:
        packed = ternary_packed(rng, n, k, p_code3=0.05)
        lin = bt.BitLinear.from_packed(packed, [0.016], n, k)
        for m in range(1, 34):
            q = rng.integers(-127, 128, size=(m, k), dtype=np.int8)
            qd = torch.from_numpy(q).cuda()
            buf, out = guarded(m, n, torch.int32)
            st = L.bt_linear_forward_q(lin._h, None, C.c_void_p(qd.data_ptr()), None, m,
                                       C.c_void_p(out.data_ptr()), bt.BT_I32, stream)
            assert st == bt.BT_OK, L.bt_last_error()
            torch.cuda.synchronize()
            assert canaries_intact(buf, m, n), ("int32 path wrote outside its output", m, n, k)
            assert np.array_equal(out.cpu().numpy(), oracle.bitlinear_i32(q, packed, n)), (m, n, k)
            # f32 activations in, f32 out: quantiser + product (tensor-core kernel from 9 tokens on)
            x = rng.normal(0, 1, (m, k)).astype(np.float32)
            xd = torch.from_numpy(x).cuda()
            buf, out = guarded(m, n, torch.float32)
            st = L.bt_linear_forward(lin._h, None, C.c_void_p(xd.data_ptr()), m, k, bt.BT_F32,
                                     C.c_void_p(out.data_ptr()), bt.BT_F32, stream)
            assert st == bt.BT_OK, L.bt_last_error()
            torch.cuda.synchronize()
            assert canaries_intact(buf, m, n), ("f32 path wrote outside its output", m, n, k)
            assert np.array_equal(out.cpu().numpy(), oracle.bitlinear_q(x, packed, [0.016], n)), (m, n, k)
    assert L.bt_device_check(0) == bt.BT_OK
