"""bt_linear_forward_noalloc: the BitLinear forward for callers that cannot allocate.

A host that has given all free device memory to its own arena, or that cannot accept the
device-wide synchronisation cudaMalloc implies, calls this entry point instead of
bt_linear_forward: outputs are caller-owned and the scratch for the quantised activations is
a fixed array inside the library.  The test drives it through the C ABI twice in a row with
different inputs (the array keeps the previous call's contents) and checks each result
against bt_linear_forward, which must agree bit for bit (the stated tolerance for f32
outputs is 1e-3 relative), and against the CPU oracle; it checks that the calls leave the
device's free memory untouched, that several bases work, and that oversize requests are refused.

This file sorts last on purpose: a run that stops at the first failure has then already
executed every other test.
"""
import ctypes as C

import numpy as np
import pytest

from gpu_util import load_bt, ternary_packed

torch = pytest.importorskip("torch")
pytestmark = pytest.mark.gpu

REL_TOL = 1e-3


def test_noalloc_matches_forward_two_calls_in_a_row(oracle):
    if not torch.cuda.is_available():
        pytest.fail("GPU tests need a CUDA device")
    bt = load_bt()
    L = bt.lib()
    rng = np.random.default_rng(77)
    n, k = 640, 1100  # k is not a multiple of 256: the padding bytes must be rewritten each call
    packed = ternary_packed(rng, n, k, p_code3=0.01)
    lin = bt.BitLinear.from_packed(packed, [0.016], n, k)
    stream = C.c_void_p(torch.cuda.current_stream().cuda_stream)
    for call, m in enumerate((8, 3)):  # second call is smaller: stale rows stay in the array
        x = torch.from_numpy(rng.normal(0, 1 + call, (m, k)).astype(np.float32)).cuda()
        expect = lin.forward(x)
        got = torch.full((m, n), float("nan"), device="cuda")
        st = L.bt_linear_forward_noalloc(lin._h, C.c_void_p(x.data_ptr()), m, k, bt.BT_F32,
                                         C.c_void_p(got.data_ptr()), bt.BT_F32, stream)
        assert st == bt.BT_OK, L.bt_last_error()
        torch.cuda.synchronize()
        e, g = expect.cpu().numpy(), got.cpu().numpy()
        assert np.abs(g - e).max() <= REL_TOL * np.abs(e).max()
        assert np.array_equal(g, e)
        ref = oracle.bitlinear_q(x.cpu().numpy(), packed, [0.016], n)  # and the CPU oracle
        assert np.abs(g - ref).max() <= REL_TOL * np.abs(ref).max()
        assert np.array_equal(g, ref)
    # bf16 in and out through the Python mirror
    xb = torch.from_numpy(rng.normal(0, 1, (2, k)).astype(np.float32)).cuda().bfloat16()
    out = torch.empty((2, n), dtype=torch.bfloat16, device="cuda")
    lin.forward_noalloc(xb, out)
    assert torch.equal(out, lin.forward(xb))
    assert L.bt_device_check(0) == bt.BT_OK


def test_noalloc_allocates_nothing_and_handles_several_bases(oracle):
    if not torch.cuda.is_available():
        pytest.fail("GPU tests need a CUDA device")
    bt = load_bt()
    L = bt.lib()
    rng = np.random.default_rng(79)
    n, k, nb = 96, 320, 2
    bases = rng.integers(-1, 2, size=(nb, n, k)).astype(np.int8)
    packed = oracle.pack_l2(bases)
    scales = np.array([0.02, 0.005], np.float32)
    lin = bt.BitLinear.from_packed(packed, scales, n, k)
    x = torch.from_numpy(rng.normal(0, 1, (5, k)).astype(np.float32)).cuda()
    out = torch.empty((5, n), device="cuda")
    lin.forward_noalloc(x, out)  # first call: symbol lookup and kernel attributes
    torch.cuda.synchronize()
    free_before, _ = torch.cuda.mem_get_info()
    for _ in range(4):
        lin.forward_noalloc(x, out)
    torch.cuda.synchronize()
    free_after, _ = torch.cuda.mem_get_info()
    assert free_after == free_before, "bt_linear_forward_noalloc changed the device's free memory"
    ref = oracle.bitlinear_q(x.cpu().numpy(), packed, scales, n, n_bases=nb)
    assert np.array_equal(out.cpu().numpy(), ref)
    # several bases with a bf16 output would need an f32 staging buffer: refused, nothing launched
    outb = torch.empty((5, n), dtype=torch.bfloat16, device="cuda")
    with pytest.raises(bt.BitTTTError) as ei:
        lin.forward_noalloc(x, outb)
    assert ei.value.status == bt.BT_ERR_ARG


def test_noalloc_rejects_oversize_requests():
    if not torch.cuda.is_available():
        pytest.fail("GPU tests need a CUDA device")
    bt = load_bt()
    L = bt.lib()
    rng = np.random.default_rng(78)
    k = 14336  # 8B MLP width: 14336 * 8 tokens fits (112 KiB), 10 tokens would not
    lin = bt.BitLinear.from_packed(ternary_packed(rng, 32, k), [1.0], 32, k)
    x = torch.zeros(10, k, device="cuda")
    y = torch.zeros(10, 32, device="cuda")
    stream = C.c_void_p(torch.cuda.current_stream().cuda_stream)
    st = L.bt_linear_forward_noalloc(lin._h, C.c_void_p(x.data_ptr()), 10, k, bt.BT_F32,
                                     C.c_void_p(y.data_ptr()), bt.BT_F32, stream)
    assert st == bt.BT_ERR_NOMEM and b"exceed the static scratch" in L.bt_last_error()
    st = L.bt_linear_forward_noalloc(lin._h, C.c_void_p(x.data_ptr()), 8, k, bt.BT_F32,
                                     C.c_void_p(y.data_ptr()), bt.BT_F32, stream)
    assert st == bt.BT_OK, L.bt_last_error()
    st = L.bt_linear_forward_noalloc(lin._h, C.c_void_p(x.data_ptr()), 2, k - 4, bt.BT_F32,
                                     C.c_void_p(y.data_ptr()), bt.BT_F32, stream)
    assert st == bt.BT_ERR_SHAPE
    torch.cuda.synchronize()
