"""Layer objects with the reference engine's names and call shapes, bound to the C ABI.

Mirrors crates/rust_engine/src/kernels/packing.rs (PackedTensor) and
crates/rust_engine/src/layers/{bit_linear,adaptive_linear}.rs.  Device buffers are torch
tensors; every computation goes through libbitttt_b200.so.
"""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass

import numpy as np

from . import (BT_BF16, BT_F32, BT_I32, check, lib)


def _torch():
    import torch
    return torch


def _ptr(t):
    return C.c_void_p(t.data_ptr())


def _stream_ptr(device_index: int):
    torch = _torch()
    return C.c_void_p(torch.cuda.current_stream(device_index).cuda_stream)


def _bt_dtype(t):
    torch = _torch()
    if t.dtype == torch.float32:
        return BT_F32
    if t.dtype == torch.bfloat16:
        return BT_BF16
    raise TypeError(f"unsupported activation dtype {t.dtype}: use float32 or bfloat16")


def pack_ternary(w: np.ndarray):
    """PackedTensor::pack (kernels/packing.rs:50-105): returns (bytes, scale)."""
    w = np.ascontiguousarray(w, np.float32).reshape(-1)
    out = np.zeros((w.size + 3) // 4, np.uint8)
    scale = C.c_float(0)
    check(lib().bt_pack_ternary(w.ctypes.data, w.size, out.ctypes.data, C.byref(scale)))
    return out, float(scale.value)


def unpack_ternary(packed: np.ndarray, n_elem: int, scale: float) -> np.ndarray:
    """PackedTensor::unpack (kernels/packing.rs:108-133)."""
    packed = np.ascontiguousarray(packed, np.uint8)
    out = np.zeros(n_elem, np.float32)
    check(lib().bt_unpack_ternary(packed.ctypes.data, n_elem, scale, out.ctypes.data))
    return out


@dataclass
class PackedTensor:
    """kernels/packing.rs:15-21: flat u8 data (4 weights per byte), scale, logical shape."""
    data: np.ndarray
    scale: float
    shape: tuple

    @staticmethod
    def pack(w: np.ndarray) -> "PackedTensor":
        data, scale = pack_ternary(w)
        return PackedTensor(data, scale, tuple(w.shape))

    @staticmethod
    def new(data: np.ndarray, shape: tuple, scale: float) -> "PackedTensor":
        return PackedTensor(np.ascontiguousarray(data, np.uint8).reshape(-1), float(scale), tuple(shape))

    def unpack(self) -> np.ndarray:
        n = int(np.prod(self.shape))
        return unpack_ternary(self.data, n, self.scale).reshape(self.shape)


class Workspace:
    """Scratch memory for forward calls; one per stream in flight."""

    def __init__(self, device: int = 0, nbytes: int = 0):
        self._h = C.c_void_p()
        check(lib().bt_workspace_create(C.byref(self._h), device, nbytes))

    def __del__(self):
        try:
            if getattr(self, "_h", None):
                lib().bt_workspace_destroy(self._h)
                self._h = None
        except Exception:
            pass


class BitLinear:
    """BitLinear / AdaptiveBitLinear of the reference (layers/bit_linear.rs:13-96,
    layers/adaptive_linear.rs:40-161) with the ternary product on the GPU.

    ``BitLinear.load(in_dim, out_dim, weight, device)`` takes the dense f32 weight like the
    reference's loader; ``precompute_packed()`` quantises and packs it
    (PackedTensor::pack) and moves it to the device.  ``BitLinear.from_packed`` takes the
    packed bytes of a converted checkpoint (``weight_packed`` + ``scales``).
    """

    def __init__(self, in_features: int, out_features: int, device: int = 0):
        self.in_features = int(in_features)
        self.out_features = int(out_features)
        self.device = int(device)
        self.weight = None
        self.packed_params: PackedTensor | None = None
        self.scales = None
        self.n_bases = 1
        self._h = None

    # -- construction ------------------------------------------------------------------
    @classmethod
    def load(cls, in_dim: int, out_dim: int, weight: np.ndarray, device: int = 0) -> "BitLinear":
        w = np.ascontiguousarray(weight, np.float32)
        if w.shape != (out_dim, in_dim):
            raise ValueError(f"weight shape {w.shape} != ({out_dim}, {in_dim})")
        self = cls(in_dim, out_dim, device)
        self.weight = w
        return self

    def precompute_packed(self) -> None:
        if self.weight is None:
            raise RuntimeError("precompute_packed: no dense weight loaded")
        self.packed_params = PackedTensor.pack(self.weight)
        self._create(self.packed_params.data, [self.packed_params.scale], 1)

    @classmethod
    def from_packed(cls, packed: np.ndarray, scales, out_dim: int, in_dim: int,
                    device: int = 0) -> "BitLinear":
        """packed: u8 [out, in/4] (one basis, in-memory layout) or [out, in/4, n_bases]
        (converted checkpoint layout)."""
        self = cls(in_dim, out_dim, device)
        packed = np.ascontiguousarray(packed, np.uint8)
        scales = np.atleast_1d(np.asarray(scales, np.float32))
        n_bases = 1 if packed.ndim <= 2 else packed.shape[2]
        if scales.size != n_bases:
            raise ValueError(f"{scales.size} scales for {n_bases} bases")
        if n_bases == 1:
            self.packed_params = PackedTensor.new(packed, (out_dim, in_dim), float(scales[0]))
        self._create(packed, scales, n_bases)
        return self

    @classmethod
    def from_l3(cls, packed_l3: np.ndarray, scales, out_dim: int, in_dim: int, device: int = 0) -> "BitLinear":
        """packed_l3: the legacy int8 layout [out, in/4, n_bases, 4] of
        tools/conversion/convert_adaptive.py:43-83 (values -1/0/+1, one byte each); converted to the
        2-bit layout on the host, then handled like any converted checkpoint."""
        w = np.ascontiguousarray(packed_l3).view(np.int8)
        if w.ndim != 4 or w.shape[0] != out_dim or w.shape[1] != in_dim // 4 or w.shape[3] != 4:
            raise ValueError(f"legacy layout has shape {w.shape}, expected ({out_dim}, {in_dim // 4}, n_bases, 4)")
        n_bases = w.shape[2]
        l2 = np.zeros((out_dim, in_dim // 4, n_bases), np.uint8)
        check(lib().bt_convert_l3_to_l2(w.ctypes.data, out_dim, in_dim, n_bases, l2.ctypes.data))
        return cls.from_packed(l2, scales, out_dim, in_dim, device)

    def _create(self, packed, scales, n_bases):
        scales = np.ascontiguousarray(scales, np.float32)
        packed = np.ascontiguousarray(packed, np.uint8)
        expect = self.out_features * (self.in_features // 4) * n_bases
        if self.in_features % 4 == 0 and packed.size != expect:
            raise ValueError(f"{packed.size} packed bytes, expected {expect}")
        h = C.c_void_p()
        check(lib().bt_linear_create(C.byref(h), packed.ctypes.data, self.out_features,
                                     self.in_features, n_bases, scales.ctypes.data, self.device))
        self._h = h
        self.scales = scales
        self.n_bases = n_bases

    def __del__(self):
        try:
            if getattr(self, "_h", None):
                lib().bt_linear_destroy(self._h)
                self._h = None
        except Exception:
            pass

    # -- forward -----------------------------------------------------------------------
    def _need_handle(self):
        if self._h is None:
            raise RuntimeError("BitLinear.forward: weights are not packed; call precompute_packed() "
                               "(the dense training path of the reference is not part of this library)")

    def forward(self, x, out_dtype=None, workspace: Workspace | None = None):
        """x: CUDA tensor [..., in_features] (f32 or bf16) -> [..., out_features].
        Leading dimensions are flattened like layers/bit_linear.rs:54-62."""
        torch = _torch()
        self._need_handle()
        if not x.is_cuda:
            raise BitTTTErrorDevice()
        x2 = x.reshape(-1, x.shape[-1]).contiguous()
        out_dtype = out_dtype or x.dtype
        y = torch.empty((x2.shape[0], self.out_features), dtype=out_dtype, device=x.device)
        check(lib().bt_linear_forward(self._h, workspace._h if workspace else None, _ptr(x2),
                                      x2.shape[0], x2.shape[1], _bt_dtype(x2), _ptr(y), _bt_dtype(y),
                                      _stream_ptr(x.device.index)))
        return y.reshape(*x.shape[:-1], self.out_features)

    __call__ = forward

    def forward_noalloc(self, x, out):
        """forward() for hosts that cannot let the library allocate device memory (an arena
        that already owns the whole GPU, or a loop that cannot afford cudaMalloc's device-wide
        synchronisation): the caller supplies `out`, and the quantised-activation scratch is
        a fixed array inside the library.  At most 8 tokens and 128 KiB of padded int8
        activations; calls that may overlap on the GPU race on that array."""
        self._need_handle()
        x2 = x.reshape(-1, x.shape[-1])
        if not x2.is_contiguous() or not out.is_contiguous():
            raise ValueError("forward_noalloc needs contiguous tensors (it will not make copies)")
        check(lib().bt_linear_forward_noalloc(self._h, _ptr(x2), x2.shape[0], x2.shape[1], _bt_dtype(x2),
                                              _ptr(out), _bt_dtype(out), _stream_ptr(x.device.index)))
        return out

    def forward_q(self, q, sx=None, workspace: Workspace | None = None):
        """q: CUDA int8 [m, in_features].  sx None -> raw int32 accumulators of basis 0;
        else f32 outputs scaled with sx [m]."""
        torch = _torch()
        self._need_handle()
        q = q.contiguous()
        if q.dtype != torch.int8 or q.shape[-1] != self.in_features:
            raise ValueError("forward_q expects int8 [m, in_features]")
        m = q.shape[0]
        if sx is None:
            out = torch.empty((m, self.out_features), dtype=torch.int32, device=q.device)
            dt, sp = BT_I32, None
        else:
            sx = sx.contiguous().float()
            out = torch.empty((m, self.out_features), dtype=torch.float32, device=q.device)
            dt, sp = BT_F32, _ptr(sx)
        check(lib().bt_linear_forward_q(self._h, workspace._h if workspace else None, _ptr(q), sp, m,
                                        _ptr(out), dt, _stream_ptr(q.device.index)))
        return out

    def forward_host(self, x: np.ndarray) -> np.ndarray:
        """Host buffers in and out (f32), copies included - the reference's calling
        convention for its CUDA path (kernels/cuda.rs:21-47)."""
        self._need_handle()
        x = np.ascontiguousarray(x, np.float32)
        lead = x.shape[:-1]
        x2 = x.reshape(-1, x.shape[-1])
        y = np.empty((x2.shape[0], self.out_features), np.float32)
        check(lib().bt_linear_forward_host(self._h, x2.ctypes.data, x2.shape[0], x2.shape[1],
                                           y.ctypes.data))
        return y.reshape(*lead, self.out_features)


class BitTTTErrorDevice(RuntimeError):
    def __init__(self):
        # wording of kernels/cuda.rs:45
        super().__init__("BitLinearCuda called on non-CUDA device")


def act_quant(x):
    """Per-token absmax int8 quantiser on the GPU: (q int8 [m,k], s f32 [m], qsum i32 [m])."""
    torch = _torch()
    x2 = x.reshape(-1, x.shape[-1]).contiguous()
    m, k = x2.shape
    q = torch.empty((m, k), dtype=torch.int8, device=x.device)
    s = torch.empty((m,), dtype=torch.float32, device=x.device)
    qs = torch.empty((m,), dtype=torch.int32, device=x.device)
    check(lib().bt_act_quant(_ptr(x2), _bt_dtype(x2), m, k, _ptr(q), _ptr(s), _ptr(qs),
                             x.device.index, _stream_ptr(x.device.index)))
    return q, s, qs
