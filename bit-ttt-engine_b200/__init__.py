"""Python host side of the B200 BitLinear library.

The compute lives in ``lib/libbitttt_b200.so`` (hand-written sm_100a CUDA behind the C ABI
of ``include/bitttt.h``).  This package binds that ABI with ctypes and mirrors the layer
interface of the reference engine (``BitLinear.load / precompute_packed / forward`` and
friends, crates/rust_engine/src/layers/) so that tests read like the reference's own.
PyTorch is used only to own device buffers and streams.

There is no CPU fallback: if the shared library is missing or cannot be loaded, import
of :func:`lib` raises.
"""
from __future__ import annotations

import ctypes as C
import os

from . import build as _build

BT_OK = 0
BT_ERR_SHAPE, BT_ERR_ALIGN, BT_ERR_DEVICE, BT_ERR_CUDA = -1, -2, -3, -4
BT_ERR_NCCL, BT_ERR_TIMEOUT, BT_ERR_NOMEM, BT_ERR_ARG = -5, -6, -7, -8
BT_F32, BT_BF16, BT_I8, BT_I32, BT_F16 = 0, 1, 2, 3, 4

_LIB = None


class BitTTTError(RuntimeError):
    def __init__(self, status: int, message: str):
        super().__init__(f"[bt_status {status}] {message}")
        self.status = status
        self.message = message


def lib_path() -> str:
    return _build.LIB_PATH


def lib() -> C.CDLL:
    """Loads libbitttt_b200.so (never builds it, never falls back)."""
    global _LIB
    if _LIB is not None:
        return _LIB
    path = lib_path()
    if not os.path.exists(path):
        raise ImportError(
            f"{path} is missing: build it with `python bit-ttt-engine_b200/build.py` "
            "(there is no CPU or PyTorch fallback)")
    L = C.CDLL(path)
    vp, i64, i32, f32 = C.c_void_p, C.c_int64, C.c_int, C.c_float
    L.bt_last_error.restype = C.c_char_p
    L.bt_version.restype = i32
    L.bt_device_count.restype = i32
    L.bt_device_check.argtypes = [i32]
    L.bt_pack_ternary.argtypes = [vp, i64, vp, C.POINTER(f32)]
    L.bt_unpack_ternary.argtypes = [vp, i64, f32, vp]
    L.bt_convert_l3_to_l2.argtypes = [vp, i64, i64, i32, vp]
    L.bt_linear_create.argtypes = [C.POINTER(vp), vp, i64, i64, i32, vp, i32]
    L.bt_linear_destroy.argtypes = [vp]
    L.bt_linear_dims.argtypes = [vp, C.POINTER(i64), C.POINTER(i64), C.POINTER(i32)]
    L.bt_workspace_create.argtypes = [C.POINTER(vp), i32, C.c_size_t]
    L.bt_workspace_destroy.argtypes = [vp]
    L.bt_linear_forward.argtypes = [vp, vp, vp, i64, i64, i32, vp, i32, vp]
    L.bt_linear_forward_noalloc.argtypes = [vp, vp, i64, i64, i32, vp, i32, vp]
    L.bt_linear_forward_q.argtypes = [vp, vp, vp, vp, i64, vp, i32, vp]
    L.bt_linear_forward_host.argtypes = [vp, vp, i64, i64, vp]
    L.bt_act_quant.argtypes = [vp, i32, i64, i64, vp, vp, vp, i32, vp]
    _LIB = L
    return L


def check(status: int) -> None:
    if status != BT_OK:
        raise BitTTTError(status, lib().bt_last_error().decode("utf-8", "replace"))


from .layers import (  # noqa: E402
    BitLinear, PackedTensor, Workspace, act_quant, pack_ternary, unpack_ternary,
)

from .model import (  # noqa: E402
    BitLlama, BitLlamaConfig, QuantizedKVCache, attn_decode, tp_unique_id, ttt_update,
)
from . import model  # noqa: E402,F401

__all__ = [
    "BitLlama", "BitLlamaConfig", "QuantizedKVCache", "attn_decode", "ttt_update",
    "lib", "lib_path", "check", "BitTTTError", "BitLinear", "PackedTensor", "Workspace",
    "act_quant", "pack_ternary", "unpack_ternary",
]
