"""Model-level mirror of the reference engine (crates/rust_engine/src/model/llama.rs,
layers/ttt.rs, layers/attention.rs, layers/kv_cache.rs) bound to the C ABI."""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass

import numpy as np

from . import check, lib
from .layers import _ptr, _stream_ptr, _torch

ARCH_TTT, ARCH_LLAMA = 0, 1
(W_Q, W_K, W_V, W_O, W_GATE, W_UP, W_DOWN, W_TTT_DOWN, W_TTT_UP) = range(9)
(T_EMBED, T_LM_HEAD, T_NORM_F, T_NORM1, T_NORM2) = range(5)


class _CModelConfig(C.Structure):
    _fields_ = [("arch", C.c_int), ("vocab_size", C.c_int), ("hidden_dim", C.c_int),
                ("num_layers", C.c_int), ("n_heads", C.c_int), ("n_kv_heads", C.c_int),
                ("intermediate_dim", C.c_int), ("inner_lr", C.c_float), ("rope_theta", C.c_double),
                ("max_position_embeddings", C.c_int), ("max_batch", C.c_int),
                ("tp_rank", C.c_int), ("tp_size", C.c_int)]


def _bind():
    L = lib()
    if getattr(L, "_model_bound", False):
        return L
    vp, i64, i32 = C.c_void_p, C.c_int64, C.c_int
    L.bt_ttt_update.argtypes = [vp, vp, i64, i64, i64, C.c_float, i64, vp, i32, vp]
    L.bt_kv_create.argtypes = [C.POINTER(vp), i64, i64, i64, i64, i32]
    L.bt_kv_reset.argtypes = [vp]
    L.bt_kv_destroy.argtypes = [vp]
    L.bt_kv_export.argtypes = [vp, i64, i64, vp, vp, vp, vp]
    L.bt_kv_import.argtypes = [vp, i64, i64, vp, vp, vp, vp]
    L.bt_kv_append.argtypes = [vp, vp, vp, vp, i64, vp]
    L.bt_attn_decode.argtypes = [vp, vp, vp, i64, i64, C.c_double, vp, vp]
    L.bt_linear_create_fused.argtypes = [C.POINTER(vp), C.POINTER(vp), C.POINTER(i64), vp, i32, i64, i32]
    L.bt_model_create.argtypes = [C.POINTER(vp), C.POINTER(_CModelConfig), i32]
    L.bt_model_set_linear.argtypes = [vp, i32, i32, vp, i64, i64, C.c_float]
    L.bt_model_set_linear_bases.argtypes = [vp, i32, i32, vp, i64, i64, i32, vp]
    L.bt_model_set_tensor.argtypes = [vp, i32, i32, vp, i64]
    L.bt_model_set_tensor_typed.argtypes = [vp, i32, i32, vp, i64, i32]
    L.bt_model_finalize.argtypes = [vp]
    L.bt_model_destroy.argtypes = [vp]
    L.bt_model_reset.argtypes = [vp]
    L.bt_model_forward_one.argtypes = [vp, vp, i32, vp, vp]
    L.bt_model_step_dev.argtypes = [vp, vp, i32, vp]
    L.bt_model_logits.restype = vp
    L.bt_model_logits.argtypes = [vp]
    L.bt_model_next.restype = vp
    L.bt_model_next.argtypes = [vp]
    L.bt_model_pos.argtypes = [vp]
    L.bt_model_ttt_state.restype = vp
    L.bt_model_ttt_state.argtypes = [vp, i32]
    L.bt_model_kv_cache.restype = vp
    L.bt_model_kv_cache.argtypes = [vp, i32]
    L.bt_model_trace_floats.restype = i64
    L.bt_model_trace_floats.argtypes = [vp, i32]
    L.bt_model_set_trace.argtypes = [vp, vp, i32]
    L.bt_model_prefill.argtypes = [vp, vp, i32, i32, i32, vp, vp]
    L.bt_model_ternary_bytes.restype = i64
    L.bt_model_ternary_bytes.argtypes = [vp]
    L.bt_tp_unique_id.argtypes = [vp]
    L.bt_model_tp_init.argtypes = [vp, vp]
    L.bt_model_seek.argtypes = [vp, i32]
    L.bt_model_tp_peer_export.argtypes = [vp, C.c_char_p]
    L.bt_model_tp_peer_import.argtypes = [vp, C.c_char_p]
    L.bt_model_tp_set_timeout.argtypes = [vp, i32]
    L.bt_model_tp_destroy.argtypes = [vp]
    L.bt_model_tp_resync.argtypes = [vp]
    L.bt_model_enqueue_products.argtypes = [vp, i32, i32, vp, C.POINTER(i32)]
    L.bt_model_launches_per_step.argtypes = [vp, i32]
    L._model_bound = True
    return L


def ttt_update(w_state, feats, inner_lr: float, chunk: int = 1):
    """TTTLayer inner update (layers/ttt.rs:52-68 / :88-113).  w_state: CUDA f32
    [batch, d, d], updated in place; feats: [batch, t_len, d] or [batch, d].  Returns z."""
    torch = _torch()
    L = _bind()
    f3 = feats if feats.dim() == 3 else feats.unsqueeze(1)
    f3 = f3.contiguous()
    batch, t_len, d = f3.shape
    z = torch.empty_like(f3)
    check(L.bt_ttt_update(_ptr(w_state), _ptr(f3), batch, t_len, d, inner_lr, chunk, _ptr(z),
                          w_state.device.index, _stream_ptr(w_state.device.index)))
    return z if feats.dim() == 3 else z.squeeze(1)


class QuantizedKVCache:
    """layers/kv_cache.rs:14-44, preallocated for `batch` sequences on the device."""

    def __init__(self, max_seq_len: int, batch: int, n_kv_heads: int, head_dim: int, device: int = 0,
                 _borrowed=None):
        self._L = _bind()
        self.batch, self.n_kv, self.head_dim, self.max_seq_len = batch, n_kv_heads, head_dim, max_seq_len
        self._owned = _borrowed is None
        if _borrowed is None:
            self._h = C.c_void_p()
            check(self._L.bt_kv_create(C.byref(self._h), batch, n_kv_heads, head_dim, max_seq_len, device))
        else:
            self._h = C.c_void_p(_borrowed)

    def reset(self):
        check(self._L.bt_kv_reset(self._h))

    def export(self, b: int, t_len: int):
        kq = np.zeros((self.n_kv, t_len, self.head_dim), np.uint8)
        vq = np.zeros_like(kq)
        ks = np.zeros((self.n_kv, t_len), np.float32)
        vs = np.zeros_like(ks)
        check(self._L.bt_kv_export(self._h, b, t_len, kq.ctypes.data, ks.ctypes.data, vq.ctypes.data,
                                   vs.ctypes.data))
        return kq, ks, vq, vs

    def export_rows(self, pos: int, batch: int):
        """The rows at position `pos` of sequences 0..batch-1: (kq [batch, n_kv, hd] u8, ks [batch, n_kv],
        vq, vs)."""
        parts = [self.export(b, pos + 1) for b in range(batch)]
        return tuple(np.stack([p[i][:, pos] for p in parts], 0) for i in range(4))

    def load(self, b: int, kq, ks, vq, vs):
        """Restores rows [0, t_len) of sequence b from arrays shaped like export()'s."""
        kq = np.ascontiguousarray(kq, np.uint8)
        vq = np.ascontiguousarray(vq, np.uint8)
        ks = np.ascontiguousarray(ks, np.float32)
        vs = np.ascontiguousarray(vs, np.float32)
        t_len = kq.shape[1]
        check(self._L.bt_kv_import(self._h, b, t_len, kq.ctypes.data, ks.ctypes.data, vq.ctypes.data, vs.ctypes.data))

    def append(self, k, v, pos):
        """QuantizedKVCache::append (layers/kv_cache.rs:50-92): k, v CUDA f32 [batch, n_kv, head_dim]
        (k already rotated), pos CUDA int32 [batch]."""
        k, v = k.contiguous(), v.contiguous()
        check(self._L.bt_kv_append(self._h, _ptr(k), _ptr(v), _ptr(pos), k.shape[0], _stream_ptr(k.device.index)))

    def __del__(self):
        try:
            if self._owned and getattr(self, "_h", None):
                self._L.bt_kv_destroy(self._h)
                self._h = None
        except Exception:
            pass


def attn_decode(cache: QuantizedKVCache, qkv, pos, n_heads: int, rope_theta: float = 10000.0):
    """Attention core of BitAttention::forward for one new token per sequence
    (layers/attention.rs:166-217): qkv CUDA f32 [batch, (n_heads+2 n_kv)*hd], pos CUDA int32
    [batch] -> [batch, n_heads*hd]."""
    torch = _torch()
    qkv = qkv.contiguous()
    batch = qkv.shape[0]
    out = torch.empty((batch, n_heads * cache.head_dim), dtype=torch.float32, device=qkv.device)
    check(cache._L.bt_attn_decode(cache._h, _ptr(qkv), _ptr(pos), batch, n_heads, rope_theta, _ptr(out),
                                  _stream_ptr(qkv.device.index)))
    return out


@dataclass
class BitLlamaConfig:
    """model/config.rs:20-59 (the fields the decode path reads)."""
    arch: str
    vocab_size: int
    hidden_dim: int
    num_layers: int
    n_heads: int
    n_kv_heads: int
    intermediate_dim: int
    inner_lr: float = 0.0
    rope_theta: float = 10000.0
    max_position_embeddings: int = 2048


class BitLlama:
    """model/llama.rs:37-272: load weights, forward_one, reset_kv_cache."""

    def __init__(self, cfg: BitLlamaConfig, max_batch: int = 1, device: int = 0, tp_rank: int = 0,
                 tp_size: int = 1):
        self._L = _bind()
        self.cfg, self.max_batch, self.device = cfg, max_batch, device
        self.tp_rank, self.tp_size = tp_rank, tp_size
        cc = _CModelConfig(ARCH_TTT if cfg.arch == "ttt" else ARCH_LLAMA, cfg.vocab_size, cfg.hidden_dim,
                           cfg.num_layers, cfg.n_heads, cfg.n_kv_heads, cfg.intermediate_dim, cfg.inner_lr,
                           cfg.rope_theta, cfg.max_position_embeddings, max_batch, tp_rank, tp_size)
        self._h = C.c_void_p()
        check(self._L.bt_model_create(C.byref(self._h), C.byref(cc), device))

    def set_linear(self, layer: int, kind: int, packed: np.ndarray, scale, n_out: int, k_in: int):
        """packed [n_out, k_in/4] with one scale, or [n_out, k_in/4, n_bases] with n_bases scales."""
        packed = np.ascontiguousarray(packed, np.uint8)
        scales = np.ascontiguousarray(np.atleast_1d(np.asarray(scale, np.float32)))
        n_bases = packed.shape[2] if packed.ndim == 3 else 1
        if scales.size != n_bases:
            raise ValueError(f"{scales.size} scales for {n_bases} bases")
        check(self._L.bt_model_set_linear_bases(self._h, layer, kind, packed.ctypes.data, n_out, k_in, n_bases,
                                                scales.ctypes.data))

    def set_tensor(self, kind: int, data: np.ndarray, layer: int = 0, f16: bool = False):
        """f16: keep the embedding / lm_head as IEEE halves on the device (a converted checkpoint's dtype)
        instead of bf16."""
        data = np.ascontiguousarray(data, np.float32)
        check(self._L.bt_model_set_tensor_typed(self._h, kind, layer, data.ctypes.data, data.size, 4 if f16 else 1))

    def finalize(self):
        check(self._L.bt_model_finalize(self._h))

    def tp_init(self, unique_id: bytes):
        """Joins the tensor-parallel communicator (collective); unique_id from tp_unique_id() of rank 0."""
        buf = (C.c_uint8 * 128).from_buffer_copy(unique_id)
        check(self._L.bt_model_tp_init(self._h, buf))

    def tp_peer_handle(self) -> bytes:
        """This rank's 64-byte CUDA IPC handle for the peer-memory exchange."""
        buf = C.create_string_buffer(64)
        check(self._L.bt_model_tp_peer_export(self._h, buf))
        return buf.raw

    def tp_peer_init(self, handles) -> None:
        """handles: the 64-byte handles of all ranks in rank order; switches the row-parallel
        projections from NCCL calls to this library's NVLink peer-memory kernels."""
        blob = b"".join(handles)
        if len(blob) != 64 * self.tp_size:
            raise ValueError("tp_peer_init expects one 64-byte handle per rank")
        check(self._L.bt_model_tp_peer_import(self._h, blob))

    def tp_set_timeout(self, milliseconds: int) -> None:
        """How long an exchange kernel waits for its peers before the step fails with BT_ERR_TIMEOUT."""
        check(self._L.bt_model_tp_set_timeout(self._h, milliseconds))

    def tp_resync(self) -> None:
        """After a timed-out exchange: every rank, with a host barrier before and after."""
        check(self._L.bt_model_tp_resync(self._h))

    def tp_destroy(self) -> None:
        check(self._L.bt_model_tp_destroy(self._h))

    def tp_peer_disable(self) -> None:
        """Back to the NCCL exchange (every rank must call it)."""
        check(self._L.bt_model_tp_peer_import(self._h, None))

    def reset_kv_cache(self):
        check(self._L.bt_model_reset(self._h))

    def seek(self, pos: int):
        """Continue from position `pos` with the caches as they are in device memory."""
        check(self._L.bt_model_seek(self._h, pos))

    @property
    def current_pos(self) -> int:
        return self._L.bt_model_pos(self._h)

    @property
    def ternary_bytes(self) -> int:
        return self._L.bt_model_ternary_bytes(self._h)

    def forward_one(self, tokens, want_logits: bool = True):
        """tokens: host ints [batch].  Returns (logits np [batch, vocab] or None, next ids)."""
        tokens = np.ascontiguousarray(tokens, np.int32).reshape(-1)
        b = tokens.size
        logits = np.empty((b, self.cfg.vocab_size), np.float32) if want_logits else None
        nxt = np.empty(b, np.int32)
        check(self._L.bt_model_forward_one(self._h, tokens.ctypes.data, b,
                                           logits.ctypes.data if want_logits else None, nxt.ctypes.data))
        return logits, nxt

    def prefill(self, tokens, ttt_chunk: int = 1, want_logits: bool = True):
        """tokens: host ints [batch, n_tokens].  Batched prefill, equivalent to n_tokens forward_one calls
        (model/llama.rs:495-498); returns (logits of the last token np [batch, vocab] or None, next ids)."""
        tokens = np.ascontiguousarray(tokens, np.int32)
        if tokens.ndim == 1:
            tokens = tokens[None, :]
        b, n = tokens.shape
        logits = np.empty((b, self.cfg.vocab_size), np.float32) if want_logits else None
        nxt = np.empty(b, np.int32)
        check(self._L.bt_model_prefill(self._h, tokens.ctypes.data, b, n, ttt_chunk,
                                       logits.ctypes.data if want_logits else None, nxt.ctypes.data))
        return logits, nxt

    def step_dev(self, tokens_dev):
        """Device-resident step on torch's current stream; results stay on the device."""
        check(self._L.bt_model_step_dev(self._h, _ptr(tokens_dev), tokens_dev.numel(),
                                        _stream_ptr(tokens_dev.device.index)))

    def set_trace(self, on: bool = True, rows: int = 0) -> None:
        """Keep the per-layer intermediate tensors of the following steps (see read_trace).
        rows: rows per tensor (default max_batch; a prefill needs sequences x tokens)."""
        torch = _torch()
        if on:
            self._trace_rows = max(rows, self.max_batch)
            n = self._L.bt_model_trace_floats(self._h, self._trace_rows)
            self._trace = torch.zeros(n, dtype=torch.float32, device=f"cuda:{self.device}")
            check(self._L.bt_model_set_trace(self._h, _ptr(self._trace), self._trace_rows))
        else:
            check(self._L.bt_model_set_trace(self._h, None, 0))  # the buffer stays readable (read_trace)

    def read_trace(self, batch: int):
        """The last traced step: a list over layers of dicts h_in, qkv, att, h_mid, act, h_out
        (numpy [batch, width]; arch ttt: qkv = down-projected features, att = TTT prediction)."""
        torch = _torch()
        torch.cuda.synchronize(self.device)
        c, tp = self.cfg, max(self.tp_size, 1)
        H, B = c.hidden_dim, self._trace_rows
        if c.arch == "ttt":
            wq = wa = H // 4
        else:
            hd = H // c.n_heads
            wq, wa = (c.n_heads // tp + 2 * (c.n_kv_heads // tp)) * hd, (c.n_heads // tp) * hd
        widths = [("h_in", H), ("qkv", wq), ("att", wa), ("h_mid", H), ("act", c.intermediate_dim // tp), ("h_out", H)]
        flat = self._trace.cpu().numpy()
        per_layer = sum(w for _, w in widths) * B
        out = []
        for li in range(c.num_layers):
            off, d = li * per_layer, {}
            for name, w in widths:
                d[name] = flat[off:off + B * w].reshape(B, w)[:batch].copy()
                off += B * w
            out.append(d)
        return out

    def enqueue_products(self, batch: int, as_in_step: bool = False) -> int:
        """Measurement aid: only the ternary-product launches of one step (state untouched);
        as_in_step: with the quantiser prologues and fused epilogues the step itself uses."""
        n = C.c_int(0)
        check(self._L.bt_model_enqueue_products(self._h, batch, int(as_in_step), _stream_ptr(self.device), C.byref(n)))
        return n.value

    def launches_per_step(self, batch: int) -> int:
        return self._L.bt_model_launches_per_step(self._h, batch)

    def next_dev(self):
        torch = _torch()
        return _wrap_dev(self._L.bt_model_next(self._h), (self.max_batch,), torch.int32, self.device)

    def logits_dev(self):
        torch = _torch()
        return _wrap_dev(self._L.bt_model_logits(self._h), (self.max_batch, self.cfg.vocab_size),
                         torch.float32, self.device)

    def ttt_state(self, layer: int):
        torch = _torch()
        d = self.cfg.hidden_dim // 4
        p = self._L.bt_model_ttt_state(self._h, layer)
        return None if not p else _wrap_dev(p, (self.max_batch, d, d), torch.float32, self.device)

    def save_memory(self, path: str) -> None:
        """TTT fast-weight states to a safetensors file, tensors `layer_{i}` (Llama::save_memory,
        model/llama.rs:575-591): `[d, d]` for a single-sequence model, `[batch, d, d]` otherwise.
        Attention blocks (which the reference's file does not cover) add their Q8 cache rows up to the
        current position as `kv_{i}.k_q / k_s / v_q / v_s` (`[batch, n_kv, T, hd]` u8, `[batch, n_kv, T]` f32)
        and the position as `kv_position`, so that a conversation can be resumed without a second prefill."""
        from .loader import write_safetensors
        torch = _torch()
        torch.cuda.synchronize(self.device)
        tensors = {}
        t_len = self.current_pos
        for li in range(self.cfg.num_layers):
            st = self.ttt_state(li)
            if st is not None:
                a = st.cpu().numpy()
                tensors[f"layer_{li}"] = a[0] if self.max_batch == 1 else a
            kv = self.kv_cache(li)
            if kv is not None and t_len > 0:
                rows = [kv.export(b, t_len) for b in range(self.max_batch)]
                for j, name in enumerate(("k_q", "k_s", "v_q", "v_s")):
                    tensors[f"kv_{li}.{name}"] = np.stack([r[j] for r in rows])
        if any(k.startswith("kv_") for k in tensors):
            tensors["kv_position"] = np.array([t_len], np.int32)
        write_safetensors(path, tensors)

    def load_memory(self, path: str) -> None:
        """Restores the states written by `save_memory`; layers missing from the file keep their
        state (Llama::load_memory, model/llama.rs:593-611).  A `[d, d]` tensor goes to every
        sequence of the batch."""
        from .loader import CheckpointError, read_safetensors
        torch = _torch()
        tensors = read_safetensors(path)
        d = self.cfg.hidden_dim // 4
        torch.cuda.synchronize(self.device)
        for li in range(self.cfg.num_layers):
            st = self.ttt_state(li)
            a = tensors.get(f"layer_{li}")
            if st is None or a is None:
                continue
            a = np.array(a, dtype=np.float32)  # a writable copy (the file is memory-mapped read-only)
            if a.shape == (d, d):
                a = np.broadcast_to(a, (self.max_batch, d, d))
            if a.shape != (self.max_batch, d, d):
                raise CheckpointError(f"{path}: layer_{li} has shape {a.shape}, expected {(d, d)} or {(self.max_batch, d, d)}")
            st.copy_(torch.from_numpy(np.array(a, dtype=np.float32)).to(st.device))
        if "kv_position" in tensors:
            t_len = int(np.array(tensors["kv_position"]).reshape(-1)[0])
            c = self.cfg
            n_kv, hd = c.n_kv_heads // max(self.tp_size, 1), c.hidden_dim // c.n_heads
            if not 0 < t_len <= c.max_position_embeddings:
                raise CheckpointError(f"{path}: kv_position {t_len} outside 1..{c.max_position_embeddings}")
            for li in range(c.num_layers):
                kv = self.kv_cache(li)
                if kv is None or f"kv_{li}.k_q" not in tensors:
                    continue
                parts = [np.array(tensors[f"kv_{li}.{name}"]) for name in ("k_q", "k_s", "v_q", "v_s")]
                if parts[0].shape != (self.max_batch, n_kv, t_len, hd) or parts[1].shape != (self.max_batch, n_kv, t_len):
                    raise CheckpointError(f"{path}: kv_{li} has shape {parts[0].shape}, expected {(self.max_batch, n_kv, t_len, hd)}")
                for b in range(self.max_batch):
                    kv.load(b, parts[0][b], parts[1][b], parts[2][b], parts[3][b])
            self.seek(t_len)
        torch.cuda.synchronize(self.device)

    def kv_cache(self, layer: int):
        p = self._L.bt_model_kv_cache(self._h, layer)
        if not p:
            return None
        c = self.cfg
        return QuantizedKVCache(c.max_position_embeddings, self.max_batch, c.n_kv_heads // max(self.tp_size, 1),
                                c.hidden_dim // c.n_heads, self.device, _borrowed=p)

    def __del__(self):
        try:
            if getattr(self, "_h", None):
                self._L.bt_model_destroy(self._h)
                self._h = None
        except Exception:
            pass


def tp_unique_id() -> bytes:
    """128-byte communicator id; create on rank 0 and send to the other ranks by any means."""
    buf = (C.c_uint8 * 128)()
    check(_bind().bt_tp_unique_id(buf))
    return bytes(buf)


def _wrap_dev(ptr: int, shape, dtype, device: int):
    """Zero-copy torch view of a device buffer owned by the library."""
    torch = _torch()
    n = int(np.prod(shape))
    itemsize = torch.empty((), dtype=dtype).element_size()

    class _Holder:
        pass
    h = _Holder()
    h.__cuda_array_interface__ = {
        "shape": (n * itemsize,), "typestr": "|u1", "data": (int(ptr), False), "version": 2,
    }
    return torch.as_tensor(h, device=f"cuda:{device}").view(dtype).reshape(shape)
