"""Python face of the CPU oracle.  TEST INFRASTRUCTURE, NOT PRODUCT CODE.

Two things live here:

* ``lib()`` - a ctypes handle on ``oracle/_build/libbitttt_oracle.so`` (the C restatement
  of the reference's CPU arithmetic, built by ``oracle/Makefile``) plus thin numpy
  wrappers around its entry points;
* a numpy/pure-Python twin of the small integer functions (``np_*``), used to cross-check
  the C code on small cases, and the model-level composition (block / one decode step)
  that strings the C functions together in the reference's order.

Parity pin status is stated in the header of ``bitttt_oracle.c``: packing is pinned by
the reference's known-answer tests and converter-generated fixtures; the ternary product
(``bitlinear_f32`` / ``bitlinear_i32``, and the multi-basis sum) is pinned against the
reference's own two CUDA kernels, compiled unchanged into ``oracle/_ref/libref_kernels.so``
(``ref_lib()``; they need a GPU to run, so that check lives in the GPU tests); every other
function is "parity unpinned" (no reference value test exists, and the reference's Rust
host code cannot be compiled in this environment).

Only tests, the smoke check and the benchmark's CPU-baseline leg may import this module.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess
from dataclasses import dataclass, field

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_SO = os.path.join(_HERE, "_build", "libbitttt_oracle.so")
_REF_SO = os.path.join(_HERE, "_ref", "libref_kernels.so")
_LIB = None
_REF_LIB = None

_f32p = np.ctypeslib.ndpointer(np.float32, flags="C_CONTIGUOUS")
_u8p = np.ctypeslib.ndpointer(np.uint8, flags="C_CONTIGUOUS")
_i8p = np.ctypeslib.ndpointer(np.int8, flags="C_CONTIGUOUS")
_i32p = np.ctypeslib.ndpointer(np.int32, flags="C_CONTIGUOUS")
_i64 = C.c_int64


def build(force: bool = False) -> str:
    """Compile the C oracle if the shared object is missing (or ``force``)."""
    src = os.path.join(_HERE, "bitttt_oracle.c")
    stale = (not os.path.exists(_SO)) or os.path.getmtime(_SO) < os.path.getmtime(src)
    if force or stale:
        subprocess.run(["make", "-C", _HERE, "-B"], check=True, capture_output=True)
    return _SO


def build_ref(reference_dir: str) -> str:
    """Compile the reference's own CUDA kernels (kernels/bit_op.cu, kernels/adaptive_bit_op.cu)
    from `reference_dir`, where they lie, into oracle/_ref/libref_kernels.so."""
    subprocess.run(["make", "-C", _HERE, "ref", f"REFERENCE={reference_dir}"], check=True, capture_output=True)
    return _REF_SO


def ref_lib():
    """ctypes handle on the reference-built kernels, or None when they were not built."""
    global _REF_LIB
    if _REF_LIB is None and os.path.exists(_REF_SO):
        L = C.CDLL(_REF_SO)
        L.ref_bit_linear_forward.argtypes = [_f32p, _u8p, _f32p, C.c_float, C.c_int, C.c_int, C.c_int]
        L.ref_adaptive_gemm_n3.argtypes = [_f32p, _i8p, _f32p, _f32p, C.c_int, C.c_int, C.c_int]
        _REF_LIB = L
    return _REF_LIB


def ref_bit_linear_forward(x, packed, n, scale):
    """The reference's bit_linear_forward kernel (kernels/bit_op.cu:4-45) run on the current
    CUDA device: x f32 [M, K], packed L1 bytes [N, K/4] -> y f32 [M, N]."""
    x = _f32(x)
    m, k = x.shape
    y = np.zeros((m, n), dtype=np.float32)
    rc = ref_lib().ref_bit_linear_forward(x, np.ascontiguousarray(packed, np.uint8).reshape(-1), y, scale, m, k, n)
    if rc != 0:
        raise RuntimeError(f"reference kernel launch failed: cudaError {rc}")
    return y


def pack_l3(bases):
    """pack_interleaved_blocks of tools/conversion/convert_adaptive.py:43-83: bases int8
    [B, N, K] with values -1/0/+1 -> bytes [N, K/4, B, 4] (one byte per weight)."""
    bases = np.ascontiguousarray(bases, np.int8)
    b, n, k = bases.shape
    return np.ascontiguousarray(bases.reshape(b, n, k // 4, 4).transpose(1, 2, 0, 3))


def ref_adaptive_gemm_n3(x, packed_l3, scales):
    """The reference's adaptive_gemm_n3_kernel_f32 (kernels/adaptive_bit_op.cu:74-161) run on the
    current CUDA device: x f32 [M, K], packed_l3 int8 [N, K/4, 3, 4], 3 scales -> y f32 [M, N]."""
    x = _f32(x)
    m, k = x.shape
    w = np.ascontiguousarray(packed_l3).view(np.int8)
    n = w.shape[0]
    assert w.shape == (n, k // 4, 3, 4)
    y = np.zeros((m, n), dtype=np.float32)
    rc = ref_lib().ref_adaptive_gemm_n3(x, w.reshape(-1), _f32(scales), y, m, k, n)
    if rc != 0:
        raise RuntimeError(f"reference kernel launch failed: cudaError {rc}")
    return y


def lib():
    global _LIB
    if _LIB is not None:
        return _LIB
    if not os.path.exists(_SO):
        build()
    L = C.CDLL(_SO)
    L.oracle_pack_l1.restype = C.c_float
    L.oracle_pack_l1.argtypes = [_f32p, _i64, _u8p]
    L.oracle_unpack_l1.argtypes = [_u8p, _i64, C.c_float, _f32p]
    L.oracle_pack_l2.argtypes = [_i8p, C.c_int, _i64, _i64, _u8p]
    L.oracle_decode_l2.argtypes = [_u8p, _f32p, C.c_int, _i64, _i64, _f32p]
    L.oracle_bitlinear_f32.argtypes = [_f32p, _i64, _i64, _u8p, _i64, C.c_float, _f32p, C.c_int]
    L.oracle_bitlinear_i32.argtypes = [_i8p, _i64, _i64, _u8p, _i64, _i32p, C.c_int]
    L.oracle_act_quant.argtypes = [_f32p, _i64, _i64, _i8p, _f32p, _i32p]
    L.oracle_bitlinear_q.argtypes = [_f32p, _i64, _i64, _u8p, C.c_int, _f32p, _i64, _f32p, C.c_int]
    L.oracle_rmsnorm.argtypes = [_f32p, _i64, _i64, _f32p, C.c_float, _f32p]
    L.oracle_silu_mul.argtypes = [_f32p, _f32p, _i64, _f32p]
    L.oracle_ttt_step.argtypes = [_f32p, _f32p, _i64, C.c_float, _f32p]
    L.oracle_ttt_chunk.argtypes = [_f32p, _f32p, _i64, _i64, C.c_float, _i64, _f32p]
    L.oracle_kv_quant.argtypes = [_f32p, _i64, _i64, _u8p, _f32p]
    L.oracle_kv_dequant.argtypes = [_u8p, _f32p, _i64, _i64, _f32p]
    L.oracle_rope.argtypes = [_f32p, _i64, _i64, _i64, C.c_double]
    L.oracle_attn_decode.argtypes = [_f32p, _f32p, _f32p, _i64, _i64, _i64, _i64, _f32p]
    L.oracle_dense_linear.argtypes = [_f32p, _i64, _i64, _f32p, _i64, _f32p, C.c_int]
    L.oracle_has_avx2.restype = C.c_int
    L.oracle_num_threads.restype = C.c_int
    _LIB = L
    return L


def _f32(a):
    return np.ascontiguousarray(a, dtype=np.float32)


# ----------------------------------------------------------------------------------------
# numpy wrappers around the C oracle
# ----------------------------------------------------------------------------------------

def pack_l1(w):
    """PackedTensor::pack (kernels/packing.rs:50-105) -> (bytes, scale)."""
    w = _f32(w).reshape(-1)
    out = np.zeros((w.size + 3) // 4, dtype=np.uint8)
    scale = lib().oracle_pack_l1(w, w.size, out)
    return out, float(scale)


def unpack_l1(packed, n_elem, scale):
    """PackedTensor::unpack (kernels/packing.rs:108-133)."""
    out = np.zeros(n_elem, dtype=np.float32)
    lib().oracle_unpack_l1(np.ascontiguousarray(packed, np.uint8), n_elem, scale, out)
    return out


def pack_l2(bases):
    """pack_2bit of tools/conversion/convert_llama_v2.py:111-151; bases int8 [B,N,K]."""
    bases = np.ascontiguousarray(bases, np.int8)
    b, n, k = bases.shape
    out = np.zeros((n, k // 4, b), dtype=np.uint8)
    lib().oracle_pack_l2(bases, b, n, k, out)
    return out


def decode_l2(packed, scales):
    """AdaptiveBitLinear::load reconstruction (layers/adaptive_linear.rs:86-109)."""
    packed = np.ascontiguousarray(packed, np.uint8)
    n, kq, b = packed.shape
    out = np.zeros((n, kq * 4), dtype=np.float32)
    lib().oracle_decode_l2(packed, _f32(scales), b, n, kq * 4, out)
    return out


def bitlinear_f32(x, packed, n, scale, threads=0):
    """BitLinearCpu::forward (kernels/cpu.rs:17-127) on f32 activations."""
    x = _f32(x)
    m, k = x.shape
    y = np.zeros((m, n), dtype=np.float32)
    lib().oracle_bitlinear_f32(x, m, k, np.ascontiguousarray(packed, np.uint8).reshape(-1), n,
                               scale, y, threads)
    return y


def bitlinear_i32(q, packed, n, threads=0):
    q = np.ascontiguousarray(q, np.int8)
    m, k = q.shape
    acc = np.zeros((m, n), dtype=np.int32)
    lib().oracle_bitlinear_i32(q, m, k, np.ascontiguousarray(packed, np.uint8).reshape(-1), n,
                               acc, threads)
    return acc


def act_quant(x):
    """Per-token absmax int8 quantiser -> (q int8 [M,K], scale f32 [M], sum_k q int32 [M])."""
    x = _f32(x)
    m, k = x.shape
    q = np.zeros((m, k), dtype=np.int8)
    s = np.zeros(m, dtype=np.float32)
    qs = np.zeros(m, dtype=np.int32)
    lib().oracle_act_quant(x, m, k, q, s, qs)
    return q, s, qs


def bitlinear_q(x, packed, scales, n, n_bases=1, threads=0):
    """act_quant -> ternary product -> scales.  packed: L1 bytes (n_bases=1) or L2
    [N,K/4,B] bytes."""
    x = _f32(x)
    m, k = x.shape
    y = np.zeros((m, n), dtype=np.float32)
    sc = _f32(np.atleast_1d(scales))
    lib().oracle_bitlinear_q(x, m, k, np.ascontiguousarray(packed, np.uint8).reshape(-1),
                             n_bases, sc, n, y, threads)
    return y


def rmsnorm(x, w, eps=1e-5):
    x = _f32(x)
    m, h = x.shape
    y = np.zeros_like(x)
    lib().oracle_rmsnorm(x, m, h, _f32(w), eps, y)
    return y


def silu_mul(g, u):
    g = _f32(g)
    out = np.zeros_like(g)
    lib().oracle_silu_mul(g, _f32(u), g.size, out)
    return out


def ttt_step(w, feat, lr):
    """In-place update of w (d x d); returns z (prediction with the old w)."""
    d = feat.shape[-1]
    z = np.zeros(d, dtype=np.float32)
    lib().oracle_ttt_step(w, _f32(feat), d, lr, z)
    return z


def ttt_chunk(w, feats, lr, chunk):
    feats = _f32(feats)
    t, d = feats.shape
    z = np.zeros((t, d), dtype=np.float32)
    lib().oracle_ttt_chunk(w, feats, t, d, lr, chunk, z)
    return z


def kv_quant(x):
    x = _f32(x)
    rows, hd = x.shape
    q = np.zeros((rows, hd), dtype=np.uint8)
    s = np.zeros(rows, dtype=np.float32)
    lib().oracle_kv_quant(x, rows, hd, q, s)
    return q, s


def kv_dequant(q, s):
    q = np.ascontiguousarray(q, np.uint8)
    rows, hd = q.shape
    out = np.zeros((rows, hd), dtype=np.float32)
    lib().oracle_kv_dequant(q, _f32(s), rows, hd, out)
    return out


def rope(x, pos, theta):
    """Half-split rotation of every row of x [rows, hd] at position pos (copy)."""
    x = _f32(x).copy()
    rows, hd = x.shape
    lib().oracle_rope(x, rows, hd, pos, float(theta))
    return x


def attn_decode(q, k, v):
    """q [n_heads, hd]; k, v [n_kv, T, hd] dequantised -> out [n_heads, hd]."""
    q, k, v = _f32(q), _f32(k), _f32(v)
    nh, hd = q.shape
    nkv, t, _ = k.shape
    out = np.zeros((nh, hd), dtype=np.float32)
    lib().oracle_attn_decode(q, k, v, nh, nkv, t, hd, out)
    return out


def dense_linear(x, w, threads=0):
    x, w = _f32(x), _f32(w)
    m, k = x.shape
    n = w.shape[0]
    y = np.zeros((m, n), dtype=np.float32)
    lib().oracle_dense_linear(x, m, k, w, n, y, threads)
    return y


# ----------------------------------------------------------------------------------------
# numpy twin of the integer functions (independent of the C code; small cases only)
# ----------------------------------------------------------------------------------------

_TERNARY = np.array([0, 1, -1, 0], dtype=np.int32)  # code table, kernels/packing.rs:9-13


def np_unpack_codes(packed_rows, k):
    """[N, ceil(K/4)] bytes -> [N, K] ternary ints (kernels/cpu.rs:110-120)."""
    p = np.asarray(packed_rows, np.uint8)
    codes = np.stack([(p >> (2 * r)) & 3 for r in range(4)], axis=-1).reshape(p.shape[0], -1)
    return _TERNARY[codes[:, :k]]


def np_pack_l1(w):
    w = np.asarray(w, np.float32).reshape(-1)
    scale = np.float32(np.float32(np.abs(w.astype(np.float64)).mean()) + np.float32(1e-6))
    ratio = (w / scale).astype(np.float32)
    q = np.clip(np.sign(ratio) * np.floor(np.abs(ratio) + np.float32(0.5)), -1, 1)
    code = np.where(q > 0.5, 1, np.where(q < -0.5, 2, 0)).astype(np.uint8)
    pad = (-code.size) % 4
    code = np.concatenate([code, np.zeros(pad, np.uint8)]).reshape(-1, 4)
    return (code[:, 0] | (code[:, 1] << 2) | (code[:, 2] << 4) | (code[:, 3] << 6)).astype(np.uint8), float(scale)


def np_act_quant(x):
    x = np.asarray(x, np.float32)
    amax = np.abs(x).max(axis=1).astype(np.float32)
    s = (amax / np.float32(127.0)).astype(np.float32)
    inv = np.where(amax > 0, np.float32(127.0) / np.where(amax > 0, amax, np.float32(1.0)), 0).astype(np.float32)
    ratio = (x * inv[:, None]).astype(np.float32)
    q = np.sign(ratio) * np.floor(np.abs(ratio) + np.float32(0.5))
    q = np.where(amax[:, None] > 0, np.clip(q, -127, 127), 0).astype(np.int8)
    return q, s


def np_bitlinear_i32(q, packed_rows, k):
    t = np_unpack_codes(packed_rows, k)
    return q.astype(np.int32) @ t.T.astype(np.int32)


# ----------------------------------------------------------------------------------------
# Model-level composition (block / decode step), reference order of operations
# ----------------------------------------------------------------------------------------

@dataclass
class Linear:
    """A packed BitLinear: L1 bytes [N, K/4] (n_bases 1) or L2 bytes [N, K/4, B]."""
    packed: np.ndarray
    scales: np.ndarray
    n: int
    k: int
    # False: the reference's own arithmetic, f32 activations straight into
    # BitLinearCpu::forward (kernels/cpu.rs:17-127), no int8 stage (single basis only)
    quantised: bool = True

    @property
    def n_bases(self):
        return 1 if self.packed.ndim == 2 else self.packed.shape[2]

    def __call__(self, x):
        if not self.quantised:
            return bitlinear_f32(x, self.packed, self.n, float(self.scales[0]))
        return bitlinear_q(x, self.packed, self.scales, self.n, self.n_bases)


@dataclass
class ModelConfig:
    arch: str
    vocab_size: int
    hidden_dim: int
    num_layers: int
    n_heads: int
    n_kv_heads: int
    intermediate_dim: int
    inner_lr: float = 0.01
    rope_theta: float = 10000.0
    rms_eps: float = 1e-5  # model/block.rs:10, model/llama.rs:13

    @property
    def head_dim(self):
        return self.hidden_dim // self.n_heads

    @property
    def d_small(self):
        return self.hidden_dim // 4  # layers/ttt.rs:29


@dataclass
class Layer:
    norm1: np.ndarray
    norm2: np.ndarray
    gate: Linear
    up: Linear
    down: Linear
    # arch == "ttt"
    ttt_down: Linear | None = None
    ttt_up: Linear | None = None
    # arch == "llama"
    q: Linear | None = None
    k: Linear | None = None
    v: Linear | None = None
    o: Linear | None = None


@dataclass
class SeqState:
    """Per-sequence state: TTT fast weights and the Q8 KV cache, per layer."""
    w: list = field(default_factory=list)          # [d_small, d_small] f32 per layer
    kq: list = field(default_factory=list)         # per layer: list over tokens of u8 [n_kv, hd]
    ks: list = field(default_factory=list)
    vq: list = field(default_factory=list)
    vs: list = field(default_factory=list)
    pos: int = 0


@dataclass
class Model:
    cfg: ModelConfig
    embed: np.ndarray     # [V, H] f32
    layers: list
    norm_f: np.ndarray    # [H]
    lm_head: np.ndarray   # [V, H] f32 (dense, model/llama.rs:23)

    def new_state(self):
        c = self.cfg
        st = SeqState()
        for _ in range(c.num_layers):
            st.w.append(np.zeros((c.d_small, c.d_small), np.float32))
            st.kq.append([]); st.ks.append([]); st.vq.append([]); st.vs.append([])
        return st

    def block(self, li, h, st):
        """BitLlamaBlock::forward (model/block.rs:87-134) for one token, h: [1, H]."""
        c, L = self.cfg, self.layers[li]
        xn = rmsnorm(h, L.norm1, c.rms_eps)
        if c.arch == "ttt":
            # TTTLayer::forward_update (layers/ttt.rs:48-74)
            feat = L.ttt_down(xn)
            z = ttt_step(st.w[li], feat[0], c.inner_lr)
            mixed = L.ttt_up(z[None, :])
        else:
            # BitAttention::forward (layers/attention.rs:149-225) with seq_len 1
            hd, nh, nkv = c.head_dim, c.n_heads, c.n_kv_heads
            q = L.q(xn).reshape(nh, hd)
            k = L.k(xn).reshape(nkv, hd)
            v = L.v(xn).reshape(nkv, hd)
            q = rope(q, st.pos, c.rope_theta)
            k = rope(k, st.pos, c.rope_theta)
            kq, ks = kv_quant(k)     # QuantizedKVCache::append (layers/kv_cache.rs:50-92)
            vq, vs = kv_quant(v)
            st.kq[li].append(kq); st.ks[li].append(ks)
            st.vq[li].append(vq); st.vs[li].append(vs)
            t = len(st.kq[li])
            kall = np.stack(st.kq[li], axis=1)            # [n_kv, T, hd]
            vall = np.stack(st.vq[li], axis=1)
            ksc = np.stack(st.ks[li], axis=1).reshape(-1)  # [n_kv*T]
            vsc = np.stack(st.vs[li], axis=1).reshape(-1)
            kd = kv_dequant(kall.reshape(nkv * t, hd), ksc).reshape(nkv, t, hd)
            vd = kv_dequant(vall.reshape(nkv * t, hd), vsc).reshape(nkv, t, hd)
            att = attn_decode(q, kd, vd).reshape(1, nh * hd)
            mixed = L.o(att)
        h = h + mixed
        xn2 = rmsnorm(h, L.norm2, c.rms_eps)
        # SwiGLU::forward (layers/swiglu.rs:29-35)
        act = silu_mul(L.gate(xn2), L.up(xn2))
        return h + L.down(act)

    def forward_one(self, token, st):
        """BitLlama::forward_one (model/llama.rs:201-272): logits [V] for one token."""
        h = self.embed[token][None, :].astype(np.float32)
        for li in range(self.cfg.num_layers):
            h = self.block(li, h, st)
        hn = rmsnorm(h, self.norm_f, self.cfg.rms_eps)
        logits = dense_linear(hn, self.lm_head)[0]
        st.pos += 1
        return logits


def model_from_weights(w, quantised: bool = True) -> Model:
    """Builds the oracle model from the synthetic checkpoint structure that the GPU model
    is built from (fields: cfg, embed, lm_head, norm_f, layers[kind -> (packed, scale, n, k)]).
    Weight-kind indices follow bt_weight_kind in include/bitttt.h."""
    (W_Q, W_K, W_V, W_O, W_GATE, W_UP, W_DOWN, W_TTT_DOWN, W_TTT_UP) = range(9)
    c = w.cfg
    cfg = ModelConfig(c.arch, c.vocab_size, c.hidden_dim, c.num_layers, c.n_heads, c.n_kv_heads,
                      c.intermediate_dim, c.inner_lr, c.rope_theta)

    def lin(layer, kind):
        if kind not in layer:
            return None
        packed, scale, n, k = layer[kind]
        packed = np.ascontiguousarray(packed)
        if packed.ndim == 3:  # converted layout, several bases
            return Linear(packed, np.asarray(scale, np.float32).reshape(-1), n, k, quantised)
        return Linear(packed.reshape(n, k // 4), np.array([scale], np.float32), n, k, quantised)

    layers = []
    for layer in w.layers:
        layers.append(Layer(layer["norm1"], layer["norm2"], lin(layer, W_GATE), lin(layer, W_UP),
                            lin(layer, W_DOWN), lin(layer, W_TTT_DOWN), lin(layer, W_TTT_UP),
                            lin(layer, W_Q), lin(layer, W_K), lin(layer, W_V), lin(layer, W_O)))
    return Model(cfg, w.embed, layers, w.norm_f, w.lm_head)
