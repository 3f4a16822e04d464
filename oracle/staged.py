"""Stage-by-stage comparison of one GPU decode step with the CPU oracle.  TEST INFRASTRUCTURE,
NOT PRODUCT CODE: used by the GPU tests and by the benchmark's self-check before it times anything."""
from __future__ import annotations

import numpy as np


def rel_err(a, b):
    return float(np.abs(a - b).max() / max(np.abs(b).max(), 1e-30))


ATT_TOL = 2e-5      # attention output vs the oracle on identical inputs (f32 accumulation on the GPU)
LOGIT_TOL = 2e-5    # dense head vs the oracle on identical hidden states
ACT_TOL = 1e-6      # silu(gate)*up: the GPU's f32 exponential against the oracle's correctly rounded one
TTT_TOL = 2e-5      # TTT prediction z on identical features and (separately advanced) state: f32 accumulation on the GPU


def staged_decode_step(oracle, ref, gpu, cfg, tokens, states, act_tol=ACT_TOL, seqs=None):
    """One decode step of a model (arch llama or ttt) checked stage by stage.

    A decode step is a chain of int8 quantisers.  A quantiser turns an input difference of a millionth
    of its step into a different rounding of a few elements, the next quantiser sees those as a much
    larger input difference, and after three or four of them two runs that started one f32 rounding
    apart are as far apart as independent quantisation noise (about 1e-2 of the logits), at any model
    width.  Comparing logits of two free-running pipelines therefore tests luck, not kernels.  Instead
    every stage of the GPU step is compared with the oracle evaluated on the GPU's own input to that
    stage (from the model's per-layer trace): the BitLinear stages bit for bit, attention and the
    dense head to f32 accumulation accuracy.  The oracle's KV state is kept identical to the GPU cache.

    The step runs twice from the same position - once on the normal path (CUDA graph from the third
    call on), once traced - and both must give the same bits.  `seqs`: the sequences to check (default:
    all; the states of the others are not advanced).  Returns (logits, next ids)."""
    tokens = np.ascontiguousarray(tokens, np.int32).reshape(-1)
    batch = tokens.size
    pos = gpu.current_pos
    is_ttt = cfg.arch == "ttt"
    saved = [gpu.ttt_state(li).clone() for li in range(cfg.num_layers)] if is_ttt else None
    logits, nxt = gpu.forward_one(tokens)
    gpu.seek(pos)
    if is_ttt:  # the fast-weight states as they were before the step
        for li in range(cfg.num_layers):
            gpu.ttt_state(li).copy_(saved[li])
    gpu.set_trace(True)
    logits_t, nxt_t = gpu.forward_one(tokens)
    gpu.set_trace(False)
    assert np.array_equal(logits, logits_t) and np.array_equal(nxt, nxt_t), "traced and normal step differ"
    tr = gpu.read_trace(batch)
    hd, nh, nkv = cfg.hidden_dim // cfg.n_heads, cfg.n_heads, cfg.n_kv_heads
    new_rows = None if is_ttt else [gpu.kv_cache(li).export_rows(pos, batch) for li in range(cfg.num_layers)]
    for b in (range(batch) if seqs is None else seqs):
        st = states[b]
        assert st.pos == pos
        for li in range(cfg.num_layers):
            L, t = ref.layers[li], tr[li]
            h_in = t["h_in"][b:b + 1]
            if li == 0:
                assert np.array_equal(h_in[0], ref.embed[int(tokens[b])]), "embedding row"
            else:
                assert np.array_equal(h_in, tr[li - 1]["h_out"][b:b + 1])
            xn = oracle.rmsnorm(h_in, L.norm1, ref.cfg.rms_eps)
            if is_ttt:
                # TTTLayer::forward_update (layers/ttt.rs:48-74): features, prediction with the old state, residual
                feat_ref = L.ttt_down(xn)
                assert np.array_equal(t["qkv"][b:b + 1], feat_ref), ("ttt down projection", li, b)
                z_ref = oracle.ttt_step(st.w[li], t["qkv"][b], ref.cfg.inner_lr)  # advances the oracle's state
                assert rel_err(t["att"][b], z_ref) <= TTT_TOL, ("ttt prediction", li, b, rel_err(t["att"][b], z_ref))
                h_mid_ref = h_in + L.ttt_up(t["att"][b:b + 1])
                assert np.array_equal(t["h_mid"][b:b + 1], h_mid_ref), ("ttt up projection + residual", li, b)
            else:
                qkv_ref = np.concatenate([L.q(xn), L.k(xn), L.v(xn)], axis=1)
                assert np.array_equal(t["qkv"][b:b + 1], qkv_ref), ("q|k|v", li, b, rel_err(t["qkv"][b:b + 1], qkv_ref))
                qkv = t["qkv"][b]
                q = oracle.rope(qkv[:nh * hd].reshape(nh, hd), pos, cfg.rope_theta)
                k = oracle.rope(qkv[nh * hd:(nh + nkv) * hd].reshape(nkv, hd), pos, cfg.rope_theta)
                v = qkv[(nh + nkv) * hd:].reshape(nkv, hd)
                kq_ref, ks_ref = oracle.kv_quant(k)
                vq_ref, vs_ref = oracle.kv_quant(v)
                kq, ks, vq, vs = (a[b] for a in new_rows[li])
                # appended rows: values exact; a rotated key can land on a rounding tie of the 8-bit grid
                assert np.array_equal(vq, vq_ref) and np.array_equal(vs, vs_ref), ("appended V row", li, b)
                assert np.abs(kq.astype(np.int32) - kq_ref.astype(np.int32)).max() <= 1, ("appended K row", li, b)
                assert rel_err(ks, ks_ref) <= 1e-6
                st.kq[li].append(kq); st.ks[li].append(ks); st.vq[li].append(vq); st.vs[li].append(vs)
                tl = len(st.kq[li])
                kd = oracle.kv_dequant(np.stack(st.kq[li], 1).reshape(nkv * tl, hd), np.stack(st.ks[li], 1).reshape(-1)).reshape(nkv, tl, hd)
                vd = oracle.kv_dequant(np.stack(st.vq[li], 1).reshape(nkv * tl, hd), np.stack(st.vs[li], 1).reshape(-1)).reshape(nkv, tl, hd)
                att_ref = oracle.attn_decode(q, kd, vd).reshape(1, -1)
                e = rel_err(t["att"][b:b + 1], att_ref)
                assert e <= ATT_TOL, ("attention", li, b, e)
                h_mid_ref = h_in + L.o(t["att"][b:b + 1])
                assert np.array_equal(t["h_mid"][b:b + 1], h_mid_ref), ("o_proj + residual", li, b, rel_err(t["h_mid"][b:b + 1], h_mid_ref))
            xn2 = oracle.rmsnorm(t["h_mid"][b:b + 1], L.norm2, ref.cfg.rms_eps)
            act_ref = oracle.silu_mul(L.gate(xn2), L.up(xn2))
            e = rel_err(t["act"][b:b + 1], act_ref)
            assert e <= act_tol, ("silu(gate)*up", li, b, e)
            h_out_ref = t["h_mid"][b:b + 1] + L.down(t["act"][b:b + 1])
            assert np.array_equal(t["h_out"][b:b + 1], h_out_ref), ("down_proj + residual", li, b, rel_err(t["h_out"][b:b + 1], h_out_ref))
        hn = oracle.rmsnorm(tr[-1]["h_out"][b:b + 1], ref.norm_f, ref.cfg.rms_eps)
        logits_ref = oracle.dense_linear(hn, ref.lm_head)[0]
        e = rel_err(logits[b], logits_ref)
        assert e <= LOGIT_TOL, ("lm_head", b, e)
        assert logits[b, nxt[b]] == logits[b].max()
        st.pos += 1
    return logits, nxt


def staged_prefill(oracle, ref, gpu, cfg, tokens, states, ttt_chunk=1, act_tol=ACT_TOL):
    """A batched prefill (bt_model_prefill) of tokens [batch, n] checked stage by stage like
    staged_decode_step: every row of every projection bit for bit on the GPU's own stage inputs, every
    token's causal attention over the GPU's cache rows, the appended K/V rows, the TTT predictions,
    and the logits of the last token.  The prefill runs twice from the same state, untraced and traced,
    and both must give the same bits.  Advances `states`.  Returns (logits, next ids)."""
    tokens = np.ascontiguousarray(tokens, np.int32)
    batch, n = tokens.shape
    pos = gpu.current_pos
    is_ttt = cfg.arch == "ttt"
    saved = [gpu.ttt_state(li).clone() for li in range(cfg.num_layers)] if is_ttt else None
    logits, nxt = gpu.prefill(tokens, ttt_chunk)
    gpu.seek(pos)
    if is_ttt:
        for li in range(cfg.num_layers):
            gpu.ttt_state(li).copy_(saved[li])
    gpu.set_trace(True, rows=batch * n)
    logits_t, nxt_t = gpu.prefill(tokens, ttt_chunk)
    gpu.set_trace(False)
    assert np.array_equal(logits, logits_t) and np.array_equal(nxt, nxt_t), "traced and normal prefill differ"
    assert gpu.current_pos == pos + n
    tr = gpu.read_trace(batch * n)
    hd, nh, nkv = cfg.hidden_dim // cfg.n_heads, cfg.n_heads, cfg.n_kv_heads
    for b in range(batch):
        st = states[b]
        assert st.pos == pos
        rows = slice(b * n, (b + 1) * n)
        for li in range(cfg.num_layers):
            L, t = ref.layers[li], tr[li]
            h_in = t["h_in"][rows]
            if li == 0:
                assert np.array_equal(h_in, ref.embed[tokens[b]]), "embedding rows"
            else:
                assert np.array_equal(h_in, tr[li - 1]["h_out"][rows])
            xn = oracle.rmsnorm(h_in, L.norm1, ref.cfg.rms_eps)
            if is_ttt:
                assert np.array_equal(t["qkv"][rows], L.ttt_down(xn)), ("ttt down projection", li, b)
                z_ref = oracle.ttt_chunk(st.w[li], t["qkv"][rows], ref.cfg.inner_lr, ttt_chunk)  # advances the oracle's state
                assert rel_err(t["att"][rows], z_ref) <= TTT_TOL, ("ttt predictions", li, b, rel_err(t["att"][rows], z_ref))
                assert np.array_equal(t["h_mid"][rows], h_in + L.ttt_up(t["att"][rows])), ("ttt up projection + residual", li, b)
            else:
                qkv_ref = np.concatenate([L.q(xn), L.k(xn), L.v(xn)], axis=1)
                assert np.array_equal(t["qkv"][rows], qkv_ref), ("q|k|v", li, b, rel_err(t["qkv"][rows], qkv_ref))
                kq_all, ks_all, vq_all, vs_all = gpu.kv_cache(li).export(b, pos + n)
                assert len(st.kq[li]) == pos
                for i in range(n):
                    qkv = t["qkv"][b * n + i]
                    k = oracle.rope(qkv[nh * hd:(nh + nkv) * hd].reshape(nkv, hd), pos + i, cfg.rope_theta)
                    v = qkv[(nh + nkv) * hd:].reshape(nkv, hd)
                    kq_ref, ks_ref = oracle.kv_quant(k)
                    vq_ref, vs_ref = oracle.kv_quant(v)
                    kq, ks, vq, vs = kq_all[:, pos + i], ks_all[:, pos + i], vq_all[:, pos + i], vs_all[:, pos + i]
                    assert np.array_equal(vq, vq_ref) and np.array_equal(vs, vs_ref), ("appended V row", li, b, i)
                    assert np.abs(kq.astype(np.int32) - kq_ref.astype(np.int32)).max() <= 1, ("appended K row", li, b, i)
                    assert rel_err(ks, ks_ref) <= 1e-6
                    st.kq[li].append(kq.copy()); st.ks[li].append(ks.copy()); st.vq[li].append(vq.copy()); st.vs[li].append(vs.copy())
                tl = pos + n
                kd = oracle.kv_dequant(np.ascontiguousarray(kq_all).reshape(nkv * tl, hd), np.ascontiguousarray(ks_all).reshape(-1)).reshape(nkv, tl, hd)
                vd = oracle.kv_dequant(np.ascontiguousarray(vq_all).reshape(nkv * tl, hd), np.ascontiguousarray(vs_all).reshape(-1)).reshape(nkv, tl, hd)
                for i in range(n):
                    q = oracle.rope(t["qkv"][b * n + i][:nh * hd].reshape(nh, hd), pos + i, cfg.rope_theta)
                    seen = pos + i + 1  # causal: the keys up to the token's own position
                    att_ref = oracle.attn_decode(q, np.ascontiguousarray(kd[:, :seen]), np.ascontiguousarray(vd[:, :seen])).reshape(-1)
                    e = rel_err(t["att"][b * n + i], att_ref)
                    assert e <= ATT_TOL, ("prefill attention", li, b, i, e)
                h_mid_ref = h_in + L.o(t["att"][rows])
                assert np.array_equal(t["h_mid"][rows], h_mid_ref), ("o_proj + residual", li, b, rel_err(t["h_mid"][rows], h_mid_ref))
            xn2 = oracle.rmsnorm(t["h_mid"][rows], L.norm2, ref.cfg.rms_eps)
            act_ref = oracle.silu_mul(L.gate(xn2), L.up(xn2))
            e = rel_err(t["act"][rows], act_ref)
            assert e <= act_tol, ("silu(gate)*up", li, b, e)
            h_out_ref = t["h_mid"][rows] + L.down(t["act"][rows])
            assert np.array_equal(t["h_out"][rows], h_out_ref), ("down_proj + residual", li, b, rel_err(t["h_out"][rows], h_out_ref))
        last = b * n + n - 1
        hn = oracle.rmsnorm(tr[-1]["h_out"][last:last + 1], ref.norm_f, ref.cfg.rms_eps)
        logits_ref = oracle.dense_linear(hn, ref.lm_head)[0]
        e = rel_err(logits[b], logits_ref)
        assert e <= LOGIT_TOL, ("lm_head", b, e)
        assert logits[b, nxt[b]] == logits[b].max()
        st.pos += n
    return logits, nxt
