#!/usr/bin/env python
"""Benchmark: ternary Llama-3-8B-shaped decode, tokens/s, plus the BitLinear GEMV roofline.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--sweep]

One "step" is one decode step (one new token per sequence) of a random-init ternary model with
the Llama-3-8B shape: 32 layers, hidden 4096, MLP 14336, 32 query / 8 KV heads, vocab 128256,
2-bit packed BitLinear weights, dense bf16 lm_head, Q8 KV cache.  The cache is first filled
by the batched prefill (the semantics of the reference CLI's prefill loop, model/llama.rs:495-498;
its rate is reported as `prefill`) so that the timed steps run at the stated context length.  Before anything is timed, the first decode step of the
model is compared with the CPU oracle.

Printed: ONE JSON line (rank 0).  The top-level keys are batch 1: `value` is device-timed
(CUDA events, tokens fed back on the device, graph replay; median of 5 timed regions of K
steps each, every region starting again at the stated context), `e2e` goes through
bt_model_forward_one with host token ids in and host next-token ids out every step,
`e2e_with_logits` also copies the logits out as the reference's loop does (model/llama.rs:507).
`roofline` is the ternary product: `frac` from the launches exactly as the step issues them
(quantiser prologues and fused epilogues included), `frac_isolated` from the plain product on
quantised activations; algorithmic bytes per launch / average launch time, measured here.
`batch64` holds the same measurements at batch 64 (the metric names both batch sizes), with
the share of the step spent in decode attention.  `cpu_baseline` is the CPU oracle timed on
this host on a bounded sample.

With --gpus N > 1 (torchrun, one rank per GPU) the model is tensor-parallel over the N GPUs:
q|k|v and gate|up split by rows, o_proj and down_proj by input columns with an
all-reduce(max) of the activation absmax and an all-reduce(sum) of the int32 accumulators
(NVLink), lm_head replicated.  All ranks decode the SAME sequences, so the total work is fixed
and the scaling is strong.
"""
from __future__ import annotations

import argparse
import importlib
import json
import os
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

METRIC = "ternary 8B decode tok/s (b=1,64); BitLinear GEMV GB/s vs 8 TB/s HBM"
UNIT = "tokens/s"
REGIONS = 5  # timed regions per measurement; the median is reported


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            d = json.load(f)
        return float(d["hbm_gbs"]), float(d.get("bf16_tflops", 0.0)), "measured"
    return 6650.0, 1590.0, "fallback"


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""
    QUERY = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,"
             "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
             "clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index, self.samples, self.proc = index, [], None

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits",
                 "-lms", "100", "-i", str(self.index)], stdout=subprocess.PIPE, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except Exception:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.samples.append(line.strip())

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for s in self.samples:
            parts = [p.strip() for p in s.split(",")]
            if len(parts) < 6:
                continue
            try:
                sm.append(float(parts[0])); mx.append(float(parts[1]))
            except ValueError:
                continue
            for name, val in zip(names, parts[2:6]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": float(np.median(sm)) if sm else None,
                "sm_max_mhz": max(mx) if mx else None, "reasons": sorted(reasons), "samples": len(sm)}


# ---------------------------------------------------------------------------------------
# workload
# ---------------------------------------------------------------------------------------

def build_8b(bt, syn, batch, max_pos, seed=4000, tp_rank=0, tp_size=1, device=0, num_layers=None, shape="8b"):
    """Random-init ternary model of the Llama-3-8B shape (or, shape="tinyllama", the TinyLlama-1.1B shape).
    Layer 0's host arrays are reused for every layer (each layer still owns its own device copy, so HBM
    traffic is real); the embedding and lm_head are one N(0, 0.02) block tiled over the vocabulary."""
    cfg = syn.LLAMA3_8B if shape == "8b" else syn.TINYLLAMA_1B
    cfg = syn.BitLlamaConfig(cfg.arch, cfg.vocab_size, cfg.hidden_dim, num_layers or cfg.num_layers, cfg.n_heads, cfg.n_kv_heads,
                             cfg.intermediate_dim, rope_theta=cfg.rope_theta, max_position_embeddings=max_pos)
    rng = np.random.default_rng(seed)
    block = syn._bf16_round(rng.normal(0, 0.02, (8016, cfg.hidden_dim)).astype(np.float32))
    table = np.tile(block, ((cfg.vocab_size + block.shape[0] - 1) // block.shape[0], 1))[:cfg.vocab_size]
    w = syn.SyntheticWeights(cfg, table, table, np.ones(cfg.hidden_dim, np.float32))
    layer = {"norm1": np.ones(cfg.hidden_dim, np.float32), "norm2": np.ones(cfg.hidden_dim, np.float32)}
    for kind, (n, k) in syn.linear_shapes(cfg).items():
        layer[kind] = (syn._ternary_codes(rng, n, k), 0.016, n, k)
    w.layers = [layer] * cfg.num_layers
    return cfg, w, syn.build_model(w, max_batch=batch, device=device, tp_rank=tp_rank, tp_size=tp_size)


def verify_first_step(model, weights, batch):
    """The benchmarked model's own first decode step (empty cache) against the CPU oracle, stage by stage
    through all layers (oracle/staged.py): q|k|v, the residual sums and silu(gate)*up bit for bit, attention
    and the 128256-row head to f32 accumulation accuracy.  Sequences 0 and batch-1 are checked; a mismatch
    raises.  Leaves the cache empty."""
    from oracle import oracle as orc
    from oracle.staged import staged_decode_step
    cfg = weights.cfg
    tokens = np.random.default_rng(3).integers(0, cfg.vocab_size, size=batch).astype(np.int32)
    ref = orc.model_from_weights(weights)
    states = [ref.new_state() for _ in range(batch)]
    model.reset_kv_cache()
    try:
        staged_decode_step(orc, ref, model, cfg, tokens, states, seqs=sorted({0, batch - 1}))
    except AssertionError as exc:
        raise SystemExit(f"bench.py: the first decode step differs from the oracle: {exc}")
    model.reset_kv_cache()
    return f"all stages of {cfg.num_layers} layers match (BitLinear stages bit-exact, attention <= 2e-5, logits <= 2e-5)"


def cpu_decode_baseline(cfg, syn, budget_s=20.0):
    """CPU oracle on the host cores: per-token time of the 8B-shaped decode estimated from a
    bounded sample - whole transformer blocks (all 7 ternary projections through the
    restatement of BitLinearCpu::forward with its AVX2+FMA inner loop and f32 activations,
    attention at a short context, norms, SwiGLU) and the dense lm_head, each timed and
    scaled to 32 layers."""
    from oracle import oracle as orc
    small = syn.BitLlamaConfig(cfg.arch, 2048, cfg.hidden_dim, 1, cfg.n_heads, cfg.n_kv_heads,
                               cfg.intermediate_dim, rope_theta=cfg.rope_theta, max_position_embeddings=64)
    w = syn.make_weights(small, seed=1, from_latent=False)
    ref = orc.model_from_weights(w, quantised=False)  # the reference's f32-activation kernel
    st = ref.new_state()
    h = np.random.default_rng(0).normal(0, 1, (1, cfg.hidden_dim)).astype(np.float32)
    ref.block(0, h, st)  # warm-up
    t0, n_blocks = time.perf_counter(), 0
    while True:
        ref.block(0, h, st)
        st.pos += 1
        n_blocks += 1
        if time.perf_counter() - t0 > budget_s * 0.6 or n_blocks >= 48:
            break
    t_block = (time.perf_counter() - t0) / n_blocks
    rows = 16032  # one eighth of the vocabulary
    head = np.random.default_rng(1).normal(0, 0.02, (rows, cfg.hidden_dim)).astype(np.float32)
    orc.dense_linear(h, head)
    t1, n_head = time.perf_counter(), 0
    while time.perf_counter() - t1 < budget_s * 0.2 or n_head < 2:
        orc.dense_linear(h, head)
        n_head += 1
    t_head = (time.perf_counter() - t1) / n_head * (cfg.vocab_size / rows)
    t_token = cfg.num_layers * t_block + t_head
    return {
        "value": 1.0 / t_token, "unit": UNIT, "cores": int(orc.lib().oracle_num_threads()), "kind": "port",
        "sample": (f"{n_blocks} transformer blocks of the 8B shape (7 BitLinear, attention at context "
                   f"<= {n_blocks + 1}, norms, SwiGLU) at batch 1 = {t_block * 1e3:.1f} ms/block, dense "
                   f"lm_head on {rows} of {cfg.vocab_size} rows scaled up = {t_head * 1e3:.1f} ms; "
                   f"token time = 32 blocks + head"),
        "ms_per_token": t_token * 1e3,
    }


def run_sweep(bt, device):
    """BitLinear shape sweep, bf16 activations in and out: per point GB/s of algorithmic bytes
    (packed weights + bf16 activations + bf16 outputs) and int8 TOP/s, plus the TTT update."""
    import ctypes as C
    import torch
    peak, bf16_tf, peak_kind = measured_peaks()
    L = bt.lib()
    rng = np.random.default_rng(0)
    for (k, n) in [(4096, 4096), (4096, 14336), (14336, 4096), (4096, 128256)]:
        # distinct weight copies so that consecutive launches do not hit L2 (126 MB)
        copies = max(2, int(400e6 // (n * k / 4))) if n * k / 4 < 200e6 else 2
        packed = rng.integers(0, 256, size=(n, k // 4), dtype=np.uint8)
        lins = [bt.BitLinear.from_packed(packed, [0.016], n, k, device=device) for _ in range(copies)]
        ws = bt.Workspace(device, 768 << 20)
        for m in (1, 8, 64, 512, 4096):
            if m * n * 2 > 3 << 30:
                continue
            x = torch.randn(m, k, device="cuda").bfloat16()
            y = torch.empty(m, n, device="cuda", dtype=torch.bfloat16)

            def run():
                st = C.c_void_p(torch.cuda.current_stream().cuda_stream)
                for lin in lins:
                    bt.check(L.bt_linear_forward(lin._h, ws._h, C.c_void_p(x.data_ptr()), m, k, bt.BT_BF16,
                                                 C.c_void_p(y.data_ptr()), bt.BT_BF16, st))
            run()  # eager once: kernel attributes are set outside the capture
            torch.cuda.synchronize()
            # one pass over all copies as a CUDA graph, so that small points measure the device and
            # not the host's launch rate
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph):
                run()
            graph.replay()
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            reps = 5 if m <= 64 else 2
            e0.record()
            for _ in range(reps):
                graph.replay()
            e1.record()
            torch.cuda.synchronize()
            us = e0.elapsed_time(e1) * 1e3 / (reps * copies)
            byts = n * k / 4 + 2 * m * k + 2 * m * n
            tops = 2.0 * m * n * k / us / 1e6
            print(json.dumps({"sweep": "bitlinear", "K": k, "N": n, "M": m, "us": us, "dtype": "bf16 in / bf16 out",
                              "kernel": "gemv_kernel (mma.sync)" if m <= 8 else "gemm_tc_kernel (tcgen05)",
                              "GBps": byts / us / 1e3, "hbm_frac": byts / us / 1e3 / peak, "peak_kind": peak_kind,
                              "int8_TOPs": tops,
                              "int8_frac_of_2x_bf16_peak": tops / (2 * bf16_tf) if bf16_tf else None,
                              "note": "quantiser kernel included; graph-replayed; weights rotate through copies larger than L2; "
                                      "int8 peak taken as twice the measured bf16 GEMM rate (derived, not measured)"}),
                  flush=True)
        del lins
    run_cpu_cases(bt, device)
    # TTT fast-weight update: S independent 64x64 states, mini-batch 16
    for s_cnt in (4, 64, 1024, 8192):
        w = torch.zeros(s_cnt, 64, 64, device="cuda")
        f = torch.randn(s_cnt, 16, 64, device="cuda")
        bt.ttt_update(w, f, 0.01, 16)
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            bt.ttt_update(w, f, 0.01, 16)
        graph.replay()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(10):
            graph.replay()
        e1.record()
        torch.cuda.synchronize()
        us = e0.elapsed_time(e1) * 1e3 / 10
        byts = s_cnt * (2 * 64 * 64 * 4 + 2 * 16 * 64 * 4)
        print(json.dumps({"sweep": "ttt_update", "states": s_cnt, "d": 64, "chunk": 16, "us": us,
                          "updates_per_s": s_cnt / us * 1e6, "GBps": byts / us / 1e3, "hbm_frac": byts / us / 1e3 / peak}),
              flush=True)


def run_cpu_cases(bt, device):
    """The two configurations the reference can run on a CPU, GPU library beside the CPU port on this host:
    (1) one BitLinear forward, 2048 x 2048 ternary weights, 8 tokens of f32 activations (plus the reference
    micro-benchmark's own shape, 8192 x 8192 with one token, bin/bench_cpu_kernel.rs:15-17), 10 warm-ups and
    100 iterations as in bin/bench_cpu_kernel.rs:54-69; (2) the tiny TTT model (4 blocks, hidden 256, MLP 688,
    vocabulary 32000): prompt of 32 ids, then 128 greedy steps at batch 1."""
    import ctypes as C
    import torch
    from oracle import oracle as orc
    syn = importlib.import_module("bit-ttt-engine_b200.synthetic")
    L = bt.lib()
    for (n, k, m) in [(2048, 2048, 8), (8192, 8192, 1)]:
        rng = np.random.default_rng(1234)
        wt = rng.integers(-1, 2, size=(n, k)).astype(np.float32) * 0.016
        packed, scale = orc.pack_l1(wt)
        x = np.random.default_rng(1235).normal(0, 1, (m, k)).astype(np.float32)
        for _ in range(10):
            y_cpu = orc.bitlinear_f32(x, packed, n, scale)
        t0 = time.perf_counter()
        for _ in range(100):
            y_cpu = orc.bitlinear_f32(x, packed, n, scale)
        cpu_us = (time.perf_counter() - t0) / 100 * 1e6
        y_q = orc.bitlinear_q(x, packed, [scale], n)  # the quantised pipeline the library implements
        lin = bt.BitLinear.from_packed(packed.reshape(n, k // 4), [scale], n, k, device=device)
        ws = bt.Workspace(device, 64 << 20)
        xd = torch.from_numpy(x).cuda()
        yd = torch.empty(m, n, device="cuda")

        def run():
            bt.check(L.bt_linear_forward(lin._h, ws._h, C.c_void_p(xd.data_ptr()), m, k, bt.BT_F32, C.c_void_p(yd.data_ptr()),
                                         bt.BT_F32, C.c_void_p(torch.cuda.current_stream().cuda_stream)))
        run()
        torch.cuda.synchronize()
        exact = bool(np.array_equal(yd.cpu().numpy(), y_q))
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            for _ in range(20):
                run()
        graph.replay()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(5):
            graph.replay()
        e1.record()
        torch.cuda.synchronize()
        gpu_us = e0.elapsed_time(e1) * 1e3 / 100
        byts = m * k * 4 + n * k / 4 + m * n * 4  # bin/bench_cpu_kernel.rs:87-91
        print(json.dumps({"sweep": "cpu_case_bitlinear", "N": n, "K": k, "M": m, "gpu_us": gpu_us, "cpu_us": cpu_us,
                          "cpu_threads": int(orc.lib().oracle_num_threads()), "cpu_GBps": byts / cpu_us / 1e3,
                          "gpu_GBps": byts / gpu_us / 1e3, "gpu_equals_quantised_oracle_bit_for_bit": exact,
                          "max_rel_diff_quantised_vs_f32_reference": float(np.abs(y_q - y_cpu).max() / np.abs(y_cpu).max()),
                          "note": "cpu = restated BitLinearCpu::forward, f32 activations; gpu = quantiser + product, weights in L2 "
                                  "(one small matrix replayed)"}), flush=True)
    cfg = syn.TINY_TTT
    w = syn.make_weights(cfg, seed=2000)
    model = syn.build_model(w, max_batch=1, device=device)
    ref = orc.model_from_weights(w)
    prompt = np.random.default_rng(7).integers(0, cfg.vocab_size, size=32).astype(np.int32)

    def gpu_run():
        model.reset_kv_cache()
        for t in prompt:
            _, nxt = model.forward_one(np.array([t], np.int32), want_logits=False)
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        for _ in range(128):
            _, nxt = model.forward_one(nxt, want_logits=False)
        torch.cuda.synchronize()
        return time.perf_counter() - t0
    gpu_run()
    gpu_s = min(gpu_run() for _ in range(3))
    st = ref.new_state()
    for t in prompt:
        logits = ref.forward_one(int(t), st)
    t0 = time.perf_counter()
    tok = int(np.flatnonzero(logits == logits.max())[-1])
    for _ in range(128):
        logits = ref.forward_one(tok, st)
        tok = int(np.flatnonzero(logits == logits.max())[-1])
    cpu_s = time.perf_counter() - t0
    print(json.dumps({"sweep": "cpu_case_tiny_ttt_decode", "decode_steps": 128, "prompt": 32,
                      "gpu_tokens_per_s": 128 / gpu_s, "cpu_tokens_per_s": 128 / cpu_s,
                      "cpu_threads": int(orc.lib().oracle_num_threads()),
                      "note": "gpu: bt_model_forward_one end to end (host id in, host id out, CUDA graph per step); cpu: the oracle "
                              "model (quantised pipeline) on the host cores"}), flush=True)


def run_reference_arm(args, rank):
    """--impl reference: the reference's CPU implementation of the path.  The reference is a
    Rust workspace with no Rust toolchain available here, so the timed code is the CPU port
    (oracle/bitttt_oracle.c, same arithmetic and AVX2 structure as kernels/cpu.rs) on all
    host threads.  Rank 0 only."""
    if rank != 0:
        return
    syn = importlib.import_module("bit-ttt-engine_b200.synthetic")
    cfg = syn.LLAMA3_8B
    vals = []
    for _ in range(max(1, min(args.steps, 3))):
        vals.append(cpu_decode_baseline(cfg, syn, budget_s=15.0))
    best = max(vals, key=lambda d: d["value"])
    line = {
        "impl": "reference", "metric": METRIC, "value": best["value"], "unit": UNIT, "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": best["ms_per_token"],
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": "Llama-3-8B-shaped ternary decode, batch 1 (CPU port of the reference kernels; "
                               "each step a bounded sample scaled to a full token)"},
        "cpu_baseline": {k: best[k] for k in ("value", "unit", "cores", "kind", "sample")},
        "e2e": {"value": best["value"], "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


# ---------------------------------------------------------------------------------------
# measurements on a built model
# ---------------------------------------------------------------------------------------

class Timer:
    def __init__(self, torch, dist, world, dev):
        self.torch, self.dist, self.world, self.dev = torch, dist, world, dev

    def barrier(self):
        if self.world > 1:
            self.dist.barrier()
        self.torch.cuda.synchronize()

    def max_over_ranks(self, v):
        t = self.torch.tensor([v], dtype=self.torch.float64, device=self.dev)
        if self.world > 1:
            self.dist.all_reduce(t, op=self.dist.ReduceOp.MAX)
        return float(t.item())


def fill_context(model, cfg, B, context, rng, tm):
    """Fills the caches with `context` positions per sequence through the batched prefill (bt_model_prefill:
    host ids in, caches filled, logits of the last token out) and reports its rate."""
    model.reset_kv_cache()
    prompt = rng.integers(0, cfg.vocab_size, size=(B, context)).astype(np.int32)
    model.prefill(prompt[:, :64], want_logits=False)  # first call: scratch allocation and kernel attributes
    model.reset_kv_cache()
    tm.barrier()
    t0 = time.perf_counter()
    model.prefill(prompt, want_logits=False)
    seconds = tm.max_over_ranks(time.perf_counter() - t0)
    return {"tokens": B * context, "batch": B, "tokens_per_sequence": context, "seconds": seconds,
            "tokens_per_s": B * context / seconds,
            "note": "bt_model_prefill end to end (host ids in, synchronous): int8 tensor-core products, causal Q8 attention"}


def fill_tokenwise(model, cfg, B, context, rng, dev, torch):
    """Token-by-token prefill (tensor-parallel models): ids fed from a device array."""
    model.reset_kv_cache()
    prompt = torch.from_numpy(rng.integers(0, cfg.vocab_size, size=(context, B)).astype(np.int32)).to(dev)
    for t in range(context):
        model.step_dev(prompt[t])
    torch.cuda.synchronize()
    return None


def time_decode(model, cfg, B, K, W, context, tm, rng):
    """Median over REGIONS timed regions of K graph-replayed steps, every region starting at `context`."""
    torch = tm.torch
    tok = torch.from_numpy(rng.integers(0, cfg.vocab_size, size=B).astype(np.int32)).to(tm.dev)
    ms_all = []
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    for region in range(REGIONS):
        model.seek(context)
        model.step_dev(tok)
        nxt = model.next_dev()
        for _ in range(W if region == 0 else 1):
            model.step_dev(nxt[:B])
        tm.barrier()
        e0.record()
        for _ in range(K):
            model.step_dev(nxt[:B])  # copies the ids device-to-device, then replays the step graph
        e1.record()
        tm.barrier()
        ms_all.append(tm.max_over_ranks(e0.elapsed_time(e1)))
    return float(np.median(ms_all)), ms_all


def time_e2e(model, cfg, B, K, context, tm, rng, want_logits):
    torch = tm.torch
    vals = []
    for region in range(3):
        model.seek(context)
        ids = rng.integers(0, cfg.vocab_size, size=B).astype(np.int32)
        for _ in range(3):
            _, ids = model.forward_one(ids, want_logits=want_logits)
        tm.barrier()
        t0 = time.perf_counter()
        for _ in range(K):
            _, ids = model.forward_one(ids, want_logits=want_logits)
        torch.cuda.synchronize()
        vals.append(tm.max_over_ranks(time.perf_counter() - t0))
    return B * K / float(np.median(vals))


def time_products(model, B, as_in_step, torch):
    """Average duration of one ternary-product launch of a decode step, replayed alone as a graph."""
    n_launch = model.enqueue_products(B, as_in_step)
    torch.cuda.synchronize()
    g = torch.cuda.CUDAGraph()
    side = torch.cuda.Stream()
    with torch.cuda.stream(side):
        with torch.cuda.graph(g, stream=side):
            model.enqueue_products(B, as_in_step)
    reps = 10
    g.replay()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(reps):
        g.replay()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) * 1e3 / reps, n_launch  # microseconds per step's worth of products


def time_attention(bt, cfg, B, context, torch, tp=1):
    """Decode attention alone, through bt_attn_decode on caches of the model's shape: microseconds
    per layer call at `context` positions (8 caches in rotation, graph-replayed)."""
    hd = cfg.hidden_dim // cfg.n_heads
    nh, nkv = cfg.n_heads // tp, cfg.n_kv_heads // tp
    layers = 8 if B <= 8 else 4
    caches = [bt.QuantizedKVCache(context + 64, B, nkv, hd, device=torch.cuda.current_device()) for _ in range(layers)]
    qkv = torch.randn(B, (nh + 2 * nkv) * hd, device="cuda")
    pos = torch.full((B,), context, dtype=torch.int32, device="cuda")
    for c in caches:
        bt.attn_decode(c, qkv, pos, nh, cfg.rope_theta)
    torch.cuda.synchronize()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        for c in caches:
            bt.attn_decode(c, qkv, pos, nh, cfg.rope_theta)
    g.replay()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(10):
        g.replay()
    e1.record()
    torch.cuda.synchronize()
    us = e0.elapsed_time(e1) * 1e3 / (10 * layers)
    byts = 2 * nkv * (context + 1) * (hd + 4) * B
    return us, byts


def product_bytes(cfg, syn, model, B):
    """Algorithmic bytes of the ternary products of one step: packed weights once + int8 activations in + f32 out."""
    shapes = syn.linear_shapes(cfg)
    act = 0
    for kinds in ([syn.W_Q, syn.W_K, syn.W_V], [syn.W_O], [syn.W_GATE, syn.W_UP], [syn.W_DOWN]):
        n = sum(shapes[k][0] for k in kinds)
        kk = shapes[kinds[0]][1]
        act += B * kk + 4 * B * n
    return model.ternary_bytes + act * cfg.num_layers


def measure_batch(bt, syn, model, cfg, B, K, W, context, tm, rng, world, peak, peak_kind):
    torch = tm.torch
    ms, ms_all = time_decode(model, cfg, B, K, W, context, tm, rng)
    e2e = time_e2e(model, cfg, B, K, context, tm, rng, want_logits=False)
    e2e_logits = time_e2e(model, cfg, B, max(8, K // 4), context, tm, rng, want_logits=True)
    us_step_plain, n_plain = time_products(model, B, False, torch)
    us_step_fused, n_fused = time_products(model, B, True, torch)
    byts = product_bytes(cfg, syn, model, B) / max(world, 1) if world > 1 else product_bytes(cfg, syn, model, B)
    us_attn, attn_bytes = time_attention(bt, cfg, B, context, torch, tp=world)
    kernel = "gemv_kernel (ternary BitLinear product, mma.sync int8)" if B <= 8 else \
             "gemm_tc_kernel (ternary BitLinear product, tcgen05 int8) + its quantiser"
    roofline = {
        "bound": "hbm", "kernel": kernel, "unit": "GB/s", "peak": peak, "peak_kind": peak_kind,
        "achieved": byts / us_step_fused / 1e3, "frac": byts / us_step_fused / 1e3 / peak,
        "achieved_isolated": byts / us_step_plain / 1e3, "frac_isolated": byts / us_step_plain / 1e3 / peak,
        "bytes_per_launch": byts / (4 * cfg.num_layers), "us_per_launch": us_step_fused / (4 * cfg.num_layers),
        "launches_per_step": n_fused, "product_us_per_step": us_step_fused,
        # dram__bytes_read.sum + dram__bytes_write.sum per product launch, mean over the four launches of a block,
        # from one ncu capture of a two-block case of the same shape (read here, not measured by this run)
        "traffic": (13750912.0 if B <= 8 else 14637952.0) if world == 1 and B in (1, 64) and cfg.hidden_dim == 4096 else None,
        "note": "frac: the four products of every block launched exactly as the decode step launches them "
                "(quantiser prologues / kernels and fused epilogues included), replayed alone; frac_isolated: the plain "
                "product on already quantised activations; bytes = packed weights once + int8 activations + f32 outputs",
    }
    return {
        "value": B * K / (ms * 1e-3), "ms_per_step": ms / K, "ms_regions": [m / K for m in ms_all],
        "e2e": {"value": e2e, "unit": UNIT, "h2d_bytes_per_step": 4 * B, "d2h_bytes_per_step": 4 * B},
        "e2e_with_logits": {"value": e2e_logits, "unit": UNIT, "h2d_bytes_per_step": 4 * B,
                            "d2h_bytes_per_step": 4 * B + 4 * B * cfg.vocab_size},
        "roofline": roofline,
        "attention": {"us_per_layer": us_attn, "share_of_step": cfg.num_layers * us_attn / (ms / K * 1e3),
                      "GBps": attn_bytes / us_attn / 1e3, "hbm_frac": attn_bytes / us_attn / 1e3 / peak,
                      "note": "bt_attn_decode alone on caches of the model's shape at this context"},
        "gpu_launches": model.launches_per_step(B) * K,
    }


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=128)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--context", type=int, default=2048, help="tokens in the KV cache before the timed steps")
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-batch64", action="store_true", help="skip the batch-64 half of the metric")
    ap.add_argument("--sweep", action="store_true",
                    help="BitLinear shape sweep (K,N in {4096x4096, 4096x14336, 14336x4096, 4096x128256}, "
                         "M in {1, 8, 64, 512, 4096}, bf16 activations) plus the TTT update: one JSON line per point")
    ap.add_argument("--profile-case", type=int, default=0, metavar="BATCH",
                    help="small case for a profiler, not a benchmark: --layers blocks of the 8B shape, BATCH sequences, "
                         "the context filled by the batched prefill, then 3 decode steps; prints a line marked profile_case")
    ap.add_argument("--layers", type=int, default=2, help="blocks of the --profile-case model")
    ap.add_argument("--shape", default="8b", choices=["8b", "tinyllama"],
                    help="8b: the metric's workload (batch 1 and 64); tinyllama: the TinyLlama-1.1B shape at batch 1 and 16 "
                         "(same measurements, a second reported configuration; use --context 512 for its stated prefill)")
    ap.add_argument("--tp-nccl", action="store_true",
                    help="with --gpus N > 1: keep the tensor-parallel exchanges on NCCL instead of the "
                         "library's peer-memory kernels")
    args = ap.parse_args()
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))

    if args.impl == "reference":
        run_reference_arm(args, rank)
        return

    import torch
    import torch.distributed as dist
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device (there is no CPU fallback)")
    torch.cuda.set_device(local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device(f"cuda:{local_rank}"))
    bt = importlib.import_module("bit-ttt-engine_b200")
    bt.lib()
    syn = importlib.import_module("bit-ttt-engine_b200.synthetic")
    if args.sweep:
        run_sweep(bt, local_rank)
        return

    if args.profile_case:
        B = args.profile_case
        cfg, _, model = build_8b(bt, syn, B, args.context + 64, device=local_rank, num_layers=args.layers)
        rng = np.random.default_rng(11)
        model.prefill(rng.integers(0, cfg.vocab_size, size=(B, args.context)).astype(np.int32), want_logits=False)
        tok = torch.from_numpy(rng.integers(0, cfg.vocab_size, size=B).astype(np.int32)).to(f"cuda:{local_rank}")
        for _ in range(3):
            model.step_dev(tok)
            tok = model.next_dev()[:B].clone()
        torch.cuda.synchronize()
        bt.check(bt.lib().bt_device_check(local_rank))
        print(json.dumps({"profile_case": True, "batch": B, "layers": args.layers, "context": args.context, "decode_steps": 3}))
        return

    K, W = args.steps, max(args.warmup, 3)
    with_b64 = not args.no_batch64
    B2 = 64 if args.shape == "8b" else 16  # the second batch size of the configuration
    B_max = B2 if with_b64 else 1
    K64 = max(8, K // 4)
    max_pos = args.context + max(W + K, 8 + K64) + 16
    cfg, weights, model = build_8b(bt, syn, B_max, max_pos, tp_rank=rank, tp_size=world, device=local_rank, shape=args.shape)
    if world > 1:
        uid = [bt.tp_unique_id() if rank == 0 else None]
        dist.broadcast_object_list(uid, src=0)
        model.tp_init(uid[0])
        if not args.tp_nccl:
            # the row-parallel exchanges as kernels over NVLink peer memory instead of NCCL calls
            # (every rank has to succeed, otherwise all of them stay on NCCL)
            ok = 1
            try:
                handles = [None] * world
                dist.all_gather_object(handles, model.tp_peer_handle())
                model.tp_peer_init(handles)
            except Exception as exc:  # noqa: BLE001
                print(f"rank {rank}: peer-memory exchange unavailable ({exc}); using NCCL", file=sys.stderr)
                ok = 0
            flag = torch.tensor([ok], device=f"cuda:{local_rank}")
            dist.all_reduce(flag, op=dist.ReduceOp.MIN)
            if int(flag.item()) == 0:
                args.tp_nccl = True
                try:
                    model.tp_peer_disable()
                except Exception:  # noqa: BLE001
                    pass
    dev = torch.device(f"cuda:{local_rank}")
    tm = Timer(torch, dist, world, dev)
    rng = np.random.default_rng(11)  # every rank feeds the same ids
    peak, _, peak_kind = measured_peaks()

    # ---- the benchmarked model's own first step against the oracle, before anything is timed ----
    verified = {"batch1": verify_first_step(model, weights, 1)} if world == 1 else {}
    if with_b64 and world == 1:
        verified[f"batch{B2}"] = verify_first_step(model, weights, B2)
    if world > 1:
        # tensor parallelism: every rank must hold the same logits bit for bit (the exchanges are exact), and the
        # sharded model must agree with the oracle on rank 0's first step within the head's accumulation accuracy
        import hashlib
        for bsz in ([1, B2] if with_b64 else [1]):
            model.reset_kv_cache()
            toks = np.random.default_rng(3).integers(0, cfg.vocab_size, size=bsz).astype(np.int32)
            logits, nxt = model.forward_one(toks)
            digest = hashlib.sha256(logits.tobytes() + nxt.tobytes()).hexdigest()
            digests = [None] * world
            dist.all_gather_object(digests, digest)
            if len(set(digests)) != 1:
                raise SystemExit(f"bench.py: the ranks' logits differ at batch {bsz}")
            verified[f"tp{world}_batch{bsz}"] = f"first-step logits and picks bit-identical on all {world} ranks"
        model.reset_kv_cache()
    del weights

    # ---- batch 1 ---------------------------------------------------------------------------
    prefill1 = fill_context(model, cfg, 1, args.context, rng, tm) if world == 1 else fill_tokenwise(model, cfg, 1, args.context, rng, dev, torch)
    sampler = ClockSampler(local_rank)
    sampler.start()
    b1 = measure_batch(bt, syn, model, cfg, 1, K, W, args.context, tm, rng, world, peak, peak_kind)
    clocks = sampler.stop()

    # ---- batch 64 --------------------------------------------------------------------------
    b64 = None
    if with_b64:
        prefill64 = fill_context(model, cfg, B2, args.context, rng, tm) if world == 1 else fill_tokenwise(model, cfg, B2, args.context, rng, dev, torch)
        b64 = measure_batch(bt, syn, model, cfg, B2, K64, W, args.context, tm, rng, world, peak, peak_kind)
        b64["steps"] = K64
        b64["unit"] = UNIT
        if prefill64 is not None:
            b64["prefill"] = prefill64

    if rank == 0:
        cpu = None if args.no_cpu_baseline else cpu_decode_baseline(cfg, syn)
        line = {
            "metric": METRIC, "value": b1["value"], "unit": UNIT, "n_gpus": world, "steps": K, "warmup": W,
            "ms_per_step": b1["ms_per_step"], "higher_is_better": True, "scaling": "strong" if world > 1 else "weak",
            "vs_baseline": None,
            "dtype": "int8 x ternary -> int32 (f32 epilogue, bf16 lm_head)", "data": "synthetic",
            "config": {"workload": f"{'Llama-3-8B' if args.shape == '8b' else 'TinyLlama-1.1B'}-shaped ternary decode, batch 1 (top level) and batch {B2} (`batch{B2}`), context {args.context}+",
                       "batch": 1, "context": args.context,
                       "parallelism": (f"tp{world} ({'NCCL' if args.tp_nccl else 'peer-memory'} exchange)") if world > 1 else "single GPU",
                       "timing": f"median of {REGIONS} regions of {K} steps, each region restarted at the stated context",
                       "l2": f"inputs larger than L2: {model.ternary_bytes / 1e9:.2f} GB of ternary tiles + {2 * cfg.vocab_size * cfg.hidden_dim / 1e9:.2f} GB lm_head per step"},
            "ms_regions": b1["ms_regions"],
            "e2e": b1["e2e"], "e2e_with_logits": b1["e2e_with_logits"],
            "gpu_launches": b1["gpu_launches"],
            "roofline": b1["roofline"], "attention": b1["attention"], "clocks": clocks,
            ("verified_against_oracle" if world == 1 else "verified_ranks_agree"): verified,
        }
        if prefill1 is not None:
            line["prefill"] = prefill1
        if b64 is not None:
            line[f"batch{B2}"] = b64
        if cpu is not None:
            line["cpu_baseline"] = {k: cpu[k] for k in ("value", "unit", "cores", "kind", "sample")}
        print(json.dumps(line), flush=True)
    bt.check(bt.lib().bt_device_check(local_rank))
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
