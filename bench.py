#!/usr/bin/env python
"""Benchmark: ternary Llama-3-8B-shaped decode, tokens/s, plus the BitLinear GEMV roofline.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--batch B] [--impl ours|reference]

One "step" is one decode step (one new token for each of the B sequences) of a random-init
ternary model with the Llama-3-8B shape: 32 layers, hidden 4096, MLP 14336, 32 query / 8 KV
heads, vocab 128256, 2-bit packed BitLinear weights, dense bf16 lm_head, Q8 KV cache.  The
cache is first filled token by token (the reference CLI's prefill, model/llama.rs:495-498)
so that the timed steps run at the stated context length.

Printed: ONE JSON line (rank 0).  `value` is device-timed (CUDA events, tokens fed back on
the device, graph replay); `e2e` goes through bt_model_forward_one with host token ids in
and host next-token ids out every step; `roofline` is the ternary GEMV alone (algorithmic
bytes per launch / average launch time, measured in this run); `cpu_baseline` is the CPU
oracle timed on this host on a bounded sample.

With --gpus N > 1 (torchrun, one rank per GPU) the model is tensor-parallel over the N GPUs:
q|k|v and gate|up split by rows, o_proj and down_proj by input columns with an
all-reduce(max) of the activation absmax and an all-reduce(sum) of the int32 accumulators
(NCCL over NVLink), lm_head replicated.  All ranks decode the SAME B sequences, so the total
work is fixed and the scaling is strong.
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


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            d = json.load(f)
        return float(d["hbm_gbs"]), "measured"
    return 6650.0, "fallback"


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

def build_8b(bt, syn, batch, max_pos, seed=4000, tp_rank=0, tp_size=1, device=0, layers=32, vocab=128256):
    """Random-init Llama-3-8B-shaped ternary model.  Layer 0's host arrays are reused for
    every layer (each layer still owns its own device copy, so HBM traffic is real); the
    embedding and lm_head are one N(0, 0.02) block tiled over the vocabulary."""
    cfg = syn.BitLlamaConfig("llama", vocab, 4096, layers, 32, 8, 14336, rope_theta=500000.0,
                             max_position_embeddings=max_pos)
    rng = np.random.default_rng(seed)
    block = rng.normal(0, 0.02, (min(8016, vocab), cfg.hidden_dim)).astype(np.float32)
    table = np.tile(block, ((vocab + block.shape[0] - 1) // block.shape[0], 1))[:vocab]
    w = syn.SyntheticWeights(cfg, table, table, np.ones(cfg.hidden_dim, np.float32))
    layer = {"norm1": np.ones(cfg.hidden_dim, np.float32), "norm2": np.ones(cfg.hidden_dim, np.float32)}
    for kind, (n, k) in syn.linear_shapes(cfg).items():
        layer[kind] = (syn._ternary_codes(rng, n, k), 0.016, n, k)
    w.layers = [layer] * cfg.num_layers
    return cfg, w, syn.build_model(w, max_batch=batch, device=device, tp_rank=tp_rank, tp_size=tp_size)


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


def run_linear_probe(bt, n, k, m):
    """Three forwards of one BitLinear (profiling aid for the product kernels)."""
    import torch
    rng = np.random.default_rng(0)
    lin = bt.BitLinear.from_packed(rng.integers(0, 256, size=(n, k // 4), dtype=np.uint8), [0.016], n, k)
    x = torch.randn(m, k, device="cuda")
    ws = bt.Workspace(0, 768 << 20)
    for _ in range(3):
        y = lin.forward(x, workspace=ws)
    torch.cuda.synchronize()
    print("linear probe done", float(y.abs().sum()), file=sys.stderr)


def run_timeline(bt, model, args, B):
    """Profiling aid: the kernels of the fused decode step (batch <= 8) write globaltimer stamps per
    CTA (entry, dependency released, activations staged, last epilogue warp done) while one step is
    captured; the replayed step is then printed launch by launch, in ns from the first stamp."""
    import ctypes as C
    import torch
    layers = args.layers
    L = bt.lib()
    model.seek(args.context)
    buf = torch.zeros(layers * 5 * 512 * 4, dtype=torch.int64, device="cuda")
    ids = np.arange(B, dtype=np.int32) + 5
    _, ids = model.forward_one(ids, want_logits=False)   # eager step: kernel attributes
    L.bt_debug_timeline.argtypes = [C.c_void_p]
    L.bt_debug_timeline(C.c_void_p(buf.data_ptr()))
    _, ids = model.forward_one(ids, want_logits=False)   # captured with the stamp slots
    L.bt_debug_timeline(None)
    for _ in range(5):
        _, ids = model.forward_one(ids, want_logits=False)
    torch.cuda.synchronize()
    t = buf.cpu().numpy().reshape(layers * 5, 512, 4)
    names = ["q|k|v", "attention", "o_proj", "gate|up", "down_proj"]
    t00 = None
    for s in range(layers * 5):
        v = t[s]
        if s % 5 == 1:  # attention: 8 stamps per CTA (entry, released, ..., partials written, arrived)
            v8 = v.reshape(256, 8)
            v = np.stack([v8[:, 0], v8[:, 1], v8[:, 6], v8[:, 7]], 1)
        used = v[:, 0] > 0
        if not used.any():
            continue
        if t00 is None:
            t00 = v[used, 0].min()
        cols = [v[used, i] - t00 for i in range(4)]
        print(f"block {s // 5} {names[s % 5]:10s} ctas {int(used.sum()):3d}  entry {int(cols[0].min()):7d}..{int(cols[0].max()):7d}"
              f"  released {int(cols[1].min()):7d}..{int(cols[1].max()):7d}  staged {int(cols[2].min()):7d}..{int(cols[2].max()):7d}"
              f" (median {int(np.median(cols[2])):7d})  done {int(cols[3].min()):7d}..{int(cols[3].max()):7d}")


def run_sweep(bt, device):
    """BASELINE config 5: per point GB/s of packed weights (HBM-bound points) and int8 TOP/s."""
    import ctypes as C
    import torch
    peak, peak_kind = measured_peaks()
    L = bt.lib()
    rng = np.random.default_rng(0)
    for (k, n) in [(4096, 4096), (4096, 14336), (14336, 4096), (4096, 128256)]:
        # distinct weight copies so that consecutive launches do not hit L2 (126 MB)
        copies = max(2, int(400e6 // (n * k / 4))) if n * k / 4 < 200e6 else 2
        packed = rng.integers(0, 256, size=(n, k // 4), dtype=np.uint8)
        lins = [bt.BitLinear.from_packed(packed, [0.016], n, k, device=device) for _ in range(copies)]
        ws = bt.Workspace(device, 768 << 20)
        for m in (1, 8, 64, 512, 4096):
            if m * n * 4 > 3 << 30:
                continue
            x = torch.randn(m, k, device="cuda")
            y = torch.empty(m, n, device="cuda")

            def run():
                st = C.c_void_p(torch.cuda.current_stream().cuda_stream)
                for lin in lins:
                    bt.check(L.bt_linear_forward(lin._h, ws._h, C.c_void_p(x.data_ptr()), m, k, 0,
                                                 C.c_void_p(y.data_ptr()), 0, st))
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
            print(json.dumps({"sweep": "bitlinear", "K": k, "N": n, "M": m, "us": us,
                              "kernel": "gemv (mma.sync)" if m <= 8 else "gemm_tc (tcgen05)",
                              "GBps": byts / us / 1e3, "hbm_frac": byts / us / 1e3 / peak, "peak_kind": peak_kind,
                              "int8_TOPs": 2.0 * m * n * k / us / 1e6,
                              "note": "quantiser kernel included; graph-replayed; weights rotate through copies larger than L2"}),
                  flush=True)
        del lins
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


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=128)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--batch", type=int, default=1)
    ap.add_argument("--context", type=int, default=2048, help="tokens in the KV cache before the timed steps")
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--layers", type=int, default=32, help="profiling aid: fewer layers of the same shape")
    ap.add_argument("--vocab", type=int, default=128256, help="profiling aid: smaller vocabulary")
    ap.add_argument("--one-step", action="store_true",
                    help="profiling aid: build the model, --seek to the context, run ONE eager decode step "
                         "(every kernel launched outside a graph) and exit without a JSON line")
    ap.add_argument("--timeline", action="store_true",
                    help="profiling aid (batch <= 8): per-launch globaltimer stamps of one graph-replayed step, "
                         "printed per block; use with --layers 2 --seek")
    ap.add_argument("--linear", type=int, nargs=3, metavar=("N", "K", "M"),
                    help="profiling aid: three bt_linear_forward calls on a random [N, K] weight with M tokens, then exit")
    ap.add_argument("--sweep", action="store_true",
                    help="BitLinear shape sweep (K,N in {4096x4096, 4096x14336, 14336x4096, 4096x128256}, "
                         "M in {1, 8, 64, 512, 4096}) plus the TTT update: one JSON line per point")
    ap.add_argument("--tp-nccl", action="store_true",
                    help="with --gpus N > 1: keep the tensor-parallel exchanges on NCCL instead of the "
                         "library's peer-memory kernels")
    ap.add_argument("--seek", action="store_true",
                    help="profiling aid: skip the token-by-token prefill and declare the (zero-filled) "
                         "cache to hold --context positions")
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

    B, K, W = args.batch, args.steps, max(args.warmup, 3)
    max_pos = args.context + W + 2 * K + 16
    if args.linear:
        run_linear_probe(bt, *args.linear)
        return
    if args.sweep:
        run_sweep(bt, local_rank)
        return
    cfg, weights, model = build_8b(bt, syn, B, max_pos, tp_rank=rank, tp_size=world, device=local_rank,
                                   layers=args.layers, vocab=args.vocab)
    del weights
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
    rng = np.random.default_rng(11)  # every rank feeds the same ids

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    if args.timeline:
        run_timeline(bt, model, args, B)
        del model
        return

    if args.one_step:
        model.seek(args.context)
        _, ids = model.forward_one(np.arange(B, dtype=np.int32) + 5, want_logits=False)
        torch.cuda.synchronize()
        print("one eager step done, next ids", ids[:4].tolist(), file=sys.stderr)
        del model
        return

    # prefill token by token, tokens fed from the host like the reference CLI
    tok = torch.from_numpy(rng.integers(0, cfg.vocab_size, size=B).astype(np.int32)).to(dev)
    prompt = torch.from_numpy(rng.integers(0, cfg.vocab_size, size=(args.context, B)).astype(np.int32)).to(dev)
    if args.seek:
        model.seek(args.context)
    else:
        for t in range(args.context):
            model.step_dev(prompt[t])
    for _ in range(W):
        model.step_dev(tok)
        tok = model.next_dev()[:B].clone()
    barrier()

    # ---- device-timed decode: K steps, greedy ids fed back on the device --------------------
    sampler = ClockSampler(local_rank)
    sampler.start()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    nxt = model.next_dev()
    barrier()
    e0.record()
    for _ in range(K):
        model.step_dev(nxt[:B])  # copies the ids device-to-device, then replays the step graph
    e1.record()
    barrier()
    ms = e0.elapsed_time(e1)
    clocks = sampler.stop()
    t = torch.tensor([ms], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms_max = float(t.item())
    value = B * K / (ms_max * 1e-3)

    # ---- end to end: host ids in, host ids out, every step ---------------------------------
    ids = rng.integers(0, cfg.vocab_size, size=B).astype(np.int32)
    for _ in range(3):
        _, ids = model.forward_one(ids, want_logits=False)
    barrier()
    t0 = time.perf_counter()
    for _ in range(K):
        _, ids = model.forward_one(ids, want_logits=False)
    torch.cuda.synchronize()
    e2e_s = time.perf_counter() - t0
    t = torch.tensor([e2e_s], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    e2e_value = B * K / float(t.item())

    # ---- roofline of the dominant kernel: the ternary GEMV launches of a step, alone -------
    peak, peak_kind = measured_peaks()
    n_launch = model.enqueue_products(B)
    torch.cuda.synchronize()
    g = torch.cuda.CUDAGraph()
    side = torch.cuda.Stream()
    with torch.cuda.stream(side):
        with torch.cuda.graph(g, stream=side):
            model.enqueue_products(B)
    reps = 10
    g.replay()
    torch.cuda.synchronize()
    e0.record()
    for _ in range(reps):
        g.replay()
    e1.record()
    torch.cuda.synchronize()
    us_per_launch = e0.elapsed_time(e1) * 1e3 / (reps * n_launch)
    groups = (B + 7) // 8
    # algorithmic bytes: packed weights once per launch + int8 activations in + f32 out
    shapes = syn.linear_shapes(cfg)
    act_bytes = 0
    for kinds in ([syn.W_Q, syn.W_K, syn.W_V], [syn.W_O], [syn.W_GATE, syn.W_UP], [syn.W_DOWN]):
        n = sum(shapes[k][0] for k in kinds)
        kk = shapes[kinds[0]][1]
        act_bytes += B * kk + 4 * B * n
    bytes_per_step = model.ternary_bytes * groups + act_bytes * cfg.num_layers
    bytes_per_launch = bytes_per_step / n_launch
    achieved = bytes_per_launch / us_per_launch / 1e3  # GB/s
    roofline = {"bound": "hbm", "kernel": "gemv_kernel (ternary BitLinear product)", "achieved": achieved,
                "peak": peak, "unit": "GB/s", "frac": achieved / peak, "peak_kind": peak_kind,
                # dram__bytes_read+write per launch, average over the four projections of a block, from the
                # ncu capture summarised in profiles/gemv_kernel_decode_layer_8b.md (batch 1, one GPU)
                "traffic": 13.75e6 if (B == 1 and world == 1) else None,
                "bytes_per_launch": bytes_per_launch, "us_per_launch": us_per_launch,
                "launches_per_step": n_launch}

    if rank == 0:
        cpu = None if args.no_cpu_baseline else cpu_decode_baseline(cfg, syn)
        line = {
            "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": K, "warmup": W,
            "ms_per_step": ms_max / K, "higher_is_better": True, "scaling": "strong" if world > 1 else "weak",
            "vs_baseline": None,
            "dtype": "int8 x ternary -> int32 (f32 epilogue, bf16 lm_head)", "data": "synthetic",
            "config": {"workload": f"Llama-3-8B-shaped ternary decode, batch {B}, context {args.context}+",
                       "batch": B, "context": args.context, "parallelism": (f"tp{world} ({'NCCL' if args.tp_nccl else 'peer-memory'} exchange)") if world > 1 else "single GPU",
                       "l2": "inputs larger than L2: 1.74 GB of ternary tiles + 1.05 GB lm_head per step"},
            "e2e": {"value": e2e_value, "unit": UNIT, "h2d_bytes_per_step": 4 * B, "d2h_bytes_per_step": 4 * B},
            "gpu_launches": model.launches_per_step(B) * K,
            "roofline": roofline, "clocks": clocks,
        }
        if cpu is not None:
            line["cpu_baseline"] = {k: cpu[k] for k in ("value", "unit", "cores", "kind", "sample")}
        print(json.dumps(line), flush=True)
    bt.check(bt.lib().bt_device_check(local_rank))
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
