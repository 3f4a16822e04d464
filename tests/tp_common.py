"""Worker functions of the tensor-parallel tests (importable by spawned processes)."""
import importlib
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
for p in (ROOT, os.path.join(ROOT, "tests")):
    if p not in sys.path:
        sys.path.insert(0, p)


def _init(rank, world, port, backend):
    import torch.distributed as dist
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group(backend, rank=rank, world_size=world)
    return dist


def cpu_row_parallel_worker(rank, world, port, result_dir):
    """Host-side logic of a row-parallel BitLinear on `world` gloo ranks: shard the packed
    columns, all-reduce(max) the per-token absmax, quantise, integer product on the shard,
    all-reduce(sum) the int32 accumulators, scale.  Must equal the unsharded oracle bit for bit."""
    import torch
    from oracle import oracle as orc
    dist = _init(rank, world, port, "gloo")
    rng = np.random.default_rng(5)  # same data on every rank
    m, n, k = 3, 48, 512
    w = rng.normal(0, 0.02, (n, k)).astype(np.float32)
    packed, sw = orc.pack_l1(w)
    packed = packed.reshape(n, k // 4)
    x = rng.normal(0, 1, (m, k)).astype(np.float32)
    cols = k // world
    x_loc = x[:, rank * cols:(rank + 1) * cols]
    p_loc = np.ascontiguousarray(packed[:, rank * cols // 4:(rank + 1) * cols // 4])
    amax = torch.from_numpy(np.abs(x_loc).max(axis=1).astype(np.float32))
    dist.all_reduce(amax, op=dist.ReduceOp.MAX)
    amax = amax.numpy()
    inv = np.where(amax > 0, np.float32(127.0) / amax, 0).astype(np.float32)
    ratio = (x_loc * inv[:, None]).astype(np.float32)
    q = np.clip(np.sign(ratio) * np.floor(np.abs(ratio) + np.float32(0.5)), -127, 127).astype(np.int8)
    acc = torch.from_numpy(orc.bitlinear_i32(q, p_loc, n))
    dist.all_reduce(acc, op=dist.ReduceOp.SUM)
    sx = (amax / np.float32(127.0)).astype(np.float32)
    y = (acc.numpy().astype(np.float32) * np.float32(sw)) * sx[:, None]
    ref = orc.bitlinear_q(x, packed, [sw], n)
    ok = bool(np.array_equal(y, ref))
    # column-parallel: rows of the output are simply split
    rows = n // world
    y_col = orc.bitlinear_q(x, np.ascontiguousarray(packed[rank * rows:(rank + 1) * rows]), [sw], rows)
    ok = ok and bool(np.array_equal(y_col, ref[:, rank * rows:(rank + 1) * rows]))
    open(os.path.join(result_dir, f"rank{rank}.txt"), "w").write("ok" if ok else "mismatch")
    dist.destroy_process_group()


def gpu_model_worker(rank, world, port, result_dir, n_tokens, use_peer=False, batch=2):
    """Tensor-parallel decode of a small llama-shaped model on `world` GPUs, checked stage by stage:
    every rank's q|k|v and silu(gate)*up slices against the oracle's slices, and the two row-parallel
    projections (o_proj, down_proj: absmax exchange + integer sum over the ranks) bit for bit against
    the oracle's unsharded projection of the gathered slices.  Every rank must hold the same hidden
    state and logits bit for bit.  use_peer: exchange over NVLink peer memory instead of NCCL.
    batch > 8 takes the tensor-core step (row quantiser + tcgen05 products, collectives over NCCL)."""
    import torch
    dist = _init(rank, world, port, "gloo")
    torch.cuda.set_device(rank)
    bt = importlib.import_module("bit-ttt-engine_b200")
    syn = importlib.import_module("bit-ttt-engine_b200.synthetic")
    from oracle import oracle as orc
    cfg = syn.BitLlamaConfig("llama", 1000, 256, 2, 8, max(4, world), 512, max_position_embeddings=64)  # KV heads: 4, or one per rank
    w = syn.make_weights(cfg, seed=3000)
    model = syn.build_model(w, max_batch=batch, device=rank, tp_rank=rank, tp_size=world)
    if use_peer:
        handles = [None] * world
        dist.all_gather_object(handles, model.tp_peer_handle())
        model.tp_peer_init(handles)
    else:
        uid = [bt.tp_unique_id() if rank == 0 else None]
        dist.broadcast_object_list(uid, src=0)
        model.tp_init(uid[0])
    ref = orc.model_from_weights(w)
    hd, nh, nkv, inter = cfg.hidden_dim // cfg.n_heads, cfg.n_heads, cfg.n_kv_heads, cfg.intermediate_dim
    nh_l, nkv_l, i_l = nh // world, nkv // world, inter // world
    tokens = np.random.default_rng(7).integers(0, cfg.vocab_size, size=(n_tokens, batch))
    worst, same, ok = 0.0, True, True
    model.set_trace(True)
    for t in range(n_tokens):
        logits, nxt = model.forward_one(tokens[t])
        mine = torch.from_numpy(logits.copy())
        theirs = mine.clone()
        dist.broadcast(theirs, src=0)
        same = same and bool(torch.equal(mine, theirs))
        tr = model.read_trace(batch)
        gathered = [None] * world
        dist.all_gather_object(gathered, [{k: v for k, v in layer.items() if k in ("att", "act")} for layer in tr])
        for b in range(batch):
            for li in range(cfg.num_layers):
                L, lt = ref.layers[li], tr[li]
                h_in = lt["h_in"][b:b + 1]
                xn = orc.rmsnorm(h_in, L.norm1, ref.cfg.rms_eps)
                q, k, v = L.q(xn)[0], L.k(xn)[0], L.v(xn)[0]
                mine_qkv = np.concatenate([q[rank * nh_l * hd:(rank + 1) * nh_l * hd], k[rank * nkv_l * hd:(rank + 1) * nkv_l * hd],
                                           v[rank * nkv_l * hd:(rank + 1) * nkv_l * hd]])
                ok = ok and bool(np.array_equal(lt["qkv"][b], mine_qkv))
                att_full = np.concatenate([gathered[r][li]["att"][b] for r in range(world)])[None, :]
                ok = ok and bool(np.array_equal(lt["h_mid"][b:b + 1], h_in + L.o(att_full)))
                xn2 = orc.rmsnorm(lt["h_mid"][b:b + 1], L.norm2, ref.cfg.rms_eps)
                act_ref = orc.silu_mul(L.gate(xn2), L.up(xn2))[0]
                mine_act = act_ref[rank * i_l:(rank + 1) * i_l]
                ok = ok and float(np.abs(lt["act"][b] - mine_act).max()) <= 1e-6 * float(np.abs(mine_act).max())
                act_full = np.concatenate([gathered[r][li]["act"][b] for r in range(world)])[None, :]
                ok = ok and bool(np.array_equal(lt["h_out"][b:b + 1], lt["h_mid"][b:b + 1] + L.down(act_full)))
            hn = orc.rmsnorm(tr[-1]["h_out"][b:b + 1], ref.norm_f, ref.cfg.rms_eps)
            r = orc.dense_linear(hn, ref.lm_head)[0]
            worst = max(worst, float(np.abs(logits[b] - r).max() / np.abs(r).max()))
    model.set_trace(False)
    # the captured path (CUDA graph with the exchanges inside) gives the same bits as the traced one
    model.reset_kv_cache()
    for t in range(3):
        logits_g, _ = model.forward_one(tokens[t])
    model.reset_kv_cache()
    model.set_trace(True)
    for t in range(3):
        logits_t, _ = model.forward_one(tokens[t])
    model.set_trace(False)
    ok = ok and bool(np.array_equal(logits_g, logits_t))
    bt.check(bt.lib().bt_device_check(rank))
    open(os.path.join(result_dir, f"rank{rank}.txt"), "w").write(f"{worst} {int(same)} {int(ok)}")
    del model
    dist.destroy_process_group()


def gpu_timeout_worker(rank, world, port, result_dir):
    """A rank that never joins: both ranks of a 2-way tensor-parallel model live on GPU 0 and
    exchange their inbox handles, but only rank 0 ever runs a step.  Its exchange kernels wait for
    flags that rank 1 never writes; the wait is bounded, so the step must come back with
    BT_ERR_TIMEOUT (no fault, no hang) and the device must stay usable.  Rank 1 launches nothing
    while rank 0 runs, so no two kernels ever wait on one another on the one GPU."""
    import time
    import torch
    dist = _init(rank, world, port, "gloo")
    torch.cuda.set_device(0)
    bt = importlib.import_module("bit-ttt-engine_b200")
    syn = importlib.import_module("bit-ttt-engine_b200.synthetic")
    from oracle import oracle as orc
    cfg = syn.BitLlamaConfig("llama", 1000, 256, 2, 8, 4, 512, max_position_embeddings=64)
    w = syn.make_weights(cfg, seed=3000)
    model = syn.build_model(w, max_batch=2, device=0, tp_rank=rank, tp_size=world)
    handles = [None] * world
    dist.all_gather_object(handles, model.tp_peer_handle())
    model.tp_peer_init(handles)
    result = "idle"
    if rank == 0:
        model.tp_set_timeout(50)
        t0 = time.perf_counter()
        try:
            model.forward_one(np.array([3, 4], np.int32))
            result = "no error"
        except bt.BitTTTError as exc:
            result = f"status {exc.status}"
        elapsed = time.perf_counter() - t0
        # the error was consumed by the failing call; the device answers and computes correctly
        clean = bt.lib().bt_device_check(0) == bt.BT_OK
        rng = np.random.default_rng(1)
        wd = rng.normal(0, 0.02, (64, 128)).astype(np.float32)
        x = rng.normal(0, 1, (2, 128)).astype(np.float32)
        lin = bt.BitLinear.load(128, 64, wd, device=0)
        lin.precompute_packed()
        y = lin.forward(torch.from_numpy(x).cuda()).cpu().numpy()
        p, s = orc.pack_l1(wd)
        usable = bool(np.array_equal(y, orc.bitlinear_q(x, p, [s], 64)))
        result += f" clean {int(clean)} usable {int(usable)} fast {int(elapsed < 20.0)}"
    dist.barrier()  # rank 1 stays alive (its inbox mapped) until rank 0 is done
    open(os.path.join(result_dir, f"rank{rank}.txt"), "w").write(result)
    del model
    dist.destroy_process_group()
