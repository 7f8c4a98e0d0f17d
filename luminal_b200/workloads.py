"""Secondary benchmark workloads (`bench.py --workload ...`): batched serving decode, tensor-parallel 70B-shape decode,
the MXFP4 MoE layer.  Each returns a dict that bench.py prints as one JSON line.  Inputs are seeded synthetic data of
the configurations' shapes; there are no checkpoints in this environment."""
import ctypes as C
import time

import numpy as np

from . import BF16, F32, BlumError, Context
from .llama import LLAMA3_8B, LLAMA3_70B, Llama
from .runtime import gen_token_ids, gen_normal, round_to_dtype


def serve64(ctx: Context, steps, warmup, batch=64, seed=2, prefill_chunk=2048, layers=None, rank=0, world=1):
    """Llama-3-8B-shape Q8_0 model, bf16 activations, paged bf16 KV (page 16, physical pages shuffled), `batch` sequences
    with context lengths uniform in [512, 4096], one decode step per bench step; one `prefill_chunk`-token prompt pass is
    timed separately.  With world > 1 every rank is a replica that serves sequences rank, rank + world, ... of the batch."""
    cfg = dict(LLAMA3_8B)
    if layers:
        cfg["layers"] = layers
    rng = np.random.default_rng(seed)
    lens = rng.integers(512, 4097, size=batch)[rank::world]
    batch = len(lens)
    total_steps = warmup + steps + 2
    pages = int(sum((n + total_steps + 15) // 16 for n in lens)) + (prefill_chunk + 15) // 16 + 8
    model = Llama(ctx, cfg, act_dtype=BF16, kv_dtype=BF16, page_size=16, max_seqs=batch + 1, max_ctx=4096 + total_steps + 16,
                  kv_pages=pages)
    model.generate_weights(0)
    ctx._check(ctx.lib.blum_memset(ctx.h, ctx.lib.blum_kv_pool_dev(model.kv.h), 0x3C, ctx.lib.blum_kv_pool_bytes(model.kv.h)))
    seqs = []
    need = [(int(n) + 15) // 16 for n in lens]
    perm = rng.permutation(int(sum(need))).astype(np.int32)          # page ids shuffled: a sequence's pages are scattered
    at = 0
    for n, npg in zip(lens, need):
        s = model.new_sequence()
        model.kv.seq_set_pages(s, perm[at:at + npg], int(n))     # contexts exist in the cache (values 0x3c3c = 0.0115), no prompt pass needed
        at += npg
        seqs.append(s)
    toks = gen_token_ids(seed, 1, batch, cfg["vocab"])
    for _ in range(max(warmup, 3)):
        toks = model.decode(seqs, toks)
    ctx.sync()
    launches0 = ctx.launches
    ctx.timer_start(5)
    t0 = time.perf_counter()
    for _ in range(steps):
        toks = model.decode(seqs, toks)
    ctx.timer_stop(5)
    ms = ctx.timer_ms(5)
    wall_ms = (time.perf_counter() - t0) * 1e3
    launches = ctx.launches - launches0
    kv_bytes = int(sum(lens)) * cfg["layers"] * 2 * cfg["kv_heads"] * cfg["head_dim"] * 2
    # one prefill chunk on a fresh sequence
    pre = model.new_sequence()
    ids = gen_token_ids(seed, 2, prefill_chunk, cfg["vocab"])
    t0 = time.perf_counter()
    model.prefill(pre, ids)
    prefill_ms = (time.perf_counter() - t0) * 1e3
    ctx.check_device_error()
    out = {"metric": "serving_decode_tokens_per_s", "value": batch * steps / (ms / 1e3), "unit": "tokens/s", "steps": steps,
           "ms_per_step": ms / steps, "dtype": "bf16", "data": "synthetic",
           "config": {"workload": "llama3-8b-shape Q8_0, batch %d decode, ctx U[512,4096], paged bf16 KV page 16, pages shuffled (seed %d)" % (batch, seed),
                      "layers": cfg["layers"]},
           "e2e": {"value": batch * steps / (wall_ms / 1e3), "unit": "tokens/s", "h2d_bytes_per_step": 16 * batch, "d2h_bytes_per_step": 4 * batch},
           "gpu_launches": int(launches),
           "bytes_per_step": {"kv": kv_bytes, "weights": model.weight_bytes},
           "achieved_GBps": (kv_bytes + model.weight_bytes) / (ms / steps) / 1e6,
           "prefill": {"tokens": prefill_chunk, "ms": prefill_ms, "tokens_per_s": prefill_chunk / (prefill_ms / 1e3)}}
    model.destroy()
    return out


def tp70b(ctx: Context, comm, rank, world, steps, warmup, batch=16, prompt=1024, layers=None, seed=3):
    """Llama-3-70B-shape Q8_0 decoder, tensor-parallel over `world` GPUs (NCCL all-reduce after o_proj and down_proj),
    bf16 activations and KV, `batch` sequences, `prompt`-token prompts, then decode steps."""
    cfg = dict(LLAMA3_70B)
    if layers:
        cfg["layers"] = layers
    model = Llama(ctx, cfg, act_dtype=BF16, kv_dtype=BF16, page_size=16, max_seqs=batch, max_ctx=prompt + warmup + steps + 24,
                  tp_rank=rank, tp_size=world)
    if world > 1:
        model.set_comm(comm)
    model.generate_weights(seed)
    seqs, toks = [], []
    t0 = time.perf_counter()
    for b in range(batch):
        s = model.new_sequence()
        seqs.append(s)
        toks.append(model.prefill(s, gen_token_ids(seed, 10 + b, prompt, cfg["vocab"])))
    ctx.sync()
    prefill_s = time.perf_counter() - t0
    def timed_steps(toks):
        for _ in range(max(warmup, 3)):
            toks = model.decode(seqs, toks)
        ctx.sync()
        ctx.timer_start(5)
        for _ in range(steps):
            toks = model.decode(seqs, toks)
        ctx.timer_stop(5)
        return toks, ctx.timer_ms(5)

    toks, ms = timed_steps(toks)
    ms_nccl, exchange = None, "none (one GPU)"
    if world > 1:
        # the same steps with the row-parallel sums done by one kernel over peer-mapped memory instead of NCCL + add
        ms_nccl, exchange = ms, "NCCL all-reduce + add"
        try:
            model.set_peer_allreduce(True)
            toks, ms = timed_steps(toks)
            exchange = "one kernel over peer-mapped memory (sum over ranks + residual + RMSNorm)"
        except BlumError as e:
            exchange = "NCCL all-reduce + add (peer mapping failed: %s)" % e.message
    ctx.check_device_error()
    # the exchanges of one step alone, back to back on the same stream: 2 per layer of [batch, hidden] bf16, as NCCL
    # all-reduce + add and as the one-kernel exchange over peer memory (which also normalises)
    ar_ms, px_ms = 0.0, None
    if world > 1:
        n_ex, H = 2 * cfg["layers"], cfg["hidden"]
        buf, res = ctx.alloc(batch * H * 2), ctx.alloc(batch * H * 2)
        ctx._check(ctx.lib.blum_memset(ctx.h, buf.ptr, 0, batch * H * 2))
        ctx._check(ctx.lib.blum_memset(ctx.h, res.ptr, 0, batch * H * 2))

        def loop(fn, timer):
            for timed in (False, True):
                if timed:
                    ctx.sync()
                    ctx.timer_start(timer)
                for i in range(n_ex * (4 if timed else 1)):
                    fn(i)
            ctx.timer_stop(timer)
            return ctx.timer_ms(timer) / 4

        def nccl_exchange(i):
            comm.allreduce_sum(buf, batch * H, BF16)
            ctx._check(ctx.lib.blum_add(ctx.h, res.ptr, buf.ptr, res.ptr, BF16, batch * H))
        ar_ms = loop(nccl_exchange, 6)
        if model.peer_allreduce:
            peer = C.c_void_p()
            ctx._check(ctx.lib.blum_peer_create(ctx.h, comm.h, H * 2, batch, 30000, C.byref(peer)))
            px_ms = loop(lambda i: ctx._check(ctx.lib.blum_allreduce_fused(ctx.h, peer, i % 2, res.ptr, None, cfg["rms_eps"], buf.ptr, res.ptr,
                                                                           BF16, batch, H)), 7)
            ctx.check_device_error()
            ctx._check(ctx.lib.blum_peer_destroy(ctx.h, peer))
        buf.free()
        res.free()
    out = {"metric": "tp_decode_tokens_per_s", "value": batch * steps / (ms / 1e3), "unit": "tokens/s", "n_gpus": world, "steps": steps,
           "ms_per_step": ms / steps, "dtype": "bf16", "data": "synthetic", "scaling": "strong",
           "config": {"workload": "llama3-70b-shape Q8_0 TP%d, batch %d, prompt %d (seed %d)" % (world, batch, prompt, seed),
                      "layers": cfg["layers"], "exchange": exchange, "exchanges": "2 per layer, %d B each" % (batch * cfg["hidden"] * 2)},
           "ms_per_step_nccl": None if ms_nccl is None else ms_nccl / steps,
           "weight_bytes_per_gpu": model.weight_bytes,
           "achieved_weight_GBps_per_gpu": model.weight_bytes / (ms / steps) / 1e6,
           "nccl_exchange_ms_per_step": ar_ms, "nccl_exchange_share": ar_ms / ((ms_nccl or ms) / steps),
           "peer_exchange_ms_per_step": px_ms, "peer_exchange_share": None if px_ms is None else px_ms / (ms / steps),
           "prefill": {"tokens": batch * prompt, "s": prefill_s, "tokens_per_s": batch * prompt / prefill_s}}
    model.destroy()
    return out


def moe_layer(ctx: Context, steps, warmup, tokens=(1, 64, 1024), hidden=2880, inter=2880, experts=32, top_k=4, seed=4):
    """One MoE feed-forward layer of the MXFP4 configuration: 32 experts, top-4, hidden = intermediate = 2880, router
    bias giving a Zipf(1.1)-like load; each token batch is captured in a CUDA graph and replayed."""
    from .moe import MoeFfn, Mxfp4Weight
    H, I, E = (hidden // 64) * 64, (inter // 64) * 64, experts       # the tensor-core path needs K % 64 == 0
    wg = Mxfp4Weight.generate(ctx, seed, 1, E, I, H)
    wu = Mxfp4Weight.generate(ctx, seed, 2, E, I, H)
    wd = Mxfp4Weight.generate(ctx, seed, 3, E, H, I)
    router = ctx.to_device(round_to_dtype(gen_normal(seed, 4, E * H, 0.02).reshape(E, H), BF16), BF16)
    bias = ctx.to_device((-1.1 * np.log(np.arange(1, E + 1))).astype(np.float32))
    layer = MoeFfn(ctx, H, I, E, top_k, router, bias, wg, wu, wd)
    rows = []
    for T in tokens:
        x = ctx.to_device(round_to_dtype(gen_normal(seed, 5, T * H).reshape(T, H), BF16), BF16)
        layer.plan(T)
        layer.enqueue(x)                                     # plain pass: sizes any workspace outside the capture
        ctx.sync()
        ctx._check(ctx.lib.blum_graph_begin(ctx.h))
        layer.enqueue(x)
        g, nk = C.c_void_p(), C.c_int()
        ctx._check(ctx.lib.blum_graph_end(ctx.h, C.byref(g), C.byref(nk)))
        for _ in range(max(warmup, 3)):
            ctx._check(ctx.lib.blum_graph_launch(ctx.h, g, nk.value))
        ctx.timer_start(6)
        for _ in range(steps):
            ctx._check(ctx.lib.blum_graph_launch(ctx.h, g, nk.value))
        ctx.timer_stop(6)
        ms = ctx.timer_ms(6) / steps
        ids = layer._plan["ids"].download(np.int32, T * top_k)
        hit = len(set(ids.tolist()))
        wbytes = hit * (wg.nbytes + wu.nbytes + wd.nbytes) // E
        flops = 2.0 * 3 * H * I * T * top_k
        rows.append({"tokens": T, "us": ms * 1e3, "experts_hit": hit, "weight_GBps": wbytes / ms / 1e6, "TFLOPs": flops / ms / 1e9,
                     "tokens_per_s": T / (ms / 1e3), "kernels": nk.value})
        ctx._check(ctx.lib.blum_graph_destroy(ctx.h, g))
    ctx.check_device_error()
    return {"metric": "moe_layer_tokens_per_s", "value": rows[-1]["tokens_per_s"], "unit": "tokens/s", "steps": steps, "dtype": "bf16",
            "data": "synthetic", "config": {"workload": "MXFP4 MoE layer, %d experts top-%d, hidden %d, intermediate %d (seed %d)" % (E, top_k, H, I, seed)},
            "per_batch": rows}


def moe_stack(ctx: Context, steps, warmup, layers=None, batches=(1, 16, 64), prompt=128, seed=4):
    """The whole MXFP4 mixture-of-experts decoder (24 layers of dense bf16 attention projections + the 32-expert top-4
    feed-forward, luminal_b200/moe_model.py): a prompt pass per sequence, then decode steps replayed from a CUDA graph per
    batch size.  The weight figure counts, per step, the dense projections once and the experts the step's tokens chose."""
    from .moe_model import MOE_CFG, MoeDecoder
    cfg = dict(MOE_CFG)
    if layers:
        cfg["layers"] = layers
    B_max = max(batches)
    model = MoeDecoder(ctx, cfg, max_seqs=B_max, max_ctx=prompt + 64, seed=seed)
    seqs, toks = [], []
    ctx.sync()
    t0 = time.perf_counter()
    for i in range(B_max):
        s = model.new_sequence()
        seqs.append(s)
        toks.append(model.prefill(s, gen_token_ids(seed, 50 + i, prompt, cfg["vocab"])))
    ctx.sync()
    prefill_s = time.perf_counter() - t0
    rows = []
    for B in batches:
        cur = list(toks[:B])
        for _ in range(max(warmup, 3)):
            cur = [int(t) for t in model.decode(seqs[:B], cur)]
        g, nk = model.step_graph(B)
        # timed: the captured step alone, replayed on fixed positions (the KV length does not grow inside the timed region)
        ctx.timer_start(6)
        for _ in range(steps):
            ctx._check(ctx.lib.blum_graph_launch(ctx.h, g, nk))
        ctx.timer_stop(6)
        ms = ctx.timer_ms(6) / steps
        hit = sum(len(set(w["ffn"]._plan["ids"].download(np.int32, B * model.k).tolist())) for w in model.layers)
        expert_bytes = 3 * model.I * model.H * 17 // 32                   # one expert's gate, up and down matrices
        dense = model.weight_bytes - model.L * model.E * expert_bytes
        rows.append({"batch": B, "ms_per_step": ms, "tokens_per_s": B / (ms / 1e3), "kernels": nk, "experts_hit_per_layer": hit / model.L,
                     "weight_GBps": (dense + hit * expert_bytes) / ms / 1e6})
    ctx.check_device_error()
    return {"metric": "moe_decode_tokens_per_s", "value": rows[-1]["tokens_per_s"], "unit": "tokens/s", "steps": steps, "dtype": "bf16",
            "data": "synthetic", "truncated_layers": bool(layers),
            "config": {"workload": "MXFP4 MoE decoder, %d layers, hidden %d, %d experts top-%d, prompt %d (seed %d)"
                       % (cfg["layers"], cfg["hidden"], cfg["experts"], cfg["top_k"], prompt, seed)},
            "prefill_tokens_per_s": B_max * prompt / prefill_s, "per_batch": rows}


def moe_ep(ctx: Context, comm, rank, world, steps, warmup, tokens_per_rank=1024, hidden=2880, inter=2880, experts=32, top_k=4, seed=4):
    """The same MoE layer with the experts sharded over `world` GPUs and `tokens_per_rank` tokens owned by every rank
    (dispatch and combine through the NCCL all-to-all).  Each call crosses the host once (per-expert counts), so the
    time is wall clock around `steps` calls, maximum over ranks taken by the caller's barrier discipline."""
    from .moe import ExpertParallelMoe, Mxfp4Weight
    H, I, E = (hidden // 64) * 64, (inter // 64) * 64, experts
    assert E % world == 0
    EL = E // world
    # this rank's experts: generated as their own stacked tensor (tensor ids keyed by rank; values are synthetic anyway)
    wg = Mxfp4Weight.generate(ctx, seed, 100 + rank, EL, I, H)
    wu = Mxfp4Weight.generate(ctx, seed, 200 + rank, EL, I, H)
    wd = Mxfp4Weight.generate(ctx, seed, 300 + rank, EL, H, I)
    router = ctx.to_device(round_to_dtype(gen_normal(seed, 4, E * H, 0.02).reshape(E, H), BF16), BF16)
    bias = ctx.to_device((-1.1 * np.log(np.arange(1, E + 1))).astype(np.float32))
    layer = ExpertParallelMoe(ctx, comm, H, I, E, top_k, router, bias, wg, wu, wd)
    T = tokens_per_rank
    x = ctx.to_device(round_to_dtype(gen_normal(seed, 5 + rank, T * H).reshape(T, H), BF16), BF16)
    for _ in range(max(warmup, 3)):
        layer.forward(x, T)
    ctx.sync()
    t0 = time.perf_counter()
    for _ in range(steps):
        layer.forward(x, T)
    ms = (time.perf_counter() - t0) * 1e3 / steps
    ctx.check_device_error()
    return {"metric": "moe_ep_layer_tokens_per_s", "value": world * T / (ms / 1e3), "unit": "tokens/s", "n_gpus": world, "steps": steps,
            "ms_per_step": ms, "dtype": "bf16", "data": "synthetic", "scaling": "weak",
            "config": {"workload": "MXFP4 MoE layer, %d experts top-%d over %d GPUs, %d tokens per GPU, hidden %d, intermediate %d (seed %d)"
                                   % (E, top_k, world, T, H, I, seed), "exchange": "NCCL send/recv all-to-all, counts through the host"}}


SWEEP_SHAPES = [(4096, 4096), (4096, 14336), (14336, 4096), (8192, 28672)]   # (K, N)
SWEEP_MS = [1, 8, 64, 512, 4096]


def sweep(ctx: Context, ms=None, shapes=None, dtype=BF16, iters=20, hbm_peak=6520.5, tc_peak=1646.8, l2_bytes=126 << 20):
    """Operator sweep of the Q8_0 matmul (seed 1): achieved HBM GB/s and TFLOP/s per (M, K, N).  Each shape is timed on
    the device over `iters` launches captured in one CUDA graph; the launches rotate through enough distinct weight
    tensors to exceed the L2, so every launch streams its weights from HBM."""
    import ctypes as C
    from .runtime import Q8Weight
    rows = []
    esz = 4 if dtype == F32 else 2
    for k, n in (shapes or SWEEP_SHAPES):
        wbytes = n * k * 34 // 32
        copies = max(2, min(16, (2 * l2_bytes + wbytes - 1) // wbytes))
        ws = [Q8Weight.generate(ctx, 1, 7000 + i, n, k) for i in range(copies)]
        arr = (C.c_void_p * copies)(*[w.h for w in ws])
        for m in (ms or SWEEP_MS):
            x = ctx.to_device(gen_normal(1, 5, m * k).reshape(m, k), dtype)
            y = ctx.alloc(m * n * esz)
            us = C.c_float()
            ctx._check(ctx.lib.blum_q8_0_matmul_timed(ctx.h, arr, copies, x.ptr, dtype, y.ptr, dtype, m, iters, C.byref(us)))
            t_ms = us.value / 1e3
            nbytes = wbytes + m * k * esz + m * n * esz
            flops = 2.0 * m * n * k
            rows.append({"K": k, "N": n, "M": m, "us": round(us.value, 2), "GBps": round(nbytes / t_ms / 1e6, 1),
                         "hbm_frac": round(nbytes / t_ms / 1e6 / hbm_peak, 3), "TFLOPs": round(flops / t_ms / 1e9, 2),
                         "tc_frac": round(flops / t_ms / 1e9 / tc_peak, 4)})
            x.free()
            y.free()
        for w in ws:
            w.free()
    ctx.check_device_error()
    return {"metric": "q8_0_matmul_operator_sweep", "unit": "us per launch", "dtype": {F32: "f32", BF16: "bf16"}.get(dtype, "f16"),
            "data": "synthetic", "config": {"workload": "Q8_0 matmul operator sweep (seed 1), bf16 in / f32 accumulate / bf16 out",
                                              "l2": "launches rotate through weight copies larger than L2"},
            "peaks": {"hbm_GBps": hbm_peak, "bf16_TFLOPs_burst": tc_peak}, "rows": rows}


def tp_parity(ctx: Context, comm, rank, world, golden_npz):
    """A small decoder that every tensor-parallel degree of one node divides, sharded over `world` ranks, seeded weights from
    the library's own generator, f32: its 8 greedy ids against the CPU oracle's (stored in the golden fixture)."""
    cfg = dict(layers=2, hidden=512, q_heads=8, kv_heads=8, head_dim=64, ffn=1024, vocab=512, rms_eps=1e-5, rope_theta=500000.0)
    model = Llama(ctx, cfg, act_dtype=F32, page_size=4, max_seqs=1, max_ctx=32, tp_rank=rank, tp_size=world)
    if world > 1:
        model.set_comm(comm)
    model.generate_weights(0)
    prompt = gen_token_ids(0, 1, 6, cfg["vocab"])
    got = [int(t) for t in model.greedy(prompt, 8)]
    want = np.load(golden_npz)["tp_greedy_ids_f32"].tolist()
    out = {"ids": got, "golden": want, "identical": got == want, "tp": world}
    if world > 1:
        try:
            model.set_peer_allreduce(True)
            peer = [int(t) for t in model.greedy(prompt, 8)]
            out["ids_peer_exchange"] = peer
            out["identical"] = out["identical"] and peer == want
        except BlumError as e:
            out["ids_peer_exchange"] = "peer mapping failed: %s" % e.message
    ctx.check_device_error()
    model.destroy()
    return out
