#!/usr/bin/env python
"""Benchmark of the Q8_0 Llama-3-8B-shaped batch-1 decode path.

  python bench.py --gpus N --steps K --warmup W [--impl reference]

A "step" is one greedy decode token of one sequence (batch 1) after a 32-token prompt, with weights
generated from seed 0 (Q8_0 linears, f32 embedding and norms, f32 activations and KV cache).  With N > 1
every rank holds a full replica and decodes its own sequence (replicas only; no collective on the data path).
One JSON line is printed by rank 0.
"""
import argparse
import json
import os
import statistics
import subprocess
import sys
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

CFG = dict(layers=32, hidden=4096, q_heads=32, kv_heads=8, head_dim=128, ffn=14336, vocab=128256,
           rms_eps=1e-5, rope_theta=500000.0)
PROMPT_LEN = 32
SEED = 0
# DRAM bytes / algorithmic bytes of decode_stream_kernel, from the ncu capture summarised in profiles/decode_stream_8b_4layers.md
NCU_TRAFFIC_RATIO = 1.003    # DRAM bytes / algorithmic bytes of decode_stream_kernel (profiles/decode_stream_8b_4layers.md)


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        p = json.load(open(path))
        return float(p["hbm_gbs"]), "measured"
    return 6650.0, "fallback"


# ------------------------------------------------------------------ clocks
class ClockSampler:
    FIELDS = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, device):
        self.device, self.proc, self.path = device, None, "/tmp/blum_clocks_%d_%d.csv" % (os.getpid(), device)

    def start(self):
        try:
            self.f = open(self.path, "w")
            self.proc = subprocess.Popen(["nvidia-smi", "-i", str(self.device), "--query-gpu=" + self.FIELDS,
                                          "--format=csv,noheader,nounits", "-lms", "100"], stdout=self.f, stderr=subprocess.DEVNULL)
        except Exception:
            self.proc = None

    def stop(self):
        out = {"sm_mhz": None, "sm_max_mhz": None, "reasons": []}
        if self.proc is None:
            return out
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        self.f.close()
        sm, mx, reasons = [], [], set()
        for line in open(self.path):
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 9:
                continue
            try:
                sm.append(float(parts[1]))
                mx.append(float(parts[2]))
            except ValueError:
                continue
            for name, val in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), parts[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        if sm:
            out = {"sm_mhz": statistics.median(sm), "sm_max_mhz": max(mx), "reasons": sorted(reasons), "samples": len(sm)}
        try:
            os.remove(self.path)
        except OSError:
            pass
        return out


# ------------------------------------------------------------------ CPU baseline (oracle port)
WORKLOAD = "llama3-8b-shape Q8_0 batch-1 greedy decode after a 32-token prompt (seed 0)"


def cpu_decode_run(steps, warmup, single_thread_tokens=1):
    """The reference's CPU arithmetic for the whole workload, end to end and without extrapolation: the full 32-layer,
    vocabulary-128256 model (weights kept quantised), the 32-token prompt pass, `warmup` untimed and `steps` timed greedy
    decode tokens on every core this process may use, then `single_thread_tokens` more tokens on ONE thread (the reference
    executor is serial and its matmul crate is used without threading, so that is its faithful figure).
    Returns (cpu_baseline dict, seconds per token on all cores)."""
    from oracle import oracle as orc
    from oracle.weights import make_weights
    try:   # torchrun exports OMP_NUM_THREADS=1 to its ranks; the baseline is meant to use every core of this process
        cores = len(os.sched_getaffinity(0))
    except AttributeError:
        cores = os.cpu_count() or 1
    orc.set_num_threads(cores)
    w = make_weights(orc, CFG, SEED)
    model = orc.Llama(CFG, w, ctx_cap=PROMPT_LEN + warmup + steps + single_thread_tokens + 2)
    prompt = orc.gen_token_ids(SEED, 1, PROMPT_LEN, CFG["vocab"])
    t0 = time.perf_counter()
    tok = orc.argmax(model.forward(prompt))
    t_prefill = time.perf_counter() - t0
    for _ in range(warmup):
        tok = orc.argmax(model.forward([tok]))
    t0 = time.perf_counter()
    for _ in range(steps):
        tok = orc.argmax(model.forward([tok]))
    t_tok = (time.perf_counter() - t0) / steps
    orc.set_num_threads(1)
    t0 = time.perf_counter()
    for _ in range(single_thread_tokens):
        tok = orc.argmax(model.forward([tok]))
    t_one = (time.perf_counter() - t0) / max(single_thread_tokens, 1)
    orc.set_num_threads(cores)
    cb = {"value": 1.0 / t_tok, "unit": "tokens/s", "cores": orc.num_threads(), "kind": "port",
          "sample": "full 32-layer model: 32-token prompt pass, %d warm-up and %d timed greedy decode tokens on all cores "
                    "(no extrapolation)" % (warmup, steps),
          "prefill_tokens_per_s": PROMPT_LEN / t_prefill,
          "single_thread": {"value": 1.0 / t_one if single_thread_tokens else None, "unit": "tokens/s", "cores": 1,
                            "sample": "%d decode token(s) of the same run on one thread" % single_thread_tokens}}
    return cb, t_tok


def run_reference(args, rank):
    """Reference arm: the reference is Rust and cannot be built here, so its CPU arithmetic runs through the oracle port:
    every step is one real decode token of the full model on all host threads (rank 0 only)."""
    if rank != 0:
        return
    steps = max(1, min(args.steps, 64))            # one real token per step; 64 tokens bound the run to a few minutes
    cb, t_tok = cpu_decode_run(steps, max(1, min(args.warmup, 3)))
    v = cb["value"]
    line = {"impl": "reference", "metric": "decode_tokens_per_s", "value": v, "unit": "tokens/s", "n_gpus": args.gpus,
            "steps": steps, "warmup": max(1, min(args.warmup, 3)), "ms_per_step": 1000.0 * t_tok, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": {"workload": WORKLOAD},
            "cpu_baseline": cb, "e2e": {"value": v, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
    print(json.dumps(line), flush=True)


# ------------------------------------------------------------------ own arm
def kernel_table(ctx, model, lib, hbm_peak, layers):
    """Per-kernel achieved HBM bandwidth of the operator-level Q8_0 GEMV entry points on this model's matrices.  Each row
    captures one launch per layer (32 different matrices: 0.6 to 4 GB per pass, so no launch finds its weights in L2) in a
    CUDA graph and times replays of it with CUDA events, so the figures are device time, not host launch time."""
    import ctypes as C
    from luminal_b200 import F32
    H, F = CFG["hidden"], CFG["ffn"]
    x = ctx.to_device(np.random.default_rng(0).standard_normal(F).astype(np.float32))
    y = ctx.alloc(max(F, CFG["vocab"]) * 4 + 1024)
    eps = CFG["rms_eps"]
    rows = {}

    def timed(name, launch, bytes_per_launch, count, reps=5):
        launch(0)                      # anything lazy (function attributes) happens outside the capture
        ctx.sync()
        ctx._check(lib.blum_graph_begin(ctx.h))
        for l in range(count):
            launch(l)
        g, nk = C.c_void_p(), C.c_int()
        ctx._check(lib.blum_graph_end(ctx.h, C.byref(g), C.byref(nk)))
        ctx._check(lib.blum_graph_launch(ctx.h, g, nk.value))
        ctx.flush_l2()                 # the first timed launch must not find its weights in L2
        ctx.sync()
        ctx.timer_start(3)
        for _ in range(reps):
            ctx._check(lib.blum_graph_launch(ctx.h, g, nk.value))
        ctx.timer_stop(3)
        ms = ctx.timer_ms(3) / (count * reps)
        ctx._check(lib.blum_graph_destroy(ctx.h, g))
        rows[name] = {"launches_per_step": count if count > 1 else 1, "us": ms * 1e3, "bytes": bytes_per_launch,
                      "GBps": bytes_per_launch / ms / 1e6, "frac_of_peak": bytes_per_launch / ms / 1e6 / hbm_peak}

    L = layers
    W = lambda l, which: lib.blum_llama_layer_weight(model.h, l, which)
    NW = lambda l, which: lib.blum_llama_norm_weight(model.h, l, which)
    qkv_rows = (CFG["q_heads"] + 2 * CFG["kv_heads"]) * CFG["head_dim"]
    timed("qkv_gemv_norm", lambda l: ctx._check(lib.blum_q8_0_matmul_fused(ctx.h, W(l, 0), x.ptr, F32, NW(l, 0), eps, None, y.ptr, F32, 1)),
          qkv_rows * H * 34 // 32 + H * 4 * 2 + qkv_rows * 4, L)
    timed("o_gemv_residual", lambda l: ctx._check(lib.blum_q8_0_matmul_fused(ctx.h, W(l, 1), x.ptr, F32, None, 0.0, y.ptr, y.ptr, F32, 1)),
          H * H * 34 // 32 + H * 4 + H * 8, L)
    timed("gate_up_gemv_swiglu", lambda l: ctx._check(lib.blum_q8_0_matmul_swiglu(ctx.h, W(l, 2), W(l, 3), x.ptr, F32, NW(l, 1), eps, y.ptr, F32, 1)),
          2 * F * H * 34 // 32 + H * 4 * 2 + F * 4, L)
    timed("down_gemv_residual", lambda l: ctx._check(lib.blum_q8_0_matmul_fused(ctx.h, W(l, 4), x.ptr, F32, None, 0.0, y.ptr, y.ptr, F32, 1)),
          H * F * 34 // 32 + F * 4 + H * 8, L)
    # the head is one 558 MB matrix: two launches per replay with the L2 flushed by its own size
    timed("head_gemv_norm", lambda l: ctx._check(lib.blum_q8_0_matmul_fused(ctx.h, W(0, 5), x.ptr, F32, NW(0, 2), eps, None, y.ptr, F32, 1)),
          CFG["vocab"] * H * 34 // 32 + H * 8 + CFG["vocab"] * 4, 1, reps=8)
    tot_b = sum(r["bytes"] * r["launches_per_step"] for r in rows.values())
    tot_us = sum(r["us"] * r["launches_per_step"] for r in rows.values())
    rows["all_gemv_launches_of_a_step"] = {"launches_per_step": sum(r["launches_per_step"] for r in rows.values()), "us": tot_us,
                                           "bytes": tot_b, "GBps": tot_b / tot_us / 1e3, "frac_of_peak": tot_b / tot_us / 1e3 / hbm_peak}
    return rows


def tp_leg(ctx, rank, world, dist):
    """The 70B-shape decoder sharded over the job's N GPUs (N = 1: unsharded, the denominator of the scaling efficiency):
    batch 16, 1024-token prompts, bf16 activations and KV, all-reduce after o_proj and down_proj; and a small decoder's
    greedy ids under the same sharding against the CPU oracle's golden ids."""
    from luminal_b200 import workloads
    comm = None
    if world > 1:
        import torch
        from luminal_b200.dist import Comm
        uid = torch.zeros(128, dtype=torch.uint8, device="cuda")
        if rank == 0:
            uid.copy_(torch.frombuffer(bytearray(Comm.unique_id()), dtype=torch.uint8))
        dist.broadcast(uid, 0)
        comm = Comm(ctx, world, rank, bytes(uid.cpu().numpy().tobytes()), init_timeout_ms=60000)
    out = {"tp_parity": workloads.tp_parity(ctx, comm, rank, world, os.path.join(ROOT, "tests", "golden", "oracle_vectors.npz"))}
    rec = workloads.tp70b(ctx, comm, rank, world, steps=8, warmup=3)
    keep = ("value", "unit", "ms_per_step", "steps", "weight_bytes_per_gpu", "achieved_weight_GBps_per_gpu", "ms_per_step_nccl",
            "nccl_exchange_ms_per_step", "nccl_exchange_share", "peer_exchange_ms_per_step", "peer_exchange_share", "prefill", "config", "dtype")
    out["tp70b"] = {k: rec[k] for k in keep if k in rec}
    out["tp70b"]["tp"] = world
    if comm is not None:
        comm.destroy()
    return out


def run_own(args, rank, world, local_rank):
    from luminal_b200 import F32, Context
    from luminal_b200.llama import Llama
    from luminal_b200.runtime import gen_token_ids

    dist = None
    if world > 1:
        import torch
        import torch.distributed as dist
        torch.cuda.set_device(local_rank)
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))

    def barrier():
        if dist is not None:
            dist.barrier()

    def max_over_ranks(v):
        if dist is None:
            return v
        import torch
        t = torch.tensor([v], dtype=torch.float64, device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    ctx = Context(local_rank)
    lib = ctx.lib
    max_ctx = PROMPT_LEN + 2 * (args.warmup + args.steps) + 8
    cfg = dict(CFG, layers=args.layers) if args.layers else CFG      # --layers: a truncated model for profiler captures only
    model = Llama(ctx, cfg, act_dtype=F32, page_size=16, max_seqs=1, max_ctx=max_ctx)
    model.generate_weights(SEED)
    prompt = gen_token_ids(SEED, 1 + rank, PROMPT_LEN, CFG["vocab"])
    hbm_peak, peak_kind = measured_peaks()

    # ---- device-resident arm: token fed back on the device, K graph replays between two events
    seq = model.new_sequence()
    tok = model.prefill(seq, prompt)
    model.decode_loop(seq, tok, max(args.warmup, 3))          # warm-up (also captures the graph)
    ctx.sync()
    launches0 = ctx.launches
    sampler = ClockSampler(local_rank)
    sampler.start()
    barrier()
    ctx.sync()
    ctx.timer_start(0)
    toks = model.decode_loop(seq, int(tok), args.steps)
    ctx.timer_stop(0)
    ms_dev = ctx.timer_ms(0)
    ctx.sync()
    barrier()
    launches = ctx.launches - launches0
    ms_dev = max_over_ranks(ms_dev)
    # the dominant kernel alone (CUDA events on the launching stream): the last step launched again, without argmax / feedback
    stream_us = None
    if lib.blum_llama_decode_path(ctx.h, model.h) == 2:
        import ctypes as C
        us = C.c_float()
        ctx._check(lib.blum_llama_stream_kernel_us(ctx.h, model.h, max(args.steps, 8), C.byref(us)))
        stream_us = us.value
    ctx_at_timing = PROMPT_LEN + max(args.warmup, 3) + args.steps
    model.kv.seq_free(seq)

    # ---- end-to-end arm: one blum_llama_decode call per token, ids from pinned host memory, token read back.
    # The prompt pass is timed too (host ids in, first token out): prefill tokens/s of the 32-token prompt.
    seq = model.new_sequence()
    ctx.sync()
    t0 = time.perf_counter()
    tok = model.prefill(seq, prompt)
    ms_prefill = max_over_ranks((time.perf_counter() - t0) * 1e3)
    for _ in range(max(args.warmup, 3)):
        tok = int(model.decode([seq], [tok])[0])
    barrier()
    ctx.sync()
    t0 = time.perf_counter()
    for _ in range(args.steps):
        tok = int(model.decode([seq], [tok])[0])
    ctx.sync()
    ms_e2e = (time.perf_counter() - t0) * 1e3
    barrier()
    clocks = sampler.stop()
    ms_e2e = max_over_ranks(ms_e2e)
    ctx.check_device_error()

    ktab = kernel_table(ctx, model, lib, hbm_peak, cfg["layers"]) if rank == 0 else None
    wbytes = model.weight_bytes
    model.destroy()
    # ---- tensor parallelism over the same N GPUs (the 70B configuration) and its parity check: every rank takes part
    tp = None
    if not args.no_tp:
        try:
            tp = tp_leg(ctx, rank, world, dist)
        except Exception as e:      # a secondary record must not cost the headline line
            tp = {"error": repr(e)}
    if rank != 0:
        if dist is not None:
            dist.destroy_process_group()
        return
    dom, allk = ktab["gate_up_gemv_swiglu"], ktab["all_gemv_launches_of_a_step"]
    tok_s = world * args.steps / (ms_dev / 1e3)
    # algorithmic bytes of one launch of the persistent decode kernel: every Q8_0 weight once, the norm weights, the
    # embedding row, and the cached K/V rows of the context (f32) read plus the new row written
    kv_bytes = cfg["layers"] * 2 * cfg["kv_heads"] * cfg["head_dim"] * 4 * (ctx_at_timing + 1)
    stream_bytes = wbytes + (2 * cfg["layers"] + 1) * cfg["hidden"] * 4 + cfg["hidden"] * 4 + kv_bytes
    if stream_us is not None:
        gbps = stream_bytes / (stream_us * 1e-6) / 1e9
        roof = {"bound": "hbm", "kernel": "decode_stream_kernel (the whole single-sequence step: %d phases, one launch)" % (5 * cfg["layers"] + 1),
                "achieved": gbps, "peak": hbm_peak, "peak_kind": peak_kind, "unit": "GB/s", "frac": gbps / hbm_peak,
                "launch_us": stream_us, "algorithmic_bytes": stream_bytes,
                # DRAM read + write of one launch, scaled by layer count from an ncu capture of a 4-layer model of the same widths
                # (profiles/decode_stream_8b_4layers.md): traffic / algorithmic bytes measured there, times this launch's bytes
                "traffic": int(stream_bytes * NCU_TRAFFIC_RATIO) if NCU_TRAFFIC_RATIO else None,
                "traffic_kind": "scaled from an ncu capture of the same kernel on a 4-layer model of the same widths",
                "frac_of_8TBps": gbps / 8000.0}
    else:
        roof = {"bound": "hbm", "kernel": "q8_gemv_i8_kernel, all launches of one decode step (M=1)",
                "achieved": allk["GBps"], "peak": hbm_peak, "peak_kind": peak_kind, "unit": "GB/s", "frac": allk["GBps"] / hbm_peak,
                "traffic": int(dom["bytes"] * 62.54 / 62.46), "traffic_kind": "per launch of the gate/up instance, scaled from an ncu capture",
                "frac_of_8TBps": allk["GBps"] / 8000.0}
    line = {
        "metric": "decode_tokens_per_s", "value": tok_s, "unit": "tokens/s", "n_gpus": world, "steps": args.steps,
        "warmup": max(args.warmup, 3), "ms_per_step": ms_dev / args.steps, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": WORKLOAD,
                   "parallelism": "replicas x%d" % world, "l2": "weights per step (7.97 GB) exceed L2 (126 MB)",
                   "kv": "f32 paged, page 16", "activations": "f32",
                   "decode_path": "persistent kernel" if stream_us is not None else "per-op kernels in a CUDA graph"},
        "e2e": {"value": world * args.steps / (ms_e2e / 1e3), "unit": "tokens/s", "h2d_bytes_per_step": 16, "d2h_bytes_per_step": 8},
        "gpu_launches": int(launches),
        "clocks": clocks,
        "prefill": {"tokens": PROMPT_LEN, "ms": ms_prefill, "tokens_per_s": world * PROMPT_LEN / (ms_prefill / 1e3),
                    "how": "blum_llama_prefill with host ids, wall clock around the call (H2D of ids and D2H of the first token inside)"},
        "roofline": roof,
        "step_roofline": {"weight_bytes_per_token": wbytes, "achieved_GBps": wbytes * args.steps / (ms_dev / 1e3) / 1e9,
                          "frac_of_measured": wbytes * args.steps / (ms_dev / 1e3) / 1e9 / hbm_peak,
                          "frac_of_8TBps": wbytes * args.steps / (ms_dev / 1e3) / 1e9 / 8000.0},
        # the operator-level GEMV entry points on the same matrices (what a luminal operator would call one by one)
        "kernels": ktab,
    }
    if args.layers:
        line["config"]["truncated"] = "%d layers instead of %d: a profiler case, not a bench value" % (cfg["layers"], CFG["layers"])
    if tp is not None:
        line["tp70b"] = tp.get("tp70b", tp)
        line["tp_parity"] = tp.get("tp_parity")
    if not args.no_cpu and world == 1:
        try:
            line["cpu_baseline"] = cpu_decode_run(8, 1)[0]
        except Exception as e:   # the baseline is a reported number, never a reason to lose the GPU line
            line["cpu_baseline"] = {"value": None, "unit": "tokens/s", "cores": None, "kind": "port", "sample": "failed: %r" % (e,)}
    print(json.dumps(line), flush=True)
    if dist is not None:
        dist.destroy_process_group()


def run_secondary(args, rank, world, local_rank):
    """Secondary configurations (not the headline metric): one JSON line each."""
    from luminal_b200 import Context, workloads
    ctx = Context(local_rank)
    if args.workload == "serve64":
        if world == 1:
            print(json.dumps(workloads.serve64(ctx, args.steps, args.warmup, layers=args.layers)), flush=True)
        else:   # replicas: the 64 sequences are dealt out over the ranks, no data-path collective; slowest rank sets the time
            import torch
            import torch.distributed as dist
            dist.init_process_group("gloo")
            out = workloads.serve64(ctx, args.steps, args.warmup, layers=args.layers, rank=rank, world=world)
            t = torch.tensor([out["ms_per_step"], out["e2e"]["value"] and 64.0 * 1e3 / world / out["e2e"]["value"]], dtype=torch.float64)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            if rank == 0:
                out.update(n_gpus=world, scaling="strong", ms_per_step=float(t[0]), value=64.0 / (float(t[0]) / 1e3))
                out["e2e"]["value"] = 64.0 / (float(t[1]) / 1e3)
                out["config"]["parallelism"] = "replicas x%d, %d sequences each" % (world, 64 // world)
                print(json.dumps(out), flush=True)
            dist.barrier()
            dist.destroy_process_group()
    elif args.workload == "sweep":
        if rank == 0:
            peaks = json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json"))) if os.path.exists(os.path.join(ROOT, "MEASURED_PEAKS.json")) else {}
            ms = [int(v) for v in args.m.split(",")] if args.m else None
            shapes = [tuple(int(v) for v in sh.split("x")) for sh in args.shapes.split(",")] if args.shapes else None
            dt = {"bf16": 2, "f16": 1, "f32": 0}[args.dtype]
            print(json.dumps(workloads.sweep(ctx, ms=ms, shapes=shapes, dtype=dt, iters=max(args.steps, 5), hbm_peak=float(peaks.get("hbm_gbs", 6650.0)),
                                             tc_peak=float(peaks.get("bf16_tflops", 1590.0)))), flush=True)
    elif args.workload == "moe":
        if rank == 0:
            print(json.dumps(workloads.moe_layer(ctx, args.steps, args.warmup)), flush=True)
    elif args.workload == "moe_stack":
        if rank == 0:
            print(json.dumps(workloads.moe_stack(ctx, args.steps, args.warmup, layers=args.layers, prompt=args.prompt or 128)), flush=True)
    else:   # tp70b / moe_ep: one process per GPU under torchrun; the NCCL id travels through a file next to the rendezvous port
        from luminal_b200.dist import Comm
        path = "/tmp/blum_nccl_id_%s" % os.environ.get("MASTER_PORT", "0")
        if rank == 0 and os.path.exists(path):
            os.remove(path)
        if world > 1:
            import torch.distributed as dist
            dist.init_process_group("gloo")
            dist.barrier()
        comm = Comm(ctx, world, rank, Comm.exchange_id_via_file(path, rank))
        if args.workload == "moe_ep":
            out = workloads.moe_ep(ctx, comm, rank, world, args.steps, args.warmup)
        else:
            out = workloads.tp70b(ctx, comm, rank, world, args.steps, args.warmup, layers=args.layers, prompt=args.prompt or 1024)
        if rank == 0:
            print(json.dumps(out), flush=True)
        comm.destroy()
        if world > 1:
            dist.barrier()
            dist.destroy_process_group()
    ctx.close()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=64)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="own", choices=["own", "reference"])
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline leg")
    ap.add_argument("--no-tp", action="store_true", help="skip the tensor-parallel 70B record and its parity check")
    ap.add_argument("--workload", default="decode8b", choices=["decode8b", "serve64", "tp70b", "moe", "moe_stack", "moe_ep", "sweep"],
                    help="decode8b (default, the headline metric) or one of the secondary configurations")
    ap.add_argument("--layers", type=int, default=None, help="truncate the model to this many layers (small cases for profiler captures; the line says so)")
    ap.add_argument("--prompt", type=int, default=None, help="tp70b only: prompt length (default 1024)")
    ap.add_argument("--m", default=None, help="sweep only: comma-separated row counts (default 1,8,64,512,4096)")
    ap.add_argument("--shapes", default=None, help="sweep only: comma-separated KxN (default: the four shapes of the operator sweep)")
    ap.add_argument("--dtype", default="bf16", choices=["bf16", "f16", "f32"], help="sweep only: activation / output type")
    args = ap.parse_args()
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if args.impl == "reference":
        run_reference(args, rank)
        return
    if args.workload != "decode8b":
        run_secondary(args, rank, world, local_rank)
        return
    run_own(args, rank, world, local_rank)


if __name__ == "__main__":
    main()
