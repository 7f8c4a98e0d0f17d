"""A mixture-of-experts decoder stack on the library's entry points: per layer RMSNorm -> dense bf16 q/k/v projection ->
RoPE + paged GQA attention -> dense bf16 o projection -> residual; RMSNorm -> MXFP4 mixture-of-experts feed-forward ->
residual; then the final norm and a dense bf16 head.  luminal has no MoE model; the layer order is that of its llama
decoder (examples/llama/src/model.rs:171-248) with the feed-forward replaced by csrc/moe.cu, and the host-side style is the
reference's: one call per operator.  A decode step for a fixed batch size is captured in a CUDA graph."""
import ctypes as C

import numpy as np

from ._lib import BF16, F32
from .llama import KvCache
from .moe import MoeFfn, Mxfp4Weight
from .runtime import Context, gen_normal, round_to_dtype

# the MXFP4 configuration: 24 layers, hidden 2880, 64 query / 8 KV heads of 64, 32 experts top-4, expert intermediate 2880
MOE_CFG = dict(layers=24, hidden=2880, q_heads=64, kv_heads=8, head_dim=64, experts=32, top_k=4, inter=2880, vocab=32768,
               rms_eps=1e-5, rope_theta=150000.0)


class MoeDecoder:
    def __init__(self, ctx: Context, cfg, max_seqs=1, max_ctx=128, page_size=16, seed=4):
        self.ctx, self.cfg = ctx, dict(cfg)
        c = self.cfg
        self.H, self.nq, self.nkv, self.d = c["hidden"], c["q_heads"], c["kv_heads"], c["head_dim"]
        self.E, self.k, self.I, self.V, self.L = c["experts"], c["top_k"], c["inter"], c["vocab"], c["layers"]
        assert self.H % 64 == 0 and (self.nq * self.d) % 64 == 0 and self.I % 64 == 0, "the tensor-core kernels need K % 64 == 0"
        self.max_seqs, self.max_ctx = max_seqs, max_ctx
        pages_per_seq = (max_ctx + page_size - 1) // page_size
        self.kv = KvCache(ctx, self.L, self.nkv, self.d, page_size, max_seqs * pages_per_seq, max_seqs, pages_per_seq, BF16)
        self.qkv_rows = (self.nq + 2 * self.nkv) * self.d
        bf = lambda tid, n, k, std: ctx.to_device(round_to_dtype(gen_normal(seed, tid, n * k, std).reshape(n, k), BF16), BF16)
        self.embed = ctx.to_device(gen_normal(seed, 10, self.V * self.H, 0.02).reshape(self.V, self.H))
        self.head = bf(11, self.V, self.H, 0.02)
        self.out_norm = ctx.to_device((1 + 0.1 * gen_normal(seed, 12, self.H)).astype(np.float32))
        self.layers = []
        bias = (-1.1 * np.log(np.arange(1, self.E + 1))).astype(np.float32)          # a Zipf(1.1)-like expert load
        for l in range(self.L):
            t = 100 * (l + 1)
            lw = dict(attn_norm=ctx.to_device((1 + 0.1 * gen_normal(seed, t + 1, self.H)).astype(np.float32)),
                      ffn_norm=ctx.to_device((1 + 0.1 * gen_normal(seed, t + 2, self.H)).astype(np.float32)),
                      wqkv=bf(t + 3, self.qkv_rows, self.H, 0.02), wo=bf(t + 4, self.H, self.nq * self.d, 0.02),
                      router=bf(t + 5, self.E, self.H, 0.02), bias=ctx.to_device(bias))
            lw["ffn"] = MoeFfn(ctx, self.H, self.I, self.E, self.k, lw["router"], lw["bias"],
                               Mxfp4Weight.generate(ctx, seed, t + 6, self.E, self.I, self.H),
                               Mxfp4Weight.generate(ctx, seed, t + 7, self.E, self.I, self.H),
                               Mxfp4Weight.generate(ctx, seed, t + 8, self.E, self.H, self.I), keep_separate=False)
            self.layers.append(lw)
        self._graphs = {}
        self._bufs = {}
        self.max_splits = 8
        self.trace = None            # a list: prefill appends (layer, x_in, x_mid, x_out, routing ids) as host arrays

    # ---- buffers of a pass over R rows
    def _rows(self, R):
        if R not in self._bufs:
            ctx, a = self.ctx, lambda n: self.ctx.alloc(max(n, 16))
            scratch = ctx.lib.blum_attn_decode_scratch_bytes(R, self.nq, self.d, self.max_splits)
            self._bufs[R] = dict(ids=a(R * 4), seq=a(R * 4), pos=a(R * 4), ctxl=a(R * 4), x=a(R * self.H * 2), xn=a(R * self.H * 2),
                                 qkv=a(R * self.qkv_rows * 2), q=a(R * self.nq * self.d * 2), attn=a(R * self.nq * self.d * 2),
                                 o=a(R * self.H * 2), logits=a(R * self.V * 4), next=a(R * 4), scratch=a(scratch))
        return self._bufs[R]

    def _mm(self, w, n, k, x, y, rows, ydt=BF16):
        self.ctx._check(self.ctx.lib.blum_bf16_matmul(self.ctx.h, w.ptr, n, k, x.ptr, y.ptr, ydt, rows))

    def new_sequence(self):
        return self.kv.seq_alloc()

    def _upload(self, buf, values):
        buf.upload(np.ascontiguousarray(values, dtype=np.int32))

    def _head(self, b, x_rows, rows):
        ctx, lib, c = self.ctx, self.ctx.lib, self.cfg
        ctx._check(lib.blum_rmsnorm(ctx.h, x_rows, None, self.out_norm.ptr, c["rms_eps"], b["xn"].ptr, None, BF16, rows, self.H))
        self._mm(self.head, self.V, self.H, b["xn"], b["logits"], rows, F32)
        ctx._check(lib.blum_argmax(ctx.h, b["logits"].ptr, F32, rows, self.V, b["next"].ptr))

    # ---- prompt pass of one sequence (eager launches; buffers are kept per prompt length)
    def prefill(self, seq, ids, want_logits=False):
        ctx, lib, c = self.ctx, self.ctx.lib, self.cfg
        T, p0 = len(ids), self.kv.seq_len(seq)
        self.kv.seq_extend(seq, p0 + T)
        ctx._check(lib.blum_kv_sync_tables(ctx.h, self.kv.h))
        b = self._rows(T)
        self._upload(b["ids"], ids)
        self._upload(b["seq"], [seq] * T)
        self._upload(b["pos"], np.arange(p0, p0 + T))
        ctx._check(lib.blum_gather(ctx.h, self.embed.ptr, F32, self.V, self.H, b["ids"].ptr, T, b["x"].ptr, BF16))
        f = None
        for l, w in enumerate(self.layers):
            x_in = ctx.to_host(b["x"], BF16, T * self.H) if self.trace is not None and f is None else None
            # residual add of the previous layer's feed-forward folded into this norm
            ctx._check(lib.blum_rmsnorm(ctx.h, b["x"].ptr, f.ptr if f is not None else None, w["attn_norm"].ptr, c["rms_eps"], b["xn"].ptr,
                                        b["x"].ptr if f is not None else None, BF16, T, self.H))
            if self.trace is not None and x_in is None:
                x_in = ctx.to_host(b["x"], BF16, T * self.H)
            self._mm(w["wqkv"], self.qkv_rows, self.H, b["xn"], b["qkv"], T)
            ctx._check(lib.blum_rope_kv_append(ctx.h, self.kv.h, l, b["qkv"].ptr, BF16, self.nq, c["rope_theta"], b["seq"].ptr, b["pos"].ptr, T, b["q"].ptr))
            ctx._check(lib.blum_attn_prefill_paged(ctx.h, self.kv.h, l, b["q"].ptr, BF16, self.nq, seq, p0, T, b["attn"].ptr))
            self._mm(w["wo"], self.H, self.nq * self.d, b["attn"], b["o"], T)
            ctx._check(lib.blum_rmsnorm(ctx.h, b["x"].ptr, b["o"].ptr, w["ffn_norm"].ptr, c["rms_eps"], b["xn"].ptr, b["x"].ptr, BF16, T, self.H))
            keep = w["ffn"].plan(T)                                 # cached per prompt length: no allocation after the first prompt
            f = w["ffn"].enqueue(b["xn"])
            if self.trace is not None:
                x_mid = ctx.to_host(b["x"], BF16, T * self.H)
                ids_l = keep["ids"].download(np.int32, T * self.k)
                fo = ctx.to_host(f, BF16, T * self.H)
                self.trace.append(dict(layer=l, x_in=x_in.reshape(T, self.H), x_mid=x_mid.reshape(T, self.H), ids=ids_l.reshape(T, self.k),
                                       ffn_out=fo.reshape(T, self.H), p0=p0, seq=seq))
        ctx._check(lib.blum_add(ctx.h, b["x"].ptr, f.ptr, b["x"].ptr, BF16, T * self.H))
        last = C.c_void_p(b["x"].ptr + (T - 1) * self.H * 2)
        self._head(b, last, 1)
        tok = int(b["next"].download(np.int32, 1)[0])
        ctx.check_device_error()
        if want_logits:
            return tok, ctx.to_host(b["logits"], F32, self.V)
        return tok

    # ---- one decode step of B sequences: the launches of a step, replayed from a CUDA graph per batch size
    def _enqueue_step(self, B, splits):
        ctx, lib, c, b = self.ctx, self.ctx.lib, self.cfg, self._rows(B)
        ctx._check(lib.blum_gather(ctx.h, self.embed.ptr, F32, self.V, self.H, b["ids"].ptr, B, b["x"].ptr, BF16))
        f = None
        for l, w in enumerate(self.layers):
            ctx._check(lib.blum_rmsnorm(ctx.h, b["x"].ptr, f.ptr if f is not None else None, w["attn_norm"].ptr, c["rms_eps"], b["xn"].ptr,
                                        b["x"].ptr if f is not None else None, BF16, B, self.H))
            self._mm(w["wqkv"], self.qkv_rows, self.H, b["xn"], b["qkv"], B)
            ctx._check(lib.blum_rope_attn_decode_paged(ctx.h, self.kv.h, l, b["qkv"].ptr, BF16, self.nq, c["rope_theta"], b["seq"].ptr,
                                                       b["ctxl"].ptr, B, splits, b["scratch"].ptr, b["attn"].ptr))
            self._mm(w["wo"], self.H, self.nq * self.d, b["attn"], b["o"], B)
            ctx._check(lib.blum_rmsnorm(ctx.h, b["x"].ptr, b["o"].ptr, w["ffn_norm"].ptr, c["rms_eps"], b["xn"].ptr, b["x"].ptr, BF16, B, self.H))
            f = w["ffn"].enqueue(b["xn"])
        ctx._check(lib.blum_add(ctx.h, b["x"].ptr, f.ptr, b["x"].ptr, BF16, B * self.H))
        self._head(b, b["x"].ptr, B)

    def decode(self, seqs, toks, want_logits=False):
        ctx, lib = self.ctx, self.ctx.lib
        B = len(seqs)
        b = self._rows(B)
        lens = [self.kv.seq_len(s) for s in seqs]
        for s, n in zip(seqs, lens):
            self.kv.seq_extend(s, n + 1)
        ctx._check(lib.blum_kv_sync_tables(ctx.h, self.kv.h))
        self._upload(b["ids"], toks)
        self._upload(b["seq"], seqs)
        self._upload(b["ctxl"], [n + 1 for n in lens])
        # context splits of the attention kernel: one per 256 cached positions of the longest sequence, a power of two
        splits = 1
        while splits < self.max_splits and splits * 256 < max(lens) + 1:
            splits *= 2
        key = (B, splits)
        if key not in self._graphs:
            for w in self.layers:
                w["ffn"].plan(B)                               # (kept per batch size: makes it the layer's current plan)
            # (every layer's planned buffers are its own, so the captured step names them all)
            self._enqueue_step(B, splits)                  # plain pass (sizes workspaces outside the capture); the captured step
                                                           # below repeats it on the same positions with the same values
            ctx.sync()
            ctx._check(lib.blum_graph_begin(ctx.h))
            self._enqueue_step(B, splits)
            g, nk = C.c_void_p(), C.c_int()
            ctx._check(lib.blum_graph_end(ctx.h, C.byref(g), C.byref(nk)))
            self._graphs[key] = (g, nk.value)
        self._last_key = key
        g, nk = self._graphs[key]
        ctx._check(lib.blum_graph_launch(ctx.h, g, nk))
        out = b["next"].download(np.int32, B)
        ctx.check_device_error()
        if want_logits:
            return out, ctx.to_host(b["logits"], F32, B * self.V).reshape(B, self.V)
        return out

    def step_graph(self, B):
        """(graph handle, kernel count) of the B-row step captured last, for timing loops."""
        assert self._last_key[0] == B
        return self._graphs[self._last_key]

    @property
    def weight_bytes(self):
        dense = self.L * (self.qkv_rows * self.H + self.H * self.nq * self.d + self.E * self.H) * 2 + self.V * self.H * 2
        return dense + self.L * 3 * self.E * self.I * self.H * 17 // 32
