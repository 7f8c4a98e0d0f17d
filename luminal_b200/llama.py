"""Host-side mirror of luminal's llama example on top of the C ABI.

`Llama` plays the role of examples/llama/src/main.rs: build the model, load (or generate) weights,
run the prompt pass, then the greedy decode loop.  `KvCache` wraps the paged KV pool that replaces
the per-layer `[1, kv_heads, pos, head_dim]` cache tensors of examples/llama/src/model.rs:85.
"""
import ctypes as C

import numpy as np

from ._lib import BF16, F16, F32, DTYPE_SIZE, LlamaCfg
from .runtime import Context, DeviceBuffer, pack_gguf_q8_0

LLAMA3_8B = dict(layers=32, hidden=4096, q_heads=32, kv_heads=8, head_dim=128, ffn=14336, vocab=128256,
                 rms_eps=1e-5, rope_theta=500000.0)
# examples/qwen/src/model.rs:6-14 (Qwen3-4B) and examples/phi/src/model.rs:5-12 (Phi-3-mini; its head_dim of 96 is not covered
# by the attention kernels here, which take 64 or 128)
QWEN3_4B = dict(layers=36, hidden=2560, q_heads=32, kv_heads=8, head_dim=128, ffn=9728, vocab=151936, rms_eps=1e-6,
                rope_theta=1000000.0, rope_mode=1, qk_norm=1, tie_head=1)
LLAMA3_70B = dict(layers=80, hidden=8192, q_heads=64, kv_heads=8, head_dim=128, ffn=28672, vocab=128256,
                  rms_eps=1e-5, rope_theta=500000.0)


class KvCache:
    """Paged KV pool + per-sequence page table (host-side allocator, device-side pages)."""

    def __init__(self, ctx: Context, layers, kv_heads, head_dim, page_size, num_pages, max_seqs, max_pages_per_seq,
                 dtype=F32, handle=None):
        self.ctx = ctx
        self.layers, self.kv_heads, self.head_dim, self.page_size = layers, kv_heads, head_dim, page_size
        self.num_pages, self.max_seqs, self.max_pages_per_seq, self.dtype = num_pages, max_seqs, max_pages_per_seq, dtype
        self.owner = handle is None
        if handle is None:
            h = C.c_void_p()
            ctx._check(ctx.lib.blum_kv_create(ctx.h, layers, kv_heads, head_dim, page_size, num_pages, max_seqs,
                                              max_pages_per_seq, dtype, C.byref(h)))
            handle = h.value
        self.h = handle

    def seq_alloc(self):
        s = C.c_int()
        self.ctx._check(self.ctx.lib.blum_kv_seq_alloc(self.ctx.h, self.h, C.byref(s)))
        return s.value

    def seq_extend(self, seq, new_len):
        self.ctx._check(self.ctx.lib.blum_kv_seq_extend(self.ctx.h, self.h, seq, new_len))

    def seq_free(self, seq):
        self.ctx._check(self.ctx.lib.blum_kv_seq_free(self.ctx.h, self.h, seq))

    def seq_set_pages(self, seq, pages, length):
        pages = np.ascontiguousarray(pages, dtype=np.int32)
        self.ctx._check(self.ctx.lib.blum_kv_seq_set_pages(self.ctx.h, self.h, seq, pages.ctypes.data, pages.size, length))

    def seq_len(self, seq):
        return self.ctx.lib.blum_kv_seq_len(self.h, seq)

    @property
    def free_pages(self):
        return self.ctx.lib.blum_kv_free_pages(self.h)

    def page_table(self):
        self.ctx._check(self.ctx.lib.blum_kv_sync_tables(self.ctx.h, self.h))
        out = np.empty(self.max_seqs * self.max_pages_per_seq, dtype=np.int32)
        self.ctx._check(self.ctx.lib.blum_memcpy_d2h(self.ctx.h, out.ctypes.data, self.ctx.lib.blum_kv_page_table_dev(self.h), out.nbytes))
        return out.reshape(self.max_seqs, self.max_pages_per_seq)

    def pool(self, np_dtype):
        """Whole pool as [layer, page, 2, kv_head, page_size, head_dim]."""
        nbytes = self.ctx.lib.blum_kv_pool_bytes(self.h)
        out = np.empty(nbytes // np.dtype(np_dtype).itemsize, dtype=np_dtype)
        self.ctx._check(self.ctx.lib.blum_memcpy_d2h(self.ctx.h, out.ctypes.data, self.ctx.lib.blum_kv_pool_dev(self.h), nbytes))
        return out.reshape(self.layers, self.num_pages, 2, self.kv_heads, self.page_size, self.head_dim)

    def append(self, layer, k: DeviceBuffer, v: DeviceBuffer, dtype, seq_ids, positions):
        s = self.ctx.to_device_raw(np.asarray(seq_ids, np.int32))
        p = self.ctx.to_device_raw(np.asarray(positions, np.int32))
        self.ctx._check(self.ctx.lib.blum_kv_append_paged(self.ctx.h, self.h, layer, k.ptr, v.ptr, dtype, s.ptr, p.ptr, len(seq_ids)))
        self.ctx.sync()

    def rope_append(self, layer, qkv: DeviceBuffer, dtype, q_heads, theta, seq_ids, positions):
        T = len(seq_ids)
        s = self.ctx.to_device_raw(np.asarray(seq_ids, np.int32))
        p = self.ctx.to_device_raw(np.asarray(positions, np.int32))
        q_out = self.ctx.alloc(max(T * q_heads * self.head_dim * DTYPE_SIZE[dtype], 16))
        self.ctx._check(self.ctx.lib.blum_rope_kv_append(self.ctx.h, self.h, layer, qkv.ptr, dtype, q_heads, float(theta),
                                                        s.ptr, p.ptr, T, q_out.ptr))
        self.ctx.sync()
        return q_out

    def gather_contiguous(self, layer, seq, which_v, out_dtype=F32):
        """[kv_heads, len, head_dim] in the reference's cache layout."""
        n = self.kv_heads * self.seq_len(seq) * self.head_dim
        out = self.ctx.alloc(max(n * DTYPE_SIZE[out_dtype], 16))
        self.ctx._check(self.ctx.lib.blum_kv_gather_contiguous(self.ctx.h, self.h, layer, seq, int(which_v), out.ptr, out_dtype))
        return self.ctx.to_host(out, out_dtype, n).reshape(self.kv_heads, -1, self.head_dim)

    def attn_decode(self, layer, q: DeviceBuffer, dtype, q_heads, seq_ids, ctx_lens, max_splits=1):
        B = len(seq_ids)
        s = self.ctx.to_device_raw(np.asarray(seq_ids, np.int32))
        c = self.ctx.to_device_raw(np.asarray(ctx_lens, np.int32))
        out = self.ctx.alloc(max(B * q_heads * self.head_dim * DTYPE_SIZE[dtype], 16))
        sb = self.ctx.lib.blum_attn_decode_scratch_bytes(B, q_heads, self.head_dim, max_splits)
        scratch = self.ctx.alloc(sb) if sb else None
        self.ctx._check(self.ctx.lib.blum_attn_decode_paged(self.ctx.h, self.h, layer, q.ptr, dtype, q_heads, s.ptr, c.ptr, B,
                                                           max_splits, scratch.ptr if scratch else None, out.ptr))
        self.ctx.sync()
        return out

    def attn_prefill(self, layer, q: DeviceBuffer, dtype, q_heads, seq, p, T):
        out = self.ctx.alloc(max(T * q_heads * self.head_dim * DTYPE_SIZE[dtype], 16))
        self.ctx._check(self.ctx.lib.blum_attn_prefill_paged(self.ctx.h, self.h, layer, q.ptr, dtype, q_heads, seq, p, T, out.ptr))
        self.ctx.sync()
        return out

    def destroy(self):
        if self.h and self.owner:
            self.ctx.lib.blum_kv_destroy(self.ctx.h, self.h)
        self.h = None


class Llama:
    """The decoder of examples/llama/src/model.rs with its weights, cache and decode loop on the device."""

    def __init__(self, ctx: Context, cfg: dict, act_dtype=F32, kv_dtype=None, page_size=16, max_seqs=1, max_ctx=128,
                 kv_pages=0, embed_q8=False, tp_rank=0, tp_size=1):
        """cfg may carry the sibling-decoder switches rope_mode (1 = half-split pairs, qwen), qk_norm and tie_head
        (examples/qwen/src/model.rs); a phi-style model is the Llama layout with rope_theta 10000 and kv_heads = q_heads."""
        self.ctx, self.cfg = ctx, dict(cfg)
        c = LlamaCfg()
        for k in ("layers", "hidden", "q_heads", "kv_heads", "head_dim", "ffn", "vocab", "rms_eps", "rope_theta"):
            setattr(c, k, cfg[k])
        c.act_dtype = act_dtype
        c.kv_dtype = act_dtype if kv_dtype is None else kv_dtype
        c.page_size, c.max_seqs, c.max_ctx, c.kv_pages = page_size, max_seqs, max_ctx, kv_pages
        c.embed_q8, c.tp_rank, c.tp_size = int(embed_q8), tp_rank, tp_size
        c.rope_mode, c.qk_norm, c.tie_head = int(cfg.get("rope_mode", 0)), int(cfg.get("qk_norm", 0)), int(cfg.get("tie_head", 0))
        self.c = c
        h = C.c_void_p()
        ctx._check(ctx.lib.blum_llama_create(ctx.h, C.byref(c), C.byref(h)))
        self.h = h.value
        pages_per_seq = (max_ctx + page_size - 1) // page_size
        self.kv = KvCache(ctx, cfg["layers"], cfg["kv_heads"] // tp_size, cfg["head_dim"], page_size,
                          kv_pages or max_seqs * pages_per_seq, max_seqs, pages_per_seq, c.kv_dtype,
                          handle=ctx.lib.blum_llama_kv(self.h))

    def set_comm(self, comm):
        """Communicator for the all-reduces of a tensor-parallel shard (tp_size > 1)."""
        self.ctx._check(self.ctx.lib.blum_llama_set_comm(self.ctx.h, self.h, comm.h))
        self.comm = comm

    def set_sampling(self, temperature=0.0, top_p=1.0, seed=0):
        """temperature 0: greedy (the reference's rule); otherwise temperature / top-p sampling keyed by (seed, sequence
        slot, position): the same seed reproduces the same tokens."""
        self.ctx._check(self.ctx.lib.blum_llama_set_sampling(self.ctx.h, self.h, float(temperature), float(top_p), int(seed)))

    def set_peer_allreduce(self, enable=True, timeout_ms=30000):
        """Tensor-parallel shards: sum row-parallel projections over peer-mapped memory in one kernel (steps of up to 64
        rows) instead of NCCL all-reduce + add.  Collective: every rank calls it.  Raises BlumError when the exchange
        areas cannot be mapped (then nothing changed and NCCL stays in use)."""
        self.ctx._check(self.ctx.lib.blum_llama_set_peer_allreduce(self.ctx.h, self.h, int(bool(enable)), int(timeout_ms)))

    @property
    def peer_allreduce(self):
        return bool(self.ctx.lib.blum_llama_peer_allreduce(self.h))

    def generate_weights(self, seed):
        self.ctx._check(self.ctx.lib.blum_llama_generate_weights(self.ctx.h, self.h, seed))

    def set_tensor(self, name, value):
        """value: f32 array, or (int8 [N,K], f16-bits [N,K/32]) for a Q8_0 tensor (full, unsharded tensor)."""
        if isinstance(value, tuple):
            raw = pack_gguf_q8_0(*value)
            self.ctx._check(self.ctx.lib.blum_llama_set_tensor(self.ctx.h, self.h, name.encode(), raw.ctypes.data, raw.nbytes, 1))
        else:
            a = np.ascontiguousarray(value, dtype=np.float32)
            self.ctx._check(self.ctx.lib.blum_llama_set_tensor(self.ctx.h, self.h, name.encode(), a.ctypes.data, a.nbytes, 0))

    def load_weights(self, weights: dict):
        for name, value in weights.items():
            self.set_tensor(name, value)

    def load_gguf(self, path):
        """Installs the decoder's tensors from a GGUF file (F32 and Q8_0 tensors, as the reference loader accepts)."""
        from .gguf import load_llama
        return load_llama(self, path)

    @property
    def weight_bytes(self):
        return self.ctx.lib.blum_llama_weight_bytes(self.h)

    def new_sequence(self):
        return self.kv.seq_alloc()

    def prefill(self, seq, ids, want_logits=False):
        ids = np.ascontiguousarray(ids, dtype=np.int32)
        nxt = C.c_int32()
        logits = np.empty(self.cfg["vocab"], np.float32) if want_logits else None
        self.ctx._check(self.ctx.lib.blum_llama_prefill(self.ctx.h, self.h, seq, ids.ctypes.data, ids.size, C.byref(nxt),
                                                       logits.ctypes.data if want_logits else None))
        return (nxt.value, logits) if want_logits else nxt.value

    def decode(self, seqs, ids, want_logits=False):
        seqs = np.ascontiguousarray(seqs, dtype=np.int32)
        ids = np.ascontiguousarray(ids, dtype=np.int32)
        out = np.empty(seqs.size, np.int32)
        logits = np.empty((seqs.size, self.cfg["vocab"]), np.float32) if want_logits else None
        self.ctx._check(self.ctx.lib.blum_llama_decode(self.ctx.h, self.h, seqs.ctypes.data, ids.ctypes.data, seqs.size,
                                                      out.ctypes.data, logits.ctypes.data if want_logits else None))
        return (out, logits) if want_logits else out

    def decode_loop(self, seq, first_token, steps):
        out = np.empty(steps, np.int32)
        self.ctx._check(self.ctx.lib.blum_llama_decode_loop(self.ctx.h, self.h, seq, int(first_token), steps, out.ctypes.data))
        return out

    def greedy(self, prompt_ids, steps):
        """Prompt pass + `steps` greedy tokens (examples/llama/src/main.rs:117-181)."""
        seq = self.new_sequence()
        tok = self.prefill(seq, prompt_ids)
        out = [tok]
        while len(out) < steps:
            tok = int(self.decode([seq], [tok])[0])
            out.append(tok)
        self.kv.seq_free(seq)
        return out

    def destroy(self):
        if self.h:
            self.ctx.lib.blum_llama_destroy(self.ctx.h, self.h)
            self.h = None
            self.kv.h = None
