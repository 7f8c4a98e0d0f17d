"""ctypes + numpy front end of the CPU oracle (test infrastructure; see oracle.c).

Only tests/, __graft_entry__.smoke() and bench.py's CPU-baseline leg may import this module.
"""
import ctypes as C
import os
import subprocess

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
LIB = os.path.join(HERE, "liboracle.so")


def build(force=False):
    src = os.path.join(HERE, "oracle.c")
    if force or not os.path.exists(LIB) or os.path.getmtime(LIB) < os.path.getmtime(src):
        subprocess.run(["make", "-C", HERE, "-B", "liboracle.so"], check=True, capture_output=True)
    return LIB


_lib = None


def lib():
    global _lib
    if _lib is None:
        build()
        L = C.CDLL(LIB)
        L.orc_f16_to_f32.restype = C.c_float
        L.orc_f16_to_f32.argtypes = [C.c_uint16]
        L.orc_f32_to_f16.restype = C.c_uint16
        L.orc_f32_to_f16.argtypes = [C.c_float]
        L.orc_argmax.restype = C.c_int32
        L.orc_sample_top_p.restype = C.c_int32
        L.orc_sample_top_p.argtypes = [C.c_void_p, C.c_int64, C.c_float, C.c_float, C.c_uint64, C.c_uint64, C.c_uint64]
        L.orc_llama_forward.restype = C.c_int
        L.orc_num_threads.restype = C.c_int
        _lib = L
    return _lib


def _p(a):
    return a.ctypes.data_as(C.c_void_p)


def _i64(v):
    return C.c_int64(int(v))


def _u64(v):
    return C.c_uint64(int(v))


# ------------------------------------------------------------------ conversions
def f16_bits_to_f32(bits):
    return np.asarray(bits, dtype=np.uint16).view(np.float16).astype(np.float32)


def round_bf16(a):
    a = np.array(a, dtype=np.float32, copy=True).reshape(-1)
    lib().orc_round_bf16(_p(a), _i64(a.size))
    return a


def bf16_bits(a):
    a = np.ascontiguousarray(a, dtype=np.float32)
    u = a.view(np.uint32).astype(np.uint64)
    return ((u + 0x7FFF + ((u >> 16) & 1)) >> 16).astype(np.uint16)


# ------------------------------------------------------------------ generators
def gen_q8_quants(seed, tensor, n):
    out = np.empty(n, dtype=np.int8)
    lib().orc_gen_q8_quants(_u64(seed), _u64(tensor), _i64(n), _p(out))
    return out


def gen_q8_scales(seed, tensor, nblocks):
    out = np.empty(nblocks, dtype=np.uint16)
    lib().orc_gen_q8_scales(_u64(seed), _u64(tensor), _i64(nblocks), _p(out))
    return out


def gen_normal(seed, tensor, n, stddev=1.0):
    out = np.empty(n, dtype=np.float32)
    lib().orc_gen_normal(_u64(seed), _u64(tensor), _i64(n), C.c_float(stddev), _p(out))
    return out


def gen_token_ids(seed, tensor, n, vocab):
    out = np.empty(n, dtype=np.int32)
    lib().orc_gen_token_ids(_u64(seed), _u64(tensor), _i64(n), C.c_int32(vocab), _p(out))
    return out


# ------------------------------------------------------------------ Q8_0
def q8_pack(q, d_bits):
    q = np.ascontiguousarray(q, dtype=np.int8)
    n, k = q.shape
    d = np.ascontiguousarray(d_bits, dtype=np.uint16).reshape(n, k // 32)
    out = np.empty(n * (k // 32) * 34, dtype=np.uint8)
    lib().orc_q8_pack(_p(q), _p(d), _i64(n), _i64(k), _p(out))
    return out


def q8_unpack(gguf_bytes, n, k):
    b = np.ascontiguousarray(gguf_bytes, dtype=np.uint8)
    q = np.empty((n, k), dtype=np.int8)
    d = np.empty((n, k // 32), dtype=np.uint16)
    lib().orc_q8_unpack(_p(b), _i64(n), _i64(k), _p(q), _p(d))
    return q, d


def q8_dequant(gguf_bytes, n, k):
    b = np.ascontiguousarray(gguf_bytes, dtype=np.uint8)
    w = np.empty((n, k), dtype=np.float32)
    lib().orc_q8_dequant(_p(b), _i64(n), _i64(k), _p(w))
    return w


def q8_matmul(gguf_bytes, n, k, x):
    """Faithful form: f32 dequantised weights, ascending-k f32 accumulation."""
    b = np.ascontiguousarray(gguf_bytes, dtype=np.uint8)
    x = np.ascontiguousarray(x, dtype=np.float32).reshape(-1, k)
    y = np.empty((x.shape[0], n), dtype=np.float32)
    lib().orc_q8_matmul(_p(b), _i64(n), _i64(k), _p(x), _i64(x.shape[0]), _p(y))
    return y


def q8_matmul_fast(q, d_bits, x):
    q = np.ascontiguousarray(q, dtype=np.int8)
    n, k = q.shape
    d = np.ascontiguousarray(d_bits, dtype=np.uint16)
    x = np.ascontiguousarray(x, dtype=np.float32).reshape(-1, k)
    y = np.empty((x.shape[0], n), dtype=np.float32)
    lib().orc_q8_matmul_fast(_p(q), _p(d), _i64(n), _i64(k), _p(x), _i64(x.shape[0]), _p(y))
    return y


def gather_f32(table, ids_f32):
    table = np.ascontiguousarray(table, dtype=np.float32)
    ids = np.ascontiguousarray(ids_f32, dtype=np.float32).reshape(-1)
    out = np.empty((ids.size, table.shape[1]), dtype=np.float32)
    lib().orc_gather_f32(_p(table), _i64(table.shape[1]), _p(ids), _i64(ids.size), _p(out))
    return out


def q8_gather(gguf_bytes, dim, ids_f32):
    b = np.ascontiguousarray(gguf_bytes, dtype=np.uint8)
    ids = np.ascontiguousarray(ids_f32, dtype=np.float32).reshape(-1)
    out = np.empty((ids.size, dim), dtype=np.float32)
    lib().orc_q8_gather(_p(b), _i64(dim), _p(ids), _i64(ids.size), _p(out))
    return out


# ------------------------------------------------------------------ row-wise
def rmsnorm(x, weight, eps):
    x = np.ascontiguousarray(x, dtype=np.float32)
    rows, dim = x.reshape(-1, x.shape[-1]).shape
    y = np.empty_like(x)
    w = None if weight is None else np.ascontiguousarray(weight, dtype=np.float32)
    lib().orc_rmsnorm(_p(x), _p(w) if w is not None else None, C.c_float(eps), _i64(rows), _i64(dim), _p(y))
    return y


def softmax(x):
    x = np.ascontiguousarray(x, dtype=np.float32)
    rows, cols = x.reshape(-1, x.shape[-1]).shape
    y = np.empty_like(x)
    lib().orc_softmax(_p(x), _i64(rows), _i64(cols), _p(y))
    return y


def swiglu(gate, up):
    gate = np.ascontiguousarray(gate, dtype=np.float32)
    up = np.ascontiguousarray(up, dtype=np.float32)
    out = np.empty_like(gate)
    lib().orc_swiglu(_p(gate), _p(up), _i64(gate.size), _p(out))
    return out


def rope(x, positions, heads, head_dim, theta):
    """x [T, heads, head_dim] -> rotated copy."""
    x = np.array(x, dtype=np.float32, copy=True)
    pos = np.ascontiguousarray(positions, dtype=np.int32)
    lib().orc_rope(_p(x), _p(pos), _i64(pos.size), C.c_int(heads), C.c_int(head_dim), C.c_float(theta))
    return x


def triu(size, diagonal):
    out = np.empty((size, size), dtype=np.float32)
    lib().orc_triu(C.c_int(size), C.c_int(diagonal), _p(out))
    return out


def argmax(v):
    v = np.ascontiguousarray(v, dtype=np.float32).reshape(-1)
    return int(lib().orc_argmax(_p(v), _i64(v.size)))


def sample_top_p(v, temperature, top_p, seed, seq, pos):
    """Temperature / top-p sample of one row of logits (orc_sample_top_p: an integer-exact specification)."""
    v = np.ascontiguousarray(v, dtype=np.float32).reshape(-1)
    return int(lib().orc_sample_top_p(v.ctypes.data, v.size, float(temperature), float(top_p), int(seed), int(seq), int(pos)))


def attention(q, kc, vc, T, p, nq, nkv, d, ctx_cap):
    q = np.ascontiguousarray(q, dtype=np.float32)
    kc = np.ascontiguousarray(kc, dtype=np.float32)
    vc = np.ascontiguousarray(vc, dtype=np.float32)
    out = np.empty((T, nq * d), dtype=np.float32)
    lib().orc_attention(_p(q), _p(kc), _p(vc), _i64(T), _i64(p), C.c_int(nq), C.c_int(nkv), C.c_int(d), _i64(ctx_cap), _p(out))
    return out


# ------------------------------------------------------------------ Llama
class _Q8(C.Structure):
    _fields_ = [("q", C.c_void_p), ("d", C.c_void_p), ("N", C.c_int64), ("K", C.c_int64)]


class _Llama(C.Structure):
    _fields_ = [
        ("layers", C.c_int32), ("hidden", C.c_int32), ("q_heads", C.c_int32), ("kv_heads", C.c_int32),
        ("head_dim", C.c_int32), ("ffn", C.c_int32), ("vocab", C.c_int32),
        ("eps", C.c_float), ("theta", C.c_float),
        ("embed", C.c_void_p), ("out_norm", C.c_void_p), ("head", _Q8),
        ("attn_norm", C.POINTER(C.c_void_p)), ("ffn_norm", C.POINTER(C.c_void_p)),
        ("wq", C.POINTER(_Q8)), ("wk", C.POINTER(_Q8)), ("wv", C.POINTER(_Q8)), ("wo", C.POINTER(_Q8)),
        ("wgate", C.POINTER(_Q8)), ("wup", C.POINTER(_Q8)), ("wdown", C.POINTER(_Q8)),
        ("kcache", C.POINTER(C.c_void_p)), ("vcache", C.POINTER(C.c_void_p)),
        ("ctx_cap", C.c_int64), ("round_mode", C.c_int32),
        ("rope_mode", C.c_int32), ("qk_norm", C.c_int32), ("tie_head", C.c_int32),
        ("q_norm", C.POINTER(C.c_void_p)), ("k_norm", C.POINTER(C.c_void_p)), ("embed_q8", _Q8),
    ]


class Llama:
    """Llama decoder of examples/llama/src/model.rs on the CPU.

    weights: dict gguf_name -> f32 array (norms, embedding) or (int8 [N,K], f16-bits [N,K/32]) tuples.
    """

    def __init__(self, cfg, weights, ctx_cap, round_mode=0):
        self.cfg = dict(cfg)
        self.keep = []   # keeps numpy arrays alive
        L = cfg["layers"]
        m = _Llama()
        for k in ("layers", "hidden", "q_heads", "kv_heads", "head_dim", "ffn", "vocab"):
            setattr(m, k, cfg[k])
        m.eps, m.theta = cfg["rms_eps"], cfg["rope_theta"]
        m.ctx_cap, m.round_mode = ctx_cap, round_mode

        def f32(name):
            a = np.ascontiguousarray(weights[name], dtype=np.float32)
            self.keep.append(a)
            return a.ctypes.data

        def q8(name):
            q, d = weights[name]
            q = np.ascontiguousarray(q, dtype=np.int8)
            d = np.ascontiguousarray(d, dtype=np.uint16)
            self.keep += [q, d]
            return _Q8(q.ctypes.data, d.ctypes.data, q.shape[0], q.shape[1])

        m.rope_mode, m.qk_norm, m.tie_head = int(cfg.get("rope_mode", 0)), int(cfg.get("qk_norm", 0)), int(cfg.get("tie_head", 0))
        m.out_norm = f32("output_norm.weight")
        if isinstance(weights["token_embd.weight"], tuple):
            m.embed_q8 = q8("token_embd.weight")           # Q8_0 embedding table (QuantizedGather)
        else:
            m.embed = f32("token_embd.weight")
        if not m.tie_head:
            m.head = q8("output.weight")
        if m.qk_norm:
            self.q_norm = (C.c_void_p * L)(*[f32("blk.%d.attn_q_norm.weight" % i) for i in range(L)])
            self.k_norm = (C.c_void_p * L)(*[f32("blk.%d.attn_k_norm.weight" % i) for i in range(L)])
            m.q_norm, m.k_norm = self.q_norm, self.k_norm
        self.attn_norm = (C.c_void_p * L)(*[f32("blk.%d.attn_norm.weight" % i) for i in range(L)])
        self.ffn_norm = (C.c_void_p * L)(*[f32("blk.%d.ffn_norm.weight" % i) for i in range(L)])
        m.attn_norm, m.ffn_norm = self.attn_norm, self.ffn_norm
        for field, gg in (("wq", "attn_q"), ("wk", "attn_k"), ("wv", "attn_v"), ("wo", "attn_output"),
                          ("wgate", "ffn_gate"), ("wup", "ffn_up"), ("wdown", "ffn_down")):
            arr = (_Q8 * L)(*[q8("blk.%d.%s.weight" % (i, gg)) for i in range(L)])
            setattr(self, field, arr)
            setattr(m, field, arr)
        kv_elems = cfg["kv_heads"] * ctx_cap * cfg["head_dim"]
        self.k = [np.zeros(kv_elems, dtype=np.float32) for _ in range(L)]
        self.v = [np.zeros(kv_elems, dtype=np.float32) for _ in range(L)]
        self.kp = (C.c_void_p * L)(*[a.ctypes.data for a in self.k])
        self.vp = (C.c_void_p * L)(*[a.ctypes.data for a in self.v])
        m.kcache, m.vcache = self.kp, self.vp
        self.m = m
        self.pos = 0

    def forward(self, ids):
        """Runs the ids at the current position; returns the logits of the last one."""
        ids = np.ascontiguousarray(ids, dtype=np.int32)
        logits = np.empty(self.cfg["vocab"], dtype=np.float32)
        rc = lib().orc_llama_forward(C.byref(self.m), _p(ids), _i64(ids.size), _i64(self.pos), _p(logits))
        if rc != 0:
            raise RuntimeError("oracle llama forward failed (%d)" % rc)
        self.pos += ids.size
        return logits

    def greedy(self, prompt_ids, steps):
        """Prefill + `steps` greedy tokens, as examples/llama/src/main.rs:117-181.  Returns (ids, top-2 gaps)."""
        out, gaps = [], []
        logits = self.forward(prompt_ids)
        for _ in range(steps):
            tok = argmax(logits)
            top2 = np.partition(logits, -2)[-2:]
            gaps.append(float(top2[1] - top2[0]))
            out.append(tok)
            if len(out) == steps:
                break
            logits = self.forward([tok])
        return out, gaps


def num_threads():
    return lib().orc_num_threads()


def set_num_threads(n):
    lib().orc_set_num_threads(C.c_int(n))
