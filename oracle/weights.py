"""Seeded model weights for the CPU oracle (TEST INFRASTRUCTURE: used by tests/, __graft_entry__.smoke() and the CPU-baseline
legs of bench.py only).  Tensor ids are FNV-1a hashes of the GGUF tensor names (examples/llama/src/model.rs:250-259), the
same rule the library's own generator applies on the device, so both sides build the same model from a seed."""
import numpy as np


def fnv1a(name):
    h = 0xCBF29CE484222325
    for ch in name.encode():
        h ^= ch
        h = (h * 0x100000001B3) & 0xFFFFFFFFFFFFFFFF
    return h


TINY_CFG = dict(layers=2, hidden=256, q_heads=8, kv_heads=2, head_dim=64, ffn=512, vocab=320,
                rms_eps=1e-5, rope_theta=500000.0)
# the sibling decoders at test size: qwen (half-split rotary pairs, per-head q/k norm, tied head over a Q8_0 embedding table,
# eps 1e-6, theta 1e6: examples/qwen/src/model.rs) and phi (interleaved pairs, theta 1e4, as many kv heads as q heads:
# examples/phi/src/model.rs)
TINY_QWEN_CFG = dict(layers=2, hidden=256, q_heads=4, kv_heads=2, head_dim=128, ffn=512, vocab=320, rms_eps=1e-6,
                     rope_theta=1000000.0, rope_mode=1, qk_norm=1, tie_head=1, embed_q8=1)
TINY_PHI_CFG = dict(layers=2, hidden=256, q_heads=4, kv_heads=4, head_dim=64, ffn=512, vocab=320, rms_eps=1e-5,
                    rope_theta=10000.0)
# a decoder that divides by every tensor-parallel degree of one node (8 kv heads, ffn / 32 and vocabulary multiples of 8)
TP_CFG = dict(layers=2, hidden=512, q_heads=8, kv_heads=8, head_dim=64, ffn=1024, vocab=512, rms_eps=1e-5, rope_theta=500000.0)
LLAMA8B_CFG = dict(layers=32, hidden=4096, q_heads=32, kv_heads=8, head_dim=128, ffn=14336, vocab=128256,
                   rms_eps=1e-5, rope_theta=500000.0)


def tensor_shapes(cfg):
    """GGUF name -> (kind, shape) for the Llama layout of examples/llama/src/model.rs:250-259."""
    H, d = cfg["hidden"], cfg["head_dim"]
    out = {"token_embd.weight": ("q8" if cfg.get("embed_q8") or cfg.get("tie_head") else "f32", (cfg["vocab"], H)),
           "output_norm.weight": ("norm", (H,))}
    if not cfg.get("tie_head"):
        out["output.weight"] = ("q8", (cfg["vocab"], H))
    for i in range(cfg["layers"]):
        p = "blk.%d." % i
        out[p + "attn_norm.weight"] = ("norm", (H,))
        out[p + "ffn_norm.weight"] = ("norm", (H,))
        if cfg.get("qk_norm"):
            out[p + "attn_q_norm.weight"] = ("norm", (d,))
            out[p + "attn_k_norm.weight"] = ("norm", (d,))
        out[p + "attn_q.weight"] = ("q8", (cfg["q_heads"] * d, H))
        out[p + "attn_k.weight"] = ("q8", (cfg["kv_heads"] * d, H))
        out[p + "attn_v.weight"] = ("q8", (cfg["kv_heads"] * d, H))
        out[p + "attn_output.weight"] = ("q8", (H, cfg["q_heads"] * d))
        out[p + "ffn_gate.weight"] = ("q8", (cfg["ffn"], H))
        out[p + "ffn_up.weight"] = ("q8", (cfg["ffn"], H))
        out[p + "ffn_down.weight"] = ("q8", (H, cfg["ffn"]))
    return out


def make_weights(gen, cfg, seed, norm_random=False):
    """Seeded weights through generator module `gen` (the oracle's or the library's host generators).

    Q8_0 linears: int8 uniform [-127,127], f16 scale |N(0,0.02)|/127; f32 embedding N(0,0.02); norm weights 1.0
    (or 1 + 0.1 N(0,1) with norm_random, to exercise the weight multiply)."""
    w = {}
    for name, (kind, shape) in tensor_shapes(cfg).items():
        tid = fnv1a(name)
        if kind == "q8":
            n, k = shape
            w[name] = (gen.gen_q8_quants(seed, tid, n * k).reshape(n, k), gen.gen_q8_scales(seed, tid, n * k // 32).reshape(n, k // 32))
        elif kind == "f32":
            w[name] = gen.gen_normal(seed, tid, int(np.prod(shape)), 0.02).reshape(shape)
        else:
            w[name] = (1.0 + 0.1 * gen.gen_normal(seed, tid, shape[0], 1.0)).astype(np.float32) if norm_random else np.ones(shape, np.float32)
    return w
