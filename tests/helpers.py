"""Shared helpers of the test-suite: tolerances, seeded model weights, a float64 numpy model."""
import numpy as np

# tolerance of the parity contract: per-kernel outputs within max-abs 1e-2 and relative 2e-2 of the f32 reference
MAX_ABS = 1e-2
REL = 2e-2


def assert_parity(got, want, max_abs=MAX_ABS, rel=REL, what=""):
    got = np.asarray(got, dtype=np.float64).reshape(-1)
    want = np.asarray(want, dtype=np.float64).reshape(-1)
    assert got.shape == want.shape, (what, got.shape, want.shape)
    assert np.isfinite(got).all(), "%s: non-finite output" % what
    err = np.abs(got - want).max() if got.size else 0.0
    scale = np.abs(want).max() if want.size else 0.0
    assert err <= max_abs, "%s: max-abs error %.3e > %.1e" % (what, err, max_abs)
    assert err <= rel * max(scale, 1e-30) or err <= 1e-6, "%s: relative error %.3e > %.1e (scale %.3e)" % (
        what, err / max(scale, 1e-30), rel, scale)
    return err


from oracle.weights import LLAMA8B_CFG, TINY_CFG, TP_CFG, TINY_PHI_CFG, TINY_QWEN_CFG, fnv1a, make_weights, tensor_shapes  # noqa: F401  (re-exported)


def f16_bits_to_f64(bits):
    return np.asarray(bits, dtype=np.uint16).view(np.float16).astype(np.float64)


def dequant64(qd):
    q, d = qd
    return q.astype(np.float64) * np.repeat(f16_bits_to_f64(d), 32, axis=1)


class NumpyLlama:
    """Independent float64 restatement of the decoder (cross-checks the C oracle in the CPU suite)."""

    def __init__(self, cfg, weights):
        self.cfg, self.w = cfg, weights
        L, nkv, d = cfg["layers"], cfg["kv_heads"], cfg["head_dim"]
        self.k = [np.zeros((nkv, 0, d)) for _ in range(L)]
        self.v = [np.zeros((nkv, 0, d)) for _ in range(L)]
        self.deq = {n: dequant64(v) for n, v in weights.items() if isinstance(v, tuple)}

    def _norm(self, x, w):
        return x / np.sqrt((x * x).mean(-1, keepdims=True) + self.cfg["rms_eps"]) * w

    def _rope(self, x, pos):
        d = self.cfg["head_dim"]
        inv = 1.0 / self.cfg["rope_theta"] ** (np.arange(d // 2) * 2.0 / d)
        a = pos[:, None, None] * inv[None, None, :]
        out = np.empty_like(x)
        if self.cfg.get("rope_mode", 0) == 1:          # half-split pairs (x[i], x[i + d/2]): examples/qwen/src/model.rs:52-77
            x0, x1 = x[..., :d // 2], x[..., d // 2:]
            out[..., :d // 2] = x0 * np.cos(a) - x1 * np.sin(a)
            out[..., d // 2:] = x1 * np.cos(a) + x0 * np.sin(a)
            return out
        x0, x1 = x[..., 0::2], x[..., 1::2]
        out[..., 0::2] = x0 * np.cos(a) - x1 * np.sin(a)
        out[..., 1::2] = x0 * np.sin(a) + x1 * np.cos(a)
        return out

    def forward(self, ids):
        c = self.cfg
        T, nq, nkv, d = len(ids), c["q_heads"], c["kv_heads"], c["head_dim"]
        p = self.k[0].shape[1]
        pos = np.arange(p, p + T, dtype=np.float64)
        emb = self.deq["token_embd.weight"] if "token_embd.weight" in self.deq else self.w["token_embd.weight"]
        x = emb[np.asarray(ids)].astype(np.float64)
        for l in range(c["layers"]):
            pre = "blk.%d." % l
            r = self._norm(x, self.w[pre + "attn_norm.weight"])
            q = (r @ self.deq[pre + "attn_q.weight"].T).reshape(T, nq, d)
            k = (r @ self.deq[pre + "attn_k.weight"].T).reshape(T, nkv, d)
            v = (r @ self.deq[pre + "attn_v.weight"].T).reshape(T, nkv, d)
            if c.get("qk_norm"):
                q = self._norm(q, self.w[pre + "attn_q_norm.weight"])
                k = self._norm(k, self.w[pre + "attn_k_norm.weight"])
            q, k = self._rope(q, pos), self._rope(k, pos)
            self.k[l] = np.concatenate([self.k[l], k.transpose(1, 0, 2)], axis=1)
            self.v[l] = np.concatenate([self.v[l], v.transpose(1, 0, 2)], axis=1)
            out = np.zeros((T, nq, d))
            for h in range(nq):
                kh, vh = self.k[l][h // (nq // nkv)], self.v[l][h // (nq // nkv)]
                s = q[:, h, :] @ kh.T / np.sqrt(d)
                j = np.arange(p + T)[None, :]
                s = s + np.where(j - p > np.arange(T)[:, None], -65504.0, 0.0)
                s = np.exp(s - s.max(-1, keepdims=True))
                out[:, h, :] = (s / s.sum(-1, keepdims=True)) @ vh
            x = x + out.reshape(T, nq * d) @ self.deq[pre + "attn_output.weight"].T
            r = self._norm(x, self.w[pre + "ffn_norm.weight"])
            g = r @ self.deq[pre + "ffn_gate.weight"].T
            u = r @ self.deq[pre + "ffn_up.weight"].T
            x = x + (u * (g / (1.0 + np.exp(-g)))) @ self.deq[pre + "ffn_down.weight"].T
        r = self._norm(x[-1:], self.w["output_norm.weight"])
        head = self.deq["token_embd.weight"] if c.get("tie_head") else self.deq["output.weight"]
        return (r @ head.T)[0]
