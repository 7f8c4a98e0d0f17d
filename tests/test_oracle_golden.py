"""Pins the CPU oracle: against the fixed-value vectors luminal's own tests carry, against numpy
float64 restatements, and against the committed golden fixtures.  No GPU needed."""
import json
import os

import numpy as np
import pytest

from helpers import TINY_CFG, TINY_PHI_CFG, TINY_QWEN_CFG, NumpyLlama, assert_parity, f16_bits_to_f64, make_weights

GOLD = os.path.join(os.path.dirname(__file__), "golden")


@pytest.fixture(scope="module")
def known():
    return json.load(open(os.path.join(GOLD, "reference_known_answers.json")))


def test_embedding_known_answer(orc, known):
    k = known["embedding"]
    w = np.array(k["weight_3x4"], np.float32).reshape(3, 4)
    assert np.array_equal(orc.gather_f32(w, k["ids_single"]).reshape(-1), np.array(k["expected_single"], np.float32))
    assert np.array_equal(orc.gather_f32(w, k["ids_batch_2x3"]).reshape(-1), np.array(k["expected_batch"], np.float32))


def test_gather_known_answer(orc, known):
    k = known["gather"]
    m = np.array(k["matrix_3x2"], np.float32).reshape(3, 2)
    assert np.array_equal(orc.gather_f32(m, k["indexes"]).reshape(-1), np.array(k["expected"], np.float32))


def test_triu_known_answer(orc, known):
    k = known["triu"]
    for diag in (-1, 0, 1):
        assert np.array_equal(orc.triu(k["size"], diag).reshape(-1), np.array(k["diag_%d" % diag], np.float32))


def test_causal_mask_is_triu_times_f16_min(orc):
    # attention_mask = triu(seq, 1) * f16::MIN padded left by prev_seq (examples/llama/src/model.rs:122-127)
    T, p = 4, 3
    mask = np.concatenate([np.zeros((T, p), np.float32), orc.triu(T, 1) * np.float32(-65504.0)], axis=1)
    j, t = np.arange(p + T)[None, :], np.arange(T)[:, None]
    assert np.array_equal(mask, np.where(j - p > t, np.float32(-65504.0), np.float32(0.0)))


@pytest.mark.parametrize("m", [1, 16])
def test_q8_matmul_reference_test_shape(orc, known, m):
    """The reference's Q8_0 tests: W[512,1024] int8 in 0..5 with unit scales, x uniform(-0.5,0.5),
    compared with the f32 matmul at 1e-3."""
    k = known["q8_matvec_shape"]
    rng = np.random.default_rng(5 + m)
    q = rng.integers(k["quant_range"][0], k["quant_range"][1], size=(k["N"], k["K"])).astype(np.int8)
    d = np.full((k["N"], k["K"] // 32), np.float16(1.0)).view(np.uint16)
    x = rng.uniform(-0.5, 0.5, size=(m, k["K"])).astype(np.float32)
    want = x.astype(np.float64) @ q.astype(np.float64).T
    got = orc.q8_matmul(orc.q8_pack(q, d), k["N"], k["K"], x)
    assert np.abs(got - want).max() < k["tolerance_abs"]
    assert np.abs(orc.q8_matmul_fast(q, d, x) - want).max() < k["tolerance_abs"]


def test_q8_block_layout(orc):
    """34-byte blocks: f16 scale then 32 int8 (crates/luminal_cuda/src/quantized.rs:30-33)."""
    q = (np.arange(64, dtype=np.int32) - 32).astype(np.int8).reshape(1, 64)
    d = np.array([[0x3C00, 0x4000]], np.uint16)   # 1.0, 2.0
    b = orc.q8_pack(q, d)
    assert b.size == 68
    assert b[0] == 0x00 and b[1] == 0x3C and b[34] == 0x00 and b[35] == 0x40
    assert np.array_equal(b[2:34].view(np.int8), q[0, :32]) and np.array_equal(b[36:68].view(np.int8), q[0, 32:])
    w = orc.q8_dequant(b, 1, 64)
    assert np.array_equal(w[0, :32], q[0, :32].astype(np.float32)) and np.array_equal(w[0, 32:], 2 * q[0, 32:].astype(np.float32))
    q2, d2 = orc.q8_unpack(b, 1, 64)
    assert np.array_equal(q2, q) and np.array_equal(d2, d)


def test_half_conversions_exhaustive(orc):
    L = orc.lib()
    allh = np.arange(65536, dtype=np.uint16)
    back = np.array([L.orc_f16_to_f32(int(h)) for h in allh], np.float32)
    ref = allh.view(np.float16).astype(np.float32)
    assert ((back == ref) | (np.isnan(back) & np.isnan(ref))).all()
    rng = np.random.default_rng(1)
    vals = np.concatenate([rng.standard_normal(4000).astype(np.float32) * s for s in (1e-8, 1e-5, 1e-3, 1, 100, 6e4)])
    with np.errstate(over="ignore"):
        want = vals.astype(np.float16).view(np.uint16)
    got = np.array([L.orc_f32_to_f16(float(v)) for v in vals], np.uint16)
    assert np.array_equal(got, want)


def test_generators_distribution(orc):
    q = orc.gen_q8_quants(1, 11, 1 << 18)
    assert q.min() == -127 and q.max() == 127 and abs(q.astype(np.float64).mean()) < 1.0
    counts = np.bincount(q.astype(np.int32) + 127, minlength=255)
    assert counts.min() > 0.8 * q.size / 255 and counts.max() < 1.2 * q.size / 255
    s = f16_bits_to_f64(orc.gen_q8_scales(1, 11, 1 << 16)) * 127
    assert abs(s.mean() - 0.02 * np.sqrt(2 / np.pi)) < 5e-4          # E|N(0,s)| = s*sqrt(2/pi)
    n = orc.gen_normal(1, 12, 1 << 16)
    assert abs(n.mean()) < 0.02 and abs(n.std() - 1) < 0.02
    ids = orc.gen_token_ids(0, 3, 4096, 128256)
    assert ids.min() >= 0 and ids.max() < 128256 and len(set(ids.tolist())) > 4000


def test_rmsnorm_against_float64(orc, known):
    k = known["rms_norm_shape"]
    rng = np.random.default_rng(0)
    x = rng.uniform(-0.5, 0.5, (k["rows"], k["dim"])).astype(np.float32)
    w = rng.uniform(-0.5, 0.5, k["dim"]).astype(np.float32)
    want = x.astype(np.float64) / np.sqrt((x.astype(np.float64) ** 2).mean(-1, keepdims=True) + k["eps"]) * w
    assert np.abs(orc.rmsnorm(x, w, k["eps"]) - want).max() < 1e-5
    assert np.abs(orc.rmsnorm(x, None, k["eps"]) * w - want).max() < 1e-5


def test_rope_against_float64(orc, known):
    k = known["rope_shape"]
    rng = np.random.default_rng(0)
    x = rng.uniform(-0.5, 0.5, (k["seq"], k["heads"], k["head_dim"])).astype(np.float32)
    got = orc.rope(x, np.arange(k["seq"]), k["heads"], k["head_dim"], k["theta"])
    d = k["head_dim"]
    inv = 1.0 / k["theta"] ** (np.arange(d // 2) * 2.0 / d)
    a = np.arange(k["seq"])[:, None, None] * inv[None, None, :]
    want = np.empty_like(x, dtype=np.float64)
    want[..., 0::2] = x[..., 0::2] * np.cos(a) - x[..., 1::2] * np.sin(a)
    want[..., 1::2] = x[..., 0::2] * np.sin(a) + x[..., 1::2] * np.cos(a)
    assert np.abs(got - want).max() < 1e-6
    # position 0 leaves the vector unchanged up to the sin(pi/2) rounding
    assert np.abs(got[0] - x[0]).max() < 1e-6


def test_softmax_swiglu_argmax(orc):
    rng = np.random.default_rng(2)
    x = rng.standard_normal((7, 129)).astype(np.float32) * 4
    e = np.exp(x.astype(np.float64) - x.max(-1, keepdims=True))
    assert np.abs(orc.softmax(x) - e / e.sum(-1, keepdims=True)).max() < 1e-6
    g, u = rng.standard_normal(1000).astype(np.float32), rng.standard_normal(1000).astype(np.float32)
    assert np.abs(orc.swiglu(g, u) - u * g / (1 + np.exp(-g.astype(np.float64)))).max() < 1e-6
    # greedy rule of examples/llama/src/main.rs:194-198: the last maximum wins; a NaN is replaced by what follows
    assert orc.argmax([1, 5, 3, 5, 2]) == 3
    assert orc.argmax([7, 7, 7]) == 2
    assert orc.argmax([1, np.nan, 0.5, 0.25]) == 2
    assert orc.argmax([3, 1, np.nan]) == 2


def test_attention_against_float64(orc):
    rng = np.random.default_rng(3)
    T, p, nq, nkv, d, cap = 3, 5, 4, 2, 16, 12
    q = rng.standard_normal((T, nq, d)).astype(np.float32)
    kc = rng.standard_normal((nkv, cap, d)).astype(np.float32)
    vc = rng.standard_normal((nkv, cap, d)).astype(np.float32)
    got = orc.attention(q, kc, vc, T, p, nq, nkv, d, cap).reshape(T, nq, d)
    for t in range(T):
        for h in range(nq):
            kh, vh = kc[h // 2, :p + T].astype(np.float64), vc[h // 2, :p + T].astype(np.float64)
            s = kh @ q[t, h].astype(np.float64) / np.sqrt(d)
            s[np.arange(p + T) - p > t] += -65504.0
            e = np.exp(s - s.max())
            assert np.abs(got[t, h] - (e / e.sum()) @ vh).max() < 1e-5


def test_llama_oracle_against_float64_model(orc):
    """Two independent restatements of examples/llama/src/model.rs agree: prefill of 5 tokens then 3 decode steps,
    KV cache carried across calls."""
    cfg = dict(TINY_CFG, layers=2)
    w = make_weights(orc, cfg, seed=7, norm_random=True)
    c_model = orc.Llama(cfg, w, ctx_cap=16)
    n_model = NumpyLlama(cfg, w)
    ids = orc.gen_token_ids(7, 1, 5, cfg["vocab"])
    a, b = c_model.forward(ids), n_model.forward(ids)
    assert_parity(a, b, max_abs=1e-4, rel=1e-4, what="prefill logits")
    for _ in range(3):
        tok = orc.argmax(a)
        assert tok == int(np.argmax(b))
        a, b = c_model.forward([tok]), n_model.forward([tok])
        assert_parity(a, b, max_abs=1e-4, rel=1e-4, what="decode logits")


@pytest.mark.parametrize("cfg", [TINY_QWEN_CFG, TINY_PHI_CFG], ids=["qwen", "phi"])
def test_sibling_decoders_against_float64_model(orc, cfg):
    """The qwen form (half-split rotary pairs, per-head q/k RMSNorm, tied head over a Q8_0 embedding table:
    examples/qwen/src/model.rs:52-105,233) and the phi form (interleaved pairs, theta 1e4, one kv head per q head:
    examples/phi/src/model.rs:50-70) of the C oracle against the independent float64 model."""
    w = make_weights(orc, cfg, seed=9, norm_random=True)
    c_model = orc.Llama(cfg, w, ctx_cap=16)
    n_model = NumpyLlama(cfg, w)
    ids = orc.gen_token_ids(9, 1, 5, cfg["vocab"])
    a, b = c_model.forward(ids), n_model.forward(ids)
    assert_parity(a, b, max_abs=1e-4, rel=1e-4, what="prefill logits")
    for _ in range(3):
        tok = orc.argmax(a)
        assert tok == int(np.argmax(b))
        a, b = c_model.forward([tok]), n_model.forward([tok])
        assert_parity(a, b, max_abs=1e-4, rel=1e-4, what="decode logits")


def test_sampler_specification(orc):
    """The temperature / top-p sampler of the oracle: frequencies follow softmax(l / T), the nucleus is the smallest set of
    most likely tokens reaching top_p (ties included), degenerate rows fall back to the greedy rule."""
    rng = np.random.default_rng(3)
    l = (rng.standard_normal(300) * 2).astype(np.float32)
    for temp in (1.0, 0.5):
        p = np.exp((l.astype(np.float64) - l.max()) / temp)
        p /= p.sum()
        n = 20000
        cnt = np.bincount([orc.sample_top_p(l, temp, 1.0, 9, 1, i) for i in range(n)], minlength=300)
        top = np.argsort(-p)[:8]
        assert np.abs(cnt[top] / n - p[top]).max() < 4 * np.sqrt(p[top].max() / n) + 1e-3
    order = np.argsort(-p)
    k = int(np.searchsorted(np.cumsum(p[order]), 0.6)) + 1
    seen = {orc.sample_top_p(l, 0.5, 0.6, 9, 0, i) for i in range(4000)}
    assert seen <= set(order[:k + 1].tolist()) and len(seen) >= k - 1
    assert {orc.sample_top_p(l, 1.0, 1e-9, 9, 0, i) for i in range(50)} == {int(np.argmax(l))}
    assert orc.sample_top_p(np.full(10, np.nan, np.float32), 1.0, 1.0, 1, 0, 0) == orc.argmax(np.full(10, np.nan, np.float32))
    inf = l.copy(); inf[7] = np.inf
    assert orc.sample_top_p(inf, 1.0, 1.0, 1, 0, 0) == 7
    assert orc.sample_top_p(l, 1.0, 0.9, 5, 2, 40) == orc.sample_top_p(l, 1.0, 0.9, 5, 2, 40)       # a pure function of its key


def test_golden_fixture_matches_oracle(orc):
    """tests/golden/oracle_vectors.npz (written by tests/golden/make_golden.py) is reproduced: integer results
    exactly, float results to 1e-6 relative (libm may differ in the last place between CPUs)."""
    g = np.load(os.path.join(GOLD, "oracle_vectors.npz"))
    from golden import make_golden
    fresh = make_golden.compute(orc)
    assert set(g.files) == set(fresh.keys())
    for k in g.files:
        if g[k].dtype.kind in "iu":
            assert np.array_equal(g[k], fresh[k]), k
        else:
            assert np.abs(g[k] - fresh[k]).max() <= 1e-6 * max(1.0, np.abs(g[k]).max()), k
