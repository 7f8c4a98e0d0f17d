"""The mixture-of-experts decoder stack (luminal_b200/moe_model.py): every layer against a numpy reference fed with the
layer's own input (a bf16 stack cannot be compared end to end: one expert choice that flips at a near-tie changes a whole
row), plus consistency of the three execution forms (prompt pass, single decode steps, batched captured steps)."""
import numpy as np
import pytest

from helpers import assert_parity
from luminal_b200 import BF16
from luminal_b200.moe_model import MoeDecoder
from luminal_b200.runtime import gen_normal, gen_token_ids, round_to_dtype

pytestmark = pytest.mark.gpu

CFG = dict(layers=3, hidden=256, q_heads=8, kv_heads=2, head_dim=64, experts=8, top_k=2, inter=128, vocab=512,
           rms_eps=1e-5, rope_theta=150000.0)
SEED = 4


def _host_layer(orc, cfg, l):
    from oracle import moe as omoe
    H, E, I = cfg["hidden"], cfg["experts"], cfg["inter"]
    qkv_rows, qd = (cfg["q_heads"] + 2 * cfg["kv_heads"]) * cfg["head_dim"], cfg["q_heads"] * cfg["head_dim"]
    t = 100 * (l + 1)
    bf = lambda tid, n, k: round_to_dtype(gen_normal(SEED, tid, n * k, 0.02).reshape(n, k), BF16)
    w = dict(attn_norm=(1 + 0.1 * gen_normal(SEED, t + 1, H)).astype(np.float32), ffn_norm=(1 + 0.1 * gen_normal(SEED, t + 2, H)).astype(np.float32),
             wqkv=bf(t + 3, qkv_rows, H), wo=bf(t + 4, H, qd), router=bf(t + 5, E, H),
             bias=(-1.1 * np.log(np.arange(1, E + 1))).astype(np.float32))
    for name, tid, (n, k) in (("wg", t + 6, (I, H)), ("wu", t + 7, (I, H)), ("wd", t + 8, (H, I))):
        w[name] = omoe.dequant_mxfp4(*omoe.gen_mxfp4(SEED, tid, E, n, k))
    return w


def test_every_layer_against_a_reference_fed_with_its_own_input(ctx, orc):
    from oracle import moe as omoe
    rb = omoe.round_bf16
    cfg = CFG
    nq, nkv, d, H, k = cfg["q_heads"], cfg["kv_heads"], cfg["head_dim"], cfg["hidden"], cfg["top_k"]
    m = MoeDecoder(ctx, cfg, max_seqs=2, max_ctx=64, seed=SEED)
    m.trace = []
    T = 24
    prompt = gen_token_ids(SEED, 1, T, cfg["vocab"])
    seq = m.new_sequence()
    m.prefill(seq, prompt)
    assert len(m.trace) == cfg["layers"]
    clear_total = 0
    for tr in m.trace:
        w = _host_layer(orc, cfg, tr["layer"])
        x_in, x_mid = tr["x_in"], tr["x_mid"]
        # ---- attention half from the layer's input
        xn = rb(orc.rmsnorm(x_in, w["attn_norm"], cfg["rms_eps"]))
        qkv = rb(xn.astype(np.float64) @ w["wqkv"].astype(np.float64).T)
        pos = np.arange(T)
        q = rb(orc.rope(qkv[:, :nq * d].reshape(T, nq, d), pos, nq, d, cfg["rope_theta"]))
        kk = rb(orc.rope(qkv[:, nq * d:(nq + nkv) * d].reshape(T, nkv, d), pos, nkv, d, cfg["rope_theta"]))
        vv = qkv[:, (nq + nkv) * d:].reshape(T, nkv, d)
        cap = 32
        kc, vc = np.zeros((nkv, cap, d), np.float32), np.zeros((nkv, cap, d), np.float32)
        kc[:, :T], vc[:, :T] = kk.transpose(1, 0, 2), vv.transpose(1, 0, 2)
        att = rb(orc.attention(q, kc, vc, T, 0, nq, nkv, d, cap))
        o = rb(att.astype(np.float64) @ w["wo"].astype(np.float64).T)
        want_mid = rb(x_in + o)
        scale = float(np.abs(want_mid).max())
        assert_parity(x_mid, want_mid, max_abs=3e-2 * scale, rel=3e-2, what="layer %d after attention" % tr["layer"])
        # ---- feed-forward half from the GPU's own mid-layer rows
        xn2 = rb(orc.rmsnorm(x_mid, w["ffn_norm"], cfg["rms_eps"]))
        want_f, ids_ref, _ = omoe.moe_ffn(xn2, w["router"], w["bias"], w["wg"], w["wu"], w["wd"], k, round_gate_up=False)
        logits = np.sort(omoe.route(xn2, w["router"], w["bias"], k)[2], axis=1)[:, ::-1]
        clear = (logits[:, k - 1] - logits[:, k]) > 1e-3 * np.abs(logits).max()
        clear_total += int(clear.sum())
        assert np.array_equal(tr["ids"][clear], ids_ref[clear]), "layer %d expert choice" % tr["layer"]
        fs = float(np.abs(want_f).max())
        assert_parity(tr["ffn_out"][clear], rb(want_f)[clear], max_abs=3e-2 * fs, rel=3e-2, what="layer %d feed-forward" % tr["layer"])
    assert clear_total >= 0.8 * T * cfg["layers"]
    ctx.check_device_error()


def test_prompt_pass_single_steps_and_batched_steps_agree(ctx, orc):
    cfg = CFG
    m = MoeDecoder(ctx, cfg, max_seqs=4, max_ctx=64, seed=SEED)
    prompts = [gen_token_ids(SEED, 20 + i, 9 + 3 * i, cfg["vocab"]) for i in range(3)]
    # whole prompt at once against prompt minus its last token + one decode step
    for p in prompts:
        s = m.new_sequence()
        _, full = m.prefill(s, p, want_logits=True)
        m.kv.seq_free(s)
        s = m.new_sequence()
        m.prefill(s, p[:-1])
        _, step = m.decode([s], [int(p[-1])], want_logits=True)
        m.kv.seq_free(s)
        assert_parity(step[0], full, max_abs=6e-2 * float(np.abs(full).max()), rel=6e-2, what="decode step against prompt pass")
    # three sequences of different lengths stepped together against each one alone
    alone = []
    for p in prompts:
        s = m.new_sequence()
        t = m.prefill(s, p)
        lg = []
        for _ in range(3):
            out, l1 = m.decode([s], [t], want_logits=True)
            t = int(out[0])
            lg.append(l1[0])
        alone.append(lg)
        m.kv.seq_free(s)
    seqs, toks = [], []
    for p in prompts:
        s = m.new_sequence()
        seqs.append(s)
        toks.append(m.prefill(s, p))
    for step in range(3):
        out, lg = m.decode(seqs, toks, want_logits=True)
        for i in range(3):
            # (the sequences follow their own greedy tokens; a row is compared while both runs fed the same token)
            assert_parity(lg[i], alone[i][step], max_abs=6e-2 * float(np.abs(alone[i][step]).max()), rel=6e-2, what="batched step %d row %d" % (step, i))
        toks = [int(np.argmax(alone[i][step][::-1])) for i in range(3)]
        toks = [len(alone[i][step]) - 1 - t for t in toks]              # last maximum, as the library's greedy rule
    ctx.check_device_error()
