"""Writes tests/golden/oracle_vectors.npz: outputs of the CPU oracle on small seeded inputs.

Run from the repository root:  python tests/golden/make_golden.py
The inputs are not stored: they are regenerated from (seed, tensor id) by the seeded generators, which
tests/test_abi.py checks are identical in the oracle and in the library.  The reference itself (Rust) cannot
run in this environment, so these are oracle outputs; the oracle in turn is pinned by the fixed-value vectors
of reference_known_answers.json.
"""
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
for p in (ROOT, os.path.dirname(HERE)):
    if p not in sys.path:
        sys.path.insert(0, p)

from helpers import TINY_CFG, TP_CFG, make_weights  # noqa: E402

Q8_CASES = [(64, 256, 1), (96, 512, 3), (40, 1024, 8)]   # (N, K, M); tensor id 100+i, activations id 200+i, seed 1
# temperature / top-p sampler: logits = gen_normal(seed 5, tensor 700, 8 x 1000, sigma 3); (temperature, top_p, seed) cases;
# row r is sampled as sequence slot r % 3 at position 10 r + case index
SAMPLE_CASES = [(1.0, 1.0, 1), (0.7, 0.9, 2), (2.0, 0.5, 3), (1.0, 0.02, 4)]


# MXFP4 mixture-of-experts layer (seed 4): hidden 64, intermediate 96, 4 experts, top-2, 9 tokens; expert weights from tensor
# ids 810-812, router id 820, tokens id 821; both forms of the gate/up products (rounded to bf16 before the SwiGLU or not)
MOE_CASE = dict(H=64, I=96, E=4, k=2, T=9)


def moe_inputs(orc):
    from oracle import moe as omoe
    c = MOE_CASE
    ws = [omoe.dequant_mxfp4(*omoe.gen_mxfp4(4, 810 + i, c["E"], n, kk)) for i, (n, kk) in enumerate(((c["I"], c["H"]), (c["I"], c["H"]), (c["H"], c["I"])))]
    router = omoe.round_bf16(orc.gen_normal(4, 820, c["E"] * c["H"], 0.02).reshape(c["E"], c["H"]))
    bias = (-0.3 * np.log(np.arange(1, c["E"] + 1))).astype(np.float32)
    x = omoe.round_bf16(orc.gen_normal(4, 821, c["T"] * c["H"]).reshape(c["T"], c["H"]))
    return x, router, bias, ws


def compute_moe(orc):
    from oracle import moe as omoe
    x, router, bias, ws = moe_inputs(orc)
    out = {}
    for key, rnd in (("moe_out", True), ("moe_out_f32_gate_up", False)):
        y, ids, gates = omoe.moe_ffn(x, router, bias, ws[0], ws[1], ws[2], MOE_CASE["k"], round_gate_up=rnd)
        out[key] = y
    out["moe_ids"], out["moe_gates"] = ids, gates
    return out


def compute(orc):
    out = {}
    for i, (n, k, m) in enumerate(Q8_CASES):
        q = orc.gen_q8_quants(1, 100 + i, n * k).reshape(n, k)
        d = orc.gen_q8_scales(1, 100 + i, n * k // 32).reshape(n, k // 32)
        x = orc.gen_normal(1, 200 + i, m * k).reshape(m, k)
        out["q8_matmul_%d" % i] = orc.q8_matmul(orc.q8_pack(q, d), n, k, x)
        out["q8_matmul_bf16in_%d" % i] = orc.q8_matmul(orc.q8_pack(q, d), n, k, orc.round_bf16(x).reshape(m, k))
    x = orc.gen_normal(1, 300, 6 * 256).reshape(6, 256)
    w = orc.gen_normal(1, 301, 256)
    out["rmsnorm"] = orc.rmsnorm(x, w, 1e-5)
    xr = orc.gen_normal(1, 302, 5 * 4 * 128).reshape(5, 4, 128)
    out["rope"] = orc.rope(xr, np.array([0, 1, 17, 511, 4095]), 4, 128, 500000.0)
    g, u = orc.gen_normal(1, 303, 777), orc.gen_normal(1, 304, 777)
    out["swiglu"] = orc.swiglu(g, u)
    out["softmax"] = orc.softmax(orc.gen_normal(1, 305, 4 * 333, 3.0).reshape(4, 333))
    T, p, nq, nkv, dd, cap = 4, 9, 8, 2, 64, 16
    qa = orc.gen_normal(1, 306, T * nq * dd).reshape(T, nq, dd)
    kc = orc.gen_normal(1, 307, nkv * cap * dd).reshape(nkv, cap, dd)
    vc = orc.gen_normal(1, 308, nkv * cap * dd).reshape(nkv, cap, dd)
    out["attention"] = orc.attention(qa, kc, vc, T, p, nq, nkv, dd, cap)
    # tiny Llama: 6-token prompt, 8 greedy steps (seed 0; prompt ids tensor id 1)
    w = make_weights(orc, TINY_CFG, seed=0)
    model = orc.Llama(TINY_CFG, w, ctx_cap=32)
    prompt = orc.gen_token_ids(0, 1, 6, TINY_CFG["vocab"])
    logits = model.forward(prompt)
    out["llama_prefill_logits"] = logits.copy()
    toks = []
    for _ in range(8):
        tok = orc.argmax(logits)
        toks.append(tok)
        logits = model.forward([tok])
    out["llama_greedy_ids"] = np.array(toks, np.int32)
    out["llama_last_logits"] = logits.copy()
    # a decoder every tensor-parallel degree of one node divides (seed 0; prompt ids tensor id 1): 6-token prompt, 8 greedy steps,
    # bf16 activations as the tensor-parallel configuration runs them
    w = make_weights(orc, TP_CFG, seed=0)
    for key, mode in (("tp_greedy_ids_f32", 0), ("tp_greedy_ids_bf16", 2)):
        model = orc.Llama(TP_CFG, w, ctx_cap=32, round_mode=mode)
        ids, gaps = model.greedy(orc.gen_token_ids(0, 1, 6, TP_CFG["vocab"]), 8)
        out[key] = np.array(ids, np.int32)
        out[key.replace("ids", "gaps")] = np.array(gaps, np.float32)
    out.update(compute_moe(orc))
    logits = orc.gen_normal(5, 700, 8 * 1000, 3.0).reshape(8, 1000)
    out["sample_ids"] = np.array([[orc.sample_top_p(logits[r], t, p, sd, r % 3, 10 * r + c) for r in range(8)]
                                  for c, (t, p, sd) in enumerate(SAMPLE_CASES)], np.int32)
    return out


if __name__ == "__main__":
    from oracle import oracle
    np.savez_compressed(os.path.join(HERE, "oracle_vectors.npz"), **compute(oracle))
    print("wrote", os.path.join(HERE, "oracle_vectors.npz"))
