"""The CPU oracle of the MXFP4 mixture-of-experts layer (oracle/moe.py): its definitions checked against hand-made cases
and an independent float64 evaluation, its committed golden vectors, and the expert-parallel sharding (every rank computes
the rows of its own experts; the combine at the owner gives the unsharded result exactly).  No GPU needed."""
import os
import sys

import numpy as np

sys.path.insert(0, os.path.join(os.path.dirname(__file__), "golden"))
from make_golden import MOE_CASE, moe_inputs  # noqa: E402
from oracle import moe as omoe  # noqa: E402

GOLD = os.path.join(os.path.dirname(__file__), "golden")


def test_mxfp4_decode_by_hand():
    # byte 0x2B: element 0 = code 0xB = -(1.5), element 1 = code 0x2 = +1.0; scale byte 126 = 2^-1
    nib = np.zeros((1, 16), np.uint8)
    nib[0, 0] = 0x2B
    nib[0, 15] = 0x7F                       # element 30 = code 0xF = -6, element 31 = code 7 = +6
    got = omoe.dequant_mxfp4(nib, np.array([[126]], np.uint8))[0]
    assert got[0] == -0.75 and got[1] == 0.5 and got[30] == -3.0 and got[31] == 3.0 and not got[2:30].any()
    assert not omoe.dequant_mxfp4(nib, np.array([[0]], np.uint8)).any()           # scale byte 0 decodes to zero
    codes = np.arange(16, dtype=np.uint8)
    packed = np.zeros((1, 16), np.uint8)
    packed[0, :8] = codes[0::2] | (codes[1::2] << 4)
    vals = omoe.dequant_mxfp4(packed, np.array([[127]], np.uint8))[0][:16]
    assert vals.tolist() == [0, .5, 1, 1.5, 2, 3, 4, 6, 0, -.5, -1, -1.5, -2, -3, -4, -6]


def test_round_bf16_ties_to_even():
    a = np.array([1.0, 1.0 + 2.0 ** -8, 1.0 + 3 * 2.0 ** -8, -(1.0 + 2.0 ** -8), 3.0e38], np.float32)
    assert omoe.round_bf16(a).tolist()[:4] == [1.0, 1.0, 1.0 + 2.0 ** -6, -1.0]


def test_routing_rules():
    H, E, k = 8, 6, 3
    w = np.zeros((E, H), np.float32)
    w[[1, 3, 4], 0] = 1.0                      # experts 1, 3, 4 tie on top, the rest tie at zero
    x = np.zeros((2, H), np.float32)
    x[:, 0] = [1.0, -1.0]                      # second token: the three are the WORST, the others tie at zero
    ids, gates, logits = omoe.route(x, w, None, k)
    assert ids.tolist() == [[1, 3, 4], [0, 2, 5]]           # ties go to the lower expert index
    assert np.allclose(gates, 1.0 / 3)
    bias = np.array([0, 0, 0, 0, 0, 5.0], np.float32)
    ids, gates, _ = omoe.route(x, w, bias, k)
    assert ids[0].tolist() == [5, 1, 3]
    e = np.exp(np.array([5.0, 1.0, 1.0]) - 5.0)
    assert np.allclose(gates[0], e / e.sum(), atol=1e-6)    # softmax over the selected logits only


def test_permutation_is_a_stable_counting_sort():
    ids = np.array([[2, 0], [1, 2], [0, 2], [2, 1]], np.int32)
    src, slot, off = omoe.permute(ids, 4)
    assert src.tolist() == [1, 4, 2, 7, 0, 3, 5, 6] and off.tolist() == [0, 2, 4, 8, 8]
    assert slot[src].tolist() == list(range(8))


def _float64_layer(x, router, bias, ws, k, round_gate_up):
    """The same layer evaluated token by token in float64 with the roundings applied explicitly."""
    T, H = x.shape
    rb = lambda a: omoe.round_bf16(np.asarray(a, np.float32)).astype(np.float64)
    out = np.zeros((T, H))
    for t in range(T):
        logits = x[t].astype(np.float64) @ router.astype(np.float64).T + bias
        order = sorted(range(len(logits)), key=lambda e: (-logits[e], e))[:k]
        g = np.exp(logits[order] - logits[order[0]])
        g /= g.sum()
        for j, e in enumerate(order):
            gate, up = ws[0][e].astype(np.float64) @ x[t], ws[1][e].astype(np.float64) @ x[t]
            if round_gate_up:
                gate, up = rb(gate), rb(up)
            mid = rb(up * (gate / (1 + np.exp(-gate))))
            out[t] += g[j] * rb(ws[2][e].astype(np.float64) @ mid)
    return out


def test_layer_against_a_float64_evaluation_and_the_golden_vectors(orc):
    x, router, bias, ws = moe_inputs(orc)
    g = np.load(os.path.join(GOLD, "oracle_vectors.npz"))
    for key, rnd in (("moe_out", True), ("moe_out_f32_gate_up", False)):
        y, ids, gates = omoe.moe_ffn(x, router, bias, ws[0], ws[1], ws[2], MOE_CASE["k"], round_gate_up=rnd)
        assert np.array_equal(y, g[key]) and np.array_equal(ids, g["moe_ids"]) and np.array_equal(gates, g["moe_gates"])
        want = _float64_layer(x, router, bias, ws, MOE_CASE["k"], rnd)
        # f32 sums of 64 / 96 products against float64: a bf16 rounding step may flip here and there
        assert np.abs(y - want).max() <= 2.0 ** -7 * np.abs(want).max()
        assert np.abs(y - want).mean() <= 1e-3 * np.abs(want).mean()
    assert np.abs(g["moe_out"] - g["moe_out_f32_gate_up"]).max() > 0          # the two forms are different roundings


def test_expert_parallel_sharding_gives_the_unsharded_layer(orc):
    """Rank r holds experts [r E/W, (r+1) E/W): it receives the rows routed to them, runs the expert, sends them back; the
    owner combines in choice order.  The same arithmetic per row, so the result is identical for every W."""
    x, router, bias, ws = moe_inputs(orc)
    c = MOE_CASE
    want, ids, gates = omoe.moe_ffn(x, router, bias, ws[0], ws[1], ws[2], c["k"])
    for W in (2, 4):
        EL = c["E"] // W
        contrib = np.zeros((c["T"], c["k"], c["H"]), np.float32)
        for r in range(W):
            mine = [w[r * EL:(r + 1) * EL] for w in ws]
            for t, j in zip(*np.nonzero((ids >= r * EL) & (ids < (r + 1) * EL))):
                e = ids[t, j] - r * EL
                gate, up = omoe.round_bf16(mine[0][e] @ x[t]), omoe.round_bf16(mine[1][e] @ x[t])
                contrib[t, j] = omoe.round_bf16(mine[2][e] @ omoe.round_bf16(up * omoe.swish(gate)))
        got = np.zeros_like(want)
        for t in range(c["T"]):
            for j in range(c["k"]):
                got[t] += gates[t, j] * contrib[t, j]
        assert np.array_equal(got, want), W
