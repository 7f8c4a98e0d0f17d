"""Temperature / top-p sampling on the device against the CPU oracle's integer-exact specification: identical token ids."""
import numpy as np
import pytest

from helpers import TINY_CFG, make_weights
from luminal_b200 import F32, BlumError
from luminal_b200.llama import Llama

pytestmark = pytest.mark.gpu


def _sample(ctx, logits, temperature, top_p, seed, seqs, poss):
    rows, cols = logits.shape
    ld = ctx.to_device(logits)
    sd, pd = ctx.to_device_raw(np.asarray(seqs, np.int32)), ctx.to_device_raw(np.asarray(poss, np.int32))
    scratch, out = ctx.alloc(rows * cols * 4), ctx.alloc(rows * 4)
    ctx._check(ctx.lib.blum_sample_top_p(ctx.h, ld.ptr, rows, cols, temperature, top_p, seed, sd.ptr, pd.ptr, scratch.ptr, out.ptr))
    return out.download(np.int32, rows)


@pytest.mark.parametrize("cols", [1000, 4097, 128256])
def test_sampler_matches_the_oracle_token_for_token(ctx, orc, cols):
    rng = np.random.default_rng(cols)
    rows = 24 if cols < 100000 else 6
    logits = (rng.standard_normal((rows, cols)) * rng.uniform(0.5, 6.0, (rows, 1))).astype(np.float32)
    seqs, poss = rng.integers(0, 8, rows), rng.integers(0, 5000, rows)
    for temperature, top_p, seed in ((1.0, 1.0, 1), (0.3, 0.9, 2), (2.5, 0.5, 3), (0.8, 0.05, 4), (1.0, 1e-6, 5), (7.0, 0.999, 6)):
        got = _sample(ctx, logits, temperature, top_p, seed, seqs, poss)
        want = [orc.sample_top_p(logits[r], temperature, top_p, seed, seqs[r], poss[r]) for r in range(rows)]
        assert got.tolist() == want, (temperature, top_p)
    ctx.check_device_error()


def test_sampler_against_golden_fixture(ctx, orc):
    import os
    from golden.make_golden import SAMPLE_CASES
    g = np.load(os.path.join(os.path.dirname(__file__), "golden", "oracle_vectors.npz"))
    logits = orc.gen_normal(5, 700, 8 * 1000, 3.0).reshape(8, 1000)
    for c, (t, p, sd) in enumerate(SAMPLE_CASES):
        got = _sample(ctx, logits, t, p, sd, [r % 3 for r in range(8)], [10 * r + c for r in range(8)])
        assert got.tolist() == g["sample_ids"][c].tolist(), c


def test_sampler_edge_rows(ctx, orc):
    cols = 777
    rng = np.random.default_rng(5)
    base = rng.standard_normal(cols).astype(np.float32)
    rows = []
    rows.append(np.zeros(cols, np.float32))                                  # all equal: every token in the nucleus
    r = base.copy(); r[::3] = -np.inf; rows.append(r)                         # -inf entries never sampled
    r = base.copy(); r[5] = np.nan; r[700] = np.nan; rows.append(r)           # NaNs weigh nothing
    r = base.copy(); r[123] = np.inf; rows.append(r)                          # +inf maximum: greedy rule
    rows.append(np.full(cols, np.nan, np.float32))                            # nothing finite: greedy rule
    rows.append(np.full(cols, -np.inf, np.float32))
    r = base.copy(); r[10] = r[20] = r[30] = 9.0; rows.append(r)              # ties at the top
    r = np.full(cols, -50.0, np.float32); r[42] = 0.0; rows.append(r)         # one token holds all the weight
    logits = np.stack(rows)
    n = len(rows)
    for trial in range(20):
        seqs, poss = [trial % 3] * n, list(range(trial * 10, trial * 10 + n))
        for temperature, top_p in ((1.0, 1.0), (0.5, 0.6)):
            got = _sample(ctx, logits, temperature, top_p, 99, seqs, poss)
            want = [orc.sample_top_p(logits[r], temperature, top_p, 99, seqs[r], poss[r]) for r in range(n)]
            assert got.tolist() == want, (trial, temperature, top_p)
            assert np.isfinite(logits[1][got[1]]) and got[2] not in (5, 700) and got[3] == 123 and got[7] == 42
    with pytest.raises(BlumError):
        _sample(ctx, logits, 0.0, 1.0, 1, [0] * n, [0] * n)                  # temperature 0 is the argmax entry point
    ctx.check_device_error()


def test_decoder_samples_reproducibly_and_like_the_oracle(ctx, orc):
    cfg = TINY_CFG
    m = Llama(ctx, cfg, act_dtype=F32, page_size=4, max_seqs=2, max_ctx=64)
    m.load_weights(make_weights(orc, cfg, seed=0))
    prompt = orc.gen_token_ids(0, 1, 6, cfg["vocab"])
    greedy = m.greedy(prompt, 10)
    m.set_sampling(1.5, 0.95, seed=11)
    seq = m.new_sequence()
    first, logits = m.prefill(seq, prompt, want_logits=True)
    assert first == orc.sample_top_p(logits, 1.5, 0.95, 11, seq, len(prompt) - 1)
    toks = [first]
    for step in range(9):                                    # captured step: the draw follows the position
        out, lg = m.decode([seq], [toks[-1]], want_logits=True)
        assert int(out[0]) == orc.sample_top_p(lg[0], 1.5, 0.95, 11, seq, len(prompt) + step)
        toks.append(int(out[0]))
    m.kv.seq_free(seq)
    seq = m.new_sequence()
    first2 = m.prefill(seq, prompt)
    rest = m.decode_loop(seq, first2, 9).tolist()              # tokens fed back on the device
    m.kv.seq_free(seq)
    assert [first2] + rest == toks
    assert toks != greedy
    m.set_sampling(1.5, 0.95, seed=12)
    assert m.greedy(prompt, 10) != toks                      # another seed, another text
    m.set_sampling(0.0)
    assert m.greedy(prompt, 10) == greedy
    ctx.check_device_error()
    m.destroy()
