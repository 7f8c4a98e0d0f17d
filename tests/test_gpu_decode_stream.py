"""The single-sequence decode step as one persistent kernel (decode_stream.cu) against the CPU oracle and against the
per-op path of the same library, on small models whose shapes exercise what the full-size model cannot reach quickly:
row groups cut by CTA boundaries (few units per CTA), several k slices per group, split attention over long contexts,
page boundaries, repacking after a weight change."""
import numpy as np
import pytest

from helpers import assert_parity, make_weights
from luminal_b200 import F32
from luminal_b200.llama import Llama

pytestmark = pytest.mark.gpu

# head_dim 128 and widths in multiples of 512 are what the persistent kernel needs
CFG_A = dict(layers=2, hidden=512, q_heads=4, kv_heads=2, head_dim=128, ffn=1024, vocab=2048, rms_eps=1e-5, rope_theta=500000.0)
CFG_B = dict(layers=3, hidden=1024, q_heads=8, kv_heads=2, head_dim=128, ffn=1536, vocab=4096, rms_eps=1e-5, rope_theta=500000.0)


def _pair(ctx, orc, cfg, seed, max_ctx, page_size=16, norm_random=True):
    w = make_weights(orc, cfg, seed=seed, norm_random=norm_random)
    m = Llama(ctx, cfg, act_dtype=F32, page_size=page_size, max_seqs=2, max_ctx=max_ctx)
    m.load_weights(w)
    return m, w


@pytest.mark.parametrize("cfg", [CFG_A, CFG_B], ids=["hidden512", "hidden1024"])
def test_stream_step_matches_oracle_and_per_op_path(ctx, orc, cfg):
    m, w = _pair(ctx, orc, cfg, seed=5, max_ctx=96, page_size=4)
    assert ctx.lib.blum_llama_decode_path(ctx.h, m.h) == 2
    ref = orc.Llama(cfg, w, ctx_cap=96)
    prompt = orc.gen_token_ids(5, 1, 7, cfg["vocab"])
    seq = m.new_sequence()
    tok, logits = m.prefill(seq, prompt, want_logits=True)
    want = ref.forward(prompt)
    assert tok == orc.argmax(want)
    ids = [tok]
    for step in range(40):                                   # crosses ten 4-token pages
        out, lg = m.decode([seq], [tok], want_logits=True)
        want = ref.forward([tok])
        assert_parity(lg[0], want, max_abs=1e-3, rel=1e-3, what="stream step %d logits" % step)
        assert int(out[0]) == orc.argmax(want), step
        tok = int(out[0])
        ids.append(tok)
    m.kv.seq_free(seq)
    ctx.check_device_error()
    # the per-op path of the same model gives the same tokens
    ctx._check(ctx.lib.blum_llama_set_decode_path(ctx.h, m.h, 1))
    assert ctx.lib.blum_llama_decode_path(ctx.h, m.h) == 1
    assert m.greedy(prompt, 41) == ids
    ctx._check(ctx.lib.blum_llama_set_decode_path(ctx.h, m.h, 0))
    # two runs of the persistent kernel are bit-identical (fixed summation order)
    seq = m.new_sequence()
    tok = m.prefill(seq, prompt)
    _, l1 = m.decode([seq], [tok], want_logits=True)
    m.kv.seq_free(seq)
    seq = m.new_sequence()
    tok = m.prefill(seq, prompt)
    _, l2 = m.decode([seq], [tok], want_logits=True)
    m.kv.seq_free(seq)
    assert np.array_equal(l1, l2)
    m.destroy()


def test_stream_step_long_context_uses_split_attention(ctx, orc):
    """700 cached positions: several 256-position tiles and more than one split per head."""
    cfg = CFG_A
    m, w = _pair(ctx, orc, cfg, seed=6, max_ctx=800)
    ref = orc.Llama(cfg, w, ctx_cap=800)
    prompt = orc.gen_token_ids(6, 1, 700, cfg["vocab"])
    seq = m.new_sequence()
    tok = m.prefill(seq, prompt)
    want = ref.forward(prompt)
    assert tok == orc.argmax(want)
    for step in range(6):
        out, lg = m.decode([seq], [tok], want_logits=True)
        want = ref.forward([tok])
        assert_parity(lg[0], want, max_abs=1e-3, rel=1e-3, what="long-context stream step %d" % step)
        tok = int(out[0])
        assert tok == orc.argmax(want)
    ctx.check_device_error()
    m.destroy()


def test_stream_decode_loop_and_repack_after_weight_change(ctx, orc):
    cfg = CFG_B
    m, w = _pair(ctx, orc, cfg, seed=7, max_ctx=64)
    prompt = orc.gen_token_ids(7, 1, 5, cfg["vocab"])
    want = m.greedy(prompt, 12)
    seq = m.new_sequence()
    first = m.prefill(seq, prompt)
    got = [first] + m.decode_loop(seq, first, 11).tolist()
    m.kv.seq_free(seq)
    assert got == want
    # new weights for one projection: the packed copy must follow
    name = "blk.1.ffn_down.weight"
    q, d = w[name]
    w2 = dict(w)
    w2[name] = (np.ascontiguousarray(q[::-1]), np.ascontiguousarray(d[::-1]))
    m.set_tensor(name, w2[name])
    ref = orc.Llama(cfg, w2, ctx_cap=64)
    ids, _ = ref.greedy(prompt, 8)
    assert m.greedy(prompt, 8) == ids
    ctx.check_device_error()
    m.destroy()


@pytest.mark.parametrize("cfg", [CFG_A, CFG_B], ids=["hidden512", "hidden1024"])
def test_prompt_chunks_take_the_packed_rows_matmul(ctx, orc, cfg):
    """Prompt chunks of the f32 configuration multiply 8 / 16 / 32 rows per pass over the stream-packed weights
    (integer mma on block-fixed-point rows): logits of the last prompt token against the oracle for every tile shape,
    a ragged last tile and more rows than one scratch block; the per-op path (GEMV, two rows per pass) agrees too."""
    m, w = _pair(ctx, orc, cfg, seed=8, max_ctx=160)
    for n in (5, 9, 17, 33, 131):
        prompt = orc.gen_token_ids(8, n, n, cfg["vocab"])
        ref = orc.Llama(cfg, w, ctx_cap=160)
        want = ref.forward(prompt)
        seq = m.new_sequence()
        tok, logits = m.prefill(seq, prompt, want_logits=True)
        m.kv.seq_free(seq)
        assert_parity(logits, want, max_abs=1e-3, rel=1e-3, what="prompt of %d tokens" % n)
        assert tok == orc.argmax(want)
        ctx._check(ctx.lib.blum_llama_set_decode_path(ctx.h, m.h, 1))
        seq = m.new_sequence()
        tok1, logits1 = m.prefill(seq, prompt, want_logits=True)
        m.kv.seq_free(seq)
        ctx._check(ctx.lib.blum_llama_set_decode_path(ctx.h, m.h, 0))
        assert tok1 == tok
        assert_parity(logits1, logits, max_abs=1e-4, rel=1e-4, what="per-op path, prompt of %d tokens" % n)
        # a second pass gives the same bits (fixed summation order)
        seq = m.new_sequence()
        _, logits2 = m.prefill(seq, prompt, want_logits=True)
        m.kv.seq_free(seq)
        assert np.array_equal(logits, logits2)
    ctx.check_device_error()
    m.destroy()
