"""End-to-end decoder on the GPU against the CPU oracle: logits within tolerance, greedy ids identical."""
import os

import numpy as np
import pytest

from helpers import LLAMA8B_CFG, TINY_CFG, TINY_PHI_CFG, TINY_QWEN_CFG, assert_parity, make_weights
from luminal_b200 import BF16, F32, BlumError, runtime
from luminal_b200.llama import Llama

pytestmark = pytest.mark.gpu
GOLD = os.path.join(os.path.dirname(__file__), "golden")


@pytest.fixture(scope="module")
def tiny(ctx, orc):
    w = make_weights(orc, TINY_CFG, seed=0)
    m = Llama(ctx, TINY_CFG, act_dtype=F32, page_size=4, max_seqs=6, max_ctx=64)
    m.load_weights(w)
    yield m, w
    m.destroy()


def test_tiny_llama_matches_golden_and_oracle(ctx, orc, tiny):
    m, w = tiny
    g = np.load(os.path.join(GOLD, "oracle_vectors.npz"))
    prompt = orc.gen_token_ids(0, 1, 6, TINY_CFG["vocab"])
    seq = m.new_sequence()
    tok, logits = m.prefill(seq, prompt, want_logits=True)
    assert_parity(logits, g["llama_prefill_logits"], max_abs=1e-3, rel=1e-3, what="prefill logits")
    toks = [tok]
    for _ in range(7):
        out, logits = m.decode([seq], [toks[-1]], want_logits=True)
        toks.append(int(out[0]))
    assert toks == g["llama_greedy_ids"].tolist()
    out, logits = m.decode([seq], [toks[-1]], want_logits=True)
    assert_parity(logits[0], g["llama_last_logits"], max_abs=1e-3, rel=1e-3, what="last logits")
    m.kv.seq_free(seq)
    ctx.check_device_error()


def test_generated_weights_equal_loaded_weights(ctx, orc, tiny):
    """blum_llama_generate_weights (device-side quants, host-side scales) builds the same model as loading the
    oracle's generated tensors by GGUF name."""
    m, w = tiny
    g = Llama(ctx, TINY_CFG, act_dtype=F32, page_size=16, max_seqs=1, max_ctx=64)
    g.generate_weights(0)
    prompt = orc.gen_token_ids(0, 2, 9, TINY_CFG["vocab"])
    assert g.greedy(prompt, 6) == m.greedy(prompt, 6)
    g.destroy()


def test_decode_loop_equals_stepwise_decode(ctx, orc, tiny):
    m, _ = tiny
    prompt = orc.gen_token_ids(0, 3, 5, TINY_CFG["vocab"])
    want = m.greedy(prompt, 12)
    seq = m.new_sequence()
    first = m.prefill(seq, prompt)
    got = [first] + m.decode_loop(seq, first, 11).tolist()
    m.kv.seq_free(seq)
    assert got == want


def test_batched_decode_equals_single_sequences(ctx, orc, tiny):
    """Ragged batch: 5 sequences of different prompt lengths decoded together give the ids each gives alone
    (more than 4 rows takes the unfused matmul path, fewer the fused GEMV path)."""
    m, _ = tiny
    prompts = [orc.gen_token_ids(0, 10 + i, n, TINY_CFG["vocab"]) for i, n in enumerate((1, 3, 7, 12, 20))]
    alone = [m.greedy(p, 6) for p in prompts]
    for group in (prompts[:2], prompts):
        seqs = [m.new_sequence() for _ in group]
        toks = [[m.prefill(s, p)] for s, p in zip(seqs, group)]
        for _ in range(5):
            out = m.decode(seqs, [t[-1] for t in toks])
            for t, o in zip(toks, out):
                t.append(int(o))
        for s in seqs:
            m.kv.seq_free(s)
        assert toks == alone[:len(group)]
    ctx.check_device_error()


def test_bf16_model_tracks_bf16_oracle(ctx, orc):
    w = make_weights(orc, TINY_CFG, seed=0)
    m = Llama(ctx, TINY_CFG, act_dtype=BF16, page_size=16, max_seqs=1, max_ctx=64)
    m.load_weights(w)
    ref = orc.Llama(TINY_CFG, w, ctx_cap=64, round_mode=2)
    prompt = orc.gen_token_ids(0, 1, 6, TINY_CFG["vocab"])
    seq = m.new_sequence()
    _, logits = m.prefill(seq, prompt, want_logits=True)
    want = ref.forward(prompt)
    # bf16 activations: 8-bit significands through 2 layers; the contract tolerance applies to the logits' scale
    assert_parity(logits, want, max_abs=5e-2 * max(1.0, np.abs(want).max()), rel=5e-2, what="bf16 logits")
    m.destroy()


def test_llama3_8b_layer_shapes(ctx, orc):
    """One layer with the real Llama-3-8B widths (hidden 4096, 32/8 heads of 128, FFN 14336) and a small vocabulary."""
    cfg = dict(layers=1, hidden=4096, q_heads=32, kv_heads=8, head_dim=128, ffn=14336, vocab=512, rms_eps=1e-5, rope_theta=500000.0)
    w = make_weights(orc, cfg, seed=0)
    ref = orc.Llama(cfg, w, ctx_cap=64)
    m = Llama(ctx, cfg, act_dtype=F32, page_size=16, max_seqs=1, max_ctx=64)
    m.generate_weights(0)
    prompt = orc.gen_token_ids(0, 1, 32, cfg["vocab"])
    seq = m.new_sequence()
    tok, logits = m.prefill(seq, prompt, want_logits=True)
    want = ref.forward(prompt)
    assert_parity(logits, want, max_abs=2e-3, rel=2e-3, what="8B-width prefill logits")
    assert tok == orc.argmax(want)
    for _ in range(4):
        out, logits = m.decode([seq], [tok], want_logits=True)
        want = ref.forward([tok])
        assert_parity(logits[0], want, max_abs=2e-3, rel=2e-3, what="8B-width decode logits")
        assert int(out[0]) == orc.argmax(want)
        tok = int(out[0])
    m.destroy()


def test_llama3_8b_full_model_32_greedy_ids(ctx, orc):
    """The configuration the benchmark times, at its own size: 32 layers, vocabulary 128 256, seed 0, f32 activations and
    KV.  A 32-token prompt and 32 greedy steps on the GPU and through the CPU oracle (weights kept quantised, all host
    cores): the 32 token ids must be identical (examples/llama/src/main.rs:152-181, sampler :194-198) and the logits of every
    step within the contract tolerance.  The top-2 logit gap of every step is printed for both sides, so that a mismatch can
    be told apart from a near-tie."""
    cfg = LLAMA8B_CFG
    m = Llama(ctx, cfg, act_dtype=F32, page_size=16, max_seqs=1, max_ctx=80)
    m.generate_weights(0)
    w = make_weights(orc, cfg, seed=0)
    ref = orc.Llama(cfg, w, ctx_cap=80)
    prompt = orc.gen_token_ids(0, 1, 32, cfg["vocab"])
    seq = m.new_sequence()
    tok, logits = m.prefill(seq, prompt, want_logits=True)
    want = ref.forward(prompt)
    got_ids, want_ids, report = [], [], []
    for step in range(32):
        wtok = orc.argmax(want)
        g2, w2 = np.partition(logits, -2)[-2:], np.partition(want, -2)[-2:]
        report.append("step %2d: gpu id %6d gap %.3e | oracle id %6d gap %.3e | max |dlogit| %.2e" % (
            step, tok, g2[1] - g2[0], wtok, w2[1] - w2[0], np.abs(logits - want).max()))
        got_ids.append(int(tok))
        want_ids.append(int(wtok))
        assert_parity(logits, want, max_abs=1e-2, rel=2e-2, what="full-size logits, step %d\n%s" % (step, "\n".join(report)))
        if tok != wtok or step == 31:
            break
        out, lg = m.decode([seq], [tok], want_logits=True)
        tok, logits = int(out[0]), lg[0]
        want = ref.forward([wtok])
    print("\n".join(report))
    assert got_ids == want_ids and len(got_ids) == 32, "\n".join(report)
    ctx.check_device_error()
    m.destroy()


def test_decode_reports_a_device_error_and_leaves_the_sequence_as_it_was(ctx, orc, tiny):
    """A page id outside the pool is caught by the kernels' index check (they skip the access and set the error word, no
    fault): the decode call must come back with ERR_DEVICE instead of a garbage token, the sequence must not have grown,
    and the same step must succeed once the table is repaired."""
    from luminal_b200 import _lib
    m, _ = tiny
    prompt = orc.gen_token_ids(0, 3, 5, TINY_CFG["vocab"])
    want = m.greedy(prompt, 3)
    seq = m.new_sequence()
    tok = m.prefill(seq, prompt)
    assert tok == want[0]
    n_before = m.kv.seq_len(seq)
    table = m.kv.page_table()                                # synchronised copy of the device table
    entry = int(seq) * m.kv.max_pages_per_seq + 1            # page of positions 4..7: the slot the next token is appended to
    good = np.array([table.reshape(-1)[entry]], np.int32)
    bad = np.array([m.kv.num_pages + 7], np.int32)
    tbl = ctx.lib.blum_kv_page_table_dev(m.kv.h)
    ctx._check(ctx.lib.blum_memcpy_h2d(ctx.h, tbl + 4 * entry, bad.ctypes.data, 4))
    ctx.sync()
    with pytest.raises(BlumError) as ei:
        m.decode([seq], [tok])
    assert ei.value.code == _lib.ERR_DEVICE
    assert m.kv.seq_len(seq) == n_before
    ctx._check(ctx.lib.blum_memcpy_h2d(ctx.h, tbl + 4 * entry, good.ctypes.data, 4))
    ctx.sync()
    ctx.check_device_error()                                 # the failed call already cleared the word
    m.kv.seq_free(seq)
    assert m.greedy(prompt, 3) == want


def test_a_second_larger_model_leaves_the_first_models_captured_step_valid(ctx, orc):
    """Model A (bf16, 5-row batches: tensor-core / small-batch GEMMs with an f32 workspace) decodes, then a larger model B is
    created on the same context and runs, which outgrows the shared workspace.  A's captured step still names the old
    buffer, which therefore must not have been freed: A decodes again and reproduces its own earlier tokens."""
    w = make_weights(orc, TINY_CFG, seed=0)
    a = Llama(ctx, TINY_CFG, act_dtype=BF16, page_size=16, max_seqs=5, max_ctx=64)
    a.load_weights(w)
    prompts = [orc.gen_token_ids(0, 40 + i, 4 + i, TINY_CFG["vocab"]) for i in range(5)]

    def run(model):
        seqs = [model.new_sequence() for _ in prompts]
        toks = [[model.prefill(s, p)] for s, p in zip(seqs, prompts)]
        for _ in range(4):
            out = model.decode(seqs, [t[-1] for t in toks])
            for t, o in zip(toks, out):
                t.append(int(o))
        for s in seqs:
            model.kv.seq_free(s)
        return toks

    first = run(a)
    big = dict(TINY_CFG, hidden=512, ffn=2048, q_heads=8, kv_heads=2, head_dim=64)
    b = Llama(ctx, big, act_dtype=BF16, page_size=16, max_seqs=8, max_ctx=2048)
    b.generate_weights(1)
    sb = b.new_sequence()
    b.prefill(sb, orc.gen_token_ids(0, 50, 300, big["vocab"]))
    assert run(a) == first
    ctx.check_device_error()
    b.destroy()
    a.destroy()


@pytest.mark.parametrize("cfg", [TINY_QWEN_CFG, TINY_PHI_CFG], ids=["qwen", "phi"])
def test_sibling_decoders_match_the_oracle(ctx, orc, cfg):
    """qwen (half-split rotary pairs, per-head q/k norm, tied head over a Q8_0 embedding table) and phi (theta 1e4, as
    many kv heads as q heads) on the same kernels: prompt pass, single-sequence decode and a 5-row batch against the
    oracle, f32 activations."""
    w = make_weights(orc, cfg, seed=9, norm_random=True)
    m = Llama(ctx, cfg, act_dtype=F32, page_size=4, max_seqs=6, max_ctx=64, embed_q8=bool(cfg.get("embed_q8")))
    m.load_weights(w)
    ref = orc.Llama(cfg, w, ctx_cap=64)
    prompt = orc.gen_token_ids(9, 1, 7, cfg["vocab"])
    seq = m.new_sequence()
    tok, logits = m.prefill(seq, prompt, want_logits=True)
    want = ref.forward(prompt)
    assert_parity(logits, want, max_abs=1e-3, rel=1e-3, what="sibling prefill logits")
    ids = [tok]
    for step in range(6):
        assert tok == orc.argmax(want)
        out, lg = m.decode([seq], [tok], want_logits=True)
        want = ref.forward([tok])
        assert_parity(lg[0], want, max_abs=1e-3, rel=1e-3, what="sibling decode logits, step %d" % step)
        tok = int(out[0])
        ids.append(tok)
    m.kv.seq_free(seq)
    # the same tokens come out of a 5-row batch (rows 1..4 are other prompts): the batched path applies the same glue
    prompts = [prompt] + [orc.gen_token_ids(9, 20 + i, 3 + i, cfg["vocab"]) for i in range(4)]
    seqs = [m.new_sequence() for _ in prompts]
    toks = [[m.prefill(s, p)] for s, p in zip(seqs, prompts)]
    for _ in range(6):
        out = m.decode(seqs, [t[-1] for t in toks])
        for t, o in zip(toks, out):
            t.append(int(o))
    assert toks[0] == ids
    ctx.check_device_error()
    m.destroy()


def test_model_error_paths(ctx, tiny):
    m, _ = tiny
    with pytest.raises(BlumError):
        m.prefill(5, [1, 2, 3])                      # sequence slot not allocated
    seq = m.new_sequence()
    with pytest.raises(BlumError):
        m.prefill(seq, [TINY_CFG["vocab"]])          # token id out of range
    with pytest.raises(BlumError):
        m.prefill(seq, list(range(65)))              # longer than max_ctx
    with pytest.raises(BlumError):
        m.set_tensor("blk.0.nope.weight", np.zeros(4, np.float32))
    with pytest.raises(BlumError):
        m.set_tensor("output_norm.weight", np.zeros(5, np.float32))   # wrong size
    m.kv.seq_free(seq)


def test_checkpoint_through_a_gguf_file(ctx, orc, tmp_path):
    """The seeded tiny model written as a GGUF v3 file (Q8_0 blocks + F32 tensors), read back through the memory map and
    installed tensor by tensor: same greedy ids as the golden sequence; a file of the wrong shape is refused."""
    from luminal_b200.gguf import GGML_F32, GGML_Q8_0, GgufError, write_gguf
    from luminal_b200.runtime import pack_gguf_q8_0
    w = make_weights(orc, TINY_CFG, 0)
    tensors = {}
    for name, v in w.items():
        if isinstance(v, tuple):
            tensors[name] = (GGML_Q8_0, v[0].shape, pack_gguf_q8_0(*v))
        else:
            a = np.ascontiguousarray(v, np.float32)
            tensors[name] = (GGML_F32, a.shape, a)
    path = str(tmp_path / "tiny.gguf")
    write_gguf(path, {"general.architecture": "llama", "llama.block_count": TINY_CFG["layers"]}, tensors)
    g = np.load(os.path.join(GOLD, "oracle_vectors.npz"))
    model = Llama(ctx, TINY_CFG, act_dtype=F32, page_size=4, max_seqs=2, max_ctx=64)
    info = model.load_gguf(path)
    assert info.version == 3 and len(info.tensors) == len(w)
    toks = model.greedy(orc.gen_token_ids(0, 1, 6, TINY_CFG["vocab"]), 8)
    assert toks == g["llama_greedy_ids"].tolist()
    model.destroy()
    bad = dict(TINY_CFG)
    bad["ffn"] = TINY_CFG["ffn"] * 2
    other = Llama(ctx, bad, act_dtype=F32, page_size=4, max_seqs=1, max_ctx=32)
    with pytest.raises(GgufError):
        other.load_gguf(path)
    other.destroy()
