"""MXFP4 mixture of experts on the GPU against the numpy oracle: exact routing and permutation, tolerance on values."""
import numpy as np
import pytest

from helpers import assert_parity
from luminal_b200 import BF16, F32
from luminal_b200.moe import MoeFfn, Mxfp4Weight
from luminal_b200.runtime import gen_normal, round_to_dtype
from oracle import moe as omoe

pytestmark = pytest.mark.gpu


def test_mxfp4_generator_and_dequant_match_the_oracle(ctx):
    E, N, K = 3, 40, 128
    w = Mxfp4Weight.generate(ctx, 4, 900, E, N, K)
    q, s = w.download()
    oq, os_ = omoe.gen_mxfp4(4, 900, E, N, K)
    assert np.array_equal(q, oq) and np.array_equal(s, os_)
    assert s.min() >= 119 and s.max() <= 127 and len(np.unique(q & 15)) == 16
    # dequantised weights through the tensor-core path: y = x W^T with x = identity rows picks out W's columns
    x = np.zeros((64, K), np.float32)
    x[np.arange(64), np.arange(64)] = 1.0
    offsets = ctx.to_device_raw(np.array([0, 64, 64, 64], np.int32))     # all 64 rows belong to expert 0
    y = ctx.alloc(64 * N * 4)
    xd = ctx.to_device(x, BF16)
    ctx._check(ctx.lib.blum_moe_grouped_gemm(ctx.h, w.h, xd.ptr, offsets.ptr, 64, y.ptr, F32, 64))
    got = ctx.to_host(y, F32, 64 * N).reshape(64, N)
    want = omoe.dequant_mxfp4(oq, os_)[0][:, :64].T
    assert np.array_equal(got, want)          # e2m1 * 2^e is exact in bf16 and each output is a single product
    ctx.check_device_error()
    w.free()


def test_stacked_gate_up_weight_layout(ctx):
    """[E, 2N, K]: every 32 rows are 16 gate rows followed by the 16 up rows of the same features, quants and scales alike."""
    E, N, K = 3, 48, 128
    g, u = Mxfp4Weight.generate(ctx, 4, 930, E, N, K), Mxfp4Weight.generate(ctx, 4, 931, E, N, K)
    st = Mxfp4Weight.stack_gate_up(g, u)
    (gq, gs), (uq, us), (sq, ss) = g.download(), u.download(), st.download()
    assert sq.shape == (E, 2 * N, K // 2) and ss.shape == (E, 2 * N, K // 32)
    for got, a, b in ((sq, gq, uq), (ss, gs, us)):
        got = got.reshape(E, N // 16, 2, 16, -1)
        assert np.array_equal(got[:, :, 0], a.reshape(E, N // 16, 16, -1))
        assert np.array_equal(got[:, :, 1], b.reshape(E, N // 16, 16, -1))
    for w in (g, u, st):
        w.free()


def _form(layer, form):
    """stream: the small-rows streaming kernel whatever the row count; fused: the tcgen05 grouped product with the SwiGLU
    epilogue; three: gate, up and down as three tcgen05 products."""
    layer.SMALL_ROWS = {"stream": 1 << 20, "fused": 0, "three": 0}[form]
    assert (layer.w_gate_up is not None) == (form != "three")


@pytest.mark.parametrize("form", ["stream", "fused", "three"])
@pytest.mark.parametrize("T", [1, 7, 64, 300])
def test_moe_ffn_against_oracle(ctx, T, form):
    fused = form != "three"
    H, I, E, k = 256, 384, 8, 2
    wg, wu, wd = (Mxfp4Weight.generate(ctx, 4, 910 + i, E, n, kk) for i, (n, kk) in enumerate(((I, H), (I, H), (H, I))))
    router = round_to_dtype(gen_normal(4, 920, E * H, 0.02).reshape(E, H), BF16)
    bias = (-1.1 * np.log(np.arange(1, E + 1))).astype(np.float32) * 0.05      # mild Zipf skew
    x = round_to_dtype(gen_normal(4, 921, T * H).reshape(T, H), BF16)
    layer = MoeFfn(ctx, H, I, E, k, ctx.to_device(router, BF16), ctx.to_device(bias), wg, wu, wd, fused_swiglu=fused)
    _form(layer, form)
    keep = {}
    out = ctx.to_host(layer.forward(ctx.to_device(x, BF16), T, out_dtype=F32, keep=keep), F32, T * H).reshape(T, H)
    ctx.check_device_error()
    deq = [omoe.dequant_mxfp4(*omoe.gen_mxfp4(4, 910 + i, E, n, kk)) for i, (n, kk) in enumerate(((I, H), (I, H), (H, I)))]
    want, ids, gates = omoe.moe_ffn(x, router, bias, deq[0], deq[1], deq[2], k, round_gate_up=not fused)
    # routing and permutation are exact
    got_ids = keep["ids"].download(np.int32, T * k).reshape(T, k)
    assert np.array_equal(got_ids, ids)
    assert np.abs(ctx.to_host(keep["gates"], F32, T * k).reshape(T, k) - gates).max() < 1e-5
    ss, so, off = omoe.permute(ids, E)
    assert np.array_equal(keep["sorted_src"].download(np.int32, T * k), ss)
    assert np.array_equal(keep["slot_of"].download(np.int32, T * k), so)
    assert np.array_equal(keep["offsets"].download(np.int32, E + 1), off)
    # values: bf16 intermediates on both sides; the accumulation order inside the MMA differs
    scale = np.abs(want).max()
    assert_parity(out, want, max_abs=max(1e-2, 2e-2 * scale), rel=2e-2, what="moe ffn T=%d" % T)
    assert np.abs(out - want).mean() < 4e-3 * scale
    for w in (wg, wu, wd) + ((layer.w_gate_up,) if fused else ()):
        w.free()


@pytest.mark.parametrize("form", ["stream", "fused", "three"])
@pytest.mark.parametrize("T", [1, 64])
def test_moe_ffn_at_the_full_layer_size(ctx, T, form):
    """The MoE configuration's own dimensions (hidden = expert intermediate = 2880, 32 experts, top-4, Zipf-skewed router
    bias): routing and permutation exact, values at the contract tolerance.  The oracle dequantises only the experts that
    are hit, from the bytes the device holds; the device generator is checked against the oracle's on expert 0."""
    H, I, E, k = 2880, 2880, 32, 4
    ws = [Mxfp4Weight.generate(ctx, 4, 940 + i, E, n, kk) for i, (n, kk) in enumerate(((I, H), (I, H), (H, I)))]
    host = [w.download() for w in ws]
    q0, s0 = omoe.gen_mxfp4(4, 940, 1, I, H)       # the stream is indexed expert-major: expert 0 is its first N*K elements
    assert np.array_equal(host[0][0][0], q0[0]) and np.array_equal(host[0][1][0], s0[0])
    router = round_to_dtype(gen_normal(4, 950, E * H, 0.02).reshape(E, H), BF16)
    bias = (-1.1 * np.log(np.arange(1, E + 1))).astype(np.float32)              # expert load roughly Zipf(1.1)
    x = round_to_dtype(gen_normal(4, 951, T * H).reshape(T, H), BF16)
    fused = form != "three"
    layer = MoeFfn(ctx, H, I, E, k, ctx.to_device(router, BF16), ctx.to_device(bias), *ws, fused_swiglu=fused)
    _form(layer, form)
    keep = {}
    out = ctx.to_host(layer.forward(ctx.to_device(x, BF16), T, out_dtype=F32, keep=keep), F32, T * H).reshape(T, H)
    ctx.check_device_error()
    expert = lambda e: tuple(omoe.dequant_mxfp4(q[e], s[e]) for q, s in host)
    want, ids, gates = omoe.moe_ffn_lazy(x, router, bias, expert, k, round_gate_up=not fused)
    assert np.array_equal(keep["ids"].download(np.int32, T * k).reshape(T, k), ids)
    assert np.abs(ctx.to_host(keep["gates"], F32, T * k).reshape(T, k) - gates).max() < 1e-5
    ss, so, off = omoe.permute(ids, E)
    assert np.array_equal(keep["sorted_src"].download(np.int32, T * k), ss)
    assert np.array_equal(keep["slot_of"].download(np.int32, T * k), so)
    assert np.array_equal(keep["offsets"].download(np.int32, E + 1), off)
    scale = np.abs(want).max()
    assert_parity(out, want, max_abs=max(1e-2, 2e-2 * scale), rel=2e-2, what="moe ffn 2880/32/top-4 T=%d" % T)
    assert np.abs(out - want).mean() < 4e-3 * scale
    for w in ws + ([layer.w_gate_up] if fused else []):
        w.free()


def test_topk_ties_go_to_the_lower_expert(ctx):
    H, E, k, T = 64, 8, 4, 3
    router = np.zeros((E, H), np.float32)
    router[[1, 3, 5, 6], 0] = 1.0            # experts 1,3,5,6 tie on top; the rest tie at zero
    x = np.zeros((T, H), np.float32)
    x[:, 0] = [1.0, 2.0, -1.0]               # negative x flips the order: 0,2,4,7 lead
    layer = MoeFfn(ctx, H, 64, E, k, ctx.to_device(router, BF16), None, None, None, None)
    ids, gates = layer.route(ctx.to_device(x, BF16), T)
    got = ids.download(np.int32, T * k).reshape(T, k)
    assert got.tolist() == [[1, 3, 5, 6], [1, 3, 5, 6], [0, 2, 4, 7]]
    assert np.allclose(ctx.to_host(gates, F32, T * k), 0.25)
    assert np.array_equal(omoe.route(x, router, None, k)[0], got)


def test_bf16_dense_matmul(ctx):
    n, k, m = 200, 256, 70
    w = round_to_dtype(gen_normal(4, 930, n * k, 0.02).reshape(n, k), BF16)
    x = round_to_dtype(gen_normal(4, 931, m * k).reshape(m, k), BF16)
    y = ctx.alloc(m * n * 4)
    wd, xd = ctx.to_device(w, BF16), ctx.to_device(x, BF16)
    ctx._check(ctx.lib.blum_bf16_matmul(ctx.h, wd.ptr, n, k, xd.ptr, y.ptr, F32, m))
    got = ctx.to_host(y, F32, m * n).reshape(m, n)
    assert_parity(got, x.astype(np.float64) @ w.astype(np.float64).T, max_abs=1e-4, rel=1e-4, what="bf16 matmul")
    ctx.check_device_error()


@pytest.mark.parametrize("m", [1, 5, 8])
@pytest.mark.parametrize("n,k", [(5120, 2880), (200, 256), (96, 2880)])
def test_bf16_dense_matmul_at_decode_row_counts(ctx, m, n, k):
    """One to eight rows take the streaming kernel (bf16_small.cu): K = 2880 is 22.5 super-blocks of 128 (a ragged last
    chunk), N = 200 / 96 leave ragged row tasks; f32 and bf16 outputs."""
    w = round_to_dtype(gen_normal(4, 960 + m, n * k, 0.02).reshape(n, k), BF16)
    x = round_to_dtype(gen_normal(4, 970 + m, m * k).reshape(m, k), BF16)
    want = x.astype(np.float64) @ w.astype(np.float64).T
    wd, xd = ctx.to_device(w, BF16), ctx.to_device(x, BF16)
    y = ctx.alloc(m * n * 4)
    ctx._check(ctx.lib.blum_bf16_matmul(ctx.h, wd.ptr, n, k, xd.ptr, y.ptr, F32, m))
    assert_parity(ctx.to_host(y, F32, m * n).reshape(m, n), want, max_abs=2e-4 * max(1.0, float(np.abs(want).max())), rel=1e-4, what="bf16 small matmul f32 out")
    ctx._check(ctx.lib.blum_bf16_matmul(ctx.h, wd.ptr, n, k, xd.ptr, y.ptr, BF16, m))
    got = ctx.to_host(y, BF16, m * n).reshape(m, n)
    assert_parity(got, want, max_abs=2.0 ** -8 * float(np.abs(want).max()) + 1e-4, rel=1e-2, what="bf16 small matmul bf16 out")
    ctx.check_device_error()
