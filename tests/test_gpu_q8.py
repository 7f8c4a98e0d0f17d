"""Q8_0 weights and matmul on the GPU against the CPU oracle (through the C ABI)."""
import json
import os

import numpy as np
import pytest

from helpers import assert_parity
from luminal_b200 import BF16, F16, F32, BlumError, _lib
from luminal_b200.ops import QuantizedGather, QuantizedMatmul
from luminal_b200.runtime import Q8Weight, gen_normal, gen_q8_quants, gen_q8_scales, pack_gguf_q8_0, round_to_dtype

pytestmark = pytest.mark.gpu
GOLD = os.path.join(os.path.dirname(__file__), "golden")


def make_q8(seed, tid, n, k):
    return gen_q8_quants(seed, tid, n * k).reshape(n, k), gen_q8_scales(seed, tid, n * k // 32).reshape(n, k // 32)


def test_repack_is_bit_exact(ctx, orc):
    """GGUF bytes -> two-plane layout -> GGUF bytes; device-side generation equals host generation."""
    for n, k in ((8, 32), (33, 96), (256, 4096), (1000, 1024)):
        q, d = make_q8(1, 50, n, k)
        gguf = pack_gguf_q8_0(q, d)
        w = Q8Weight.from_gguf_bytes(ctx, gguf, n, k)
        pq, pd = w.planes()
        assert np.array_equal(pq, q) and np.array_equal(pd, d)
        assert np.array_equal(w.to_gguf_bytes(), gguf)
        g = Q8Weight.generate(ctx, 1, 50, n, k)
        gq, gd = g.planes()
        assert np.array_equal(gq, q) and np.array_equal(gd, d)
        dev = ctx.to_device_raw(gguf)
        w2 = Q8Weight.from_device_gguf_bytes(ctx, dev, n, k)
        assert np.array_equal(w2.planes()[0], q)


def test_slice_and_concat(ctx):
    q, d = make_q8(1, 51, 96, 256)
    w = Q8Weight.from_gguf_bytes(ctx, pack_gguf_q8_0(q, d), 96, 256)
    s = w.slice(32, 40, 64, 128)
    sq, sd = s.planes()
    assert np.array_equal(sq, q[32:72, 64:192]) and np.array_equal(sd, d[32:72, 2:6])
    a, b = w.slice(0, 32, 0, 256), w.slice(32, 64, 0, 256)
    c = Q8Weight.concat_rows(ctx, [b, a])
    cq, cd = c.planes()
    assert np.array_equal(cq, np.concatenate([q[32:], q[:32]])) and np.array_equal(cd, np.concatenate([d[32:], d[:32]]))
    with pytest.raises(BlumError):
        w.slice(0, 8, 16, 64)          # K must be cut on 32-element block boundaries
    with pytest.raises(BlumError):
        w.slice(90, 8, 0, 256)


@pytest.mark.parametrize("dtype,tol", [(F32, 2e-4), (BF16, None), (F16, None)])
@pytest.mark.parametrize("n,k", [(512, 1024), (8, 32), (100, 96), (1031, 4096), (4096, 14336 // 4)])
def test_matmul_parity_small_m(ctx, orc, dtype, tol, n, k):
    q, d = make_q8(1, 60, n, k)
    w = Q8Weight.from_gguf_bytes(ctx, pack_gguf_q8_0(q, d), n, k)
    for m in (1, 2, 3, 4, 5, 8):
        x = round_to_dtype(gen_normal(1, 61 + m, m * k).reshape(m, k), dtype)
        want = orc.q8_matmul_fast(q, d, x)
        out = QuantizedMatmul(ctx, dtype).process(ctx.to_device(x, dtype), w, m)
        got = ctx.to_host(out, dtype, m * n).reshape(m, n)
        if dtype == F32:
            assert_parity(got, want, max_abs=tol, rel=tol, what="f32 q8 matmul M=%d" % m)
        else:
            # output rounding to a 16-bit type: half an ulp of the result on top of the contract tolerance
            assert_parity(got, want, what="16-bit q8 matmul M=%d" % m)
            assert_parity(got, round_to_dtype(want, dtype), max_abs=2e-2 * max(1e-3, np.abs(want).max()), what="rounded")
    ctx.check_device_error()


def test_matmul_reference_test_shape(ctx, orc):
    """Shape and tolerance class of luminal's own Q8_0 tests (W[512,1024] in 0..5, unit scales, 1e-3)."""
    k = json.load(open(os.path.join(GOLD, "reference_known_answers.json")))["q8_matvec_shape"]
    rng = np.random.default_rng(0)
    q = rng.integers(0, 5, size=(k["N"], k["K"])).astype(np.int8)
    d = np.full((k["N"], k["K"] // 32), np.float16(1.0)).view(np.uint16)
    w = Q8Weight.from_gguf_bytes(ctx, pack_gguf_q8_0(q, d), k["N"], k["K"])
    for m in (k["M_matvec"], k["M_matmul"]):
        x = rng.uniform(-0.5, 0.5, size=(m, k["K"])).astype(np.float32)
        out = QuantizedMatmul(ctx, F32).process(ctx.to_device(x), w, m)
        got = ctx.to_host(out, F32, m * k["N"]).reshape(m, k["N"])
        assert np.abs(got - x.astype(np.float64) @ q.astype(np.float64).T).max() < k["tolerance_abs"]


def test_matmul_against_golden_fixture(ctx):
    from golden.make_golden import Q8_CASES
    g = np.load(os.path.join(GOLD, "oracle_vectors.npz"))
    for i, (n, k, m) in enumerate(Q8_CASES):
        w = Q8Weight.generate(ctx, 1, 100 + i, n, k)
        x = gen_normal(1, 200 + i, m * k).reshape(m, k)
        got = ctx.to_host(QuantizedMatmul(ctx, F32).process(ctx.to_device(x), w, m), F32, m * n).reshape(m, n)
        assert_parity(got, g["q8_matmul_%d" % i], max_abs=2e-4, rel=2e-4, what="golden f32 %d" % i)
        got = ctx.to_host(QuantizedMatmul(ctx, BF16, F32).process(ctx.to_device(x, BF16), w, m), F32, m * n).reshape(m, n)
        if m <= 2:      # GEMV family: f32-grade
            assert_parity(got, g["q8_matmul_bf16in_%d" % i], max_abs=2e-4, rel=2e-4, what="golden bf16-in %d" % i)
        else:           # tensor-core path: weights rounded to bf16, contract tolerance
            assert_parity(got, g["q8_matmul_bf16in_%d" % i], what="golden bf16-in %d (tensor cores)" % i)


def test_both_gemv_kernels_agree(ctx, orc):
    """f32 activations take the integer-dot-product kernel, 16-bit activations the float-form kernel: same product."""
    n, k = 648, 2048                                   # N not a multiple of the rows a CTA covers
    q, d = make_q8(1, 70, n, k)
    w = Q8Weight.from_gguf_bytes(ctx, pack_gguf_q8_0(q, d), n, k)
    for m in (1, 2):
        x = round_to_dtype(gen_normal(1, 71 + m, m * k).reshape(m, k), BF16)      # exactly representable in both
        want = orc.q8_matmul_fast(q, d, x)
        for dtype in (F32, BF16):
            got = ctx.to_host(QuantizedMatmul(ctx, dtype, F32).process(ctx.to_device(x, dtype), w, m), F32, m * n).reshape(m, n)
            assert_parity(got, want, max_abs=2e-4, rel=2e-4, what="gemv M=%d in=%s" % (m, dtype))
    ctx.check_device_error()


def test_fused_norm_residual_and_swiglu(ctx, orc):
    n, k = 768, 1024
    q, d = make_q8(1, 80, n, k)
    q2, d2 = make_q8(1, 81, n, k)
    w = Q8Weight.from_gguf_bytes(ctx, pack_gguf_q8_0(q, d), n, k)
    w2 = Q8Weight.from_gguf_bytes(ctx, pack_gguf_q8_0(q2, d2), n, k)
    for m in (1, 3):
        x = gen_normal(1, 82, m * k).reshape(m, k) * 3
        nw = (1 + 0.1 * gen_normal(1, 83, k)).astype(np.float32)
        res = gen_normal(1, 84, m * n).reshape(m, n)
        xn = orc.rmsnorm(x, nw, 1e-5)
        want = res + orc.q8_matmul_fast(q, d, xn)
        xd, nwd, resd, out = ctx.to_device(x), ctx.to_device(nw), ctx.to_device(res), ctx.alloc(m * n * 4)
        ctx._check(ctx.lib.blum_q8_0_matmul_fused(ctx.h, w.h, xd.ptr, F32, nwd.ptr, 1e-5, resd.ptr, out.ptr, F32, m))
        assert_parity(ctx.to_host(out, F32, m * n), want, max_abs=5e-4, rel=5e-4, what="fused norm+residual M=%d" % m)
        # residual aliasing the output (x += W y)
        ctx._check(ctx.lib.blum_q8_0_matmul_fused(ctx.h, w.h, xd.ptr, F32, nwd.ptr, 1e-5, resd.ptr, resd.ptr, F32, m))
        assert_parity(ctx.to_host(resd, F32, m * n), want, max_abs=5e-4, rel=5e-4, what="aliased residual")
        want_sw = orc.swiglu(orc.q8_matmul_fast(q, d, xn), orc.q8_matmul_fast(q2, d2, xn))
        ctx._check(ctx.lib.blum_q8_0_matmul_swiglu(ctx.h, w.h, w2.h, xd.ptr, F32, nwd.ptr, 1e-5, out.ptr, F32, m))
        assert_parity(ctx.to_host(out, F32, m * n), want_sw, max_abs=5e-4, rel=5e-4, what="swiglu M=%d" % m)


def test_quantized_gather(ctx, orc):
    n, k = 300, 256
    q, d = make_q8(1, 90, n, k)
    gguf = pack_gguf_q8_0(q, d)
    w = Q8Weight.from_gguf_bytes(ctx, gguf, n, k)
    ids = np.array([0, 299, 17, 17, 5.9], np.float32)   # ids travel as f32 and are truncated
    got = ctx.to_host(QuantizedGather(ctx, k, F32).process(ids, w), F32, ids.size * k).reshape(-1, k)
    assert np.array_equal(got, orc.q8_gather(gguf, k, ids))


def test_error_paths(ctx):
    lib = ctx.lib
    w = Q8Weight.generate(ctx, 1, 95, 32, 64)
    buf = ctx.alloc(1024)
    assert lib.blum_q8_0_matmul(ctx.h, w.h, None, F32, buf.ptr, F32, 1) == _lib.ERR_INVALID
    assert b"null" in lib.blum_last_error(ctx.h)
    assert lib.blum_q8_0_matmul(ctx.h, w.h, buf.ptr, 7, buf.ptr, F32, 1) == _lib.ERR_INVALID
    assert lib.blum_q8_0_matmul(ctx.h, w.h, buf.ptr, F32, buf.ptr, F32, -3) == _lib.ERR_INVALID
    assert lib.blum_q8_0_matmul(ctx.h, w.h, buf.ptr, F32, buf.ptr, F32, 0) == 0       # empty input is a no-op
    h = np.zeros(1, np.uint64)
    assert lib.blum_q8_0_weight_from_gguf_bytes(ctx.h, buf.ptr, 4, 48, h.ctypes.data) == _lib.ERR_INVALID   # K % 32 != 0
    assert lib.blum_q8_0_weight_from_gguf_bytes(ctx.h, buf.ptr, 0, 64, h.ctypes.data) == _lib.ERR_INVALID
    ctx.sync()


@pytest.mark.parametrize("k,n", [(4096, 4096), (4096, 14336), (14336, 4096), (8192, 28672)])
def test_full_size_properties(ctx, k, n):
    """Sizes of the operator sweep, checked through size-independent properties instead of the (slow) oracle:
    linearity in x, a row subset against the oracle-free exact integer model, and scale homogeneity."""
    w = Q8Weight.generate(ctx, 1, 1000 + k + n, n, k)
    mm = QuantizedMatmul(ctx, F32)
    x1, x2 = gen_normal(1, 1, k), gen_normal(1, 2, k)
    y1 = ctx.to_host(mm.process(ctx.to_device(x1), w, 1), F32, n)
    y2 = ctx.to_host(mm.process(ctx.to_device(x2), w, 1), F32, n)
    y12 = ctx.to_host(mm.process(ctx.to_device(x1 + 2 * x2), w, 1), F32, n)
    assert_parity(y12, y1 + 2 * y2, max_abs=1e-3, rel=1e-3, what="linearity")
    # rows 0, n/2 and n-1 against float64 math on the generated values
    rows = [0, n // 2, n - 1]
    q = np.stack([gen_q8_quants(1, 1000 + k + n, (r + 1) * k)[-k:] for r in rows]) if n * k < (1 << 26) else None
    if q is not None:
        d = np.stack([gen_q8_scales(1, 1000 + k + n, (r + 1) * k // 32)[-(k // 32):] for r in rows])
        wrow = q.astype(np.float64) * np.repeat(d.view(np.float16).astype(np.float64), 32, axis=1)
        assert_parity(y1[rows], wrow @ x1.astype(np.float64), max_abs=1e-3, rel=1e-3, what="row subset")
    # two rows of x at once equal the two single-row results
    y = ctx.to_host(mm.process(ctx.to_device(np.stack([x1, x2])), w, 2), F32, 2 * n).reshape(2, n)
    assert_parity(y[0], y1, max_abs=1e-6, rel=1e-6, what="row 0 of M=2")
    assert_parity(y[1], y2, max_abs=1e-6, rel=1e-6, what="row 1 of M=2")
