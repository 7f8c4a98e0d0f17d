"""Row-wise / elementwise kernels on the GPU against the CPU oracle and the golden fixtures."""
import json
import os

import numpy as np
import pytest

from helpers import assert_parity
from luminal_b200 import BF16, F16, F32, BlumError
from luminal_b200 import ops
from luminal_b200.runtime import gen_normal, round_to_dtype

pytestmark = pytest.mark.gpu
GOLD = os.path.join(os.path.dirname(__file__), "golden")


@pytest.fixture(scope="module")
def gold():
    return np.load(os.path.join(GOLD, "oracle_vectors.npz"))


def test_embedding_known_answer(ctx):
    k = json.load(open(os.path.join(GOLD, "reference_known_answers.json")))["embedding"]
    table = ctx.to_device(np.array(k["weight_3x4"], np.float32))
    g = ops.CudaGather(ctx, 4, F32)
    assert np.array_equal(ctx.to_host(g.process(k["ids_single"], table, 3), F32, 12), np.array(k["expected_single"], np.float32))
    assert np.array_equal(ctx.to_host(g.process(k["ids_batch_2x3"], table, 3), F32, 24), np.array(k["expected_batch"], np.float32))


def test_gather_out_of_range_sets_error_word(ctx):
    table = ctx.to_device(np.arange(12, dtype=np.float32))
    ops.CudaGather(ctx, 4, F32).process([5.0], table, 3)
    with pytest.raises(BlumError):
        ctx.check_device_error()
    ctx.check_device_error()   # cleared by the read


@pytest.mark.parametrize("dtype", [F32, BF16, F16])
@pytest.mark.parametrize("rows,dim", [(15, 32), (1, 4096), (7, 8192), (3, 2880 - 2880 % 8)])
def test_rmsnorm(ctx, orc, dtype, rows, dim):
    x = round_to_dtype(gen_normal(2, 1, rows * dim).reshape(rows, dim) * 2, dtype)
    w = (1 + 0.2 * gen_normal(2, 2, dim)).astype(np.float32)
    norm = ops.CudaStdNorm(ctx, 1e-5, dtype)
    got = ctx.to_host(norm.process(ctx.to_device(x, dtype), rows, dim, ctx.to_device(w)), dtype, rows * dim)
    tol = 1e-5 if dtype == F32 else 2e-2
    assert_parity(got, orc.rmsnorm(x, w, 1e-5), max_abs=tol * 8, rel=tol, what="rmsnorm")
    got = ctx.to_host(norm.process(ctx.to_device(x, dtype), rows, dim), dtype, rows * dim)
    assert_parity(got, orc.rmsnorm(x, None, 1e-5), max_abs=tol * 8, rel=tol, what="stdnorm")


def test_rmsnorm_with_residual(ctx, orc):
    rows, dim = 5, 1024
    x, r = gen_normal(2, 3, rows * dim).reshape(rows, dim), gen_normal(2, 4, rows * dim).reshape(rows, dim)
    w = (1 + 0.2 * gen_normal(2, 5, dim)).astype(np.float32)
    xd, rd, wd = ctx.to_device(x), ctx.to_device(r), ctx.to_device(w)
    y, s = ctx.alloc(rows * dim * 4), ctx.alloc(rows * dim * 4)
    ctx._check(ctx.lib.blum_rmsnorm(ctx.h, xd.ptr, rd.ptr, wd.ptr, 1e-5, y.ptr, s.ptr, F32, rows, dim))
    assert np.array_equal(ctx.to_host(s, F32, rows * dim).reshape(rows, dim), x + r)
    assert_parity(ctx.to_host(y, F32, rows * dim), orc.rmsnorm(x + r, w, 1e-5), max_abs=1e-5, rel=1e-5, what="residual norm")


def test_rmsnorm_golden(ctx, gold):
    x, w = gen_normal(1, 300, 6 * 256).reshape(6, 256), gen_normal(1, 301, 256)
    got = ctx.to_host(ops.CudaStdNorm(ctx, 1e-5, F32).process(ctx.to_device(x), 6, 256, ctx.to_device(w)), F32, 6 * 256)
    assert_parity(got, gold["rmsnorm"], max_abs=2e-5, rel=1e-5, what="rmsnorm golden")


@pytest.mark.parametrize("dtype", [F32, BF16])
def test_rope(ctx, orc, gold, dtype):
    pos = np.array([0, 1, 17, 511, 4095])
    x = round_to_dtype(gen_normal(1, 302, 5 * 4 * 128).reshape(5, 4, 128), dtype)
    buf = ops.rope_interleaved(ctx, ctx.to_device(x, dtype), pos, 4, 128, 500000.0, dtype)
    got = ctx.to_host(buf, dtype, x.size).reshape(x.shape)
    if dtype == F32:
        assert_parity(got, gold["rope"], max_abs=5e-4, rel=5e-4, what="rope golden")
        assert_parity(got, orc.rope(x, pos, 4, 128, 500000.0), max_abs=5e-4, rel=5e-4, what="rope")
        assert np.abs(got[0] - x[0]).max() < 1e-6        # position 0 is the identity
    else:
        assert_parity(got, orc.rope(x, pos, 4, 128, 500000.0), what="rope bf16")
    # the reference's own RoPE test shape (heads 8, seq 2, head_dim 4, theta 1e6)
    x2 = round_to_dtype(gen_normal(1, 310, 2 * 8 * 4).reshape(2, 8, 4), dtype)
    got2 = ctx.to_host(ops.rope_interleaved(ctx, ctx.to_device(x2, dtype), [0, 1], 8, 4, 1e6, dtype), dtype, 64)
    assert_parity(got2, orc.rope(x2, [0, 1], 8, 4, 1e6), what="rope reference shape")


@pytest.mark.parametrize("dtype", [F32, BF16, F16])
def test_swiglu_add(ctx, orc, gold, dtype):
    for n in (777, 14336, 5):
        g = round_to_dtype(gen_normal(1, 303, n), dtype)
        u = round_to_dtype(gen_normal(1, 304, n), dtype)
        got = ctx.to_host(ops.swiglu(ctx, ctx.to_device(g, dtype), ctx.to_device(u, dtype), n, dtype), dtype, n)
        if dtype == F32:
            assert_parity(got, orc.swiglu(g, u), max_abs=1e-6, rel=1e-6, what="swiglu")
        else:   # one rounding to the 16-bit output type: an ulp relative to each element
            want = orc.swiglu(g, u)
            assert np.all(np.abs(got - want) <= 2.0 ** -7 * np.abs(want) + 1e-6), "swiglu 16-bit"
        got = ctx.to_host(ops.add(ctx, ctx.to_device(g, dtype), ctx.to_device(u, dtype), n, dtype), dtype, n)
        assert np.array_equal(got, round_to_dtype(g + u, dtype))
    if dtype == F32:
        g, u = gen_normal(1, 303, 777), gen_normal(1, 304, 777)
        got = ctx.to_host(ops.swiglu(ctx, ctx.to_device(g), ctx.to_device(u), 777), F32, 777)
        assert_parity(got, gold["swiglu"], max_abs=1e-6, rel=1e-6, what="swiglu golden")


def test_softmax(ctx, orc, gold):
    x = gen_normal(1, 305, 4 * 333, 3.0).reshape(4, 333)
    got = ctx.to_host(ops.CudaSoftmax(ctx, F32).process(ctx.to_device(x), 4, 333), F32, x.size).reshape(x.shape)
    assert_parity(got, gold["softmax"], max_abs=1e-6, rel=1e-5, what="softmax golden")
    assert np.abs(got.sum(-1) - 1).max() < 1e-5
    big = gen_normal(1, 306, 2 * 4097, 5.0).reshape(2, 4097)
    got = ctx.to_host(ops.CudaSoftmax(ctx, F32).process(ctx.to_device(big), 2, 4097), F32, big.size).reshape(big.shape)
    assert_parity(got, orc.softmax(big), max_abs=2e-5, rel=1e-4, what="softmax wide")   # summation order differs


def test_argmax_greedy_rule(ctx, orc):
    """examples/llama/src/main.rs:194-198: last maximum wins; NaN rows follow the sequential fold."""
    rows = [np.array([1, 5, 3, 5, 2], np.float32), np.array([7, 7, 7, 7, 7], np.float32),
            np.array([1, np.nan, 0.5, 0.25, 0.1], np.float32), np.array([3, 1, 2, 0, np.nan], np.float32)]
    x = np.stack(rows)
    got = ops.argmax(ctx, ctx.to_device_raw(x), 4, 5)
    assert got.tolist() == [orc.argmax(r) for r in rows] == [3, 4, 2, 4]
    v = gen_normal(3, 1, 128256)
    v[[5, 99999, 128255]] = 9.0   # three equal maxima: the last index is returned
    assert ops.argmax(ctx, ctx.to_device(v), 1, 128256)[0] == 128255 == orc.argmax(v)
    m = gen_normal(3, 2, 3 * 1000).reshape(3, 1000)
    assert ops.argmax(ctx, ctx.to_device(m), 3, 1000).tolist() == [orc.argmax(r) for r in m]


def test_argmax_rows_split_over_several_ctas(ctx, orc):
    """Wide f32 rows are split over CTAs that join 64-bit {value, index} keys: ties across parts, signed zeros, -inf rows,
    NaN rows, odd widths (the scalar-load form), and a second call on the same context (the records return to zero)."""
    for cols in (128256, 32768, 9001):
        m = gen_normal(3, 40 + cols % 7, 6 * cols).reshape(6, cols)
        m[0, [3, cols // 2, cols - 2]] = 11.0                       # equal maxima in different parts: the last one
        m[1, :] = -np.inf                                           # every element equal: the last index
        m[2, :] = -1.0
        m[2, [17, cols - 100]] = [0.0, -0.0]                        # +0 then -0 compare equal: the later index
        m[3, [5, cols - 9]] = [-0.0, 0.0]
        m[3, m[3] > 0] = -1.0
        m[4, cols // 3] = np.nan                                    # the sequential fold of the reference
        want = [orc.argmax(r) for r in m]
        assert want[0] == cols - 2 and want[1] == cols - 1 and want[2] == cols - 100 and want[3] == cols - 9
        d = ctx.to_device(m)
        for _ in range(2):
            assert ops.argmax(ctx, d, 6, cols).tolist() == want, cols
    one = gen_normal(3, 77, 128256)
    assert ops.argmax(ctx, ctx.to_device(one), 1, 128256)[0] == orc.argmax(one)
    ctx.check_device_error()
