"""Q8_0 tensor-core GEMM (tcgen05 + TMEM) against the CPU oracle, through blum_q8_0_matmul with bf16 activations."""
import numpy as np
import pytest

from helpers import assert_parity
from luminal_b200 import BF16, F32
from luminal_b200.ops import QuantizedMatmul
from luminal_b200.runtime import Q8Weight, gen_normal, gen_q8_quants, gen_q8_scales, round_to_dtype

pytestmark = pytest.mark.gpu


def make_q8(seed, tid, n, k):
    return gen_q8_quants(seed, tid, n * k).reshape(n, k), gen_q8_scales(seed, tid, n * k // 32).reshape(n, k // 32)


def check(ctx, orc, n, k, m, out_dtype, tid):
    q, d = make_q8(1, tid, n, k)
    w = Q8Weight.generate(ctx, 1, tid, n, k)
    x = round_to_dtype(gen_normal(1, tid + 1, m * k).reshape(m, k), BF16)
    want = orc.q8_matmul_fast(q, d, x)
    out = QuantizedMatmul(ctx, BF16, out_dtype).process(ctx.to_device(x, BF16), w, m)
    got = ctx.to_host(out, out_dtype, m * n).reshape(m, n)
    ctx.check_device_error()
    # bf16 weights (8-bit significand of q*d) and, for bf16 output, one more rounding: the contract tolerance
    # (a bf16 result near 4 already carries a rounding step of 2^-7 * 4 / 2 = 0.016 / 2, hence the scale term)
    tol = 1e-2 if out_dtype == F32 else max(1e-2, 2.0 ** -8 * np.abs(want).max() + 5e-3)
    assert_parity(got, want, max_abs=tol, what="tc gemm N=%d K=%d M=%d" % (n, k, m))
    # and it has to be far better than the contract on average: a layout or descriptor mistake is not subtle
    assert np.abs(got - want).mean() < 2e-3 * max(np.abs(want).mean(), 1e-6) + (2e-3 if out_dtype == BF16 else 0) * np.abs(want).mean()
    w.free()


@pytest.mark.parametrize("m", [9, 16, 32, 33, 64, 100, 128, 129, 256, 300])
def test_tc_gemm_small_shapes(ctx, orc, m):
    check(ctx, orc, 256, 512, m, F32, 300)
    check(ctx, orc, 200, 1024, m, BF16, 310)      # N not a multiple of the 128-row tile


@pytest.mark.parametrize("n,k,m", [(4096, 4096, 64), (1024, 4096, 512), (512, 14336, 64), (14336, 4096, 16)])
def test_tc_gemm_model_shapes(ctx, orc, n, k, m):
    check(ctx, orc, n, k, m, BF16, 320)


@pytest.mark.parametrize("k,n", [(4096, 4096), (4096, 14336), (14336, 4096), (8192, 28672)])
def test_operator_sweep_sizes_on_a_sub_block(ctx, k, n):
    """Every (K, N) of the operator sweep at M in {8, 64, 512, 4096} (and two ragged row counts), bf16 in and out: several token tiles at full N,
    split-K at full size and the ragged last tiles.  The full products are too slow for the CPU oracle, so a sub-block is
    checked instead: up to 64 rows of x (first, last and scattered) times 256 output columns (the first and the last
    128-row weight tile plus scattered ones), computed in float64 from the host generator's quants and scales."""
    tid = 2000 + k + n
    w = Q8Weight.generate(ctx, 1, tid, n, k)
    q, d = make_q8(1, tid, n, k)
    rng = np.random.default_rng(k + n)
    cols = np.unique(np.concatenate([np.arange(0, 64), np.arange(n - 64, n), rng.integers(64, n - 64, 128)]))
    wsub = q[cols].astype(np.float64) * np.repeat(d[cols].view(np.float16).astype(np.float64), 32, axis=1)
    mm = QuantizedMatmul(ctx, BF16, BF16)
    # 700 and 1300 rows: CTAs that hold two 256-row token tiles meet a ragged and a wholly empty second tile
    for m in (8, 64, 512, 4096) + ((700, 1300) if n == 14336 else ()):
        x = round_to_dtype(gen_normal(1, tid + m, m * k).reshape(m, k), BF16)
        rows = np.unique(np.concatenate([np.arange(0, min(m, 8)), np.arange(max(m - 8, 0), m), rng.integers(0, m, 48)]))
        got = ctx.to_host(mm.process(ctx.to_device(x, BF16), w, m), BF16, m * n).reshape(m, n)[np.ix_(rows, cols)]
        ctx.check_device_error()
        want = x[rows].astype(np.float64) @ wsub.T
        tol = max(1e-2, 2.0 ** -8 * np.abs(want).max() + 5e-3)       # as in check(): one bf16 rounding step of the output
        assert_parity(got, want, max_abs=tol, what="tc gemm sub-block N=%d K=%d M=%d" % (n, k, m))
        assert np.abs(got - want).mean() < 4e-3 * np.abs(want).mean()
        if m == 700:
            # the same ragged product with f32 output (two token tiles per CTA, f32 stores): no output rounding
            got32 = ctx.to_host(QuantizedMatmul(ctx, BF16, F32).process(ctx.to_device(x, BF16), w, m), F32, m * n).reshape(m, n)[np.ix_(rows, cols)]
            ctx.check_device_error()
            assert_parity(got32, want, max_abs=1e-2, what="tc gemm sub-block f32 out N=%d K=%d M=%d" % (n, k, m))
    w.free()


def test_tc_gemm_matches_gemv_on_same_rows(ctx, orc):
    """Row 0 of an M=64 tensor-core product equals the M=1 GEMV of the same row (different kernels, same math)."""
    n, k = 1024, 2048
    w = Q8Weight.generate(ctx, 1, 330, n, k)
    x = round_to_dtype(gen_normal(1, 331, 64 * k).reshape(64, k), BF16)
    big = ctx.to_host(QuantizedMatmul(ctx, BF16, F32).process(ctx.to_device(x, BF16), w, 64), F32, 64 * n).reshape(64, n)
    one = ctx.to_host(QuantizedMatmul(ctx, BF16, F32).process(ctx.to_device(x[:1], BF16), w, 1), F32, n)
    assert_parity(big[0], one, max_abs=5e-3, rel=5e-3, what="tc gemm row vs gemv")


@pytest.mark.parametrize("m", [3, 4, 5, 8, 15, 16])
def test_small_batch_kernel_shapes(ctx, orc, m):
    """Batches of 3..16 rows take the register-streaming mma.sync kernel (K a multiple of 256): ragged N (not a multiple
    of its 32-row tasks), K of one and of several chunks with a partial last 512-chunk, f32 and bf16 outputs, a shape with
    more row blocks than one, and a model shape."""
    check(ctx, orc, 100, 256, m, F32, 340)        # N ragged, a single chunk
    check(ctx, orc, 1000, 1280, m, BF16, 350)     # several chunks; 2.5 chunks of 512
    check(ctx, orc, 2100, 768, m, F32, 355)       # several row blocks, the last one ragged
    check(ctx, orc, 4096, 4096, m, BF16, 360)


def test_small_batch_kernel_matches_gemv_on_same_rows(ctx, orc):
    """Every row of an M=8 product equals the M=1 GEMV of that row up to the bf16 rounding of the weights."""
    n, k = 512, 2048
    w = Q8Weight.generate(ctx, 1, 370, n, k)
    x = round_to_dtype(gen_normal(1, 371, 8 * k).reshape(8, k), BF16)
    big = ctx.to_host(QuantizedMatmul(ctx, BF16, F32).process(ctx.to_device(x, BF16), w, 8), F32, 8 * n).reshape(8, n)
    for r in (0, 7):
        one = ctx.to_host(QuantizedMatmul(ctx, BF16, F32).process(ctx.to_device(x[r:r + 1], BF16), w, 1), F32, n)
        assert_parity(big[r], one, max_abs=5e-3, rel=5e-3, what="small-batch kernel row %d vs gemv" % r)
    w.free()
