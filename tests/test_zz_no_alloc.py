"""The allocation-free split-decode attention entry point (blum_attn_decode_paged_static).

It exists for callers that must not allocate while serving - a runtime that handed all device memory out at
start-up, or a decode thread that cannot afford the device-wide synchronisation of cudaMalloc/cudaFree - and keeps
its split partials in a buffer built into the library.  The test drives it through the C ABI and checks it against
the ordinary entry point (caller-provided scratch) on two calls in a row, so that whatever the first call left in
the shared buffer is shown not to leak into the second.  This file sorts last on purpose: a run that stops at the
first failure has already run every other test.
"""
import ctypes

import numpy as np
import pytest

from luminal_b200 import BF16, F32, _lib
from luminal_b200.llama import KvCache
from luminal_b200.runtime import gen_normal, round_to_dtype

pytestmark = pytest.mark.gpu


def _setup(ctx, dtype, lens, nq, nkv, d, seed):
    ps = 16
    pages = sum((n + ps - 1) // ps for n in lens)
    kv = KvCache(ctx, 1, nkv, d, ps, num_pages=pages, max_seqs=len(lens), max_pages_per_seq=(max(lens) + ps - 1) // ps, dtype=dtype)
    for i, n in enumerate(lens):
        s = kv.seq_alloc()
        kv.seq_extend(s, n)
        k = round_to_dtype(gen_normal(seed, 10 + i, n * nkv * d).reshape(n, nkv * d), dtype)
        v = round_to_dtype(gen_normal(seed, 40 + i, n * nkv * d).reshape(n, nkv * d), dtype)
        kv.append(0, ctx.to_device(k, dtype), ctx.to_device(v, dtype), dtype, [s] * n, list(range(n)))
    q = ctx.to_device(round_to_dtype(gen_normal(seed, 99, len(lens) * nq * d), dtype), dtype)
    return kv, q


def _free_device_bytes():
    try:
        rt = ctypes.CDLL("libcudart.so.12")      # the runtime libblum.so is linked against, already loaded
    except OSError:
        rt = ctypes.CDLL("libcudart.so")
    free, total = ctypes.c_size_t(), ctypes.c_size_t()
    assert rt.cudaMemGetInfo(ctypes.byref(free), ctypes.byref(total)) == 0
    return free.value


def _oracle_attention(orc, kv, q_host, lens, nq, nkv, d, seed, dtype):
    """Decode attention of every sequence through the CPU oracle: the cache is rebuilt in the reference's contiguous
    [kv_heads, ctx, head_dim] layout from the same seeded rows the pool was filled with."""
    out = []
    for i, n in enumerate(lens):
        k = round_to_dtype(gen_normal(seed, 10 + i, n * nkv * d).reshape(n, nkv, d), dtype)
        v = round_to_dtype(gen_normal(seed, 40 + i, n * nkv * d).reshape(n, nkv, d), dtype)
        kc, vc = np.ascontiguousarray(k.transpose(1, 0, 2)), np.ascontiguousarray(v.transpose(1, 0, 2))
        out.append(orc.attention(q_host[i].reshape(1, nq * d), kc, vc, 1, n - 1, nq, nkv, d, n)[0])
    return np.concatenate(out)


def _static(ctx, kv, q, dtype, nq, lens, splits):
    B = len(lens)
    seqs = ctx.to_device_raw(np.arange(B, dtype=np.int32))
    cl = ctx.to_device_raw(np.asarray(lens, np.int32))
    out = ctx.alloc(B * nq * kv.head_dim * (4 if dtype == F32 else 2))
    ctx._check(ctx.lib.blum_attn_decode_paged_static(ctx.h, kv.h, 0, q.ptr, dtype, nq, seqs.ptr, cl.ptr, B, splits, out.ptr))
    return ctx.to_host(out, dtype, B * nq * kv.head_dim)


@pytest.mark.parametrize("dtype", [F32, BF16])
def test_static_scratch_matches_caller_scratch_twice(ctx, orc, dtype):
    nq, nkv, d = 8, 2, 128
    # first call: long contexts, many splits; second call: different data and fewer splits over the same buffer
    for seed, lens, splits in ((11, [900, 33, 512, 700], 7), (12, [64, 300], 3)):
        kv, q = _setup(ctx, dtype, lens, nq, nkv, d, seed)
        want = ctx.to_host(kv.attn_decode(0, q, dtype, nq, list(range(len(lens))), lens, max_splits=splits), dtype, len(lens) * nq * d)
        got = _static(ctx, kv, q, dtype, nq, lens, splits)
        tol = 2e-5 if dtype == F32 else 1e-2          # same tolerances as the attention tests
        assert np.abs(got - want).max() <= tol * max(1.0, np.abs(want).max())
        # and against the CPU oracle directly, so that this test does not lean on the sibling entry point being right
        q_host = round_to_dtype(gen_normal(seed, 99, len(lens) * nq * d), dtype).reshape(len(lens), nq * d)
        ref = _oracle_attention(orc, kv, q_host, lens, nq, nkv, d, seed, dtype)
        assert np.abs(got - ref).max() <= tol * max(1.0, np.abs(ref).max())
        kv.destroy()
    ctx.check_device_error()


def test_static_scratch_call_allocates_no_device_memory(ctx):
    """Free device memory is the same before and after a warm call (the first call on a device only looks an address up).
    Inputs, outputs and index arrays are the caller's and exist before the measurement starts."""
    lens, nq = [700, 90], 8
    kv, q = _setup(ctx, F32, lens, nq, 2, 128, 14)
    _static(ctx, kv, q, F32, nq, lens, 5)                      # warm: address lookup, page table upload, kernel load
    seqs = ctx.to_device_raw(np.arange(2, dtype=np.int32))
    cl = ctx.to_device_raw(np.asarray(lens, np.int32))
    out = ctx.alloc(2 * nq * 128 * 4)
    ctx.sync()
    before = _free_device_bytes()
    for _ in range(3):
        ctx._check(ctx.lib.blum_attn_decode_paged_static(ctx.h, kv.h, 0, q.ptr, F32, nq, seqs.ptr, cl.ptr, 2, 5, out.ptr))
    ctx.sync()
    assert _free_device_bytes() == before
    kv.destroy()


def test_static_scratch_rejects_oversized_requests(ctx):
    kv, q = _setup(ctx, F32, [40], 8, 2, 128, 13)
    cap = ctx.lib.blum_attn_decode_static_scratch_bytes()
    assert cap == 8 << 20
    seqs = ctx.to_device_raw(np.zeros(1, np.int32))
    cl = ctx.to_device_raw(np.array([40], np.int32))
    out = ctx.alloc(8 * 128 * 4)
    too_many_rows = cap // (8 * 4 * 130 * 4) + 1          # B that no longer fits with 4 splits
    rc = ctx.lib.blum_attn_decode_paged_static(ctx.h, kv.h, 0, q.ptr, F32, 8, seqs.ptr, cl.ptr, too_many_rows, 4, out.ptr)
    assert rc == _lib.ERR_INVALID
    msg = ctx.lib.blum_last_error(ctx.h).decode()
    assert "scratch" in msg and str(cap) in msg
    # a single split needs no scratch at all and is always accepted
    ctx._check(ctx.lib.blum_attn_decode_paged_static(ctx.h, kv.h, 0, q.ptr, F32, 8, seqs.ptr, cl.ptr, 1, 1, out.ptr))
    ctx.sync()
    kv.destroy()
