"""Tensor-parallel decoder over NCCL: one process per GPU (needs at least 2 GPUs; skipped otherwise)."""
import multiprocessing as mp
import os
import sys
import tempfile

import numpy as np
import pytest

pytestmark = pytest.mark.gpu
GOLD = os.path.join(os.path.dirname(__file__), "golden")


def _gpu_count():
    try:
        import ctypes
        rt = ctypes.CDLL("libcudart.so")
        n = ctypes.c_int()
        return n.value if rt.cudaGetDeviceCount(ctypes.byref(n)) == 0 else 0
    except OSError:
        return 0


def _run_ranks(target, size, per_item_timeout=240):
    """Starts one daemon child per rank, collects one result tuple each (last field = traceback or None) and ALWAYS
    terminates and joins every child, whatever happened: a rank that failed after the communicator was set up leaves
    its peer inside a collective that cannot complete, so the parent ends the peers as soon as the first failure
    is reported or a result does not arrive in time."""
    ctxm = mp.get_context("spawn")
    q = ctxm.Queue()
    results = []
    with tempfile.TemporaryDirectory() as td:
        procs = [ctxm.Process(target=target, args=(r, size, os.path.join(td, "nccl_id"), q), daemon=True) for r in range(size)]
        try:
            for p in procs:
                p.start()
            for _ in range(size):
                try:
                    item = q.get(timeout=per_item_timeout)
                except Exception:
                    results.append((None, "no result from a rank within %d s" % per_item_timeout))
                    break
                results.append(item)
                if item[-1] is not None:      # a rank failed: do not wait for its peers
                    break
        finally:
            failed = any(r[-1] is not None for r in results) or len(results) < size
            for p in procs:
                if not failed:
                    p.join(timeout=60)
                if p.is_alive():
                    p.terminate()             # this exact child only
                    p.join(timeout=10)
                if p.is_alive():
                    p.kill()
                    p.join(timeout=10)
    for r in results:
        assert r[-1] is None, "rank %s failed:\n%s" % (r[0], r[-1])
    assert len(results) == size
    return results


def _rank_main(rank, size, id_path, out_q):
    try:
        here = os.path.dirname(os.path.abspath(__file__))
        for p in (os.path.dirname(here), here):
            if p not in sys.path:
                sys.path.insert(0, p)
        os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
        from helpers import TINY_CFG, make_weights
        from luminal_b200 import F32, Context
        from luminal_b200.dist import Comm
        from luminal_b200.llama import Llama
        from oracle import oracle as orc
        ctx = Context(rank)
        comm = Comm(ctx, size, rank, Comm.exchange_id_via_file(id_path, rank))
        # plain all-reduce first
        buf = ctx.to_device(np.full(1000, rank + 1, np.float32))
        comm.allreduce_sum(buf, 1000, F32)
        ar = ctx.to_host(buf, F32, 1000)
        model = Llama(ctx, TINY_CFG, act_dtype=F32, page_size=4, max_seqs=2, max_ctx=64, tp_rank=rank, tp_size=size)
        model.set_comm(comm)
        model.load_weights(make_weights(orc, TINY_CFG, seed=0))     # every rank is handed the full tensors and keeps its window
        prompt = orc.gen_token_ids(0, 1, 6, TINY_CFG["vocab"])
        toks = model.greedy(prompt, 8)
        ctx.check_device_error()
        model.destroy()
        comm.destroy()
        out_q.put((rank, ar.tolist()[:3], toks, None))
    except Exception as e:   # report instead of hanging the parent
        import traceback
        out_q.put((rank, None, None, traceback.format_exc()))


@pytest.mark.skipif(_gpu_count() < 2, reason="needs 2 GPUs")
def test_tensor_parallel_greedy_ids_match_golden():
    size = 2
    g = np.load(os.path.join(GOLD, "oracle_vectors.npz"))
    results = _run_ranks(_rank_main, size)
    for rank, ar, toks, err in results:
        assert err is None, "rank %d failed:\n%s" % (rank, err)
        assert ar == [3.0, 3.0, 3.0]                       # 1 + 2 summed over the two ranks
        assert toks == g["llama_greedy_ids"].tolist(), (rank, toks)


def _ep_rank_main(rank, size, id_path, out_q):
    try:
        here = os.path.dirname(os.path.abspath(__file__))
        for p in (os.path.dirname(here), here):
            if p not in sys.path:
                sys.path.insert(0, p)
        os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
        from luminal_b200 import BF16, F32, Context
        from luminal_b200.dist import Comm
        from luminal_b200.moe import ExpertParallelMoe, MoeFfn, Mxfp4Weight
        from luminal_b200.runtime import gen_normal, round_to_dtype
        ctx = Context(rank)
        comm = Comm(ctx, size, rank, Comm.exchange_id_via_file(id_path, rank))
        H, I, E, k, T = 256, 384, 8, 2, 70 + 30 * rank          # ranks own different numbers of tokens
        EL = E // size
        full = [Mxfp4Weight.generate(ctx, 4, 910 + i, E, n, kk) for i, (n, kk) in enumerate(((I, H), (I, H), (H, I)))]
        mine = []
        for w in full:                                           # this rank's slice of the stacked experts
            q, s = w.download()
            mine.append(Mxfp4Weight.from_host(ctx, q[rank * EL:(rank + 1) * EL], s[rank * EL:(rank + 1) * EL], EL, w.N, w.K))
        router = ctx.to_device(round_to_dtype(gen_normal(4, 920, E * H, 0.02).reshape(E, H), BF16), BF16)
        bias = ctx.to_device((-0.05 * 1.1 * np.log(np.arange(1, E + 1))).astype(np.float32))
        x = ctx.to_device(round_to_dtype(gen_normal(4, 930 + rank, T * H).reshape(T, H), BF16), BF16)
        # the sharded layer multiplies gate, up and down as three tensor-core products: bit identity is against that form
        want = ctx.to_host(MoeFfn(ctx, H, I, E, k, router, bias, *full, fused_swiglu=False).forward(x, T, out_dtype=F32), F32, T * H)
        ep = ExpertParallelMoe(ctx, comm, H, I, E, k, router, bias, *mine)
        got = ctx.to_host(ep.forward(x, T, out_dtype=F32), F32, T * H)
        got2 = ctx.to_host(ep.forward(x, T, out_dtype=F32), F32, T * H)
        ctx.check_device_error()
        comm.destroy()
        out_q.put((rank, bool(np.array_equal(got, want)), bool(np.array_equal(got2, want)), float(np.abs(want).max()), None))
    except Exception:   # report instead of hanging the parent
        import traceback
        out_q.put((rank, None, None, None, traceback.format_exc()))


@pytest.mark.skipif(_gpu_count() < 2, reason="needs 2 GPUs")
def test_expert_parallel_moe_equals_the_single_gpu_layer():
    """Experts sharded over 2 ranks, tokens owned by their rank, rows exchanged with the NCCL all-to-all: every token's
    output is bit-identical to the unsharded layer run on the same GPU (each row's product does not depend on its neighbours)."""
    results = _run_ranks(_ep_rank_main, 2)
    for rank, same, same2, peak, err in results:
        assert err is None, "rank %d failed:\n%s" % (rank, err)
        assert same and same2 and peak > 0, (rank, same, same2, peak)


def _peer_rank_main(rank, size, id_path, out_q):
    try:
        import ctypes as C
        here = os.path.dirname(os.path.abspath(__file__))
        for p in (os.path.dirname(here), here):
            if p not in sys.path:
                sys.path.insert(0, p)
        os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
        from helpers import TINY_CFG, make_weights
        from luminal_b200 import BF16, F32, Context
        from luminal_b200.dist import Comm
        from luminal_b200.llama import Llama
        from luminal_b200.runtime import gen_normal, round_to_dtype
        from oracle import oracle as orc
        ctx = Context(rank)
        lib = ctx.lib
        comm = Comm(ctx, size, rank, Comm.exchange_id_via_file(id_path, rank))
        # --- the exchange kernel against numpy: every rank's partial product is regenerated from its seed on every rank
        worst = 0.0
        for dtype, dim, rows in ((F32, 512, 5), (BF16, 1024, 16), (BF16, 8192, 3)):
            es = 4 if dtype == F32 else 2
            peer = C.c_void_p()
            ctx._check(lib.blum_peer_create(ctx.h, comm.h, dim * es, 16, 30000, C.byref(peer)))
            nw = (1 + 0.1 * gen_normal(9, 5, dim)).astype(np.float32)
            nwd = ctx.to_device(nw)
            xn, xo = ctx.alloc(rows * dim * es), ctx.alloc(rows * dim * es)
            for call in range(12):                       # slots alternate; the same area is reused many times
                slot = call % 2
                parts = [round_to_dtype(gen_normal(9, 100 * call + r, rows * dim).reshape(rows, dim), dtype) for r in range(size)]
                x = round_to_dtype(gen_normal(9, 100 * call + 50, rows * dim).reshape(rows, dim), dtype)
                mine = ctx.to_device(parts[rank], dtype)
                ctx._check(lib.blum_memcpy_d2d(ctx.h, lib.blum_peer_slot(peer, slot), mine.ptr, rows * dim * es))
                xd = ctx.to_device(x, dtype)
                with_norm = call % 3 != 2
                ctx._check(lib.blum_allreduce_fused(ctx.h, peer, slot, xd.ptr, nwd.ptr if with_norm else None, 1e-5,
                                                    xn.ptr if with_norm else None, xo.ptr, dtype, rows, dim))
                got = ctx.to_host(xo, dtype, rows * dim).reshape(rows, dim)
                acc = np.zeros((rows, dim), np.float32)
                for r in range(size):
                    acc = acc + parts[r].astype(np.float32)
                want = round_to_dtype(x.astype(np.float32) + round_to_dtype(acc, dtype).astype(np.float32), dtype)
                assert np.array_equal(got, want), ("sum", dtype, call)
                if with_norm:
                    gn = ctx.to_host(xn, dtype, rows * dim).reshape(rows, dim).astype(np.float64)
                    w64 = want.astype(np.float64)
                    wn = w64 / np.sqrt((w64 * w64).mean(axis=1, keepdims=True) + 1e-5) * nw
                    worst = max(worst, float(np.abs(gn - wn).max() / (np.abs(wn).max())))
            # the same slot twice in a row is refused on the host, nothing is launched
            rc = lib.blum_allreduce_fused(ctx.h, peer, 1, xd.ptr, None, 1e-5, None, xo.ptr, dtype, rows, dim)
            assert rc == -4, rc
            ctx.check_device_error()
            ctx._check(lib.blum_peer_destroy(ctx.h, peer))
        # --- the decoder with the exchange kernel gives the ids of the NCCL path (eager prefill + captured decode steps)
        model = Llama(ctx, TINY_CFG, act_dtype=F32, page_size=4, max_seqs=2, max_ctx=64, tp_rank=rank, tp_size=size)
        model.set_comm(comm)
        model.load_weights(make_weights(orc, TINY_CFG, seed=0))
        prompt = orc.gen_token_ids(0, 1, 6, TINY_CFG["vocab"])
        ids_nccl = model.greedy(prompt, 8)
        model.set_peer_allreduce(True)
        assert model.peer_allreduce
        ids_peer = model.greedy(prompt, 8)
        ids_peer2 = model.greedy(prompt, 8)
        model.set_peer_allreduce(False)
        ids_back = model.greedy(prompt, 8)
        ctx.check_device_error()
        model.destroy()
        comm.destroy()
        out_q.put((rank, ids_nccl, ids_peer, ids_peer2, ids_back, worst, None))
    except Exception:   # report instead of hanging the parent
        import traceback
        out_q.put((rank, None, None, None, None, None, traceback.format_exc()))


@pytest.mark.skipif(_gpu_count() < 2, reason="needs 2 GPUs")
def test_peer_memory_exchange_kernel_and_decoder():
    """Sum over ranks + residual + RMSNorm as one kernel over peer-mapped memory: bit-exact sums against numpy, the
    decoder's greedy ids equal to the NCCL path and to the golden ids."""
    g = np.load(os.path.join(GOLD, "oracle_vectors.npz"))
    results = _run_ranks(_peer_rank_main, 2)
    for rank, ids_nccl, ids_peer, ids_peer2, ids_back, worst, err in results:
        assert err is None, "rank %d failed:\n%s" % (rank, err)
        assert ids_peer == ids_nccl == ids_peer2 == ids_back == g["llama_greedy_ids"].tolist(), (rank, ids_nccl, ids_peer)
        assert worst < 1e-2, worst          # bf16 rows: half an ulp of the normalised value
