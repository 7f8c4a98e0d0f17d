"""Multi-GPU host logic: NCCL communicator handle and the tensor-parallel shard rule.

luminal itself has no distributed code (device 0 is hard-coded, crates/luminal_cuda/src/quantized.rs:247); this is the
host side of the additions in csrc/comm.cu.  One process per GPU.
"""
import ctypes as C
import os
import time

from . import _lib


def tp_window(name, cfg, rank, size):
    """Window (row0, rows, col0, cols) of the FULL tensor `name` that tensor-parallel rank `rank` of `size` holds.

    Column-parallel (rows cut): attn_q/k/v by heads, ffn_gate/up, output head by vocabulary.
    Row-parallel (columns cut, always on 32-element Q8_0 block boundaries): attn_output, ffn_down.
    Everything else (norms, embedding) is replicated: the whole tensor.
    """
    d, H = cfg["head_dim"], cfg["hidden"]
    nq, nkv, ffn, vocab = cfg["q_heads"], cfg["kv_heads"], cfg["ffn"], cfg["vocab"]
    assert nkv % size == 0 and ffn % (32 * size) == 0 and vocab % size == 0, "shapes do not divide by the TP degree"
    kind = name.split(".")[-2] if name.startswith("blk.") else name.rsplit(".", 1)[0]
    if kind == "attn_q":
        r = nq // size * d
        return (rank * r, r, 0, H)
    if kind in ("attn_k", "attn_v"):
        r = nkv // size * d
        return (rank * r, r, 0, H)
    if kind in ("ffn_gate", "ffn_up"):
        r = ffn // size
        return (rank * r, r, 0, H)
    if kind == "output":
        r = vocab // size
        return (rank * r, r, 0, H)
    if kind == "attn_output":
        c = nq // size * d
        assert c % 32 == 0
        return (0, H, rank * c, c)
    if kind == "ffn_down":
        c = ffn // size
        assert c % 32 == 0
        return (0, H, rank * c, c)
    return None   # replicated


class Comm:
    """NCCL communicator bound to one context (one GPU, one process)."""

    def __init__(self, ctx, nranks, rank, unique_id: bytes, init_timeout_ms=120000):
        """init_timeout_ms: give up (BlumError, ERR_COMM) if a rank has not joined in that time; 0 waits for ever."""
        assert len(unique_id) == 128
        self.ctx, self.nranks, self.rank = ctx, nranks, rank
        h = C.c_void_p()
        ctx._check(ctx.lib.blum_comm_init_rank(ctx.h, nranks, rank, unique_id, int(init_timeout_ms), C.byref(h)))
        self.h = h.value

    @staticmethod
    def unique_id() -> bytes:
        buf = C.create_string_buffer(128)
        rc = _lib.load().blum_comm_unique_id(buf)
        if rc != 0:
            raise RuntimeError("ncclGetUniqueId failed (%d)" % rc)
        return buf.raw

    @staticmethod
    def exchange_id_via_file(path, rank, timeout_s=120.0) -> bytes:
        """Rank 0 writes the id to `path` (atomically); the others wait for it.  Enough for one node."""
        if rank == 0:
            uid = Comm.unique_id()
            tmp = path + ".tmp"
            with open(tmp, "wb") as f:
                f.write(uid)
            os.replace(tmp, path)
            return uid
        t0 = time.time()
        while not os.path.exists(path):
            if time.time() - t0 > timeout_s:
                raise TimeoutError("rank %d: no NCCL id at %s after %.0f s" % (rank, path, timeout_s))
            time.sleep(0.01)
        return open(path, "rb").read()

    # timeout_ms = 0 only enqueues the collective; > 0 waits for it and aborts the communicator if a peer never arrives

    def allreduce_sum(self, buf, count, dtype, timeout_ms=0):
        self.ctx._check(self.ctx.lib.blum_allreduce_sum(self.ctx.h, self.h, buf.ptr, count, dtype, int(timeout_ms)))

    def allgather(self, send, recv, bytes_per_rank, timeout_ms=0):
        self.ctx._check(self.ctx.lib.blum_allgather(self.ctx.h, self.h, send.ptr, recv.ptr, bytes_per_rank, int(timeout_ms)))

    def alltoallv(self, send, send_bytes, send_offsets, recv, recv_bytes, recv_offsets, timeout_ms=0):
        """Variable all-to-all in bytes; the four lists are per-peer host values."""
        arr = lambda v: (C.c_int64 * self.nranks)(*[int(x) for x in v])
        self.ctx._check(self.ctx.lib.blum_alltoallv(self.ctx.h, self.h, send.ptr, arr(send_bytes), arr(send_offsets), recv.ptr,
                                                    arr(recv_bytes), arr(recv_offsets), int(timeout_ms)))

    def destroy(self):
        if self.h:
            self.ctx.lib.blum_comm_destroy(self.ctx.h, self.h)
            self.h = None


def ep_exchange_plan(counts, rank, experts_per_rank):
    """Host bookkeeping of one expert-parallel dispatch.

    `counts[s][e]` = (token, choice) pairs that source rank s routed to GLOBAL expert e (every rank holds the whole matrix
    after an all-gather of its own row).  Rank d owns experts [d*EL, (d+1)*EL).  A rank's rows are sorted by global
    expert, so the rows for destination d are one contiguous run.  Returns, in rows:
      send_rows[d], send_off[d]   what this rank sends to d and where it starts in its sorted row buffer
      recv_rows[s], recv_off[s]   what arrives from s and where it lands (source-major)
      recv_expert[j]              LOCAL expert of received row j (each source's run is sorted by expert)
    """
    import numpy as np
    counts = np.asarray(counts, dtype=np.int64)
    W, E = counts.shape
    EL = experts_per_rank
    assert W * EL == E, "experts do not divide over the ranks"
    per_dest = counts.reshape(W, W, EL).sum(axis=2)              # [source][dest]
    send_rows = per_dest[rank]
    recv_rows = per_dest[:, rank]
    send_off = np.concatenate([[0], np.cumsum(send_rows)[:-1]])
    recv_off = np.concatenate([[0], np.cumsum(recv_rows)[:-1]])
    mine = counts[:, rank * EL:(rank + 1) * EL]                  # [source][local expert]
    recv_expert = np.concatenate([np.repeat(np.arange(EL, dtype=np.int32), mine[s]) for s in range(W)]) if recv_rows.sum() else np.zeros(0, np.int32)
    return dict(send_rows=send_rows, send_off=send_off, recv_rows=recv_rows, recv_off=recv_off, recv_expert=recv_expert.astype(np.int32))
