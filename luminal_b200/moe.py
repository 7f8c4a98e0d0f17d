"""Host-side driver of the MXFP4 mixture-of-experts feed-forward (csrc/moe.cu): route -> permute -> grouped GEMMs ->
SwiGLU -> grouped GEMM -> un-permute.  luminal has no MoE; this mirrors the op-by-op style of its operators (each step
allocates its output and returns a device buffer)."""
import ctypes as C

import numpy as np

from ._lib import BF16, F32
from .runtime import Context, DeviceBuffer


class Mxfp4Weight:
    """E stacked expert matrices [N, K] in MXFP4 on the device."""

    def __init__(self, ctx, handle, E, N, K):
        self.ctx, self.h, self.E, self.N, self.K = ctx, handle, E, N, K

    @classmethod
    def from_host(cls, ctx, nibbles, scales, E, N, K):
        nibbles = np.ascontiguousarray(nibbles, dtype=np.uint8)
        scales = np.ascontiguousarray(scales, dtype=np.uint8)
        assert nibbles.size == E * N * K // 2 and scales.size == E * N * K // 32
        h = C.c_void_p()
        ctx._check(ctx.lib.blum_mxfp4_weight_from_host(ctx.h, nibbles.ctypes.data, scales.ctypes.data, E, N, K, C.byref(h)))
        return cls(ctx, h.value, E, N, K)

    @classmethod
    def generate(cls, ctx, seed, tensor_id, E, N, K):
        h = C.c_void_p()
        ctx._check(ctx.lib.blum_mxfp4_weight_generate(ctx.h, seed, tensor_id, E, N, K, C.byref(h)))
        return cls(ctx, h.value, E, N, K)

    @classmethod
    def stack_gate_up(cls, gate, up):
        """[E, 2N, K]: 16 gate rows, then the 16 up rows of the same features, and so on (the fused SwiGLU product's layout)."""
        h = C.c_void_p()
        gate.ctx._check(gate.ctx.lib.blum_mxfp4_weight_stack_gate_up(gate.ctx.h, gate.h, up.h, C.byref(h)))
        return cls(gate.ctx, h.value, gate.E, 2 * gate.N, gate.K)

    def download(self):
        q = np.empty(self.E * self.N * self.K // 2, np.uint8)
        s = np.empty(self.E * self.N * self.K // 32, np.uint8)
        self.ctx._check(self.ctx.lib.blum_mxfp4_weight_download(self.ctx.h, self.h, q.ctypes.data, s.ctypes.data))
        return q.reshape(self.E, self.N, self.K // 2), s.reshape(self.E, self.N, self.K // 32)

    @property
    def nbytes(self):
        return self.E * self.N * self.K * 17 // 32

    def free(self):
        if self.h:
            self.ctx.lib.blum_mxfp4_weight_free(self.ctx.h, self.h)
            self.h = None


class MoeFfn:
    """One MoE feed-forward layer: bf16 router [E, H] (+ f32 bias), MXFP4 gate/up [E, I, H] and down [E, H, I]."""

    def __init__(self, ctx: Context, hidden, inter, experts, top_k, router_w: DeviceBuffer, router_bias, w_gate, w_up, w_down,
                 fused_swiglu=True, keep_separate=True):
        """fused_swiglu: gate and up are multiplied as ONE grouped product over a stacked copy of the two weights, with the
        SwiGLU in its epilogue (gate and up sums are then not rounded to bf16 before it).  keep_separate=False frees the two
        separate weights once the stacked copy exists."""
        self.ctx, self.H, self.I, self.E, self.k = ctx, hidden, inter, experts, top_k
        self.router_w, self.router_bias = router_w, router_bias
        self.w_gate, self.w_up, self.w_down = w_gate, w_up, w_down
        self.w_gate_up = None
        if fused_swiglu and w_gate is not None and inter % 16 == 0:
            self.w_gate_up = Mxfp4Weight.stack_gate_up(w_gate, w_up)
            if not keep_separate:
                w_gate.free()
                w_up.free()
                self.w_gate = self.w_up = None

    # rows (token, choice pairs) up to which the streaming kernel (csrc/moe_small.cu) runs both expert products; above it the
    # tcgen05 grouped GEMMs do
    SMALL_ROWS = 1024

    def _small(self, n):
        return self.w_gate_up is not None and n <= self.SMALL_ROWS and self.H % 32 == 0 and self.I % 32 == 0

    def _experts(self, xp, offsets, n, hint, g, u, mid, yp, slot_of, gates, T, out, out_dtype):
        """From the rows sorted by expert to the layer output: SwiGLU of the gate / up products, down product, combine."""
        ctx, lib = self.ctx, self.ctx.lib
        if self._small(n):
            ctx._check(lib.blum_moe_experts_small(ctx.h, self.w_gate_up.h, self.w_down.h, xp.ptr, offsets.ptr, n, slot_of.ptr, gates.ptr,
                                                  T, self.k, out.ptr, out_dtype))
            return
        self._gate_up_swiglu(xp, offsets, n, hint, g, u, mid)
        ctx._check(lib.blum_moe_grouped_gemm(ctx.h, self.w_down.h, mid.ptr, offsets.ptr, n, yp.ptr, BF16, hint))
        ctx._check(lib.blum_moe_unpermute(ctx.h, yp.ptr, slot_of.ptr, gates.ptr, T, self.k, self.H, out.ptr, out_dtype))

    def _gate_up_swiglu(self, xp, offsets, n, hint, g, u, mid):
        ctx, lib = self.ctx, self.ctx.lib
        if self.w_gate_up is not None:
            ctx._check(lib.blum_moe_grouped_gemm_swiglu(ctx.h, self.w_gate_up.h, xp.ptr, offsets.ptr, n, mid.ptr, hint))
            return
        ctx._check(lib.blum_moe_grouped_gemm(ctx.h, self.w_gate.h, xp.ptr, offsets.ptr, n, g.ptr, BF16, hint))
        ctx._check(lib.blum_moe_grouped_gemm(ctx.h, self.w_up.h, xp.ptr, offsets.ptr, n, u.ptr, BF16, hint))
        ctx._check(lib.blum_swiglu(ctx.h, g.ptr, u.ptr, mid.ptr, BF16, n * self.I))

    def route(self, x: DeviceBuffer, T):
        ids, gates = self.ctx.alloc(max(T * self.k * 4, 16)), self.ctx.alloc(max(T * self.k * 4, 16))
        self.ctx._check(self.ctx.lib.blum_moe_route_topk(self.ctx.h, x.ptr, self.router_w.ptr,
                                                        self.router_bias.ptr if self.router_bias else None, T, self.H, self.E,
                                                        self.k, ids.ptr, gates.ptr))
        return ids, gates

    def permute(self, ids: DeviceBuffer, T):
        n = T * self.k
        sorted_src, slot_of, offsets = self.ctx.alloc(max(n * 4, 16)), self.ctx.alloc(max(n * 4, 16)), self.ctx.alloc((self.E + 1) * 4)
        self.ctx._check(self.ctx.lib.blum_moe_permute(self.ctx.h, ids.ptr, n, self.E, sorted_src.ptr, slot_of.ptr, offsets.ptr))
        return sorted_src, slot_of, offsets

    def plan(self, T, out_dtype=BF16):
        """Pre-allocates every intermediate of a T-token step (so that `enqueue` allocates nothing and can be captured).
        Plans are kept per (T, out_dtype): planning the same shape again only makes it the current one."""
        ctx, n = self.ctx, T * self.k
        if not hasattr(self, "_plans"):
            self._plans = {}
        if (T, out_dtype) in self._plans:
            self._plan = self._plans[(T, out_dtype)]
            return self._plan
        a = lambda nbytes: ctx.alloc(max(nbytes, 16))
        self._plan = self._plans[(T, out_dtype)] = dict(T=T, out_dtype=out_dtype, ids=a(n * 4), gates=a(n * 4), sorted_src=a(n * 4), slot_of=a(n * 4),
                          offsets=a((self.E + 1) * 4), xp=a(n * self.H * 2),
                          g=a(n * self.I * 2) if self.w_gate_up is None else None, u=a(n * self.I * 2) if self.w_gate_up is None else None,
                          mid=a(n * self.I * 2), yp=a(n * self.H * 2), out=a(T * self.H * (4 if out_dtype == F32 else 2)))
        return self._plan

    def enqueue(self, x: DeviceBuffer):
        """Issues the whole layer on the context's stream using the planned buffers; returns the output buffer."""
        p, ctx, lib = self._plan, self.ctx, self.ctx.lib
        T, n, hint = p["T"], p["T"] * self.k, max(1, p["T"] * self.k // self.E)
        ctx._check(lib.blum_moe_route_topk(ctx.h, x.ptr, self.router_w.ptr, self.router_bias.ptr if self.router_bias else None,
                                           T, self.H, self.E, self.k, p["ids"].ptr, p["gates"].ptr))
        ctx._check(lib.blum_moe_permute(ctx.h, p["ids"].ptr, n, self.E, p["sorted_src"].ptr, p["slot_of"].ptr, p["offsets"].ptr))
        ctx._check(lib.blum_moe_gather_rows(ctx.h, x.ptr, p["sorted_src"].ptr, n, self.k, self.H, p["xp"].ptr))
        self._experts(p["xp"], p["offsets"], n, hint, p["g"], p["u"], p["mid"], p["yp"], p["slot_of"], p["gates"], T, p["out"], p["out_dtype"])
        return p["out"]

    def forward(self, x: DeviceBuffer, T, out_dtype=BF16, keep=None):
        """x bf16 [T, H] -> out [T, H].  `keep`, if a dict, receives the intermediate device buffers."""
        ctx, lib, n = self.ctx, self.ctx.lib, T * self.k
        ids, gates = self.route(x, T)
        sorted_src, slot_of, offsets = self.permute(ids, T)
        xp = ctx.alloc(max(n * self.H * 2, 16))
        ctx._check(lib.blum_moe_gather_rows(ctx.h, x.ptr, sorted_src.ptr, n, self.k, self.H, xp.ptr))
        hint = max(1, n // self.E)
        sep = self.w_gate_up is None
        g, u = (ctx.alloc(max(n * self.I * 2, 16)), ctx.alloc(max(n * self.I * 2, 16))) if sep else (None, None)
        mid = ctx.alloc(max(n * self.I * 2, 16))
        yp = ctx.alloc(max(n * self.H * 2, 16))
        out = ctx.alloc(max(T * self.H * (4 if out_dtype == F32 else 2), 16))
        self._experts(xp, offsets, n, hint, g, u, mid, yp, slot_of, gates, T, out, out_dtype)
        ctx.sync()
        if keep is not None:
            keep.update(ids=ids, gates=gates, sorted_src=sorted_src, slot_of=slot_of, offsets=offsets, xp=xp, yp=yp)
        return out


class ExpertParallelMoe:
    """The same layer with the experts sharded over the ranks of a communicator (rank r holds experts
    [r*E/W, (r+1)*E/W)); router and tokens stay with the rank that owns the tokens.

    dispatch: route -> sort pairs by global expert -> all-gather of the per-expert counts -> all-to-all of the rows;
    experts: rows re-sorted by local expert -> grouped GEMMs -> back to arrival order;
    combine: all-to-all back -> gate-weighted un-permute at the owner.
    The exchange is NCCL send/recv (blum_alltoallv); the counts cross the host once per layer call."""

    def __init__(self, ctx: Context, comm, hidden, inter, experts, top_k, router_w, router_bias, w_gate, w_up, w_down):
        assert experts % comm.nranks == 0
        self.ctx, self.comm = ctx, comm
        self.H, self.I, self.E, self.k = hidden, inter, experts, top_k
        self.EL = experts // comm.nranks
        assert w_gate.E == self.EL and w_up.E == self.EL and w_down.E == self.EL, "pass this rank's expert slice"
        self.router_w, self.router_bias = router_w, router_bias
        self.w_gate, self.w_up, self.w_down = w_gate, w_up, w_down
        self._local = MoeFfn(ctx, hidden, inter, experts, top_k, router_w, router_bias, None, None, None)   # route / permute only

    def plan(self, T, out_dtype=BF16):
        """Allocates every buffer of a T-token call once, sized for the worst case on the receiving side (all pairs of
        all ranks routed to this rank's experts), so that `forward` itself allocates nothing."""
        ctx, W, H, I, n = self.ctx, self.comm.nranks, self.H, self.I, T * self.k
        a = lambda nbytes: ctx.alloc(max(int(nbytes), 16))
        nmax = W * n
        self._plan = dict(T=T, out_dtype=out_dtype, ids=a(n * 4), gates=a(n * 4), sorted_src=a(n * 4), slot_of=a(n * 4),
                          offsets=a((self.E + 1) * 4), xp=a(n * H * 2), all_off=a(W * (self.E + 1) * 4), recv=a(nmax * H * 2),
                          out_rows=a(nmax * H * 2), ids2=a(nmax * 4), s2=a(nmax * 4), slot2=a(nmax * 4), off2=a((self.EL + 1) * 4),
                          xq=a(nmax * H * 2), g=a(nmax * I * 2), u=a(nmax * I * 2), mid=a(nmax * I * 2), yq=a(nmax * H * 2),
                          yp=a(n * H * 2), out=a(T * H * (4 if out_dtype == F32 else 2)))
        return self._plan

    def forward(self, x: DeviceBuffer, T, out_dtype=BF16):
        from .dist import ep_exchange_plan
        ctx, lib, comm = self.ctx, self.ctx.lib, self.comm
        W, r, H, k, n = comm.nranks, comm.rank, self.H, self.k, T * self.k
        b = getattr(self, "_plan", None)
        if b is None or b["T"] != T or b["out_dtype"] != out_dtype:
            b = self.plan(T, out_dtype)
        bias = self.router_bias.ptr if self.router_bias else None
        ctx._check(lib.blum_moe_route_topk(ctx.h, x.ptr, self.router_w.ptr, bias, T, H, self.E, k, b["ids"].ptr, b["gates"].ptr))
        ctx._check(lib.blum_moe_permute(ctx.h, b["ids"].ptr, n, self.E, b["sorted_src"].ptr, b["slot_of"].ptr, b["offsets"].ptr))
        ctx._check(lib.blum_moe_gather_rows(ctx.h, x.ptr, b["sorted_src"].ptr, n, k, H, b["xp"].ptr))
        # per-expert counts of every rank (offsets are the exclusive prefix sums of this rank's counts)
        comm.allgather(b["offsets"], b["all_off"], (self.E + 1) * 4)
        off = b["all_off"].download(np.int32, W * (self.E + 1)).reshape(W, self.E + 1)
        plan = ep_exchange_plan(np.diff(off, axis=1), r, self.EL)
        nr = int(plan["recv_rows"].sum())
        rb = H * 2
        comm.alltoallv(b["xp"], plan["send_rows"] * rb, plan["send_off"] * rb, b["recv"], plan["recv_rows"] * rb, plan["recv_off"] * rb)
        if nr:
            b["ids2"].upload(plan["recv_expert"])
            ctx._check(lib.blum_moe_permute(ctx.h, b["ids2"].ptr, nr, self.EL, b["s2"].ptr, b["slot2"].ptr, b["off2"].ptr))
            ctx._check(lib.blum_moe_gather_rows(ctx.h, b["recv"].ptr, b["s2"].ptr, nr, 1, H, b["xq"].ptr))
            hint = max(1, nr // self.EL)
            ctx._check(lib.blum_moe_grouped_gemm(ctx.h, self.w_gate.h, b["xq"].ptr, b["off2"].ptr, nr, b["g"].ptr, BF16, hint))
            ctx._check(lib.blum_moe_grouped_gemm(ctx.h, self.w_up.h, b["xq"].ptr, b["off2"].ptr, nr, b["u"].ptr, BF16, hint))
            ctx._check(lib.blum_swiglu(ctx.h, b["g"].ptr, b["u"].ptr, b["mid"].ptr, BF16, nr * self.I))
            ctx._check(lib.blum_moe_grouped_gemm(ctx.h, self.w_down.h, b["mid"].ptr, b["off2"].ptr, nr, b["yq"].ptr, BF16, hint))
            ctx._check(lib.blum_moe_gather_rows(ctx.h, b["yq"].ptr, b["slot2"].ptr, nr, 1, H, b["out_rows"].ptr))   # back to arrival order
        comm.alltoallv(b["out_rows"], plan["recv_rows"] * rb, plan["recv_off"] * rb, b["yp"], plan["send_rows"] * rb, plan["send_off"] * rb)
        ctx._check(lib.blum_moe_unpermute(ctx.h, b["yp"].ptr, b["slot_of"].ptr, b["gates"].ptr, T, k, H, b["out"].ptr, out_dtype))
        ctx.sync()
        return b["out"]
