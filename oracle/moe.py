"""CPU oracle of the MXFP4 mixture-of-experts feed-forward (numpy).  TEST INFRASTRUCTURE: only tests/ and the
CPU-baseline legs of bench.py may import it.

luminal has no MoE, top-k or MXFP4 code, so nothing in the reference pins these semantics: PARITY UNPINNED, this file
is the arbiter.  Definitions (shared with luminal_b200/csrc/moe.cu):
  * MXFP4: e2m1 codes (sign, 2-bit exponent, 1-bit mantissa; magnitudes 0, .5, 1, 1.5, 2, 3, 4, 6), element 2i in the low
    nibble of byte i, one e8m0 scale 2^(e-127) per 32 elements along K;
  * router logits in f32, top-k with ties to the LOWER expert index, gates = softmax over the selected logits;
  * (token, choice) pairs sorted by expert, stable; expert = Wdown((Wup x) * swish(Wgate x));
  * activations are bf16: every op output is rounded to bf16 (round to nearest even), the combine accumulates in f32.
"""
import numpy as np

E2M1 = np.array([0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0], np.float32)
M64 = (1 << 64) - 1
GOLDEN = 0x9E3779B97F4A7C15


def _mix64_int(z):
    z = ((z ^ (z >> 30)) * 0xBF58476D1CE4E5B9) & M64
    z = ((z ^ (z >> 27)) * 0x94D049BB133111EB) & M64
    return z ^ (z >> 31)


def gen_key(seed, tensor):
    return _mix64_int(_mix64_int((seed + GOLDEN) & M64) ^ ((tensor * 0xD1B54A32D192ED03 + 0x8CB92BA72F3D8DD7) & M64))


def gen_hash(key, idx):
    """splitmix64 finaliser of key + idx*golden, vectorised over a uint64 index array."""
    with np.errstate(over="ignore"):
        z = np.uint64(key) + idx.astype(np.uint64) * np.uint64(GOLDEN)
        z = (z ^ (z >> np.uint64(30))) * np.uint64(0xBF58476D1CE4E5B9)
        z = (z ^ (z >> np.uint64(27))) * np.uint64(0x94D049BB133111EB)
        return z ^ (z >> np.uint64(31))


def gen_mxfp4(seed, tensor, E, N, K):
    """Same stream as blum_mxfp4_weight_generate: codes uniform over 16 values, block exponents uniform in [-8, 0]."""
    n = E * N * K
    codes = (gen_hash(gen_key(seed, tensor), np.arange(n, dtype=np.uint64)) >> np.uint64(60)).astype(np.uint8)
    nibbles = (codes[0::2] | (codes[1::2] << 4)).astype(np.uint8).reshape(E, N, K // 2)
    h = gen_hash(gen_key(seed, tensor ^ (0x5CA1E5 << 40)), np.arange(n // 32, dtype=np.uint64))
    scales = (119 + (((h >> np.uint64(32)) * np.uint64(9)) >> np.uint64(32))).astype(np.uint8).reshape(E, N, K // 32)
    return nibbles, scales


def dequant_mxfp4(nibbles, scales):
    """[..., K/2] bytes + [..., K/32] e8m0 -> f32 [..., K]."""
    lo, hi = nibbles & 15, nibbles >> 4
    codes = np.stack([lo, hi], axis=-1).reshape(nibbles.shape[:-1] + (nibbles.shape[-1] * 2,))
    vals = np.where(codes & 8, -E2M1[codes & 7], E2M1[codes & 7]).astype(np.float32)
    sc = np.where(scales == 0, 0.0, np.exp2(scales.astype(np.float32) - 127.0)).astype(np.float32)
    return vals * np.repeat(sc, 32, axis=-1)


def round_bf16(a):
    a = np.ascontiguousarray(a, dtype=np.float32)
    u = a.view(np.uint32).astype(np.uint64)
    r = ((u + 0x7FFF + ((u >> 16) & 1)) >> 16).astype(np.uint32) << 16
    return r.view(np.float32)


def route(x, router_w, router_bias, k):
    logits = x.astype(np.float32) @ router_w.astype(np.float32).T
    if router_bias is not None:
        logits = logits + router_bias.astype(np.float32)
    order = np.argsort(-logits, axis=1, kind="stable")[:, :k]            # ties -> lower expert index
    sel = np.take_along_axis(logits, order, axis=1)
    e = np.exp2((sel - sel[:, :1]) * np.float32(1.4426950408889634))
    return order.astype(np.int32), (e / e.sum(1, keepdims=True)).astype(np.float32), logits


def permute(ids, E):
    flat = ids.reshape(-1)
    sorted_src = np.argsort(flat, kind="stable").astype(np.int32)
    slot_of = np.empty_like(sorted_src)
    slot_of[sorted_src] = np.arange(flat.size, dtype=np.int32)
    offsets = np.concatenate([[0], np.cumsum(np.bincount(flat, minlength=E))]).astype(np.int32)
    return sorted_src, slot_of, offsets


def swish(g):
    # g / (1 + exp(-g)); the exponent is capped so that very negative g gives g * tiny instead of an overflow warning
    g = np.asarray(g, np.float32)
    return g * (np.float32(1.0) / (np.float32(1.0) + np.exp(np.minimum(-g, np.float32(88.0)))))


def moe_ffn_lazy(x, router_w, router_bias, expert, k, round_gate_up=True):
    """x [T,H] (bf16 values); expert(e) -> (wg [I,H], wu [I,H], wd [H,I]) as f32, called once per expert that is hit
    (full-size layers hold gigabytes of dequantised weights otherwise).  Returns (out f32 [T,H], ids, gates).
    round_gate_up: the gate and up products are stored as bf16 before the SwiGLU (the three-product form); False is the
    one-product form, whose epilogue applies the SwiGLU to the f32 sums."""
    T = x.shape[0]
    ids, gates, _ = route(x, router_w, router_bias, k)
    out = np.zeros((T, x.shape[1]), np.float32)
    contrib = np.zeros((T, k, x.shape[1]), np.float32)
    for e in np.unique(ids):
        wg, wu, wd = expert(int(e))
        for t, j in zip(*np.nonzero(ids == e)):
            g, u = wg @ x[t], wu @ x[t]
            if round_gate_up:
                g, u = round_bf16(g), round_bf16(u)
            mid = round_bf16(u * swish(g))
            contrib[t, j] = round_bf16(wd @ mid)
    for t in range(T):                       # the combine adds the k choices in choice order, in f32
        for j in range(k):
            out[t] += gates[t, j] * contrib[t, j]
    return out, ids, gates


def moe_ffn(x, router_w, router_bias, wg, wu, wd, k, round_gate_up=True):
    """x [T,H] (bf16 values); wg/wu f32 [E,I,H]; wd f32 [E,H,I] (already dequantised).  Returns (out f32 [T,H], ids, gates)."""
    return moe_ffn_lazy(x, router_w, router_bias, lambda e: (wg[e], wu[e], wd[e]), k, round_gate_up)
