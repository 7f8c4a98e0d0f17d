// Temperature / top-p sampling on the device, one CTA per row of logits.
//
// luminal's llama example samples greedily on the host (examples/llama/src/main.rs:194-198: a 513 KB copy and a scan per
// token); blum_argmax replaces that.  This sampler is an addition with no counterpart there.  It is specified in integers
// wherever a result could depend on the order of operations, so that 1024 threads reproduce a sequential scan bit for bit:
//   m    = the largest logit that is not a NaN (a row without one is sampled greedily)
//   z_i  = (l_i - m) * (1 / temperature), each operation rounded to f32
//   w_i  = trunc(2^30 * e^z_i) by sample_weight below (a fixed sequence of f32 operations); NaN and -inf give 0
//   W    = sum of w_i;  P = max(1, (uint64)((double)top_p * (double)W)), P = W for top_p >= 1
//   tau  = the largest integer with S(tau) = sum of the w_i >= tau  >=  P;  the nucleus is {i : w_i >= tau}
//   r    = floor(u * S(tau) / 2^64), u = mix64(mix64(seed + GOLDEN * (seq + 1)) + pos)
//   the sampled token is the first index i of the nucleus, in index order, whose running sum of w exceeds r.
// (seq, pos) are the row's sequence slot and position, read from device memory, so a captured step draws a new number every
// replay.  tau is found by a radix selection over the 31 weight bits (11 + 10 + 10) with 64-bit sums per bucket in shared
// memory; the pick is a block-wide exclusive scan over contiguous chunks.  Five passes over the row's weights (513 KB for
// the Llama-3 vocabulary, L2-resident): HBM-irrelevant, a few tens of microseconds.
#include "common.cuh"
#include <math.h>

#define SP_THREADS 1024

__device__ __forceinline__ uint32_t sample_weight(float z) {
    if (!(z > -21.5f)) return 0u;                      // also NaN; 2^30 e^-21.5 < 1
    if (z > 0.f) z = 0.f;
    const float t = __fmul_rn(z, 1.44269504f);
    const float n = rintf(t);                          // round to nearest even
    const float f = __fsub_rn(t, n);                   // exact, |f| <= 0.5 (never fused with the multiply above)
    float p = 1.5403530e-4f;                           // 2^f = e^(f ln 2), Taylor coefficients, Horner with fused multiply-adds
    p = __fmaf_rn(p, f, 1.3333558e-3f);
    p = __fmaf_rn(p, f, 9.6181291e-3f);
    p = __fmaf_rn(p, f, 5.5504109e-2f);
    p = __fmaf_rn(p, f, 2.4022651e-1f);
    p = __fmaf_rn(p, f, 6.9314718e-1f);
    p = __fmaf_rn(p, f, 1.0f);
    const float sc = __uint_as_float((uint32_t)(127 + 30 + (int)n) << 23);      // 2^(n + 30), n in [-32, 0]
    return (uint32_t)__float2uint_rz(__fmul_rn(p, sc));
}

__device__ __forceinline__ unsigned long long sp_block_sum(unsigned long long v, unsigned long long* red) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    __syncthreads();                                   // red may still be read from an earlier call
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = v;
    __syncthreads();
    unsigned long long s = 0;
    for (int w = 0; w < SP_THREADS / 32; w++) s += red[w];
    return s;
}

// rows [rows][3*max_rows...] layout of the decoder: seq ids at rows_seq, positions at rows_pos (either may be null: 0)
__global__ void __launch_bounds__(SP_THREADS) sample_top_p_kernel(const float* __restrict__ logits, int64_t cols, float inv_t, float top_p,
                                                                  unsigned long long seed, const int32_t* __restrict__ rows_seq,
                                                                  const int32_t* __restrict__ rows_pos, uint32_t* __restrict__ wbuf,
                                                                  int32_t* __restrict__ out) {
    __shared__ unsigned long long hist[2048];
    __shared__ unsigned long long red[SP_THREADS / 32];
    __shared__ float fred[SP_THREADS / 32];
    __shared__ uint32_t s_prefix;
    __shared__ unsigned long long s_above;
    __shared__ int s_pick;
    const int tid = threadIdx.x;
    const float* l = logits + (size_t)blockIdx.x * cols;
    uint32_t* w = wbuf + (size_t)blockIdx.x * cols;

    // ---- m
    float m = -INFINITY;
    for (int64_t i = tid; i < cols; i += SP_THREADS) { const float v = l[i]; if (v == v) m = fmaxf(m, v); }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
    if ((tid & 31) == 0) fred[tid >> 5] = m;
    __syncthreads();
    for (int k = 0; k < SP_THREADS / 32; k++) m = fmaxf(m, fred[k]);
    if (!(m > -INFINITY)) {
        // no finite logit: the greedy rule of the reference, sequentially (a degenerate row; not worth a parallel path)
        if (tid == 0) {
            float cur = l[0]; int ci = 0;
            for (int64_t j = 1; j < cols; j++) { const float v = l[j]; if (!(cur > v)) { cur = v; ci = (int)j; } }
            out[blockIdx.x] = ci;
        }
        return;
    }
    // ---- w, W
    unsigned long long part = 0;
    for (int64_t i = tid; i < cols; i += SP_THREADS) {
        const uint32_t wi = sample_weight(__fmul_rn(__fsub_rn(l[i], m), inv_t));
        w[i] = wi;
        part += wi;
    }
    const unsigned long long W = sp_block_sum(part, red);
    unsigned long long P = top_p >= 1.f ? W : (unsigned long long)((double)top_p * (double)W);
    if (P < 1) P = 1;

    // ---- tau by radix selection: digits of 11, 10 and 10 bits from the top of the 31-bit weights
    if (tid == 0) { s_prefix = 0u; s_above = 0ull; }
    const int shifts[3] = {20, 10, 0}, bits[3] = {11, 10, 10};
    for (int level = 0; level < 3; level++) {
        const int sh = shifts[level], nb = 1 << bits[level];
        for (int b = tid; b < nb; b += SP_THREADS) hist[b] = 0ull;
        __syncthreads();
        const uint32_t prefix = s_prefix;
        const int hs = sh + bits[level];                       // bits above this digit must equal the prefix
        for (int64_t i = tid; i < cols; i += SP_THREADS) {
            const uint32_t wi = w[i];                          // this thread's own stores
            if (wi != 0u && (hs >= 31 || (wi >> hs) == (prefix >> hs))) atomicAdd(&hist[(wi >> sh) & (uint32_t)(nb - 1)], (unsigned long long)wi);
        }
        __syncthreads();
        if (tid == 0) {
            // the highest digit d whose S(low edge of d) = above + sum of buckets >= d reaches P
            unsigned long long cum = s_above;
            int d = nb - 1;
            for (; d > 0; d--) {
                if (cum + hist[d] >= P) break;
                cum += hist[d];
            }
            s_above = cum;
            s_prefix = prefix | ((uint32_t)d << sh);
        }
        __syncthreads();
    }
    const uint32_t tau = s_prefix > 0u ? s_prefix : 1u;

    // ---- S(tau) and the pick: contiguous chunks, block-wide exclusive scan of the chunk sums
    const int64_t chunk = (cols + SP_THREADS - 1) / SP_THREADS;
    const int64_t i0 = (int64_t)tid * chunk, i1 = i0 + chunk < cols ? i0 + chunk : cols;
    unsigned long long mine = 0;
    __syncthreads();                                           // other threads' weights are read now
    for (int64_t i = i0; i < i1; i++) { const uint32_t wi = w[i]; if (wi >= tau) mine += wi; }
    // inclusive scan within the warp, then over the warp totals
    unsigned long long inc = mine;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        const unsigned long long v = __shfl_up_sync(0xffffffffu, inc, o);
        if ((tid & 31) >= o) inc += v;
    }
    if ((tid & 31) == 31) red[tid >> 5] = inc;
    if (tid == 0) s_pick = -1;
    __syncthreads();
    unsigned long long before = 0, S = 0;
    for (int k = 0; k < SP_THREADS / 32; k++) { if (k < (tid >> 5)) before += red[k]; S += red[k]; }
    const unsigned long long excl = before + inc - mine;
    const unsigned long long sq = (unsigned long long)(rows_seq ? rows_seq[blockIdx.x] : 0), ps = (unsigned long long)(rows_pos ? rows_pos[blockIdx.x] : 0);
    const unsigned long long u = blum_mix64(blum_mix64(seed + BLUM_GOLDEN * (sq + 1ull)) + ps);
    const unsigned long long r = __umul64hi(u, S);
    if (mine > 0 && r >= excl && r < excl + mine) {
        unsigned long long run = excl;
        for (int64_t i = i0; i < i1; i++) {
            const uint32_t wi = w[i];
            if (wi >= tau) { run += wi; if (run > r) { s_pick = (int)i; break; } }
        }
    }
    __syncthreads();
    if (tid == 0) {
        int pick = s_pick;
        if (pick < 0) {                                        // no weight at all (a +inf logit): the greedy rule
            float cur = l[0]; pick = 0;
            for (int64_t j = 1; j < cols; j++) { const float v = l[j]; if (!(cur > v)) { cur = v; pick = (int)j; } }
        }
        out[blockIdx.x] = pick;
    }
}

extern "C" int blum_sample_top_p(blum_ctx* ctx, const float* logits, int64_t rows, int64_t cols, float temperature, float top_p,
                                 uint64_t seed, const int32_t* row_seq, const int32_t* row_pos, void* scratch, int32_t* out_idx) {
    if (!ctx) return BLUM_ERR_INVALID;
    BLUM_REQUIRE(ctx, logits && out_idx && scratch && rows >= 0 && cols > 0 && cols < (1ll << 31), "sample_top_p: bad argument");
    BLUM_REQUIRE(ctx, temperature > 0.f && top_p > 0.f, "sample_top_p: temperature and top_p must be positive (temperature 0 is blum_argmax)");
    if (rows == 0) return BLUM_OK;
    sample_top_p_kernel<<<(unsigned)rows, SP_THREADS, 0, ctx->stream>>>(logits, cols, 1.0f / temperature, top_p, (unsigned long long)seed, row_seq,
                                                                      row_pos, (uint32_t*)scratch, out_idx);
    BLUM_LAUNCH_CHECK(ctx);
    return BLUM_OK;
}
