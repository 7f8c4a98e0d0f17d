/*
 * oracle.c - CPU restatement of luminal's arithmetic for the Q8_0 transformer-decoding path.
 *
 * THIS IS TEST INFRASTRUCTURE.  It is the checker that the CUDA library is compared against and
 * the CPU baseline that bench.py times; nothing in the product path may call it.
 *
 * Every function restates the semantics of the cited luminal source (paths relative to the luminal
 * tree); no code is copied.  The reference cannot be built in this environment (it is Rust), so the
 * restatement is pinned against the fixed-value tests the reference carries (embedding known-answer,
 * gather, triu, Q8_0 matvec with unit scales; see tests/golden/).  End-to-end greedy token ids,
 * paged-KV indexing and bf16 results have no golden values in the reference: for those rows parity
 * is "unpinned" and this file is the only arbiter.
 *
 * Conventions: all arithmetic in f32 unless noted; reductions run in ascending index order
 * (src/op.rs:200-409: SumReduce / MaxReduce fold left to right in f32).  The *_fast variants use
 * vectorised partial sums and OpenMP and are the timed CPU baseline; they agree with the faithful
 * forms to rounding.
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>
#ifdef _OPENMP
#include <omp.h>
#endif

/* ------------------------------------------------------------------ half / bfloat16 in software */
float orc_f16_to_f32(uint16_t h) {
    uint32_t sign = (uint32_t)(h & 0x8000u) << 16, exp = (h >> 10) & 0x1f, man = h & 0x3ffu, bits;
    if (exp == 0) {
        if (man == 0) bits = sign;
        else { /* subnormal: renormalise */
            int e = -1;
            do { man <<= 1; e++; } while (!(man & 0x400u));
            bits = sign | ((uint32_t)(127 - 15 - e) << 23) | ((man & 0x3ffu) << 13);
        }
    } else if (exp == 31) bits = sign | 0x7f800000u | (man << 13);
    else bits = sign | ((exp + 112) << 23) | (man << 13);
    float f; memcpy(&f, &bits, 4); return f;
}

uint16_t orc_f32_to_f16(float f) { /* round to nearest even */
    uint32_t x; memcpy(&x, &f, 4);
    uint32_t sign = (x >> 16) & 0x8000u, absx = x & 0x7fffffffu;
    if (absx >= 0x7f800000u) return (uint16_t)(sign | 0x7c00u | ((absx > 0x7f800000u) ? 0x200u : 0));
    if (absx >= 0x477ff000u) return (uint16_t)(sign | 0x7c00u);          /* rounds to inf */
    if (absx < 0x33000001u) return (uint16_t)sign;                      /* rounds to zero */
    int32_t e = (int32_t)(absx >> 23) - 127;
    uint32_t man = (absx & 0x7fffffu) | 0x800000u;
    uint32_t shift, half;
    if (e < -14) { shift = (uint32_t)(13 + (-14 - e)); half = 0; }       /* subnormal result */
    else { shift = 13; half = (uint32_t)(e + 15) << 10; }
    uint32_t m = man >> shift, rem = man & ((1u << shift) - 1), halfway = 1u << (shift - 1);
    if (e >= -14) m &= 0x3ffu;
    uint32_t r = half + m;   /* mantissa carry propagates into the exponent correctly */
    if (rem > halfway || (rem == halfway && (r & 1))) r++;
    return (uint16_t)(sign | r);
}

float orc_bf16_to_f32(uint16_t b) { uint32_t x = (uint32_t)b << 16; float f; memcpy(&f, &x, 4); return f; }
uint16_t orc_f32_to_bf16(float f) {
    uint32_t x; memcpy(&x, &f, 4);
    if ((x & 0x7fffffffu) > 0x7f800000u) return 0x7fc0;
    return (uint16_t)((x + 0x7fffu + ((x >> 16) & 1u)) >> 16);
}
void orc_round_bf16(float* a, int64_t n) { for (int64_t i = 0; i < n; i++) a[i] = orc_bf16_to_f32(orc_f32_to_bf16(a[i])); }
void orc_round_f16(float* a, int64_t n) { for (int64_t i = 0; i < n; i++) a[i] = orc_f16_to_f32(orc_f32_to_f16(a[i])); }

/* ------------------------------------------------------------------ seeded generators
 * h(seed, tensor, i) = mix64(key(seed, tensor) + i * 0x9E3779B97F4A7C15) with the splitmix64 finaliser. */
static uint64_t mix64(uint64_t z) {
    z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
    z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
    return z ^ (z >> 31);
}
static uint64_t gen_key(uint64_t seed, uint64_t tensor) {
    return mix64(mix64(seed + 0x9E3779B97F4A7C15ull) ^ (tensor * 0xD1B54A32D192ED03ull + 0x8CB92BA72F3D8DD7ull));
}
static uint64_t gen_hash(uint64_t key, uint64_t i) { return mix64(key + i * 0x9E3779B97F4A7C15ull); }
static double gen_uniform(uint64_t key, uint64_t i) { return ((double)(gen_hash(key, i) >> 11) + 0.5) / 9007199254740992.0; }
static double gen_gauss(uint64_t key, uint64_t i) {
    double u1 = gen_uniform(key, 2 * i), u2 = gen_uniform(key, 2 * i + 1);
    return sqrt(-2.0 * log(u1)) * cos(6.283185307179586476925286766559 * u2);
}
/* int8 quants uniform on [-127,127] */
void orc_gen_q8_quants(uint64_t seed, uint64_t tensor, int64_t n, int8_t* out) {
    uint64_t key = gen_key(seed, tensor);
#pragma omp parallel for schedule(static)
    for (int64_t i = 0; i < n; i++) out[i] = (int8_t)((int)(((gen_hash(key, (uint64_t)i) >> 32) * 255ull) >> 32) - 127);
}
/* f16 block scales |N(0,0.02)|/127 */
void orc_gen_q8_scales(uint64_t seed, uint64_t tensor, int64_t nblocks, uint16_t* out) {
    uint64_t key = gen_key(seed, tensor ^ (0x5ca1e5ull << 40));
#pragma omp parallel for schedule(static)
    for (int64_t i = 0; i < nblocks; i++) out[i] = orc_f32_to_f16((float)(fabs(0.02 * gen_gauss(key, (uint64_t)i)) / 127.0));
}
void orc_gen_normal(uint64_t seed, uint64_t tensor, int64_t n, float stddev, float* out) {
    uint64_t key = gen_key(seed, tensor);
#pragma omp parallel for schedule(static)
    for (int64_t i = 0; i < n; i++) out[i] = (float)((double)stddev * gen_gauss(key, (uint64_t)i));
}
void orc_gen_token_ids(uint64_t seed, uint64_t tensor, int64_t n, int32_t vocab, int32_t* out) {
    uint64_t key = gen_key(seed, tensor);
    for (int64_t i = 0; i < n; i++) out[i] = (int32_t)(((gen_hash(key, (uint64_t)i) >> 32) * (uint64_t)vocab) >> 32);
}

/* ------------------------------------------------------------------ Q8_0
 * Storage: crates/luminal_cuda/src/quantized.rs:30-33 - 34-byte blocks {f16 d; int8 qs[32]}, block (n,kb)
 * at byte 34*(n*K/32+kb).  Dequantisation w = (float)q * f16_to_f32(d): examples/llama/src/loader.rs:227-241. */
void orc_q8_pack(const int8_t* q, const uint16_t* d, int64_t N, int64_t K, uint8_t* bytes) {
    for (int64_t b = 0; b < N * (K / 32); b++) {
        memcpy(bytes + 34 * b, d + b, 2);
        memcpy(bytes + 34 * b + 2, q + 32 * b, 32);
    }
}
void orc_q8_unpack(const uint8_t* bytes, int64_t N, int64_t K, int8_t* q, uint16_t* d) {
    for (int64_t b = 0; b < N * (K / 32); b++) {
        memcpy(d + b, bytes + 34 * b, 2);
        memcpy(q + 32 * b, bytes + 34 * b + 2, 32);
    }
}
void orc_q8_dequant(const uint8_t* bytes, int64_t N, int64_t K, float* w) {
    for (int64_t b = 0; b < N * (K / 32); b++) {
        uint16_t d; memcpy(&d, bytes + 34 * b, 2);
        float df = orc_f16_to_f32(d);
        const int8_t* q = (const int8_t*)(bytes + 34 * b + 2);
        for (int i = 0; i < 32; i++) w[32 * b + i] = (float)q[i] * df;
    }
}

/* Faithful form: dequantise to f32 as the CPU loader does, then y[m,n] = sum_k x[m,k]*w[n,k] in ascending k
 * (matmul = broadcast multiply + SumReduce: src/hl_ops/matmul.rs:4-103, src/op.rs SumReduce). */
void orc_q8_matmul(const uint8_t* bytes, int64_t N, int64_t K, const float* x, int64_t M, float* y) {
    float* wrow = (float*)malloc((size_t)K * sizeof(float));
    for (int64_t n = 0; n < N; n++) {
        orc_q8_dequant(bytes + 34 * n * (K / 32), 1, K, wrow);
        for (int64_t m = 0; m < M; m++) {
            float acc = 0.f;
            for (int64_t k = 0; k < K; k++) acc += x[m * K + k] * wrow[k];
            y[m * N + n] = acc;
        }
    }
    free(wrow);
}

/* Baseline form on the two-plane layout: per block sum(q*x) then *d (the order of the reference GPU kernel,
 * crates/luminal_cuda/src/quantized.rs:88-97), vector partial sums, OpenMP over rows. */
void orc_q8_matmul_fast(const int8_t* q, const uint16_t* d, int64_t N, int64_t K, const float* x, int64_t M, float* y) {
    const int64_t KB = K / 32;
#pragma omp parallel for schedule(static)
    for (int64_t n = 0; n < N; n++) {
        const int8_t* qr = q + n * K;
        for (int64_t m = 0; m < M; m++) {
            const float* xr = x + m * K;
            float acc = 0.f;
            for (int64_t b = 0; b < KB; b++) {
                float s = 0.f;
#pragma omp simd reduction(+ : s)
                for (int i = 0; i < 32; i++) s += (float)qr[32 * b + i] * xr[32 * b + i];
                acc += s * orc_f16_to_f32(d[n * KB + b]);
            }
            y[m * N + n] = acc;
        }
    }
}

/* Embedding: out[t,:] = E[id_t,:]; ids travel as f32 and are truncated (crates/luminal_nn/src/embedding.rs:43-57;
 * crates/luminal_cpu/src/binary.rs:175-191). */
void orc_gather_f32(const float* table, int64_t dim, const float* ids_f32, int64_t T, float* out) {
    for (int64_t t = 0; t < T; t++) memcpy(out + t * dim, table + (int64_t)ids_f32[t] * dim, (size_t)dim * sizeof(float));
}
void orc_q8_gather(const uint8_t* bytes, int64_t dim, const float* ids_f32, int64_t T, float* out) {
    for (int64_t t = 0; t < T; t++) orc_q8_dequant(bytes + 34 * (int64_t)ids_f32[t] * (dim / 32), 1, dim, out + t * dim);
}

/* ------------------------------------------------------------------ row-wise pieces */
/* RMSNorm: x * recip(sqrt(sum(x^2) * recip(H) + eps)) * w  (src/hl_ops/unary.rs:93-104, src/hl_ops/reduction.rs:38-45,
 * crates/luminal_nn/src/norm.rs:58-70). weight may be NULL. */
void orc_rmsnorm(const float* x, const float* weight, float eps, int64_t rows, int64_t dim, float* y) {
    const float inv_n = 1.0f / (float)dim;
    for (int64_t r = 0; r < rows; r++) {
        float s = 0.f;
        for (int64_t k = 0; k < dim; k++) s += x[r * dim + k] * x[r * dim + k];
        const float rs = 1.0f / sqrtf(s * inv_n + eps);
        for (int64_t k = 0; k < dim; k++) y[r * dim + k] = x[r * dim + k] * rs * (weight ? weight[k] : 1.0f);
    }
}

/* Softmax over the last dim: e = exp2((x - max) * (1/ln2)); p = e * recip(sum e)  (src/hl_ops/unary.rs:34-36,126-130). */
void orc_softmax(const float* x, int64_t rows, int64_t cols, float* y) {
    for (int64_t r = 0; r < rows; r++) {
        float m = x[r * cols];
        for (int64_t j = 1; j < cols; j++) m = fmaxf(m, x[r * cols + j]);
        float s = 0.f;
        for (int64_t j = 0; j < cols; j++) { float e = exp2f((x[r * cols + j] - m) * 1.4426950408889634f); y[r * cols + j] = e; s += e; }
        const float inv = 1.0f / s;
        for (int64_t j = 0; j < cols; j++) y[r * cols + j] *= inv;
    }
}

/* swish(g) = g * 1/(1+exp(-g)); out = up * swish(gate)  (src/hl_ops/unary.rs:169-177, examples/llama/src/model.rs:27-31). */
void orc_swiglu(const float* gate, const float* up, int64_t n, float* out) {
    for (int64_t i = 0; i < n; i++) out[i] = up[i] * (gate[i] * (1.0f / (1.0f + expf(-gate[i]))));
}

/* RoPE on x [T, heads, head_dim], interleaved pairs (examples/llama/src/model.rs:52-72):
 * f_i = recip(exp(((2 i) * (1/d)) * ln(theta))) (F32Pow: src/hl_ops/binary.rs:301-309); a = pos * f_i;
 * cos(a) = sin(pi/2 - a) (src/hl_ops/unary.rs:64-66). */
void orc_rope_inv_freq(float theta, int head_dim, float* inv_freq) {
    const float ln_theta = logf(fabsf(theta)), inv_d = 1.0f / (float)head_dim;
    for (int i = 0; i < head_dim / 2; i++) inv_freq[i] = 1.0f / expf((((float)i) * 2.0f) * inv_d * ln_theta);
}
void orc_rope(float* x, const int32_t* positions, int64_t T, int heads, int head_dim, float theta) {
    float inv_freq[256];
    orc_rope_inv_freq(theta, head_dim, inv_freq);
    for (int64_t t = 0; t < T; t++)
        for (int h = 0; h < heads; h++)
            for (int i = 0; i < head_dim / 2; i++) {
                const float a = (float)positions[t] * inv_freq[i];
                const float sn = sinf(a), cs = sinf(1.5707964f - a);
                float* p = x + (t * heads + h) * head_dim + 2 * i;
                const float x0 = p[0], x1 = p[1];
                p[0] = x0 * cs - x1 * sn;
                p[1] = x0 * sn + x1 * cs;
            }
}

/* Half-split RoPE of the qwen decoder (examples/qwen/src/model.rs:52-77): freqs = [f, f], rotated = [-x[d/2:], x[:d/2]],
 * out = x * cos(freqs) + rotated * sin(freqs); so pair (x[i], x[i + d/2]) is rotated by pos * f_i. */
void orc_rope_half(float* x, const int32_t* positions, int64_t T, int heads, int head_dim, float theta) {
    float inv_freq[256];
    orc_rope_inv_freq(theta, head_dim, inv_freq);
    const int h2 = head_dim / 2;
    for (int64_t t = 0; t < T; t++)
        for (int h = 0; h < heads; h++)
            for (int i = 0; i < h2; i++) {
                const float a = (float)positions[t] * inv_freq[i];
                const float sn = sinf(a), cs = sinf(1.5707964f - a);
                float* p = x + (t * heads + h) * head_dim;
                const float x0 = p[i], x1 = p[i + h2];
                p[i] = x0 * cs - x1 * sn;
                p[i + h2] = x1 * cs + x0 * sn;
            }
}

/* triu(size, diagonal): 1 where col - row >= diagonal (src/hl_ops/other.rs:103-109). */
void orc_triu(int size, int diagonal, float* out) {
    for (int r = 0; r < size; r++) for (int c = 0; c < size; c++) out[r * size + c] = (c - r >= diagonal) ? 1.0f : 0.0f;
}

/* Greedy sampler (examples/llama/src/main.rs:194-198): position_max_by(partial_cmp.unwrap_or(Equal)) keeps the
 * running maximum unless it is strictly greater than the next element; so the LAST maximum wins and a NaN is
 * replaced by whatever follows it. */
int32_t orc_argmax(const float* v, int64_t n) {
    int64_t best = 0; float cur = v[0];
    for (int64_t i = 1; i < n; i++) if (!(cur > v[i])) { cur = v[i]; best = i; }
    return (int32_t)best;
}

/* Temperature / top-p sampler.  The reference only samples greedily (examples/llama/src/main.rs:194-198); this sampler has
 * no counterpart there and is specified here, in integers wherever a result could depend on the order of operations, so
 * that a parallel implementation reproduces it bit for bit:
 *   m    = the largest logit that is not a NaN (a row without one falls back to the greedy rule)
 *   z_i  = (l_i - m) * (1 / temperature), each operation rounded to f32
 *   w_i  = trunc(2^30 * e^z_i) by orc_sample_weight below (a fixed sequence of f32 operations); NaN and -inf give 0
 *   W    = sum of w_i;  P = max(1, (uint64)((double)top_p * (double)W)), P = W for top_p >= 1
 *   tau  = the largest integer with S(tau) = sum of the w_i >= tau  >=  P;  the nucleus is {i : w_i >= tau}
 *   r    = floor(u * S(tau) / 2^64), u = mix64(mix64(seed + GOLDEN * (seq + 1)) + pos)
 *   the sampled token is the first index i of the nucleus, in index order, whose running sum of w exceeds r. */
static uint32_t orc_sample_weight(float z) {
    if (!(z > -21.5f)) return 0;                      /* also NaN; 2^30 e^-21.5 < 1 */
    if (z > 0.f) z = 0.f;
    const float t = z * 1.44269504f;
    const float n = rintf(t);                         /* round to nearest even */
    const float f = t - n;                            /* exact, |f| <= 0.5 */
    float p = 1.5403530e-4f;                          /* 2^f = e^(f ln 2), Taylor coefficients, Horner with fused multiply-adds */
    p = fmaf(p, f, 1.3333558e-3f);
    p = fmaf(p, f, 9.6181291e-3f);
    p = fmaf(p, f, 5.5504109e-2f);
    p = fmaf(p, f, 2.4022651e-1f);
    p = fmaf(p, f, 6.9314718e-1f);
    p = fmaf(p, f, 1.0f);
    union { uint32_t u; float v; } sc;
    sc.u = (uint32_t)(127 + 30 + (int)n) << 23;       /* 2^(n + 30), n in [-32, 0] */
    return (uint32_t)(p * sc.v);                      /* exact scaling, then truncation */
}

int32_t orc_sample_top_p(const float* logits, int64_t n, float temperature, float top_p, uint64_t seed, uint64_t seq, uint64_t pos) {
    float m = -INFINITY; int any = 0;
    for (int64_t i = 0; i < n; i++) if (logits[i] == logits[i]) { if (!any || logits[i] > m) m = logits[i]; any = 1; }
    if (!any || !(m > -INFINITY) || !(temperature > 0.f)) return orc_argmax(logits, n);
    const float inv_t = 1.0f / temperature;
    uint32_t* w = (uint32_t*)malloc((size_t)n * sizeof(uint32_t));
    uint64_t W = 0;
    for (int64_t i = 0; i < n; i++) {
        const float d = logits[i] - m;
        w[i] = orc_sample_weight(d * inv_t);
        W += w[i];
    }
    uint64_t P = top_p >= 1.f ? W : (uint64_t)((double)top_p * (double)W);
    if (P < 1) P = 1;
    uint32_t lo = 1, hi = 0x7fffffffu;                /* S(lo) >= P always holds for lo = 1 */
    while (lo < hi) {
        const uint32_t mid = lo + (hi - lo + 1) / 2;
        uint64_t S = 0;
        for (int64_t i = 0; i < n; i++) if (w[i] >= mid) S += w[i];
        if (S >= P) lo = mid; else hi = mid - 1;
    }
    const uint32_t tau = lo;
    uint64_t S = 0;
    for (int64_t i = 0; i < n; i++) if (w[i] >= tau) S += w[i];
    const uint64_t u = mix64(mix64(seed + 0x9E3779B97F4A7C15ull * (seq + 1)) + pos);
    const uint64_t r = (uint64_t)(((unsigned __int128)u * S) >> 64);
    uint64_t run = 0; int32_t pick = -1;
    for (int64_t i = 0; i < n && pick < 0; i++)
        if (w[i] >= tau) { run += w[i]; if (run > r) pick = (int32_t)i; }
    free(w);
    return pick < 0 ? orc_argmax(logits, n) : pick;
}

/* ------------------------------------------------------------------ attention
 * q [T, nq, d]; K,V contiguous caches [nkv, ctx_cap, d] holding p+T valid positions (the new rows already
 * appended at p..p+T, examples/llama/src/model.rs:108-110).  Scores S = (q.k)/sqrt(d) for j in [0,p+T), plus
 * -65504 where j - p > t (additive f16::MIN mask, model.rs:116-127), softmax, out = P.V; q head h uses kv head
 * h / (nq/nkv) (model.rs:113-119).  out [T, nq*d]. */
void orc_attention(const float* q, const float* kc, const float* vc, int64_t T, int64_t p, int nq, int nkv, int d,
                   int64_t ctx_cap, float* out) {
    const int g = nq / nkv;
    const int64_t L = p + T;
    const float inv_sqrt_d = 1.0f / sqrtf((float)d);
#pragma omp parallel for collapse(2) schedule(static)
    for (int64_t t = 0; t < T; t++)
        for (int h = 0; h < nq; h++) {
            float* s = (float*)malloc((size_t)L * sizeof(float));
            const float* qv = q + (t * nq + h) * d;
            const float* kh = kc + (int64_t)(h / g) * ctx_cap * d;
            const float* vh = vc + (int64_t)(h / g) * ctx_cap * d;
            for (int64_t j = 0; j < L; j++) {
                float a = 0.f;
                for (int c = 0; c < d; c++) a += qv[c] * kh[j * d + c];
                s[j] = a * inv_sqrt_d + ((j - p > t) ? -65504.0f : 0.0f);
            }
            orc_softmax(s, 1, L, s);
            float* o = out + (t * nq + h) * d;
            for (int c = 0; c < d; c++) o[c] = 0.f;
            for (int64_t j = 0; j < L; j++)
                for (int c = 0; c < d; c++) o[c] += s[j] * vh[j * d + c];
            free(s);
        }
}

/* ------------------------------------------------------------------ Llama forward (examples/llama/src/model.rs:171-248)
 * Weights stay quantised (two-plane form) and are dequantised on the fly: int8 * f16 is exact in f32, so this equals
 * the reference CPU loader's f32 weights bit for bit. */
typedef struct orc_q8 { const int8_t* q; const uint16_t* d; int64_t N, K; } orc_q8;
typedef struct orc_llama {
    int32_t layers, hidden, q_heads, kv_heads, head_dim, ffn, vocab;
    float eps, theta;
    const float* embed;                 /* [vocab, hidden] f32 */
    const float* out_norm;              /* [hidden] */
    orc_q8 head;                        /* [vocab, hidden] */
    const float** attn_norm;            /* per layer [hidden] */
    const float** ffn_norm;
    orc_q8 *wq, *wk, *wv, *wo, *wgate, *wup, *wdown;   /* per layer */
    float** kcache;                     /* per layer [kv_heads, ctx_cap, head_dim] */
    float** vcache;
    int64_t ctx_cap;
    int32_t round_mode;                 /* 0: f32 activations; 2: round activations to bf16 after every op */
    /* sibling decoders (all zero / NULL = Llama): examples/qwen/src/model.rs, examples/phi/src/model.rs */
    int32_t rope_mode;                  /* 0 interleaved pairs, 1 half-split pairs */
    int32_t qk_norm;                    /* per-head RMSNorm with weight on q and k before RoPE (qwen model.rs:93-105) */
    int32_t tie_head;                   /* logits = x . embedding^T (qwen model.rs:233) */
    const float** q_norm;               /* per layer [head_dim] */
    const float** k_norm;
    orc_q8 embed_q8;                    /* Q8_0 embedding table (q == NULL: the f32 table `embed` is used) */
} orc_llama;

static void act_round(const orc_llama* m, float* a, int64_t n) { if (m->round_mode == 2) orc_round_bf16(a, n); else if (m->round_mode == 1) orc_round_f16(a, n); }
static void linear(const orc_q8* w, const float* x, int64_t M, float* y) { orc_q8_matmul_fast(w->q, w->d, w->N, w->K, x, M, y); }

/* Runs T tokens at positions [p, p+T); writes logits of the LAST position (examples/llama/src/main.rs:58-61).
 * Returns 0, or -1 on allocation failure / cache overflow. */
int orc_llama_forward(const orc_llama* m, const int32_t* ids, int64_t T, int64_t p, float* logits) {
    const int H = m->hidden, nq = m->q_heads, nkv = m->kv_heads, d = m->head_dim, F = m->ffn;
    if (p + T > m->ctx_cap) return -1;
    float* x = (float*)malloc((size_t)T * H * 4), *r = (float*)malloc((size_t)T * H * 4);
    float* qb = (float*)malloc((size_t)T * nq * d * 4), *kb = (float*)malloc((size_t)T * nkv * d * 4), *vb = (float*)malloc((size_t)T * nkv * d * 4);
    float* ao = (float*)malloc((size_t)T * nq * d * 4), *y = (float*)malloc((size_t)T * H * 4);
    float* gt = (float*)malloc((size_t)T * F * 4), *up = (float*)malloc((size_t)T * F * 4);
    int32_t* pos = (int32_t*)malloc((size_t)T * 4);
    if (!x || !r || !qb || !kb || !vb || !ao || !y || !gt || !up || !pos) return -1;
    for (int64_t t = 0; t < T; t++) {
        pos[t] = (int32_t)(p + t);
        if (m->embed_q8.q) {           /* w = (float)q * d, row ids[t] (crates/luminal_cuda/src/quantized.rs:202-233) */
            const int8_t* qr = m->embed_q8.q + (int64_t)ids[t] * H;
            const uint16_t* dr = m->embed_q8.d + (int64_t)ids[t] * (H / 32);
            for (int k = 0; k < H; k++) x[t * H + k] = (float)qr[k] * orc_f16_to_f32(dr[k / 32]);
        } else memcpy(x + t * H, m->embed + (int64_t)ids[t] * H, (size_t)H * 4);
    }
    act_round(m, x, T * H);
    for (int l = 0; l < m->layers; l++) {
        orc_rmsnorm(x, m->attn_norm[l], m->eps, T, H, r); act_round(m, r, T * H);
        linear(&m->wq[l], r, T, qb); linear(&m->wk[l], r, T, kb); linear(&m->wv[l], r, T, vb);
        act_round(m, qb, T * nq * d); act_round(m, kb, T * nkv * d); act_round(m, vb, T * nkv * d);
        if (m->qk_norm) {              /* LayerNorm(head_dim, weight, no bias, no mean) over every head */
            orc_rmsnorm(qb, m->q_norm[l], m->eps, T * nq, d, qb); orc_rmsnorm(kb, m->k_norm[l], m->eps, T * nkv, d, kb);
            act_round(m, qb, T * nq * d); act_round(m, kb, T * nkv * d);
        }
        if (m->rope_mode == 1) { orc_rope_half(qb, pos, T, nq, d, m->theta); orc_rope_half(kb, pos, T, nkv, d, m->theta); }
        else { orc_rope(qb, pos, T, nq, d, m->theta); orc_rope(kb, pos, T, nkv, d, m->theta); }
        act_round(m, qb, T * nq * d); act_round(m, kb, T * nkv * d);
        for (int64_t t = 0; t < T; t++)
            for (int h = 0; h < nkv; h++) {
                memcpy(m->kcache[l] + ((int64_t)h * m->ctx_cap + p + t) * d, kb + (t * nkv + h) * d, (size_t)d * 4);
                memcpy(m->vcache[l] + ((int64_t)h * m->ctx_cap + p + t) * d, vb + (t * nkv + h) * d, (size_t)d * 4);
            }
        orc_attention(qb, m->kcache[l], m->vcache[l], T, p, nq, nkv, d, m->ctx_cap, ao); act_round(m, ao, T * nq * d);
        linear(&m->wo[l], ao, T, y);
        for (int64_t i = 0; i < T * H; i++) x[i] += y[i];
        act_round(m, x, T * H);
        orc_rmsnorm(x, m->ffn_norm[l], m->eps, T, H, r); act_round(m, r, T * H);
        linear(&m->wgate[l], r, T, gt); linear(&m->wup[l], r, T, up);
        orc_swiglu(gt, up, T * F, gt); act_round(m, gt, T * F);
        linear(&m->wdown[l], gt, T, y);
        for (int64_t i = 0; i < T * H; i++) x[i] += y[i];
        act_round(m, x, T * H);
    }
    orc_rmsnorm(x + (T - 1) * H, m->out_norm, m->eps, 1, H, r); act_round(m, r, H);
    linear(m->tie_head ? &m->embed_q8 : &m->head, r, 1, logits);
    free(x); free(r); free(qb); free(kb); free(vb); free(ao); free(y); free(gt); free(up); free(pos);
    return 0;
}

int orc_num_threads(void) {
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}
void orc_set_num_threads(int n) {
#ifdef _OPENMP
    omp_set_num_threads(n);
#else
    (void)n;
#endif
}
