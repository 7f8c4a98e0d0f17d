// Elementwise / row-wise family: gathers, RMSNorm(+residual), interleaved RoPE, SwiGLU, add,
// row softmax and the greedy argmax.  All are bound by HBM (or L2) bandwidth; every kernel moves
// 16 bytes per thread per access and computes in f32.
//
// They stand in for luminal's CudaStdNorm (crates/luminal_cuda/src/unary.rs:170-302), CudaSoftmax
// (unary.rs:493-593), CudaGather (binary.rs:279-344), QuantizedGather (quantized.rs:170-233) and
// the generated FusedElementwiseOp kernels (elementwise_fusion.rs:432-453) that carry RoPE, SwiGLU
// and the residual adds of examples/llama/src/model.rs.
#include "common.cuh"
#include <math.h>

template <typename T> struct Vec16 { static constexpr int N = 16 / sizeof(T); };

template <typename T>
__device__ __forceinline__ void load_vec(const T* p, float* o) {
    constexpr int N = Vec16<T>::N;
    const int4 raw = *reinterpret_cast<const int4*>(p);
    const T* e = reinterpret_cast<const T*>(&raw);
#pragma unroll
    for (int i = 0; i < N; i++) o[i] = to_f32<T>(e[i]);
}
template <typename T>
__device__ __forceinline__ void store_vec(T* p, const float* v) {
    constexpr int N = Vec16<T>::N;
    int4 raw;
    T* e = reinterpret_cast<T*>(&raw);
#pragma unroll
    for (int i = 0; i < N; i++) e[i] = from_f32<T>(v[i]);
    *reinterpret_cast<int4*>(p) = raw;
}

// ------------------------------------------------------------------ gathers
template <typename TI, typename TO>
__global__ void gather_rows_kernel(const TI* __restrict__ table, int64_t rows, int64_t dim,
                                   const int32_t* __restrict__ ids, int64_t T, TO* __restrict__ out, int* err) {
    const int64_t t = blockIdx.x;
    int64_t id = ids[t];
    if (id < 0 || id >= rows) { if (threadIdx.x == 0) atomicOr(err, 0x10); id = 0; }
    for (int64_t j = threadIdx.x; j < dim; j += blockDim.x)
        out[t * dim + j] = from_f32<TO>(to_f32<TI>(table[id * dim + j]));
}

template <typename TO>
__global__ void q8_gather_kernel(const int8_t* __restrict__ q, const __half* __restrict__ d, int64_t rows, int64_t dim,
                                 const int32_t* __restrict__ ids, TO* __restrict__ out, int* err) {
    const int64_t t = blockIdx.x;
    int64_t id = ids[t];
    if (id < 0 || id >= rows) { if (threadIdx.x == 0) atomicOr(err, 0x10); id = 0; }
    for (int64_t j = threadIdx.x; j < dim; j += blockDim.x) {
        const float w = (float)q[id * dim + j] * __half2float(d[id * (dim >> 5) + (j >> 5)]);
        out[t * dim + j] = from_f32<TO>(w);
    }
}

// ------------------------------------------------------------------ RMSNorm
// one CTA per row; the row is read once from global and kept in registers (dim <= 16 * blockDim * VPT)
template <typename T, int VPT>
__global__ void __launch_bounds__(256) rmsnorm_kernel(const T* __restrict__ x, const T* __restrict__ residual,
                                                      const float* __restrict__ weight, float eps, T* __restrict__ y,
                                                      T* __restrict__ sum_out, int64_t dim) {
    constexpr int N = Vec16<T>::N;
    __shared__ float red[8];
    __shared__ float rs_sh;
    const int64_t row = blockIdx.x;
    const T* xr = x + row * dim;
    float v[VPT][N];
    float ss = 0.f;
#pragma unroll
    for (int i = 0; i < VPT; i++) {
        const int64_t k = ((int64_t)i * blockDim.x + threadIdx.x) * N;
        if (k < dim) {
            load_vec<T>(xr + k, v[i]);
            if (residual) {
                float r[N];
                load_vec<T>(residual + row * dim + k, r);
#pragma unroll
                for (int j = 0; j < N; j++) v[i][j] = to_f32<T>(from_f32<T>(v[i][j] + r[j]));
                if (sum_out) store_vec<T>(sum_out + row * dim + k, v[i]);
            }
#pragma unroll
            for (int j = 0; j < N; j++) ss += v[i][j] * v[i][j];
        }
    }
    ss = warp_sum(ss);
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = ss;
    __syncthreads();
    if (threadIdx.x == 0) {
        float s = 0.f;
        for (int w = 0; w < (int)(blockDim.x >> 5); w++) s += red[w];
        rs_sh = rsqrtf(s / (float)dim + eps);
    }
    __syncthreads();
    const float rs = rs_sh;
#pragma unroll
    for (int i = 0; i < VPT; i++) {
        const int64_t k = ((int64_t)i * blockDim.x + threadIdx.x) * N;
        if (k < dim) {
            float o[N];
#pragma unroll
            for (int j = 0; j < N; j++) o[j] = v[i][j] * rs * (weight ? weight[k + j] : 1.f);
            store_vec<T>(y + row * dim + k, o);
        }
    }
}

// ------------------------------------------------------------------ RoPE (interleaved pairs)
template <typename T>
__global__ void rope_kernel(T* __restrict__ x, const int32_t* __restrict__ positions, int64_t T_, int heads,
                            int head_dim, const RopeFreqs f) {
    const int half = head_dim >> 1;
    const int64_t total = T_ * heads * half;
    for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
        const int pi = (int)(i % half);
        const int64_t th = i / half;
        const int64_t t = th / heads;
        const float a = (float)positions[t] * f.inv_freq[pi];
        const float sn = sinf(a), cs = sinf(1.5707964f - a);   // cos(x) = sin(pi/2 - x), src/hl_ops/unary.rs:64-66
        T* p = x + th * head_dim + 2 * pi;
        const float x0 = to_f32<T>(p[0]), x1 = to_f32<T>(p[1]);
        p[0] = from_f32<T>(x0 * cs - x1 * sn);
        p[1] = from_f32<T>(x0 * sn + x1 * cs);
    }
}

// Per-head RMSNorm (optional) + RoPE of the q and k heads of fused qkv rows, in place: one warp per (token, head).
// Values are rounded to the activation type where the reference's ops would round them (after the norm, after the rotation).
template <typename T>
__global__ void qk_norm_rope_kernel(T* __restrict__ qkv, const int32_t* __restrict__ positions, int64_t T_, int nq, int nkv, int d,
                                    const float* __restrict__ qw, const float* __restrict__ kw, float eps, const RopeFreqs f, int mode) {
    const int lane = threadIdx.x & 31;
    const int64_t warp = (blockIdx.x * (int64_t)blockDim.x + threadIdx.x) >> 5, nwarps = ((int64_t)gridDim.x * blockDim.x) >> 5;
    const int heads = nq + nkv, row = (nq + 2 * nkv) * d, half = d >> 1;
    for (int64_t i = warp; i < T_ * heads; i += nwarps) {
        const int64_t t = i / heads;
        const int h = (int)(i - t * heads);
        T* p = qkv + t * row + (int64_t)h * d;
        const float* w = h < nq ? qw : kw;
        float rs = 1.f;
        if (w) {
            float ss = 0.f;
            for (int c = lane; c < d; c += 32) { const float v = to_f32<T>(p[c]); ss += v * v; }
            rs = rsqrtf(warp_sum(ss) / (float)d + eps);
        }
        const float pos = (float)positions[t];
        for (int pi = lane; pi < half; pi += 32) {
            const int i0 = mode == 0 ? 2 * pi : pi, i1 = mode == 0 ? 2 * pi + 1 : pi + half;
            float x0 = to_f32<T>(p[i0]), x1 = to_f32<T>(p[i1]);
            if (w) { x0 = to_f32<T>(from_f32<T>(x0 * rs * w[i0])); x1 = to_f32<T>(from_f32<T>(x1 * rs * w[i1])); }
            const float a = pos * f.inv_freq[pi];
            const float sn = sinf(a), cs = sinf(1.5707964f - a);
            p[i0] = from_f32<T>(x0 * cs - x1 * sn);
            p[i1] = from_f32<T>(x1 * cs + x0 * sn);
        }
    }
}

void blum_rope_freqs(float theta, int head_dim, RopeFreqs* f) {
    // f_i = recip(exp(((2 i) * (1/d)) * ln(theta))) in f32, as examples/llama/src/model.rs:56-57 with
    // F32Pow = exp(t * ln|base|) (src/hl_ops/binary.rs:301-309)
    // theta <= 0 asks for no rotation at all (all angles zero): the rotation was applied by an earlier kernel
    if (!(theta > 0.f)) { for (int i = 0; i < 128; i++) f->inv_freq[i] = 0.f; return; }
    const float ln_theta = logf(fabsf(theta));
    const float inv_d = 1.0f / (float)head_dim;
    for (int i = 0; i < head_dim / 2 && i < 128; i++) {
        const float t = ((float)i * 2.0f) * inv_d;
        f->inv_freq[i] = 1.0f / expf(t * ln_theta);
    }
}

// ------------------------------------------------------------------ SwiGLU, add
// rows of [gate | up] (2 F columns: one matmul over the stacked gate / up matrix) -> out [R][F]
template <typename T>
__global__ void swiglu_rows_kernel(const T* __restrict__ gu, T* __restrict__ out, int64_t R, int64_t F) {
    constexpr int N = Vec16<T>::N;
    const int64_t per_row = F / N, nv = R * per_row;
    for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < nv; i += (int64_t)gridDim.x * blockDim.x) {
        const int64_t r = i / per_row, c = (i - r * per_row) * N;
        float g[N], u[N], o[N];
        load_vec<T>(gu + r * 2 * F + c, g);
        load_vec<T>(gu + r * 2 * F + F + c, u);
#pragma unroll
        for (int j = 0; j < N; j++) o[j] = u[j] * (g[j] * (1.f / (1.f + expf(-g[j]))));
        store_vec<T>(out + r * F + c, o);
    }
}

template <typename T>
__global__ void swiglu_kernel(const T* __restrict__ gate, const T* __restrict__ up, T* __restrict__ out, int64_t n) {
    constexpr int N = Vec16<T>::N;
    const int64_t nv = n / N;
    for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < nv; i += (int64_t)gridDim.x * blockDim.x) {
        float g[N], u[N], o[N];
        load_vec<T>(gate + i * N, g);
        load_vec<T>(up + i * N, u);
#pragma unroll
        for (int j = 0; j < N; j++) o[j] = u[j] * (g[j] * (1.f / (1.f + expf(-g[j]))));
        store_vec<T>(out + i * N, o);
    }
    if (blockIdx.x == 0 && threadIdx.x < (n % N)) {
        const int64_t i = nv * N + threadIdx.x;
        const float g = to_f32<T>(gate[i]), u = to_f32<T>(up[i]);
        out[i] = from_f32<T>(u * (g * (1.f / (1.f + expf(-g)))));
    }
}

template <typename T>
__global__ void add_kernel(const T* __restrict__ a, const T* __restrict__ b, T* __restrict__ out, int64_t n) {
    constexpr int N = Vec16<T>::N;
    const int64_t nv = n / N;
    for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < nv; i += (int64_t)gridDim.x * blockDim.x) {
        float x[N], y[N];
        load_vec<T>(a + i * N, x);
        load_vec<T>(b + i * N, y);
#pragma unroll
        for (int j = 0; j < N; j++) x[j] += y[j];
        store_vec<T>(out + i * N, x);
    }
    if (blockIdx.x == 0 && threadIdx.x < (n % N)) {
        const int64_t i = nv * N + threadIdx.x;
        out[i] = from_f32<T>(to_f32<T>(a[i]) + to_f32<T>(b[i]));
    }
}

// ------------------------------------------------------------------ softmax (one CTA per row)
template <typename T>
__global__ void __launch_bounds__(256) softmax_kernel(const T* __restrict__ x, T* __restrict__ y, int64_t cols) {
    __shared__ float red[8];
    __shared__ float bc;
    const T* xr = x + blockIdx.x * cols;
    T* yr = y + blockIdx.x * cols;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = blockDim.x >> 5;
    float m = -INFINITY;
    for (int64_t j = threadIdx.x; j < cols; j += blockDim.x) m = fmaxf(m, to_f32<T>(xr[j]));
    m = warp_max(m);
    if (lane == 0) red[warp] = m;
    __syncthreads();
    if (threadIdx.x == 0) { float v = red[0]; for (int w = 1; w < nw; w++) v = fmaxf(v, red[w]); bc = v; }
    __syncthreads();
    m = bc;
    float s = 0.f;
    // exp(x) = exp2(x * 1/ln2)  (src/hl_ops/unary.rs:34-36)
    for (int64_t j = threadIdx.x; j < cols; j += blockDim.x) s += exp2f((to_f32<T>(xr[j]) - m) * 1.4426950408889634f);
    s = warp_sum(s);
    __syncthreads();
    if (lane == 0) red[warp] = s;
    __syncthreads();
    if (threadIdx.x == 0) { float v = 0.f; for (int w = 0; w < nw; w++) v += red[w]; bc = 1.f / v; }
    __syncthreads();
    const float inv = bc;
    for (int64_t j = threadIdx.x; j < cols; j += blockDim.x)
        yr[j] = from_f32<T>(exp2f((to_f32<T>(xr[j]) - m) * 1.4426950408889634f) * inv);
}

// ------------------------------------------------------------------ argmax
// examples/llama/src/main.rs:194-198 folds `position_max_by(partial_cmp.unwrap_or(Equal))`: the running
// maximum is replaced whenever it is not strictly greater than the next element.  Without NaNs that is
// "the last index holding the maximum", which is order-independent and is what the parallel path
// computes.  A row that contains a NaN takes the sequential path so the fold is reproduced exactly.
template <typename T>
__global__ void __launch_bounds__(1024) argmax_kernel(const T* __restrict__ x, int64_t cols, int32_t* __restrict__ out) {
    __shared__ float sv[32];
    __shared__ int si[32];
    __shared__ int snan;
    const T* xr = x + blockIdx.x * cols;
    if (threadIdx.x == 0) snan = 0;
    __syncthreads();
    float bv = -INFINITY; int bi = -1; bool has_nan = false;
    for (int64_t j = threadIdx.x; j < cols; j += blockDim.x) {
        const float v = to_f32<T>(xr[j]);
        if (v != v) has_nan = true;
        if (v > bv || (v == bv && (int)j > bi) || bi < 0) { bv = v; bi = (int)j; }
    }
    if (has_nan) snan = 1;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
        const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
        if (oi >= 0 && (bi < 0 || ov > bv || (ov == bv && oi > bi))) { bv = ov; bi = oi; }
    }
    if ((threadIdx.x & 31) == 0) { sv[threadIdx.x >> 5] = bv; si[threadIdx.x >> 5] = bi; }
    __syncthreads();
    if (threadIdx.x == 0) {
        if (snan) {
            float cur = to_f32<T>(xr[0]); int ci = 0;
            for (int64_t j = 1; j < cols; j++) {
                const float v = to_f32<T>(xr[j]);
                if (!(cur > v)) { cur = v; ci = (int)j; }
            }
            out[blockIdx.x] = ci;
        } else {
            for (int w = 1; w < (int)(blockDim.x >> 5); w++) {
                if (si[w] >= 0 && (bi < 0 || sv[w] > bv || (sv[w] == bv && si[w] > bi))) { bv = sv[w]; bi = si[w]; }
            }
            out[blockIdx.x] = bi;
        }
    }
}

// The same rule with a row split over several CTAs (a 128256-column row is 0.5 MB: one CTA per row reaches a fraction of
// the memory rate).  Every CTA folds its part into a 64-bit key {order-preserving image of the value, index} and joins
// it with atomicMax: the largest key is the last index holding the maximum.  The CTA that arrives last at the row's
// counter writes the index and returns the row's scratch record to zero, so one launch does the whole job.
// -0.0 enters as +0.0 (the two compare equal in the reference's fold); a row with a NaN is folded sequentially.
struct ArgmaxRec { unsigned long long key; unsigned int nan, arrived; };

__global__ void __launch_bounds__(512) argmax_split_kernel(const float* __restrict__ x, int64_t cols, int splits, ArgmaxRec* __restrict__ rec,
                                                           int32_t* __restrict__ out) {
    __shared__ unsigned long long sk[16];
    __shared__ int snan;
    const int row = blockIdx.x / splits, part = blockIdx.x - row * splits;
    const float* xr = x + (size_t)row * cols;
    // parts are whole float4 groups when the row allows it
    const int64_t per = (((cols + splits - 1) / splits) + 3) & ~(int64_t)3;
    const int64_t beg = per * part, end = min(cols, beg + per);
    if (threadIdx.x == 0) snan = 0;
    __syncthreads();
    unsigned long long best = 0;
    bool has_nan = false;
    auto take = [&](float v, int64_t j) {
        if (v != v) has_nan = true;
        if (v == 0.f) v = 0.f;
        const unsigned int b = __float_as_uint(v);
        const unsigned long long k = ((unsigned long long)(b ^ ((b >> 31) ? 0xffffffffu : 0x80000000u)) << 32) | (unsigned int)j;
        best = k > best ? k : best;
    };
    if ((cols & 3) == 0 && ((uintptr_t)x & 15) == 0) {
        for (int64_t j = beg + 4 * (int64_t)threadIdx.x; j < end; j += 4 * (int64_t)blockDim.x) {
            const float4 v = *reinterpret_cast<const float4*>(xr + j);
            take(v.x, j); take(v.y, j + 1); take(v.z, j + 2); take(v.w, j + 3);
        }
    } else {
        for (int64_t j = beg + threadIdx.x; j < end; j += blockDim.x) take(xr[j], j);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const unsigned long long ok = __shfl_xor_sync(0xffffffffu, best, o);
        best = ok > best ? ok : best;
    }
    if (has_nan) snan = 1;
    if ((threadIdx.x & 31) == 0) sk[threadIdx.x >> 5] = best;
    __syncthreads();
    if (threadIdx.x == 0) {
        for (int w = 1; w < (int)(blockDim.x >> 5); w++) best = sk[w] > best ? sk[w] : best;
        ArgmaxRec* r = rec + row;
        atomicMax(&r->key, best);
        if (snan) atomicOr(&r->nan, 1u);
        __threadfence();
        if (atomicAdd(&r->arrived, 1u) == (unsigned)splits - 1) {
            __threadfence();
            const unsigned long long k = atomicMax(&r->key, 0ull);
            int idx = (int)(unsigned int)k;
            if (atomicOr(&r->nan, 0u)) {
                float cur = xr[0]; idx = 0;
                for (int64_t j = 1; j < cols; j++) {
                    const float v = xr[j];
                    if (!(cur > v)) { cur = v; idx = (int)j; }
                }
            }
            out[row] = idx;
            r->key = 0; r->nan = 0;
            __threadfence();
            r->arrived = 0;
        }
    }
}

// Vocabulary-parallel argmax: each rank reduces its slice to (max value, global index) per row; the pairs of all
// ranks are then merged with the same "last maximum wins" rule (a higher rank holds higher global indices).
__global__ void __launch_bounds__(1024) argmax_pairs_kernel(const float* __restrict__ x, int64_t cols, int index_offset,
                                                            int32_t* __restrict__ pairs) {
    __shared__ float sv[32];
    __shared__ int si[32];
    const float* xr = x + blockIdx.x * cols;
    float bv = -INFINITY; int bi = -1;
    for (int64_t j = threadIdx.x; j < cols; j += blockDim.x) {
        const float v = xr[j];
        if (bi < 0 || v > bv || (v == bv && (int)j > bi)) { bv = v; bi = (int)j; }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
        const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
        if (oi >= 0 && (bi < 0 || ov > bv || (ov == bv && oi > bi))) { bv = ov; bi = oi; }
    }
    if ((threadIdx.x & 31) == 0) { sv[threadIdx.x >> 5] = bv; si[threadIdx.x >> 5] = bi; }
    __syncthreads();
    if (threadIdx.x == 0) {
        for (int w = 1; w < (int)(blockDim.x >> 5); w++)
            if (si[w] >= 0 && (bi < 0 || sv[w] > bv || (sv[w] == bv && si[w] > bi))) { bv = sv[w]; bi = si[w]; }
        pairs[2 * blockIdx.x] = __float_as_int(bv);
        pairs[2 * blockIdx.x + 1] = bi + index_offset;
    }
}

__global__ void pick_pairs_kernel(const int32_t* __restrict__ pairs, int nranks, int64_t rows, int32_t* __restrict__ out) {
    const int64_t r = blockIdx.x * (int64_t)blockDim.x + threadIdx.x;
    if (r >= rows) return;
    float bv = -INFINITY; int bi = -1;
    for (int k = 0; k < nranks; k++) {
        const float v = __int_as_float(pairs[((int64_t)k * rows + r) * 2]);
        const int i = pairs[((int64_t)k * rows + r) * 2 + 1];
        if (bi < 0 || v > bv || (v == bv && i > bi)) { bv = v; bi = i; }
    }
    out[r] = bi;
}

int blum_argmax_pairs(blum_ctx* ctx, const float* logits, int64_t rows, int64_t cols, int index_offset, int32_t* pairs) {
    BLUM_REQUIRE(ctx, logits && pairs && rows > 0 && cols > 0, "argmax_pairs: bad argument");
    argmax_pairs_kernel<<<(unsigned)rows, 1024, 0, ctx->stream>>>(logits, cols, index_offset, pairs);
    BLUM_LAUNCH_CHECK(ctx);
    return BLUM_OK;
}
int blum_pick_pairs(blum_ctx* ctx, const int32_t* pairs, int nranks, int64_t rows, int32_t* out_idx) {
    BLUM_REQUIRE(ctx, pairs && out_idx && nranks > 0 && rows > 0, "pick_pairs: bad argument");
    pick_pairs_kernel<<<(unsigned)((rows + 127) / 128), 128, 0, ctx->stream>>>(pairs, nranks, rows, out_idx);
    BLUM_LAUNCH_CHECK(ctx);
    return BLUM_OK;
}

static inline unsigned grid_for(const blum_ctx* ctx, int64_t work_items, int block) {
    int64_t g = (work_items + block - 1) / block;
    const int64_t cap = (int64_t)ctx->sm_count * 8;
    if (g > cap) g = cap;
    if (g < 1) g = 1;
    return (unsigned)g;
}

extern "C" {

int blum_gather(blum_ctx* ctx, const void* table, blum_dtype tdt, int64_t rows, int64_t dim, const int32_t* ids,
                int64_t T, void* out, blum_dtype odt) {
    if (!ctx) return BLUM_ERR_INVALID;
    BLUM_REQUIRE(ctx, table && ids && out && rows > 0 && dim > 0 && T >= 0, "gather: bad argument");
    if (T == 0) return BLUM_OK;
    BLUM_DISPATCH_DTYPE(tdt, TI, BLUM_DISPATCH_DTYPE(odt, TO,
        (gather_rows_kernel<TI, TO><<<(unsigned)T, 256, 0, ctx->stream>>>((const TI*)table, rows, dim, ids, T, (TO*)out, ctx->dev_error))));
    BLUM_LAUNCH_CHECK(ctx);
    return BLUM_OK;
}

int blum_q8_0_gather(blum_ctx* ctx, const blum_q8_weight* w, const int32_t* ids, int64_t T, void* out, blum_dtype odt) {
    if (!ctx) return BLUM_ERR_INVALID;
    BLUM_REQUIRE(ctx, w && ids && out && T >= 0, "q8 gather: bad argument");
    if (T == 0) return BLUM_OK;
    BLUM_DISPATCH_DTYPE(odt, TO,
        (q8_gather_kernel<TO><<<(unsigned)T, 256, 0, ctx->stream>>>(w->q, w->d, w->N, w->K, ids, (TO*)out, ctx->dev_error)));
    BLUM_LAUNCH_CHECK(ctx);
    return BLUM_OK;
}

int blum_rmsnorm(blum_ctx* ctx, const void* x, const void* residual, const float* weight, float eps, void* y,
                 void* sum_out, blum_dtype dt, int64_t rows, int64_t dim) {
    if (!ctx) return BLUM_ERR_INVALID;
    BLUM_REQUIRE(ctx, x && y && rows >= 0 && dim > 0, "rmsnorm: bad argument");
    const int N = 16 / (int)blum_dtype_size(dt);
    BLUM_REQUIRE(ctx, dim % N == 0, "rmsnorm: dim %lld must be a multiple of %d", (long long)dim, N);
    BLUM_REQUIRE(ctx, dim <= (int64_t)256 * N * 8, "rmsnorm: dim %lld too large", (long long)dim);
    if (rows == 0) return BLUM_OK;
    const int vpt = (int)((dim / N + 255) / 256);
    BLUM_DISPATCH_DTYPE(dt, T, {
        if (vpt <= 1) rmsnorm_kernel<T, 1><<<(unsigned)rows, 256, 0, ctx->stream>>>((const T*)x, (const T*)residual, weight, eps, (T*)y, (T*)sum_out, dim);
        else if (vpt <= 2) rmsnorm_kernel<T, 2><<<(unsigned)rows, 256, 0, ctx->stream>>>((const T*)x, (const T*)residual, weight, eps, (T*)y, (T*)sum_out, dim);
        else if (vpt <= 4) rmsnorm_kernel<T, 4><<<(unsigned)rows, 256, 0, ctx->stream>>>((const T*)x, (const T*)residual, weight, eps, (T*)y, (T*)sum_out, dim);
        else rmsnorm_kernel<T, 8><<<(unsigned)rows, 256, 0, ctx->stream>>>((const T*)x, (const T*)residual, weight, eps, (T*)y, (T*)sum_out, dim);
    });
    BLUM_LAUNCH_CHECK(ctx);
    return BLUM_OK;
}

int blum_rope_interleaved(blum_ctx* ctx, void* x, blum_dtype dt, const int32_t* positions, int64_t T, int heads,
                          int head_dim, float theta) {
    if (!ctx) return BLUM_ERR_INVALID;
    BLUM_REQUIRE(ctx, x && positions && T >= 0 && heads > 0, "rope: bad argument");
    BLUM_REQUIRE(ctx, head_dim > 0 && head_dim % 2 == 0 && head_dim <= 256, "rope: head_dim must be even and <= 256");
    if (T == 0) return BLUM_OK;
    RopeFreqs f;
    blum_rope_freqs(theta, head_dim, &f);
    const int64_t total = T * heads * (head_dim / 2);
    BLUM_DISPATCH_DTYPE(dt, TT, (rope_kernel<TT><<<grid_for(ctx, total, 256), 256, 0, ctx->stream>>>((TT*)x, positions, T, heads, head_dim, f)));
    BLUM_LAUNCH_CHECK(ctx);
    return BLUM_OK;
}

int blum_qk_norm_rope(blum_ctx* ctx, void* qkv, blum_dtype dt, const int32_t* positions, int64_t T, int q_heads, int kv_heads,
                      int head_dim, const float* q_norm_w, const float* k_norm_w, float eps, float theta, int rope_mode) {
    if (!ctx) return BLUM_ERR_INVALID;
    BLUM_REQUIRE(ctx, qkv && positions && T >= 0 && q_heads > 0 && kv_heads > 0, "qk_norm_rope: bad argument");
    BLUM_REQUIRE(ctx, head_dim > 0 && head_dim % 2 == 0 && head_dim <= 256, "qk_norm_rope: head_dim %d not supported", head_dim);
    BLUM_REQUIRE(ctx, rope_mode == 0 || rope_mode == 1, "qk_norm_rope: rope_mode must be 0 (interleaved) or 1 (half-split)");
    BLUM_REQUIRE(ctx, (q_norm_w == nullptr) == (k_norm_w == nullptr), "qk_norm_rope: give both norm weights or neither");
    if (T == 0) return BLUM_OK;
    RopeFreqs f;
    blum_rope_freqs(theta, head_dim, &f);
    const int64_t warps = T * (q_heads + kv_heads);
    BLUM_DISPATCH_DTYPE(dt, TT, (qk_norm_rope_kernel<TT><<<grid_for(ctx, warps * 32, 256), 256, 0, ctx->stream>>>(
        (TT*)qkv, positions, T, q_heads, kv_heads, head_dim, q_norm_w, k_norm_w, eps, f, rope_mode)));
    BLUM_LAUNCH_CHECK(ctx);
    return BLUM_OK;
}

int blum_swiglu(blum_ctx* ctx, const void* gate, const void* up, void* out, blum_dtype dt, int64_t n) {
    if (!ctx) return BLUM_ERR_INVALID;
    BLUM_REQUIRE(ctx, gate && up && out && n >= 0, "swiglu: bad argument");
    if (n == 0) return BLUM_OK;
    BLUM_DISPATCH_DTYPE(dt, T, (swiglu_kernel<T><<<grid_for(ctx, n / 4 + 1, 256), 256, 0, ctx->stream>>>((const T*)gate, (const T*)up, (T*)out, n)));
    BLUM_LAUNCH_CHECK(ctx);
    return BLUM_OK;
}

}  // extern "C"
int blum_swiglu_rows(blum_ctx* ctx, const void* gate_up, void* out, int dt, int64_t R, int64_t F) {
    BLUM_REQUIRE(ctx, gate_up && out && R >= 0 && F > 0 && F % 8 == 0, "swiglu rows: bad argument");
    if (R == 0) return BLUM_OK;
    BLUM_DISPATCH_DTYPE(dt, T, (swiglu_rows_kernel<T><<<grid_for(ctx, R * F / 4 + 1, 256), 256, 0, ctx->stream>>>((const T*)gate_up, (T*)out, R, F)));
    BLUM_LAUNCH_CHECK(ctx);
    return BLUM_OK;
}
extern "C" {

int blum_add(blum_ctx* ctx, const void* a, const void* b, void* out, blum_dtype dt, int64_t n) {
    if (!ctx) return BLUM_ERR_INVALID;
    BLUM_REQUIRE(ctx, a && b && out && n >= 0, "add: bad argument");
    if (n == 0) return BLUM_OK;
    BLUM_DISPATCH_DTYPE(dt, T, (add_kernel<T><<<grid_for(ctx, n / 4 + 1, 256), 256, 0, ctx->stream>>>((const T*)a, (const T*)b, (T*)out, n)));
    BLUM_LAUNCH_CHECK(ctx);
    return BLUM_OK;
}

int blum_softmax(blum_ctx* ctx, const void* x, void* y, blum_dtype dt, int64_t rows, int64_t cols) {
    if (!ctx) return BLUM_ERR_INVALID;
    BLUM_REQUIRE(ctx, x && y && rows >= 0 && cols > 0, "softmax: bad argument");
    if (rows == 0) return BLUM_OK;
    BLUM_DISPATCH_DTYPE(dt, T, (softmax_kernel<T><<<(unsigned)rows, 256, 0, ctx->stream>>>((const T*)x, (T*)y, cols)));
    BLUM_LAUNCH_CHECK(ctx);
    return BLUM_OK;
}

int blum_argmax(blum_ctx* ctx, const void* logits, blum_dtype dt, int64_t rows, int64_t cols, int32_t* out_idx) {
    if (!ctx) return BLUM_ERR_INVALID;
    BLUM_REQUIRE(ctx, logits && out_idx && rows >= 0 && cols > 0 && cols < (1ll << 31), "argmax: bad argument");
    if (rows == 0) return BLUM_OK;
    if (dt == BLUM_F32 && cols >= 8192 && rows <= BLUM_ARGMAX_ROWS && rows < 4 * (int64_t)ctx->sm_count) {
        int splits = (int)((4 * (int64_t)ctx->sm_count + rows - 1) / rows);
        splits = (int)std::min<int64_t>(splits, cols / 4096);
        argmax_split_kernel<<<(unsigned)(rows * splits), 512, 0, ctx->stream>>>((const float*)logits, cols, splits, (ArgmaxRec*)ctx->argmax_ws, out_idx);
        BLUM_LAUNCH_CHECK(ctx);
        return BLUM_OK;
    }
    BLUM_DISPATCH_DTYPE(dt, T, (argmax_kernel<T><<<(unsigned)rows, 1024, 0, ctx->stream>>>((const T*)logits, cols, out_idx)));
    BLUM_LAUNCH_CHECK(ctx);
    return BLUM_OK;
}

}  // extern "C"
