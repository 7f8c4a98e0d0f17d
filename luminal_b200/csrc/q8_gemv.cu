// Q8_0 GEMV family: y[M,N] = x[M,K] * W^T for small M (decode), bound by HBM bandwidth.
//
// Stands in for the matvec kernel of QuantizedMatmul (crates/luminal_cuda/src/quantized.rs:28-109
// in luminal), which reads 34-byte blocks with byte loads and re-streams W once per row of x.
// Here W is the two-plane layout of q8_weight.cu and is streamed exactly once for up to
// GEMV_MAX_MT rows of x:
//   * a CTA stages its rows of x in shared memory as f32 (optionally folding the RMSNorm weight
//     in and computing rsqrt(mean(x^2)+eps) on the fly);
//   * each warp owns R consecutive rows of W at a time; every lane issues one 128-bit streaming
//     load per row per 512-element chunk (U chunks in flight), so a warp reads 512 contiguous
//     bytes per row per chunk;
//   * int8 -> f32 conversion and FMA in f32 (same arithmetic as the reference:
//     sum_block(q * x) * d, f32 accumulate), one warp-shuffle reduction per row at the end;
//   * row groups are dealt round-robin over (CTA, warp) so that every SM pulls the same share.
// Algorithmic bytes per launch: N*K*34/32 (weights) + M*K*sizeof(x) + M*N*sizeof(y).
#include "common.cuh"

#define GEMV_MAX_MT 4

struct GemvF32Params {
    const int8_t* q;  const __half* d;     // weight (gate weight in SwiGLU mode)
    const int8_t* q2; const __half* d2;    // up weight in SwiGLU mode, else null
    const void* x;    void* y;
    const void* residual;                  // y's dtype and shape, or null
    const float* norm_w;                   // f32 [K] or null
    float eps;
    int N, K;
    int m0, mt, M;                         // rows [m0, m0+mt) of x are handled by this launch
};

__device__ __forceinline__ float dot16(const int4& v, const float* xv) {
    const int w[4] = {v.x, v.y, v.z, v.w};
    float s = 0.f;
#pragma unroll
    for (int j = 0; j < 4; j++) {
#pragma unroll
        for (int b = 0; b < 4; b++) {
            const int qv = (int)(signed char)((unsigned)w[j] >> (8 * b));
            s = fmaf((float)qv, xv[4 * j + b], s);
        }
    }
    return s;
}

// Shared-memory slot of x[k..k+4) (k % 4 == 0).  Within each 512-element chunk the four float4
// pieces of a lane's 16 values are stored 32 float4 apart, so that lane l reading piece j touches
// float4 (j*32 + l): consecutive lanes, no bank conflicts.
__device__ __forceinline__ int xs_slot(int k) {
    return (k & ~511) + ((((k & 15) >> 2) * 32 + ((k & 511) >> 4)) << 2);
}

template <typename TX>
__device__ __forceinline__ void load4_f32(const TX* p, float* o);
template <> __device__ __forceinline__ void load4_f32<float>(const float* p, float* o) {
    const float4 v = *reinterpret_cast<const float4*>(p);
    o[0] = v.x; o[1] = v.y; o[2] = v.z; o[3] = v.w;
}
template <> __device__ __forceinline__ void load4_f32<__half>(const __half* p, float* o) {
    const uint2 v = *reinterpret_cast<const uint2*>(p);
    const __half2 a = *reinterpret_cast<const __half2*>(&v.x), b = *reinterpret_cast<const __half2*>(&v.y);
    o[0] = __low2float(a); o[1] = __high2float(a); o[2] = __low2float(b); o[3] = __high2float(b);
}
template <> __device__ __forceinline__ void load4_f32<__nv_bfloat16>(const __nv_bfloat16* p, float* o) {
    const uint2 v = *reinterpret_cast<const uint2*>(p);
    o[0] = __uint_as_float(v.x << 16); o[1] = __uint_as_float(v.x & 0xffff0000u);
    o[2] = __uint_as_float(v.y << 16); o[3] = __uint_as_float(v.y & 0xffff0000u);
}

// MT rows of x, R rows of W per warp pass, U chunks in flight.  SWIGLU: rows come in (gate, up) pairs.
template <typename TX, typename TY, int MT, int R, int U, bool SWIGLU>
__global__ void __launch_bounds__(256) q8_gemv_kernel(const GemvF32Params p) {
    extern __shared__ __align__(16) float xs[];   // [MT][KP]
    __shared__ float red[MT][8];
    __shared__ float rs_sh[MT];

    const int K = p.K, N = p.N, KP = (p.K + 511) & ~511;   // KP: padded row stride of xs
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, nwarps = blockDim.x >> 5;

    // ---- stage x (f32), fold the norm weight, sum of squares per row
    const TX* xg = reinterpret_cast<const TX*>(p.x) + (size_t)p.m0 * K;
    float ss[MT];
#pragma unroll
    for (int m = 0; m < MT; m++) ss[m] = 0.f;
    for (int k = tid * 4; k < K; k += blockDim.x * 4) {
        float nw[4] = {1.f, 1.f, 1.f, 1.f};
        if (p.norm_w) load4_f32<float>(p.norm_w + k, nw);
#pragma unroll
        for (int m = 0; m < MT; m++) {
            float v[4];
            load4_f32<TX>(xg + (size_t)m * K + k, v);
            ss[m] += v[0] * v[0] + v[1] * v[1] + v[2] * v[2] + v[3] * v[3];
            *reinterpret_cast<float4*>(xs + m * KP + xs_slot(k)) = make_float4(v[0] * nw[0], v[1] * nw[1], v[2] * nw[2], v[3] * nw[3]);
        }
    }
    if (p.norm_w) {
#pragma unroll
        for (int m = 0; m < MT; m++) {
            const float s = warp_sum(ss[m]);
            if (lane == 0) red[m][warp] = s;
        }
    }
    __syncthreads();
    if (p.norm_w) {
        if (tid < MT) {
            float s = 0.f;
            for (int w = 0; w < nwarps; w++) s += red[tid][w];
            rs_sh[tid] = rsqrtf(s / (float)K + p.eps);
        }
        __syncthreads();
    }

    // ---- stream W
    const int kb_per_row = K >> 5;
    const int groups = (N + R - 1) / R;
    for (int g = blockIdx.x + gridDim.x * warp; g < groups; g += gridDim.x * nwarps) {
        const int row0 = g * R;
        float acc[R][MT], acc2[SWIGLU ? R : 1][MT];
#pragma unroll
        for (int r = 0; r < R; r++)
#pragma unroll
            for (int m = 0; m < MT; m++) { acc[r][m] = 0.f; if (SWIGLU) acc2[r][m] = 0.f; }

        const int8_t* qrow[R];
        const __half* drow[R];
#pragma unroll
        for (int r = 0; r < R; r++) {
            const int row = min(row0 + r, N - 1);
            qrow[r] = p.q + (size_t)row * K;
            drow[r] = p.d + (size_t)row * kb_per_row;
        }
        const size_t off2_q = SWIGLU ? (size_t)(p.q2 - p.q) : 0;
        const size_t off2_d = SWIGLU ? (size_t)(p.d2 - p.d) : 0;

        for (int kbase = lane * 16; kbase < K; kbase += 512 * U) {
            int4 wq[U][R], wq2[SWIGLU ? U : 1][SWIGLU ? R : 1];
            __half ws[U][R], ws2[SWIGLU ? U : 1][SWIGLU ? R : 1];
#pragma unroll
            for (int u = 0; u < U; u++) {
                const int k = kbase + u * 512;
                if (k < K) {
#pragma unroll
                    for (int r = 0; r < R; r++) {
                        wq[u][r] = ld_stream_16(qrow[r] + k);
                        ws[u][r] = __ldg(drow[r] + (k >> 5));
                        if (SWIGLU) {
                            wq2[u][r] = ld_stream_16(qrow[r] + off2_q + k);
                            ws2[u][r] = __ldg(drow[r] + off2_d + (k >> 5));
                        }
                    }
                }
            }
#pragma unroll
            for (int u = 0; u < U; u++) {
                const int k = kbase + u * 512;
                if (k < K) {
#pragma unroll
                    for (int m = 0; m < MT; m++) {
                        float xv[16];
#pragma unroll
                        for (int j = 0; j < 4; j++) {
                            const float4 t = *reinterpret_cast<const float4*>(xs + m * KP + (k & ~511) + (j * 32 + lane) * 4);
                            xv[4 * j] = t.x; xv[4 * j + 1] = t.y; xv[4 * j + 2] = t.z; xv[4 * j + 3] = t.w;
                        }
#pragma unroll
                        for (int r = 0; r < R; r++) {
                            acc[r][m] = fmaf(dot16(wq[u][r], xv), __half2float(ws[u][r]), acc[r][m]);
                            if (SWIGLU) acc2[r][m] = fmaf(dot16(wq2[u][r], xv), __half2float(ws2[u][r]), acc2[r][m]);
                        }
                    }
                }
            }
        }

        // ---- reduce across the warp, epilogue
#pragma unroll
        for (int r = 0; r < R; r++) {
#pragma unroll
            for (int m = 0; m < MT; m++) {
                float s = warp_sum(acc[r][m]);
                float s2 = SWIGLU ? warp_sum(acc2[r][m]) : 0.f;
                const int row = row0 + r;
                if (lane == 0 && row < N) {
                    if (p.norm_w) { s *= rs_sh[m]; s2 *= rs_sh[m]; }
                    if (SWIGLU) {
                        // up * (gate * 1/(1+exp(-gate)))
                        s = s2 * (s * (1.f / (1.f + __expf(-s))));
                    }
                    const size_t o = (size_t)(p.m0 + m) * N + row;
                    if (p.residual) s += to_f32<TY>(reinterpret_cast<const TY*>(p.residual)[o]);
                    reinterpret_cast<TY*>(p.y)[o] = from_f32<TY>(s);
                }
            }
        }
    }
}

// launch shape of the float form: rows per warp, 32-block steps in flight per lane, warps per CTA, CTAs per SM
struct GemvVariant { int R, U, warps, ctas_per_sm; };
static const GemvVariant kGemvShape = {2, 2, 8, 2};

template <typename TX, typename TY, int MT, int R, int U, bool SWIGLU>
static int launch_one(blum_ctx* ctx, const GemvF32Params& p, int warps, int ctas_per_sm) {
    auto kern = q8_gemv_kernel<TX, TY, MT, R, U, SWIGLU>;
    const size_t smem = (size_t)MT * ((p.K + 511) & ~511) * sizeof(float);
    BLUM_REQUIRE(ctx, smem + 1024 <= ctx->smem_optin, "q8 gemv: K=%d with %d rows of x needs %zu B of shared memory", p.K, MT, smem);
    if (smem + 2048 > 48 * 1024) BLUM_CUDA(ctx, cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    const int groups = (p.N + R - 1) / R;
    int grid = ctx->sm_count * ctas_per_sm;
    const int need = (groups + warps - 1) / warps;
    if (grid > need) grid = need;
    if (grid < 1) grid = 1;
    kern<<<grid, warps * 32, smem, ctx->stream>>>(p);
    BLUM_LAUNCH_CHECK(ctx);
    return BLUM_OK;
}

template <typename TX, typename TY, int MT, bool SWIGLU>
static int launch_ru(blum_ctx* ctx, const GemvF32Params& p, const GemvVariant& v) {
    if constexpr (SWIGLU) return launch_one<TX, TY, MT, 1, 2, true>(ctx, p, v.warps, v.ctas_per_sm);
    else return launch_one<TX, TY, MT, 2, 2, false>(ctx, p, v.warps, v.ctas_per_sm);
}

template <typename TX, typename TY, bool SWIGLU>
static int launch_mt(blum_ctx* ctx, GemvF32Params p, const GemvVariant& v) {
    // rows of x in chunks of up to GEMV_MAX_MT; W is re-read once per chunk
    // as many rows of x per pass as fit in shared memory as f32
    int max_mt = (int)((ctx->smem_optin - 2048) / ((size_t)((p.K + 511) & ~511) * sizeof(float)));
    if (max_mt > GEMV_MAX_MT) max_mt = GEMV_MAX_MT;
    BLUM_REQUIRE(ctx, max_mt >= 1, "q8 gemv: K=%d does not fit in shared memory", p.K);
    for (int m0 = 0; m0 < p.M; m0 += max_mt) {
        p.m0 = m0;
        p.mt = (p.M - m0 < max_mt) ? p.M - m0 : max_mt;
        int rc;
        switch (p.mt) {
            case 1: rc = launch_ru<TX, TY, 1, SWIGLU>(ctx, p, v); break;
            case 2: rc = launch_ru<TX, TY, 2, SWIGLU>(ctx, p, v); break;
            case 3: rc = launch_ru<TX, TY, 3, SWIGLU>(ctx, p, v); break;
            default: rc = launch_ru<TX, TY, 4, SWIGLU>(ctx, p, v); break;
        }
        if (rc) return rc;
    }
    return BLUM_OK;
}

template <bool SWIGLU>
static int launch_types(blum_ctx* ctx, const GemvF32Params& p, int xdt, int ydt, const GemvVariant& v) {
#define TT(xd, yd, TX, TY) if (xdt == xd && ydt == yd) return launch_mt<TX, TY, SWIGLU>(ctx, p, v)
    TT(BLUM_F32, BLUM_F32, float, float);
    TT(BLUM_BF16, BLUM_BF16, __nv_bfloat16, __nv_bfloat16);
    TT(BLUM_F16, BLUM_F16, __half, __half);
    TT(BLUM_BF16, BLUM_F32, __nv_bfloat16, float);
    TT(BLUM_F16, BLUM_F32, __half, float);
#undef TT
    return blum_fail(ctx, BLUM_ERR_INVALID, "q8 gemv: unsupported dtype pair (%d,%d)", xdt, ydt);
}

// integer-dot-product form (q8_gemv_i8.cu)
bool blum_gemv_i8_supported(int xdt, int ydt);
int blum_gemv_i8_dispatch(blum_ctx* ctx, const blum_q8_weight* w, const blum_q8_weight* w_up, const void* x, int xdt,
                          const float* norm_w, float eps, const void* residual, void* y, int ydt, int64_t M);

// M <= 2 with a supported dtype pair takes the integer-dot-product kernel, everything else the float form
int blum_gemv_dispatch(blum_ctx* ctx, const blum_q8_weight* w, const blum_q8_weight* w_up, const void* x, int xdt,
                       const float* norm_w, float eps, const void* residual, void* y, int ydt, int64_t M) {
    if (M <= 2 && blum_gemv_i8_supported(xdt, ydt))
        return blum_gemv_i8_dispatch(ctx, w, w_up, x, xdt, norm_w, eps, residual, y, ydt, M);
    BLUM_REQUIRE(ctx, w && x && y, "q8 matmul: null argument");
    BLUM_REQUIRE(ctx, M >= 1, "q8 matmul: M must be >= 1 (got %lld)", (long long)M);
    BLUM_REQUIRE(ctx, xdt >= 0 && xdt <= 2 && ydt >= 0 && ydt <= 2, "q8 matmul: bad dtype");
    BLUM_REQUIRE(ctx, w->N < (1ll << 31) && w->K < (1ll << 31), "q8 matmul: dimension too large");
    BLUM_REQUIRE(ctx, ((uintptr_t)x % 16) == 0 && ((uintptr_t)y % 4) == 0, "q8 matmul: x must be 16-byte aligned");
    if (w_up) BLUM_REQUIRE(ctx, w_up->N == w->N && w_up->K == w->K, "q8 swiglu: gate and up weights differ in shape");
    GemvF32Params p;
    p.q = w->q; p.d = w->d;
    p.q2 = w_up ? w_up->q : nullptr; p.d2 = w_up ? w_up->d : nullptr;
    p.x = x; p.y = y; p.residual = residual; p.norm_w = norm_w; p.eps = eps;
    p.N = (int)w->N; p.K = (int)w->K; p.M = (int)M; p.m0 = 0; p.mt = 1;
    if (w_up) return launch_types<true>(ctx, p, xdt, ydt, kGemvShape);
    return launch_types<false>(ctx, p, xdt, ydt, kGemvShape);
}
