// Q8_0 GEMV, integer-dot-product form (M <= 2): the decode kernel.
//
// Same job as q8_gemv.cu (y = x * W^T for the reference's QuantizedMatmul,
// crates/luminal_cuda/src/quantized.rs:28-109 in luminal), built so that the SM's instruction issue rate
// is not what limits an HBM-bound stream:
//   * x is staged once per CTA as block fixed point: for every 32-element block (the Q8_0 block)
//     x_i = xfix_i * 2^(e-21) with |xfix_i| <= 2^22, e the exponent of the block's largest |x_i|;
//     xfix is split into three byte planes (xfix = a*65536 + b*256 + c, a signed, b and c unsigned).
//     The rounding error of x is at most 2^-22 of the block maximum, i.e. f32-grade.
//   * sum_i q_i * xfix_i is then EXACT integer arithmetic: three dp4a per four weights straight on the
//     packed int8 words (no per-weight int->float conversion, no byte extraction);
//   * per (row, block): f = 65536*A + 256*B + C, acc += f * (d * 2^(e-21)) in f32 - the same
//     "block sum times block scale" order as the reference kernel (quantized.rs:88-97);
//   * a lane owns one whole block per step and reads it with one 256-bit streaming load, so a warp
//     reads 1 KiB contiguous per row per step; R rows x U steps are in flight per lane.
// Algorithmic bytes per launch: N*K*34/32 + M*K*sizeof(x) + M*N*sizeof(y).
#include "common.cuh"

struct GemvI8Params {
    const int8_t* q;  const __half* d;
    const int8_t* q2; const __half* d2;
    const void* x;    void* y;
    const void* residual;
    const float* norm_w;
    float eps;
    int N, K;
    int m0, mt, M;
    unsigned long long* trace;
};

struct W256 { int v[8]; };

__device__ __forceinline__ W256 ld_stream_32(const void* p) {
    W256 r;
    asm volatile("ld.global.nc.L1::no_allocate.L2::128B.v8.s32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
                 : "=r"(r.v[0]), "=r"(r.v[1]), "=r"(r.v[2]), "=r"(r.v[3]), "=r"(r.v[4]), "=r"(r.v[5]), "=r"(r.v[6]), "=r"(r.v[7])
                 : "l"(p));
    return r;
}
__device__ __forceinline__ int dp4a_ss(int a, int b, int c) {
    int d; asm("dp4a.s32.s32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c)); return d;
}
__device__ __forceinline__ int dp4a_su(int a, int b, int c) {
    int d; asm("dp4a.s32.u32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c)); return d;
}

template <typename TX> __device__ __forceinline__ void ld4(const TX* p, float* o);
template <> __device__ __forceinline__ void ld4<float>(const float* p, float* o) {
    const float4 v = *reinterpret_cast<const float4*>(p);
    o[0] = v.x; o[1] = v.y; o[2] = v.z; o[3] = v.w;
}
template <> __device__ __forceinline__ void ld4<__half>(const __half* p, float* o) {
    const uint2 v = *reinterpret_cast<const uint2*>(p);
    const __half2 a = *reinterpret_cast<const __half2*>(&v.x), b = *reinterpret_cast<const __half2*>(&v.y);
    o[0] = __low2float(a); o[1] = __high2float(a); o[2] = __low2float(b); o[3] = __high2float(b);
}
template <> __device__ __forceinline__ void ld4<__nv_bfloat16>(const __nv_bfloat16* p, float* o) {
    const uint2 v = *reinterpret_cast<const uint2*>(p);
    o[0] = __uint_as_float(v.x << 16); o[1] = __uint_as_float(v.x & 0xffff0000u);
    o[2] = __uint_as_float(v.y << 16); o[3] = __uint_as_float(v.y & 0xffff0000u);
}

// Shared-memory layout of one row of x: per 1024-element step `it`, plane p (0..2), half j (0..1):
// 32 lanes x 16 bytes, so that lane l reading piece (p, j) touches consecutive 16-byte slots.
__device__ __forceinline__ int limb_offset(int k, int plane) {
    const int it = k >> 10, lane = (k & 1023) >> 5, o = k & 31;
    return ((it * 3 + plane) * 2 + (o >> 4)) * 512 + lane * 16 + (o & 15);
}

template <typename TX, typename TY, int MT, int R, int U, int THREADS, bool SWIGLU>
__global__ void __launch_bounds__(THREADS) q8_gemv_i8_kernel(const GemvI8Params p) {
    extern __shared__ __align__(16) unsigned char smem[];
    __shared__ float red[MT][THREADS / 32];
    __shared__ float rs_sh[MT];

    const int K = p.K, N = p.N;
    const int NIT = (K + 1023) >> 10;                 // 1024-element steps per row
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    constexpr int NW = THREADS / 32;
    unsigned char* limbs = smem;                      // [MT][NIT * 3072]
    float* xscale = reinterpret_cast<float*>(smem + (size_t)MT * NIT * 3072);   // [MT][NIT * 32]

    // ---- before touching x (which the previous kernel may still be writing): let the next kernel start its
    // own prologue, and pull this warp's first rows towards L2 so the stream is already moving
    blum_trace(p.trace, 0);
    pdl_launch_dependents();
    // The first step of this warp's first row group is loaded into registers right away: the weights do not depend on
    // the previous kernel, so the HBM latency of the first loads overlaps the wait and the staging of x.
    const int KB = K >> 5;
    W256 wq[U][R], wq2[SWIGLU ? U : 1][SWIGLU ? R : 1];
    float ws[U][R], ws2[SWIGLU ? U : 1][SWIGLU ? R : 1];
    bool preloaded = false;
    {
        const int g0 = blockIdx.x + gridDim.x * warp;
        if (g0 * R < N) {
            preloaded = true;
#pragma unroll
            for (int u = 0; u < U; u++) {
                const int kb = u * 32 + lane;
                if (kb < KB) {
#pragma unroll
                    for (int r = 0; r < R; r++) {
                        const int row = min(g0 * R + r, N - 1);
                        wq[u][r] = ld_stream_32(p.q + (size_t)row * K + (size_t)kb * 32);
                        ws[u][r] = __half2float(__ldg(p.d + (size_t)row * KB + kb));
                        if (SWIGLU) {
                            wq2[u][r] = ld_stream_32(p.q2 + (size_t)row * K + (size_t)kb * 32);
                            ws2[u][r] = __half2float(__ldg(p.d2 + (size_t)row * KB + kb));
                        }
                    }
                }
            }
            const int lines = min(K >> 7, 64);                 // 128-byte lines per row, at most 8 KiB per row
#pragma unroll
            for (int r = 0; r < R; r++) {
                const int row = min(g0 * R + r, N - 1);
                for (int l = lane; l < lines; l += 32) {
                    asm volatile("prefetch.global.L2 [%0];" ::"l"(p.q + (size_t)row * K + (size_t)l * 128));
                    if (SWIGLU) asm volatile("prefetch.global.L2 [%0];" ::"l"(p.q2 + (size_t)row * K + (size_t)l * 128));
                }
            }
        }
    }
    pdl_wait();
    blum_trace(p.trace, 1);

    // ---- stage x: fold the norm weight, block maximum, fixed point, three byte planes
    const TX* xg = reinterpret_cast<const TX*>(p.x) + (size_t)p.m0 * K;
    float ss[MT];
#pragma unroll
    for (int m = 0; m < MT; m++) ss[m] = 0.f;
    const int KP = NIT << 10;
    for (int k = tid * 4; k < KP; k += THREADS * 4) {
        float nw[4] = {1.f, 1.f, 1.f, 1.f};
        if (p.norm_w && k < K) ld4<float>(p.norm_w + k, nw);
#pragma unroll
        for (int m = 0; m < MT; m++) {
            float v[4] = {0.f, 0.f, 0.f, 0.f};
            if (k < K) ld4<TX>(xg + (size_t)m * K + k, v);
            ss[m] += v[0] * v[0] + v[1] * v[1] + v[2] * v[2] + v[3] * v[3];
#pragma unroll
            for (int i = 0; i < 4; i++) v[i] *= nw[i];
            float mx = fmaxf(fmaxf(fabsf(v[0]), fabsf(v[1])), fmaxf(fabsf(v[2]), fabsf(v[3])));
            mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
            mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
            mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 4));     // 8 lanes x 4 = one 32-element block
            const int E = (int)((__float_as_uint(mx) >> 23) & 0xffu);
            // xfix = x * 2^(21 - (E-127)); blocks whose maximum is below 2^-105 are treated as zero
            const float up = (E >= 22 && E < 255) ? __uint_as_float((unsigned)(275 - E) << 23) : 0.f;
            const float down = (E == 255) ? __uint_as_float(0x7fc00000u) : (E >= 22 ? __uint_as_float((unsigned)(E - 21) << 23) : 0.f);
            unsigned pa = 0, pb = 0, pc = 0;
#pragma unroll
            for (int i = 0; i < 4; i++) {
                const int xf = __float2int_rn(v[i] * up);
                pa |= ((unsigned)(xf >> 16) & 0xffu) << (8 * i);
                pb |= ((unsigned)(xf >> 8) & 0xffu) << (8 * i);
                pc |= ((unsigned)xf & 0xffu) << (8 * i);
            }
            unsigned char* base = limbs + (size_t)m * NIT * 3072;
            *reinterpret_cast<unsigned*>(base + limb_offset(k, 0)) = pa;
            *reinterpret_cast<unsigned*>(base + limb_offset(k, 1)) = pb;
            *reinterpret_cast<unsigned*>(base + limb_offset(k, 2)) = pc;
            if ((k & 31) == 0) xscale[m * NIT * 32 + (k >> 5)] = down;
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
            for (int w = 0; w < NW; w++) s += red[tid][w];
            rs_sh[tid] = rsqrtf(s / (float)K + p.eps);
        }
        __syncthreads();
    }

    blum_trace(p.trace, 2);
    // ---- stream W
    const int groups = (N + R - 1) / R;
    for (int g = blockIdx.x + gridDim.x * warp; g < groups; g += gridDim.x * NW) {
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
            drow[r] = p.d + (size_t)row * KB;
        }
        const ptrdiff_t off2_q = SWIGLU ? (p.q2 - p.q) : 0;
        const ptrdiff_t off2_d = SWIGLU ? (p.d2 - p.d) : 0;

        for (int it0 = 0; it0 < NIT; it0 += U) {
            const bool skip_loads = preloaded;       // true only for the very first step of the first group
            preloaded = false;
#pragma unroll
            for (int u = 0; u < U; u++) {
                const int kb = (it0 + u) * 32 + lane;
                if (kb < KB && !skip_loads) {
#pragma unroll
                    for (int r = 0; r < R; r++) {
                        wq[u][r] = ld_stream_32(qrow[r] + (size_t)kb * 32);
                        ws[u][r] = __half2float(__ldg(drow[r] + kb));
                        if (SWIGLU) {
                            wq2[u][r] = ld_stream_32(qrow[r] + off2_q + (size_t)kb * 32);
                            ws2[u][r] = __half2float(__ldg(drow[r] + off2_d + kb));
                        }
                    }
                }
            }
#pragma unroll
            for (int u = 0; u < U; u++) {
                const int it = it0 + u;
                const int kb = it * 32 + lane;
                if (kb < KB) {
#pragma unroll
                    for (int m = 0; m < MT; m++) {
                        const unsigned char* base = limbs + (size_t)m * NIT * 3072 + (size_t)it * 3072 + lane * 16;
                        int xa[8], xb[8], xc[8];
#pragma unroll
                        for (int j = 0; j < 2; j++) {
                            const int4 ta = *reinterpret_cast<const int4*>(base + (0 * 2 + j) * 512);
                            const int4 tb = *reinterpret_cast<const int4*>(base + (1 * 2 + j) * 512);
                            const int4 tc = *reinterpret_cast<const int4*>(base + (2 * 2 + j) * 512);
                            xa[4 * j] = ta.x; xa[4 * j + 1] = ta.y; xa[4 * j + 2] = ta.z; xa[4 * j + 3] = ta.w;
                            xb[4 * j] = tb.x; xb[4 * j + 1] = tb.y; xb[4 * j + 2] = tb.z; xb[4 * j + 3] = tb.w;
                            xc[4 * j] = tc.x; xc[4 * j + 1] = tc.y; xc[4 * j + 2] = tc.z; xc[4 * j + 3] = tc.w;
                        }
                        const float xs = xscale[m * NIT * 32 + kb];
#pragma unroll
                        for (int r = 0; r < R; r++) {
                            int A = 0, B = 0, C = 0;
#pragma unroll
                            for (int i = 0; i < 8; i++) {
                                A = dp4a_ss(wq[u][r].v[i], xa[i], A);
                                B = dp4a_su(wq[u][r].v[i], xb[i], B);
                                C = dp4a_su(wq[u][r].v[i], xc[i], C);
                            }
                            const float f = fmaf((float)A, 65536.f, fmaf((float)B, 256.f, (float)C));
                            acc[r][m] = fmaf(f, ws[u][r] * xs, acc[r][m]);
                            if (SWIGLU) {
                                int A2 = 0, B2 = 0, C2 = 0;
#pragma unroll
                                for (int i = 0; i < 8; i++) {
                                    A2 = dp4a_ss(wq2[u][r].v[i], xa[i], A2);
                                    B2 = dp4a_su(wq2[u][r].v[i], xb[i], B2);
                                    C2 = dp4a_su(wq2[u][r].v[i], xc[i], C2);
                                }
                                const float f2 = fmaf((float)A2, 65536.f, fmaf((float)B2, 256.f, (float)C2));
                                acc2[r][m] = fmaf(f2, ws2[u][r] * xs, acc2[r][m]);
                            }
                        }
                    }
                }
            }
        }

#pragma unroll
        for (int r = 0; r < R; r++) {
#pragma unroll
            for (int m = 0; m < MT; m++) {
                float s = warp_sum(acc[r][m]);
                float s2 = SWIGLU ? warp_sum(acc2[r][m]) : 0.f;
                const int row = row0 + r;
                if (lane == 0 && row < N) {
                    if (p.norm_w) { s *= rs_sh[m]; s2 *= rs_sh[m]; }
                    if (SWIGLU) s = s2 * (s * (1.f / (1.f + __expf(-s))));
                    const size_t o = (size_t)(p.m0 + m) * N + row;
                    if (p.residual) s += to_f32<TY>(reinterpret_cast<const TY*>(p.residual)[o]);
                    reinterpret_cast<TY*>(p.y)[o] = from_f32<TY>(s);
                }
            }
        }
    }
    blum_trace(p.trace, 3);
}

template <typename TX, typename TY, int MT, int R, int U, int THREADS, bool SWIGLU>
static int launch_i8(blum_ctx* ctx, const GemvI8Params& p, int ctas_per_sm) {
    auto kern = q8_gemv_i8_kernel<TX, TY, MT, R, U, THREADS, SWIGLU>;
    const int nit = (p.K + 1023) >> 10;
    const size_t smem = (size_t)MT * nit * (3072 + 128);
    BLUM_REQUIRE(ctx, smem + 4096 <= ctx->smem_optin, "q8 gemv: K=%d needs %zu B of shared memory", p.K, smem);
    if (smem + 2048 > 48 * 1024) BLUM_CUDA(ctx, cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    const int groups = (p.N + R - 1) / R;
    constexpr int NW = THREADS / 32;
    int grid = ctx->sm_count * ctas_per_sm;
    const int need = (groups + NW - 1) / NW;
    if (grid > need) grid = need;
    if (grid < 1) grid = 1;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(grid); cfg.blockDim = dim3(THREADS); cfg.dynamicSmemBytes = smem; cfg.stream = ctx->stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = ctx->pdl ? 1 : 0;
    cfg.attrs = attr; cfg.numAttrs = 1;
    BLUM_CUDA(ctx, cudaLaunchKernelEx(&cfg, kern, p));
    ctx->launches++;
    return BLUM_OK;
}

// One CTA of 32 warps per SM stages x once per SM; one row per warp pass keeps the row groups fine-grained; two
// 32-weight blocks per lane in flight.  (Smaller CTAs that could share an SM with the next kernel were measured and
// lose: half the warps cannot issue the dp4a work at stream rate.)
template <typename TX, typename TY, int MT, bool SWIGLU>
static int launch_i8_v(blum_ctx* ctx, const GemvI8Params& p) {
    return launch_i8<TX, TY, MT, 1, 2, 1024, SWIGLU>(ctx, p, 1);
}

template <bool SWIGLU>
static int launch_i8_types(blum_ctx* ctx, GemvI8Params p, int xdt, int ydt) {
    for (int m0 = 0; m0 < p.M; m0 += 2) {
        p.m0 = m0;
        p.mt = (p.M - m0 < 2) ? 1 : 2;
        int rc = BLUM_ERR_INVALID;
#define TT(xd, yd, TX, TY)                                                                  \
        if (xdt == xd && ydt == yd)                                                         \
            rc = (p.mt == 1) ? launch_i8_v<TX, TY, 1, SWIGLU>(ctx, p) : launch_i8_v<TX, TY, 2, SWIGLU>(ctx, p)
        TT(BLUM_F32, BLUM_F32, float, float);
        TT(BLUM_BF16, BLUM_BF16, __nv_bfloat16, __nv_bfloat16);
        TT(BLUM_F16, BLUM_F16, __half, __half);
        TT(BLUM_BF16, BLUM_F32, __nv_bfloat16, float);
        TT(BLUM_F16, BLUM_F32, __half, float);
#undef TT
        if (rc) return rc == BLUM_ERR_INVALID && ctx->err.empty() ? blum_fail(ctx, rc, "q8 gemv: unsupported dtype pair (%d,%d)", xdt, ydt) : rc;
    }
    return BLUM_OK;
}

bool blum_gemv_i8_supported(int xdt, int ydt) {
    return (xdt == ydt) || (ydt == BLUM_F32 && xdt != BLUM_F32);
}

int blum_gemv_i8_dispatch(blum_ctx* ctx, const blum_q8_weight* w, const blum_q8_weight* w_up, const void* x, int xdt,
                          const float* norm_w, float eps, const void* residual, void* y, int ydt, int64_t M) {
    BLUM_REQUIRE(ctx, w && x && y, "q8 matmul: null argument");
    BLUM_REQUIRE(ctx, M >= 1, "q8 matmul: M must be >= 1 (got %lld)", (long long)M);
    BLUM_REQUIRE(ctx, xdt >= 0 && xdt <= 2 && ydt >= 0 && ydt <= 2, "q8 matmul: bad dtype");
    BLUM_REQUIRE(ctx, w->N < (1ll << 31) && w->K < (1ll << 31), "q8 matmul: dimension too large");
    BLUM_REQUIRE(ctx, ((uintptr_t)x % 16) == 0, "q8 matmul: x must be 16-byte aligned");
    if (w_up) BLUM_REQUIRE(ctx, w_up->N == w->N && w_up->K == w->K, "q8 swiglu: gate and up weights differ in shape");
    GemvI8Params p;
    p.q = w->q; p.d = w->d;
    p.q2 = w_up ? w_up->q : nullptr; p.d2 = w_up ? w_up->d : nullptr;
    p.x = x; p.y = y; p.residual = residual; p.norm_w = norm_w; p.eps = eps;
    p.N = (int)w->N; p.K = (int)w->K; p.M = (int)M; p.m0 = 0; p.mt = 1;
    p.trace = blum_trace_slot(ctx);
    ctx->err.clear();
    if (w_up) return launch_i8_types<true>(ctx, p, xdt, ydt);
    return launch_i8_types<false>(ctx, p, xdt, ydt);
}
