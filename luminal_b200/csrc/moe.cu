// Mixture-of-experts feed-forward with MXFP4 expert weights: routing, token permutation, grouped GEMM, combine.
//
// luminal has no MoE, top-k or MXFP4 code; these are additions and their semantics are fixed here (the CPU checker used by
// the tests restates them):
//   * router: logits[t,e] = sum_h x[t,h] * Wr[e,h] (+ bias[e]) in f32 from bf16 inputs;
//   * top-k: the k largest logits, ties resolved towards the LOWER expert index; gates = softmax over the k selected
//     logits (equal to the renormalised full softmax);
//   * permutation: (token, choice) pairs sorted by expert, stable in token order then choice order within an expert;
//   * expert: y = Wdown( (Wup x) * swish(Wgate x) ); weights MXFP4 = e2m1 codes with one e8m0 scale per 32 elements
//     along K (element 2i in the low nibble of byte i), dequantised exactly to bf16 for the tensor cores;
//   * combine: out[t] = sum_j gate[t,j] * y_{expert(t,j)}[t] accumulated in f32 in choice order.
// The grouped GEMM is the tcgen05 kernel of q8_gemm_tc.cu in grouped mode (one launch for all experts).
#include "common.cuh"
#include <string.h>


enum { WF_Q8_0 = 0, WF_MXFP4 = 1, WF_BF16 = 2 };

__global__ void mxfp4_generate_kernel(uint8_t* __restrict__ q, uint8_t* __restrict__ s, int64_t nbytes, int64_t nblocks,
                                      uint64_t key_q, uint64_t key_s) {
    const int64_t stride = (int64_t)gridDim.x * blockDim.x;
    for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < nbytes; i += stride) {
        const uint32_t lo = (uint32_t)(blum_gen_hash(key_q, (uint64_t)(2 * i)) >> 60);        // 16 codes, uniform
        const uint32_t hi = (uint32_t)(blum_gen_hash(key_q, (uint64_t)(2 * i + 1)) >> 60);
        q[i] = (uint8_t)(lo | (hi << 4));
    }
    for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < nblocks; i += stride)
        s[i] = (uint8_t)(119 + (((blum_gen_hash(key_s, (uint64_t)i) >> 32) * 9ull) >> 32));   // exponent uniform in [-8, 0]
}

// one CTA per token, 32 warps; warp w computes the logits of experts w, w+32, ... (all loads of a pass of 1024 columns in
// flight together: at one token the kernel is nothing but load latency); warp 0 then selects
#define MOE_ROUTE_WARPS 32
__global__ void __launch_bounds__(32 * MOE_ROUTE_WARPS) moe_route_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ wr,
                                                        const float* __restrict__ bias, int H, int E, int k,
                                                        int32_t* __restrict__ ids, float* __restrict__ gates) {
    __shared__ float logits[256];
    const int t = blockIdx.x, lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const __nv_bfloat16* xr = x + (size_t)t * H;
    for (int e = warp; e < E; e += MOE_ROUTE_WARPS) {
        const __nv_bfloat16* w = wr + (size_t)e * H;
        float acc = 0.f;
        for (int h0 = lane * 8; h0 < H; h0 += 1024) {
            uint4 a[4], b[4];
#pragma unroll
            for (int u = 0; u < 4; u++) {
                const int h = h0 + u * 256;
                if (h < H) { a[u] = *reinterpret_cast<const uint4*>(xr + h); b[u] = *reinterpret_cast<const uint4*>(w + h); }
            }
#pragma unroll
            for (int u = 0; u < 4; u++) {
                if (h0 + u * 256 < H) {
                    const uint32_t aw[4] = {a[u].x, a[u].y, a[u].z, a[u].w}, bw[4] = {b[u].x, b[u].y, b[u].z, b[u].w};
#pragma unroll
                    for (int i = 0; i < 4; i++) {
                        acc = fmaf(__uint_as_float(aw[i] << 16), __uint_as_float(bw[i] << 16), acc);
                        acc = fmaf(__uint_as_float(aw[i] & 0xffff0000u), __uint_as_float(bw[i] & 0xffff0000u), acc);
                    }
                }
            }
        }
        acc = warp_sum(acc);
        if (lane == 0) logits[e] = acc + (bias ? bias[e] : 0.f);
    }
    __syncthreads();
    if (warp == 0) {
        float sel_v[8]; int sel_i[8];
        for (int j = 0; j < k; j++) {
            float bv = -INFINITY; int bi = 0x7fffffff;
            for (int e = lane; e < E; e += 32) {
                const float v = logits[e];
                if (v > bv || (v == bv && e < bi)) { bv = v; bi = e; }
            }
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) {
                const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
                const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
                if (ov > bv || (ov == bv && oi < bi)) { bv = ov; bi = oi; }
            }
            sel_v[j] = bv; sel_i[j] = bi;
            if (lane == 0) logits[bi] = -INFINITY;
            __syncwarp();
        }
        if (lane == 0) {
            float m = sel_v[0], sum = 0.f, ex[8];
            for (int j = 0; j < k; j++) { ex[j] = exp2f((sel_v[j] - m) * 1.4426950408889634f); sum += ex[j]; }
            const float inv = 1.f / sum;
            for (int j = 0; j < k; j++) { ids[(size_t)t * k + j] = sel_i[j]; gates[(size_t)t * k + j] = ex[j] * inv; }
        }
    }
}

// Stable counting sort of the T*k (token, choice) pairs by expert: one CTA of 32 warps, a warp per expert (round-robin when
// there are more than 32).  A warp reads 32 pairs per step; the ballot of "this pair chose my expert" gives the count in the
// first pass and, with the prefix of lower lanes, each pair's sorted row in the second - pair order inside an expert is kept.
__global__ void __launch_bounds__(1024) moe_permute_kernel(const int32_t* __restrict__ ids, int n, int E, int32_t* __restrict__ sorted_src,
                                                           int32_t* __restrict__ slot_of, int32_t* __restrict__ offsets, int* err) {
    __shared__ int counts[257];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, warps = blockDim.x >> 5;
    for (int e = warp; e < E; e += warps) {
        int c = 0;
        for (int i0 = 0; i0 < n; i0 += 32) {
            const int i = i0 + lane;
            c += __popc(__ballot_sync(0xffffffffu, i < n && ids[i] == e));
        }
        if (lane == 0) counts[e] = c;
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        int run = 0;
        for (int j = 0; j < E; j++) { const int c = counts[j]; counts[j] = run; offsets[j] = run; run += c; }
        offsets[E] = run;
        if (run != n) atomicOr(err, 0x2000);       // an expert id outside [0,E)
    }
    __syncthreads();
    for (int e = warp; e < E; e += warps) {
        int pos = counts[e];
        for (int i0 = 0; i0 < n; i0 += 32) {
            const int i = i0 + lane;
            const bool mine = i < n && ids[i] == e;
            const unsigned m = __ballot_sync(0xffffffffu, mine);
            if (mine) {
                const int r = pos + __popc(m & ((1u << lane) - 1u));
                sorted_src[r] = i;
                slot_of[i] = r;
            }
            pos += __popc(m);
        }
    }
}

// xp[r, :] = x[sorted_src[r] / k, :]
__global__ void moe_gather_rows_kernel(const __nv_bfloat16* __restrict__ x, const int32_t* __restrict__ sorted_src, int k,
                                       int H, __nv_bfloat16* __restrict__ xp) {
    const int r = blockIdx.x;
    const int t = sorted_src[r] / k;
    const uint4* src = reinterpret_cast<const uint4*>(x + (size_t)t * H);
    uint4* dst = reinterpret_cast<uint4*>(xp + (size_t)r * H);
    for (int i = threadIdx.x; i < H / 8; i += blockDim.x) dst[i] = src[i];
}

// out[t, :] = sum_j gates[t,j] * yp[slot_of[t*k+j], :]
template <typename TO>
__global__ void moe_unpermute_kernel(const __nv_bfloat16* __restrict__ yp, const int32_t* __restrict__ slot_of,
                                     const float* __restrict__ gates, int k, int H, TO* __restrict__ out) {
    const int t = blockIdx.x;
    __shared__ float g_s[8];
    __shared__ int slot_s[8];
    if (threadIdx.x < k) { g_s[threadIdx.x] = gates[(size_t)t * k + threadIdx.x]; slot_s[threadIdx.x] = slot_of[(size_t)t * k + threadIdx.x]; }
    __syncthreads();
    // two columns per thread, the k rows of a column pair requested together (H is even)
    for (int h = 2 * threadIdx.x; h < H; h += 2 * blockDim.x) {
        uint32_t v[8];
#pragma unroll
        for (int j = 0; j < 8; j++) if (j < k) v[j] = *reinterpret_cast<const uint32_t*>(yp + (size_t)slot_s[j] * H + h);
        float a0 = 0.f, a1 = 0.f;
#pragma unroll
        for (int j = 0; j < 8; j++)
            if (j < k) {
                a0 = fmaf(g_s[j], __uint_as_float(v[j] << 16), a0);
                a1 = fmaf(g_s[j], __uint_as_float(v[j] & 0xffff0000u), a1);
            }
        out[(size_t)t * H + h] = from_f32<TO>(a0);
        out[(size_t)t * H + h + 1] = from_f32<TO>(a1);
    }
}

// rows of the stacked weight: 32-row groups, 16 gate rows then the 16 up rows of the same features; one 16-byte word per thread
__global__ void mxfp4_stack_kernel(const uint4* __restrict__ g, const uint4* __restrict__ u, uint4* __restrict__ out, int64_t rows_out,
                                   int64_t N, int words_per_row) {
    const int64_t total = rows_out * words_per_row;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
        const int64_t r = i / words_per_row, w = i - r * words_per_row;
        const int64_t e = r / (2 * N), rr = r - e * 2 * N;          // row inside the expert's 2N stacked rows
        const int64_t src = e * N + (rr >> 5) * 16 + (rr & 15);
        out[i] = ((rr & 16) ? u : g)[src * words_per_row + w];
    }
}

extern "C" {

int blum_mxfp4_weight_free(blum_ctx* ctx, blum_mxfp4_weight* w) {
    if (!ctx) return BLUM_ERR_INVALID;
    if (!w) return BLUM_OK;
    cudaSetDevice(ctx->device);
    cudaStreamSynchronize(ctx->stream);
    if (w->q) cudaFree(w->q);
    if (w->s) cudaFree(w->s);
    delete w;
    return BLUM_OK;
}

static int mxfp4_alloc(blum_ctx* ctx, int E, int64_t N, int64_t K, blum_mxfp4_weight** out) {
    BLUM_REQUIRE(ctx, out != nullptr, "mxfp4 weight: null output");
    *out = nullptr;
    BLUM_REQUIRE(ctx, E > 0 && N > 0 && K > 0 && K % 64 == 0, "mxfp4 weight: need E>0, N>0, K %% 64 == 0");
    BLUM_CUDA(ctx, cudaSetDevice(ctx->device));
    blum_mxfp4_weight* w = new blum_mxfp4_weight();
    w->E = E; w->N = N; w->K = K;
    cudaError_t e = cudaMalloc((void**)&w->q, (size_t)E * N * K / 2);
    if (e == cudaSuccess) e = cudaMalloc((void**)&w->s, (size_t)E * N * K / 32);
    if (e != cudaSuccess) {
        if (w->q) cudaFree(w->q);
        delete w;
        return blum_fail(ctx, BLUM_ERR_OOM, "mxfp4 weight: cudaMalloc failed: %s", cudaGetErrorString(e));
    }
    *out = w;
    return BLUM_OK;
}

/* E stacked expert matrices [N,K]: packed e2m1 bytes [E*N*K/2] and e8m0 scale bytes [E*N*K/32] from the host. */
int blum_mxfp4_weight_from_host(blum_ctx* ctx, const void* nibbles, const void* scales, int E, int64_t N, int64_t K,
                                blum_mxfp4_weight** out) {
    if (!ctx) return BLUM_ERR_INVALID;
    BLUM_REQUIRE(ctx, nibbles && scales, "mxfp4 weight: null data");
    int rc = mxfp4_alloc(ctx, E, N, K, out);
    if (rc) return rc;
    BLUM_CUDA(ctx, cudaMemcpyAsync((*out)->q, nibbles, (size_t)E * N * K / 2, cudaMemcpyHostToDevice, ctx->stream));
    BLUM_CUDA(ctx, cudaMemcpyAsync((*out)->s, scales, (size_t)E * N * K / 32, cudaMemcpyHostToDevice, ctx->stream));
    BLUM_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
    return BLUM_OK;
}

/* Seeded weights: codes uniform over the 16 e2m1 values, block exponents uniform in [-8, 0]. */
int blum_mxfp4_weight_generate(blum_ctx* ctx, uint64_t seed, uint64_t tensor_id, int E, int64_t N, int64_t K,
                               blum_mxfp4_weight** out) {
    if (!ctx) return BLUM_ERR_INVALID;
    int rc = mxfp4_alloc(ctx, E, N, K, out);
    if (rc) return rc;
    mxfp4_generate_kernel<<<ctx->sm_count * 8, 256, 0, ctx->stream>>>((*out)->q, (*out)->s, (int64_t)E * N * K / 2, (int64_t)E * N * K / 32,
                                                                     blum_gen_key(seed, tensor_id), blum_gen_key(seed, tensor_id ^ (0x5ca1e5ull << 40)));
    BLUM_LAUNCH_CHECK(ctx);
    return BLUM_OK;
}

int blum_mxfp4_weight_stack_gate_up(blum_ctx* ctx, const blum_mxfp4_weight* gate, const blum_mxfp4_weight* up, blum_mxfp4_weight** out) {
    if (!ctx) return BLUM_ERR_INVALID;
    BLUM_REQUIRE(ctx, gate && up && out, "mxfp4 stack: null argument");
    BLUM_REQUIRE(ctx, gate->E == up->E && gate->N == up->N && gate->K == up->K, "mxfp4 stack: gate and up differ in shape");
    BLUM_REQUIRE(ctx, gate->N % 16 == 0, "mxfp4 stack: need N %% 16 == 0");      // (K %% 64 == 0: a row's K/2 quant bytes are whole 16-byte words)
    const int64_t N = gate->N, K = gate->K;
    int rc = mxfp4_alloc(ctx, gate->E, 2 * N, K, out);
    if (rc) return rc;
    const int64_t rows_out = (int64_t)gate->E * 2 * N;
    mxfp4_stack_kernel<<<ctx->sm_count * 8, 256, 0, ctx->stream>>>((const uint4*)gate->q, (const uint4*)up->q, (uint4*)(*out)->q, rows_out, N, (int)(K / 32));
    BLUM_LAUNCH_CHECK(ctx);
    // the scale plane has K/32 bytes per row, not a multiple of 16 in general: it is copied 16 rows at a time as whole rows
    BLUM_CUDA(ctx, cudaMemcpy2DAsync((*out)->s, (size_t)32 * (K / 32), gate->s, (size_t)16 * (K / 32), (size_t)16 * (K / 32), (size_t)(gate->E * N / 16),
                                     cudaMemcpyDeviceToDevice, ctx->stream));
    BLUM_CUDA(ctx, cudaMemcpy2DAsync((*out)->s + (size_t)16 * (K / 32), (size_t)32 * (K / 32), up->s, (size_t)16 * (K / 32), (size_t)16 * (K / 32),
                                     (size_t)(gate->E * N / 16), cudaMemcpyDeviceToDevice, ctx->stream));
    BLUM_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
    return BLUM_OK;
}

int blum_mxfp4_weight_download(blum_ctx* ctx, const blum_mxfp4_weight* w, void* nibbles_out, void* scales_out) {
    if (!ctx) return BLUM_ERR_INVALID;
    BLUM_REQUIRE(ctx, w && nibbles_out && scales_out, "mxfp4 download: null argument");
    BLUM_CUDA(ctx, cudaMemcpyAsync(nibbles_out, w->q, (size_t)w->E * w->N * w->K / 2, cudaMemcpyDeviceToHost, ctx->stream));
    BLUM_CUDA(ctx, cudaMemcpyAsync(scales_out, w->s, (size_t)w->E * w->N * w->K / 32, cudaMemcpyDeviceToHost, ctx->stream));
    BLUM_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
    return BLUM_OK;
}

int blum_moe_route_topk(blum_ctx* ctx, const void* x_bf16, const void* router_w_bf16, const float* router_bias, int64_t T,
                        int H, int E, int k, int32_t* ids_out, float* gates_out) {
    if (!ctx) return BLUM_ERR_INVALID;
    BLUM_REQUIRE(ctx, x_bf16 && router_w_bf16 && ids_out && gates_out, "moe_route: null argument");
    BLUM_REQUIRE(ctx, T >= 0 && H > 0 && H % 8 == 0 && E > 0 && E <= 256 && k > 0 && k <= 8 && k <= E, "moe_route: need H %% 8 == 0, E <= 256, k <= 8");
    if (T == 0) return BLUM_OK;
    moe_route_kernel<<<(unsigned)T, 32 * MOE_ROUTE_WARPS, 0, ctx->stream>>>((const __nv_bfloat16*)x_bf16, (const __nv_bfloat16*)router_w_bf16, router_bias,
                                                          H, E, k, ids_out, gates_out);
    BLUM_LAUNCH_CHECK(ctx);
    return BLUM_OK;
}

/* ids [T*k] -> sorted_src [T*k] (index of the (token, choice) pair at each sorted row), slot_of [T*k] (its inverse),
 * offsets [E+1] (first sorted row of every expert). */
int blum_moe_permute(blum_ctx* ctx, const int32_t* ids, int64_t n_pairs, int E, int32_t* sorted_src, int32_t* slot_of,
                     int32_t* offsets) {
    if (!ctx) return BLUM_ERR_INVALID;
    BLUM_REQUIRE(ctx, ids && sorted_src && slot_of && offsets && n_pairs >= 0 && E > 0 && E <= 256, "moe_permute: bad argument");
    moe_permute_kernel<<<1, 1024, 0, ctx->stream>>>(ids, (int)n_pairs, E, sorted_src, slot_of, offsets, ctx->dev_error);
    BLUM_LAUNCH_CHECK(ctx);
    return BLUM_OK;
}

int blum_moe_gather_rows(blum_ctx* ctx, const void* x_bf16, const int32_t* sorted_src, int64_t n_pairs, int k, int H, void* xp_bf16) {
    if (!ctx) return BLUM_ERR_INVALID;
    BLUM_REQUIRE(ctx, x_bf16 && sorted_src && xp_bf16 && k > 0 && H % 8 == 0, "moe_gather_rows: bad argument");
    if (n_pairs == 0) return BLUM_OK;
    moe_gather_rows_kernel<<<(unsigned)n_pairs, 128, 0, ctx->stream>>>((const __nv_bfloat16*)x_bf16, sorted_src, k, H, (__nv_bfloat16*)xp_bf16);
    BLUM_LAUNCH_CHECK(ctx);
    return BLUM_OK;
}

/* yp[r, :] = xp[r, :] * W_e^T for the rows r of expert e (offsets from blum_moe_permute). */
int blum_moe_grouped_gemm(blum_ctx* ctx, const blum_mxfp4_weight* w, const void* xp_bf16, const int32_t* offsets, int64_t n_rows,
                          void* yp, blum_dtype y_dtype, int rows_per_expert_hint) {
    if (!ctx) return BLUM_ERR_INVALID;
    BLUM_REQUIRE(ctx, w && xp_bf16 && offsets && yp, "moe_grouped_gemm: null argument");
    if (n_rows == 0) return BLUM_OK;
    return blum_tc_gemm(ctx, WF_MXFP4, w->q, w->s, (int64_t)w->E * w->N, (int)w->N, (int)w->K, xp_bf16, n_rows, yp, y_dtype,
                        offsets, w->E, rows_per_expert_hint);
}

int blum_moe_grouped_gemm_swiglu(blum_ctx* ctx, const blum_mxfp4_weight* w, const void* xp_bf16, const int32_t* offsets, int64_t n_rows,
                                 void* mid_bf16, int rows_per_expert_hint) {
    if (!ctx) return BLUM_ERR_INVALID;
    BLUM_REQUIRE(ctx, w && xp_bf16 && offsets && mid_bf16, "moe_grouped_gemm_swiglu: null argument");
    BLUM_REQUIRE(ctx, w->N % 32 == 0, "moe_grouped_gemm_swiglu: the weight is not a stacked gate/up weight");
    if (n_rows == 0) return BLUM_OK;
    return blum_tc_gemm(ctx, WF_MXFP4, w->q, w->s, (int64_t)w->E * w->N, (int)w->N, (int)w->K, xp_bf16, n_rows, mid_bf16, BLUM_BF16,
                        offsets, w->E, rows_per_expert_hint, 1);
}

int blum_moe_unpermute(blum_ctx* ctx, const void* yp_bf16, const int32_t* slot_of, const float* gates, int64_t T, int k, int H,
                       void* out, blum_dtype out_dtype) {
    if (!ctx) return BLUM_ERR_INVALID;
    BLUM_REQUIRE(ctx, yp_bf16 && slot_of && gates && out && k > 0 && k <= 8 && H > 0 && H % 2 == 0, "moe_unpermute: need k <= 8 and an even H");
    if (T == 0) return BLUM_OK;
    if (out_dtype == BLUM_F32) moe_unpermute_kernel<float><<<(unsigned)T, 256, 0, ctx->stream>>>((const __nv_bfloat16*)yp_bf16, slot_of, gates, k, H, (float*)out);
    else if (out_dtype == BLUM_BF16) moe_unpermute_kernel<__nv_bfloat16><<<(unsigned)T, 256, 0, ctx->stream>>>((const __nv_bfloat16*)yp_bf16, slot_of, gates, k, H, (__nv_bfloat16*)out);
    else return blum_fail(ctx, BLUM_ERR_INVALID, "moe_unpermute: output must be f32 or bf16");
    BLUM_LAUNCH_CHECK(ctx);
    return BLUM_OK;
}

}  // extern "C"
