// Fused GQA attention over the paged KV cache.
//
// Replaces the chain the reference runs per layer (examples/llama/src/model.rs:113-136 in luminal):
// materialise the 4x GQA-expanded K and V, cuBLAS batched QK^T (crates/luminal_cuda/src/matmul.rs:59-107),
// a fused scale + additive causal mask, CudaSoftmax (crates/luminal_cuda/src/unary.rs:493-593), cuBLAS PV and a
// head-merge copy.  Here one kernel streams each K/V page once for all query heads of a KV head, keeps an
// online softmax (max, sum) in f32, and splits long contexts over CTAs whose partial (max, sum, out)
// triples a second kernel merges ("split-K decode").
//
// A "query row" is one token of one sequence: at decode there is one row per sequence, at prefill one row
// per new token with ctx = position + 1, which is exactly the reference's causal mask: positions j with
// j - p > t receive -65504 before the softmax and their exp2 underflows to 0 in f32, so leaving them out
// changes nothing.
// Algorithmic bytes per row per layer: 2 * kv_heads * head_dim * ctx * sizeof(kv element).
#include "kv.cuh"
#include <math.h>

#define LOG2E 1.4426950408889634f

template <typename TC>
__device__ __forceinline__ void load8(const TC* p, float* o);
template <> __device__ __forceinline__ void load8<float>(const float* p, float* o) {
    const float4 a = *reinterpret_cast<const float4*>(p), b = *reinterpret_cast<const float4*>(p + 4);
    o[0] = a.x; o[1] = a.y; o[2] = a.z; o[3] = a.w; o[4] = b.x; o[5] = b.y; o[6] = b.z; o[7] = b.w;
}
template <> __device__ __forceinline__ void load8<__nv_bfloat16>(const __nv_bfloat16* p, float* o) {
    const uint4 v = *reinterpret_cast<const uint4*>(p);
    const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
    for (int i = 0; i < 4; i++) { o[2 * i] = __uint_as_float(w[i] << 16); o[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u); }
}
template <> __device__ __forceinline__ void load8<__half>(const __half* p, float* o) {
    const uint4 v = *reinterpret_cast<const uint4*>(p);
    const __half2* h = reinterpret_cast<const __half2*>(&v);
#pragma unroll
    for (int i = 0; i < 4; i++) { o[2 * i] = __low2float(h[i]); o[2 * i + 1] = __high2float(h[i]); }
}

struct AttnParams {
    KvView kv;
    int layer, max_seqs;
    const void* q;            // [rows, nq, D]
    void* out;                // [rows, nq, D]
    float* part_o;            // [rows, nq, splits, D]   (splits > 1)
    float* part_ml;           // [rows, nq, splits, 2]
    const int32_t* seq_ids;   // [rows]
    const int32_t* ctx_lens;  // [rows]
    int nq;
    float scale;              // 1/sqrt(D)
    int* err;
};

// grid (splits, kv_heads, rows); block D threads.  TILE = D/2 positions per iteration.
template <typename TQ, typename TC, int G, int D>
__global__ void __launch_bounds__(D) attn_rows_kernel(const AttnParams p) {
    constexpr int TILE = D / 2;
    constexpr int QPAD = D / 2 + 4;              // the two halves of q land in different banks
    __shared__ __align__(16) float qs[G][2][QPAD];
    __shared__ float sc[G][TILE];
    __shared__ float corr[G];

    const int split = blockIdx.x, nsplit = gridDim.x, kvh = blockIdx.y, row = blockIdx.z;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    constexpr int NW = D / 32;
    const KvView& kv = p.kv;
    const int ps = kv.page_size;

    int seq = p.seq_ids[row];
    int ctx = p.ctx_lens[row];
    bool bad = false;
    if (seq < 0 || seq >= p.max_seqs || ctx < 0 || (ctx + ps - 1) / ps > kv.max_pages_per_seq) { bad = true; ctx = 0; seq = 0; }
    if (bad && tid == 0) atomicOr(p.err, 0x100);

    // this split's position range, cut on page boundaries
    const int npages = (ctx + ps - 1) / ps;
    const int pages_per_split = (npages + nsplit - 1) / nsplit;
    const int c0 = min(ctx, split * pages_per_split * ps);
    const int c1 = min(ctx, (split + 1) * pages_per_split * ps);

    // q of the G heads of this kv head
    const TQ* qg = reinterpret_cast<const TQ*>(p.q) + ((int64_t)row * p.nq + (int64_t)kvh * G) * D;
    for (int i = tid; i < G * D; i += D) {
        const int g = i / D, c = i % D;
        qs[g][c / (D / 2)][c % (D / 2)] = to_f32<TQ>(qg[i]);
    }
    __syncthreads();

    const TC* pool = reinterpret_cast<const TC*>(kv.pool);
    const int32_t* table = kv.table + (int64_t)seq * kv.max_pages_per_seq;

    float m_run[G], l_run[G], o_acc[G];
#pragma unroll
    for (int g = 0; g < G; g++) { m_run[g] = -INFINITY; l_run[g] = 0.f; o_acc[g] = 0.f; }

    const int jj = tid >> 1, half = tid & 1;
    for (int t0 = c0; t0 < c1; t0 += TILE) {
        // ---- scores for TILE positions: two threads per position, D/2 dims each
        {
            const int pos = t0 + jj;
            float acc[G];
#pragma unroll
            for (int g = 0; g < G; g++) acc[g] = 0.f;
            if (pos < c1) {
                int32_t page = table[pos / ps];
                if (page < 0 || page >= kv.num_pages) { atomicOr(p.err, 0x200); page = 0; }
                const TC* kr = pool + kv_tile_offset(kv, p.layer, page, 0, kvh, pos % ps) + half * (D / 2);
#pragma unroll
                for (int c = 0; c < D / 2; c += 8) {
                    float kvv[8];
                    load8<TC>(kr + c, kvv);
#pragma unroll
                    for (int g = 0; g < G; g++) {
                        const float4 qa = *reinterpret_cast<const float4*>(&qs[g][half][c]);
                        const float4 qb = *reinterpret_cast<const float4*>(&qs[g][half][c + 4]);
                        acc[g] += kvv[0] * qa.x + kvv[1] * qa.y + kvv[2] * qa.z + kvv[3] * qa.w +
                                  kvv[4] * qb.x + kvv[5] * qb.y + kvv[6] * qb.z + kvv[7] * qb.w;
                    }
                }
            }
#pragma unroll
            for (int g = 0; g < G; g++) {
                const float s = acc[g] + __shfl_xor_sync(0xffffffffu, acc[g], 1);
                if (half == 0) sc[g][jj] = (pos < c1) ? s * p.scale : -INFINITY;
            }
        }
        __syncthreads();
        // ---- online softmax per head (one warp per head, round-robin)
#pragma unroll
        for (int g = 0; g < G; g++) {
            if (g % NW == warp) {   // every thread carries the same running max, so any warp can take a head
                float mx = -INFINITY;
                for (int j = lane; j < TILE; j += 32) mx = fmaxf(mx, sc[g][j]);
                mx = warp_max(mx);
                const float m_new = fmaxf(m_run[g], mx);
                for (int j = lane; j < TILE; j += 32) sc[g][j] = exp2f((sc[g][j] - m_new) * LOG2E);
                if (lane == 0) corr[g] = m_new;
            }
        }
        __syncthreads();
        // ---- every thread rescales its copy of (m, l) and its output column, then adds the tile
#pragma unroll
        for (int g = 0; g < G; g++) {
            const float m_new = corr[g];
            const float c = (m_run[g] == -INFINITY) ? 0.f : exp2f((m_run[g] - m_new) * LOG2E);
            l_run[g] *= c;
            o_acc[g] *= c;
            m_run[g] = m_new;
        }
        const int tile_n = min(TILE, c1 - t0);
        for (int j = 0; j < tile_n; j++) {
            const int pos = t0 + j;
            int32_t page = table[pos / ps];
            if (page < 0 || page >= kv.num_pages) page = 0;
            const float vv = to_f32<TC>(pool[kv_tile_offset(kv, p.layer, page, 1, kvh, pos % ps) + tid]);
#pragma unroll
            for (int g = 0; g < G; g++) {
                const float pj = sc[g][j];
                l_run[g] += pj;
                o_acc[g] = fmaf(pj, vv, o_acc[g]);
            }
        }
        __syncthreads();
    }

    // ---- write
#pragma unroll
    for (int g = 0; g < G; g++) {
        const int h = kvh * G + g;
        if (nsplit == 1) {
            const float inv = l_run[g] > 0.f ? 1.f / l_run[g] : 0.f;
            reinterpret_cast<TQ*>(p.out)[((int64_t)row * p.nq + h) * D + tid] = from_f32<TQ>(o_acc[g] * inv);
        } else {
            const int64_t base = ((int64_t)row * p.nq + h) * nsplit + split;
            p.part_o[base * D + tid] = o_acc[g];
            if (tid == 0) { p.part_ml[base * 2] = m_run[g]; p.part_ml[base * 2 + 1] = l_run[g]; }
        }
    }
}

// merges split partials: grid (nq, rows), block D
template <typename TQ, int D>
__global__ void __launch_bounds__(D) attn_combine_kernel(const float* __restrict__ part_o, const float* __restrict__ part_ml,
                                                         int nq, int nsplit, TQ* __restrict__ out) {
    const int h = blockIdx.x, row = blockIdx.y, tid = threadIdx.x;
    const int64_t base = ((int64_t)row * nq + h) * nsplit;
    float m = -INFINITY;
    for (int s = 0; s < nsplit; s++) m = fmaxf(m, part_ml[(base + s) * 2]);
    float l = 0.f, o = 0.f;
    for (int s = 0; s < nsplit; s++) {
        const float ms = part_ml[(base + s) * 2];
        if (ms == -INFINITY) continue;
        const float w = exp2f((ms - m) * LOG2E);
        l += w * part_ml[(base + s) * 2 + 1];
        o += w * part_o[(base + s) * D + tid];
    }
    out[((int64_t)row * nq + h) * D + tid] = from_f32<TQ>(l > 0.f ? o / l : 0.f);
}

// merge of split partials for callers in other translation units
int blum_attn_combine(blum_ctx* ctx, const float* part_o, const float* part_ml, int nq, int nsplit, int rows, int head_dim,
                      void* out, int dtype) {
    const dim3 grid(nq, rows);
#define COMBINE(T, D) attn_combine_kernel<T, D><<<grid, D, 0, ctx->stream>>>(part_o, part_ml, nq, nsplit, (T*)out)
    if (head_dim == 128) {
        if (dtype == BLUM_F32) COMBINE(float, 128); else if (dtype == BLUM_F16) COMBINE(__half, 128); else COMBINE(__nv_bfloat16, 128);
    } else if (head_dim == 64) {
        if (dtype == BLUM_F32) COMBINE(float, 64); else if (dtype == BLUM_F16) COMBINE(__half, 64); else COMBINE(__nv_bfloat16, 64);
    } else {
        return blum_fail(ctx, BLUM_ERR_INVALID, "attention combine: unsupported head_dim %d", head_dim);
    }
#undef COMBINE
    BLUM_LAUNCH_CHECK(ctx);
    return BLUM_OK;
}

__global__ void prefill_rows_kernel(int32_t* seq_ids, int32_t* ctx_lens, int seq, int p, int T) {
    const int t = blockIdx.x * blockDim.x + threadIdx.x;
    if (t < T) { seq_ids[t] = seq; ctx_lens[t] = p + t + 1; }
}

template <typename TQ, typename TC, int G, int D>
static int launch_attn(blum_ctx* ctx, const AttnParams& p, int rows, int nsplit) {
    dim3 grid(nsplit, p.kv.kv_heads, rows);
    attn_rows_kernel<TQ, TC, G, D><<<grid, D, 0, ctx->stream>>>(p);
    BLUM_LAUNCH_CHECK(ctx);
    if (nsplit > 1) {
        attn_combine_kernel<TQ, D><<<dim3(p.nq, rows), D, 0, ctx->stream>>>(p.part_o, p.part_ml, p.nq, nsplit, (TQ*)p.out);
        BLUM_LAUNCH_CHECK(ctx);
    }
    return BLUM_OK;
}

template <typename TQ, typename TC>
static int launch_attn_gd(blum_ctx* ctx, const AttnParams& p, int rows, int nsplit, int g, int d) {
#define GD(gg, dd) if (g == gg && d == dd) return launch_attn<TQ, TC, gg, dd>(ctx, p, rows, nsplit)
    GD(1, 128); GD(2, 128); GD(4, 128); GD(8, 128);
    GD(1, 64);  GD(2, 64);  GD(4, 64);  GD(8, 64);
#undef GD
    return blum_fail(ctx, BLUM_ERR_INVALID, "attention: unsupported group size %d / head_dim %d", g, d);
}

int blum_attn_rows(blum_ctx* ctx, blum_kv* kv, int layer, const void* q, int dtype, int q_heads, const int32_t* seq_ids,
                   const int32_t* ctx_lens, int64_t rows, int nsplit, void* scratch, void* out) {
    BLUM_REQUIRE(ctx, kv && q && out && seq_ids && ctx_lens, "attention: null argument");
    BLUM_REQUIRE(ctx, layer >= 0 && layer < kv->layers, "attention: layer %d outside [0,%d)", layer, kv->layers);
    BLUM_REQUIRE(ctx, q_heads > 0 && q_heads % kv->kv_heads == 0, "attention: q_heads %d not a multiple of kv_heads %d", q_heads, kv->kv_heads);
    BLUM_REQUIRE(ctx, rows >= 0 && rows < 65536, "attention: too many rows");
    if (rows == 0) return BLUM_OK;
    if (nsplit < 1) nsplit = 1;
    BLUM_REQUIRE(ctx, nsplit == 1 || scratch, "attention: split decode needs a scratch buffer");
    int rc = blum_kv_sync_tables(ctx, kv);
    if (rc) return rc;
    AttnParams p;
    p.kv = kv_view(kv); p.layer = layer; p.max_seqs = kv->max_seqs;
    p.q = q; p.out = out; p.seq_ids = seq_ids; p.ctx_lens = ctx_lens; p.nq = q_heads;
    p.scale = 1.0f / sqrtf((float)kv->head_dim);
    p.err = ctx->dev_error;
    p.part_o = (float*)scratch;
    p.part_ml = p.part_o ? p.part_o + (size_t)rows * q_heads * nsplit * kv->head_dim : nullptr;
    const int g = q_heads / kv->kv_heads, d = kv->head_dim;
    if (dtype == BLUM_F32 && kv->dtype == BLUM_F32) return launch_attn_gd<float, float>(ctx, p, (int)rows, nsplit, g, d);
    if (dtype == BLUM_BF16 && kv->dtype == BLUM_BF16) return launch_attn_gd<__nv_bfloat16, __nv_bfloat16>(ctx, p, (int)rows, nsplit, g, d);
    if (dtype == BLUM_F16 && kv->dtype == BLUM_F16) return launch_attn_gd<__half, __half>(ctx, p, (int)rows, nsplit, g, d);
    if (dtype == BLUM_F32 && kv->dtype == BLUM_BF16) return launch_attn_gd<float, __nv_bfloat16>(ctx, p, (int)rows, nsplit, g, d);
    return blum_fail(ctx, BLUM_ERR_INVALID, "attention: unsupported dtype pair (%d,%d)", dtype, kv->dtype);
}

extern "C" {

size_t blum_attn_decode_scratch_bytes(int64_t B, int q_heads, int head_dim, int max_splits) {
    if (B <= 0 || q_heads <= 0 || head_dim <= 0 || max_splits <= 1) return 0;
    return (size_t)B * q_heads * max_splits * (head_dim + 2) * sizeof(float);
}

int blum_attn_decode_paged(blum_ctx* ctx, blum_kv* kv, int layer, const void* q, blum_dtype dtype, int q_heads,
                           const int32_t* seq_ids, const int32_t* ctx_lens, int64_t B, int max_splits, void* scratch,
                           void* out) {
    if (!ctx) return BLUM_ERR_INVALID;
    return blum_attn_rows(ctx, kv, layer, q, dtype, q_heads, seq_ids, ctx_lens, B, max_splits, scratch, out);
}

}  // extern "C"

// ------------------------------------------------------------------ split decode without any allocation
// Scratch for the split partials lives in the library image itself: BLUM_ATTN_STATIC_FLOATS floats (8 MiB) of
// device memory that every GPU which loads the library keeps until the process exits.
#define BLUM_ATTN_STATIC_FLOATS (2u << 20)
static __device__ __align__(256) float g_attn_static_scratch[BLUM_ATTN_STATIC_FLOATS];
// In host code the array's name only stands for the symbol; the device address has to be asked for, once per
// device, while that device is current.
static float* g_attn_static_ptr[64] = {};

static int attn_static_scratch(blum_ctx* ctx, float** out) {
    BLUM_REQUIRE(ctx, ctx->device >= 0 && ctx->device < 64, "static attention scratch: device index %d not supported", ctx->device);
    if (!g_attn_static_ptr[ctx->device]) {
        // the lookup answers for the CURRENT device: make the context's device current for it and put the caller's back
        int prev = -1;
        BLUM_CUDA(ctx, cudaGetDevice(&prev));
        if (prev != ctx->device) BLUM_CUDA(ctx, cudaSetDevice(ctx->device));
        float* ptr = nullptr;
        const cudaError_t e = cudaGetSymbolAddress((void**)&ptr, g_attn_static_scratch);
        if (prev != ctx->device) cudaSetDevice(prev);
        if (e != cudaSuccess || !ptr)
            return blum_fail(ctx, BLUM_ERR_CUDA, "static attention scratch: cudaGetSymbolAddress failed on device %d: %s", ctx->device,
                             cudaGetErrorString(e));
        g_attn_static_ptr[ctx->device] = ptr;
    }
    *out = g_attn_static_ptr[ctx->device];
    return BLUM_OK;
}

extern "C" {

size_t blum_attn_decode_static_scratch_bytes(void) { return (size_t)BLUM_ATTN_STATIC_FLOATS * sizeof(float); }

int blum_attn_decode_paged_static(blum_ctx* ctx, blum_kv* kv, int layer, const void* q, blum_dtype dtype, int q_heads,
                                  const int32_t* seq_ids, const int32_t* ctx_lens, int64_t B, int max_splits, void* out) {
    if (!ctx) return BLUM_ERR_INVALID;
    BLUM_REQUIRE(ctx, kv != nullptr, "attention (static scratch): null kv");
    const size_t need = blum_attn_decode_scratch_bytes(B, q_heads, kv->head_dim, max_splits);
    if (need > blum_attn_decode_static_scratch_bytes())
        return blum_fail(ctx, BLUM_ERR_INVALID,
                         "attention (static scratch): B=%lld x q_heads=%d x splits=%d needs %zu bytes of scratch, the built-in "
                         "buffer holds %zu; lower max_splits or use blum_attn_decode_paged with your own scratch",
                         (long long)B, q_heads, max_splits, need, blum_attn_decode_static_scratch_bytes());
    float* scratch = nullptr;
    int rc = attn_static_scratch(ctx, &scratch);
    if (rc) return rc;
    // every split writes its whole (max, sum, out) record, so nothing left by an earlier call is read
    return blum_attn_rows(ctx, kv, layer, q, dtype, q_heads, seq_ids, ctx_lens, B, max_splits, scratch, out);
}

int blum_attn_prefill_paged(blum_ctx* ctx, blum_kv* kv, int layer, const void* q, blum_dtype dtype, int q_heads, int seq,
                            int64_t p, int64_t T, void* out) {
    if (!ctx) return BLUM_ERR_INVALID;
    BLUM_REQUIRE(ctx, kv != nullptr, "attention prefill: null kv");
    BLUM_REQUIRE(ctx, T >= 0 && T < 65536 && p >= 0, "attention prefill: bad range");
    if (T == 0) return BLUM_OK;
    if (seq < 0 || seq >= kv->max_seqs || kv->seq_len[seq] < p + T)
        return blum_fail(ctx, BLUM_ERR_STATE, "attention prefill: sequence %d does not hold %lld tokens", seq, (long long)(p + T));
    if (q_heads > 0 && q_heads % kv->kv_heads == 0 && blum_attn_prefill_mma_covers(dtype, kv->dtype, kv->head_dim, kv->page_size))
        return blum_attn_prefill_mma(ctx, kv, layer, q, dtype, q_heads, seq, p, T, out);
    int32_t* rows = nullptr;
    BLUM_CUDA(ctx, cudaMallocAsync((void**)&rows, (size_t)2 * T * sizeof(int32_t), ctx->stream));
    prefill_rows_kernel<<<(unsigned)((T + 255) / 256), 256, 0, ctx->stream>>>(rows, rows + T, seq, (int)p, (int)T);
    int rc = BLUM_OK;
    if (cudaGetLastError() != cudaSuccess) rc = blum_fail(ctx, BLUM_ERR_CUDA, "attention prefill: launch failed");
    else ctx->launches++;
    if (!rc) rc = blum_attn_rows(ctx, kv, layer, q, dtype, q_heads, rows, rows + T, T, 1, nullptr, out);
    cudaFreeAsync(rows, ctx->stream);
    return rc;
}

}  // extern "C"
