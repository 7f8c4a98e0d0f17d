// Decode-step attention fused with RoPE and the KV append: one launch per layer.
//
// Per layer the reference runs RoPE on q and k as generated elementwise kernels, rebuilds the whole K/V cache
// tensors to append one row (examples/llama/src/model.rs:104-110,140 in luminal), materialises the GQA-expanded
// K/V, then cuBLAS QK^T, scale+mask, CudaSoftmax and cuBLAS PV (model.rs:113-136).  Here a CTA owns one
// (sequence, kv head, split): it rotates its q heads and (split 0) the new k, writes the new k/v row into its page
// slot, and attends over the cached positions plus the new token, whose k/v it already holds in shared memory.
// K/V tiles are staged in shared memory with cp.async, double buffered; the first tile (which depends only on
// data older than the previous kernel) is requested before the programmatic-dependent-launch wait, so the
// kernel's latency after q/k/v arrive is a couple of memory round trips instead of one per position.
// Algorithmic bytes per (sequence, layer): 2*kv_heads*head_dim*ctx*sizeof(kv) read + one k/v row written.
#include "attn_decode.cuh"
#include <stdlib.h>

template <typename TC> __device__ __forceinline__ void ld8(const TC* p, float* o);
template <> __device__ __forceinline__ void ld8<float>(const float* p, float* o) {
    const float4 a = *reinterpret_cast<const float4*>(p), b = *reinterpret_cast<const float4*>(p + 4);
    o[0] = a.x; o[1] = a.y; o[2] = a.z; o[3] = a.w; o[4] = b.x; o[5] = b.y; o[6] = b.z; o[7] = b.w;
}
template <> __device__ __forceinline__ void ld8<__nv_bfloat16>(const __nv_bfloat16* p, float* o) {
    const uint4 v = *reinterpret_cast<const uint4*>(p);
    const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
    for (int i = 0; i < 4; i++) { o[2 * i] = __uint_as_float(w[i] << 16); o[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u); }
}
template <> __device__ __forceinline__ void ld8<__half>(const __half* p, float* o) {
    const uint4 v = *reinterpret_cast<const uint4*>(p);
    const __half2* h = reinterpret_cast<const __half2*>(&v);
#pragma unroll
    for (int i = 0; i < 4; i++) { o[2 * i] = __low2float(h[i]); o[2 * i + 1] = __high2float(h[i]); }
}

// grid (splits, kv_heads, rows); block D threads
template <typename TS, typename TC, int G, int D>
__global__ void __launch_bounds__(D) attn_decode_fused_kernel(const FusedAttnParams p) {
    constexpr int TILE = D / 2;
    constexpr int QPAD = D / 2 + 4;
    constexpr int ROWB = attn_row_bytes<TC, D>();      // padded row: consecutive rows start in different banks
    constexpr int CPR = D * (int)sizeof(TC) / 16;      // 16-byte chunks per row
    extern __shared__ __align__(16) unsigned char tiles[];   // [2 buffers][K|V][TILE][ROWB]
    __shared__ __align__(16) float qs[G][2][QPAD];
    __shared__ __align__(16) float knew[D], vnew[D];
    __shared__ float sc[G][TILE];
    __shared__ float corr[G];
    __shared__ int32_t pages[2][TILE];                 // page ids of the tile in each buffer

    blum_trace(p.trace, 0);
    pdl_launch_dependents();
    const int split = blockIdx.x, nsplit = gridDim.x, kvh = blockIdx.y, row = blockIdx.z;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    constexpr int NW = D / 32;
    const KvView& kv = p.kv;
    const int ps = kv.page_size, nkv = kv.kv_heads;

    // Everything up to the dependency wait reads only data that is older than the previous kernel: sequence id,
    // length, page table and the cached K/V rows.  The first tile is already on its way when q/k/v arrive.
    int seq = p.seq_ids[row];
    int ctx = p.ctx_lens[row];
    if (seq < 0 || seq >= p.max_seqs || ctx < 1 || (ctx + ps - 1) / ps > kv.max_pages_per_seq) {
        if (tid == 0) atomicOr(p.err, 0x100);
        seq = 0; ctx = 1;
    }
    const int pos = ctx - 1;                           // position of the new token
    const int32_t* table = kv.table + (int64_t)seq * kv.max_pages_per_seq;
    TC* pool = reinterpret_cast<TC*>(kv.pool);

    // cached positions [0, pos) split on page boundaries
    const int npages = (pos + ps - 1) / ps;
    const int pages_per_split = (npages + nsplit - 1) / nsplit;
    const int c0 = min(pos, split * pages_per_split * ps);
    const int c1 = min(pos, (split + 1) * pages_per_split * ps);
    const int ntiles = (c1 - c0 + TILE - 1) / TILE;

    // issues the copies of tile `t` into buffer `t & 1` (page ids first, then 16-byte chunks of K and V rows)
    auto load_pages = [&](int t) {
        const int t0 = c0 + t * TILE, tile_n = min(TILE, c1 - t0);
        const int first_pg = t0 / ps, n_pg = (t0 + tile_n - 1) / ps - first_pg + 1;
        if (tid < n_pg) {
            int32_t page = table[first_pg + tid];
            if (page < 0 || page >= kv.num_pages) { atomicOr(p.err, 0x200); page = 0; }
            pages[t & 1][tid] = page;
        }
    };
    auto issue_tile = [&](int t) {
        const int t0 = c0 + t * TILE, tile_n = min(TILE, c1 - t0);
        const int first_pg = t0 / ps;
        unsigned char* kb = tiles + (size_t)(t & 1) * 2 * TILE * ROWB;
        unsigned char* vb = kb + (size_t)TILE * ROWB;
        for (int i = tid; i < tile_n * CPR; i += D) {
            const int j = i / CPR, c = i % CPR, posj = t0 + j;
            const int32_t page = pages[t & 1][posj / ps - first_pg];
            const unsigned char* ksrc = reinterpret_cast<const unsigned char*>(pool + kv_tile_offset(kv, p.layer, page, 0, kvh, posj % ps));
            const unsigned char* vsrc = reinterpret_cast<const unsigned char*>(pool + kv_tile_offset(kv, p.layer, page, 1, kvh, posj % ps));
            cp_async_16(kb + (size_t)j * ROWB + c * 16, ksrc + c * 16);
            cp_async_16(vb + (size_t)j * ROWB + c * 16, vsrc + c * 16);
        }
        cp_async_commit();
    };
    if (ntiles > 0) { load_pages(0); __syncthreads(); issue_tile(0); }

    // rotation angles and the append slot depend only on the position: compute them before the wait as well
    constexpr int NPAIR = ((G + 1) * (D / 2) + D - 1) / D;
    float rsn[NPAIR], rcs[NPAIR];
#pragma unroll
    for (int it = 0; it < NPAIR; it++) {
        const int pi = (tid + it * D) % (D / 2);
        const float a = (float)pos * p.freqs.inv_freq[pi];
        rsn[it] = sinf(a); rcs[it] = sinf(1.5707964f - a);          // cos(x) = sin(pi/2 - x), as the reference computes it
    }
    const int32_t new_page = (split == 0) ? table[pos / ps] : 0;

    pdl_wait();
    blum_trace(p.trace, 1);

    // ---- RoPE of this kv head's q heads and (for the new row) k; v is copied
    const TS* rowp = reinterpret_cast<const TS*>(p.qkv) + (int64_t)row * (p.nq + 2 * nkv) * D;
#pragma unroll
    for (int it = 0; it < NPAIR; it++) {
        const int i = tid + it * D;
        if (i < (G + 1) * (D / 2)) {
            const int h = i / (D / 2), pi = i % (D / 2);
            const TS* src = (h < G) ? rowp + ((int64_t)kvh * G + h) * D : rowp + ((int64_t)p.nq + kvh) * D;
            const float sn = rsn[it], cs = rcs[it];
            const float x0 = to_f32<TS>(src[2 * pi]), x1 = to_f32<TS>(src[2 * pi + 1]);
            // every value is rounded to the activation type where the reference's op output would be
            const float r0 = to_f32<TS>(from_f32<TS>(x0 * cs - x1 * sn)), r1 = to_f32<TS>(from_f32<TS>(x0 * sn + x1 * cs));
            if (h < G) {
                const int e0 = 2 * pi, e1 = 2 * pi + 1;
                qs[h][e0 / (D / 2)][e0 % (D / 2)] = r0;
                qs[h][e1 / (D / 2)][e1 % (D / 2)] = r1;
            } else {
                knew[2 * pi] = to_f32<TC>(from_f32<TC>(r0));
                knew[2 * pi + 1] = to_f32<TC>(from_f32<TC>(r1));
            }
        }
    }
    vnew[tid] = to_f32<TC>(from_f32<TC>(to_f32<TS>(rowp[((int64_t)p.nq + nkv + kvh) * D + tid])));
    __syncthreads();
    if (split == 0) {   // append the new row to its page slot
        if (new_page < 0 || new_page >= kv.num_pages) { if (tid == 0) atomicOr(p.err, 0x40); }
        else {
            pool[kv_tile_offset(kv, p.layer, new_page, 0, kvh, pos % ps) + tid] = from_f32<TC>(knew[tid]);
            pool[kv_tile_offset(kv, p.layer, new_page, 1, kvh, pos % ps) + tid] = from_f32<TC>(vnew[tid]);
        }
    }
    blum_trace(p.trace, 2);

    float m_run[G], l_run[G], o_acc[G];
#pragma unroll
    for (int g = 0; g < G; g++) { m_run[g] = -INFINITY; l_run[g] = 0.f; o_acc[g] = 0.f; }

    const int jj = tid >> 1, half = tid & 1;
    for (int t = 0; t < ntiles; t++) {
        const int t0 = c0 + t * TILE, tile_n = min(TILE, c1 - t0);
        // next tile: its page ids now, its copies after the barrier below (the buffer it uses was last read in tile t-1)
        if (t + 1 < ntiles) load_pages(t + 1);
        __syncthreads();
        if (t + 1 < ntiles) { issue_tile(t + 1); cp_async_wait<1>(); } else { cp_async_wait<0>(); }
        __syncthreads();
        const unsigned char* kb = tiles + (size_t)(t & 1) * 2 * TILE * ROWB;
        const unsigned char* vb = kb + (size_t)TILE * ROWB;
        {   // scores: two threads per position, D/2 dims each
            float acc[G];
#pragma unroll
            for (int g = 0; g < G; g++) acc[g] = 0.f;
            if (jj < tile_n) {
                const TC* kr = reinterpret_cast<const TC*>(kb + (size_t)jj * ROWB) + half * (D / 2);
#pragma unroll
                for (int c = 0; c < D / 2; c += 8) {
                    float kvv[8];
                    ld8<TC>(kr + c, kvv);
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
                if (half == 0) sc[g][jj] = (jj < tile_n) ? s * p.scale : -INFINITY;
            }
        }
        __syncthreads();
#pragma unroll
        for (int g = 0; g < G; g++) {
            if (g % NW == warp) {
                float mx = -INFINITY;
                for (int j = lane; j < TILE; j += 32) mx = fmaxf(mx, sc[g][j]);
                mx = warp_max(mx);
                const float m_new = fmaxf(m_run[g], mx);
                for (int j = lane; j < TILE; j += 32) sc[g][j] = exp2f((sc[g][j] - m_new) * LOG2E);
                if (lane == 0) corr[g] = m_new;
            }
        }
        __syncthreads();
#pragma unroll
        for (int g = 0; g < G; g++) {
            const float m_new = corr[g];
            const float c = (m_run[g] == -INFINITY) ? 0.f : exp2f((m_run[g] - m_new) * LOG2E);
            l_run[g] *= c; o_acc[g] *= c; m_run[g] = m_new;
        }
        for (int j = 0; j < tile_n; j++) {
            const float vv = to_f32<TC>(reinterpret_cast<const TC*>(vb + (size_t)j * ROWB)[tid]);
#pragma unroll
            for (int g = 0; g < G; g++) {
                const float pj = sc[g][j];
                l_run[g] += pj;
                o_acc[g] = fmaf(pj, vv, o_acc[g]);
            }
        }
    }
    __syncthreads();

    // ---- the new token itself (split 0): score from shared memory
    if (split == 0) {
        float part[G];
#pragma unroll
        for (int g = 0; g < G; g++) part[g] = qs[g][tid / (D / 2)][tid % (D / 2)] * knew[tid];
#pragma unroll
        for (int g = 0; g < G; g++) {
            const float s = warp_sum(part[g]);
            if (lane == 0) sc[g][warp] = s;
        }
        __syncthreads();
#pragma unroll
        for (int g = 0; g < G; g++) {
            float s = 0.f;
#pragma unroll
            for (int w = 0; w < NW; w++) s += sc[g][w];
            s *= p.scale;
            const float m_new = fmaxf(m_run[g], s);
            const float c = (m_run[g] == -INFINITY) ? 0.f : exp2f((m_run[g] - m_new) * LOG2E);
            const float pj = exp2f((s - m_new) * LOG2E);
            l_run[g] = l_run[g] * c + pj;
            o_acc[g] = fmaf(pj, vnew[tid], o_acc[g] * c);
            m_run[g] = m_new;
        }
    }

#pragma unroll
    for (int g = 0; g < G; g++) {
        const int h = kvh * G + g;
        if (nsplit == 1) {
            const float inv = l_run[g] > 0.f ? 1.f / l_run[g] : 0.f;
            reinterpret_cast<TS*>(p.out)[((int64_t)row * p.nq + h) * D + tid] = from_f32<TS>(o_acc[g] * inv);
        } else {
            const int64_t base = ((int64_t)row * p.nq + h) * nsplit + split;
            p.part_o[base * D + tid] = o_acc[g];
            if (tid == 0) { p.part_ml[base * 2] = m_run[g]; p.part_ml[base * 2 + 1] = l_run[g]; }
        }
    }
    blum_trace(p.trace, 3);
}

int blum_attn_combine(blum_ctx* ctx, const float* part_o, const float* part_ml, int nq, int nsplit, int rows, int head_dim,
                      void* out, int dtype);

template <typename TS, typename TC, int G, int D>
static int launch_fused(blum_ctx* ctx, const FusedAttnParams& p, int rows, int nsplit) {
    cudaLaunchConfig_t cfg = {};
    constexpr int smem = attn_smem_bytes<TC, D>();
    auto kern = attn_decode_fused_kernel<TS, TC, G, D>;
    if (smem + 8192 > 48 * 1024) BLUM_CUDA(ctx, cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
    cfg.gridDim = dim3(nsplit, p.kv.kv_heads, rows); cfg.blockDim = dim3(D); cfg.dynamicSmemBytes = smem; cfg.stream = ctx->stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = ctx->pdl ? 1 : 0;
    cfg.attrs = attr; cfg.numAttrs = 1;
    BLUM_CUDA(ctx, cudaLaunchKernelEx(&cfg, kern, p));
    ctx->launches++;
    return BLUM_OK;
}

template <typename TS, typename TC>
static int launch_fused_gd(blum_ctx* ctx, const FusedAttnParams& p, int rows, int nsplit, int g, int d) {
#define GD(gg, dd) if (g == gg && d == dd) return launch_fused<TS, TC, gg, dd>(ctx, p, rows, nsplit)
    GD(1, 128); GD(2, 128); GD(4, 128); GD(8, 128);
    GD(1, 64);  GD(2, 64);  GD(4, 64);  GD(8, 64);
#undef GD
    return blum_fail(ctx, BLUM_ERR_INVALID, "fused decode attention: unsupported group size %d / head_dim %d", g, d);
}

// RoPE + KV append + attention for one new token per row.  The sequences must already be extended to hold the
// new position (ctx_lens[b] - 1) and the page table synchronised.
int blum_attn_decode_fused(blum_ctx* ctx, blum_kv* kv, int layer, const void* qkv, int dtype, int q_heads, float theta,
                           const int32_t* seq_ids, const int32_t* ctx_lens, int64_t rows, int nsplit, void* scratch, void* out) {
    BLUM_REQUIRE(ctx, kv && qkv && out && seq_ids && ctx_lens, "fused decode attention: null argument");
    BLUM_REQUIRE(ctx, layer >= 0 && layer < kv->layers, "fused decode attention: layer %d outside [0,%d)", layer, kv->layers);
    BLUM_REQUIRE(ctx, q_heads > 0 && q_heads % kv->kv_heads == 0, "fused decode attention: q_heads %d not a multiple of kv_heads %d",
                 q_heads, kv->kv_heads);
    BLUM_REQUIRE(ctx, rows >= 0 && rows < 65536, "fused decode attention: too many rows");
    if (rows == 0) return BLUM_OK;
    if (nsplit < 1) nsplit = 1;
    BLUM_REQUIRE(ctx, nsplit == 1 || scratch, "fused decode attention: split decode needs a scratch buffer");
    int rc = blum_kv_sync_tables(ctx, kv);
    if (rc) return rc;
    FusedAttnParams p;
    p.kv = kv_view(kv); p.layer = layer; p.max_seqs = kv->max_seqs;
    p.qkv = qkv; p.out = out; p.seq_ids = seq_ids; p.ctx_lens = ctx_lens; p.nq = q_heads;
    p.scale = 1.0f / sqrtf((float)kv->head_dim);
    blum_rope_freqs(theta, kv->head_dim, &p.freqs);
    p.err = ctx->dev_error;
    p.trace = blum_trace_slot(ctx);
    p.part_o = (float*)scratch;
    p.part_ml = p.part_o ? p.part_o + (size_t)rows * q_heads * nsplit * kv->head_dim : nullptr;
    const int g = q_heads / kv->kv_heads, d = kv->head_dim;
    if (blum_attn_decode_mma_covers(dtype, kv->dtype, g, d, kv->page_size)) rc = blum_attn_decode_mma_launch(ctx, p, dtype, (int)rows, nsplit, g, d);
    else if (dtype == BLUM_F32 && kv->dtype == BLUM_F32) rc = launch_fused_gd<float, float>(ctx, p, (int)rows, nsplit, g, d);
    else if (dtype == BLUM_BF16 && kv->dtype == BLUM_BF16) rc = launch_fused_gd<__nv_bfloat16, __nv_bfloat16>(ctx, p, (int)rows, nsplit, g, d);
    else if (dtype == BLUM_F16 && kv->dtype == BLUM_F16) rc = launch_fused_gd<__half, __half>(ctx, p, (int)rows, nsplit, g, d);
    else if (dtype == BLUM_F32 && kv->dtype == BLUM_BF16) rc = launch_fused_gd<float, __nv_bfloat16>(ctx, p, (int)rows, nsplit, g, d);
    else return blum_fail(ctx, BLUM_ERR_INVALID, "fused decode attention: unsupported dtype pair (%d,%d)", dtype, kv->dtype);
    if (rc) return rc;
    if (nsplit > 1) return blum_attn_combine(ctx, p.part_o, p.part_ml, q_heads, nsplit, (int)rows, d, out, dtype);
    return BLUM_OK;
}

extern "C" int blum_rope_attn_decode_paged(blum_ctx* ctx, blum_kv* kv, int layer, const void* qkv, blum_dtype dtype, int q_heads,
                                           float theta, const int32_t* seq_ids, const int32_t* ctx_lens, int64_t B,
                                           int max_splits, void* scratch, void* out) {
    if (!ctx) return BLUM_ERR_INVALID;
    return blum_attn_decode_fused(ctx, kv, layer, qkv, dtype, q_heads, theta, seq_ids, ctx_lens, B, max_splits, scratch, out);
}
