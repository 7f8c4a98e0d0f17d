// One decode step of the Llama decoder (batch 1, f32 activations and KV cache) as ONE persistent kernel with a
// continuous weight stream.
//
// The reference executes a decode step as ~10^3 graph nodes, one allocation and one launch each
// (src/graph.rs:191-224 in luminal), the quantised matmuls as one 64-thread-block matvec launch per projection
// (crates/luminal_cuda/src/quantized.rs:28-109,116-168).  A batch-1 step is bound by reading the 8 GB of Q8_0
// weights once; every kernel boundary, dependency wait and re-staging of x is time with no weight bytes in flight.
// Here the weights of the whole step are one statically ordered stream:
//   * grid = one CTA per SM (cooperative launch, so all CTAs are co-resident); per matrix every CTA owns one
//     contiguous range of 8.5 KB units (16 rows x 512 k, repacked once at load so that a unit is contiguous in
//     HBM and already in the register layout of the MMA operand);
//   * warp 0 is the producer: one elected thread issues cp.async.bulk copies of consecutive units into a ring of
//     shared-memory stages (mbarrier complete_tx), limited only by free stages - it runs ahead across phase
//     boundaries, so HBM keeps streaming while the compute warps sit in a grid barrier, stage x or run attention;
//   * warps 1-8 consume: x is staged once per phase per CTA as block fixed point (per 32-element block
//     x_i = xfix_i * 2^(e-21), |xfix_i| <= 2^22, split into three signed byte planes), so that the dot product of
//     a Q8_0 block with x is exact integer arithmetic on the legacy tensor path: one mma.sync.m16n8k32.s8 covers
//     16 rows x one block, the three planes of x are three columns of B (k is permuted inside a block so that
//     both operands are plain 8/16-byte shared-memory loads); per (row, block): acc_plane += float(int) * (d * 2^e),
//     result = 65536 acc_0 + 256 acc_1 + acc_2 - the block-sum-times-block-scale order of the reference kernel;
//   * phases of a layer: [RMSNorm + q/k/v] -> [RoPE + KV append + attention] -> [o_proj + residual] ->
//     [RMSNorm + gate/up + SwiGLU] -> [down + residual]; after the last layer [RMSNorm + LM head].  Phases are
//     separated by grid barriers (monotonic 64-bit counter, bounded spin); a 16-row group whose k-range is cut by
//     a CTA boundary is finished by the CTA that holds its first slice, which adds the partial sums the later
//     CTAs publish (flag + bounded wait; the later CTAs reach those slices first, so the wait is normally over
//     before it starts); all sums run in a fixed order, so results are reproducible bit for bit.
// Every wait is bounded by wall-clock time; on expiry the CTA raises the abort word, every later wait in the grid
// becomes a no-op, the error word is set and the producer waits for its copies in flight before the CTA exits.
// Algorithmic bytes per launch: all Q8_0 weights of the model once (N*K*34/32 each) + the KV rows of the context.
#include "decode_stream.cuh"
#include <cooperative_groups.h>

#define DS_TIMEOUT_NS 2000000000ull       // every wait gives up after 2 s
#define LOG2E 1.4426950408889634f

__device__ __forceinline__ uint32_t ds_smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void ds_mbar_init(uint64_t* bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(ds_smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void ds_mbar_arrive(uint64_t* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(ds_smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void ds_mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(ds_smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool ds_mbar_try(uint64_t* bar, uint32_t parity) {
    uint32_t ok;
    asm volatile("{\n\t.reg .pred q;\n\tmbarrier.try_wait.parity.shared::cta.b64 q, [%1], %2;\n\tselp.u32 %0, 1, 0, q;\n\t}"
                 : "=r"(ok) : "r"(ds_smem_u32(bar)), "r"(parity) : "memory");
    return ok != 0;
}
__device__ __forceinline__ void ds_bulk_load(void* dst, const void* src, uint32_t bytes, uint64_t* bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(ds_smem_u32(dst)), "l"(src), "r"(bytes), "r"(ds_smem_u32(bar)) : "memory");
}
__device__ __forceinline__ unsigned long long ds_ld_acquire(const unsigned long long* p) {
    unsigned long long v;
    asm volatile("ld.acquire.gpu.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ void ds_st_release(unsigned long long* p, unsigned long long v) {
    asm volatile("st.release.gpu.global.u64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
}
__device__ __forceinline__ void ds_named_sync() { asm volatile("bar.sync 1, %0;" ::"n"(DS_CONSUMER_THREADS) : "memory"); }

// records a timeout: error word for the host, abort word for every other CTA, abort flag for this CTA
__device__ __noinline__ void ds_give_up(int* err, unsigned long long* ctr, volatile int* s_abort) {
    *s_abort = 1;
    atomicOr(err, 0x400);
    atomicExch(ctr + 2, 1ull);
}
__device__ __forceinline__ bool ds_aborted(const DsParams& p, volatile int* s_abort) {
    if (*s_abort) return true;
    if (*reinterpret_cast<volatile unsigned long long*>(p.ctr + 2) != 0ull) { *s_abort = 1; return true; }
    return false;
}
// bounded wait on an mbarrier phase; a no-op once the grid has aborted
__device__ __forceinline__ void ds_mbar_wait(uint64_t* bar, uint32_t parity, const DsParams& p, volatile int* s_abort) {
    if (*s_abort) return;
    if (ds_mbar_try(bar, parity)) return;
    const unsigned long long t0 = blum_globaltimer();
    for (uint32_t spin = 1;; spin++) {
        if (ds_mbar_try(bar, parity)) return;
        if ((spin & 63u) == 0u) {
            if (ds_aborted(p, s_abort)) return;
            if (blum_globaltimer() - t0 > DS_TIMEOUT_NS) { ds_give_up(p.err, p.ctr, s_abort); return; }
        }
    }
}
// bounded wait until *word >= target (acquire)
__device__ __forceinline__ void ds_wait_ge(const unsigned long long* word, unsigned long long target, const DsParams& p,
                                           volatile int* s_abort) {
    if (*s_abort) return;
    if (ds_ld_acquire(word) >= target) return;
    const unsigned long long t0 = blum_globaltimer();
    for (uint32_t spin = 1;; spin++) {
        if (ds_ld_acquire(word) >= target) return;
        if (spin > 16u) __nanosleep(32);
        if ((spin & 63u) == 0u) {
            if (ds_aborted(p, s_abort)) return;
            if (blum_globaltimer() - t0 > DS_TIMEOUT_NS) { ds_give_up(p.err, p.ctr, s_abort); return; }
        }
    }
}

// grid barrier of the compute warps (the producer warp does not take part: its schedule is static)
__device__ __forceinline__ void ds_grid_sync(const DsParams& p, unsigned long long target, int tid_c, volatile int* s_abort) {
    ds_named_sync();
    if (tid_c == 0 && !*s_abort) {
        __threadfence();
        atomicAdd(p.ctr, 1ull);
        ds_wait_ge(p.ctr, target, p, s_abort);
        __threadfence();
    }
    ds_named_sync();
}

__device__ __forceinline__ float4 ds_ldcg4(const float* p) { return __ldcg(reinterpret_cast<const float4*>(p)); }

struct DsShared {
    uint64_t full[DS_MAX_STAGES], empty[DS_MAX_STAGES];
    float4 red[2][DS_CONSUMER_WARPS][32];           // cross-warp reduction of a group segment, double buffered
    float wred[DS_CONSUMER_WARPS];                  // sum of squares per warp
    float q[128], knew[128], vnew[128];
    float sc[DS_ATTN_TILE];
    long long koff[DS_ATTN_TILE];
    float o_half[2][128];
    float l_half[2];
    unsigned long long seq;
    int abort;
};

// ---- x of a phase -> block fixed point in shared memory (three signed byte planes + one scale per 32 elements)
// planes: [K/32][3][32] bytes; scales: [K/32] floats.  Returns rsqrt(mean(x^2) + eps) when a norm weight is folded in.
__device__ __forceinline__ float ds_stage_x(const DsParams& p, const DsPhase& P, DsShared& sh, unsigned char* xpl, float* xsc,
                                            int tid_c, int cta) {
    const int K = P.K, lane = tid_c & 31, cw = tid_c >> 5;
    const float* src;
    bool copy_to_xres = false;
    if (P.kind == DS_QKV) {
        if (P.layer == 0) {
            int id = p.rows[0];
            if (id < 0 || id >= p.vocab) { if (tid_c == 0) atomicOr(p.err, 0x100); id = 0; }
            src = p.embed + (size_t)id * p.H;
            copy_to_xres = (cta == 0);
        } else src = p.xres;
    } else if (P.kind == DS_O) src = p.attn;
    else if (P.kind == DS_DOWN) src = p.mid;
    else src = p.xres;
    const bool combine = (P.kind == DS_O) && p.nsplit > 1;
    float ss = 0.f;
    // one step of four consecutive elements: norm weight, block maximum over the 8 lanes of a 32-element block, digits
    auto put = [&](float (&v)[4], int k) {
        if (copy_to_xres) *reinterpret_cast<float4*>(p.xres + k) = make_float4(v[0], v[1], v[2], v[3]);
        ss += v[0] * v[0] + v[1] * v[1] + v[2] * v[2] + v[3] * v[3];
        if (P.norm_w) {
            const float4 nw = __ldg(reinterpret_cast<const float4*>(P.norm_w + k));
            v[0] *= nw.x; v[1] *= nw.y; v[2] *= nw.z; v[3] *= nw.w;
        }
        float mx = fmaxf(fmaxf(fabsf(v[0]), fabsf(v[1])), fmaxf(fabsf(v[2]), fabsf(v[3])));
        mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
        mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
        mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 4));     // 8 lanes x 4 = one 32-element block
        const int E = (int)((__float_as_uint(mx) >> 23) & 0xffu);
        // xfix = x * 2^(21 - (E-127)); blocks whose maximum is below 2^-105 count as zero; a non-finite block poisons its sums
        const float up = (E >= 22 && E < 255) ? __uint_as_float((unsigned)(275 - E) << 23) : 0.f;
        const float down = (E == 255) ? __uint_as_float(0x7fc00000u) : (E >= 22 ? __uint_as_float((unsigned)(E - 21) << 23) : 0.f);
        unsigned pa = 0, pb = 0, pc = 0;
#pragma unroll
        for (int i = 0; i < 4; i++) {
            const int xf = __float2int_rn(v[i] * up);
            const int lo = (int)(signed char)(xf & 0xff);          // balanced digits: all three planes are signed bytes
            const int x1 = (xf - lo) >> 8;
            const int mi = (int)(signed char)(x1 & 0xff);
            const int hi = (x1 - mi) >> 8;
            pa |= ((unsigned)hi & 0xffu) << (8 * i);
            pb |= ((unsigned)mi & 0xffu) << (8 * i);
            pc |= ((unsigned)lo & 0xffu) << (8 * i);
        }
        unsigned char* blk = xpl + (size_t)(k >> 5) * 96 + (k & 31);
        *reinterpret_cast<unsigned*>(blk) = pa;
        *reinterpret_cast<unsigned*>(blk + 32) = pb;
        *reinterpret_cast<unsigned*>(blk + 64) = pc;
        if ((k & 31) == 0) xsc[k >> 5] = down;
    };
    if (!combine) {
        constexpr int STEP = DS_CONSUMER_THREADS * 4;
        for (int k0 = tid_c * 4; k0 < K; k0 += STEP * 8) {       // the loads of eight steps are in flight together
            float4 buf[8];
#pragma unroll
            for (int i = 0; i < 8; i++) if (k0 + i * STEP < K) buf[i] = ds_ldcg4(src + k0 + i * STEP);
#pragma unroll
            for (int i = 0; i < 8; i++) {
                if (k0 + i * STEP < K) {
                    float v[4] = {buf[i].x, buf[i].y, buf[i].z, buf[i].w};
                    put(v, k0 + i * STEP);
                }
            }
        }
    } else {
        for (int k = tid_c * 4; k < K; k += DS_CONSUMER_THREADS * 4) {
            // merge the split attention partials of head k/128: weights exp2((m_s - m_max) log2 e)
            const int h = k >> 7, c = k & 127;
            const float* base = p.attn_part + (size_t)h * p.nsplit * 130;
            float mmax = -INFINITY;
            for (int s = 0; s < p.nsplit; s++) mmax = fmaxf(mmax, __ldcg(base + s * 130 + 128));
            float den = 0.f;
            float v[4] = {0.f, 0.f, 0.f, 0.f};
            for (int s = 0; s < p.nsplit; s++) {
                const float ms = __ldcg(base + s * 130 + 128);
                const float w = (ms == -INFINITY) ? 0.f : exp2f((ms - mmax) * LOG2E);
                den = fmaf(__ldcg(base + s * 130 + 129), w, den);
                const float2 o01 = __ldcg(reinterpret_cast<const float2*>(base + s * 130 + c));
                const float2 o23 = __ldcg(reinterpret_cast<const float2*>(base + s * 130 + c + 2));
                v[0] = fmaf(o01.x, w, v[0]); v[1] = fmaf(o01.y, w, v[1]); v[2] = fmaf(o23.x, w, v[2]); v[3] = fmaf(o23.y, w, v[3]);
            }
            const float inv = den > 0.f ? 1.f / den : 0.f;
#pragma unroll
            for (int i = 0; i < 4; i++) v[i] *= inv;
            put(v, k);
        }
    }
    if (P.norm_w) {
        ss = warp_sum(ss);
        if (lane == 0) sh.wred[cw] = ss;
    }
    ds_named_sync();
    float rs = 1.f;
    if (P.norm_w) {
        float s = 0.f;
#pragma unroll
        for (int w = 0; w < DS_CONSUMER_WARPS; w++) s += sh.wred[w];
        rs = rsqrtf(s / (float)K + p.eps);
    }
    return rs;
}

// ---- RoPE + KV append + attention of the new token; items (q head, split) are dealt round robin to the CTAs
__device__ __forceinline__ void ds_attention(const DsParams& p, int layer, DsShared& sh, int tid_c, int cta, int ncta,
                                             volatile int* s_abort) {
    const int lane = tid_c & 31, cw = tid_c >> 5;
    const KvView& kv = p.kv;
    const int ps = kv.page_size, G = p.nq / p.nkv;
    int seq = p.rows[p.max_rows], ctx = p.rows[3 * p.max_rows];
    if (seq < 0 || seq >= p.max_seqs || ctx < 1 || (ctx + ps - 1) / ps > kv.max_pages_per_seq) {
        if (tid_c == 0) atomicOr(p.err, 0x100);
        seq = 0; ctx = 1;
    }
    const int pos = ctx - 1;
    const int32_t* table = kv.table + (size_t)seq * kv.max_pages_per_seq;
    float* pool = reinterpret_cast<float*>(kv.pool);
    const long long vdelta = (long long)kv.kv_heads * ps * 128;       // K tile -> V tile of the same (page, head)
    const int hh = tid_c >> 7, c = tid_c & 127;
    const int nitems = p.nq * p.nsplit;
    for (int item = cta; item < nitems; item += ncta) {
        const int h = item % p.nq, split = item / p.nq, kvh = h / G;
        // rotary embedding of q (threads 0..63) and of the new k (64..127); v is copied (128..255)
        if (tid_c < 128) {
            const int pi = tid_c & 63;
            const float a = (float)pos * p.freqs.inv_freq[pi];
            const float sn = sinf(a), cs = sinf(1.5707964f - a);       // cos(x) = sin(pi/2 - x), as the reference computes it
            const float* s2 = p.qkv + (size_t)((tid_c < 64) ? h : p.nq + kvh) * 128 + 2 * pi;
            const float2 x = __ldcg(reinterpret_cast<const float2*>(s2));
            float* dst = (tid_c < 64) ? sh.q : sh.knew;
            dst[2 * pi] = x.x * cs - x.y * sn;
            dst[2 * pi + 1] = x.x * sn + x.y * cs;
        } else {
            sh.vnew[c] = __ldcg(p.qkv + (size_t)(p.nq + p.nkv + kvh) * 128 + c);
        }
        ds_named_sync();
        if (split == 0 && h % G == 0) {     // one item per kv head appends the new row to its page slot
            const int32_t page = table[pos / ps];
            if (page < 0 || page >= kv.num_pages) { if (tid_c == 0) atomicOr(p.err, 0x40); }
            else {
                const long long o = kv_tile_offset(kv, layer, page, 0, kvh, pos % ps);
                if (hh == 0) pool[o + c] = sh.knew[c]; else pool[o + vdelta + c] = sh.vnew[c];
            }
        }
        const float4 q4 = *reinterpret_cast<const float4*>(&sh.q[lane * 4]);
        // cached positions [0, pos) split on page boundaries
        const int npages = (pos + ps - 1) / ps, pages_per_split = (npages + p.nsplit - 1) / p.nsplit;
        const int c0 = min(pos, split * pages_per_split * ps), c1 = min(pos, (split + 1) * pages_per_split * ps);
        float m_run = -INFINITY, l_run = 0.f, o_acc = 0.f;
        for (int t0 = c0; t0 < c1; t0 += DS_ATTN_TILE) {
            const int n = min(DS_ATTN_TILE, c1 - t0);
            if (tid_c < n) {
                const int pj = t0 + tid_c;
                int32_t page = table[pj / ps];
                if (page < 0 || page >= kv.num_pages) { atomicOr(p.err, 0x200); page = 0; }
                sh.koff[tid_c] = kv_tile_offset(kv, layer, page, 0, kvh, pj % ps);
            }
            ds_named_sync();
            for (int j0 = cw; j0 < n; j0 += DS_CONSUMER_WARPS * 4) {       // four independent rows per warp in flight
                float4 kr[4];
#pragma unroll
                for (int i = 0; i < 4; i++) {
                    const int j = j0 + i * DS_CONSUMER_WARPS;
                    kr[i] = (j < n) ? __ldg(reinterpret_cast<const float4*>(pool + sh.koff[j]) + lane) : make_float4(0.f, 0.f, 0.f, 0.f);
                }
#pragma unroll
                for (int i = 0; i < 4; i++) {
                    const int j = j0 + i * DS_CONSUMER_WARPS;
                    const float dot = warp_sum(kr[i].x * q4.x + kr[i].y * q4.y + kr[i].z * q4.z + kr[i].w * q4.w);
                    if (lane == 0 && j < n) sh.sc[j] = dot * p.scale;
                }
            }
            ds_named_sync();
            float mx = -INFINITY;
            for (int j = lane; j < n; j += 32) mx = fmaxf(mx, sh.sc[j]);
            mx = warp_max(mx);
            const float m_new = fmaxf(m_run, mx);
            const float corr = (m_run == -INFINITY) ? 0.f : exp2f((m_run - m_new) * LOG2E);
            ds_named_sync();                                               // every warp has read the raw scores
            if (tid_c < n) sh.sc[tid_c] = exp2f((sh.sc[tid_c] - m_new) * LOG2E);
            ds_named_sync();
            o_acc *= corr; l_run *= corr; m_run = m_new;
#pragma unroll 8
            for (int j = hh; j < n; j += 2) {
                const float pj = sh.sc[j];
                o_acc = fmaf(pj, __ldg(pool + sh.koff[j] + vdelta + c), o_acc);
                l_run += pj;
            }
            ds_named_sync();                                               // sc / koff are rewritten by the next tile
        }
        if (split == 0) {       // the new token itself: its k and v are still in shared memory
            const float4 k4 = *reinterpret_cast<const float4*>(&sh.knew[lane * 4]);
            const float s = warp_sum(k4.x * q4.x + k4.y * q4.y + k4.z * q4.z + k4.w * q4.w) * p.scale;
            const float m_new = fmaxf(m_run, s);
            const float corr = (m_run == -INFINITY) ? 0.f : exp2f((m_run - m_new) * LOG2E);
            const float pj = exp2f((s - m_new) * LOG2E);
            o_acc *= corr; l_run *= corr; m_run = m_new;
            if (hh == 0) { o_acc = fmaf(pj, sh.vnew[c], o_acc); l_run += pj; }
        }
        sh.o_half[hh][c] = o_acc;
        if (c == 0) sh.l_half[hh] = l_run;
        ds_named_sync();
        if (hh == 0) {
            const float o = sh.o_half[0][c] + sh.o_half[1][c], l = sh.l_half[0] + sh.l_half[1];
            if (p.nsplit == 1) p.attn[(size_t)h * 128 + c] = o * (l > 0.f ? 1.f / l : 0.f);
            else {
                float* dst = p.attn_part + ((size_t)h * p.nsplit + split) * 130;
                dst[c] = o;
                if (c == 0) { dst[128] = m_run; dst[129] = l; }
            }
        }
        ds_named_sync();                                                   // shared scratch is reused by the next item
    }
    (void)s_abort;
}

__global__ void __launch_bounds__(DS_THREADS, 1) decode_stream_kernel(const __grid_constant__ DsParams p) {
    extern __shared__ __align__(128) unsigned char dyn[];
    __shared__ __align__(16) DsShared sh;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int cta = blockIdx.x, ncta = gridDim.x;
    const int NS = p.nstages;
    unsigned char* ring = dyn;
    unsigned char* xpl = dyn + (size_t)NS * DS_UNIT_BYTES;
    float* xsc = reinterpret_cast<float*>(xpl + (size_t)p.kmax * 3);
    volatile int* s_abort = &sh.abort;

    if (tid == 0) {
        for (int s = 0; s < NS; s++) { ds_mbar_init(&sh.full[s], 1); ds_mbar_init(&sh.empty[s], DS_CONSUMER_WARPS); }
        sh.abort = 0;
        sh.seq = *reinterpret_cast<volatile unsigned long long*>(p.ctr + 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();

    if (warp == 0) {
        // ------------------------------------------------------------ producer: the static weight stream
        if (lane == 0) {
            int slot = 0;
            uint32_t wrap = 0;           // completed passes over the ring
            long long issued = 0;
            bool stop = false;
            for (int ph = 0; ph < p.nphases && !stop; ph++) {
                const DsPhase P = p.phases[ph];
                if (!P.w) continue;
                const long long units = (long long)P.groups * P.S;
                const long long u0 = units * cta / ncta, u1 = units * (cta + 1) / ncta;
                const unsigned char* src = P.w + (size_t)u0 * DS_UNIT_BYTES;
                for (long long u = u0; u < u1; u++, src += DS_UNIT_BYTES) {
                    if (wrap > 0) ds_mbar_wait(&sh.empty[slot], (wrap - 1) & 1u, p, s_abort);
                    if (*s_abort) { stop = true; break; }
                    ds_mbar_expect_tx(&sh.full[slot], DS_UNIT_BYTES);
                    ds_bulk_load(ring + (size_t)slot * DS_UNIT_BYTES, src, DS_UNIT_BYTES, &sh.full[slot]);
                    issued++;
                    if (++slot == NS) { slot = 0; wrap++; }
                }
            }
            if (stop) {
                // aborted: wait (bounded) for the copies still in flight before this CTA's shared memory is released
                const long long back = issued < NS ? issued : NS;
                int s2 = slot; uint32_t w2 = wrap;
                for (long long i = 0; i < back; i++) {
                    if (--s2 < 0) { s2 = NS - 1; w2--; }
                    const unsigned long long t0 = blum_globaltimer();
                    while (!ds_mbar_try(&sh.full[s2], w2 & 1u) && blum_globaltimer() - t0 < DS_TIMEOUT_NS) {}
                }
            }
        }
        return;
    }

    // ---------------------------------------------------------------- consumers
    const int tid_c = tid - 32, cw = warp - 1;
    const int g = lane >> 2, t = lane & 3;
    const unsigned long long seq = sh.seq;
    int slot = 0;
    uint32_t wrap = 0;
    unsigned segcount = 0;
    int barrier_idx = 0;
    for (int ph = 0; ph < p.nphases; ph++) {
        const DsPhase P = p.phases[ph];
        if (P.kind == DS_ATTN) {
            ds_attention(p, P.layer, sh, tid_c, cta, ncta, s_abort);
        } else {
            const float rs = ds_stage_x(p, P, sh, xpl, xsc, tid_c, cta);
            const int S = P.S;
            const long long units = (long long)P.groups * S;
            const long long u0 = units * cta / ncta, u1 = units * (cta + 1) / ncta;
            const unsigned long long epoch = seq * (unsigned long long)(p.nphases + 1) + (unsigned long long)ph + 1ull;
            float acc0 = 0.f, acc1 = 0.f, acc2 = 0.f, acc3 = 0.f;
            long long seg_start = u0;
            long long grp = u0 / S;
            int s = (int)(u0 - grp * S);
            for (long long u = u0; u < u1; u++) {
                ds_mbar_wait(&sh.full[slot], wrap & 1u, p, s_abort);
                const unsigned char* st = ring + (size_t)slot * DS_UNIT_BYTES;
                const int kb0 = s * DS_UNIT_BLOCKS + 2 * cw;                     // this warp's two blocks of the slice
                const uint32_t d_lo = *reinterpret_cast<const uint32_t*>(st + 8192 + g * 32 + cw * 4);
                const uint32_t d_hi = *reinterpret_cast<const uint32_t*>(st + 8192 + (g + 8) * 32 + cw * 4);
                const float2 xs2 = *reinterpret_cast<const float2*>(xsc + kb0);
                const float2 dl = __half22float2(*reinterpret_cast<const __half2*>(&d_lo));
                const float2 dh = __half22float2(*reinterpret_cast<const __half2*>(&d_hi));
#pragma unroll
                for (int jj = 0; jj < 2; jj++) {
                    const int4 a = *reinterpret_cast<const int4*>(st + (size_t)(2 * cw + jj) * 512 + lane * 16);
                    // columns 0..2 of B are the three planes of x; the other columns are zero (select, so the warp stays converged)
                    int2 b = *reinterpret_cast<const int2*>(xpl + (size_t)(kb0 + jj) * 96 + min(g, 2) * 32 + t * 8);
                    b.x = g < 3 ? b.x : 0; b.y = g < 3 ? b.y : 0;
                    int d0, d1, d2, d3;
                    asm volatile("mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%10,%10,%10};"
                                 : "=r"(d0), "=r"(d1), "=r"(d2), "=r"(d3)
                                 : "r"(a.x), "r"(a.y), "r"(a.z), "r"(a.w), "r"(b.x), "r"(b.y), "r"(0));
                    const float xs = jj ? xs2.y : xs2.x;
                    const float sl = (jj ? dl.y : dl.x) * xs, shi = (jj ? dh.y : dh.x) * xs;
                    acc0 = fmaf((float)d0, sl, acc0);
                    acc1 = fmaf((float)d1, sl, acc1);
                    acc2 = fmaf((float)d2, shi, acc2);
                    acc3 = fmaf((float)d3, shi, acc3);
                }
                __syncwarp();
                if (lane == 0) ds_mbar_arrive(&sh.empty[slot]);
                if (++slot == NS) { slot = 0; wrap++; }

                const bool group_end = (s == S - 1);
                if (group_end || u == u1 - 1) {
                    // ---- end of this CTA's segment of the group: sum the warps' partial sums in a fixed order
                    const unsigned par = segcount & 1u;
                    sh.red[par][cw][lane] = make_float4(acc0, acc1, acc2, acc3);
                    ds_named_sync();
                    if (cw == (int)(segcount % DS_CONSUMER_WARPS)) {
                        float4 v = sh.red[par][0][lane];
#pragma unroll
                        for (int w = 1; w < DS_CONSUMER_WARPS; w++) {
                            const float4 o = sh.red[par][w][lane];
                            v.x += o.x; v.y += o.y; v.z += o.z; v.w += o.w;
                        }
                        // lane t=0 of a row pair holds planes 0 and 1 (columns 0, 1), lane t=1 plane 2 (column 2)
                        const float p2_lo = __shfl_down_sync(0xffffffffu, v.x, 1), p2_hi = __shfl_down_sync(0xffffffffu, v.z, 1);
                        float r_lo = fmaf(v.x, 65536.f, fmaf(v.y, 256.f, p2_lo));
                        float r_hi = fmaf(v.z, 65536.f, fmaf(v.w, 256.f, p2_hi));
                        const bool has_head = (seg_start == grp * S);
                        if (!has_head) {
                            // a later slice range of a group that starts in an earlier CTA: publish the partial sums
                            if (t == 0) { p.part[(size_t)cta * 32 + g] = r_lo; p.part[(size_t)cta * 32 + g + 8] = r_hi; }
                            __syncwarp();
                            if (lane == 0) { __threadfence(); ds_st_release(p.ctr + 8 + cta, epoch); }
                        } else {
                            if (!group_end) {
                                // the group continues in later CTAs: add their partial sums in CTA order
                                const long long gend = (grp + 1) * S;
                                for (int c2 = cta + 1; c2 < ncta; c2++) {
                                    const long long r0 = units * c2 / ncta, r1 = units * (c2 + 1) / ncta;
                                    if (r0 >= gend) break;
                                    if (r1 <= r0) continue;
                                    if (lane == 0) ds_wait_ge(p.ctr + 8 + c2, epoch, p, s_abort);
                                    __syncwarp();
                                    if (t == 0) { r_lo += __ldcg(p.part + (size_t)c2 * 32 + g); r_hi += __ldcg(p.part + (size_t)c2 * 32 + g + 8); }
                                }
                            }
                            if (t == 0) {
                                const long long row = grp * DS_UNIT_ROWS + g;
                                if (P.kind == DS_QKV) { p.qkv[row] = r_lo * rs; p.qkv[row + 8] = r_hi * rs; }
                                else if (P.kind == DS_HEAD) { p.logits[row] = r_lo * rs; p.logits[row + 8] = r_hi * rs; }
                                else if (P.kind == DS_GATEUP) {
                                    const float gate = r_lo * rs, upv = r_hi * rs;         // rows 0-7 of a group are gate rows, 8-15 the up rows
                                    p.mid[grp * 8 + g] = upv * (gate * (1.f / (1.f + __expf(-gate))));
                                } else {                                                  // o_proj / down: residual add in place
                                    p.xres[row] = __ldcg(p.xres + row) + r_lo;
                                    p.xres[row + 8] = __ldcg(p.xres + row + 8) + r_hi;
                                }
                            }
                        }
                    }
                    segcount++;
                    acc0 = acc1 = acc2 = acc3 = 0.f;
                    seg_start = u + 1;
                }
                if (group_end) { s = 0; grp++; } else s++;
            }
        }
        if (ph + 1 < p.nphases) {
            barrier_idx++;
            ds_grid_sync(p, (seq * (unsigned long long)p.nbarriers + (unsigned long long)barrier_idx) * (unsigned long long)ncta, tid_c, s_abort);
        }
    }
    if (cta == 0 && tid_c == 0 && !*s_abort) *reinterpret_cast<volatile unsigned long long*>(p.ctr + 1) = seq + 1ull;
}

// ------------------------------------------------------------------ packing
// thread per 16-byte operand piece (512 per unit) or per block scale (256 per unit)
__global__ void ds_pack_kernel(const int8_t* __restrict__ q, const __half* __restrict__ d, const int8_t* __restrict__ q2,
                               const __half* __restrict__ d2, long long groups, int K, unsigned char* __restrict__ out) {
    const int S = K / DS_UNIT_K, KB = K / 32;
    const long long total = groups * S * 768;
    for (long long idx = blockIdx.x * (long long)blockDim.x + threadIdx.x; idx < total; idx += (long long)gridDim.x * blockDim.x) {
        const long long u = idx / 768;
        const int r = (int)(idx - u * 768);
        const long long grp = u / S;
        const int s = (int)(u - grp * S);
        unsigned char* unit = out + (size_t)u * DS_UNIT_BYTES;
        if (r < 512) {
            const int j = r >> 5, lane = r & 31, g = lane >> 2, c = lane & 3;
            const int8_t *lo, *hi;
            if (q2) { lo = q + (size_t)(grp * 8 + g) * K; hi = q2 + (size_t)(grp * 8 + g) * K; }       // 8 gate rows, then the 8 up rows
            else { lo = q + (size_t)(grp * 16 + g) * K; hi = q + (size_t)(grp * 16 + g + 8) * K; }
            const int kbase = s * DS_UNIT_K + j * 32 + 8 * c;
            const int2 a = *reinterpret_cast<const int2*>(lo + kbase), b = *reinterpret_cast<const int2*>(hi + kbase);
            *reinterpret_cast<int4*>(unit + j * 512 + lane * 16) = make_int4(a.x, b.x, a.y, b.y);
        } else {
            const int r2 = r - 512, row = r2 >> 4, j = r2 & 15;
            const __half* src;
            if (q2) src = (row < 8) ? d + (size_t)(grp * 8 + row) * KB : d2 + (size_t)(grp * 8 + row - 8) * KB;
            else src = d + (size_t)(grp * 16 + row) * KB;
            reinterpret_cast<__half*>(unit + 8192)[row * 16 + j] = src[s * DS_UNIT_BLOCKS + j];
        }
    }
}

size_t blum_ds_packed_bytes(int64_t rows_total, int64_t K) { return (size_t)(rows_total / DS_UNIT_ROWS) * (size_t)(K / DS_UNIT_K) * DS_UNIT_BYTES; }

// Packs w (or gate = w and up = w_up interleaved in groups of 8 + 8 rows) into stream units.
int blum_ds_pack(blum_ctx* ctx, const blum_q8_weight* w, const blum_q8_weight* w_up, unsigned char* out) {
    BLUM_REQUIRE(ctx, w && out, "stream pack: null argument");
    const int64_t rows = w_up ? 2 * w->N : w->N;
    BLUM_REQUIRE(ctx, w->K % DS_UNIT_K == 0 && rows % DS_UNIT_ROWS == 0 && (!w_up || (w_up->N == w->N && w_up->K == w->K && w->N % 8 == 0)),
                 "stream pack: shape [%lld,%lld] is not a multiple of the 16 x 512 unit", (long long)rows, (long long)w->K);
    ds_pack_kernel<<<ctx->sm_count * 8, 256, 0, ctx->stream>>>(w->q, w->d, w_up ? w_up->q : nullptr, w_up ? w_up->d : nullptr,
                                                               rows / DS_UNIT_ROWS, (int)w->K, out);
    BLUM_LAUNCH_CHECK(ctx);
    return BLUM_OK;
}

size_t blum_ds_smem_bytes(int nstages, int kmax) { return (size_t)nstages * DS_UNIT_BYTES + (size_t)kmax * 3 + (size_t)kmax / 32 * 4 + 128; }

int blum_ds_launch(blum_ctx* ctx, const DsParams& p) {
    static bool attr_set[64] = {};
    const size_t smem = blum_ds_smem_bytes(p.nstages, p.kmax);
    if (ctx->device >= 0 && ctx->device < 64 && !attr_set[ctx->device]) {
        BLUM_CUDA(ctx, cudaFuncSetAttribute(decode_stream_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)(ctx->smem_optin - 20 * 1024)));
        attr_set[ctx->device] = true;
    }
    void* args[] = {(void*)&p};
    BLUM_CUDA(ctx, cudaLaunchCooperativeKernel((const void*)decode_stream_kernel, dim3(ctx->sm_count), dim3(DS_THREADS), args, smem, ctx->stream));
    ctx->launches++;
    return BLUM_OK;
}
