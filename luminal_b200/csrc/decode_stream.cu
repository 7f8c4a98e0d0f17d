// One decode step of the Llama decoder (batch 1, f32 activations and KV cache) as ONE persistent kernel with a
// continuous weight stream and data-driven hand-over between its phases.
//
// The reference executes a decode step as ~10^3 graph nodes, one allocation and one launch each
// (src/graph.rs:191-224 in luminal), the quantised matmuls as one 64-thread-block matvec launch per projection
// (crates/luminal_cuda/src/quantized.rs:28-109,116-168).  A batch-1 step is bound by reading the 8 GB of Q8_0
// weights once; every kernel boundary, dependency wait and re-staging of x is time with no weight bytes in flight.
// Here the weights of the whole step are one statically ordered stream:
//   * grid = one CTA per SM (cooperative launch, so all CTAs are co-resident); per matrix every CTA owns one
//     contiguous range of 8.5 KB units (16 rows x 512 k, repacked once at load so that a unit is contiguous in
//     HBM and already in the register layout of the MMA operand);
//   * the ring: one shared-memory stage per warp.  A warp waits for its unit (mbarrier complete_tx), consumes it and
//     at once requests the unit a whole ring further down the CTA's stream into the same stage with one
//     cp.async.bulk - across phase boundaries, so HBM keeps streaming while the CTA waits for activations;
//   * x is staged once per phase per CTA as block fixed point (per 32-element block x_i = xfix_i * 2^(e-21),
//     |xfix_i| <= 2^22, split into three signed byte planes), so that the dot product of a Q8_0 block with x is
//     exact integer arithmetic on the legacy tensor path: one mma.sync.m16n8k32.s8 covers 16 rows x one block, the
//     three planes of x are three columns of B (k is permuted inside a block so that both operands are plain
//     8/16-byte shared-memory loads); per (row, block): acc_plane += float(int) * (d * 2^e),
//     result = 65536 acc_0 + 256 acc_1 + acc_2 - the block-sum-times-block-scale order of the reference kernel;
//   * phases of a layer: [RMSNorm + q/k/v] -> [RoPE + KV append + attention] -> [o_proj + residual] ->
//     [RMSNorm + gate/up + SwiGLU] -> [down + residual]; after the last layer [RMSNorm + LM head];
//   * hand-over without grid barriers: every activation that crosses CTAs is a 64-bit word {f32 value, 32-bit tag},
//     written with one store and read with one load, so a word is seen whole or not at all.  The tag names the
//     launch and the producing phase; a reader that finds an older tag loads again (bounded).  No fence, no counter,
//     no barrier stands between a producer's store and a consumer's load, and a CTA waits only for the values it
//     reads.  (A buffer's next version is written two or more phases later; those writers have by then consumed
//     values that every reader of the old version contributed to, so no reader can still be waiting for it.)
//   * a 16-row group whose k-range is cut by a CTA boundary is finished by the CTA that holds its first slice,
//     which adds the partial sums the later CTAs publish (tagged words again; fetched while the stream still runs);
//     all sums run in a fixed order, so results are reproducible bit for bit.
// Every wait is bounded by wall-clock time; on expiry the CTA raises the abort word, every later wait in the grid
// becomes a no-op, the error word is set, and a warp waits for its copy in flight before it exits.
// Algorithmic bytes per launch: all Q8_0 weights of the model once (N*K*34/32 each) + the KV rows of the context.
#include "decode_stream.cuh"

#define DS_TIMEOUT_NS 2000000000ull       // every wait gives up after 2 s
#define LOG2E 1.4426950408889634f

__device__ __forceinline__ uint32_t ds_smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void ds_mbar_init(uint64_t* bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(ds_smem_u32(bar)), "r"(count));
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
// weights are read once: their lines are the first to leave L2 again
__device__ __forceinline__ void ds_bulk_load(void* dst, const void* src, uint32_t bytes, uint64_t* bar, uint64_t policy) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint [%0], [%1], %2, [%3], %4;"
                 ::"r"(ds_smem_u32(dst)), "l"(src), "r"(bytes), "r"(ds_smem_u32(bar)), "l"(policy) : "memory");
}
__device__ __forceinline__ void ds_bulk_prefetch(const void* src, uint32_t bytes) {
    asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(src), "r"(bytes) : "memory");
}
// tagged words: {value, tag} in one naturally aligned 64-bit access
__device__ __forceinline__ void ds_st_tagged(unsigned long long* p, float v, uint32_t tag) {
    const unsigned long long w = ((unsigned long long)tag << 32) | (unsigned long long)__float_as_uint(v);
    asm volatile("st.relaxed.gpu.global.b64 [%0], %1;" ::"l"(p), "l"(w) : "memory");
}
__device__ __forceinline__ unsigned long long ds_ld_word(const unsigned long long* p) {
    unsigned long long v;
    asm volatile("ld.relaxed.gpu.global.b64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ ulonglong2 ds_ld_word2(const unsigned long long* p) {
    ulonglong2 v;
    asm volatile("ld.relaxed.gpu.global.v2.b64 {%0, %1}, [%2];" : "=l"(v.x), "=l"(v.y) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ uint32_t ds_tag_of(unsigned long long w) { return (uint32_t)(w >> 32); }
__device__ __forceinline__ float ds_val_of(unsigned long long w) { return __uint_as_float((uint32_t)w); }

// The first wait that gives up also records where: ctr[3] = site (1 weight stage, 2 activation word, 3 attention
// input, 4 partial sums of a split group, 6 a slot of the per-unit sums), ctr[4] = CTA, ctr[5], ctr[6] = what it waited for and what it saw.
__device__ __noinline__ void ds_give_up(int* err, unsigned long long* ctr, volatile int* s_abort, int site, long long a, long long b) {
    *s_abort = 1;
    atomicOr(err, 0x400);
    if (atomicCAS(ctr + 3, 0ull, (unsigned long long)site) == 0ull) {
        ctr[4] = blockIdx.x; ctr[5] = (unsigned long long)a; ctr[6] = (unsigned long long)b;
    }
    atomicExch(ctr + 2, 1ull);
}
__device__ __forceinline__ bool ds_aborted(const DsParams& p, volatile int* s_abort) {
    if (*s_abort) return true;
    if (*reinterpret_cast<volatile unsigned long long*>(p.ctr + 2) != 0ull) { *s_abort = 1; return true; }
    return false;
}
// bounded wait on an mbarrier phase; a no-op once the grid has aborted
__device__ __forceinline__ void ds_mbar_wait(uint64_t* bar, uint32_t parity, const DsParams& p, volatile int* s_abort, int site, long long what) {
    if (*s_abort) return;
    if (ds_mbar_try(bar, parity)) return;
    const unsigned long long t0 = blum_globaltimer();
    for (uint32_t spin = 1;; spin++) {
        if (ds_mbar_try(bar, parity)) return;
        if ((spin & 63u) == 0u) {
            if (ds_aborted(p, s_abort)) return;
            if (blum_globaltimer() - t0 > DS_TIMEOUT_NS) { ds_give_up(p.err, p.ctr, s_abort, site, what, parity); return; }
        }
    }
}
// bounded wait for a tagged word; returns the word (whatever it holds once the grid has aborted)
__device__ __forceinline__ unsigned long long ds_wait_word(const unsigned long long* ptr, uint32_t tag, const DsParams& p,
                                                           volatile int* s_abort, int site) {
    unsigned long long w = ds_ld_word(ptr);
    if (ds_tag_of(w) == tag || *s_abort) return w;
    const unsigned long long t0 = blum_globaltimer();
    for (uint32_t spin = 1;; spin++) {
        w = ds_ld_word(ptr);
        if (ds_tag_of(w) == tag) return w;
        if ((spin & 63u) == 0u) {
            if (ds_aborted(p, s_abort)) return w;
            if (blum_globaltimer() - t0 > DS_TIMEOUT_NS) { ds_give_up(p.err, p.ctr, s_abort, site, (long long)tag, (long long)ds_tag_of(w)); return w; }
        }
    }
}
__device__ __forceinline__ float ds_wait_value(const unsigned long long* ptr, uint32_t tag, const DsParams& p, volatile int* s_abort, int site) {
    return ds_val_of(ds_wait_word(ptr, tag, p, s_abort, site));
}

__device__ __forceinline__ void ds_sync() { __syncthreads(); }
__device__ __forceinline__ int ds_sync_and(int pred) { return __syncthreads_and(pred); }

static_assert(DS_PARTIAL_SLOTS * 16 >= DS_WARPS * 128, "the attention phase borrows the partial-sum slots as [DS_WARPS][128]");
struct DsShared {
    uint64_t full[DS_STAGES];
    float partial[DS_PARTIAL_SLOTS][16];            // per-unit row sums waiting for the rest of their group (the attention phase
                                                    // borrows it as [DS_WARPS][128])
    int gcnt[DS_PARTIAL_SLOTS];                     // units of a group deposited so far (indexed by group % slots)
    int pbusy[DS_PARTIAL_SLOTS];                    // 1 while a slot of `partial` holds sums that have not been added up yet
    int xstate[DS_MAX_SLICES];                      // 4 * phase + {1: being staged, 2: staged} per 512-element slice of x
    float xss[DS_MAX_SLICES];                       // sum of squares of each staged slice (RMSNorm)
    float q[128], knew[128], vnew[128];
    float rsn[64], rcs[64];                         // rotation of the step's position
    float sc[DS_ATTN_TILE];
    long long koff[DS_ATTN_TILE];
    float l_part[DS_WARPS];                         // every warp's share of the softmax denominator (its share of P V lives in `partial`)
    unsigned long long seq;
    int abort;
    float pp_sum[16];                               // partial sums of the later CTAs for this CTA's last group
    int pp_state;                                   // phase + 1: pp_sum is valid for that phase
    unsigned long long amax;                        // largest (ordered logit, row) key of this CTA's head rows; 0: none
    int amax_nan;                                   // a head row of this CTA was a NaN
    int2 range[DS_MAX_PHASES];                      // this CTA's units [x, y) of every phase
};

// tag of what phase `ph` of launch `seq` writes (ph = -1: the embedding row that CTA 0 copies into the residual stream)
__device__ __forceinline__ uint32_t ds_tag(unsigned long long seq, int nphases, int ph) {
    return (uint32_t)((seq + 1ull) * (unsigned long long)(nphases + 2) + (unsigned long long)(ph + 1));
}

// ---- x of a phase -> block fixed point in shared memory (three signed byte planes + one scale per 32 elements)
// planes: [K/32][3][32] bytes; scales: [K/32] floats.  x is the previous phase's output: tagged words that are loaded
// again until they carry that phase's tag.  x is staged lazily, one 512-element slice (the k range of one unit) at a time,
// by the warp that first needs it: a unit only needs its own slice, so a warp starts on its weights as soon as that slice
// has arrived instead of waiting for the slowest producer of the whole vector, and the round trips of the hand-over
// overlap with the other warps' work.  sh.xstate[s] = 4 * phase + {1: a warp is staging it, 2: staged}.
__device__ __noinline__ void ds_stage_slice(const DsParams& p, int kind, int layer, const float* norm_w, int ph, unsigned long long seq,
                                            DsShared& sh, unsigned char* xpl, float* xsc, int lane, int slice, volatile int* s_abort) {
    const uint32_t tag = ds_tag(seq, p.nphases, ph - 1);
    const unsigned long long* src = kind == DS_O ? p.attn : kind == DS_DOWN ? p.mid : p.xres;
    const bool from_embed = (kind == DS_QKV && layer == 0);
    const bool combine = (kind == DS_O) && p.nsplit > 1;
    const int kbase = slice * DS_UNIT_K;
    float ss = 0.f;
    // one step of four consecutive elements: norm weight, block maximum over the 8 lanes of a 32-element block, digits
    auto put = [&](float (&v)[4], int k, const float4 nw) {      // nw: the norm weights of these four elements (ones without a norm)
        ss += v[0] * v[0] + v[1] * v[1] + v[2] * v[2] + v[3] * v[3];
        v[0] *= nw.x; v[1] *= nw.y; v[2] *= nw.z; v[3] *= nw.w;
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
    auto norm_at = [&](int k) { return norm_w ? __ldg(reinterpret_cast<const float4*>(norm_w + k)) : make_float4(1.f, 1.f, 1.f, 1.f); };
    constexpr int PASS = 128;                                     // elements a warp covers per pass (4 per lane)
    if (from_embed) {
        // layer 0 reads the embedding row itself
        int id = p.rows[0];
        if (id < 0 || id >= p.vocab) { if (lane == 0) atomicOr(p.err, 0x100); id = 0; }
        const float* erow = p.embed + (size_t)id * p.H;
#pragma unroll
        for (int i = 0; i < DS_UNIT_K / PASS; i++) {
            const int k = kbase + i * PASS + lane * 4;
            const float4 e = __ldg(reinterpret_cast<const float4*>(erow + k));
            float v[4] = {e.x, e.y, e.z, e.w};
            put(v, k, norm_at(k));
        }
    } else if (!combine) {
        // Two halves of 8 words per lane.  The norm weights do not depend on the words and are requested with them; the second
        // half's first request goes out before the first half is digitised, so that its round trip overlaps that work.  Words
        // that still carry an older tag are requested together again: one round trip per attempt, however many are late.
        // (All 16 words of a lane polled as one round was measured slower: twice the polling traffic while producers are late.)
        const int kA = kbase + lane * 4, kB = kA + 2 * PASS;
        ulonglong2 bufA[2][2], bufB[2][2];
        auto request = [&](ulonglong2 (&buf)[2][2], int k0, unsigned ready) {
#pragma unroll
            for (int i = 0; i < 2; i++)
                if (!((ready >> i) & 1u)) { buf[i][0] = ds_ld_word2(src + k0 + i * PASS); buf[i][1] = ds_ld_word2(src + k0 + i * PASS + 2); }
        };
        auto arrived = [&](const ulonglong2 (&buf)[2][2], unsigned ready) {
#pragma unroll
            for (int i = 0; i < 2; i++)
                if (ds_tag_of(buf[i][0].x) == tag && ds_tag_of(buf[i][0].y) == tag && ds_tag_of(buf[i][1].x) == tag && ds_tag_of(buf[i][1].y) == tag)
                    ready |= 1u << i;
            return ready;
        };
        auto wait_all = [&](ulonglong2 (&buf)[2][2], int k0) {       // first request already issued
            unsigned ready = 0;
            const unsigned long long t0 = blum_globaltimer();
            for (uint32_t spin = 0;; spin++) {
                ready = arrived(buf, ready);
                if (__all_sync(0xffffffffu, ready == 3u || *s_abort)) break;
                if (lane == 0 && (spin & 15u) == 15u && !ds_aborted(p, s_abort) && blum_globaltimer() - t0 > DS_TIMEOUT_NS)
                    ds_give_up(p.err, p.ctr, s_abort, 2, (long long)tag, (long long)k0);
                request(buf, k0, ready);
            }
        };
        const float4 nwA0 = norm_at(kA), nwA1 = norm_at(kA + PASS);
        request(bufA, kA, 0u);
        wait_all(bufA, kA);
        const float4 nwB0 = norm_at(kB), nwB1 = norm_at(kB + PASS);
        request(bufB, kB, 0u);
#pragma unroll
        for (int i = 0; i < 2; i++) {
            float v[4] = {ds_val_of(bufA[i][0].x), ds_val_of(bufA[i][0].y), ds_val_of(bufA[i][1].x), ds_val_of(bufA[i][1].y)};
            put(v, kA + i * PASS, i ? nwA1 : nwA0);
        }
        wait_all(bufB, kB);
#pragma unroll
        for (int i = 0; i < 2; i++) {
            float v[4] = {ds_val_of(bufB[i][0].x), ds_val_of(bufB[i][0].y), ds_val_of(bufB[i][1].x), ds_val_of(bufB[i][1].y)};
            put(v, kB + i * PASS, i ? nwB1 : nwB0);
        }
    } else {
        for (int i = 0; i < DS_UNIT_K / PASS; i++) {
            const int k = kbase + i * PASS + lane * 4;
            // merge the split attention partials of head k/128: weights exp2((m_s - m_max) log2 e)
            const int h = k >> 7, c = k & 127;
            const unsigned long long* base = p.attn_part + (size_t)h * p.nsplit * 130;
            float mmax = -INFINITY;
            for (int s = 0; s < p.nsplit; s++) mmax = fmaxf(mmax, ds_wait_value(base + s * 130 + 128, tag, p, s_abort, 2));
            float den = 0.f;
            float v[4] = {0.f, 0.f, 0.f, 0.f};
            for (int s = 0; s < p.nsplit; s++) {
                const float ms = ds_wait_value(base + s * 130 + 128, tag, p, s_abort, 2);
                const float w = (ms == -INFINITY) ? 0.f : exp2f((ms - mmax) * LOG2E);
                den = fmaf(ds_wait_value(base + s * 130 + 129, tag, p, s_abort, 2), w, den);
#pragma unroll
                for (int e = 0; e < 4; e++) v[e] = fmaf(ds_wait_value(base + s * 130 + c + e, tag, p, s_abort, 2), w, v[e]);
            }
            const float inv = den > 0.f ? 1.f / den : 0.f;
#pragma unroll
            for (int e = 0; e < 4; e++) v[e] *= inv;
            put(v, k, norm_at(k));
        }
    }
    ss = warp_sum(ss);
    if (lane == 0) sh.xss[slice] = ss;
}

// makes sure slice `slice` of the phase's x is in shared memory: stages it, or waits for the warp that does
__device__ __forceinline__ void ds_ensure_slice(const DsParams& p, const DsPhase& P, int ph, unsigned long long seq, DsShared& sh,
                                                unsigned char* xpl, float* xsc, int lane, int slice, volatile int* s_abort) {
    const int ready = ph * 4 + 2, busy = ph * 4 + 1;
    int r = 0;
    if (lane == 0) {
        const int v = *reinterpret_cast<volatile int*>(&sh.xstate[slice]);
        if (v == ready) r = 0;
        else if (v == busy) r = 2;
        else r = (atomicCAS(&sh.xstate[slice], v, busy) == v) ? 1 : 2;
    }
    r = __shfl_sync(0xffffffffu, r, 0);
    if (r == 1) {
        ds_stage_slice(p, P.kind, P.layer, P.norm_w, ph, seq, sh, xpl, xsc, lane, slice, s_abort);
        __syncwarp();
        if (lane == 0) { __threadfence_block(); *reinterpret_cast<volatile int*>(&sh.xstate[slice]) = ready; }
    } else if (r == 2) {
        if (lane == 0) {
            const unsigned long long t0 = blum_globaltimer();
            for (uint32_t spin = 1; *reinterpret_cast<volatile int*>(&sh.xstate[slice]) != ready && !*s_abort; spin++)
                if ((spin & 1023u) == 0u && (ds_aborted(p, s_abort) || blum_globaltimer() - t0 > DS_TIMEOUT_NS)) {
                    if (!*s_abort) ds_give_up(p.err, p.ctr, s_abort, 7, slice, ph);
                    break;
                }
        }
        __syncwarp();
    }
    __threadfence_block();
}

// (sequence, context length) of the step, validated
__device__ __forceinline__ void ds_step_row(const DsParams& p, int tid_c, int& seq, int& ctx) {
    seq = p.rows[p.max_rows]; ctx = p.rows[3 * p.max_rows];
    const int ps = p.kv.page_size;
    if (seq < 0 || seq >= p.max_seqs || ctx < 1 || (ctx + ps - 1) / ps > p.kv.max_pages_per_seq) {
        if (tid_c == 0) atomicOr(p.err, 0x100);
        seq = 0; ctx = 1;
    }
}
// cached positions [c0, c1) of split `split` (split on page boundaries)
__device__ __forceinline__ void ds_split_range(const DsParams& p, int pos, int split, int& c0, int& c1) {
    const int ps = p.kv.page_size;
    const int npages = (pos + ps - 1) / ps, pages_per_split = (npages + p.nsplit - 1) / p.nsplit;
    c0 = min(pos, split * pages_per_split * ps); c1 = min(pos, (split + 1) * pages_per_split * ps);
}
// row offsets of tile [t0, t0 + n) of kv head kvh into koff
__device__ __forceinline__ void ds_tile_offsets(const DsParams& p, DsShared& sh, int layer, const int32_t* table, int kvh, int t0, int n, int tid_c) {
    if (tid_c < n) {
        const int pj = t0 + tid_c, ps = p.kv.page_size;
        int32_t page = table[pj / ps];
        if (page < 0 || page >= p.kv.num_pages) { atomicOr(p.err, 0x200); page = 0; }
        sh.koff[tid_c] = kv_tile_offset(p.kv, layer, page, 0, kvh, pj % ps);
    }
}

// ---- RoPE + KV append + attention of the new token; items (q head, split) are dealt round robin to the CTAs
__device__ __forceinline__ void ds_attention(const DsParams& p, int layer, int ph, unsigned long long seqno, DsShared& sh, int tid_c,
                                             int cta, int ncta, volatile int* s_abort) {
    const int nitems = p.nq * p.nsplit;
    if (cta >= nitems) return;
    const int lane = tid_c & 31, cw = tid_c >> 5;
    const KvView& kv = p.kv;
    const int ps = kv.page_size, G = p.nq / p.nkv;
    const uint32_t tag_in = ds_tag(seqno, p.nphases, ph - 1), tag_out = ds_tag(seqno, p.nphases, ph);
    int seq, ctx;
    ds_step_row(p, tid_c, seq, ctx);
    const int pos = ctx - 1;
    const int32_t* table = kv.table + (size_t)seq * kv.max_pages_per_seq;
    float* pool = reinterpret_cast<float*>(kv.pool);
    const long long vdelta = (long long)kv.kv_heads * ps * 128;       // K tile -> V tile of the same (page, head)
    const int part = tid_c >> 7, c = tid_c & 127;                     // partition of the positions for P V, and the dim
    if (tid_c < 64) {
        const float a = (float)pos * p.freqs.inv_freq[tid_c];
        sh.rsn[tid_c] = sinf(a); sh.rcs[tid_c] = sinf(1.5707964f - a);   // cos(x) = sin(pi/2 - x), as the reference computes it
    }
    for (int item = cta; item < nitems; item += ncta) {
        const int h = item % p.nq, split = item / p.nq, kvh = h / G;
        int c0, c1;
        ds_split_range(p, pos, split, c0, c1);
        // Nothing up to here depends on the new token: the row offsets of the first tile, and L2 prefetches of its cached
        // K and V rows (the weight stream has long pushed them out of L2), go out before q/k/v are waited for.
        if (c1 > c0) {
            const int n0 = min(DS_ATTN_TILE, c1 - c0);
            ds_tile_offsets(p, sh, layer, table, kvh, c0, n0, tid_c);
            if (tid_c < n0) {
                const float* kr = pool + sh.koff[tid_c];
#pragma unroll
                for (int l = 0; l < 4; l++) {                                    // a row of 128 floats is four 128-byte lines
                    asm volatile("prefetch.global.L2 [%0];" ::"l"(kr + l * 32));
                    asm volatile("prefetch.global.L2 [%0];" ::"l"(kr + vdelta + l * 32));
                }
            }
        }
        ds_sync();                                                  // rsn / rcs / koff are written
        // rotary embedding of q (threads 0..63) and of the new k (64..127); v is copied (128..255)
        if (tid_c < 128) {
            const int pi = tid_c & 63;
            const float sn = sh.rsn[pi], cs = sh.rcs[pi];
            const unsigned long long* s2 = p.qkv + (size_t)((tid_c < 64) ? h : p.nq + kvh) * 128 + 2 * pi;
            ulonglong2 w = ds_ld_word2(s2);
            if (ds_tag_of(w.x) != tag_in) w.x = ds_wait_word(s2, tag_in, p, s_abort, 3);
            if (ds_tag_of(w.y) != tag_in) w.y = ds_wait_word(s2 + 1, tag_in, p, s_abort, 3);
            const float x0 = ds_val_of(w.x), x1 = ds_val_of(w.y);
            float* dst = (tid_c < 64) ? sh.q : sh.knew;
            dst[2 * pi] = x0 * cs - x1 * sn;
            dst[2 * pi + 1] = x0 * sn + x1 * cs;
        } else if (tid_c < 256) {
            sh.vnew[c] = ds_wait_value(p.qkv + (size_t)(p.nq + p.nkv + kvh) * 128 + c, tag_in, p, s_abort, 3);
        }
        ds_sync();
        if (split == 0 && h % G == 0 && tid_c < 256) {     // one item per kv head appends the new row to its page slot
            const int32_t page = table[pos / ps];
            if (page < 0 || page >= kv.num_pages) { if (tid_c == 0) atomicOr(p.err, 0x40); }
            else {
                const long long o = kv_tile_offset(kv, layer, page, 0, kvh, pos % ps);
                if (part == 0) pool[o + c] = sh.knew[c]; else pool[o + vdelta + c] = sh.vnew[c];
            }
        }
        const float4 q4 = *reinterpret_cast<const float4*>(&sh.q[lane * 4]);
        // Both products give a warp whole rows (a lane holds four of the 128 dims) and keep eight rows per warp in flight: a
        // tile of up to 128 positions is ONE round of loads for the scores and one for P V (the rows come from L2 or HBM, so
        // rounds, not bytes, are what a short context costs).
        float m_run = -INFINITY, l_run = 0.f;
        float4 o4 = make_float4(0.f, 0.f, 0.f, 0.f);
        for (int t0 = c0; t0 < c1; t0 += DS_ATTN_TILE) {
            const int n = min(DS_ATTN_TILE, c1 - t0);
            if (t0 > c0) { ds_tile_offsets(p, sh, layer, table, kvh, t0, n, tid_c); ds_sync(); }
            for (int j0 = cw; j0 < n; j0 += DS_WARPS * 8) {
                float4 kr[8];
#pragma unroll
                for (int i = 0; i < 8; i++) {
                    const int j = j0 + i * DS_WARPS;
                    kr[i] = (j < n) ? __ldg(reinterpret_cast<const float4*>(pool + sh.koff[j]) + lane) : make_float4(0.f, 0.f, 0.f, 0.f);
                }
#pragma unroll
                for (int i = 0; i < 8; i++) {
                    const int j = j0 + i * DS_WARPS;
                    const float dot = warp_sum(kr[i].x * q4.x + kr[i].y * q4.y + kr[i].z * q4.z + kr[i].w * q4.w);
                    if (lane == 0 && j < n) sh.sc[j] = dot * p.scale;
                }
            }
            // the V rows of this warp's first eight positions do not depend on the scores: requested now, they arrive while the
            // softmax goes through its three barriers
            float4 vr[8];
#pragma unroll
            for (int i = 0; i < 8; i++) {
                const int j = cw + i * DS_WARPS;
                vr[i] = (j < n) ? __ldg(reinterpret_cast<const float4*>(pool + sh.koff[j] + vdelta) + lane) : make_float4(0.f, 0.f, 0.f, 0.f);
            }
            ds_sync();
            float mx = -INFINITY;
            for (int j = lane; j < n; j += 32) mx = fmaxf(mx, sh.sc[j]);
            mx = warp_max(mx);
            const float m_new = fmaxf(m_run, mx);
            const float corr = (m_run == -INFINITY) ? 0.f : exp2f((m_run - m_new) * LOG2E);
            ds_sync();                                               // every warp has read the raw scores
            if (tid_c < n) sh.sc[tid_c] = exp2f((sh.sc[tid_c] - m_new) * LOG2E);
            ds_sync();
            o4.x *= corr; o4.y *= corr; o4.z *= corr; o4.w *= corr; l_run *= corr; m_run = m_new;
            for (int j0 = cw; j0 < n; j0 += DS_WARPS * 8) {
                if (j0 != cw) {
#pragma unroll
                    for (int i = 0; i < 8; i++) {
                        const int j = j0 + i * DS_WARPS;
                        vr[i] = (j < n) ? __ldg(reinterpret_cast<const float4*>(pool + sh.koff[j] + vdelta) + lane) : make_float4(0.f, 0.f, 0.f, 0.f);
                    }
                }
#pragma unroll
                for (int i = 0; i < 8; i++) {
                    const int j = j0 + i * DS_WARPS;
                    const float pj = (j < n) ? sh.sc[j] : 0.f;
                    o4.x = fmaf(pj, vr[i].x, o4.x); o4.y = fmaf(pj, vr[i].y, o4.y); o4.z = fmaf(pj, vr[i].z, o4.z); o4.w = fmaf(pj, vr[i].w, o4.w);
                    l_run += pj;
                }
            }
            ds_sync();                                               // sc / koff are rewritten by the next tile
        }
        if (split == 0) {       // the new token itself: its k and v are still in shared memory
            const float4 k4 = *reinterpret_cast<const float4*>(&sh.knew[lane * 4]);
            const float s = warp_sum(k4.x * q4.x + k4.y * q4.y + k4.z * q4.z + k4.w * q4.w) * p.scale;
            const float m_new = fmaxf(m_run, s);
            const float corr = (m_run == -INFINITY) ? 0.f : exp2f((m_run - m_new) * LOG2E);
            const float pj = exp2f((s - m_new) * LOG2E);
            o4.x *= corr; o4.y *= corr; o4.z *= corr; o4.w *= corr; l_run *= corr; m_run = m_new;
            if (cw == 0) {
                const float4 v4 = *reinterpret_cast<const float4*>(&sh.vnew[lane * 4]);
                o4.x = fmaf(pj, v4.x, o4.x); o4.y = fmaf(pj, v4.y, o4.y); o4.z = fmaf(pj, v4.z, o4.z); o4.w = fmaf(pj, v4.w, o4.w);
                l_run += pj;
            }
        }
        // every warp's share of P V, [warp][128]: in the 8 KB of `partial`, which only the unit loops of the weight phases use
        // (a CTA-wide barrier lies between them and this point, and another between here and the next weight phase)
        float (*o_part)[128] = reinterpret_cast<float (*)[128]>(&sh.partial[0][0]);
        *reinterpret_cast<float4*>(&o_part[cw][lane * 4]) = o4;
        if (lane == 0) sh.l_part[cw] = l_run;
        ds_sync();
        if (part == 0) {
            float o = 0.f, l = 0.f;
#pragma unroll
            for (int i = 0; i < DS_WARPS; i++) { o += o_part[i][c]; l += sh.l_part[i]; }
            if (p.nsplit == 1) ds_st_tagged(p.attn + (size_t)h * 128 + c, o * (l > 0.f ? 1.f / l : 0.f), tag_out);
            else {
                unsigned long long* dst = p.attn_part + ((size_t)h * p.nsplit + split) * 130;
                ds_st_tagged(dst + c, o, tag_out);
                if (c == 0) { ds_st_tagged(dst + 128, m_run, tag_out); ds_st_tagged(dst + 129, l, tag_out); }
            }
        }
        ds_sync();                                                   // shared scratch is reused by the next item
    }
}

// position of a CTA in its static weight stream (the units of all phases, in phase order)
struct DsCursor {
    int ph, u, u1;
    const unsigned char* base;
};
// first and one-past-last unit of CTA `cta` among `units` (an even split of the unit list over the grid)
__device__ __forceinline__ int ds_range_lo(int units, int cta, int ncta) { return (int)(((unsigned long long)(unsigned)units * (unsigned)cta) / (unsigned)ncta); }
__device__ __forceinline__ void ds_cursor_seek(const DsPhase* phases, int nphases, const DsShared& sh, DsCursor& c) {   // first unit at or after phase c.ph
    for (; c.ph < nphases; c.ph++) {
        const int2 r = sh.range[c.ph];
        if (r.x < r.y) { c.u = r.x; c.u1 = r.y; c.base = phases[c.ph].w; return; }
    }
    c.u = c.u1 = 0; c.base = nullptr;
}
__device__ __forceinline__ void ds_cursor_advance(const DsPhase* phases, int nphases, const DsShared& sh, DsCursor& c, int k) {
    while (k > 0 && c.base) {
        const int avail = c.u1 - c.u;
        if (k < avail) { c.u += k; k = 0; }
        else { k -= avail; c.ph++; ds_cursor_seek(phases, nphases, sh, c); }
    }
}

// Partial sums of the later CTAs that hold slices of the group ending at unit `gend` (whose first slices this CTA holds),
// added in CTA order.  `block` = false only looks: returns false if one of them has not been published yet.
__device__ __forceinline__ bool ds_fetch_partners(const DsParams& p, int units, int gend, int cta, int ncta, uint32_t tag, int lane,
                                                  bool block, volatile int* s_abort, float& sum) {
    sum = 0.f;
    for (int c2 = cta + 1; c2 < ncta; c2++) {
        const int r0 = ds_range_lo(units, c2, ncta), r1 = ds_range_lo(units, c2 + 1, ncta);
        if (r0 >= gend) break;
        if (r1 <= r0) continue;
        const unsigned long long* src = p.part + (size_t)c2 * 16 + (lane & 15);
        unsigned long long w = block ? ds_wait_word(src, tag, p, s_abort, 4) : ds_ld_word(src);
        if (!__all_sync(0xffffffffu, ds_tag_of(w) == tag || *s_abort)) return false;
        sum += ds_val_of(w);
    }
    return true;
}

// PROF: the development counters and timestamps (blum_llama_stream_profile); the product launches the kernel without them:
// they cost clock reads per unit and registers the unit loop has no room for
template <bool PROF>
__global__ void __launch_bounds__(DS_THREADS, 1) decode_stream_kernel(const __grid_constant__ DsParams p) {
    extern __shared__ __align__(128) unsigned char dyn[];
    __shared__ __align__(16) DsShared sh;
    const int tid_c = threadIdx.x, cw = tid_c >> 5, lane = tid_c & 31;
    const int cta = blockIdx.x, ncta = gridDim.x;
    constexpr int NS = DS_STAGES;
    unsigned char* ring = dyn;
    unsigned char* xpl = dyn + (size_t)NS * DS_UNIT_BYTES;
    float* xsc = reinterpret_cast<float*>(xpl + (size_t)p.kmax * 3);
    volatile int* s_abort = &sh.abort;

    // the phase table and this CTA's share of every phase's units: read all the time, so they live in shared memory
    DsPhase* phases = reinterpret_cast<DsPhase*>(xsc + p.kmax / 32);
    for (int i = tid_c; i < p.nphases; i += DS_THREADS) {
        const DsPhase P = p.phases[i];
        phases[i] = P;
        // short phases hand out whole 16-row groups (a group cut between two CTAs costs a round trip at the very end of the
        // phase, more than the uneven share does); long ones are cut to the unit
        if (!P.w) sh.range[i] = make_int2(0, 0);
        else if (P.whole) sh.range[i] = make_int2(ds_range_lo(P.groups, cta, ncta) * P.S, ds_range_lo(P.groups, cta + 1, ncta) * P.S);
        else sh.range[i] = make_int2(ds_range_lo(P.groups * P.S, cta, ncta), ds_range_lo(P.groups * P.S, cta + 1, ncta));
    }
    if (tid_c == 0) {
        for (int s = 0; s < NS; s++) ds_mbar_init(&sh.full[s], 1);
        sh.abort = 0;
        sh.seq = *reinterpret_cast<volatile unsigned long long*>(p.ctr + 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    for (int i = tid_c; i < DS_PARTIAL_SLOTS; i += DS_THREADS) { sh.gcnt[i] = 0; sh.pbusy[i] = 0; }
    for (int i = tid_c; i < DS_MAX_SLICES; i += DS_THREADS) sh.xstate[i] = 0;
    if (tid_c == 0) { sh.pp_state = 0; sh.amax = 0ull; sh.amax_nan = 0; }
    __syncthreads();

    // ---- the weight stream.  Unit number n of this CTA's stream (all phases, in order) lives in ring stage n % NS, and
    // stage i belongs to warp i: the warp waits for the unit, consumes it and at once requests unit n + NS into the same
    // stage with one bulk copy (mbarrier complete_tx).  The requests of a warp therefore run ahead of its compute by a
    // whole ring, across phase boundaries: while the CTA waits for activations or runs attention, the next phase's first
    // units are landing.  (A stage has a single consumer, so that consumer sees every phase of the stage's barrier in
    // order and no "stage free" barrier is needed.)
    DsCursor rf = {0, 0, 0, nullptr};             // the unit this warp requests next
    ds_cursor_seek(phases, p.nphases, sh, rf);
    ds_cursor_advance(phases, p.nphases, sh, rf, cw);
    bool outstanding = false;                     // a copy into this warp's stage is in flight or unconsumed
    int rf_n = cw, req_n = 0;                     // stream numbers of `rf` and of the outstanding request
    int pf_n = -1;                                // highest stream number this warp has pulled into L2
    uint64_t evict_first;                         // weights are read once: their lines leave L2 first
    asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(evict_first));
    auto request = [&]() {                        // lane 0 only
        if (rf.base && !*s_abort) {
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");     // the stage was last read through the generic proxy
            ds_mbar_expect_tx(&sh.full[cw], DS_UNIT_BYTES);
            ds_bulk_load(ring + (size_t)cw * DS_UNIT_BYTES, rf.base + (size_t)rf.u * DS_UNIT_BYTES, DS_UNIT_BYTES, &sh.full[cw], evict_first);
            outstanding = true; req_n = rf_n;
        }
    };
    if (lane == 0) { request(); ds_cursor_advance(phases, p.nphases, sh, rf, NS); rf_n += NS; }

    const int g = lane >> 2, t = lane & 3;
    const unsigned long long seq = sh.seq;
    if (cta == 0) {
        // the embedding row of the step's token becomes the residual stream (tag of "phase -1"): the first o_proj adds to it
        int id = p.rows[0];
        if (id < 0 || id >= p.vocab) id = 0;             // reported by the staging of layer 0
        const uint32_t tag0 = ds_tag(seq, p.nphases, -1);
        for (int k = tid_c; k < p.H; k += DS_THREADS) ds_st_tagged(p.xres + k, __ldg(p.embed + (size_t)id * p.H + k), tag0);
    }
    int nbase = 0;                        // units of this CTA consumed in earlier phases
    auto now = [&]() -> long long { if constexpr (PROF) return clock64(); else return 0; };
    const long long ct0 = now();
    long long c_full = 0, c_stage = 0, c_attn = 0, c_seg = 0;
    long long k_stage[6] = {0, 0, 0, 0, 0, 0}, k_loop[6] = {0, 0, 0, 0, 0, 0};
    for (int ph = 0; ph < p.nphases; ph++) {
        const DsPhase P = phases[ph];
        if (P.kind == DS_ATTN) {
            const long long a0 = now();
            ds_attention(p, P.layer, ph, seq, sh, tid_c, cta, ncta, s_abort);
            c_attn += now() - a0;
            if constexpr (PROF) k_loop[DS_ATTN] += now() - a0;
            continue;
        }
        const int S = P.S, units = P.groups * S;
        const int u0 = sh.range[ph].x, u1 = sh.range[ph].y;
        if (u1 <= u0) continue;                   // nothing of this matrix here: its x is not needed either
        const uint32_t tag = ds_tag(seq, p.nphases, ph);
        long long* tl = (PROF && p.prof && P.layer == p.prof_layer && tid_c == 0) ? p.prof + (size_t)ncta * 32 + (size_t)cta * 64 + P.kind * 8 : nullptr;
        if (tl) tl[0] = (long long)blum_globaltimer();
        ds_sync();                          // the previous phase's warps are done with x and the reduction scratch
        if (tl) tl[1] = (long long)blum_globaltimer();
        // The ring is full and stays so while x is waited for and staged.  So that HBM does not idle meanwhile, every warp
        // pulls the next units of its stage into L2 (a bounded distance ahead: more of it fills the queues that the
        // activation words have to pass through); the requests that follow the stall then hit L2.
        auto pull_ahead = [&]() {            // lane 0 only
            DsCursor pc = rf;
            int pn = rf_n;
            for (int d = 0; d < DS_PREFETCH_UNITS && pc.base; d++) {
                if (pn > pf_n) { ds_bulk_prefetch(pc.base + (size_t)pc.u * DS_UNIT_BYTES, DS_UNIT_BYTES); pf_n = pn; }
                ds_cursor_advance(phases, p.nphases, sh, pc, NS);
                pn += NS;
            }
        };
        if (lane == 0) pull_ahead();
        if (tl) tl[2] = (long long)blum_globaltimer();
        if (ph + 1 < p.nphases) {                 // the norm weight of the phase after this one: towards L2, out of the way
            const DsPhase N = phases[ph + 1 + (phases[ph + 1].kind == DS_ATTN ? 1 : 0)];
            if (N.norm_w) for (int k = tid_c * 32; k < N.K; k += DS_THREADS * 32) asm volatile("prefetch.global.L2 [%0];" ::"l"(N.norm_w + k));
        }
        const long long l0 = now();
        // the last group of the range continues in later CTAs if the range ends inside it
        const bool split_tail = (u1 % S != 0) && ((u1 / S) * S >= u0);
        const int first = (cw - nbase % NS + NS) % NS;
        for (int u = u0 + first; u < u1; u += NS) {
            const int n = nbase + (u - u0);
            const uint32_t par = (uint32_t)((n / NS) & 1);
            const int grp = u / S;
            const int s = u - grp * S;
            // The partial sums the later CTAs publish for this CTA's last group are fetched while the stream is still
            // running (one warp looks once per unit until they are there), so that finishing the group does not start a
            // chain of round trips at the very end of the phase.
            if (split_tail && cw == NS - 1 && *reinterpret_cast<volatile int*>(&sh.pp_state) != ph + 1) {
                float sum;
                if (ds_fetch_partners(p, units, (u1 / S + 1) * S, cta, ncta, tag, lane, false, s_abort, sum)) {
                    if (lane < 16) sh.pp_sum[lane] = sum;
                    __syncwarp();
                    if (lane == 0) { __threadfence_block(); *reinterpret_cast<volatile int*>(&sh.pp_state) = ph + 1; }
                }
            }
            {
                const long long e0 = now();
                ds_ensure_slice(p, P, ph, seq, sh, xpl, xsc, lane, s, s_abort);
                if constexpr (PROF) { if (cw == 0) { c_stage += now() - e0; k_stage[P.kind] += now() - e0; } }
                if (tl && u == u0 + first) tl[3] = (long long)blum_globaltimer();
            }
            const long long f0 = now();
            ds_mbar_wait(&sh.full[cw], par, p, s_abort, 1, n);
            c_full += now() - f0;
            const unsigned char* st = ring + (size_t)cw * DS_UNIT_BYTES;
            // block scales of this lane's two rows and the scales of x for the slice's 16 blocks
            uint32_t dlo[8], dhi[8];
            {
                const uint4 a0 = *reinterpret_cast<const uint4*>(st + 8192 + g * 32), a1 = *reinterpret_cast<const uint4*>(st + 8192 + g * 32 + 16);
                const uint4 b0 = *reinterpret_cast<const uint4*>(st + 8192 + (g + 8) * 32), b1 = *reinterpret_cast<const uint4*>(st + 8192 + (g + 8) * 32 + 16);
                dlo[0] = a0.x; dlo[1] = a0.y; dlo[2] = a0.z; dlo[3] = a0.w; dlo[4] = a1.x; dlo[5] = a1.y; dlo[6] = a1.z; dlo[7] = a1.w;
                dhi[0] = b0.x; dhi[1] = b0.y; dhi[2] = b0.z; dhi[3] = b0.w; dhi[4] = b1.x; dhi[5] = b1.y; dhi[6] = b1.z; dhi[7] = b1.w;
            }
            const int kb0 = s * DS_UNIT_BLOCKS;
            const unsigned char* xb = xpl + (size_t)kb0 * 96 + min(g, 2) * 32 + t * 8;
            float acc0 = 0.f, acc1 = 0.f, acc2 = 0.f, acc3 = 0.f;
#pragma unroll
            for (int j = 0; j < DS_UNIT_BLOCKS; j++) {
                const int4 a = *reinterpret_cast<const int4*>(st + j * 512 + lane * 16);
                // columns 0..2 of B are the three planes of x; the other columns are zero (select, so the warp stays converged)
                int2 b = *reinterpret_cast<const int2*>(xb + j * 96);
                b.x = g < 3 ? b.x : 0; b.y = g < 3 ? b.y : 0;
                int d0, d1, d2, d3;
                asm volatile("mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%10,%10,%10};"
                             : "=r"(d0), "=r"(d1), "=r"(d2), "=r"(d3)
                             : "r"(a.x), "r"(a.y), "r"(a.z), "r"(a.w), "r"(b.x), "r"(b.y), "r"(0));
                const float xs = xsc[kb0 + j];
                const float2 dl = __half22float2(*reinterpret_cast<const __half2*>(&dlo[j >> 1]));
                const float2 dh = __half22float2(*reinterpret_cast<const __half2*>(&dhi[j >> 1]));
                const float sl = ((j & 1) ? dl.y : dl.x) * xs, shi = ((j & 1) ? dh.y : dh.x) * xs;
                acc0 = fmaf((float)d0, sl, acc0);
                acc1 = fmaf((float)d1, sl, acc1);
                acc2 = fmaf((float)d2, shi, acc2);
                acc3 = fmaf((float)d3, shi, acc3);
            }
            __syncwarp();                                           // every lane has read the stage
            if (lane == 0) { outstanding = false; request(); ds_cursor_advance(phases, p.nphases, sh, rf, NS); rf_n += NS; }

            // ---- the unit's 16 row sums: lane t=0 of a row pair holds planes 0 and 1 (columns 0, 1), lane t=1 plane 2
            const long long g0c = now();
            const float p2_lo = __shfl_down_sync(0xffffffffu, acc0, 1), p2_hi = __shfl_down_sync(0xffffffffu, acc2, 1);
            const int pslot = n & (DS_PARTIAL_SLOTS - 1);
            // The warps are not coupled to each other: one whose units keep hitting L2 can run many units ahead of one whose
            // copy is late.  A slot of `partial` is therefore taken only once the group that used it before has been added up.
            if (lane == 0 && *reinterpret_cast<volatile int*>(&sh.pbusy[pslot]) && !*s_abort) {
                const unsigned long long t0 = blum_globaltimer();
                for (uint32_t spin = 1; *reinterpret_cast<volatile int*>(&sh.pbusy[pslot]); spin++)
                    if ((spin & 255u) == 0u && (ds_aborted(p, s_abort) || blum_globaltimer() - t0 > DS_TIMEOUT_NS)) {
                        if (!*s_abort) ds_give_up(p.err, p.ctr, s_abort, 6, n, grp);
                        break;
                    }
            }
            __syncwarp();
            if (t == 0) {
                sh.partial[pslot][g] = fmaf(acc0, 65536.f, fmaf(acc1, 256.f, p2_lo));
                sh.partial[pslot][g + 8] = fmaf(acc2, 65536.f, fmaf(acc3, 256.f, p2_hi));
            }
            // the warp that deposits the last unit of the group's segment in this CTA finishes the group
            const int seg_first = max(u0, grp * S), seg_end = min(u1, (grp + 1) * S);      // units [seg_first, seg_end)
            __syncwarp();
            int last = 0;
            if (lane == 0) {
                sh.pbusy[pslot] = 1;
                __threadfence_block();
                const int gi = grp & (DS_PARTIAL_SLOTS - 1);
                last = (atomicAdd(&sh.gcnt[gi], 1) == (seg_end - seg_first) - 1);
                if (last) sh.gcnt[gi] = 0;
            }
            last = __shfl_sync(0xffffffffu, last, 0);
            if (last) {
                __threadfence_block();
                float v = 0.f;                                               // lane = row of the group (lanes 0..15)
                if (lane < 16)
                    for (int uu = seg_first; uu < seg_end; uu++)             // fixed order: reproducible bit for bit
                        v += sh.partial[(nbase + (uu - u0)) & (DS_PARTIAL_SLOTS - 1)][lane];
                __syncwarp();                                                // every lane has read the slots: hand them back
                if (lane == 0) {
                    __threadfence_block();
                    for (int uu = seg_first; uu < seg_end; uu++) sh.pbusy[(nbase + (uu - u0)) & (DS_PARTIAL_SLOTS - 1)] = 0;
                }
                const bool has_head = (seg_first == grp * S), has_tail = (seg_end == (grp + 1) * S);
                if (!has_head) {
                    // a later slice range of a group that starts in an earlier CTA: publish the partial sums
                    if (lane < 16) ds_st_tagged(p.part + (size_t)cta * 16 + lane, v, tag);
                } else {
                    if (!has_tail) {
                        // the group continues in later CTAs: their partial sums, summed in CTA order, are added as one term
                        float sum;
                        if (*reinterpret_cast<volatile int*>(&sh.pp_state) == ph + 1) { __threadfence_block(); sum = lane < 16 ? sh.pp_sum[lane] : 0.f; }
                        else ds_fetch_partners(p, units, (grp + 1) * S, cta, ncta, tag, lane, true, s_abort, sum);
                        v += sum;
                    }
                    const int row = grp * DS_UNIT_ROWS + lane;
                    // RMSNorm scale: every slice's sum of squares, in slice order (a group that continues in later CTAs has
                    // not needed all slices here yet)
                    float rs = 1.f;
                    if (P.norm_w) {
                        if (!has_tail)
                            for (int sl = 0; sl < S; sl++) ds_ensure_slice(p, P, ph, seq, sh, xpl, xsc, lane, sl, s_abort);
                        float ssq = 0.f;
                        for (int sl = 0; sl < S; sl++) ssq += sh.xss[sl];
                        rs = rsqrtf(ssq / (float)P.K + p.eps);
                    }
                    if (P.kind == DS_GATEUP) {
                        const float upv = __shfl_down_sync(0xffffffffu, v, 8) * rs;         // rows 0-7 of a group are gate rows, 8-15 the up rows
                        const float gate = v * rs;
                        if (lane < 8) ds_st_tagged(p.mid + grp * 8 + lane, upv * (gate * (1.f / (1.f + __expf(-gate)))), tag);
                    } else if (lane < 16) {
                        if (P.kind == DS_QKV) ds_st_tagged(p.qkv + row, v * rs, tag);
                        else if (P.kind == DS_HEAD) {
                            const float lv = v * rs;
                            p.logits[row] = lv;
                            if (p.pick) {
                                // greedy rule of the reference: the LAST index holding the maximum.  Keys order like the
                                // values (both zeros alike) with the row in the low half, so the larger row wins a tie.
                                const bool isnan = lv != lv;
                                uint32_t b = __float_as_uint(lv == 0.f ? 0.f : lv);
                                b = (b & 0x80000000u) ? ~b : (b | 0x80000000u);
                                unsigned long long key = isnan ? 0ull : ((unsigned long long)b << 32) | (uint32_t)row;
#pragma unroll
                                for (int o = 8; o > 0; o >>= 1) {
                                    const unsigned long long other = __shfl_xor_sync(0x0000ffffu, key, o);
                                    key = other > key ? other : key;
                                }
                                const unsigned anynan = __ballot_sync(0x0000ffffu, isnan);
                                if (lane == 0) {
                                    atomicMax(&sh.amax, key);
                                    if (anynan) sh.amax_nan = 1;
                                }
                            }
                        }
                        else {                                                              // o_proj / down: residual add in place
                            // the residual row was written two or three phases ago: one L2 read here.  (Fetching a CTA's residual
                            // rows into shared memory at the start of the phase put a round trip and a barrier in front of
                            // every o_proj / down phase and was 10 us per step slower.)
                            const uint32_t rtag = ds_tag(seq, p.nphases, P.kind == DS_O ? ph - 3 : ph - 2);
                            const float base = ds_wait_value(p.xres + row, rtag, p, s_abort, 2);
                            ds_st_tagged(p.xres + row, base + v, tag);
                        }
                    }
                }
            }
            c_seg += now() - g0c;
        }
        nbase += u1 - u0;
        if constexpr (PROF) k_loop[P.kind] += now() - l0;
        if (tl) tl[4] = (long long)blum_globaltimer();
    }
    // a copy this warp requested and never consumed (only after an abort) has to land before the CTA's shared memory goes away
    if (lane == 0 && outstanding) {
        const unsigned long long t0 = blum_globaltimer();
        while (!ds_mbar_try(&sh.full[cw], (uint32_t)((req_n / NS) & 1)) && blum_globaltimer() - t0 < DS_TIMEOUT_NS) {}
    }
    if (PROF && p.prof && tid_c == 0) {
        long long* o = p.prof + cta * 32;
        for (int k = 0; k < 6; k++) { o[8 + 3 * k] = k_stage[k]; o[9 + 3 * k] = k_loop[k]; o[10 + 3 * k] = 0; }
        o[0] = now() - ct0; o[1] = c_full; o[2] = 0; o[3] = c_stage; o[4] = c_attn; o[5] = c_seg; o[6] = 0; o[7] = 0;
    }
    if (p.pick) {
        // ---- next token inside the kernel: every CTA publishes its best (key, row); CTA 0 takes the maximum, and only when
        // a NaN was seen anywhere replays the reference's sequential fold over the finished logits
        ds_sync();                                                   // this CTA's head rows are all accounted for
        const uint32_t atag = ds_tag(seq, p.nphases, p.nphases);
        if (tid_c == 0) {
            const unsigned long long key = sh.amax;
            __threadfence();                                         // this CTA's logits before its word
            ds_st_tagged(p.amax + (size_t)cta * 2, __uint_as_float((uint32_t)(key >> 32)), atag);
            ds_st_tagged(p.amax + (size_t)cta * 2 + 1, __int_as_float(sh.amax_nan ? -2 : (key ? (int)(uint32_t)key : -1)), atag);
        }
        if (cta == 0) {
            ds_sync();
            if (tid_c == 0) { sh.amax = 0ull; sh.amax_nan = 0; }
            ds_sync();
            for (int c = tid_c; c < ncta; c += DS_THREADS) {
                const unsigned long long hi = ds_wait_word(p.amax + (size_t)c * 2, atag, p, s_abort, 8);
                const unsigned long long lo = ds_wait_word(p.amax + (size_t)c * 2 + 1, atag, p, s_abort, 8);
                const int r = (int)(uint32_t)lo;
                if (r == -2) sh.amax_nan = 1;
                else if (r >= 0) atomicMax(&sh.amax, ((hi & 0xffffffffull) << 32) | (uint32_t)r);
            }
            ds_sync();
            if (tid_c == 0 && !*s_abort) {
                int tok = (int)(uint32_t)sh.amax;
                if (sh.amax_nan) {
                    __threadfence();
                    float cur = *reinterpret_cast<volatile float*>(p.logits); tok = 0;
                    for (int j = 1; j < p.vocab; j++) { const float v = *reinterpret_cast<volatile float*>(p.logits + j); if (!(cur > v)) { cur = v; tok = j; } }
                }
                p.next[0] = tok;
                if (p.pick == 2) {
                    // every CTA has finished every phase (its word is here), so nobody reads the row any more
                    p.rows[0] = tok;
                    p.rows[2 * p.max_rows] += 1;
                    p.rows[3 * p.max_rows] += 1;
                    if (p.hist) p.hist[p.hist_step] = tok;
                }
            }
        }
    }
    // the launch number makes the next launch's tags new; whoever reads it has started, and nobody can finish before everybody
    // who has work has started (they all feed the last phase)
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

size_t blum_ds_smem_bytes(int kmax) { return (size_t)DS_STAGES * DS_UNIT_BYTES + (size_t)kmax * 3 + (size_t)kmax / 32 * 4 + DS_MAX_PHASES * sizeof(DsPhase) + 128; }

int blum_ds_launch(blum_ctx* ctx, const DsParams& p) {
    static bool attr_set[64] = {};
    const size_t smem = blum_ds_smem_bytes(p.kmax);
    if (ctx->device >= 0 && ctx->device < 64 && !attr_set[ctx->device]) {
        BLUM_CUDA(ctx, cudaFuncSetAttribute(decode_stream_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)(ctx->smem_optin - 24 * 1024)));
        BLUM_CUDA(ctx, cudaFuncSetAttribute(decode_stream_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)(ctx->smem_optin - 24 * 1024)));
        attr_set[ctx->device] = true;
    }
    void* args[] = {(void*)&p};
    const void* kern = p.prof ? (const void*)decode_stream_kernel<true> : (const void*)decode_stream_kernel<false>;
    BLUM_CUDA(ctx, cudaLaunchCooperativeKernel(kern, dim3(ctx->sm_count), dim3(DS_THREADS), args, smem, ctx->stream));
    ctx->launches++;
    return BLUM_OK;
}
