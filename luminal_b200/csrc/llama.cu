// Llama-architecture decoder as one object: weights, paged KV pool, work buffers and captured
// CUDA graphs of the decode step.
//
// The reference builds this model as a graph of ~10^3 primitive nodes per token
// (examples/llama/src/model.rs:171-248 in luminal) and interprets it node by node with one allocation
// and one launch each (src/graph.rs:191-224); the decode loop copies 128 256 logits to the host and
// takes the argmax there (examples/llama/src/main.rs:152-181,194-198).  Here a single-sequence decode step
// (f32 activations and cache, head_dim 128, dimensions in multiples of 512) is ONE persistent kernel with a
// continuous weight stream (decode_stream.cu) followed by the on-device argmax.  Other small batches
// (up to GEMV_ROWS rows) are 5 launches per layer, captured once in a CUDA graph and replayed:
//   [RMSNorm + fused q/k/v GEMV] [RoPE + KV append + paged GQA attention]
//   [o_proj GEMV + residual] [RMSNorm + gate/up GEMV + SwiGLU] [down GEMV + residual]
// plus the embedding gather, the [final norm + LM head GEMV] and the argmax; only token ids cross PCIe.
// Steps with more rows (prefill, large batches) run the unfused sequence norm -> matmul -> elementwise
// through the same entry points a luminal operator would call.
#include "kv.cuh"
#include "decode_stream.cuh"
#include <algorithm>
#include <map>
#include <stdlib.h>
#include <string.h>
#include <string>

#define GEMV_ROWS 4   // rows of x up to which the fused GEMV kernels are used

struct LayerW {
    float* attn_norm = nullptr;
    float* ffn_norm = nullptr;
    float *q_norm = nullptr, *k_norm = nullptr;     // per-head norm weights [head_dim] (qk_norm models)
    blum_q8_weight *wqkv = nullptr, *wo = nullptr, *wgate = nullptr, *wup = nullptr, *wdown = nullptr;
    blum_q8_weight* wgu = nullptr;     // gate rows then up rows in one allocation: wgate / wup are views of it
};

// The batch-1 step as one persistent kernel (decode_stream.cu): stream-packed copies of the weights, the phase table and
// the counters its grid barriers use.
struct StreamPlan {
    bool built = false;
    uint64_t weights_version = 0;          // version of the model's weights the packed copy was made from
    unsigned char* packed = nullptr;
    DsPhase* d_phases = nullptr;
    std::vector<DsPhase> h_phases;         // host copy: where each matrix's packed units start
    int nphases = 0, kmax = 0, grid = 0;
    unsigned long long* words = nullptr;   // tagged activation words: xres | qkv | attn | mid | part | attn_part
    size_t words_bytes = 0;
    unsigned long long *xres = nullptr, *qkv = nullptr, *attn = nullptr, *mid = nullptr, *part = nullptr, *attn_part = nullptr, *amax = nullptr;
    unsigned long long* ctr = nullptr;
    size_t ctr_bytes = 0;
    long long* prof = nullptr;             // development aid (blum_llama_stream_profile)
    int64_t last_ctx_len = 1;              // context length of the last launch (blum_llama_stream_kernel_us)
};
#define DS_MAX_SPLITS 16

struct blum_llama {
    blum_llama_cfg cfg;
    StreamPlan sp;
    int decode_path = 0;                          // 0: persistent stream kernel when the shape allows it, 1: per-op kernels in a CUDA graph
    int stream_state = -1;                        // -1 unknown, 0 unsupported, 1 supported
    int pack_state = -1;                          // the same for the packed copy alone (the rows matmul)
    uint64_t weights_version = 1;
    int nq = 0, nkv = 0, ffn = 0, vocab = 0;      // local (tensor-parallel shard) sizes
    float* embed_f32 = nullptr;
    blum_q8_weight* embed_q8 = nullptr;
    float* out_norm = nullptr;
    blum_q8_weight* head = nullptr;
    std::vector<LayerW> L;
    blum_kv* kv = nullptr;
    int max_rows = 0;
    void *x = nullptr, *xn = nullptr, *qkv = nullptr, *q = nullptr, *attn = nullptr, *mid = nullptr, *gate = nullptr, *up = nullptr;
    float* logits = nullptr;                      // [max_seqs][vocab]
    int32_t* d_rows = nullptr;                    // ids | seq | pos | ctx, each [max_rows]
    int32_t* d_next = nullptr;                    // [max_seqs]
    int32_t* d_pairs = nullptr;                   // tensor parallel: [tp_size][max_seqs] (max logit bits, global index)
    int32_t* d_hist = nullptr;                    // device-resident loop history
    int hist_cap = 0;
    int32_t* h_rows = nullptr;                    // pinned mirror of d_rows
    int32_t* h_next = nullptr;                    // pinned
    void* attn_scratch = nullptr;
    int max_splits = 1;
    int pre_seq = -1; int64_t pre_p0 = 0;                    // the prompt chunk forward_rows is running (prefill only)
    std::map<std::pair<int, int>, cudaGraphExec_t> graphs;   // (rows, nsplit) -> captured decode step
    std::map<std::pair<int, int>, int> graph_nodes;          // kernel nodes per captured step
    blum_comm* comm = nullptr;
    float temperature = 0.f, top_p = 1.f;   // temperature 0: greedy (the reference's sampler)
    uint64_t sample_seed = 0;
    void* sample_scratch = nullptr;    // integer weights of the sampled rows [max_seqs][vocab]
    void* rows_scratch = nullptr;      // digitised activations and partial sums of the prompt-chunk matmul (prefill_rows.cu)
    size_t rows_scratch_bytes = 0;
    blum_peer* peer = nullptr;         // peer-mapped exchange area: row-parallel sums without a library collective
    int64_t weight_bytes = 0;
};

uint64_t blum_fnv1a(const char* s) {
    uint64_t h = 0xcbf29ce484222325ull;
    for (; *s; s++) { h ^= (uint8_t)*s; h *= 0x100000001b3ull; }
    return h;
}

__global__ void fill_f32_kernel(float* p, int64_t n, float v) {
    for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x) p[i] = v;
}

// after a device-resident step: feed the sampled token back and advance position / context
__global__ void advance_rows_kernel(int32_t* rows, int max_rows, const int32_t* next, int32_t* hist, int step, int B) {
    const int b = threadIdx.x;
    if (b < B) {
        rows[b] = next[b];
        rows[2 * max_rows + b] += 1;
        rows[3 * max_rows + b] += 1;
        if (hist) hist[step * B + b] = next[b];
    }
}

static size_t act_bytes(const blum_llama* m, int64_t elems) { return (size_t)elems * blum_dtype_size(m->cfg.act_dtype); }

#define TRY(call) do { int rc__ = (call); if (rc__) return rc__; } while (0)

// next-token choice for `rows` rows of logits: the reference's greedy rule, or the temperature / top-p sampler keyed by
// (seed, sequence slot, position) of each row
static int pick_tokens(blum_ctx* ctx, blum_llama* m, int rows, const int32_t* seq, const int32_t* pos) {
    if (m->temperature > 0.f)
        return blum_sample_top_p(ctx, m->logits, rows, m->vocab, m->temperature, m->top_p, m->sample_seed, seq, pos, m->sample_scratch, m->d_next);
    return blum_argmax(ctx, m->logits, BLUM_F32, rows, m->vocab, m->d_next);
}

static bool stream_supported(blum_ctx* ctx, blum_llama* m);
static int build_stream_plan(blum_ctx* ctx, blum_llama* m);

static bool pack_supported(blum_ctx* ctx, blum_llama* m);
static int ensure_packed(blum_ctx* ctx, blum_llama* m);

// More than four rows of f32 activations (prompt chunks, small batches): the projections read the stream-packed weights once
// per 32 rows on the integer tensor path (prefill_rows.cu).  Blocks of ROWS_BLOCK rows share one scratch area.  With 16-bit
// activations the kernels that convert the weights are as fast or faster at these row counts (measured: 55 against 69 us
// at 16 rows on 8192 x 28672) and need no second copy of the weights, so those models do not take this path.
#define ROWS_BLOCK 128
static int rows_mm(blum_ctx* ctx, blum_llama* m, int phase, const void* x, int64_t ldx, void* y, int64_t ldy, int R, int swiglu, int ydt = -1) {
    const DsPhase& P = m->sp.h_phases[(size_t)phase];
    const int64_t rows_total = (int64_t)P.groups * DS_UNIT_ROWS;
    const int adt = m->cfg.act_dtype;
    if (ydt < 0) ydt = adt;
    const size_t xs = blum_dtype_size((blum_dtype)adt), ys = blum_dtype_size((blum_dtype)ydt);
    for (int r0 = 0; r0 < R; r0 += ROWS_BLOCK) {
        const int n = std::min(ROWS_BLOCK, R - r0);
        TRY(blum_rows_matmul(ctx, P.w, rows_total, P.K, (const char*)x + (size_t)r0 * ldx * xs, adt, ldx, n, swiglu,
                             (char*)y + (size_t)r0 * ldy * ys, ydt, ldy, m->rows_scratch, m->rows_scratch_bytes));
    }
    return BLUM_OK;
}

// ------------------------------------------------------------------ forward for R rows
// rows are described by d_rows (ids, seq, pos, ctx); head_rows = rows whose logits are needed
// (all for decode, the last one for prefill); everything is enqueued on ctx->stream.
static int forward_rows(blum_ctx* ctx, blum_llama* m, int R, int nsplit, bool last_row_only) {
    const blum_llama_cfg& c = m->cfg;
    const blum_dtype adt = (blum_dtype)c.act_dtype;
    const int H = c.hidden, d = c.head_dim;
    const int32_t *ids = m->d_rows, *seq = m->d_rows + m->max_rows, *pos = m->d_rows + 2 * m->max_rows, *ctxl = m->d_rows + 3 * m->max_rows;
    if (m->embed_q8) TRY(blum_q8_0_gather(ctx, m->embed_q8, ids, R, m->x, adt));
    else TRY(blum_gather(ctx, m->embed_f32, BLUM_F32, c.vocab, H, ids, R, m->x, adt));
    const bool fused = R <= GEMV_ROWS;
    // more rows than the GEMV takes at once and the model has (or can have) the stream-packed weights
    const bool rows_path = !fused && m->decode_path == 0 && adt == BLUM_F32 && pack_supported(ctx, m);
    if (rows_path) TRY(ensure_packed(ctx, m));
    // Programmatic dependent launch belongs to the fused GEMV chain, where every kernel lets its successor start early.
    // Outside it (row counts that take the GEMM kernels) the attribute buys nothing and is switched off.
    struct PdlGuard {
        blum_ctx* c; bool saved;
        PdlGuard(blum_ctx* c_, bool keep) : c(c_), saved(c_->pdl) { if (!keep) c->pdl = false; }
        ~PdlGuard() { c->pdl = saved; }
    } pdl_guard(ctx, fused);
    for (int l = 0; l < c.layers; l++) {
        const LayerW& w = m->L[l];
        if (fused) {
            TRY(blum_gemv_dispatch(ctx, w.wqkv, nullptr, m->x, adt, w.attn_norm, c.rms_eps, nullptr, m->qkv, adt, R));
        } else {
            // (for l > 0 the previous layer's down-projection add already produced xn = rmsnorm(x) with this layer's weight)
            if (l == 0) TRY(blum_rmsnorm(ctx, m->x, nullptr, w.attn_norm, c.rms_eps, m->xn, nullptr, adt, R, H));
            if (rows_path) TRY(rows_mm(ctx, m, 5 * l, m->xn, H, m->qkv, (int64_t)(m->nq + 2 * m->nkv) * d, R, 0));
            else TRY(blum_q8_0_matmul(ctx, w.wqkv, m->xn, adt, m->qkv, adt, R));
        }
        // The sibling decoders (per-head q/k norm, half-split rotary pairs) get their glue from one extra kernel that works in
        // place on the fused rows; the kernels after it then rotate by zero angles.
        float theta = c.rope_theta;
        if (c.qk_norm || c.rope_mode != 0) {
            TRY(blum_qk_norm_rope(ctx, m->qkv, adt, pos, R, m->nq, m->nkv, d, c.qk_norm ? w.q_norm : nullptr, c.qk_norm ? w.k_norm : nullptr,
                                  c.rms_eps, c.rope_theta, c.rope_mode));
            theta = 0.f;
        }
        if (!last_row_only) {
            // decode: every row is the next token of its own sequence -> RoPE + append + attention in one launch
            TRY(blum_attn_decode_fused(ctx, m->kv, l, m->qkv, adt, m->nq, theta, seq, ctxl, R, nsplit, m->attn_scratch, m->attn));
        } else {
            TRY(blum_rope_kv_append(ctx, m->kv, l, m->qkv, adt, m->nq, theta, seq, pos, R, m->q));
            if (m->pre_seq >= 0 && blum_attn_prefill_mma_covers(adt, m->kv->dtype, d, m->kv->page_size))
                TRY(blum_attn_prefill_mma(ctx, m->kv, l, m->q, adt, m->nq, m->pre_seq, m->pre_p0, R, m->attn));
            else
                TRY(blum_attn_rows(ctx, m->kv, l, m->q, adt, m->nq, seq, ctxl, R, nsplit, m->attn_scratch, m->attn));
        }
        // row-parallel projections: with tensor parallelism every rank holds a K-slice, the partial products are
        // summed over ranks (NCCL all-reduce) and only then added to the residual stream
        const bool tp = c.tp_size > 1;
        if (tp && !m->comm) return blum_fail(ctx, BLUM_ERR_STATE, "llama: tp_size=%d but no communicator was set (blum_llama_set_comm)", c.tp_size);
        // with a peer-mapped exchange area and few rows, the projection writes its partial product into the area and one
        // kernel sums over ranks, adds the residual and normalises (peer_reduce.cu); otherwise NCCL does the sum
        const bool pull = tp && m->peer && R <= blum_peer_max_rows(m->peer);
        void* part0 = pull ? blum_peer_slot(m->peer, 0) : nullptr;
        void* part1 = pull ? blum_peer_slot(m->peer, 1) : nullptr;
        if (fused) {
            if (!tp) {
                TRY(blum_gemv_dispatch(ctx, w.wo, nullptr, m->attn, adt, nullptr, 0.f, m->x, m->x, adt, R));
            } else if (pull) {
                TRY(blum_gemv_dispatch(ctx, w.wo, nullptr, m->attn, adt, nullptr, 0.f, nullptr, part0, adt, R));
                TRY(blum_allreduce_fused(ctx, m->peer, 0, m->x, nullptr, 0.f, nullptr, m->x, adt, R, H));
            } else {
                TRY(blum_gemv_dispatch(ctx, w.wo, nullptr, m->attn, adt, nullptr, 0.f, nullptr, m->xn, adt, R));
                TRY(blum_allreduce_sum(ctx, m->comm, m->xn, (int64_t)R * H, adt, 0));
                TRY(blum_add(ctx, m->x, m->xn, m->x, adt, (int64_t)R * H));
            }
            TRY(blum_gemv_dispatch(ctx, w.wgate, w.wup, m->x, adt, w.ffn_norm, c.rms_eps, nullptr, m->mid, adt, R));
            if (!tp) {
                TRY(blum_gemv_dispatch(ctx, w.wdown, nullptr, m->mid, adt, nullptr, 0.f, m->x, m->x, adt, R));
            } else if (pull) {
                TRY(blum_gemv_dispatch(ctx, w.wdown, nullptr, m->mid, adt, nullptr, 0.f, nullptr, part1, adt, R));
                TRY(blum_allreduce_fused(ctx, m->peer, 1, m->x, nullptr, 0.f, nullptr, m->x, adt, R, H));
            } else {
                TRY(blum_gemv_dispatch(ctx, w.wdown, nullptr, m->mid, adt, nullptr, 0.f, nullptr, m->xn, adt, R));
                TRY(blum_allreduce_sum(ctx, m->comm, m->xn, (int64_t)R * H, adt, 0));
                TRY(blum_add(ctx, m->x, m->xn, m->x, adt, (int64_t)R * H));
            }
        } else {
            // residual add and the following RMSNorm in one kernel: x <- x + proj (rounded as the separate add would),
            // xn <- rmsnorm(x) * weight.  The projection lands in the gate buffer, which is free here.
            if (rows_path) TRY(rows_mm(ctx, m, 5 * l + 2, m->attn, (int64_t)m->nq * d, pull ? part0 : m->gate, H, R, 0));
            else TRY(blum_q8_0_matmul(ctx, w.wo, m->attn, adt, pull ? part0 : m->gate, adt, R));
            if (pull) {
                TRY(blum_allreduce_fused(ctx, m->peer, 0, m->x, w.ffn_norm, c.rms_eps, m->xn, m->x, adt, R, H));
            } else {
                if (tp) TRY(blum_allreduce_sum(ctx, m->comm, m->gate, (int64_t)R * H, adt, 0));
                TRY(blum_rmsnorm(ctx, m->x, m->gate, w.ffn_norm, c.rms_eps, m->xn, m->x, adt, R, H));
            }
            if (rows_path) {
                TRY(rows_mm(ctx, m, 5 * l + 3, m->xn, H, m->mid, m->ffn, R, 1));       // SwiGLU in the finishing pass
                TRY(rows_mm(ctx, m, 5 * l + 4, m->mid, m->ffn, pull ? part1 : m->gate, H, R, 0));
            } else {
                TRY(blum_q8_0_matmul(ctx, w.wgu, m->xn, adt, m->gate, adt, R));            // [R][gate | up]
                TRY(blum_swiglu_rows(ctx, m->gate, m->mid, adt, R, m->ffn));
                TRY(blum_q8_0_matmul(ctx, w.wdown, m->mid, adt, pull ? part1 : m->gate, adt, R));
            }
            if (pull) {
                const bool more = l + 1 < c.layers;
                TRY(blum_allreduce_fused(ctx, m->peer, 1, m->x, more ? m->L[l + 1].attn_norm : nullptr, c.rms_eps, more ? m->xn : nullptr, m->x, adt, R, H));
            } else {
                if (tp) TRY(blum_allreduce_sum(ctx, m->comm, m->gate, (int64_t)R * H, adt, 0));
                if (l + 1 < c.layers) TRY(blum_rmsnorm(ctx, m->x, m->gate, m->L[l + 1].attn_norm, c.rms_eps, m->xn, m->x, adt, R, H));
                else TRY(blum_add(ctx, m->x, m->gate, m->x, adt, (int64_t)R * H));
            }
        }
    }
    // head: the reference computes logits for every position and keeps the last (examples/llama/src/main.rs:58-61);
    // only the kept rows are computed here
    const int HR = last_row_only ? 1 : R;
    const char* xh = (const char*)m->x + (last_row_only ? act_bytes(m, (int64_t)(R - 1) * H) : 0);
    if (HR <= GEMV_ROWS) {
        TRY(blum_gemv_dispatch(ctx, m->head, nullptr, xh, adt, m->out_norm, c.rms_eps, nullptr, m->logits, BLUM_F32, HR));
    } else {
        TRY(blum_rmsnorm(ctx, xh, nullptr, m->out_norm, c.rms_eps, m->xn, nullptr, adt, HR, H));
        if (rows_path) TRY(rows_mm(ctx, m, 5 * c.layers, m->xn, H, m->logits, m->vocab, HR, 0, BLUM_F32));
        else TRY(blum_q8_0_matmul(ctx, m->head, m->xn, adt, m->logits, BLUM_F32, HR));
    }
    if (c.tp_size > 1) {
        // vocabulary-parallel head: local (max, global index) per row, all-gather of the pairs, final pick
        TRY(blum_argmax_pairs(ctx, m->logits, HR, m->vocab, c.tp_rank * m->vocab, m->d_pairs + (size_t)c.tp_rank * HR * 2));
        TRY(blum_allgather(ctx, m->comm, m->d_pairs + (size_t)c.tp_rank * HR * 2, m->d_pairs, (int64_t)HR * 8, 0));
        TRY(blum_pick_pairs(ctx, m->d_pairs, c.tp_size, HR, m->d_next));
        return BLUM_OK;
    }
    TRY(pick_tokens(ctx, m, HR, seq + (last_row_only ? R - 1 : 0), pos + (last_row_only ? R - 1 : 0)));
    return BLUM_OK;
}

static int pick_nsplit(const blum_ctx* ctx, const blum_llama* m, int R, int64_t max_ctx_len) {
    // enough CTAs for several waves (ragged context lengths balance out), but no split shorter than 256 positions
    int by_grid = (6 * ctx->sm_count + R * m->nkv - 1) / (R * m->nkv);
    int by_len = (int)((max_ctx_len + 255) / 256);
    int n = by_grid < by_len ? by_grid : by_len;
    if (n > m->max_splits) n = m->max_splits;
    return n < 1 ? 1 : n;
}

// ------------------------------------------------------------------ persistent stream kernel: plan and launch
static bool stream_supported(blum_ctx* ctx, blum_llama* m) {
    if (m->stream_state >= 0) return m->stream_state == 1;
    const blum_llama_cfg& c = m->cfg;
    const int d = c.head_dim, H = c.hidden, qd = m->nq * d;
    bool ok = c.tp_size == 1 && c.act_dtype == BLUM_F32 && c.kv_dtype == BLUM_F32 && d == 128 && !c.embed_q8 && !c.qk_norm && c.rope_mode == 0 && !c.tie_head;
    ok = ok && H % DS_UNIT_K == 0 && qd % DS_UNIT_K == 0 && m->ffn % DS_UNIT_K == 0 && 5 * c.layers + 1 <= DS_MAX_PHASES;
    ok = ok && ((m->nq + 2 * m->nkv) * d) % DS_UNIT_ROWS == 0 && H % DS_UNIT_ROWS == 0 && m->ffn % 8 == 0 && m->vocab % DS_UNIT_ROWS == 0;
    int coop = 0;
    if (ok) ok = cudaDeviceGetAttribute(&coop, cudaDevAttrCooperativeLaunch, ctx->device) == cudaSuccess && coop != 0;
    if (ok) {
        const int kmax = std::max(H, std::max(qd, m->ffn));
        // ring (one stage per warp) + x as three byte planes + its block scales, beside ~22 KB of static shared memory
        ok = blum_ds_smem_bytes(kmax) + 24 * 1024 <= ctx->smem_optin;
        m->sp.kmax = kmax; m->sp.grid = ctx->sm_count;
    }
    m->stream_state = ok ? 1 : 0;
    return ok;
}

static void free_stream_plan(blum_llama* m) {
    StreamPlan& sp = m->sp;
    void* bufs[] = {sp.packed, sp.d_phases, sp.words, sp.ctr, sp.prof};
    sp.prof = nullptr; sp.words = nullptr;
    for (void* b : bufs) if (b) cudaFree(b);
    sp.packed = nullptr; sp.d_phases = nullptr; sp.ctr = nullptr;
    sp.built = false;
}

static int build_stream_plan(blum_ctx* ctx, blum_llama* m);

// The packed copy doubles the weight memory: models the persistent kernel covers always have it; others get it when their
// shapes fit the 16 x 512 unit and the device has room for it beside what is already allocated.
static bool pack_supported(blum_ctx* ctx, blum_llama* m) {
    if (m->pack_state >= 0) return m->pack_state == 1;
    bool ok = stream_supported(ctx, m);
    if (!ok && m->cfg.act_dtype == BLUM_F32) {
        const blum_llama_cfg& c = m->cfg;
        const int d = c.head_dim, H = c.hidden;
        const int64_t qkv_rows = (int64_t)(m->nq + 2 * m->nkv) * d, qd = (int64_t)m->nq * d;
        ok = H % DS_UNIT_K == 0 && qd % DS_UNIT_K == 0 && m->ffn % DS_UNIT_K == 0 && 5 * c.layers + 1 <= DS_MAX_PHASES &&
             qkv_rows % DS_UNIT_ROWS == 0 && H % DS_UNIT_ROWS == 0 && m->ffn % 8 == 0 && m->vocab % DS_UNIT_ROWS == 0 && m->head != nullptr;
        if (ok) {
            const size_t total = (blum_ds_packed_bytes(qkv_rows, H) + blum_ds_packed_bytes(H, qd) + blum_ds_packed_bytes(2ll * m->ffn, H) +
                                  blum_ds_packed_bytes(H, m->ffn)) * (size_t)c.layers + blum_ds_packed_bytes(m->vocab, H);
            size_t free_b = 0, total_b = 0;
            ok = cudaMemGetInfo(&free_b, &total_b) == cudaSuccess && free_b > total + ((size_t)4 << 30);
        }
    }
    m->pack_state = ok ? 1 : 0;
    return ok;
}
// Everything the packed-rows matmul needs exists after this call (never inside a stream capture: it allocates).
static int ensure_packed(blum_ctx* ctx, blum_llama* m) {
    if (!m->sp.built || m->sp.weights_version != m->weights_version) TRY(build_stream_plan(ctx, m));
    if (!m->rows_scratch) {
        const int H = m->cfg.hidden, d = m->cfg.head_dim;
        int64_t nk = std::max<int64_t>((int64_t)(H / DS_UNIT_K) * 2 * m->ffn, (int64_t)(m->ffn / DS_UNIT_K) * H);
        nk = std::max<int64_t>(nk, (int64_t)(H / DS_UNIT_K) * (m->nq + 2 * m->nkv) * d);
        nk = std::max<int64_t>(nk, (int64_t)(H / DS_UNIT_K) * m->vocab);
        m->rows_scratch_bytes = blum_rows_scratch_bytes(ROWS_BLOCK, std::max<int64_t>(std::max(H, m->ffn), (int64_t)m->nq * d), nk);
        BLUM_CUDA(ctx, cudaMalloc(&m->rows_scratch, m->rows_scratch_bytes));
    }
    return BLUM_OK;
}

// Packs every matrix of the model into stream units (once per set of weights) and writes the phase table.
static int build_stream_plan(blum_ctx* ctx, blum_llama* m) {
    StreamPlan& sp = m->sp;
    const blum_llama_cfg& c = m->cfg;
    const int d = c.head_dim, H = c.hidden, L = c.layers;
    const int64_t qkv_rows = (int64_t)(m->nq + 2 * m->nkv) * d, qd = (int64_t)m->nq * d;
    const size_t b_qkv = blum_ds_packed_bytes(qkv_rows, H), b_o = blum_ds_packed_bytes(H, qd), b_gu = blum_ds_packed_bytes(2ll * m->ffn, H),
                 b_down = blum_ds_packed_bytes(H, m->ffn), b_head = blum_ds_packed_bytes(m->vocab, H);
    const size_t total = (b_qkv + b_o + b_gu + b_down) * (size_t)L + b_head;
    if (!sp.packed) {
        cudaError_t e = cudaMalloc((void**)&sp.packed, total);
        if (e == cudaSuccess) e = cudaMalloc((void**)&sp.d_phases, sizeof(DsPhase) * (size_t)(5 * L + 1));
        const size_t n_x = (size_t)H, n_qkv = (size_t)qkv_rows, n_attn = (size_t)qd, n_mid = (size_t)m->ffn, n_part = (size_t)sp.grid * 16,
                     n_ap = (size_t)m->nq * DS_MAX_SPLITS * 130;
        sp.words_bytes = (n_x + n_qkv + n_attn + n_mid + n_part + n_ap + 2 * (size_t)sp.grid) * sizeof(unsigned long long);
        if (e == cudaSuccess) e = cudaMalloc((void**)&sp.words, sp.words_bytes);
        if (e == cudaSuccess) {
            sp.xres = sp.words; sp.qkv = sp.xres + n_x; sp.attn = sp.qkv + n_qkv; sp.mid = sp.attn + n_attn; sp.part = sp.mid + n_mid;
            sp.attn_part = sp.part + n_part; sp.amax = sp.attn_part + n_ap;
        }
        sp.ctr_bytes = 8 * sizeof(unsigned long long);
        if (e == cudaSuccess) e = cudaMalloc((void**)&sp.ctr, sp.ctr_bytes);
        if (e != cudaSuccess) {
            free_stream_plan(m);
            return blum_fail(ctx, BLUM_ERR_OOM, "llama: no memory for the stream-packed weights (%zu bytes): %s", total, cudaGetErrorString(e));
        }
    }
    BLUM_CUDA(ctx, cudaMemsetAsync(sp.ctr, 0, sp.ctr_bytes, ctx->stream));
    BLUM_CUDA(ctx, cudaMemsetAsync(sp.words, 0, sp.words_bytes, ctx->stream));     // tag 0 is never a valid tag
    std::vector<DsPhase> ph;
    unsigned char* at = sp.packed;
    auto add = [&](int kind, int layer, const blum_q8_weight* w, const blum_q8_weight* w_up, const float* norm_w, size_t bytes) -> int {
        DsPhase P = {};
        P.kind = kind; P.layer = layer; P.norm_w = norm_w;
        if (w) {
            TRY(blum_ds_pack(ctx, w, w_up, at));
            P.w = at; P.K = (int)w->K; P.S = (int)(w->K / DS_UNIT_K); P.groups = (int)((w_up ? 2 * w->N : w->N) / DS_UNIT_ROWS);
            // a phase whose whole share fits the ring is short: whole groups per CTA
            P.whole = ((int64_t)P.groups * P.S <= (int64_t)2 * DS_STAGES * sp.grid) ? 1 : 0;
            at += bytes;
        }
        ph.push_back(P);
        return BLUM_OK;
    };
    for (int l = 0; l < L; l++) {
        const LayerW& w = m->L[l];
        TRY(add(DS_QKV, l, w.wqkv, nullptr, w.attn_norm, b_qkv));
        TRY(add(DS_ATTN, l, nullptr, nullptr, nullptr, 0));
        TRY(add(DS_O, l, w.wo, nullptr, nullptr, b_o));
        TRY(add(DS_GATEUP, l, w.wgate, w.wup, w.ffn_norm, b_gu));
        TRY(add(DS_DOWN, l, w.wdown, nullptr, nullptr, b_down));
    }
    TRY(add(DS_HEAD, L, m->head, nullptr, m->out_norm, b_head));
    sp.nphases = (int)ph.size();
    BLUM_CUDA(ctx, cudaMemcpyAsync(sp.d_phases, ph.data(), sizeof(DsPhase) * ph.size(), cudaMemcpyHostToDevice, ctx->stream));
    BLUM_CUDA(ctx, cudaStreamSynchronize(ctx->stream));      // ph is a host temporary
    sp.h_phases = ph;
    sp.built = true;
    sp.weights_version = m->weights_version;
    return BLUM_OK;
}

// pick: 0 logits only, 1 greedy token into d_next[0], 2 also fed back into the step's row (hist[hist_step] records it)
static int run_stream_launch(blum_ctx* ctx, blum_llama* m, int64_t max_ctx_len, int pick = 0, int hist_step = 0) {
    StreamPlan& sp = m->sp;
    if (!sp.built || sp.weights_version != m->weights_version) TRY(build_stream_plan(ctx, m));
    sp.last_ctx_len = max_ctx_len;
    const blum_llama_cfg& c = m->cfg;
    DsParams p = {};
    p.phases = sp.d_phases; p.nphases = sp.nphases;
    p.kv = kv_view(m->kv); p.max_seqs = m->kv->max_seqs; p.max_rows = m->max_rows;
    p.rows = m->d_rows; p.embed = m->embed_f32;
    p.xres = sp.xres; p.qkv = sp.qkv; p.attn = sp.attn; p.mid = sp.mid; p.logits = m->logits;
    p.part = sp.part; p.attn_part = sp.attn_part; p.amax = sp.amax; p.ctr = sp.ctr;
    p.H = c.hidden; p.nq = m->nq; p.nkv = m->nkv; p.ffn = m->ffn; p.vocab = m->vocab;
    // enough (head, split) items to occupy the grid once contexts are long; one split per 256 cached positions at most
    int nsplit = (int)std::min<int64_t>(DS_MAX_SPLITS, std::max<int64_t>(1, max_ctx_len / 256));
    p.nsplit = nsplit; p.kmax = sp.kmax;
    p.eps = c.rms_eps; p.scale = 1.0f / sqrtf((float)c.head_dim);
    blum_rope_freqs(c.rope_theta, c.head_dim, &p.freqs);
    p.err = ctx->dev_error;
    p.prof = sp.prof;
    p.prof_layer = 3;
    p.pick = pick; p.next = m->d_next; p.hist = m->d_hist; p.hist_step = hist_step;
    return blum_ds_launch(ctx, p);
}
// feed_step >= 0: the caller wants the token fed back on the device (decode loop); *fed says whether this step did it
static int run_stream_step(blum_ctx* ctx, blum_llama* m, int64_t max_ctx_len, int feed_step, bool* fed) {
    if (m->temperature > 0.f) {            // the sampler is a kernel of its own
        TRY(run_stream_launch(ctx, m, max_ctx_len));
        return pick_tokens(ctx, m, 1, m->d_rows + m->max_rows, m->d_rows + 2 * m->max_rows);
    }
    if (feed_step >= 0 && fed) *fed = true;
    return run_stream_launch(ctx, m, max_ctx_len, feed_step >= 0 ? 2 : 1, feed_step >= 0 ? feed_step : 0);
}

static int run_decode_step(blum_ctx* ctx, blum_llama* m, int R, int nsplit, int64_t max_ctx_len, int feed_step = -1, bool* fed = nullptr) {
    if (R == 1 && m->decode_path != 1 && stream_supported(ctx, m)) return run_stream_step(ctx, m, max_ctx_len, feed_step, fed);
    if (R > GEMV_ROWS && m->decode_path == 0 && m->cfg.act_dtype == BLUM_F32 && pack_supported(ctx, m))
        TRY(ensure_packed(ctx, m));          // allocations and packing happen outside the capture below
    auto key = std::make_pair(R, nsplit);
    auto it = m->graphs.find(key);
    if (it == m->graphs.end()) {
        TRY(blum_kv_sync_tables(ctx, m->kv));
        cudaGraph_t graph = nullptr;
        const int64_t launches_before = ctx->launches;
        BLUM_CUDA(ctx, cudaStreamBeginCapture(ctx->stream, cudaStreamCaptureModeThreadLocal));
        int rc = forward_rows(ctx, m, R, nsplit, false);
        cudaError_t e = cudaStreamEndCapture(ctx->stream, &graph);
        ctx->launches = launches_before;   // captured, not launched
        if (rc) { if (graph) cudaGraphDestroy(graph); return rc; }
        if (e != cudaSuccess) return blum_fail(ctx, BLUM_ERR_CUDA, "graph capture failed: %s", cudaGetErrorString(e));
        cudaGraphExec_t exec = nullptr;
        e = cudaGraphInstantiate(&exec, graph, 0);
        size_t nodes = 0;
        cudaGraphGetNodes(graph, nullptr, &nodes);
        cudaGraphDestroy(graph);
        if (e != cudaSuccess) return blum_fail(ctx, BLUM_ERR_CUDA, "graph instantiate failed: %s", cudaGetErrorString(e));
        m->graphs[key] = exec;
        m->graph_nodes[key] = (int)nodes;
        it = m->graphs.find(key);
    }
    BLUM_CUDA(ctx, cudaGraphLaunch(it->second, ctx->stream));
    ctx->launches += m->graph_nodes[key];
    return BLUM_OK;
}

// ------------------------------------------------------------------ weights
struct TensorRef { blum_q8_weight* w; int64_t dst_row0, nrows, K_full, src_row0, k0; float* f32; int64_t f32_n; bool is_embed; };

// Resolves a GGUF tensor name (examples/llama/src/model.rs:250-259) to its place in this shard.
static bool resolve_tensor(blum_llama* m, const char* name, TensorRef* r) {
    const blum_llama_cfg& c = m->cfg;
    const int d = c.head_dim, H = c.hidden, tp = c.tp_size, rk = c.tp_rank;
    memset(r, 0, sizeof *r);
    if (!strcmp(name, "token_embd.weight")) {
        if (m->embed_q8) { *r = TensorRef{m->embed_q8, 0, c.vocab, H, 0, 0, nullptr, 0, true}; }
        else { r->f32 = m->embed_f32; r->f32_n = (int64_t)c.vocab * H; r->is_embed = true; }
        return true;
    }
    if (!strcmp(name, "output_norm.weight")) { r->f32 = m->out_norm; r->f32_n = H; return true; }
    if (!strcmp(name, "output.weight")) {
        if (c.tie_head) return false;            // the head is the embedding table
        *r = TensorRef{m->head, 0, m->vocab, H, (int64_t)rk * m->vocab, 0, nullptr, 0, false};
        return true;
    }
    int l = -1; char rest[64];
    if (sscanf(name, "blk.%d.%63s", &l, rest) != 2 || l < 0 || l >= c.layers) return false;
    LayerW& w = m->L[l];
    const int64_t nq_rows = (int64_t)m->nq * d, nkv_rows = (int64_t)m->nkv * d;
    if (!strcmp(rest, "attn_norm.weight")) { r->f32 = w.attn_norm; r->f32_n = H; return true; }
    if (!strcmp(rest, "ffn_norm.weight")) { r->f32 = w.ffn_norm; r->f32_n = H; return true; }
    if (c.qk_norm && !strcmp(rest, "attn_q_norm.weight")) { r->f32 = w.q_norm; r->f32_n = d; return true; }
    if (c.qk_norm && !strcmp(rest, "attn_k_norm.weight")) { r->f32 = w.k_norm; r->f32_n = d; return true; }
    if (!strcmp(rest, "attn_q.weight")) { *r = TensorRef{w.wqkv, 0, nq_rows, H, rk * nq_rows, 0, nullptr, 0, false}; return true; }
    if (!strcmp(rest, "attn_k.weight")) { *r = TensorRef{w.wqkv, nq_rows, nkv_rows, H, rk * nkv_rows, 0, nullptr, 0, false}; return true; }
    if (!strcmp(rest, "attn_v.weight")) { *r = TensorRef{w.wqkv, nq_rows + nkv_rows, nkv_rows, H, rk * nkv_rows, 0, nullptr, 0, false}; return true; }
    if (!strcmp(rest, "attn_output.weight")) { *r = TensorRef{w.wo, 0, H, (int64_t)c.q_heads * d, 0, rk * nq_rows, nullptr, 0, false}; return true; }
    if (!strcmp(rest, "ffn_gate.weight")) { *r = TensorRef{w.wgate, 0, m->ffn, H, (int64_t)rk * m->ffn, 0, nullptr, 0, false}; return true; }
    if (!strcmp(rest, "ffn_up.weight")) { *r = TensorRef{w.wup, 0, m->ffn, H, (int64_t)rk * m->ffn, 0, nullptr, 0, false}; return true; }
    if (!strcmp(rest, "ffn_down.weight")) { *r = TensorRef{w.wdown, 0, H, c.ffn, 0, (int64_t)rk * m->ffn, nullptr, 0, false}; return true; }
    (void)tp;
    return false;
}

static void layer_names(int l, std::vector<std::string>* out) {
    static const char* kinds[] = {"attn_norm", "ffn_norm", "attn_q", "attn_k", "attn_v", "attn_output", "ffn_gate", "ffn_up", "ffn_down"};
    for (const char* k : kinds) out->push_back("blk." + std::to_string(l) + "." + k + ".weight");
}

extern "C" {

uint64_t blum_llama_tensor_id(const char* gguf_name) { return gguf_name ? blum_fnv1a(gguf_name) : 0; }

int blum_llama_destroy(blum_ctx* ctx, blum_llama* m) {
    if (!ctx) return BLUM_ERR_INVALID;
    if (!m) return BLUM_OK;
    cudaSetDevice(ctx->device);
    cudaStreamSynchronize(ctx->stream);
    for (auto& g : m->graphs) cudaGraphExecDestroy(g.second);
    free_stream_plan(m);
    if (m->peer) blum_peer_destroy(ctx, m->peer);
    for (auto& w : m->L) {
        if (w.attn_norm) cudaFree(w.attn_norm);
        if (w.ffn_norm) cudaFree(w.ffn_norm);
        if (w.q_norm) cudaFree(w.q_norm);
        if (w.k_norm) cudaFree(w.k_norm);
        blum_q8_0_weight_free(ctx, w.wqkv); blum_q8_0_weight_free(ctx, w.wo); blum_q8_0_weight_free(ctx, w.wgate);
        blum_q8_0_weight_free(ctx, w.wup); blum_q8_0_weight_free(ctx, w.wdown); blum_q8_0_weight_free(ctx, w.wgu);
    }
    if (!m->cfg.tie_head) blum_q8_0_weight_free(ctx, m->head);
    blum_q8_0_weight_free(ctx, m->embed_q8);
    void* bufs[] = {m->sample_scratch, m->rows_scratch, m->embed_f32, m->out_norm, m->x, m->xn, m->qkv, m->q, m->attn, m->mid, m->gate, m->logits,
                    m->d_rows, m->d_next, m->d_hist, m->attn_scratch, m->d_pairs};
    for (void* b : bufs) if (b) cudaFree(b);
    if (m->h_rows) cudaFreeHost(m->h_rows);
    if (m->h_next) cudaFreeHost(m->h_next);
    blum_kv_destroy(ctx, m->kv);
    delete m;
    return BLUM_OK;
}

int blum_llama_create(blum_ctx* ctx, const blum_llama_cfg* cfg, blum_llama** out) {
    if (!ctx) return BLUM_ERR_INVALID;
    BLUM_REQUIRE(ctx, cfg && out, "llama_create: null argument");
    *out = nullptr;
    const blum_llama_cfg& c = *cfg;
    BLUM_REQUIRE(ctx, c.layers > 0 && c.hidden > 0 && c.q_heads > 0 && c.kv_heads > 0 && c.head_dim > 0 && c.ffn > 0 && c.vocab > 0,
                 "llama_create: non-positive dimension");
    BLUM_REQUIRE(ctx, c.q_heads % c.kv_heads == 0, "llama_create: q_heads must be a multiple of kv_heads");
    BLUM_REQUIRE(ctx, c.hidden % 32 == 0 && c.ffn % 32 == 0 && (c.q_heads * c.head_dim) % 32 == 0, "llama_create: dims must be multiples of 32");
    BLUM_REQUIRE(ctx, c.head_dim == 64 || c.head_dim == 128, "llama_create: head_dim must be 64 or 128");
    BLUM_REQUIRE(ctx, c.act_dtype >= 0 && c.act_dtype <= 2 && c.kv_dtype >= 0 && c.kv_dtype <= 2, "llama_create: bad dtype");
    BLUM_REQUIRE(ctx, c.page_size > 0 && c.max_seqs > 0 && c.max_ctx > 0, "llama_create: bad cache geometry");
    const int tp = c.tp_size > 0 ? c.tp_size : 1;
    BLUM_REQUIRE(ctx, c.tp_rank >= 0 && c.tp_rank < tp, "llama_create: tp_rank outside [0,tp_size)");
    BLUM_REQUIRE(ctx, (c.rope_mode == 0 || c.rope_mode == 1) && (c.qk_norm == 0 || c.qk_norm == 1) && (c.tie_head == 0 || c.tie_head == 1),
                 "llama_create: rope_mode, qk_norm and tie_head must be 0 or 1");
    BLUM_REQUIRE(ctx, !c.tie_head || (c.embed_q8 && tp == 1), "llama_create: a tied head needs a Q8_0 embedding table (embed_q8 = 1) and no tensor parallelism");
    BLUM_REQUIRE(ctx, c.kv_heads % tp == 0 && c.ffn % (32 * tp) == 0 && c.vocab % tp == 0,
                 "llama_create: kv_heads, ffn/32 and vocab must divide by tp_size=%d", tp);
    BLUM_CUDA(ctx, cudaSetDevice(ctx->device));
    blum_llama* m = new blum_llama();
    m->cfg = c; m->cfg.tp_size = tp;
    m->nq = c.q_heads / tp; m->nkv = c.kv_heads / tp; m->ffn = c.ffn / tp; m->vocab = c.vocab / tp;
    const int H = c.hidden, d = c.head_dim;
    int rc = BLUM_OK;
    auto fail = [&](int code) { blum_llama_destroy(ctx, m); return code; };
#define ALLOC(ptr, bytes) do { cudaError_t e__ = cudaMalloc((void**)&(ptr), (bytes)); \
        if (e__ != cudaSuccess) { blum_fail(ctx, BLUM_ERR_OOM, "llama_create: cudaMalloc(%zu) failed: %s", (size_t)(bytes), cudaGetErrorString(e__)); return fail(BLUM_ERR_OOM); } } while (0)
    if (c.embed_q8) { rc = blum_q8_alloc(ctx, c.vocab, H, &m->embed_q8); if (rc) return fail(rc); }
    else ALLOC(m->embed_f32, (size_t)c.vocab * H * 4);
    ALLOC(m->out_norm, (size_t)H * 4);
    if (c.tie_head) m->head = m->embed_q8;        // borrowed: freed once, as the embedding
    else { rc = blum_q8_alloc(ctx, m->vocab, H, &m->head); if (rc) return fail(rc); }
    m->L.resize(c.layers);
    for (auto& w : m->L) {
        ALLOC(w.attn_norm, (size_t)H * 4);
        ALLOC(w.ffn_norm, (size_t)H * 4);
        if (c.qk_norm) { ALLOC(w.q_norm, (size_t)d * 4); ALLOC(w.k_norm, (size_t)d * 4); }
        if ((rc = blum_q8_alloc(ctx, (int64_t)(m->nq + 2 * m->nkv) * d, H, &w.wqkv))) return fail(rc);
        if ((rc = blum_q8_alloc(ctx, H, (int64_t)m->nq * d, &w.wo))) return fail(rc);
        // gate and up share one allocation so that the matrix kernels multiply both in one pass over x
        if ((rc = blum_q8_alloc(ctx, 2ll * m->ffn, H, &w.wgu))) return fail(rc);
        w.wgate = new blum_q8_weight(); w.wup = new blum_q8_weight();
        w.wgate->N = w.wup->N = m->ffn; w.wgate->K = w.wup->K = H; w.wgate->owns = w.wup->owns = false;
        w.wgate->q = w.wgu->q; w.wgate->d = w.wgu->d;
        w.wup->q = w.wgu->q + (size_t)m->ffn * H; w.wup->d = w.wgu->d + (size_t)m->ffn * (H / 32);
        if ((rc = blum_q8_alloc(ctx, H, m->ffn, &w.wdown))) return fail(rc);
    }
    const int64_t per_layer = ((int64_t)(m->nq + 2 * m->nkv) * d * H + (int64_t)H * m->nq * d + 3ll * m->ffn * H);
    m->weight_bytes = (per_layer * c.layers + (int64_t)m->vocab * H) * 34 / 32;
    const int pages_per_seq = (c.max_ctx + c.page_size - 1) / c.page_size;
    const int64_t pages = c.kv_pages > 0 ? c.kv_pages : (int64_t)c.max_seqs * pages_per_seq;
    rc = blum_kv_create(ctx, c.layers, m->nkv, d, c.page_size, pages, c.max_seqs, pages_per_seq, (blum_dtype)c.kv_dtype, &m->kv);
    if (rc) return fail(rc);
    m->max_rows = c.max_seqs > 2048 ? c.max_seqs : (c.max_ctx < 2048 ? (c.max_ctx > c.max_seqs ? c.max_ctx : c.max_seqs) : 2048);
    const int R = m->max_rows;
    ALLOC(m->x, act_bytes(m, (int64_t)R * H));
    ALLOC(m->xn, act_bytes(m, (int64_t)R * H));
    ALLOC(m->qkv, act_bytes(m, (int64_t)R * (m->nq + 2 * m->nkv) * d));
    ALLOC(m->q, act_bytes(m, (int64_t)R * m->nq * d));
    ALLOC(m->attn, act_bytes(m, (int64_t)R * m->nq * d));
    ALLOC(m->mid, act_bytes(m, (int64_t)R * m->ffn));
    ALLOC(m->gate, act_bytes(m, (int64_t)R * std::max<int64_t>(2ll * m->ffn, H)));   // [gate | up]; also takes the o / down projections before they join x
    ALLOC(m->logits, (size_t)c.max_seqs * m->vocab * 4);
    {   // split-K workspace of the tensor-core GEMM for the widest projection, so that captured steps never allocate
        const int64_t widest = std::max<int64_t>((int64_t)(m->nq + 2 * m->nkv) * d, std::max<int64_t>(2ll * m->ffn, H));
        // (+ the digitised rows of the integer-path matmul: 32 rows of two byte planes and one scale per block)
        const int64_t kmax = std::max<int64_t>((int64_t)m->nq * d, std::max<int64_t>(m->ffn, H));
        if ((rc = blum_gemm_ws_reserve(ctx, (size_t)R * widest * sizeof(float) + (size_t)kmax * 72 + 4096))) return fail(rc);
    }
    ALLOC(m->d_rows, (size_t)4 * R * 4);
    ALLOC(m->d_next, (size_t)c.max_seqs * 4);
    ALLOC(m->d_pairs, (size_t)tp * c.max_seqs * 8);
    m->max_splits = 32;
    ALLOC(m->attn_scratch, blum_attn_decode_scratch_bytes(c.max_seqs, m->nq, d, m->max_splits) + 16);
    if (cudaHostAlloc((void**)&m->h_rows, (size_t)4 * R * 4, cudaHostAllocDefault) != cudaSuccess ||
        cudaHostAlloc((void**)&m->h_next, (size_t)(c.max_seqs + 1) * 4, cudaHostAllocDefault) != cudaSuccess) {
        blum_fail(ctx, BLUM_ERR_OOM, "llama_create: pinned allocation failed");
        return fail(BLUM_ERR_OOM);
    }
#undef ALLOC
    *out = m;
    return BLUM_OK;
}

blum_kv* blum_llama_kv(blum_llama* m) { return m ? m->kv : nullptr; }
blum_q8_weight* blum_llama_layer_weight(blum_llama* m, int layer, int which) {
    if (!m) return nullptr;
    if (which == 5) return m->head;
    if (layer < 0 || layer >= (int)m->L.size()) return nullptr;
    const LayerW& w = m->L[layer];
    switch (which) {
        case 0: return w.wqkv; case 1: return w.wo; case 2: return w.wgate; case 3: return w.wup; case 4: return w.wdown;
        default: return nullptr;
    }
}
const float* blum_llama_norm_weight(blum_llama* m, int layer, int which) {
    if (!m) return nullptr;
    if (which == 2) return m->out_norm;
    if (layer < 0 || layer >= (int)m->L.size()) return nullptr;
    return which == 0 ? m->L[layer].attn_norm : which == 1 ? m->L[layer].ffn_norm : nullptr;
}
int64_t blum_llama_weight_bytes(const blum_llama* m) { return m ? m->weight_bytes : -1; }
int blum_llama_set_decode_path(blum_ctx* ctx, blum_llama* m, int path) {
    if (!ctx) return BLUM_ERR_INVALID;
    BLUM_REQUIRE(ctx, m && (path == 0 || path == 1), "llama_set_decode_path: path must be 0 (automatic) or 1 (per-op kernels)");
    m->decode_path = path;
    return BLUM_OK;
}
int blum_llama_decode_path(blum_ctx* ctx, blum_llama* m) {
    if (!ctx || !m) return BLUM_ERR_INVALID;
    return (m->decode_path != 1 && stream_supported(ctx, m)) ? 2 : 1;
}
// Development aid: cycle counters of the last persistent-kernel launch, averaged over CTAs: [0] consumer total, [1] waiting
// for weight stages, [2] grid barriers, [3] staging x, [4] attention, [5] group reductions, [6] producer waiting for a free
// stage, [7] producer total, [8 + 3 k + {0, 1, 2}] staging / unit loop / following barrier of phase kind k.  The first call
// switches the counters on (they are filled by the launches that follow).
int blum_llama_stream_profile(blum_ctx* ctx, blum_llama* m, double* out, int per_cta) {
    if (!ctx || !m || !out) return BLUM_ERR_INVALID;
    StreamPlan& sp = m->sp;
    if (!stream_supported(ctx, m)) return blum_fail(ctx, BLUM_ERR_STATE, "stream profile: the model does not use the persistent kernel");
    const size_t n = (size_t)sp.grid * 96;
    if (!sp.prof) {
        BLUM_CUDA(ctx, cudaMalloc((void**)&sp.prof, n * sizeof(long long)));
        BLUM_CUDA(ctx, cudaMemsetAsync(sp.prof, 0, n * sizeof(long long), ctx->stream));
    }
    std::vector<long long> h(n);
    BLUM_CUDA(ctx, cudaMemcpyAsync(h.data(), sp.prof, n * sizeof(long long), cudaMemcpyDeviceToHost, ctx->stream));
    BLUM_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
    // out: [32] averages over CTAs, then [32] maxima, then [32] minima; with per_cta also the raw [grid][32] table
    for (int i = 0; i < 32; i++) {
        double s = 0, mx = -1e300, mn = 1e300;
        for (int c = 0; c < sp.grid; c++) { const double v = (double)h[(size_t)c * 32 + i]; s += v; mx = v > mx ? v : mx; mn = v < mn ? v : mn; }
        out[i] = s / sp.grid; out[32 + i] = mx; out[64 + i] = mn;
    }
    if (per_cta) for (size_t i = 0; i < n; i++) out[96 + i] = (double)h[i];      // [grid][32] counters, then [grid][64] timeline of one layer
    return BLUM_OK;
}
// Development aid: average device time of the persistent decode kernel alone.  The step that was run last is launched again
// `iters` times between two CUDA events (same token, same position: every launch recomputes the same step and rewrites the
// same KV slot with the same values), without the argmax and token feedback kernels that follow it in a real step.
int blum_llama_stream_kernel_us(blum_ctx* ctx, blum_llama* m, int iters, float* avg_us) {
    if (!ctx || !m || !avg_us || iters < 1) return BLUM_ERR_INVALID;
    if (m->decode_path == 1 || !stream_supported(ctx, m) || !m->sp.built)
        return blum_fail(ctx, BLUM_ERR_STATE, "stream kernel timing: run a single-sequence decode step on the persistent path first");
    cudaEvent_t a, b;
    BLUM_CUDA(ctx, cudaEventCreate(&a));
    BLUM_CUDA(ctx, cudaEventCreate(&b));
    int rc = BLUM_OK;
    cudaEventRecord(a, ctx->stream);
    for (int i = 0; i < iters && !rc; i++) rc = run_stream_launch(ctx, m, m->sp.last_ctx_len);
    cudaEventRecord(b, ctx->stream);
    const cudaError_t e = cudaEventSynchronize(b);
    float ms = 0.f;
    cudaEventElapsedTime(&ms, a, b);
    cudaEventDestroy(a); cudaEventDestroy(b);
    if (rc) return rc;
    if (e != cudaSuccess) return blum_fail(ctx, BLUM_ERR_CUDA, "stream kernel timing: %s", cudaGetErrorString(e));
    *avg_us = ms * 1000.f / (float)iters;
    return blum_check_device_error(ctx);
}
int blum_llama_set_comm(blum_ctx* ctx, blum_llama* m, blum_comm* comm) {
    if (!ctx || !m) return BLUM_ERR_INVALID;
    if (m->peer && comm != m->comm) { blum_peer_destroy(ctx, m->peer); m->peer = nullptr; }
    m->comm = comm;
    return BLUM_OK;
}

// Rows up to this count take the one-kernel exchange; larger row counts (prompt chunks) keep NCCL, whose ring / in-switch
// algorithms move each byte once where the one-shot pull reads every peer's whole partial product.
#define LLAMA_PEER_MAX_ROWS 64

int blum_llama_set_peer_allreduce(blum_ctx* ctx, blum_llama* m, int enable, int timeout_ms) {
    if (!ctx) return BLUM_ERR_INVALID;
    BLUM_REQUIRE(ctx, m != nullptr, "llama_set_peer_allreduce: null model");
    if ((enable != 0) == (m->peer != nullptr)) return BLUM_OK;
    BLUM_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
    for (auto& g : m->graphs) cudaGraphExecDestroy(g.second);      // captured steps name the buffers of the other path
    m->graphs.clear();
    if (!enable) {
        blum_peer_destroy(ctx, m->peer);
        m->peer = nullptr;
        return BLUM_OK;
    }
    if (m->cfg.tp_size <= 1 || !m->comm) return blum_fail(ctx, BLUM_ERR_STATE, "llama_set_peer_allreduce: needs tp_size > 1 and a communicator");
    return blum_peer_create(ctx, m->comm, (int64_t)act_bytes(m, m->cfg.hidden), LLAMA_PEER_MAX_ROWS, timeout_ms, &m->peer);
}
int blum_llama_peer_allreduce(const blum_llama* m) { return m && m->peer ? 1 : 0; }

int blum_llama_set_sampling(blum_ctx* ctx, blum_llama* m, float temperature, float top_p, uint64_t seed) {
    if (!ctx) return BLUM_ERR_INVALID;
    BLUM_REQUIRE(ctx, m != nullptr, "llama_set_sampling: null model");
    BLUM_REQUIRE(ctx, temperature >= 0.f && top_p > 0.f, "llama_set_sampling: temperature must be >= 0 and top_p > 0");
    if (temperature > 0.f && m->cfg.tp_size > 1)
        return blum_fail(ctx, BLUM_ERR_STATE, "llama_set_sampling: a vocabulary-parallel head only samples greedily");
    BLUM_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
    if (temperature > 0.f && !m->sample_scratch)
        BLUM_CUDA(ctx, cudaMalloc(&m->sample_scratch, (size_t)std::max(m->cfg.max_seqs, 1) * (size_t)m->vocab * 4));
    for (auto& g : m->graphs) cudaGraphExecDestroy(g.second);      // captured steps end in the other kernel
    m->graphs.clear();
    m->temperature = temperature; m->top_p = top_p; m->sample_seed = seed;
    return BLUM_OK;
}

int blum_llama_generate_weights(blum_ctx* ctx, blum_llama* m, uint64_t seed) {
    if (!ctx) return BLUM_ERR_INVALID;
    BLUM_REQUIRE(ctx, m != nullptr, "llama_generate_weights: null model");
    m->weights_version++;
    std::vector<std::string> names = {"token_embd.weight", "output_norm.weight"};
    if (!m->cfg.tie_head) names.push_back("output.weight");
    for (int l = 0; l < m->cfg.layers; l++) {
        layer_names(l, &names);
        if (m->cfg.qk_norm) { names.push_back("blk." + std::to_string(l) + ".attn_q_norm.weight"); names.push_back("blk." + std::to_string(l) + ".attn_k_norm.weight"); }
    }
    std::vector<float> host;
    for (const std::string& name : names) {
        TensorRef r;
        if (!resolve_tensor(m, name.c_str(), &r)) return blum_fail(ctx, BLUM_ERR_STATE, "unknown tensor %s", name.c_str());
        const uint64_t tid = blum_fnv1a(name.c_str());
        if (r.w) {
            TRY(blum_q8_generate_window(ctx, r.w, r.dst_row0, r.nrows, seed, tid, r.K_full, r.src_row0, r.k0));
        } else if (r.is_embed) {
            // f32 embedding ~ N(0, 0.02), generated on the host in slabs
            const int64_t slab = (int64_t)1 << 24;
            host.resize((size_t)(r.f32_n < slab ? r.f32_n : slab));
            const uint64_t key = blum_gen_key(seed, tid);
            for (int64_t o = 0; o < r.f32_n; o += slab) {
                const int64_t n = (r.f32_n - o < slab) ? r.f32_n - o : slab;
                blum_gen_normal_range(key, o, n, 0.02f, host.data());
                BLUM_CUDA(ctx, cudaMemcpyAsync(r.f32 + o, host.data(), (size_t)n * 4, cudaMemcpyHostToDevice, ctx->stream));
                BLUM_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
            }
        } else {
            fill_f32_kernel<<<32, 256, 0, ctx->stream>>>(r.f32, r.f32_n, 1.0f);   // norm weights = 1
            BLUM_LAUNCH_CHECK(ctx);
        }
    }
    BLUM_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
    return BLUM_OK;
}

int blum_llama_set_tensor(blum_ctx* ctx, blum_llama* m, const char* gguf_name, const void* host_bytes, size_t nbytes,
                          int is_q8_0) {
    if (!ctx) return BLUM_ERR_INVALID;
    BLUM_REQUIRE(ctx, m && gguf_name && host_bytes, "llama_set_tensor: null argument");
    TensorRef r;
    if (!resolve_tensor(m, gguf_name, &r)) return blum_fail(ctx, BLUM_ERR_INVALID, "llama_set_tensor: unknown tensor '%s'", gguf_name);
    m->weights_version++;                      // stream-packed copies are rebuilt before the next single-sequence step
    if (r.w) {
        BLUM_REQUIRE(ctx, is_q8_0, "llama_set_tensor: '%s' must be Q8_0", gguf_name);
        // the caller passes the FULL tensor; its row count follows from the byte count
        const size_t row_bytes = (size_t)(r.K_full / 32) * 34;
        BLUM_REQUIRE(ctx, nbytes % row_bytes == 0 && (int64_t)(nbytes / row_bytes) >= r.src_row0 + r.nrows,
                     "llama_set_tensor: '%s' has %zu bytes, not a [>=%lld, %lld] Q8_0 tensor", gguf_name, nbytes,
                     (long long)(r.src_row0 + r.nrows), (long long)r.K_full);
        return blum_q8_fill_from_host_gguf(ctx, r.w, r.dst_row0, r.nrows, host_bytes, r.K_full, r.src_row0, r.k0);
    }
    BLUM_REQUIRE(ctx, !is_q8_0, "llama_set_tensor: '%s' must be f32", gguf_name);
    BLUM_REQUIRE(ctx, nbytes == (size_t)r.f32_n * 4, "llama_set_tensor: '%s' expects %lld f32 values", gguf_name, (long long)r.f32_n);
    BLUM_CUDA(ctx, cudaMemcpyAsync(r.f32, host_bytes, nbytes, cudaMemcpyHostToDevice, ctx->stream));
    BLUM_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
    return BLUM_OK;
}

// uploads the first R entries of the four row arrays
static int upload_rows(blum_ctx* ctx, blum_llama* m, int R) {
    for (int a = 0; a < 4; a++)
        BLUM_CUDA(ctx, cudaMemcpyAsync(m->d_rows + (size_t)a * m->max_rows, m->h_rows + (size_t)a * m->max_rows, (size_t)R * 4,
                                       cudaMemcpyHostToDevice, ctx->stream));
    return BLUM_OK;
}

int blum_llama_prefill(blum_ctx* ctx, blum_llama* m, int seq, const int32_t* host_ids, int64_t T, int32_t* next_token,
                       float* logits_out) {
    if (!ctx) return BLUM_ERR_INVALID;
    BLUM_REQUIRE(ctx, m && host_ids && T > 0, "llama_prefill: bad argument");
    const int64_t p0 = blum_kv_seq_len(m->kv, seq);
    if (p0 < 0) return blum_fail(ctx, BLUM_ERR_STATE, "llama_prefill: sequence %d is not allocated", seq);
    for (int64_t i = 0; i < T; i++)
        BLUM_REQUIRE(ctx, host_ids[i] >= 0 && host_ids[i] < m->cfg.vocab, "llama_prefill: token id %d out of range", host_ids[i]);
    TRY(blum_kv_seq_extend(ctx, m->kv, seq, p0 + T));
    TRY(blum_kv_sync_tables(ctx, m->kv));
    for (int64_t o = 0; o < T; o += m->max_rows) {
        const int R = (int)((T - o < m->max_rows) ? T - o : m->max_rows);
        BLUM_CUDA(ctx, cudaStreamSynchronize(ctx->stream));   // h_rows is reused
        for (int i = 0; i < R; i++) {
            m->h_rows[i] = host_ids[o + i];
            m->h_rows[m->max_rows + i] = seq;
            m->h_rows[2 * m->max_rows + i] = (int32_t)(p0 + o + i);
            m->h_rows[3 * m->max_rows + i] = (int32_t)(p0 + o + i + 1);
        }
        TRY(upload_rows(ctx, m, R));
        m->pre_seq = seq; m->pre_p0 = p0 + o;
        const int frc = forward_rows(ctx, m, R, 1, true);
        m->pre_seq = -1;
        if (frc) return frc;
    }
    BLUM_CUDA(ctx, cudaMemcpyAsync(m->h_next, m->d_next, 4, cudaMemcpyDeviceToHost, ctx->stream));
    if (logits_out) BLUM_CUDA(ctx, cudaMemcpyAsync(logits_out, m->logits, (size_t)m->vocab * 4, cudaMemcpyDeviceToHost, ctx->stream));
    BLUM_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
    if (next_token) *next_token = m->h_next[0];
    return blum_check_device_error(ctx);
}

// Reads the device error word in the same synchronisation as the step's result: h_next[max_seqs] mirrors it.
static int finish_step(blum_ctx* ctx, blum_llama* m, const char* what) {
    int32_t* h_err = m->h_next + m->cfg.max_seqs;
    BLUM_CUDA(ctx, cudaMemcpyAsync(h_err, ctx->dev_error, sizeof(int), cudaMemcpyDeviceToHost, ctx->stream));
    BLUM_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
    if (*h_err != 0) {
        const int word = *h_err;
        BLUM_CUDA(ctx, cudaMemsetAsync(ctx->dev_error, 0, sizeof(int), ctx->stream));
        // a stream kernel that gave up leaves its barrier counters mid-way: start the next launch from zero
        unsigned long long where[8] = {};
        if (m->sp.ctr) {
            cudaMemcpyAsync(where, m->sp.ctr, sizeof where, cudaMemcpyDeviceToHost, ctx->stream);
            cudaStreamSynchronize(ctx->stream);
            // launch numbers start again from zero, so the tags the words still carry would come round again: clear them too
            BLUM_CUDA(ctx, cudaMemsetAsync(m->sp.ctr, 0, m->sp.ctr_bytes, ctx->stream));
            BLUM_CUDA(ctx, cudaMemsetAsync(m->sp.words, 0, m->sp.words_bytes, ctx->stream));
        }
        if (where[3])
            return blum_fail(ctx, BLUM_ERR_DEVICE, "%s: device error word = 0x%x; the persistent decode kernel gave up a wait (site %llu: 1 weight "
                             "stage, 2 activation word, 3 attention input, 4 split-group partial) in CTA %llu, waited for %llu, saw %llu; launch %llu",
                             what, word, where[3], where[4], where[5], where[6], where[1]);
        return blum_fail(ctx, BLUM_ERR_DEVICE, "%s: device error word = 0x%x (bounded wait expired or bad page / sequence index)", what, word);
    }
    return BLUM_OK;
}

int blum_llama_decode(blum_ctx* ctx, blum_llama* m, const int32_t* seq_ids, const int32_t* host_ids, int64_t B,
                      int32_t* next_tokens, float* logits_out) {
    if (!ctx) return BLUM_ERR_INVALID;
    BLUM_REQUIRE(ctx, m && seq_ids && host_ids && next_tokens, "llama_decode: null argument");
    BLUM_REQUIRE(ctx, B > 0 && B <= m->cfg.max_seqs, "llama_decode: batch %lld outside [1,%d]", (long long)B, m->cfg.max_seqs);
    // validate every row before any sequence grows, so that a rejected call leaves the cache as it was
    for (int b = 0; b < B; b++) {
        if (blum_kv_seq_len(m->kv, seq_ids[b]) < 0) return blum_fail(ctx, BLUM_ERR_STATE, "llama_decode: sequence %d is not allocated", seq_ids[b]);
        BLUM_REQUIRE(ctx, host_ids[b] >= 0 && host_ids[b] < m->cfg.vocab, "llama_decode: token id %d out of range", host_ids[b]);
        for (int a = 0; a < b; a++) BLUM_REQUIRE(ctx, seq_ids[a] != seq_ids[b], "llama_decode: sequence %d appears twice in the batch", seq_ids[b]);
    }
    std::vector<int64_t> old_len((size_t)B);
    int64_t max_len = 0;
    int grown = 0, rc = BLUM_OK;
    for (int b = 0; b < B && !rc; b++) {
        const int64_t len = blum_kv_seq_len(m->kv, seq_ids[b]);
        old_len[b] = len;
        rc = blum_kv_seq_extend(ctx, m->kv, seq_ids[b], len + 1);
        if (rc) break;
        grown = b + 1;
        m->h_rows[b] = host_ids[b];
        m->h_rows[m->max_rows + b] = seq_ids[b];
        m->h_rows[2 * m->max_rows + b] = (int32_t)len;
        m->h_rows[3 * m->max_rows + b] = (int32_t)len + 1;
        if (len + 1 > max_len) max_len = len + 1;
    }
    // a failed step must not leave sequences one token longer than what the cache holds (pages stay with the sequence)
    auto roll_back = [&]() { for (int b = 0; b < grown; b++) m->kv->seq_len[seq_ids[b]] = old_len[b]; };
    if (!rc) rc = blum_kv_sync_tables(ctx, m->kv);
    if (!rc) rc = upload_rows(ctx, m, (int)B);
    if (!rc) rc = run_decode_step(ctx, m, (int)B, pick_nsplit(ctx, m, (int)B, max_len), max_len);
    if (!rc) {
        cudaError_t e = cudaMemcpyAsync(m->h_next, m->d_next, (size_t)B * 4, cudaMemcpyDeviceToHost, ctx->stream);
        if (e == cudaSuccess && logits_out) e = cudaMemcpyAsync(logits_out, m->logits, (size_t)B * m->vocab * 4, cudaMemcpyDeviceToHost, ctx->stream);
        if (e != cudaSuccess) rc = blum_fail(ctx, BLUM_ERR_CUDA, "llama_decode: result copy failed: %s", cudaGetErrorString(e));
    }
    if (!rc) rc = finish_step(ctx, m, "llama_decode");
    if (rc) { roll_back(); return rc; }
    memcpy(next_tokens, m->h_next, (size_t)B * 4);
    return BLUM_OK;
}

int blum_llama_decode_loop(blum_ctx* ctx, blum_llama* m, int seq, int32_t first_token, int steps, int32_t* tokens_out) {
    if (!ctx) return BLUM_ERR_INVALID;
    BLUM_REQUIRE(ctx, m && steps > 0, "llama_decode_loop: bad argument");
    const int64_t len = blum_kv_seq_len(m->kv, seq);
    if (len < 0) return blum_fail(ctx, BLUM_ERR_STATE, "llama_decode_loop: sequence %d is not allocated", seq);
    BLUM_REQUIRE(ctx, first_token >= 0 && first_token < m->cfg.vocab, "llama_decode_loop: token id out of range");
    if (m->hist_cap < steps) {     // grown before the sequence is, so that a failed allocation changes nothing
        if (m->d_hist) cudaFree(m->d_hist);
        m->d_hist = nullptr; m->hist_cap = 0;
        BLUM_CUDA(ctx, cudaMalloc((void**)&m->d_hist, (size_t)steps * 4));
        m->hist_cap = steps;
    }
    TRY(blum_kv_seq_extend(ctx, m->kv, seq, len + steps));
    auto body = [&]() -> int {
        TRY(blum_kv_sync_tables(ctx, m->kv));
        m->h_rows[0] = first_token;
        m->h_rows[m->max_rows] = seq;
        m->h_rows[2 * m->max_rows] = (int32_t)len;
        m->h_rows[3 * m->max_rows] = (int32_t)len + 1;
        TRY(upload_rows(ctx, m, 1));
        const int nsplit = pick_nsplit(ctx, m, 1, len + steps);
        for (int s = 0; s < steps; s++) {
            bool fed = false;
            TRY(run_decode_step(ctx, m, 1, nsplit, len + steps, s, &fed));
            if (!fed) {
                advance_rows_kernel<<<1, 32, 0, ctx->stream>>>(m->d_rows, m->max_rows, m->d_next, m->d_hist, s, 1);
                BLUM_LAUNCH_CHECK(ctx);
            }
        }
        if (tokens_out) BLUM_CUDA(ctx, cudaMemcpyAsync(tokens_out, m->d_hist, (size_t)steps * 4, cudaMemcpyDeviceToHost, ctx->stream));
        return finish_step(ctx, m, "llama_decode_loop");
    };
    const int rc = body();
    if (rc) m->kv->seq_len[seq] = len;
    return rc;
}

}  // extern "C"
