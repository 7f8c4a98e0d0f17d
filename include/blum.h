/*
 * blum.h - C ABI of libblum.so: sm_100a kernels for the CUDA hot path that luminal's
 * inference compiler runs for Q8_0-quantized transformer decoding.
 *
 * Each entry point names the reference interface it stands in for (paths are relative
 * to the luminal source tree), or says that the reference has no counterpart.  Hooks that
 * exist for tests, benches and development (seeded generators, timers, traces) are declared
 * in blum_dev.h, not here.  The convention throughout:
 *   - every function returns an int status: 0 = ok, <0 = error (see blum_status);
 *     nothing aborts, traps or throws across this boundary (the reference panics
 *     instead: crates/luminal_cuda/src/quantized.rs:144,163);
 *   - blum_last_error(ctx) returns a human-readable message for the last failure;
 *   - device pointers are plain `void*` owned by the caller, exactly like the
 *     `CudaSlice<T>` inside `CudaData<T>` (crates/luminal_cuda/src/lib.rs:83-100);
 *   - all compute calls are asynchronous and ordered on the context's stream
 *     (the reference launches everything on device 0's default stream);
 *   - a context is bound to one device and is used from one host thread at a time.
 */
#ifndef BLUM_H
#define BLUM_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef enum blum_status {
    BLUM_OK = 0,
    BLUM_ERR_INVALID = -1,   /* bad argument (null pointer, unsupported shape or dtype)  */
    BLUM_ERR_CUDA = -2,      /* a CUDA runtime call failed; message holds the CUDA error  */
    BLUM_ERR_OOM = -3,       /* device or page-pool memory exhausted                      */
    BLUM_ERR_STATE = -4,     /* call made in the wrong state (e.g. sequence not allocated)*/
    BLUM_ERR_DEVICE = -5,    /* a kernel recorded an error word (bounded wait ran out, bad index) */
    BLUM_ERR_COMM = -6       /* NCCL failure                                             */
} blum_status;

/* Element types of activations / outputs.  The reference's CudaFloat covers f32 and
 * f16 (crates/luminal_cuda/src/lib.rs:54-81); bf16 is an addition. */
typedef enum blum_dtype { BLUM_F32 = 0, BLUM_F16 = 1, BLUM_BF16 = 2 } blum_dtype;

typedef struct blum_ctx blum_ctx;
typedef struct blum_q8_weight blum_q8_weight;
typedef struct blum_kv blum_kv;
typedef struct blum_llama blum_llama;
typedef struct blum_comm blum_comm;
typedef struct blum_peer blum_peer;

/* ------------------------------------------------------------------ lifecycle */

/* Replaces CudaContext::new(0) + default_stream() (crates/luminal_cuda/src/quantized.rs:247,142). */
int blum_ctx_create(int device, blum_ctx** out);
int blum_ctx_destroy(blum_ctx* ctx);
/* Run on a caller-owned cudaStream_t (pass 0 for the legacy default stream) so that ordering with untouched luminal
 * ops is kept: the reference launches everything on `device.default_stream()` (crates/luminal_cuda/src/quantized.rs:142). */
int blum_ctx_set_stream(blum_ctx* ctx, void* cuda_stream);
void* blum_ctx_stream(blum_ctx* ctx);
/* Message of the last failed call on this context.  No counterpart: the reference panics with its message
 * (crates/luminal_cuda/src/quantized.rs:144,163). */
const char* blum_last_error(blum_ctx* ctx);
/* Device ordinal and SM count of the context; the reference has a fixed device 0 (crates/luminal_cuda/src/quantized.rs:247). */
int blum_ctx_device(blum_ctx* ctx);
int blum_ctx_sm_count(blum_ctx* ctx);
/* Library version string and the gencode it was built for.  No counterpart: the reference compiles its kernels at run time
 * (crates/luminal_cuda/src/lib.rs:237-258). */
const char* blum_version(void);

/* ------------------------------------------------------------------ buffers
 * Stand-ins for stream.alloc / memcpy_stod / memcpy_dtov used by the copy ops
 * (crates/luminal_cuda/src/prim.rs:31-47,60-75).  Host<->device copies are stream-ordered;
 * the d2h form synchronises the stream before returning, as memcpy_dtov does. */
int blum_dev_alloc(blum_ctx* ctx, size_t bytes, void** dptr);
int blum_dev_free(blum_ctx* ctx, void* dptr);
int blum_memset(blum_ctx* ctx, void* dptr, int byte, size_t bytes);
int blum_memcpy_h2d(blum_ctx* ctx, void* dst_dev, const void* src_host, size_t bytes);
int blum_memcpy_d2h(blum_ctx* ctx, void* dst_host, const void* src_dev, size_t bytes);
int blum_memcpy_d2d(blum_ctx* ctx, void* dst_dev, const void* src_dev, size_t bytes);
int blum_host_alloc_pinned(blum_ctx* ctx, size_t bytes, void** hptr);
int blum_host_free_pinned(blum_ctx* ctx, void* hptr);
int blum_sync(blum_ctx* ctx);
/* Reads and clears the device error word that bounded waits / index checks write. */
int blum_check_device_error(blum_ctx* ctx);

/* Replay a fixed sequence of calls as one CUDA graph: everything issued on this context between begin and end is
 * captured instead of executed (no counterpart in luminal's CUDA crate; its Metal backend batches command buffers).
 * Calls that allocate or synchronise must happen before begin. */
int blum_graph_begin(blum_ctx* ctx);
int blum_graph_end(blum_ctx* ctx, void** graph_exec_out, int* n_kernels_out);
int blum_graph_launch(blum_ctx* ctx, void* graph_exec, int n_kernels);
int blum_graph_destroy(blum_ctx* ctx, void* graph_exec);

/* ------------------------------------------------------------------ Q8_0 weights
 * A Q8_0 tensor [N,K] arrives as raw GGUF bytes: 34-byte blocks {f16 d; int8 qs[32]} in
 * row-major block order (crates/luminal_cuda/src/quantized.rs:30-33; uploaded as CudaData<u8>
 * by examples/llama/src/loader.rs:156-158).  It is repacked once into two planes
 * (int8 [N][K] and f16 [N][K/32]) so that kernels can use 128-bit loads and TMA. */
int blum_q8_0_weight_from_gguf_bytes(blum_ctx* ctx, const void* dev_bytes, int64_t N, int64_t K,
                                     blum_q8_weight** out);
int blum_q8_0_weight_from_host_gguf_bytes(blum_ctx* ctx, const void* host_bytes, int64_t N, int64_t K,
                                          blum_q8_weight** out);
/* New weight whose rows are the rows of `parts[0..n)` stacked along N (fused q/k/v, gate/up). */
int blum_q8_0_weight_concat_rows(blum_ctx* ctx, blum_q8_weight* const* parts, int nparts,
                                 blum_q8_weight** out);
/* Rows [n0,n0+n) x columns [k0,k0+k) as a new weight (tensor-parallel shards; k0,k multiples of 32). */
int blum_q8_0_weight_slice(blum_ctx* ctx, const blum_q8_weight* w, int64_t n0, int64_t n,
                           int64_t k0, int64_t k, blum_q8_weight** out);
/* Writes the weight back out in GGUF block order (device buffer of N*K*34/32 bytes). */
int blum_q8_0_weight_to_gguf_bytes(blum_ctx* ctx, const blum_q8_weight* w, void* dev_bytes);
int blum_q8_0_weight_free(blum_ctx* ctx, blum_q8_weight* w);
int64_t blum_q8_0_weight_rows(const blum_q8_weight* w);
int64_t blum_q8_0_weight_cols(const blum_q8_weight* w);
const void* blum_q8_0_weight_quants(const blum_q8_weight* w);
const void* blum_q8_0_weight_scales(const blum_q8_weight* w);

/* ------------------------------------------------------------------ Q8_0 matmul
 * y[M,N] = x[M,K] * W^T with f32 accumulation.  Replaces QuantizedMatmul<T>::process
 * (crates/luminal_cuda/src/quantized.rs:116-168), which launches one matvec per row of x.
 * M <= 16 runs the bandwidth-bound GEMV family; larger M runs the tcgen05 GEMM.
 * x and y are dense row-major; x_dtype / y_dtype may differ. */
int blum_q8_0_matmul(blum_ctx* ctx, const blum_q8_weight* w, const void* x, blum_dtype x_dtype,
                     void* y, blum_dtype y_dtype, int64_t M);

/* Fused forms used by the decoder step (all optional pieces may be NULL / 0):
 *   xn      = norm_weight ? x * rsqrt(mean(x^2)+eps) * norm_weight : x        (per row of x)
 *   acc     = xn * W^T
 *   y       = residual ? residual + acc : acc
 * norm_weight is f32 [K]; residual has y's shape and dtype and may alias y. */
int blum_q8_0_matmul_fused(blum_ctx* ctx, const blum_q8_weight* w, const void* x, blum_dtype x_dtype,
                           const float* norm_weight, float eps, const void* residual,
                           void* y, blum_dtype y_dtype, int64_t M);
/* y[M,N] = (xn * Wup^T) * swish(xn * Wgate^T), the SwiGLU of examples/llama/src/model.rs:27-31. */
int blum_q8_0_matmul_swiglu(blum_ctx* ctx, const blum_q8_weight* w_gate, const blum_q8_weight* w_up,
                            const void* x, blum_dtype x_dtype, const float* norm_weight, float eps,
                            void* y, blum_dtype y_dtype, int64_t M);
/* Embedding row dequantisation; replaces QuantizedGather<T>::process
 * (crates/luminal_cuda/src/quantized.rs:202-233).  ids are int32 on the device. */
int blum_q8_0_gather(blum_ctx* ctx, const blum_q8_weight* w, const int32_t* ids, int64_t T,
                     void* out, blum_dtype out_dtype);
/* f32 / f16 / bf16 table gather; replaces CudaGather (crates/luminal_cuda/src/binary.rs:279-344). */
int blum_gather(blum_ctx* ctx, const void* table, blum_dtype table_dtype, int64_t rows, int64_t dim,
                const int32_t* ids, int64_t T, void* out, blum_dtype out_dtype);

/* ------------------------------------------------------------------ elementwise family
 * RMSNorm: y = x * rsqrt(mean(x^2)+eps) [* weight]; replaces CudaStdNorm + the trailing
 * multiply (crates/luminal_cuda/src/unary.rs:170-302; crates/luminal_nn/src/norm.rs:58-70).
 * With `residual` non-null: s = x + residual is written to sum_out (may alias x) and normalised. */
int blum_rmsnorm(blum_ctx* ctx, const void* x, const void* residual, const float* weight, float eps,
                 void* y, void* sum_out, blum_dtype dtype, int64_t rows, int64_t dim);
/* Per-head RMSNorm (optional) followed by rotary embedding, in place on the q and k heads of fused rows
 * qkv [T, (q_heads + 2*kv_heads) * head_dim]: the glue of the qwen decoder (examples/qwen/src/model.rs:52-77,93-105).
 * norm weights f32 [head_dim] or NULL (no norm); rope_mode as in blum_llama_cfg; v is left as it is. */
int blum_qk_norm_rope(blum_ctx* ctx, void* qkv, blum_dtype dtype, const int32_t* positions, int64_t T, int q_heads,
                      int kv_heads, int head_dim, const float* q_norm_w, const float* k_norm_w, float eps, float theta,
                      int rope_mode);
/* Interleaved-pair rotary embedding of examples/llama/src/model.rs:52-72 applied in place to
 * x [T, heads, head_dim]; positions int32 [T]. */
int blum_rope_interleaved(blum_ctx* ctx, void* x, blum_dtype dtype, const int32_t* positions,
                          int64_t T, int heads, int head_dim, float theta);
/* out = up * gate * sigmoid(gate)  (examples/llama/src/model.rs:27-31; src/hl_ops/unary.rs:169-177). */
int blum_swiglu(blum_ctx* ctx, const void* gate, const void* up, void* out, blum_dtype dtype, int64_t n);
int blum_add(blum_ctx* ctx, const void* a, const void* b, void* out, blum_dtype dtype, int64_t n);
/* Row softmax; replaces CudaSoftmax (crates/luminal_cuda/src/unary.rs:493-593); f32 accumulation. */
int blum_softmax(blum_ctx* ctx, const void* x, void* y, blum_dtype dtype, int64_t rows, int64_t cols);
/* Greedy sampler of examples/llama/src/main.rs:194-198 on the device: index of the maximum of each
 * row; among equal maxima the LAST index wins (Iterator::max_by semantics); NaNs compare equal. */
int blum_argmax(blum_ctx* ctx, const void* logits, blum_dtype dtype, int64_t rows, int64_t cols,
                int32_t* out_idx);
/* Temperature / top-p sampler, one token per row of f32 logits (no counterpart in the reference, which only has the
 * greedy rule above).  Integer-exact specification, so every implementation gives the same token: m = largest non-NaN
 * logit; z = (l - m) * (1 / temperature) in f32; w = trunc(2^30 e^z) by a fixed sequence of f32 operations; W = sum w;
 * P = max(1, (uint64)((double)top_p * W)) (W for top_p >= 1); tau = largest integer with S(tau) = sum of the w >= tau
 * reaching P; r = floor(u * S(tau) / 2^64) with u = mix64(mix64(seed + GOLDEN * (seq + 1)) + pos); the token is the first
 * index with w >= tau, in index order, whose running sum of w exceeds r.  row_seq / row_pos: device int32 [rows] (NULL:
 * zeros).  scratch: device memory of rows * cols * 4 bytes.  A row without a finite logit, or whose maximum is +inf, is
 * sampled greedily. */
int blum_sample_top_p(blum_ctx* ctx, const float* logits, int64_t rows, int64_t cols, float temperature, float top_p,
                      uint64_t seed, const int32_t* row_seq, const int32_t* row_pos, void* scratch, int32_t* out_idx);

/* ------------------------------------------------------------------ paged KV cache
 * The reference cache is one contiguous [1, kv_heads, pos, head_dim] tensor per layer that is
 * rebuilt on every step (examples/llama/src/model.rs:108-110,140).  Here: a pool of pages
 * [layer][page][k|v][kv_head][page_size][head_dim], a per-sequence page table, append in place. */
int blum_kv_create(blum_ctx* ctx, int layers, int kv_heads, int head_dim, int page_size,
                   int64_t num_pages, int max_seqs, int max_pages_per_seq, blum_dtype dtype,
                   blum_kv** out);
int blum_kv_destroy(blum_ctx* ctx, blum_kv* kv);
/* Host-side page allocator.  seq_alloc returns a sequence slot; seq_extend grows it to hold
 * `new_len` tokens (allocating pages as needed); seq_free returns its pages to the pool. */
int blum_kv_seq_alloc(blum_ctx* ctx, blum_kv* kv, int* seq_out);
int blum_kv_seq_extend(blum_ctx* ctx, blum_kv* kv, int seq, int64_t new_len);
int blum_kv_seq_free(blum_ctx* ctx, blum_kv* kv, int seq);
int64_t blum_kv_seq_len(const blum_kv* kv, int seq);
int64_t blum_kv_free_pages(const blum_kv* kv);
/* Uses caller-chosen physical pages for a sequence (tests: shuffled page ids). */
int blum_kv_seq_set_pages(blum_ctx* ctx, blum_kv* kv, int seq, const int32_t* pages, int npages,
                          int64_t len);
/* Copies the page table (int32 [max_seqs][max_pages_per_seq]) to the device if it changed. */
int blum_kv_sync_tables(blum_ctx* ctx, blum_kv* kv);
const int32_t* blum_kv_page_table_dev(const blum_kv* kv);
void* blum_kv_pool_dev(const blum_kv* kv);
size_t blum_kv_pool_bytes(const blum_kv* kv);

/* Writes k,v [T, kv_heads, head_dim] of layer `layer` at (seq_ids[t], positions[t]).
 * Replaces concat_along + contiguous (examples/llama/src/model.rs:109-110,140). */
int blum_kv_append_paged(blum_ctx* ctx, blum_kv* kv, int layer, const void* k, const void* v,
                         blum_dtype dtype, const int32_t* seq_ids, const int32_t* positions, int64_t T);
/* qkv [T, (q_heads+2*kv_heads)*head_dim] -> rotary on q and k, q_out [T, q_heads*head_dim],
 * k and v appended to the cache: the per-token glue of examples/llama/src/model.rs:89-110. */
int blum_rope_kv_append(blum_ctx* ctx, blum_kv* kv, int layer, const void* qkv, blum_dtype dtype,
                        int q_heads, float theta, const int32_t* seq_ids, const int32_t* positions,
                        int64_t T, void* q_out);
/* Gathers a sequence's K or V of one layer into contiguous [kv_heads, len, head_dim] (reference layout). */
int blum_kv_gather_contiguous(blum_ctx* ctx, blum_kv* kv, int layer, int seq, int which_v,
                              void* out, blum_dtype out_dtype);

/* ------------------------------------------------------------------ attention
 * Decode: one query token per sequence, q [B, q_heads, head_dim], softmax(q k^T / sqrt(d)) v over
 * the first ctx_lens[b] cached positions of sequence seq_ids[b]; split over KV chunks and merged.
 * Replaces the cuBLAS QK^T + scale/mask + CudaSoftmax + cuBLAS PV chain
 * (examples/llama/src/model.rs:113-136; crates/luminal_cuda/src/matmul.rs:59-107; unary.rs:493-593).
 * `scratch` holds split partials: blum_attn_decode_scratch_bytes(...) bytes. */
size_t blum_attn_decode_scratch_bytes(int64_t B, int q_heads, int head_dim, int max_splits);
int blum_attn_decode_paged(blum_ctx* ctx, blum_kv* kv, int layer, const void* q, blum_dtype dtype,
                           int q_heads, const int32_t* seq_ids, const int32_t* ctx_lens, int64_t B,
                           int max_splits, void* scratch, void* out);
/* The whole per-token attention glue of examples/llama/src/model.rs:89-136 in one launch: qkv [B, (q_heads+2*kv_heads)*
 * head_dim] -> RoPE on q and k, the new k/v row written at position ctx_lens[b]-1 of sequence seq_ids[b] (which must
 * already be extended to that length), attention over positions [0, ctx_lens[b]); out [B, q_heads*head_dim]. */
int blum_rope_attn_decode_paged(blum_ctx* ctx, blum_kv* kv, int layer, const void* qkv, blum_dtype dtype, int q_heads,
                                float theta, const int32_t* seq_ids, const int32_t* ctx_lens, int64_t B,
                                int max_splits, void* scratch, void* out);

/* Split decode attention for callers that may not allocate.  No counterpart in the reference: luminal allocates
 * a fresh output (and any workspace) inside every Operator::process call.  Some integrations cannot do that on the
 * serving path: a runtime that reserves all device memory at start-up and leaves none for later cudaMalloc calls,
 * or a latency-critical decode thread that must avoid cudaMalloc/cudaFree because they synchronise the whole device
 * and can fail under memory pressure in the middle of a request.  This entry point computes exactly what
 * blum_attn_decode_paged computes, but keeps the split partials in a buffer that is part of the library image
 * (blum_attn_decode_static_scratch_bytes() = 8 MiB of device memory, held by every GPU that loads the library
 * until the process exits).  It never calls cudaMalloc, cudaFree or any allocating routine.
 *   - Limit: B * q_heads * max_splits * (head_dim + 2) * 4 bytes must fit in the buffer; larger requests are
 *     rejected with BLUM_ERR_INVALID and a message naming both sizes.
 *   - The first call on a device looks the buffer's device address up (one cudaGetSymbolAddress with that device made
 *     current for the lookup and the caller's device restored afterwards); make that first call before starting any
 *     stream capture.  Like every launch of this library, the call expects the context's device to be current.
 *   - If sequences grew since the last call (blum_kv_seq_extend / seq_alloc / seq_free), the page table is uploaded
 *     inside this call, which waits for the stream.  Call blum_kv_sync_tables() yourself after growing sequences
 *     and before a capture or a latency-critical call; with a clean table this entry point only launches kernels.
 *   - All calls on a device share the one buffer.  Calls that may overlap on the GPU (different streams, or
 *     different contexts on the same device) race on it; calls ordered on one stream are safe, and nothing
 *     written by an earlier call is ever read by a later one. */
size_t blum_attn_decode_static_scratch_bytes(void);
int blum_attn_decode_paged_static(blum_ctx* ctx, blum_kv* kv, int layer, const void* q, blum_dtype dtype,
                                  int q_heads, const int32_t* seq_ids, const int32_t* ctx_lens, int64_t B,
                                  int max_splits, void* out);
/* Prefill: T new tokens of one sequence at positions [p, p+T) attending causally to [0, p+t]. */
int blum_attn_prefill_paged(blum_ctx* ctx, blum_kv* kv, int layer, const void* q, blum_dtype dtype,
                            int q_heads, int seq, int64_t p, int64_t T, void* out);

/* ------------------------------------------------------------------ dense bf16 matmul and MXFP4 mixture of experts
 * No counterpart in the reference (luminal has no MoE, top-k, MXFP4 or bf16 code); semantics are stated in csrc/moe.cu:
 * top-k ties go to the lower expert index, gates are the softmax over the selected logits, (token, choice) pairs are
 * sorted by expert, stable in token order; expert = Wdown((Wup x) * swish(Wgate x)). */
typedef struct blum_mxfp4_weight blum_mxfp4_weight;
/* y[M,N] = x[M,K] * W^T, W dense bf16 [N,K] (router / attention projections of the MoE configuration), tcgen05. */
int blum_bf16_matmul(blum_ctx* ctx, const void* w_bf16, int64_t N, int64_t K, const void* x_bf16, void* y,
                     blum_dtype y_dtype, int64_t M);
/* E stacked expert matrices [N,K] in MXFP4: packed e2m1 (element 2i in the low nibble of byte i), one e8m0 scale byte
 * per 32 elements along K. */
int blum_mxfp4_weight_from_host(blum_ctx* ctx, const void* nibbles, const void* scales, int E, int64_t N, int64_t K,
                                blum_mxfp4_weight** out);
int blum_mxfp4_weight_download(blum_ctx* ctx, const blum_mxfp4_weight* w, void* nibbles_out, void* scales_out);
int blum_mxfp4_weight_free(blum_ctx* ctx, blum_mxfp4_weight* w);
int blum_moe_route_topk(blum_ctx* ctx, const void* x_bf16, const void* router_w_bf16, const float* router_bias,
                        int64_t T, int H, int E, int k, int32_t* ids_out, float* gates_out);
int blum_moe_permute(blum_ctx* ctx, const int32_t* ids, int64_t n_pairs, int E, int32_t* sorted_src,
                     int32_t* slot_of, int32_t* offsets);
int blum_moe_gather_rows(blum_ctx* ctx, const void* x_bf16, const int32_t* sorted_src, int64_t n_pairs, int k, int H,
                         void* xp_bf16);
int blum_moe_grouped_gemm(blum_ctx* ctx, const blum_mxfp4_weight* w, const void* xp_bf16, const int32_t* offsets,
                          int64_t n_rows, void* yp, blum_dtype y_dtype, int rows_per_expert_hint);
/* Gate and up matrices [E,I,K] as one weight [E,2I,K] whose rows alternate 16 gate rows and the 16 up rows of the same
 * features (I % 16 == 0), the layout blum_moe_grouped_gemm_swiglu multiplies. */
int blum_mxfp4_weight_stack_gate_up(blum_ctx* ctx, const blum_mxfp4_weight* gate, const blum_mxfp4_weight* up,
                                    blum_mxfp4_weight** out);
/* mid[r, :] = (xp[r,:] Wup_e^T) * swish(xp[r,:] Wgate_e^T) in ONE product over the stacked weight: gate and up sums stay
 * f32 until the SwiGLU in the epilogue (the two-product form rounds both to bf16 first).  mid is bf16 [n_rows, I]. */
int blum_moe_grouped_gemm_swiglu(blum_ctx* ctx, const blum_mxfp4_weight* w_gate_up, const void* xp_bf16,
                                 const int32_t* offsets, int64_t n_rows, void* mid_bf16, int rows_per_expert_hint);
/* The expert half of the layer for small row counts (decode steps), in a streaming kernel without tensor-memory
 * hand-overs, from the rows sorted by expert to the gate-weighted sum of each token's k choices: two products (gate/up
 * over the stacked weight, SwiGLU applied while the second product stages its input, down) and the combine.  Numerics as
 * the tensor-core path with the SwiGLU epilogue: f32 gate/up sums, mid and down rows rounded to bf16.  Workspace comes
 * from the context (blum_moe_experts_small_ws_bytes; reserved on the first call, which must not be a captured one). */
int64_t blum_moe_experts_small_ws_bytes(int E, int64_t n_rows, int64_t inter, int64_t hidden);
int blum_moe_experts_small(blum_ctx* ctx, const blum_mxfp4_weight* w_gate_up, const blum_mxfp4_weight* w_down,
                           const void* xp_bf16, const int32_t* offsets, int64_t n_rows, const int32_t* slot_of,
                           const float* gates, int64_t T, int k, void* out, blum_dtype out_dtype);
int blum_moe_unpermute(blum_ctx* ctx, const void* yp_bf16, const int32_t* slot_of, const float* gates, int64_t T,
                       int k, int H, void* out, blum_dtype out_dtype);

/* ------------------------------------------------------------------ multi-GPU (no counterpart in the reference:
 * luminal hard-codes device 0, crates/luminal_cuda/src/quantized.rs:247)
 * One process per GPU.  Rank 0 calls blum_comm_unique_id and hands the 128 bytes to every rank out of band; each rank
 * then calls blum_comm_init_rank with its own context.  Collectives run on the context's stream (NCCL over NVLink).
 * Timeouts: every call that can wait for another rank takes timeout_ms.  For the init, timeout_ms > 0 gives up when a rank
 * has not joined in time (0 blocks as ncclCommInitRank does).  For a collective, timeout_ms = 0 only enqueues it (it may
 * then be captured in a CUDA graph); timeout_ms > 0 makes the call return when the collective has finished, and if it has
 * not finished in time (a peer never arrived) or NCCL reports an asynchronous error, a host watchdog aborts the
 * communicator - which ends the waiting kernel, so the context and its stream stay usable - and the call returns
 * BLUM_ERR_COMM.  An aborted communicator fails every later call at once; destroy it and build a new one. */
int blum_comm_unique_id(void* out_128_bytes);
int blum_comm_init_rank(blum_ctx* ctx, int nranks, int rank, const void* id_128_bytes, int timeout_ms, blum_comm** out);
int blum_comm_destroy(blum_ctx* ctx, blum_comm* comm);
int blum_comm_rank(const blum_comm* comm);
int blum_comm_size(const blum_comm* comm);
/* In-place sum over ranks (tensor-parallel exchange after the row-parallel o_proj / down_proj). */
int blum_allreduce_sum(blum_ctx* ctx, blum_comm* comm, void* buf, int64_t count, blum_dtype dtype, int timeout_ms);
int blum_allgather(blum_ctx* ctx, blum_comm* comm, const void* send, void* recv, int64_t bytes_per_rank, int timeout_ms);
/* Variable all-to-all in bytes (expert-parallel dispatch / combine); the four arrays are host int64 [size]. */
int blum_alltoallv(blum_ctx* ctx, blum_comm* comm, const void* send, const int64_t* send_bytes,
                   const int64_t* send_offsets, void* recv, const int64_t* recv_bytes, const int64_t* recv_offsets,
                   int timeout_ms);

/* Row-parallel exchange without a library collective (no counterpart in the reference; the unsharded computation is the
 * o_proj / down_proj matmul, the residual add of examples/llama/src/model.rs:180,186 and the RMSNorm of
 * crates/luminal_nn/src/norm.rs:62-65).  blum_peer_create is collective over `comm`: every rank allocates an exchange
 * area of two slots of max_rows rows of row_bytes, exports it with a CUDA IPC handle and maps every peer's (one process
 * per GPU with peer access; any failure on any rank fails the call on every rank with BLUM_ERR_COMM and nothing is left
 * mapped).  A projection kernel writes its partial product [rows][dim] into blum_peer_slot(peer, slot); then
 * blum_allreduce_fused, ONE kernel with one CTA per row, announces the row to every peer, waits for theirs (bounded to one
 * second: on expiry bit 0x10000 of the device error word is set and the call's results are undefined, the context stays
 * usable), loads the row of every rank with plain peer loads over NVLink, sums in rank order in f32 (so every rank gets
 * identical bits), rounds to `dtype`, adds the residual row x into x_out (x_out may be x) and, when xn_out is given, writes
 * rmsnorm(x_out) * norm_w there.  Consecutive calls must alternate slot 0 and 1 on every rank (BLUM_ERR_STATE otherwise):
 * that is what makes a slot safe to overwrite two exchanges later.  Row counts above max_rows are for NCCL. */
int blum_peer_create(blum_ctx* ctx, blum_comm* comm, int64_t row_bytes, int max_rows, int timeout_ms, blum_peer** out);
int blum_peer_destroy(blum_ctx* ctx, blum_peer* peer);
void* blum_peer_slot(blum_peer* peer, int slot);
int blum_peer_max_rows(const blum_peer* peer);
int blum_allreduce_fused(blum_ctx* ctx, blum_peer* peer, int slot, const void* x, const float* norm_w, float eps,
                         void* xn_out, void* x_out, blum_dtype dtype, int rows, int64_t dim);

/* ------------------------------------------------------------------ Llama decoder
 * The model of examples/llama/src/model.rs as one object: weights, KV pool, scratch and a
 * captured CUDA graph of the single-token step (the reference executes ~10^3 nodes per token
 * through Graph::execute, src/graph.rs:191-224). */
typedef struct blum_llama_cfg {
    int32_t layers, hidden, q_heads, kv_heads, head_dim, ffn, vocab;
    float   rms_eps, rope_theta;
    int32_t act_dtype;       /* blum_dtype of activations */
    int32_t kv_dtype;        /* blum_dtype of the KV cache */
    int32_t page_size;       /* tokens per KV page */
    int32_t max_seqs;        /* concurrent sequences */
    int32_t max_ctx;         /* longest context per sequence */
    int64_t kv_pages;        /* pages in the pool (0 = max_seqs * ceil(max_ctx/page_size)) */
    int32_t embed_q8;        /* 1: embedding table is Q8_0, 0: f32 */
    int32_t tp_rank, tp_size;/* tensor-parallel shard of this object (0,1 = unsharded) */
    /* the sibling decoders of examples/llama: all zero = Llama */
    int32_t rope_mode;       /* 0: interleaved pairs (x[2i], x[2i+1]) as examples/llama/src/model.rs:52-72 and examples/phi/src/model.rs:50-70;
                                1: half-split pairs (x[i], x[i+d/2]) as examples/qwen/src/model.rs:52-77 */
    int32_t qk_norm;         /* 1: per-head RMSNorm with weight on q and k before RoPE (examples/qwen/src/model.rs:93-105,160-161);
                                tensors blk.N.attn_q_norm.weight / attn_k_norm.weight, f32 [head_dim] */
    int32_t tie_head;        /* 1: logits = x * token_embd^T (examples/qwen/src/model.rs:233: embedding.reverse); needs embed_q8 = 1, no output.weight */
} blum_llama_cfg;

int blum_llama_create(blum_ctx* ctx, const blum_llama_cfg* cfg, blum_llama** out);
int blum_llama_destroy(blum_ctx* ctx, blum_llama* m);
/* Installs one tensor by GGUF name ("blk.3.attn_q.weight", "token_embd.weight", ...;
 * examples/llama/src/model.rs:250-259) from host bytes: Q8_0 blocks or f32. */
int blum_llama_set_tensor(blum_ctx* ctx, blum_llama* m, const char* gguf_name, const void* host_bytes,
                          size_t nbytes, int is_q8_0);
uint64_t blum_llama_tensor_id(const char* gguf_name);
int blum_llama_set_comm(blum_ctx* ctx, blum_llama* m, blum_comm* comm);
/* Next-token rule of prefill / decode / decode_loop.  temperature = 0 (the default) is the reference's greedy rule
 * (examples/llama/src/main.rs:194-198); temperature > 0 samples with blum_sample_top_p keyed by (seed, sequence slot,
 * position), so the same seed reproduces the same text.  No counterpart in the reference for temperature > 0. */
int blum_llama_set_sampling(blum_ctx* ctx, blum_llama* m, float temperature, float top_p, uint64_t seed);
/* Tensor-parallel models only (no counterpart in the reference): enable = 1 makes steps of up to 64 rows sum their
 * row-parallel projections with blum_allreduce_fused over a peer-mapped area (collective: every rank must call it);
 * enable = 0 returns to NCCL all-reduce + add.  Larger row counts always use NCCL. */
int blum_llama_set_peer_allreduce(blum_ctx* ctx, blum_llama* m, int enable, int timeout_ms);
int blum_llama_peer_allreduce(const blum_llama* m);
blum_kv* blum_llama_kv(blum_llama* m);
/* Prefill `T` prompt tokens (host int32 ids) of sequence `seq` starting at its current length;
 * returns the greedy next token.  logits_out (host f32 [vocab]) may be NULL. */
int blum_llama_prefill(blum_ctx* ctx, blum_llama* m, int seq, const int32_t* host_ids, int64_t T,
                       int32_t* next_token, float* logits_out);
/* One decode step for `B` sequences: host ids in, greedy tokens out (pinned or pageable host
 * memory).  This is the call the decode loop of examples/llama/src/main.rs:152-181 maps to. */
int blum_llama_decode(blum_ctx* ctx, blum_llama* m, const int32_t* seq_ids, const int32_t* host_ids,
                      int64_t B, int32_t* next_tokens, float* logits_out);
/* Device-resident loop: runs `steps` greedy steps for one sequence feeding each token back on the
 * device, tokens_out host int32 [steps].  Used for device-only throughput timing. */
int blum_llama_decode_loop(blum_ctx* ctx, blum_llama* m, int seq, int32_t first_token, int steps,
                           int32_t* tokens_out);
/* How a single-sequence decode step is executed.  The reference has one way (Graph::execute interprets the node list,
 * src/graph.rs:191-224); here there are two: path 0 (default) runs the step as one persistent kernel with a continuous
 * weight stream when the model allows it (f32 activations and cache, head_dim 128, no tensor parallelism, hidden / ffn /
 * q width multiples of 512) and falls back to path 1 otherwise; path 1 always replays the captured graph of per-op
 * kernels.  blum_llama_decode_path returns the path a single-sequence step takes now: 2 = persistent kernel, 1 = graph. */
int blum_llama_set_decode_path(blum_ctx* ctx, blum_llama* m, int path);
int blum_llama_decode_path(blum_ctx* ctx, blum_llama* m);
/* Bytes of Q8_0 weights read per decoded token (algorithmic). */
int64_t blum_llama_weight_bytes(const blum_llama* m);

#ifdef __cplusplus
}
#endif
#endif /* BLUM_H */
