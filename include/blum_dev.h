/*
 * blum_dev.h - development, test and bench hooks of libblum.so.
 *
 * None of these stands in for a reference interface: they generate the seeded synthetic inputs the tests and benches
 * share, time launches on the device, record traces and expose a model's own tensors for per-kernel timing.  A host
 * program that uses libblum.so as a drop-in for luminal's CUDA kernels needs only blum.h.
 */
#ifndef BLUM_DEV_H
#define BLUM_DEV_H

#include "blum.h"

#ifdef __cplusplus
extern "C" {
#endif

/* Development aid: per-launch device timestamps (globaltimer ns) of the kernels that support it (decode GEMV and
 * fused decode attention).  Enable BEFORE the launches are issued or captured; each such launch then takes the next
 * record {earliest CTA start, latest dependency-wait return, latest prologue end, latest CTA end}.  A captured graph
 * keeps writing to the records it was captured with; blum_trace_reset clears them between replays. */
int blum_trace_enable(blum_ctx* ctx, int max_launches);
int blum_trace_reset(blum_ctx* ctx);
int blum_trace_read(blum_ctx* ctx, uint64_t* out, int max_records, int* n_records);

/* Timing on the context's stream (cudaEvent pairs); slot in [0,64). */
int blum_timer_start(blum_ctx* ctx, int slot);
int blum_timer_stop(blum_ctx* ctx, int slot);
int blum_timer_elapsed_ms(blum_ctx* ctx, int slot, float* ms); /* synchronises on the stop event */
/* Writes `bytes` of a private scratch buffer (> L2) so the next kernel starts cold. */
int blum_flush_l2(blum_ctx* ctx);

/* ------------------------------------------------------------------ seeded generators
 * Counter-based inputs shared by tests and benches: h = mix64(key(seed,tensor_id) + index).
 * Integer parts run on the device; scales / normals are made on the host in double and
 * uploaded, so host and device agree bit for bit. */
int blum_gen_q8_quants_host(uint64_t seed, uint64_t tensor_id, int64_t n, int8_t* out);
int blum_gen_q8_scales_host(uint64_t seed, uint64_t tensor_id, int64_t nblocks, uint16_t* out_f16);
int blum_gen_normal_host(uint64_t seed, uint64_t tensor_id, int64_t n, float stddev, float* out);
int blum_gen_token_ids_host(uint64_t seed, uint64_t tensor_id, int64_t n, int32_t vocab, int32_t* out);

/* Generates quants on the device from (seed, tensor_id) and uploads host-made scales
 * (nblocks = N*K/32 f16 values, e.g. from blum_gen_q8_scales_host). */
int blum_q8_0_weight_generate(blum_ctx* ctx, uint64_t seed, uint64_t tensor_id, int64_t N, int64_t K,
                              const uint16_t* host_scales_f16, blum_q8_weight** out);

/* Measurement helper: captures `iters` matmul launches (cycling through ws[0..nws) so that consecutive
 * launches read different weights) in one CUDA graph and returns the average device time per launch.
 * The kernel is the one blum_q8_0_matmul picks. */
int blum_q8_0_matmul_timed(blum_ctx* ctx, blum_q8_weight* const* ws, int nws, const void* x, blum_dtype x_dtype,
                           void* y, blum_dtype y_dtype, int64_t M, int iters, float* avg_us);

/* E stacked MXFP4 expert matrices from the seeded generator (codes uniform over 16 values, block exponents in [-8, 0]). */
int blum_mxfp4_weight_generate(blum_ctx* ctx, uint64_t seed, uint64_t tensor_id, int E, int64_t N, int64_t K,
                               blum_mxfp4_weight** out);

/* Fills all weights from the seeded generator (Q8_0 linears, N(0,0.02) f32 embedding, norm = 1).
 * tensor ids follow blum_llama_tensor_id(). */
int blum_llama_generate_weights(blum_ctx* ctx, blum_llama* m, uint64_t seed);

/* Average device time (CUDA events) of the persistent decode kernel alone: the step run last is launched `iters` more
 * times (see csrc/llama.cu). */
int blum_llama_stream_kernel_us(blum_ctx* ctx, blum_llama* m, int iters, float* avg_us);
/* Development aid: average per-CTA cycle counters of the persistent decode kernel (see csrc/llama.cu). */
int blum_llama_stream_profile(blum_ctx* ctx, blum_llama* m, double* out, int per_cta);

/* Borrowed handles to the model's own tensors, for per-kernel timing: which = 0 fused q/k/v, 1 attn_output,
 * 2 ffn_gate, 3 ffn_up, 4 ffn_down, 5 output head (layer ignored).  Norm weights: 0 attn_norm, 1 ffn_norm, 2 output_norm. */
blum_q8_weight* blum_llama_layer_weight(blum_llama* m, int layer, int which);
const float* blum_llama_norm_weight(blum_llama* m, int layer, int which);
/* Plays one failure scenario of the multi-GPU entry points against host stubs of NCCL (no GPU, no second rank): 1 the init
 * fails, 2 a collective returns an error, 3 a peer never arrives at a collective (the watchdog must abort the communicator
 * after timeout_ms), 4 a rank never joins the init, 5 everything works.  Returns the status the entry points returned
 * (BLUM_ERR_STATE if the aborted communicator misbehaved afterwards) and copies their message out. */
int blum_comm_selftest(int scenario, int timeout_ms, char* message_out, int message_cap);
/* Number of kernels launched by this library on ctx since creation (bench bookkeeping). */
int64_t blum_launch_count(blum_ctx* ctx);

/* Average device time of the packed-rows matmul (the integer-path kernel the decoder uses for 5 .. 128 rows) on one matrix:
 * `copies` packed copies are cycled so that every launch streams from HBM; `iters` launches in one CUDA graph. */
int blum_rows_matmul_timed(blum_ctx* ctx, const blum_q8_weight* w, int M, blum_dtype x_dtype, int copies, int iters, float* avg_us);

#ifdef __cplusplus
}
#endif
#endif /* BLUM_DEV_H */
