// Context, buffers, timers and the seeded input generators of libblum.so.
#include "common.cuh"
#include <stdarg.h>
#include <math.h>
#include <string.h>

int blum_fail(blum_ctx* ctx, int code, const char* fmt, ...) {
    char buf[512];
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(buf, sizeof buf, fmt, ap);
    va_end(ap);
    if (ctx) ctx->err = buf;
    return code;
}

extern "C" {

const char* blum_version(void) { return "blum 0.1 (sm_100a)"; }

int blum_ctx_create(int device, blum_ctx** out) {
    if (!out) return BLUM_ERR_INVALID;
    *out = nullptr;
    blum_ctx* ctx = new blum_ctx();
    ctx->device = device;
    cudaError_t e = cudaSetDevice(device);
    if (e != cudaSuccess) { delete ctx; return BLUM_ERR_CUDA; }
    cudaDeviceProp prop;
    e = cudaGetDeviceProperties(&prop, device);
    if (e != cudaSuccess) { delete ctx; return BLUM_ERR_CUDA; }
    ctx->sm_count = prop.multiProcessorCount;
    ctx->smem_optin = prop.sharedMemPerBlockOptin;
    e = cudaStreamCreateWithFlags(&ctx->stream, cudaStreamNonBlocking);
    if (e != cudaSuccess) { delete ctx; return BLUM_ERR_CUDA; }
    ctx->own_stream = true;
    e = cudaMalloc(&ctx->dev_error, sizeof(int));
    if (e != cudaSuccess) { cudaStreamDestroy(ctx->stream); delete ctx; return BLUM_ERR_CUDA; }
    cudaMemset(ctx->dev_error, 0, sizeof(int));
    e = cudaMalloc(&ctx->argmax_ws, (size_t)BLUM_ARGMAX_ROWS * 16);
    if (e != cudaSuccess) { cudaFree(ctx->dev_error); cudaStreamDestroy(ctx->stream); delete ctx; return BLUM_ERR_CUDA; }
    cudaMemset(ctx->argmax_ws, 0, (size_t)BLUM_ARGMAX_ROWS * 16);
    *out = ctx;
    return BLUM_OK;
}

int blum_ctx_destroy(blum_ctx* ctx) {
    if (!ctx) return BLUM_ERR_INVALID;
    cudaSetDevice(ctx->device);
    cudaStreamSynchronize(ctx->stream);
    for (int i = 0; i < 64; i++) {
        if (ctx->ev_start[i]) cudaEventDestroy(ctx->ev_start[i]);
        if (ctx->ev_stop[i]) cudaEventDestroy(ctx->ev_stop[i]);
    }
    if (ctx->flush_buf) cudaFree(ctx->flush_buf);
    if (ctx->gemm_ws) cudaFree(ctx->gemm_ws);
    for (void* r : ctx->retired) cudaFree(r);
    if (ctx->trace) cudaFree(ctx->trace);
    if (ctx->dev_error) cudaFree(ctx->dev_error);
    if (ctx->argmax_ws) cudaFree(ctx->argmax_ws);
    if (ctx->own_stream) cudaStreamDestroy(ctx->stream);
    delete ctx;
    return BLUM_OK;
}

int blum_ctx_set_stream(blum_ctx* ctx, void* s) {
    if (!ctx) return BLUM_ERR_INVALID;
    if (ctx->own_stream) { cudaStreamSynchronize(ctx->stream); cudaStreamDestroy(ctx->stream); }
    ctx->stream = (cudaStream_t)s;
    ctx->own_stream = false;
    return BLUM_OK;
}
void* blum_ctx_stream(blum_ctx* ctx) { return ctx ? (void*)ctx->stream : nullptr; }
const char* blum_last_error(blum_ctx* ctx) { return ctx ? ctx->err.c_str() : "null context"; }
int blum_ctx_device(blum_ctx* ctx) { return ctx ? ctx->device : -1; }
int blum_ctx_sm_count(blum_ctx* ctx) { return ctx ? ctx->sm_count : -1; }
int64_t blum_launch_count(blum_ctx* ctx) { return ctx ? ctx->launches : -1; }

int blum_dev_alloc(blum_ctx* ctx, size_t bytes, void** dptr) {
    if (!ctx || !dptr) return BLUM_ERR_INVALID;
    *dptr = nullptr;
    if (bytes == 0) bytes = 16;
    BLUM_CUDA(ctx, cudaSetDevice(ctx->device));
    BLUM_CUDA(ctx, cudaMalloc(dptr, bytes));
    return BLUM_OK;
}
int blum_dev_free(blum_ctx* ctx, void* dptr) {
    if (!ctx) return BLUM_ERR_INVALID;
    if (!dptr) return BLUM_OK;
    BLUM_CUDA(ctx, cudaSetDevice(ctx->device));
    BLUM_CUDA(ctx, cudaFree(dptr));
    return BLUM_OK;
}
int blum_memset(blum_ctx* ctx, void* dptr, int byte, size_t bytes) {
    if (!ctx || (!dptr && bytes)) return BLUM_ERR_INVALID;
    BLUM_CUDA(ctx, cudaMemsetAsync(dptr, byte, bytes, ctx->stream));
    return BLUM_OK;
}
int blum_memcpy_h2d(blum_ctx* ctx, void* dst, const void* src, size_t bytes) {
    if (!ctx || ((!dst || !src) && bytes)) return blum_fail(ctx, BLUM_ERR_INVALID, "memcpy_h2d: null pointer");
    if (!bytes) return BLUM_OK;
    BLUM_CUDA(ctx, cudaMemcpyAsync(dst, src, bytes, cudaMemcpyHostToDevice, ctx->stream));
    return BLUM_OK;
}
int blum_memcpy_d2h(blum_ctx* ctx, void* dst, const void* src, size_t bytes) {
    if (!ctx || ((!dst || !src) && bytes)) return blum_fail(ctx, BLUM_ERR_INVALID, "memcpy_d2h: null pointer");
    if (bytes) BLUM_CUDA(ctx, cudaMemcpyAsync(dst, src, bytes, cudaMemcpyDeviceToHost, ctx->stream));
    BLUM_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
    return BLUM_OK;
}
int blum_memcpy_d2d(blum_ctx* ctx, void* dst, const void* src, size_t bytes) {
    if (!ctx || ((!dst || !src) && bytes)) return blum_fail(ctx, BLUM_ERR_INVALID, "memcpy_d2d: null pointer");
    if (bytes) BLUM_CUDA(ctx, cudaMemcpyAsync(dst, src, bytes, cudaMemcpyDeviceToDevice, ctx->stream));
    return BLUM_OK;
}
int blum_host_alloc_pinned(blum_ctx* ctx, size_t bytes, void** hptr) {
    if (!ctx || !hptr) return BLUM_ERR_INVALID;
    BLUM_CUDA(ctx, cudaSetDevice(ctx->device));
    BLUM_CUDA(ctx, cudaHostAlloc(hptr, bytes ? bytes : 16, cudaHostAllocDefault));
    return BLUM_OK;
}
int blum_host_free_pinned(blum_ctx* ctx, void* hptr) {
    if (!ctx) return BLUM_ERR_INVALID;
    if (hptr) BLUM_CUDA(ctx, cudaFreeHost(hptr));
    return BLUM_OK;
}
int blum_sync(blum_ctx* ctx) {
    if (!ctx) return BLUM_ERR_INVALID;
    BLUM_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
    return BLUM_OK;
}
int blum_check_device_error(blum_ctx* ctx) {
    if (!ctx) return BLUM_ERR_INVALID;
    int word = 0;
    BLUM_CUDA(ctx, cudaMemcpyAsync(&word, ctx->dev_error, sizeof(int), cudaMemcpyDeviceToHost, ctx->stream));
    BLUM_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
    if (word != 0) {
        BLUM_CUDA(ctx, cudaMemsetAsync(ctx->dev_error, 0, sizeof(int), ctx->stream));
        return blum_fail(ctx, BLUM_ERR_DEVICE, "device error word = 0x%x", word);
    }
    return BLUM_OK;
}

/* Stream capture for callers that want to replay a fixed sequence of calls as one CUDA graph (what the Metal backend's
 * command-buffer compiler does for luminal, crates/luminal_metal/src/command_buffer.rs; the CUDA crate has nothing like it). */
int blum_graph_begin(blum_ctx* ctx) {
    if (!ctx) return BLUM_ERR_INVALID;
    ctx->launches_at_capture = ctx->launches;
    BLUM_CUDA(ctx, cudaStreamBeginCapture(ctx->stream, cudaStreamCaptureModeThreadLocal));
    return BLUM_OK;
}
int blum_graph_end(blum_ctx* ctx, void** graph_exec_out, int* n_kernels_out) {
    if (!ctx || !graph_exec_out) return BLUM_ERR_INVALID;
    *graph_exec_out = nullptr;
    cudaGraph_t graph = nullptr;
    const cudaError_t e = cudaStreamEndCapture(ctx->stream, &graph);
    const int captured = (int)(ctx->launches - ctx->launches_at_capture);
    ctx->launches = ctx->launches_at_capture;          // captured, not executed
    if (e != cudaSuccess) return blum_fail(ctx, BLUM_ERR_CUDA, "graph capture failed: %s", cudaGetErrorString(e));
    cudaGraphExec_t exec = nullptr;
    const cudaError_t e2 = cudaGraphInstantiate(&exec, graph, 0);
    cudaGraphDestroy(graph);
    if (e2 != cudaSuccess) return blum_fail(ctx, BLUM_ERR_CUDA, "graph instantiate failed: %s", cudaGetErrorString(e2));
    *graph_exec_out = (void*)exec;
    if (n_kernels_out) *n_kernels_out = captured;
    return BLUM_OK;
}
int blum_graph_launch(blum_ctx* ctx, void* graph_exec, int n_kernels) {
    if (!ctx || !graph_exec) return BLUM_ERR_INVALID;
    BLUM_CUDA(ctx, cudaGraphLaunch((cudaGraphExec_t)graph_exec, ctx->stream));
    ctx->launches += n_kernels;
    return BLUM_OK;
}
int blum_graph_destroy(blum_ctx* ctx, void* graph_exec) {
    if (!ctx) return BLUM_ERR_INVALID;
    if (graph_exec) { cudaStreamSynchronize(ctx->stream); cudaGraphExecDestroy((cudaGraphExec_t)graph_exec); }
    return BLUM_OK;
}

int blum_trace_enable(blum_ctx* ctx, int max_launches) {
    if (!ctx || max_launches < 0) return BLUM_ERR_INVALID;
    if (ctx->trace) { cudaFree(ctx->trace); ctx->trace = nullptr; }
    ctx->trace_cap = 0; ctx->trace_next = 0;
    if (max_launches == 0) return BLUM_OK;
    BLUM_CUDA(ctx, cudaMalloc((void**)&ctx->trace, (size_t)max_launches * 32));
    ctx->trace_cap = max_launches;
    return blum_trace_reset(ctx);
}
int blum_trace_reset(blum_ctx* ctx) {
    if (!ctx || !ctx->trace) return BLUM_ERR_INVALID;
    std::vector<unsigned long long> init((size_t)ctx->trace_cap * 4, 0ull);
    for (int i = 0; i < ctx->trace_cap; i++) init[4 * (size_t)i] = ~0ull;
    BLUM_CUDA(ctx, cudaMemcpyAsync(ctx->trace, init.data(), init.size() * 8, cudaMemcpyHostToDevice, ctx->stream));
    BLUM_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
    return BLUM_OK;
}
int blum_trace_read(blum_ctx* ctx, uint64_t* out, int max_records, int* n_records) {
    if (!ctx || !ctx->trace || !out || !n_records) return BLUM_ERR_INVALID;
    const int n = ctx->trace_next < max_records ? ctx->trace_next : max_records;
    BLUM_CUDA(ctx, cudaMemcpyAsync(out, ctx->trace, (size_t)n * 32, cudaMemcpyDeviceToHost, ctx->stream));
    BLUM_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
    *n_records = n;
    return BLUM_OK;
}

int blum_timer_start(blum_ctx* ctx, int slot) {
    if (!ctx || slot < 0 || slot >= 64) return BLUM_ERR_INVALID;
    if (!ctx->ev_start[slot]) {
        BLUM_CUDA(ctx, cudaEventCreate(&ctx->ev_start[slot]));
        BLUM_CUDA(ctx, cudaEventCreate(&ctx->ev_stop[slot]));
    }
    BLUM_CUDA(ctx, cudaEventRecord(ctx->ev_start[slot], ctx->stream));
    return BLUM_OK;
}
int blum_timer_stop(blum_ctx* ctx, int slot) {
    if (!ctx || slot < 0 || slot >= 64 || !ctx->ev_stop[slot]) return BLUM_ERR_INVALID;
    BLUM_CUDA(ctx, cudaEventRecord(ctx->ev_stop[slot], ctx->stream));
    return BLUM_OK;
}
int blum_timer_elapsed_ms(blum_ctx* ctx, int slot, float* ms) {
    if (!ctx || !ms || slot < 0 || slot >= 64 || !ctx->ev_stop[slot]) return BLUM_ERR_INVALID;
    BLUM_CUDA(ctx, cudaEventSynchronize(ctx->ev_stop[slot]));
    BLUM_CUDA(ctx, cudaEventElapsedTime(ms, ctx->ev_start[slot], ctx->ev_stop[slot]));
    return BLUM_OK;
}

__global__ void flush_kernel(int4* buf, size_t n, int v) {
    size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x;
    size_t stride = (size_t)gridDim.x * blockDim.x;
    for (; i < n; i += stride) buf[i] = make_int4(v, v, v, v);
}

int blum_flush_l2(blum_ctx* ctx) {
    if (!ctx) return BLUM_ERR_INVALID;
    if (!ctx->flush_buf) {
        ctx->flush_bytes = (size_t)256 << 20;   // 2x the 126 MB L2
        BLUM_CUDA(ctx, cudaMalloc(&ctx->flush_buf, ctx->flush_bytes));
    }
    flush_kernel<<<ctx->sm_count * 4, 512, 0, ctx->stream>>>((int4*)ctx->flush_buf, ctx->flush_bytes / 16,
                                                             (int)ctx->launches);
    BLUM_LAUNCH_CHECK(ctx);
    ctx->launches--;   // the flush is bookkeeping, not product work
    return BLUM_OK;
}

// ------------------------------------------------------------------ host generators
static inline double gen_uniform(uint64_t key, uint64_t i) {
    return ((double)(blum_gen_hash(key, i) >> 11) + 0.5) * (1.0 / 9007199254740992.0);
}
static inline double gen_normal(uint64_t key, uint64_t i) {
    const double u1 = gen_uniform(key, 2 * i), u2 = gen_uniform(key, 2 * i + 1);
    return sqrt(-2.0 * log(u1)) * cos(6.283185307179586476925286766559 * u2);
}
}  // extern "C"

// f16 scales |N(0,0.02)|/127 of blocks [first_block, first_block+nblocks) of a tensor
int blum_gen_q8_scales_range(uint64_t seed, uint64_t tensor_id, int64_t first_block, int64_t nblocks, uint16_t* out) {
    if (!out || nblocks < 0 || first_block < 0) return BLUM_ERR_INVALID;
    // scales use a key derived from the tensor's id so that they are independent of its quants
    const uint64_t key = blum_gen_key(seed, tensor_id ^ (0x5ca1e5ull << 40));
#pragma omp parallel for schedule(static)
    for (int64_t i = 0; i < nblocks; i++) {
        const float s = (float)(fabs(0.02 * gen_normal(key, (uint64_t)(first_block + i))) / 127.0);
        const __half h = __float2half_rn(s);
        uint16_t bits;
        memcpy(&bits, &h, 2);
        out[i] = bits;
    }
    return BLUM_OK;
}

void blum_gen_normal_range(uint64_t key, int64_t first, int64_t n, float stddev, float* out) {
#pragma omp parallel for schedule(static)
    for (int64_t i = 0; i < n; i++) out[i] = (float)((double)stddev * gen_normal(key, (uint64_t)(first + i)));
}

extern "C" {
int blum_gen_q8_quants_host(uint64_t seed, uint64_t tensor_id, int64_t n, int8_t* out) {
    if (!out || n < 0) return BLUM_ERR_INVALID;
    const uint64_t key = blum_gen_key(seed, tensor_id);
#pragma omp parallel for schedule(static)
    for (int64_t i = 0; i < n; i++) out[i] = (int8_t)blum_gen_quant(key, (uint64_t)i);
    return BLUM_OK;
}

int blum_gen_q8_scales_host(uint64_t seed, uint64_t tensor_id, int64_t nblocks, uint16_t* out) {
    return blum_gen_q8_scales_range(seed, tensor_id, 0, nblocks, out);
}

int blum_gen_normal_host(uint64_t seed, uint64_t tensor_id, int64_t n, float stddev, float* out) {
    if (!out || n < 0) return BLUM_ERR_INVALID;
    blum_gen_normal_range(blum_gen_key(seed, tensor_id), 0, n, stddev, out);
    return BLUM_OK;
}

int blum_gen_token_ids_host(uint64_t seed, uint64_t tensor_id, int64_t n, int32_t vocab, int32_t* out) {
    if (!out || n < 0 || vocab <= 0) return BLUM_ERR_INVALID;
    const uint64_t key = blum_gen_key(seed, tensor_id);
    for (int64_t i = 0; i < n; i++)
        out[i] = (int32_t)(((blum_gen_hash(key, (uint64_t)i) >> 32) * (uint64_t)vocab) >> 32);
    return BLUM_OK;
}

}  // extern "C"
