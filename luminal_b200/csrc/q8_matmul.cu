// Dispatcher of the Q8_0 matmul entry points: picks the GEMV family (M <= 2, or f32 activations), the register-streaming
// mma.sync kernel (3 <= M <= 16, bf16 activations) or the tcgen05 GEMM (larger M, tensor-core-bound).  Replaces QuantizedMatmul<T>::process
// (crates/luminal_cuda/src/quantized.rs:116-168 in luminal).
#include "common.cuh"

int blum_gemv_dispatch(blum_ctx* ctx, const blum_q8_weight* w, const blum_q8_weight* w_up, const void* x, int xdt,
                       const float* norm_w, float eps, const void* residual, void* y, int ydt, int64_t M);
int blum_gemm_tc_supported(const blum_ctx* ctx, const blum_q8_weight* w, int xdt, int ydt, int64_t M);
int blum_gemm_tc_dispatch(blum_ctx* ctx, const blum_q8_weight* w, const void* x, int xdt, void* y, int ydt, int64_t M);

int blum_gemm_small_supported(const blum_q8_weight* w, int xdt, int ydt, int64_t M);
int blum_gemm_small_dispatch(blum_ctx* ctx, const blum_q8_weight* w, const void* x, int xdt, void* y, int ydt, int64_t M);

// M at or above which the tensor-core kernels take over from the GEMV family, and the largest M of the small-batch kernel.
#define BLUM_GEMM_MIN_M 3
#define BLUM_GEMM_SMALL_MAX_M 16   // measured: 25 vs 33 us at M=16 on 4096x14336; the small-batch kernel holds 16 tokens

extern "C" {

int blum_q8_0_matmul(blum_ctx* ctx, const blum_q8_weight* w, const void* x, blum_dtype xdt, void* y, blum_dtype ydt,
                     int64_t M) {
    if (!ctx) return BLUM_ERR_INVALID;
    if (M == 0) return BLUM_OK;
    if (M >= BLUM_GEMM_MIN_M && M <= BLUM_GEMM_SMALL_MAX_M && w && blum_gemm_small_supported(w, xdt, ydt, M))
        return blum_gemm_small_dispatch(ctx, w, x, xdt, y, ydt, M);
    if (M >= BLUM_GEMM_MIN_M && w && blum_gemm_tc_supported(ctx, w, xdt, ydt, M))
        return blum_gemm_tc_dispatch(ctx, w, x, xdt, y, ydt, M);
    return blum_gemv_dispatch(ctx, w, nullptr, x, xdt, nullptr, 0.f, nullptr, y, ydt, M);
}

int blum_q8_0_matmul_fused(blum_ctx* ctx, const blum_q8_weight* w, const void* x, blum_dtype xdt,
                           const float* norm_weight, float eps, const void* residual, void* y, blum_dtype ydt,
                           int64_t M) {
    if (!ctx) return BLUM_ERR_INVALID;
    if (M == 0) return BLUM_OK;
    return blum_gemv_dispatch(ctx, w, nullptr, x, xdt, norm_weight, eps, residual, y, ydt, M);
}

int blum_q8_0_matmul_timed(blum_ctx* ctx, blum_q8_weight* const* ws, int nws, const void* x, blum_dtype xdt, void* y,
                           blum_dtype ydt, int64_t M, int iters, float* avg_us) {
    if (!ctx) return BLUM_ERR_INVALID;
    BLUM_REQUIRE(ctx, ws && nws > 0 && iters > 0 && avg_us, "matmul_timed: bad argument");
    // one plain launch first: lets every path size its workspaces outside the capture
    {
        const int rc0 = blum_q8_0_matmul(ctx, ws[0], x, xdt, y, ydt, M);
        if (rc0) return rc0;
        BLUM_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
    }
    cudaGraph_t graph = nullptr;
    const int64_t launches_before = ctx->launches;
    BLUM_CUDA(ctx, cudaStreamBeginCapture(ctx->stream, cudaStreamCaptureModeThreadLocal));
    int rc = BLUM_OK;
    for (int i = 0; i < iters && !rc; i++) {
        const blum_q8_weight* w = ws[i % nws];
        rc = blum_q8_0_matmul(ctx, w, x, xdt, y, ydt, M);
    }
    cudaError_t e = cudaStreamEndCapture(ctx->stream, &graph);
    ctx->launches = launches_before;
    if (rc) { if (graph) cudaGraphDestroy(graph); return rc; }
    if (e != cudaSuccess) return blum_fail(ctx, BLUM_ERR_CUDA, "matmul_timed: capture failed: %s", cudaGetErrorString(e));
    cudaGraphExec_t exec = nullptr;
    e = cudaGraphInstantiate(&exec, graph, 0);
    cudaGraphDestroy(graph);
    if (e != cudaSuccess) return blum_fail(ctx, BLUM_ERR_CUDA, "matmul_timed: instantiate failed: %s", cudaGetErrorString(e));
    cudaEvent_t a, b;
    cudaEventCreate(&a); cudaEventCreate(&b);
    cudaGraphLaunch(exec, ctx->stream);                 // warm-up pass
    cudaEventRecord(a, ctx->stream);
    cudaGraphLaunch(exec, ctx->stream);
    cudaEventRecord(b, ctx->stream);
    e = cudaEventSynchronize(b);
    float ms = 0.f;
    cudaEventElapsedTime(&ms, a, b);
    cudaEventDestroy(a); cudaEventDestroy(b);
    cudaGraphExecDestroy(exec);
    if (e != cudaSuccess) return blum_fail(ctx, BLUM_ERR_CUDA, "matmul_timed: %s", cudaGetErrorString(e));
    ctx->launches += 2 * (int64_t)iters;
    *avg_us = ms * 1000.f / (float)iters;
    return BLUM_OK;
}

int blum_q8_0_matmul_swiglu(blum_ctx* ctx, const blum_q8_weight* w_gate, const blum_q8_weight* w_up, const void* x,
                            blum_dtype xdt, const float* norm_weight, float eps, void* y, blum_dtype ydt, int64_t M) {
    if (!ctx) return BLUM_ERR_INVALID;
    BLUM_REQUIRE(ctx, w_gate && w_up, "q8 swiglu: null weight");
    if (M == 0) return BLUM_OK;
    return blum_gemv_dispatch(ctx, w_gate, w_up, x, xdt, norm_weight, eps, nullptr, y, ydt, M);
}

}  // extern "C"
