// Internal definitions shared by the translation units of libblum.so.
#pragma once
#include <cuda_runtime.h>
#include <cuda_fp16.h>
#include <cuda_bf16.h>
#include <stdint.h>
#include <stdio.h>
#include <string>
#include <vector>
#include "../../include/blum.h"
#include "../../include/blum_dev.h"

#define BLUM_ARGMAX_ROWS 2048

struct blum_ctx {
    int device = 0;
    int sm_count = 0;
    size_t smem_optin = 0;
    cudaStream_t stream = nullptr;
    bool own_stream = false;
    std::string err;
    int* dev_error = nullptr;          // device error word written by kernels
    cudaEvent_t ev_start[64] = {};
    cudaEvent_t ev_stop[64] = {};
    void* flush_buf = nullptr;
    size_t flush_bytes = 0;
    int64_t launches = 0;
    int64_t launches_at_capture = 0;
    bool pdl = true;                   // launch chained kernels with programmatic dependent launch
    unsigned long long* trace = nullptr;   // device [trace_cap][4] timestamps, or null (development aid)
    int trace_cap = 0, trace_next = 0;
    void* gemm_ws = nullptr;           // f32 workspace of the split-K tensor-core GEMM (grown on demand)
    size_t gemm_ws_bytes = 0;
    void* argmax_ws = nullptr;         // BLUM_ARGMAX_ROWS zeroed 16-byte records of the split argmax (each launch leaves them zero)
    std::vector<void*> retired;        // outgrown workspaces: captured graphs may still name them, freed with the context
};

// next trace record of this context (null when tracing is off or the buffer is full)
static inline unsigned long long* blum_trace_slot(blum_ctx* ctx) {
    if (!ctx->trace || ctx->trace_next >= ctx->trace_cap) return nullptr;
    return ctx->trace + 4 * (size_t)(ctx->trace_next++);
}

struct blum_q8_weight {
    int64_t N = 0, K = 0;
    int8_t* q = nullptr;    // [N][K]
    __half* d = nullptr;    // [N][K/32]
    bool owns = true;
};

struct blum_mxfp4_weight {
    int E = 0;
    int64_t N = 0, K = 0;
    uint8_t* q = nullptr;      // [E*N][K/2] packed e2m1
    uint8_t* s = nullptr;      // [E*N][K/32] e8m0
};

int blum_fail(blum_ctx* ctx, int code, const char* fmt, ...);
int blum_swiglu_rows(blum_ctx* ctx, const void* gate_up, void* out, int dt, int64_t R, int64_t F);

#define BLUM_CUDA(ctx, call)                                                              \
    do {                                                                                  \
        cudaError_t e__ = (call);                                                         \
        if (e__ != cudaSuccess)                                                           \
            return blum_fail((ctx), (e__ == cudaErrorMemoryAllocation) ? BLUM_ERR_OOM     \
                                                                       : BLUM_ERR_CUDA,   \
                             "%s failed: %s (%s:%d)", #call, cudaGetErrorString(e__),     \
                             __FILE__, __LINE__);                                         \
    } while (0)

#define BLUM_REQUIRE(ctx, cond, ...)                                    \
    do {                                                                \
        if (!(cond)) return blum_fail((ctx), BLUM_ERR_INVALID, __VA_ARGS__); \
    } while (0)

// Checks the launch itself (configuration errors); execution errors surface at the next sync.
#define BLUM_LAUNCH_CHECK(ctx)                                                            \
    do {                                                                                  \
        cudaError_t e__ = cudaGetLastError();                                             \
        if (e__ != cudaSuccess)                                                           \
            return blum_fail((ctx), BLUM_ERR_CUDA, "kernel launch failed: %s (%s:%d)",    \
                             cudaGetErrorString(e__), __FILE__, __LINE__);                \
        (ctx)->launches++;                                                                \
    } while (0)

static inline size_t blum_dtype_size(int dt) { return dt == BLUM_F32 ? 4 : 2; }

// ------------------------------------------------------------------ generator (host + device)
// h(seed, tensor, i) = mix64(key(seed, tensor) + i * GOLDEN)
#define BLUM_GOLDEN 0x9E3779B97F4A7C15ull

__host__ __device__ static inline uint64_t blum_mix64(uint64_t z) {
    z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
    z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
    return z ^ (z >> 31);
}
__host__ __device__ static inline uint64_t blum_gen_key(uint64_t seed, uint64_t tensor_id) {
    return blum_mix64(blum_mix64(seed + BLUM_GOLDEN) ^ (tensor_id * 0xD1B54A32D192ED03ull + 0x8CB92BA72F3D8DD7ull));
}
__host__ __device__ static inline uint64_t blum_gen_hash(uint64_t key, uint64_t i) {
    return blum_mix64(key + i * BLUM_GOLDEN);
}
// uniform integer in [-127, 127]
__host__ __device__ static inline int blum_gen_quant(uint64_t key, uint64_t i) {
    uint64_t h = blum_gen_hash(key, i);
    return (int)(((h >> 32) * 255ull) >> 32) - 127;
}

// ------------------------------------------------------------------ device helpers
template <typename T> __device__ __forceinline__ float to_f32(T v);
template <> __device__ __forceinline__ float to_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ float to_f32<__half>(__half v) { return __half2float(v); }
template <> __device__ __forceinline__ float to_f32<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }

template <typename T> __device__ __forceinline__ T from_f32(float v);
template <> __device__ __forceinline__ float from_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ __half from_f32<__half>(float v) { return __float2half_rn(v); }
template <> __device__ __forceinline__ __nv_bfloat16 from_f32<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}

// 128-bit streaming load that does not allocate in L1 (weights are read once).
__device__ __forceinline__ int4 ld_stream_16(const void* p) {
    int4 r;
    asm volatile("ld.global.nc.L1::no_allocate.L2::128B.v4.s32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r.x), "=r"(r.y), "=r"(r.z), "=r"(r.w) : "l"(p));
    return r;
}

// Q8_0 dequantisation to bf16 for the tensor-core kernels, 2 instructions per weight plus the pack.
// Byte u = q + 128 dropped into bits 8..15 of the float 1.0 gives f = 1 + u * 2^-15.  With D = d * 2^15 and
// c = -(1 + 2^-8) * D (both exact: c has 9 x 11 significant bits), fma(f, D, c) = (u - 128) * d = q * d with a single
// rounding of a value that f32 holds exactly, so the result equals (float)q * d bit for bit (for finite d).
// Two weights share one packed-f32 fma.
struct Q8Scale { uint64_t D2, c2; };
__device__ __forceinline__ Q8Scale q8_scale_consts(float d) {
    const float D = d * 32768.f, c = D * -1.00390625f;
    Q8Scale s;
    asm("mov.b64 %0, {%1, %1};" : "=l"(s.D2) : "r"(__float_as_uint(D)));
    asm("mov.b64 %0, {%1, %1};" : "=l"(s.c2) : "r"(__float_as_uint(c)));
    return s;
}
// w: four int8 weights; lo = bf16x2(q0*d, q1*d), hi = bf16x2(q2*d, q3*d)
__device__ __forceinline__ void q8_dequant4(uint32_t w, const Q8Scale& s, uint32_t& lo, uint32_t& hi) {
    const uint32_t wx = w ^ 0x80808080u;
    uint64_t a01, a23, r01, r23;
    asm("mov.b64 %0, {%1, %2};" : "=l"(a01) : "r"(__byte_perm(wx, 0x3F800000u, 0x7604)), "r"(__byte_perm(wx, 0x3F800000u, 0x7614)));
    asm("mov.b64 %0, {%1, %2};" : "=l"(a23) : "r"(__byte_perm(wx, 0x3F800000u, 0x7624)), "r"(__byte_perm(wx, 0x3F800000u, 0x7634)));
    asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(r01) : "l"(a01), "l"(s.D2), "l"(s.c2));
    asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(r23) : "l"(a23), "l"(s.D2), "l"(s.c2));
    uint32_t f0, f1, f2, f3;
    asm("mov.b64 {%0, %1}, %2;" : "=r"(f0), "=r"(f1) : "l"(r01));
    asm("mov.b64 {%0, %1}, %2;" : "=r"(f2), "=r"(f3) : "l"(r23));
    asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(lo) : "r"(f1), "r"(f0));   // first source goes to the upper half
    asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(hi) : "r"(f3), "r"(f2));
}

// Timestamps of a launch for the tracing aid: [0] earliest CTA start, [1] latest return from the dependency wait,
// [2] latest end of the prologue, [3] latest CTA end (globaltimer nanoseconds).
__device__ __forceinline__ unsigned long long blum_globaltimer() {
    unsigned long long t; asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t)); return t;
}
__device__ __forceinline__ void blum_trace(unsigned long long* rec, int which) {
    if (rec && threadIdx.x == 0) {
        const unsigned long long t = blum_globaltimer();
        if (which == 0) atomicMin(rec, t); else atomicMax(rec + which, t);
    }
}

// Programmatic dependent launch: wait for the producing grid's memory / let the next grid start.
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

// inverse frequencies of the rotary embedding, computed on the host (head_dim/2 <= 128 entries)
struct RopeFreqs { float inv_freq[128]; };
void blum_rope_freqs(float theta, int head_dim, RopeFreqs* f);

// internal entry points shared between translation units
int blum_gen_q8_scales_range(uint64_t seed, uint64_t tensor_id, int64_t first_block, int64_t nblocks, uint16_t* out);
void blum_gen_normal_range(uint64_t key, int64_t first, int64_t n, float stddev, float* out);
int blum_q8_alloc(blum_ctx* ctx, int64_t N, int64_t K, blum_q8_weight** out);
int blum_q8_generate_window(blum_ctx* ctx, blum_q8_weight* w, int64_t dst_row0, int64_t nrows, uint64_t seed,
                            uint64_t tensor_id, int64_t K_full, int64_t src_row0, int64_t k0);
int blum_q8_fill_from_host_gguf(blum_ctx* ctx, blum_q8_weight* w, int64_t dst_row0, int64_t nrows, const void* host_bytes,
                                int64_t K_full, int64_t src_row0, int64_t k0);
int blum_gemv_dispatch(blum_ctx* ctx, const blum_q8_weight* w, const blum_q8_weight* w_up, const void* x, int xdt,
                       const float* norm_w, float eps, const void* residual, void* y, int ydt, int64_t M);
struct blum_kv;
int blum_attn_rows(blum_ctx* ctx, blum_kv* kv, int layer, const void* q, int dtype, int q_heads, const int32_t* seq_ids,
                   const int32_t* ctx_lens, int64_t rows, int nsplit, void* scratch, void* out);

// tensor-core causal attention of tokens [p0, p0 + T) of one sequence (attn_prefill_mma.cu); `covers` says whether a
// configuration is supported (16-bit activations and KV of the same type, head_dim 64/128, page size dividing 64 or a multiple of it)
bool blum_attn_prefill_mma_covers(int dtype, int kv_dtype, int d, int page_size);
int blum_attn_prefill_mma(blum_ctx* ctx, blum_kv* kv, int layer, const void* q, int dtype, int q_heads, int seq, int64_t p0, int64_t T,
                          void* out);
int blum_attn_decode_fused(blum_ctx* ctx, blum_kv* kv, int layer, const void* qkv, int dtype, int q_heads, float theta,
                           const int32_t* seq_ids, const int32_t* ctx_lens, int64_t rows, int nsplit, void* scratch, void* out);

int blum_argmax_pairs(blum_ctx* ctx, const float* logits, int64_t rows, int64_t cols, int index_offset, int32_t* pairs);
int blum_pick_pairs(blum_ctx* ctx, const int32_t* pairs, int nranks, int64_t rows, int32_t* out_idx);

int blum_gemm_ws_reserve(blum_ctx* ctx, size_t bytes);
int blum_bf16_small_supported(int64_t N, int64_t K, int ydt, int64_t M);
int blum_bf16_small_dispatch(blum_ctx* ctx, const void* w, int64_t N, int64_t K, const void* x, void* y, int ydt, int64_t M);
int blum_tc_gemm(blum_ctx* ctx, int wf, const void* wdata, const void* scales, int64_t w_rows, int N, int K, const void* x,
                 int64_t M, void* y, int ydt, const int* group_offsets, int groups, int rows_per_group_hint, int swiglu = 0);

// dispatch helpers -----------------------------------------------------------------------------
#define BLUM_DISPATCH_DTYPE(dt, T, ...)                                  \
    do {                                                                 \
        if ((dt) == BLUM_F32) { using T = float; __VA_ARGS__; }          \
        else if ((dt) == BLUM_F16) { using T = __half; __VA_ARGS__; }    \
        else { using T = __nv_bfloat16; __VA_ARGS__; }                   \
    } while (0)
