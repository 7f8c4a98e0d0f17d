// Dense bf16 matmul for a few rows of x (the dispatcher sends up to eight; the kernel takes up to sixteen): y[M,N] = x[M,K] * W^T, W bf16 [N,K] (the attention projections, the router
// and the head of the MoE configuration at decode batch sizes).  luminal has no bf16 type; the op restated is its Matmul
// (crates/luminal_cuda/src/matmul.rs:18-111) on a weight that is not quantised.
//
// At these row counts the tcgen05 kernel (q8_gemm_tc.cu) is bound by its per-k-step hand-over chain (15 us for the 24-30 MB
// projections of a 2880-wide model; this kernel 12.8 us at one row, level with it at sixteen).  This is q8_gemm_small.cu without the dequantisation: every warp streams its own weight
// rows from global memory straight into registers, where they already ARE mma.sync A fragments, and multiplies them with B
// fragments of x read from shared memory.
//   * a lane reads 16 bytes (8 bf16) per row and request; a request of a quarter-warp covers 32 consecutive k.  The k order
//     inside a 128-wide super-block is permuted so that a lane's 8 values are its A-fragment elements of two k16 steps:
//     step s = 2 r + t (request r, half t), lane quarter q  <->  k = 32 r + 8 q + 4 t + {0..3};  x is stored in shared
//     memory in the matching order, laid out so that one ldmatrix.x4 yields the B fragments of both 8-row token tiles;
//   * work item of a warp = 32 weight rows x 64 k (two requests per row: 128 bytes per lane in flight while the previous
//     item is multiplied); CTA = (k chunk of 512, block of rows);
//   * K must be a multiple of 32 (a request lies wholly inside or outside the row: 2880 = 22.5 super-blocks is fine);
//   * partial sums over the k chunks are added into an f32 workspace that is cleared before and converted after the launch.
// Algorithmic bytes: N*K*2 + M*K*2 + M*N*sizeof(y); flops 2*M*N*K.
#include "common.cuh"
#include <math.h>

#define BS_WARPS 8
#define BS_THREADS (BS_WARPS * 32)
#define BS_TN 16
#define BS_TASK_ROWS 32
#define BS_KC 512
#define BS_ROWB (BS_KC * 2 + 16)       // bytes of a token's row in the x image (16 past a multiple of 128: no ldmatrix bank conflicts)

struct Bf16SmallParams {
    const __nv_bfloat16* w;   // [N][K]
    const __nv_bfloat16* x;   // [M][K]
    float* ws;                // [M][N] zeroed partial sums
    int N, K, M;
    int rows_per_cta;         // multiple of BS_TASK_ROWS
};

__device__ __forceinline__ uint4 bs_ld_stream_16(const void* p) {
    uint4 r;
    asm volatile("ld.global.nc.L1::no_allocate.L2::128B.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(r.x), "=r"(r.y), "=r"(r.z), "=r"(r.w) : "l"(p));
    return r;
}
__device__ __forceinline__ void bs_mma(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3]) : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void bs_ldsm_x4(uint32_t (&r)[4], uint32_t saddr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(saddr));
}

// grid (k chunks, row blocks); block BS_THREADS; dynamic shared memory BS_TN * BS_ROWB.
__global__ void __launch_bounds__(BS_THREADS, 2) bf16_small_kernel(const Bf16SmallParams p) {
    extern __shared__ __align__(16) unsigned char xs[];
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int hr = lane >> 2, qq = lane & 3;
    const int K = p.K, N = p.N;
    const int k0 = blockIdx.x * BS_KC, kc_len = min(BS_KC, K - k0);
    const int nhalf = (kc_len + 63) >> 6;                           // 64-wide halves of super-blocks in this chunk
    const int cta_row0 = blockIdx.y * p.rows_per_cta;
    const int cta_rows = min(p.rows_per_cta, N - cta_row0);
    const int ntasks = (cta_rows + BS_TASK_ROWS - 1) / BS_TASK_ROWS;
    const uint32_t xs_s = (uint32_t)__cvta_generic_to_shared(xs);

    struct Raw { uint4 w[2][2][2]; };                                // [m tile][row hr / hr + 8][request of the half]
    auto load_unit = [&](int g, int hf, Raw& r) {
        const int row0 = cta_row0 + g * BS_TASK_ROWS;
#pragma unroll
        for (int t = 0; t < 2; t++)
#pragma unroll
            for (int h = 0; h < 2; h++) {
                const __nv_bfloat16* rp = p.w + (size_t)min(row0 + 16 * t + 8 * h + hr, N - 1) * K + k0 + hf * 64 + qq * 8;
#pragma unroll
                for (int rq = 0; rq < 2; rq++) {
                    if (hf * 64 + rq * 32 < kc_len) r.w[t][h][rq] = bs_ld_stream_16(rp + rq * 32);
                    else r.w[t][h][rq] = make_uint4(0u, 0u, 0u, 0u);
                }
            }
    };
    // the CTA's (task, half) units, task-major, are dealt to the warps as contiguous ranges of equal length (+-1)
    Raw cur, nxt;
    const int units = ntasks * nhalf;
    const int u0 = (units * warp) / BS_WARPS, niter = (units * (warp + 1)) / BS_WARPS - u0;
    int g = u0 / nhalf, hf = u0 - g * nhalf;
    if (niter > 0) load_unit(g, hf, cur);

    // ---- x image: 4-byte k pairs; pair (super-block b, request r, quarter q, half t, pair h) -> byte (8 b + 2 r + t) * 32 + 16 h + 4 q
    {
        const int pairs = (((kc_len + 127) >> 7) * 128) >> 1;
        for (int i = tid; i < BS_TN * pairs; i += BS_THREADS) {
            const int n = i / pairs, j = i - n * pairs;
            const int kk = 2 * j, b = kk >> 7, r = (kk >> 5) & 3, q = (kk >> 3) & 3, t = (kk >> 2) & 1, h = (kk >> 1) & 1;
            const uint32_t off = (uint32_t)(n * BS_ROWB + (b * 8 + 2 * r + t) * 32 + h * 16 + q * 4);
            uint32_t v = 0u;
            if (n < p.M && kk < kc_len) v = *reinterpret_cast<const uint32_t*>(p.x + (size_t)n * K + k0 + kk);
            *reinterpret_cast<uint32_t*>(xs + off) = v;
        }
    }
    __syncthreads();

    float acc[2][2][4];
#pragma unroll
    for (int t = 0; t < 2; t++)
#pragma unroll
        for (int nt = 0; nt < 2; nt++) { acc[t][nt][0] = acc[t][nt][1] = acc[t][nt][2] = acc[t][nt][3] = 0.f; }
    // ldmatrix.x4 lane role: matrix = lane / 8 -> (token tile, b0 / b1 half), row = lane % 8
    const uint32_t xlane = xs_s + (uint32_t)((((lane >> 4) & 1) * 8 + (lane & 7)) * BS_ROWB + ((lane >> 3) & 1) * 16);

    for (int it = 0; it < niter; it++) {
        int g2 = g, hf2 = hf + 1;
        if (hf2 == nhalf) { hf2 = 0; g2 = g + 1; }
        const bool last_of_task = hf2 == 0 || it + 1 == niter;
        if (it + 1 < niter) load_unit(g2, hf2, nxt);
#pragma unroll
        for (int rq = 0; rq < 2; rq++)
#pragma unroll
            for (int t2 = 0; t2 < 2; t2++) {
                // step s = 2 * (request within the super-block) + t2; this half holds requests 2 * (hf & 1) + rq
                const int s = 2 * (2 * (hf & 1) + rq) + t2;
                uint32_t b[4];
                bs_ldsm_x4(b, xlane + (uint32_t)(((hf >> 1) * 8 + s) * 32));
#pragma unroll
                for (int t = 0; t < 2; t++) {
                    const uint4 wa = cur.w[t][0][rq], wb = cur.w[t][1][rq];
                    const uint32_t a0 = t2 ? wa.z : wa.x, a2 = t2 ? wa.w : wa.y;       // row hr: pairs (0,1) and (2,3) of this step
                    const uint32_t a1 = t2 ? wb.z : wb.x, a3 = t2 ? wb.w : wb.y;       // row hr + 8
                    bs_mma(acc[t][0], a0, a1, a2, a3, b[0], b[1]);
                    bs_mma(acc[t][1], a0, a1, a2, a3, b[2], b[3]);
                }
            }
        if (last_of_task) {
            const int row0 = cta_row0 + g * BS_TASK_ROWS;
#pragma unroll
            for (int t = 0; t < 2; t++) {
                const int ra = row0 + 16 * t + hr, rb = ra + 8;
#pragma unroll
                for (int nt = 0; nt < 2; nt++) {
                    const int tok = nt * 8 + qq * 2;
                    if (tok < p.M) {
                        if (ra < N) atomicAdd(p.ws + (size_t)tok * N + ra, acc[t][nt][0]);
                        if (rb < N) atomicAdd(p.ws + (size_t)tok * N + rb, acc[t][nt][2]);
                    }
                    if (tok + 1 < p.M) {
                        if (ra < N) atomicAdd(p.ws + (size_t)(tok + 1) * N + ra, acc[t][nt][1]);
                        if (rb < N) atomicAdd(p.ws + (size_t)(tok + 1) * N + rb, acc[t][nt][3]);
                    }
                    acc[t][nt][0] = acc[t][nt][1] = acc[t][nt][2] = acc[t][nt][3] = 0.f;
                }
            }
        }
        cur = nxt;
        g = g2; hf = hf2;
    }
}

__global__ void bf16_small_out_kernel(const float* __restrict__ src, __nv_bfloat16* __restrict__ dst, int64_t n) {
    for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x) dst[i] = __float2bfloat16_rn(src[i]);
}

int blum_bf16_small_supported(int64_t N, int64_t K, int ydt, int64_t M) {
    return M >= 1 && M <= BS_TN && K % 32 == 0 && N >= 1 && N < (1ll << 31) / BS_TN && (ydt == BLUM_BF16 || ydt == BLUM_F32);
}

int blum_bf16_small_dispatch(blum_ctx* ctx, const void* w, int64_t N64, int64_t K64, const void* x, void* y, int ydt, int64_t M) {
    BLUM_REQUIRE(ctx, blum_bf16_small_supported(N64, K64, ydt, M), "bf16 small matmul: unsupported configuration (M <= 16, K %% 32 == 0)");
    const int N = (int)N64, K = (int)K64;
    Bf16SmallParams p;
    p.w = (const __nv_bfloat16*)w; p.x = (const __nv_bfloat16*)x; p.N = N; p.K = K; p.M = (int)M;
    const int nchunks = (K + BS_KC - 1) / BS_KC, total_tasks = (N + BS_TASK_ROWS - 1) / BS_TASK_ROWS;
    // tasks per CTA: about two waves of two CTAs per SM, every warp at least two units (a unit is a task's 64-wide half)
    int tpc = (int)((int64_t)nchunks * total_tasks / (4 * ctx->sm_count)) + 1;
    if (tpc < 2) tpc = 2;
    if (tpc > total_tasks) tpc = total_tasks;
    p.rows_per_cta = tpc * BS_TASK_ROWS;
    const size_t need = (size_t)M * N * sizeof(float);
    float* ws = (float*)y;
    if (ydt != BLUM_F32) {
        const int rc = blum_gemm_ws_reserve(ctx, need);
        if (rc) return rc;
        ws = (float*)ctx->gemm_ws;
    }
    BLUM_CUDA(ctx, cudaMemsetAsync(ws, 0, need, ctx->stream));
    p.ws = ws;
    const dim3 grid(nchunks, (N + p.rows_per_cta - 1) / p.rows_per_cta);
    bf16_small_kernel<<<grid, BS_THREADS, BS_TN * BS_ROWB, ctx->stream>>>(p);
    BLUM_LAUNCH_CHECK(ctx);
    if (ydt != BLUM_F32) {
        bf16_small_out_kernel<<<ctx->sm_count * 2, 256, 0, ctx->stream>>>(ws, (__nv_bfloat16*)y, (int64_t)M * N);
        BLUM_LAUNCH_CHECK(ctx);
    }
    return BLUM_OK;
}
