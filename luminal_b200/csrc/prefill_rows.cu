// Q8_0 matmul for a few rows of f32 activations (prompt chunks and small batches of the f32 configuration) over the
// stream-packed weights of the persistent decode kernel, without converting a single weight:
// y[M,N] = x[M,K] * W^T on the integer tensor path (mma.sync.m16n8k32 s8 x s8 -> s32).
//
// The reference runs one matvec launch per row of x and re-reads W each time (crates/luminal_cuda/src/quantized.rs:156-164
// in luminal); the f32 GEMV of this library re-reads W once per two rows, and the kernels that convert every weight to
// bf16 first (q8_gemm_tc.cu, q8_gemm_small.cu) are bound by that conversion, ~4.4 issued instructions per weight.  Here the
// activations are converted instead - M rows against N of the weights.  x becomes block fixed point: per 32 elements and
// row one power-of-two scale and P signed byte planes, the balanced base-256 digits of x * 2^(8 P - 3 - e); f32 takes P = 3
// (the decode kernel's representation, exact to 2^-22 of the block maximum).  With P = 2 and 16-bit inputs the same kernel was
// measured against the weight-converting kernels and lost (69 against 55 us at 16 rows on 8192 x 28672: the integer MMAs
// and the per-block scaling cost more per row of x than they save per weight), so only f32 is dispatched.  A 32-element
// block of a weight row is one MMA k-step per plane: exact integer block sums, combined over the planes as
// p0 * 65536 + (p1 * 256 + p2) (the bracket in integers), scaled by d_w * 2^e in f32.
//
//   rows_digitise_kernel   x [M][K] -> planes [tile][chunk][block][P][TOK][32] int8, scales [tile][chunk][block][TOK]
//   rows_mma_kernel<NT,P>  persistent CTAs of 16 warps.  A unit (16 rows x 512 k = 8704 contiguous bytes: 16 operand
//                          fragments in MMA register layout + the block scales) arrives in a warp's own shared-memory stage
//                          with one bulk copy completing an mbarrier; the warp re-arms the stage for its next unit as soon
//                          as it has consumed one (16 units = 139 KB in flight per SM, the decode kernel's weight stream).
//                          The CTA holds the planes of one k chunk; a warp multiplies the units of one 16-row group inside
//                          the chunk and stores its [16][TOK] partial sums into ws [tile][chunk][TOK][N]: every element is
//                          written by exactly one warp, no atomics.
//   rows_finish_kernel     y = sum over chunks in chunk order (reproducible bit for bit), or swiglu(gate, up) for the
//                          interleaved gate / up matrix, in the output type
// TOK = 8 NT rows of x per tile (NT = 1, 2, 4); the k chunk is as wide as 64 KB of planes allow.
// Every mbarrier wait is bounded (bit 0x400 of the device error word); a warp waits for a copy it started before it returns.
// Algorithmic bytes: N*K*34/32 per tile pass + the planes once per CTA and chunk from L2.
#include "common.cuh"
#include "attn_mma.cuh"
#include "decode_stream.cuh"

#define RW_WARPS 16
#define RW_THREADS (RW_WARPS * 32)
#define RW_PLANE_BYTES 65536

struct RowsParams {
    const unsigned char* packed;      // stream units of this matrix: [group][S][8704]
    int groups, S;                    // 16-row groups, 512-wide units per group
    int uc;                           // units of a group inside one k chunk
    int nchunks, ntiles, N;
    const unsigned char* planes;
    const float* xscale;
    float* ws;                        // [tile][chunk][TOK][N]
    int* err;
};

// one warp per 32-element block of a row
template <typename T, int P>
__global__ void __launch_bounds__(256) rows_digitise_kernel(const T* __restrict__ x, int64_t ldx, int M, int K, int TOK, int cb,
                                                            unsigned char* __restrict__ planes, float* __restrict__ xscale) {
    const int lane = threadIdx.x & 31;
    const int KB = K >> 5, nchunks = KB / cb;
    const int ntok = ((M + TOK - 1) / TOK) * TOK;
    const int64_t total = (int64_t)ntok * KB;
    constexpr int SH = 8 * P - 3;                              // xfix = x * 2^(SH - (E-127)): the top digit stays within +-64
    for (int64_t i = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5); i < total; i += (int64_t)gridDim.x * (blockDim.x >> 5)) {
        const int tok = (int)(i / KB), b = (int)(i - (int64_t)tok * KB);
        const float v = tok < M ? to_f32<T>(x[(int64_t)tok * ldx + (int64_t)b * 32 + lane]) : 0.f;
        float mx = fabsf(v);
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
        // blocks whose maximum is below 2^(SH+1-127) count as zero; a non-finite block poisons its sums
        const int E = (int)((__float_as_uint(mx) >> 23) & 0xffu);
        const float up = (E >= SH + 1 && E < 255) ? __uint_as_float((unsigned)(254 + SH - E) << 23) : 0.f;
        const float down = (E == 255) ? __uint_as_float(0x7fc00000u) : (E >= SH + 1 ? __uint_as_float((unsigned)(E - SH) << 23) : 0.f);
        int rest = __float2int_rn(v * up);
        int digit[P];
#pragma unroll
        for (int pl = P - 1; pl > 0; pl--) { digit[pl] = (int)(signed char)(rest & 0xff); rest = (rest - digit[pl]) >> 8; }
        digit[0] = rest;
        const int tile = tok / TOK, tt = tok - tile * TOK, chunk = b / cb, lb = b - chunk * cb;
        const size_t cbase = (size_t)tile * nchunks + chunk;
        unsigned char* dst = planes + ((cbase * cb + lb) * P * TOK + tt) * 32 + lane;
#pragma unroll
        for (int pl = 0; pl < P; pl++) dst[(size_t)pl * TOK * 32] = (unsigned char)digit[pl];
        if (lane == 0) xscale[(cbase * cb + lb) * TOK + tt] = down;
    }
}

__device__ __forceinline__ void rw_bulk_load(uint32_t dst_s, const void* src, uint32_t bytes, uint64_t* bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(dst_s), "l"(src), "r"(bytes), "r"(smem_addr(bar)) : "memory");
}

template <int NT, int P>
__global__ void __launch_bounds__(RW_THREADS, 1) rows_mma_kernel(const RowsParams p) {
    constexpr int TOK = 8 * NT;
    extern __shared__ __align__(128) unsigned char smem[];
    unsigned char* ring = smem;                                                        // [RW_WARPS][DS_UNIT_BYTES]
    unsigned char* planes_s = smem + RW_WARPS * DS_UNIT_BYTES;
    float* xsc_s = reinterpret_cast<float*>(planes_s + RW_PLANE_BYTES);                // [cb][TOK]
    __shared__ __align__(8) uint64_t full[RW_WARPS];
    __shared__ int s_abort;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, g = lane >> 2, t = lane & 3;
    const int uc = p.uc, cb = uc * 16;
    // work items (tile, chunk, group), group fastest: a CTA's contiguous range crosses few (tile, chunk) boundaries
    const long long per_tc = p.groups, total = (long long)p.ntiles * p.nchunks * per_tc;
    const long long w0 = total * blockIdx.x / gridDim.x, w1 = total * (blockIdx.x + 1) / gridDim.x;
    if (tid == 0) {
        for (int i = 0; i < RW_WARPS; i++) mbar_init(&full[i], 1);
        s_abort = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    __syncthreads();
    if (w0 >= w1) return;

    // ---- this warp's units in order: inside every (tile, chunk) segment of the CTA's range it takes items warp, warp + 16, ...
    // unit number n of the warp -> (item, unit inside the item); false past the end
    auto unit_at = [&](int n, long long& item, int& ui) -> bool {
        long long lo = w0;
        int base = 0;
        while (lo < w1) {
            const long long seg_end = min(w1, (lo / per_tc + 1) * per_tc);
            const long long cnt = seg_end - lo;                                    // items of the segment
            const int mine = cnt > warp ? (int)((cnt - warp + RW_WARPS - 1) / RW_WARPS) : 0;
            if (n < base + mine * uc) { const int r = (n - base) / uc; ui = (n - base) - r * uc; item = lo + warp + (long long)r * RW_WARPS; return true; }
            base += mine * uc;
            lo = seg_end;
        }
        return false;
    };
    const uint32_t stage_s = smem_addr(ring + (size_t)warp * DS_UNIT_BYTES);
    int req = -1, got = -1;                // lane 0: last unit requested / last unit seen complete
    auto request = [&](int n) {            // lane 0
        long long item; int ui;
        if (!unit_at(n, item, ui)) return;
        req = n;
        const int grp = (int)(item % per_tc), chunk = (int)((item / per_tc) % p.nchunks);
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");               // the stage was last read through the generic proxy
        mbar_expect_tx(&full[warp], DS_UNIT_BYTES);
        rw_bulk_load(stage_s, p.packed + ((size_t)grp * p.S + (size_t)chunk * uc + ui) * DS_UNIT_BYTES, DS_UNIT_BYTES, &full[warp]);
    };
    if (lane == 0) request(0);

    long long staged = -1;
    int n = 0;                             // units this warp has consumed
    for (long long lo = w0; lo < w1;) {
        const long long tc = lo / per_tc, seg_end = min(w1, (tc + 1) * per_tc);
        if (tc != staged) {
            __syncthreads();               // everybody is done with the previous chunk's planes
            const int4* src = reinterpret_cast<const int4*>(p.planes + (size_t)tc * cb * P * TOK * 32);
            int4* dst = reinterpret_cast<int4*>(planes_s);
            for (int i = tid; i < cb * P * TOK * 2; i += RW_THREADS) dst[i] = __ldg(src + i);
            for (int i = tid; i < cb * TOK; i += RW_THREADS) xsc_s[i] = __ldg(p.xscale + (size_t)tc * cb * TOK + i);
            staged = tc;
            __syncthreads();
        }
        float* out = p.ws + (size_t)tc * TOK * p.N;
        for (long long item = lo + warp; item < seg_end; item += RW_WARPS) {
            const int grp = (int)(item % per_tc);
            float acc[NT][4];
#pragma unroll
            for (int nt = 0; nt < NT; nt++) acc[nt][0] = acc[nt][1] = acc[nt][2] = acc[nt][3] = 0.f;
            for (int ui = 0; ui < uc; ui++, n++) {
                bool ok = s_abort == 0 && mbar_wait_bounded(&full[warp], (uint32_t)n & 1u);
                if (ok) got = n;
                else if (lane == 0 && !s_abort) { s_abort = 1; atomicOr(p.err, 0x400); }
                ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
                if (ok) {
                    const unsigned char* st = ring + (size_t)warp * DS_UNIT_BYTES;
                    const __half* dsc = reinterpret_cast<const __half*>(st + 8192);          // block scales [16 rows][16 blocks]
#pragma unroll 4
                    for (int j = 0; j < DS_UNIT_BLOCKS; j++) {
                        const int4 av = *reinterpret_cast<const int4*>(st + j * 512 + lane * 16);
                        const float wlo = __half2float(dsc[g * 16 + j]), whi = __half2float(dsc[(g + 8) * 16 + j]);
                        const int lb = ui * 16 + j;
                        const unsigned char* pb = planes_s + (size_t)lb * P * TOK * 32 + g * 32 + t * 8;
#pragma unroll
                        for (int nt = 0; nt < NT; nt++) {
                            int d[P][4];
#pragma unroll
                            for (int pl = 0; pl < P; pl++) {
                                const int2 b = *reinterpret_cast<const int2*>(pb + (size_t)(pl * TOK + nt * 8) * 32);
                                asm volatile("mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%10,%10,%10};"
                                             : "=r"(d[pl][0]), "=r"(d[pl][1]), "=r"(d[pl][2]), "=r"(d[pl][3])
                                             : "r"(av.x), "r"(av.y), "r"(av.z), "r"(av.w), "r"(b.x), "r"(b.y), "r"(0));
                            }
                            const float2 xs = *reinterpret_cast<const float2*>(xsc_s + lb * TOK + nt * 8 + 2 * t);
                            const float s00 = wlo * xs.x, s01 = wlo * xs.y, s10 = whi * xs.x, s11 = whi * xs.y;
                            float f[4];
#pragma unroll
                            for (int e = 0; e < 4; e++) {
                                if (P == 3) f[e] = fmaf((float)d[0][e], 65536.f, (float)(d[P - 2][e] * 256 + d[P - 1][e]));
                                else f[e] = (float)(d[0][e] * 256 + d[P - 1][e]);
                            }
                            acc[nt][0] = fmaf(f[0], s00, acc[nt][0]);
                            acc[nt][1] = fmaf(f[1], s01, acc[nt][1]);
                            acc[nt][2] = fmaf(f[2], s10, acc[nt][2]);
                            acc[nt][3] = fmaf(f[3], s11, acc[nt][3]);
                        }
                    }
                }
                __syncwarp();                                  // every lane has read the stage
                if (lane == 0 && !s_abort) request(n + 1);
            }
            // ---- the item's [16 rows][TOK] partial sums: this warp is their only writer
            const int ra = grp * 16 + g;
#pragma unroll
            for (int nt = 0; nt < NT; nt++) {
                const int tok = nt * 8 + 2 * t;
                out[(size_t)tok * p.N + ra] = acc[nt][0];
                out[(size_t)(tok + 1) * p.N + ra] = acc[nt][1];
                out[(size_t)tok * p.N + ra + 8] = acc[nt][2];
                out[(size_t)(tok + 1) * p.N + ra + 8] = acc[nt][3];
            }
        }
        lo = seg_end;
    }
    // a copy this warp started and never consumed (only after a wait ran out) has to land before shared memory goes away
    if (lane == 0 && req > got) mbar_wait_bounded(&full[warp], (uint32_t)req & 1u);
}

// y[m][n] = sum over chunks of ws, in chunk order; swiglu: rows 0-7 of a 16-row group are gate rows, 8-15 the up rows
template <typename TY>
__global__ void rows_finish_kernel(const float* __restrict__ ws, int M, int TOK, int nchunks, int N, int swiglu, TY* __restrict__ y, int64_t ldy) {
    const int NO = swiglu ? N / 2 : N;
    const int64_t total = (int64_t)M * NO;
    for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
        const int m = (int)(i / NO), n = (int)(i - (int64_t)m * NO);
        const int tile = m / TOK, tt = m - tile * TOK;
        const float* base = ws + ((size_t)tile * nchunks * TOK + tt) * N;
        if (!swiglu) {
            float v = 0.f;
            for (int c = 0; c < nchunks; c++) v += base[(size_t)c * TOK * N + n];
            y[(int64_t)m * ldy + n] = from_f32<TY>(v);
        } else {
            const int row = (n >> 3) * 16 + (n & 7);
            float gate = 0.f, up = 0.f;
            for (int c = 0; c < nchunks; c++) { gate += base[(size_t)c * TOK * N + row]; up += base[(size_t)c * TOK * N + row + 8]; }
            y[(int64_t)m * ldy + n] = from_f32<TY>(up * (gate * (1.f / (1.f + __expf(-gate)))));
        }
    }
}

static void rows_pick(int M, int S, int P, int* nt_out, int* uc_out) {
    const int NT = M <= 8 ? 1 : M <= 16 ? 2 : 4;
    int uc = 1;
    while (uc * 2 * (8 * NT) * P * DS_UNIT_K <= RW_PLANE_BYTES && S % (uc * 2) == 0) uc *= 2;
    *nt_out = NT; *uc_out = uc;
}

size_t blum_rows_scratch_bytes(int M, int64_t K_max, int64_t nk_max) {
    // planes + scales for M rounded up to 32 rows, and the partial sums: nk_max = max over matrices of (K / 512) * N,
    // an upper bound of nchunks * N
    const size_t mp = (size_t)((M + 31) / 32) * 32;
    return mp * (size_t)K_max * 3 + mp * (size_t)(K_max / 32) * 4 + mp * (size_t)nk_max * 4 + 1024;
}

// y [M][ldy] = x [M][ldx] * W^T over the packed units; x f32 / bf16 / f16, y likewise; swiglu: W is the interleaved gate / up
// matrix and y gets N / 2 columns.  scratch: blum_rows_scratch_bytes.
int blum_rows_matmul(blum_ctx* ctx, const unsigned char* packed, int64_t rows_total, int64_t K, const void* x, int xdt, int64_t ldx, int M,
                     int swiglu, void* y, int ydt, int64_t ldy, void* scratch, size_t scratch_bytes) {
    BLUM_REQUIRE(ctx, packed && x && y && scratch && M > 0, "rows matmul: bad argument");
    BLUM_REQUIRE(ctx, K % DS_UNIT_K == 0 && rows_total % DS_UNIT_ROWS == 0, "rows matmul: shape is not a multiple of the 16 x 512 unit");
    const int S = (int)(K / DS_UNIT_K), groups = (int)(rows_total / DS_UNIT_ROWS), N = (int)rows_total;
    BLUM_REQUIRE(ctx, xdt == BLUM_F32, "rows matmul: f32 activations only");
    constexpr int P = 3;
    int NT = 1, uc = 1;
    rows_pick(M, S, P, &NT, &uc);
    const int TOK = 8 * NT, nchunks = S / uc, ntiles = (M + TOK - 1) / TOK, cb = uc * 16;
    const size_t mp = (size_t)ntiles * TOK;
    const size_t b_planes = mp * (size_t)K * P, b_scale = mp * (size_t)(K / 32) * 4, b_ws = (size_t)ntiles * nchunks * TOK * N * 4;
    const size_t o_scale = (b_planes + 255) & ~(size_t)255, o_ws = (o_scale + b_scale + 255) & ~(size_t)255;
    BLUM_REQUIRE(ctx, o_ws + b_ws <= scratch_bytes, "rows matmul: scratch too small (%zu > %zu)", o_ws + b_ws, scratch_bytes);
    unsigned char* planes = (unsigned char*)scratch;
    float* xscale = (float*)((char*)scratch + o_scale);
    float* ws = (float*)((char*)scratch + o_ws);
    const int dg = ctx->sm_count * 4;
    rows_digitise_kernel<float, 3><<<dg, 256, 0, ctx->stream>>>((const float*)x, ldx, M, (int)K, TOK, cb, planes, xscale);
    BLUM_LAUNCH_CHECK(ctx);
    RowsParams p;
    p.packed = packed; p.groups = groups; p.S = S; p.uc = uc; p.nchunks = nchunks; p.ntiles = ntiles; p.N = N;
    p.planes = planes; p.xscale = xscale; p.ws = ws; p.err = ctx->dev_error;
    const size_t smem = (size_t)RW_WARPS * DS_UNIT_BYTES + RW_PLANE_BYTES + 4096;
    const long long total = (long long)ntiles * nchunks * groups;
    const int grid = (int)std::min<long long>((total + RW_WARPS - 1) / RW_WARPS, ctx->sm_count);
    static bool attr_set[6] = {};
#define RW_LAUNCH(NTV, PV, IDX)                                                                                                     \
    do {                                                                                                                            \
        if (!attr_set[IDX]) {                                                                                                       \
            BLUM_CUDA(ctx, cudaFuncSetAttribute(rows_mma_kernel<NTV, PV>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem)); \
            attr_set[IDX] = true;                                                                                                   \
        }                                                                                                                           \
        rows_mma_kernel<NTV, PV><<<grid, RW_THREADS, smem, ctx->stream>>>(p);                                                       \
    } while (0)
    if (NT == 1) RW_LAUNCH(1, 3, 0); else if (NT == 2) RW_LAUNCH(2, 3, 1); else RW_LAUNCH(4, 3, 2);
#undef RW_LAUNCH
    BLUM_LAUNCH_CHECK(ctx);
    const int NO = swiglu ? N / 2 : N;
    const unsigned fg = (unsigned)std::min<int64_t>(((int64_t)M * NO + 255) / 256, (int64_t)ctx->sm_count * 8);
    if (ydt == BLUM_F32) rows_finish_kernel<float><<<fg, 256, 0, ctx->stream>>>(ws, M, TOK, nchunks, N, swiglu, (float*)y, ldy);
    else if (ydt == BLUM_BF16) rows_finish_kernel<__nv_bfloat16><<<fg, 256, 0, ctx->stream>>>(ws, M, TOK, nchunks, N, swiglu, (__nv_bfloat16*)y, ldy);
    else rows_finish_kernel<__half><<<fg, 256, 0, ctx->stream>>>(ws, M, TOK, nchunks, N, swiglu, (__half*)y, ldy);
    BLUM_LAUNCH_CHECK(ctx);
    return BLUM_OK;
}

// Development aid: average device time of the packed-rows matmul on one matrix (packs `copies` distinct copies so that every
// launch streams from HBM, captures `iters` launches in a CUDA graph and times a replay).
extern "C" int blum_rows_matmul_timed(blum_ctx* ctx, const blum_q8_weight* w, int M, blum_dtype xdt, int copies, int iters, float* avg_us) {
    if (!ctx) return BLUM_ERR_INVALID;
    BLUM_REQUIRE(ctx, w && avg_us && M > 0 && M <= 128 && copies > 0 && iters > 0, "rows_matmul_timed: bad argument");
    const size_t pb = blum_ds_packed_bytes(w->N, w->K);
    const size_t sb = blum_rows_scratch_bytes(M, w->K, (w->K / DS_UNIT_K) * w->N);
    const size_t es = blum_dtype_size(xdt);
    unsigned char* packed = nullptr; void *scratch = nullptr, *x = nullptr, *y = nullptr;
    cudaError_t e = cudaMalloc((void**)&packed, pb * (size_t)copies);
    if (e == cudaSuccess) e = cudaMalloc(&scratch, sb);
    if (e == cudaSuccess) e = cudaMalloc(&x, (size_t)M * w->K * es);
    if (e == cudaSuccess) e = cudaMalloc(&y, (size_t)M * w->N * es);
    int rc = e == cudaSuccess ? BLUM_OK : blum_fail(ctx, BLUM_ERR_OOM, "rows_matmul_timed: %s", cudaGetErrorString(e));
    if (!rc) { cudaMemsetAsync(x, 0, (size_t)M * w->K * es, ctx->stream); }
    for (int c = 0; c < copies && !rc; c++) rc = blum_ds_pack(ctx, w, nullptr, packed + (size_t)c * pb);
    auto run = [&](int c) { return blum_rows_matmul(ctx, packed + (size_t)(c % copies) * pb, w->N, w->K, x, xdt, w->K, M, 0, y, xdt, w->N, scratch, sb); };
    if (!rc) rc = run(0);
    if (!rc && cudaStreamSynchronize(ctx->stream) != cudaSuccess) rc = BLUM_ERR_CUDA;
    cudaGraph_t graph = nullptr; cudaGraphExec_t exec = nullptr;
    if (!rc) {
        const int64_t before = ctx->launches;
        cudaStreamBeginCapture(ctx->stream, cudaStreamCaptureModeThreadLocal);
        for (int i = 0; i < iters && !rc; i++) rc = run(i);
        e = cudaStreamEndCapture(ctx->stream, &graph);
        ctx->launches = before;
        if (!rc && e != cudaSuccess) rc = blum_fail(ctx, BLUM_ERR_CUDA, "rows_matmul_timed: capture: %s", cudaGetErrorString(e));
        if (!rc && cudaGraphInstantiate(&exec, graph, 0) != cudaSuccess) rc = BLUM_ERR_CUDA;
    }
    if (!rc) {
        cudaEvent_t a, b;
        cudaEventCreate(&a); cudaEventCreate(&b);
        cudaGraphLaunch(exec, ctx->stream);
        cudaEventRecord(a, ctx->stream);
        cudaGraphLaunch(exec, ctx->stream);
        cudaEventRecord(b, ctx->stream);
        float ms = 0.f;
        if (cudaEventSynchronize(b) != cudaSuccess) rc = BLUM_ERR_CUDA;
        cudaEventElapsedTime(&ms, a, b);
        cudaEventDestroy(a); cudaEventDestroy(b);
        *avg_us = ms * 1000.f / (float)iters;
    }
    if (exec) cudaGraphExecDestroy(exec);
    if (graph) cudaGraphDestroy(graph);
    cudaStreamSynchronize(ctx->stream);
    if (packed) cudaFree(packed);
    if (scratch) cudaFree(scratch);
    if (x) cudaFree(x);
    if (y) cudaFree(y);
    return rc ? rc : blum_check_device_error(ctx);
}
