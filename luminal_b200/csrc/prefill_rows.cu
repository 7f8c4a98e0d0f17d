// Q8_0 matmul for a few rows of f32 activations (a prompt chunk of the f32 configuration) over the stream-packed
// weights of the persistent decode kernel: y[M,N] = x[M,K] * W^T with every weight read once per 8 / 16 / 32 rows.
//
// The reference runs one matvec launch per row of x and re-reads W each time (crates/luminal_cuda/src/quantized.rs:156-164
// in luminal); the f32 GEMV of this library re-reads W once per two rows.  Here the arithmetic is the decode kernel's:
// x becomes block fixed point (three signed byte planes and one power-of-two scale per 32 elements and row), the products
// run as exact integer mma.sync.m16n8k32 (16 weight rows x 8 activation rows per instruction, one instruction per
// plane), and each 32-element block sum is scaled by d_w * 2^e in f32.  The three plane sums of a block are combined
// as (p0 * 65536 + (p1 * 256 + p2)) - the second term in integers - so a block contributes one f32 value, rounded once.
//
//   rows_digitise_kernel   x f32 [M][K] -> planes [tile][chunk][block][plane][TOK][32] int8, scales [tile][chunk][block][TOK]
//   rows_mma_kernel<NT>    persistent CTAs of 16 warps; a step = the 16 units (16 rows x 512 k each) of consecutive
//                          row groups inside one k chunk; every warp streams its unit's 16 operand fragments from global
//                          memory into registers (four fragments ahead, running on into the next step's unit), multiplies
//                          them with the chunk's planes held in shared memory, and the warps of a group add their
//                          partial sums through shared memory in a fixed order into ws [tile][chunk][TOK][N]
//   rows_finish_kernel     y = sum over chunks in order (fixed order: results are reproducible bit for bit), or
//                          swiglu(gate, up) for the interleaved gate/up matrix
// TOK = 8 NT activation rows per tile (NT = 1, 2, 4); the k chunk is 4096 / NT wide at most so that the planes fit
// (98 KB).  Algorithmic bytes: N*K*34/32 per tile pass + the planes once per CTA and chunk from L2.
#include "common.cuh"
#include "decode_stream.cuh"

#define RW_WARPS 16
#define RW_THREADS (RW_WARPS * 32)
#define RW_PREFETCH 4
#define RW_PLANE_BYTES 98304          // uc * 16 blocks * 3 planes * TOK * 32 with uc * NT <= 8

struct RowsParams {
    const unsigned char* packed;      // stream units of this matrix: [group][S][8704]
    int groups, S;                    // 16-row groups, 512-wide units per group
    int uc;                           // units of a group inside one k chunk (1, 2, 4 or 8)
    int nchunks, ntiles;
    const unsigned char* planes;
    const float* xscale;
    float* ws;                        // [tile][chunk][TOK][N]
};

__device__ __forceinline__ int4 rw_ld_stream(const void* p) {
    int4 v;
    asm volatile("ld.global.nc.L1::no_allocate.L2::128B.v4.s32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
    return v;
}

// one thread block per (row of x, 1024 elements): a warp digitises one 32-element block per pass
__global__ void __launch_bounds__(256) rows_digitise_kernel(const float* __restrict__ x, int64_t ldx, int M, int K, int TOK, int uc,
                                                            unsigned char* __restrict__ planes, float* __restrict__ xscale) {
    const int lane = threadIdx.x & 31;
    const int KB = K >> 5, cb = uc * 16;                       // blocks per row, blocks per chunk
    const int ntok = ((M + TOK - 1) / TOK) * TOK;
    const int64_t total = (int64_t)ntok * KB;
    for (int64_t i = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5); i < total; i += (int64_t)gridDim.x * (blockDim.x >> 5)) {
        const int tok = (int)(i / KB), b = (int)(i - (int64_t)tok * KB);
        const float v = tok < M ? x[(int64_t)tok * ldx + (int64_t)b * 32 + lane] : 0.f;
        float mx = fabsf(v);
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
        // the decode kernel's representation: xfix = x * 2^(21 - (E-127)), three balanced base-256 digits
        const int E = (int)((__float_as_uint(mx) >> 23) & 0xffu);
        const float up = (E >= 22 && E < 255) ? __uint_as_float((unsigned)(275 - E) << 23) : 0.f;
        const float down = (E == 255) ? __uint_as_float(0x7fc00000u) : (E >= 22 ? __uint_as_float((unsigned)(E - 21) << 23) : 0.f);
        const int xf = __float2int_rn(v * up);
        const int lo = (int)(signed char)(xf & 0xff);
        const int x1 = (xf - lo) >> 8;
        const int mi = (int)(signed char)(x1 & 0xff);
        const int hi = (x1 - mi) >> 8;
        const int tile = tok / TOK, tt = tok - tile * TOK, chunk = b / cb, lb = b - chunk * cb;
        const int nchunks = KB / cb;
        const size_t cbase = (size_t)tile * nchunks + chunk;
        unsigned char* dst = planes + ((cbase * cb + lb) * 3 * TOK + tt) * 32 + lane;
        dst[0] = (unsigned char)hi;
        dst[(size_t)TOK * 32] = (unsigned char)mi;
        dst[(size_t)TOK * 64] = (unsigned char)lo;
        if (lane == 0) xscale[(cbase * cb + lb) * TOK + tt] = down;
    }
}

template <int NT>
__global__ void __launch_bounds__(RW_THREADS, 1) rows_mma_kernel(const RowsParams p) {
    constexpr int TOK = 8 * NT, PSTRIDE = TOK + 2;             // partial sums: [warp][row][PSTRIDE]
    extern __shared__ __align__(16) unsigned char smem[];
    unsigned char* planes_s = smem;
    float* xsc_s = reinterpret_cast<float*>(smem + RW_PLANE_BYTES);                        // [cb][TOK]
    float* part_s = xsc_s + 128 * TOK / NT;                                                // [2][RW_WARPS][16][PSTRIDE]
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, g = lane >> 2, t = lane & 3;
    const int uc = p.uc, gps = RW_WARPS / uc, cb = uc * 16;
    const int steps_per_chunk = (p.groups + gps - 1) / gps;
    const long long total = (long long)p.ntiles * p.nchunks * steps_per_chunk;
    const long long w0 = total * blockIdx.x / gridDim.x, w1 = total * (blockIdx.x + 1) / gridDim.x;
    if (w0 >= w1) return;
    const int N = p.groups * DS_UNIT_ROWS;
    const int gi = warp / uc, ui = warp - gi * uc;

    auto unit_of = [&](long long w) -> const unsigned char* {
        const int step = (int)(w % steps_per_chunk);
        const int chunk = (int)((w / steps_per_chunk) % p.nchunks);
        const int grp = step * gps + gi;
        if (grp >= p.groups) return nullptr;
        return p.packed + ((size_t)grp * p.S + (size_t)chunk * uc + ui) * DS_UNIT_BYTES;
    };
    const unsigned char* unit = unit_of(w0);
    int4 a[RW_PREFETCH];
#pragma unroll
    for (int i = 0; i < RW_PREFETCH; i++) a[i] = unit ? rw_ld_stream(unit + i * 512 + lane * 16) : make_int4(0, 0, 0, 0);
    uint4 sc[4];                                                 // block scales of rows g and g + 8 of the unit: 16 halves each
    auto load_scales = [&](const unsigned char* u, uint4 (&s)[4]) {
        if (u) {
            s[0] = *reinterpret_cast<const uint4*>(u + 8192 + g * 32);       s[1] = *reinterpret_cast<const uint4*>(u + 8192 + g * 32 + 16);
            s[2] = *reinterpret_cast<const uint4*>(u + 8192 + (g + 8) * 32); s[3] = *reinterpret_cast<const uint4*>(u + 8192 + (g + 8) * 32 + 16);
        }
    };
    load_scales(unit, sc);

    long long staged = -1;                                       // tile * nchunks + chunk whose planes are in shared memory
    int buf = 0;
    for (long long w = w0; w < w1; w++) {
        const int step = (int)(w % steps_per_chunk);
        const long long tc = w / steps_per_chunk;                // tile * nchunks + chunk
        const int chunk = (int)(tc % p.nchunks), tile = (int)(tc / p.nchunks);
        if (tc != staged) {
            __syncthreads();                                     // everybody is done with the previous chunk's planes
            const int4* src = reinterpret_cast<const int4*>(p.planes + (size_t)tc * cb * 3 * TOK * 32);
            int4* dst = reinterpret_cast<int4*>(planes_s);
            for (int i = tid; i < cb * 3 * TOK * 2; i += RW_THREADS) dst[i] = __ldg(src + i);
            for (int i = tid; i < cb * TOK; i += RW_THREADS) xsc_s[i] = __ldg(p.xscale + (size_t)tc * cb * TOK + i);
            staged = tc;
            __syncthreads();
        }
        const unsigned char* next = (w + 1 < w1) ? unit_of(w + 1) : nullptr;
        uint4 scn[4] = {sc[0], sc[1], sc[2], sc[3]};
        float acc[NT][4];
#pragma unroll
        for (int nt = 0; nt < NT; nt++) acc[nt][0] = acc[nt][1] = acc[nt][2] = acc[nt][3] = 0.f;
#pragma unroll
        for (int j = 0; j < DS_UNIT_BLOCKS; j++) {
            const int4 av = a[j % RW_PREFETCH];
            {   // refill: this unit's fragment j + RW_PREFETCH, or the next step's unit running on
                const int jn = j + RW_PREFETCH;
                const unsigned char* srcu = jn < DS_UNIT_BLOCKS ? unit : next;
                if (srcu) a[j % RW_PREFETCH] = rw_ld_stream(srcu + (jn & (DS_UNIT_BLOCKS - 1)) * 512 + lane * 16);
            }
            if (j == 8) load_scales(next, scn);
            if (unit) {
                const int lb = ui * 16 + j;
                const uint32_t wlo = reinterpret_cast<const uint32_t*>(&sc[0])[j >> 1], whi = reinterpret_cast<const uint32_t*>(&sc[2])[j >> 1];
                const float2 dl = __half22float2(*reinterpret_cast<const __half2*>(&wlo));
                const float2 dh = __half22float2(*reinterpret_cast<const __half2*>(&whi));
                const float dlo = (j & 1) ? dl.y : dl.x, dhi = (j & 1) ? dh.y : dh.x;
                const unsigned char* pb = planes_s + (size_t)lb * 3 * TOK * 32 + g * 32 + t * 8;
#pragma unroll
                for (int nt = 0; nt < NT; nt++) {
                    int d[3][4];
#pragma unroll
                    for (int pl = 0; pl < 3; pl++) {
                        const int2 b = *reinterpret_cast<const int2*>(pb + (size_t)(pl * TOK + nt * 8) * 32);
                        asm volatile("mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%10,%10,%10};"
                                     : "=r"(d[pl][0]), "=r"(d[pl][1]), "=r"(d[pl][2]), "=r"(d[pl][3])
                                     : "r"(av.x), "r"(av.y), "r"(av.z), "r"(av.w), "r"(b.x), "r"(b.y), "r"(0));
                    }
                    const float2 xs = *reinterpret_cast<const float2*>(xsc_s + lb * TOK + nt * 8 + 2 * t);
                    const float s00 = dlo * xs.x, s01 = dlo * xs.y, s10 = dhi * xs.x, s11 = dhi * xs.y;
                    acc[nt][0] = fmaf(fmaf((float)d[0][0], 65536.f, (float)(d[1][0] * 256 + d[2][0])), s00, acc[nt][0]);
                    acc[nt][1] = fmaf(fmaf((float)d[0][1], 65536.f, (float)(d[1][1] * 256 + d[2][1])), s01, acc[nt][1]);
                    acc[nt][2] = fmaf(fmaf((float)d[0][2], 65536.f, (float)(d[1][2] * 256 + d[2][2])), s10, acc[nt][2]);
                    acc[nt][3] = fmaf(fmaf((float)d[0][3], 65536.f, (float)(d[1][3] * 256 + d[2][3])), s11, acc[nt][3]);
                }
            }
        }
        // ---- the unit's [16 rows][TOK] partial sums -> shared memory; the group's units are added in unit order
        float* mine = part_s + ((size_t)buf * RW_WARPS + warp) * 16 * PSTRIDE;
#pragma unroll
        for (int nt = 0; nt < NT; nt++) {
            *reinterpret_cast<float2*>(mine + g * PSTRIDE + nt * 8 + 2 * t) = make_float2(acc[nt][0], acc[nt][1]);
            *reinterpret_cast<float2*>(mine + (g + 8) * PSTRIDE + nt * 8 + 2 * t) = make_float2(acc[nt][2], acc[nt][3]);
        }
        __syncthreads();
        float* out = p.ws + ((size_t)tile * p.nchunks + chunk) * TOK * N;
        for (int e = tid; e < gps * 16 * TOK; e += RW_THREADS) {
            const int r = e & 15, gg = (e >> 4) % gps, tok = e / (16 * gps);
            const int grp = step * gps + gg;
            if (grp < p.groups) {
                float v = 0.f;
                for (int u = 0; u < uc; u++) v += part_s[(((size_t)buf * RW_WARPS + gg * uc + u) * 16 + r) * PSTRIDE + tok];
                out[(size_t)tok * N + grp * 16 + r] = v;
            }
        }
        buf ^= 1;                                                // the next step writes the other half: one barrier per step
        unit = next;
        sc[0] = scn[0]; sc[1] = scn[1]; sc[2] = scn[2]; sc[3] = scn[3];
    }
}

// y[m][n] = sum over chunks of ws, in chunk order; swiglu: rows 0-7 of a 16-row group are gate rows, 8-15 the up rows
__global__ void rows_finish_kernel(const float* __restrict__ ws, int M, int TOK, int nchunks, int N, int swiglu, float* __restrict__ y, int64_t ldy) {
    const int NO = swiglu ? N / 2 : N;
    const int64_t total = (int64_t)M * NO;
    for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
        const int m = (int)(i / NO), n = (int)(i - (int64_t)m * NO);
        const int tile = m / TOK, tt = m - tile * TOK;
        const float* base = ws + ((size_t)tile * nchunks * TOK + tt) * N;
        if (!swiglu) {
            float v = 0.f;
            for (int c = 0; c < nchunks; c++) v += base[(size_t)c * TOK * N + n];
            y[(int64_t)m * ldy + n] = v;
        } else {
            const int row = (n >> 3) * 16 + (n & 7);
            float gate = 0.f, up = 0.f;
            for (int c = 0; c < nchunks; c++) { gate += base[(size_t)c * TOK * N + row]; up += base[(size_t)c * TOK * N + row + 8]; }
            y[(int64_t)m * ldy + n] = up * (gate * (1.f / (1.f + __expf(-gate))));
        }
    }
}

// rows per tile and units per chunk for M rows and S units per group; 0 when the shape is not covered
static int rows_pick(int M, int S, int* uc_out) {
    const int NT = M <= 8 ? 1 : M <= 16 ? 2 : 4;
    int uc = 8 / NT;
    while (uc > 1 && S % uc != 0) uc >>= 1;
    *uc_out = uc;
    return NT;
}

size_t blum_rows_scratch_bytes(int M, int64_t K_max, int64_t nk_max) {
    // planes + scales for M rounded up to 32 rows, and the partial sums: nk_max = max over matrices of (K / 512) * N,
    // an upper bound of nchunks * N
    const size_t mp = (size_t)((M + 31) / 32) * 32;
    return mp * (size_t)K_max * 3 + mp * (size_t)(K_max / 32) * 4 + mp * (size_t)nk_max * 4 + 1024;
}

// y [M][ldy] f32 = x [M][ldx] f32 * W^T over the packed units; swiglu: W is the interleaved gate / up matrix and y gets
// N / 2 columns.  scratch: blum_rows_scratch_bytes.  Returns BLUM_ERR_INVALID for shapes it does not cover.
int blum_rows_matmul(blum_ctx* ctx, const unsigned char* packed, int64_t rows_total, int64_t K, const float* x, int64_t ldx, int M,
                     int swiglu, float* y, int64_t ldy, void* scratch, size_t scratch_bytes) {
    BLUM_REQUIRE(ctx, packed && x && y && scratch && M > 0, "rows matmul: bad argument");
    BLUM_REQUIRE(ctx, K % DS_UNIT_K == 0 && rows_total % DS_UNIT_ROWS == 0, "rows matmul: shape is not a multiple of the 16 x 512 unit");
    const int S = (int)(K / DS_UNIT_K), groups = (int)(rows_total / DS_UNIT_ROWS), N = (int)rows_total;
    int uc = 1;
    const int NT = rows_pick(M, S, &uc), TOK = 8 * NT;
    const int nchunks = S / uc, ntiles = (M + TOK - 1) / TOK;
    const size_t mp = (size_t)ntiles * TOK;
    const size_t b_planes = mp * (size_t)K * 3, b_scale = mp * (size_t)(K / 32) * 4, b_ws = (size_t)ntiles * nchunks * TOK * N * 4;
    const size_t o_scale = (b_planes + 255) & ~(size_t)255, o_ws = (o_scale + b_scale + 255) & ~(size_t)255;
    BLUM_REQUIRE(ctx, o_ws + b_ws <= scratch_bytes, "rows matmul: scratch too small (%zu > %zu)", o_ws + b_ws, scratch_bytes);
    unsigned char* planes = (unsigned char*)scratch;
    float* xscale = (float*)((char*)scratch + o_scale);
    float* ws = (float*)((char*)scratch + o_ws);
    rows_digitise_kernel<<<ctx->sm_count * 4, 256, 0, ctx->stream>>>(x, ldx, M, (int)K, TOK, uc, planes, xscale);
    BLUM_LAUNCH_CHECK(ctx);
    RowsParams p;
    p.packed = packed; p.groups = groups; p.S = S; p.uc = uc; p.nchunks = nchunks; p.ntiles = ntiles;
    p.planes = planes; p.xscale = xscale; p.ws = ws;
    const size_t smem = RW_PLANE_BYTES + (size_t)128 * 8 * 4 + (size_t)2 * RW_WARPS * 16 * (TOK + 2) * 4;
    const int gps = RW_WARPS / uc;
    const long long total = (long long)ntiles * nchunks * ((groups + gps - 1) / gps);
    const int grid = (int)std::min<long long>(total, ctx->sm_count);
    static bool attr_set[3] = {};
#define RW_LAUNCH(NTV, IDX)                                                                                                        \
    do {                                                                                                                           \
        if (!attr_set[IDX]) {                                                                                                      \
            BLUM_CUDA(ctx, cudaFuncSetAttribute(rows_mma_kernel<NTV>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)(RW_PLANE_BYTES + 4096 + 2 * RW_WARPS * 16 * 34 * 4))); \
            attr_set[IDX] = true;                                                                                                  \
        }                                                                                                                          \
        rows_mma_kernel<NTV><<<grid, RW_THREADS, smem, ctx->stream>>>(p);                                                          \
    } while (0)
    if (NT == 1) RW_LAUNCH(1, 0); else if (NT == 2) RW_LAUNCH(2, 1); else RW_LAUNCH(4, 2);
#undef RW_LAUNCH
    BLUM_LAUNCH_CHECK(ctx);
    const int NO = swiglu ? N / 2 : N;
    rows_finish_kernel<<<(unsigned)std::min<int64_t>(((int64_t)M * NO + 255) / 256, (int64_t)ctx->sm_count * 8), 256, 0, ctx->stream>>>(
        ws, M, TOK, nchunks, N, swiglu, y, ldy);
    BLUM_LAUNCH_CHECK(ctx);
    return BLUM_OK;
}
