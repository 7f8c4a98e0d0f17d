// The experts of an MXFP4 mixture-of-experts layer at small row counts (decode steps: a few rows per expert).
//
// luminal has no MoE; the op being restated is csrc/moe.cu's  mid = (xp Wup^T) * swish(xp Wgate^T),  yp = mid Wdown^T  over
// rows sorted by expert.  With ~10 rows per expert the tcgen05 kernel (q8_gemm_tc.cu, grouped mode) is bound by its per
// k-step hand-over chain: 45 k-steps of ~1000 cycles per CTA whatever the row count.  This kernel has no hand-overs.  Like
// q8_gemm_small.cu, every warp streams its own weight rows from global memory straight into registers, decodes them in
// registers to bf16 A fragments (e2m1 value x 2^e, exact in bf16, the same product the tcgen05 kernel forms) and multiplies
// them with B fragments of the expert's rows of x read from shared memory (mma.sync m16n8k16, f32 accumulate).
//   * work item = (token tile of <= 16 rows of one expert, block of weight rows, k chunk of 512); the tiles that exist are
//     listed on the device from the expert offsets, the grid is sized by their bound (experts + rows / 16);
//   * a lane reads 16 bytes per row and request = the 32 weights of ONE scale block; the k order inside a 128-wide
//     super-block is permuted so that these are exactly the lane's A-fragment elements of eight k16 steps (step s, lane
//     quarter q <-> k = 32 q + 4 s + {0..3}); x is stored in shared memory in the matching order;
//   * byte -> two bf16 values through a table in shared memory replicated per lane (entry i of lane l at word 32 i + l:
//     no bank conflicts whatever the 32 bytes are); the block scale is one bf16x2 multiply per pair;
//   * K need not be a multiple of 128 or 512 (2880 = 22.5 super-blocks): lanes whose quarter lies past K hold zero fragments;
//   * partial sums over the k chunks are added into an f32 workspace.  The second product builds its x image straight from
//     the first one's sums (stacked order: 16 gate rows, then the 16 up rows of the same features), applying the SwiGLU
//     and the bf16 rounding on the way; the combine reads the second product's sums, rounds them to bf16 and adds the
//     token's k choices weighted by their gates.  Per layer: tile list, one memset, two products, combine.
// Algorithmic bytes per product: tiles * N * K * 17/32 from L2 / HBM (experts hit * N * K * 17/32 from HBM) + rows * K * 2.
#include "common.cuh"
#include <math.h>

#define MS_WARPS 8
#define MS_THREADS (MS_WARPS * 32)
#define MS_TN 16            // rows of x per tile (padded)
#define MS_TASK_ROWS 32     // weight rows of a warp task: two m16 tiles
#define MS_KC 512           // k chunk
#define MS_ROWB (MS_KC * 2 + 16)
static_assert(MS_THREADS == 256, "one thread per table entry");

struct MoeSmallParams {
    const uint8_t* q;         // [E*N][K/2] packed e2m1
    const uint8_t* s;         // [E*N][K/32] e8m0
    const __nv_bfloat16* x;   // [rows][K], rows sorted by expert; or null:
    const float* gu;          // [rows][2K] f32 gate/up sums in the stacked order (16 gate, 16 up): x = bf16(up * swish(gate))
    const int* tiles;         // {count, (expert, first row) ...}
    const int* offsets;       // [E+1]
    float* ws;                // [rows][N] zeroed partial sums
    int N, K;
    int rows_per_cta;         // multiple of MS_TASK_ROWS
};

struct MsW128 { uint32_t v[4]; };
__device__ __forceinline__ MsW128 ms_ld_stream_16(const void* p) {
    MsW128 r;
    asm volatile("ld.global.nc.L1::no_allocate.L2::128B.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(r.v[0]), "=r"(r.v[1]), "=r"(r.v[2]), "=r"(r.v[3]) : "l"(p));
    return r;
}
__device__ __forceinline__ void ms_mma(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3]) : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void ms_ldsm_x4(uint32_t (&r)[4], uint32_t saddr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(saddr));
}
__device__ __forceinline__ uint32_t ms_lds(uint32_t saddr) {
    uint32_t v;
    asm volatile("ld.shared.u32 %0, [%1];" : "=r"(v) : "r"(saddr));
    return v;
}
__device__ __forceinline__ float ms_e2m1(int code) {
    const int m = code & 7;
    const float mag = m == 0 ? 0.f : m == 1 ? 0.5f : (float)(2 + (m & 1)) * 0.25f * (float)(1 << (m >> 1));
    return (code & 8) ? -mag : mag;
}

// shared memory: [x image: MS_TN rows of MS_ROWB bytes][table: 256 entries x 32 lanes x 4 bytes][scale slab: rows_per_cta x 16 bytes]
static int ms_smem_bytes(int rows_per_cta) { return MS_TN * MS_ROWB + 256 * 32 * 4 + rows_per_cta * (MS_KC / 32); }

// grid (k chunks, row blocks, tile slots); block MS_THREADS.
__global__ void __launch_bounds__(MS_THREADS, 2) moe_small_kernel(const MoeSmallParams p) {
    extern __shared__ __align__(16) unsigned char xs[];
    if ((int)blockIdx.z >= p.tiles[0]) return;
    const int expert = p.tiles[1 + 2 * blockIdx.z], m0 = p.tiles[2 + 2 * blockIdx.z];
    const int M = min(MS_TN, p.offsets[expert + 1] - m0);            // rows of x in this tile
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int hr = lane >> 2, qq = lane & 3;
    const int K = p.K, N = p.N, KB = K >> 5, KH = K >> 1;
    const int k0 = blockIdx.x * MS_KC, kc_len = min(MS_KC, K - k0), nsb = (kc_len + 127) >> 7;
    const int cta_row0 = blockIdx.y * p.rows_per_cta;
    const int cta_rows = min(p.rows_per_cta, N - cta_row0);
    const int ntasks = (cta_rows + MS_TASK_ROWS - 1) / MS_TASK_ROWS;
    const uint32_t xs_s = (uint32_t)__cvta_generic_to_shared(xs);
    const uint32_t lut_s = xs_s + MS_TN * MS_ROWB;
    const uint32_t slab_s = lut_s + 256 * 32 * 4;
    const size_t wrow0 = (size_t)expert * N;                          // the expert's first row in the stacked tensor

    struct Raw { MsW128 w[2][2]; };                                   // [m tile][row hr / hr + 8]: one scale block each
    // N is a multiple of 32: every row of a task exists, the four rows of a lane are 8 rows apart
    const uint8_t* qbase = p.q + (wrow0 + (size_t)(cta_row0 + hr)) * KH + (k0 >> 1) + qq * 16;
    const size_t row8 = (size_t)8 * KH;
    auto load_block = [&](int g, int sb, Raw& r) {
        const bool live = sb * 128 + qq * 32 < kc_len;               // this lane's quarter of the super-block lies inside K
        const uint8_t* q0 = qbase + (size_t)g * (MS_TASK_ROWS * (size_t)KH) + sb * 64;
#pragma unroll
        for (int t = 0; t < 2; t++)
#pragma unroll
            for (int h = 0; h < 2; h++) {
                if (live) r.w[t][h] = ms_ld_stream_16(q0 + (2 * t + h) * row8);
                else r.w[t][h].v[0] = r.w[t][h].v[1] = r.w[t][h].v[2] = r.w[t][h].v[3] = 0u;      // code 0 = +0.0
            }
    };
    // The CTA's (task, super-block) units, task-major, are dealt to the warps as contiguous ranges of equal length (+-1).
    // A warp keeps the next two units in flight while it multiplies the current one.
    Raw cur, nx1, nx2;
    const int units = ntasks * nsb;
    const int u0 = (units * warp) / MS_WARPS, niter = (units * (warp + 1)) / MS_WARPS - u0;
    int g = u0 / nsb, sb = u0 - g * nsb;
    auto unit_at = [&](int u, int& gg, int& ss) { gg = u / nsb; ss = u - gg * nsb; };
    if (niter > 0) load_block(g, sb, cur);
    if (niter > 1) { int gg, ss; unit_at(u0 + 1, gg, ss); load_block(gg, ss, nx1); }

    // ---- the table, the x image (4-byte k pairs, zero past K and past the tile's rows) and the scale slab
    {
        // thread b holds entry b (MS_THREADS == 256) and writes it into the 32 lane slots, starting at its own lane so that
        // the stores of a warp fall into 32 different banks
        __nv_bfloat162 v = __floats2bfloat162_rn(ms_e2m1(tid & 15), ms_e2m1(tid >> 4));
        uint32_t* tab = reinterpret_cast<uint32_t*>(xs + MS_TN * MS_ROWB) + tid * 32;
#pragma unroll 8
        for (int j = 0; j < 32; j++) tab[(j + lane) & 31] = *reinterpret_cast<uint32_t*>(&v);
    }
    {
        const int pairs = (nsb * 128) >> 1;
        for (int i = tid; i < MS_TN * pairs; i += MS_THREADS) {
            const int n = i / pairs, j = i - n * pairs;
            const int kk = 2 * j, b = kk >> 7, q = (kk >> 5) & 3, s = (kk >> 2) & 7, h = (kk >> 1) & 1;
            const uint32_t off = (uint32_t)(n * MS_ROWB + (b * 8 + s) * 32 + h * 16 + q * 4);
            uint32_t v = 0u;
            if (n < M && kk < kc_len) {
                if (p.gu) {
                    // features f, f + 1 (f even): gate sums at (f >> 4) * 32 + (f & 15), up sums 16 further
                    const int f = k0 + kk;
                    const float* src = p.gu + (size_t)(m0 + n) * 2 * K + (f >> 4) * 32 + (f & 15);
                    const float2 g = *reinterpret_cast<const float2*>(src), u = *reinterpret_cast<const float2*>(src + 16);
                    __nv_bfloat162 m2 = __floats2bfloat162_rn(u.x * (g.x * (1.f / (1.f + expf(-g.x)))), u.y * (g.y * (1.f / (1.f + expf(-g.y)))));
                    v = *reinterpret_cast<uint32_t*>(&m2);
                } else {
                    v = *reinterpret_cast<const uint32_t*>(p.x + (size_t)(m0 + n) * K + k0 + kk);
                }
            }
            *reinterpret_cast<uint32_t*>(xs + off) = v;
        }
        // scale bytes of the CTA's rows for this chunk: up to 16 per row (fewer in the last chunk), rows past N repeat the last
        const int spr = (kc_len + 31) >> 5;
        for (int i = tid; i < ntasks * MS_TASK_ROWS * 16; i += MS_THREADS) {
            const int r = i >> 4, c = i & 15;
            const int row = min(cta_row0 + r, N - 1);
            xs[MS_TN * MS_ROWB + 256 * 32 * 4 + i] = c < spr ? p.s[(wrow0 + row) * KB + (k0 >> 5) + c] : (uint8_t)0;
        }
    }
    __syncthreads();
    if (niter == 0) return;

    float acc[2][2][4];
#pragma unroll
    for (int t = 0; t < 2; t++)
#pragma unroll
        for (int nt = 0; nt < 2; nt++) { acc[t][nt][0] = acc[t][nt][1] = acc[t][nt][2] = acc[t][nt][3] = 0.f; }
    const uint32_t xlane = xs_s + (uint32_t)((((lane >> 4) & 1) * 8 + (lane & 7)) * MS_ROWB + ((lane >> 3) & 1) * 16);
    const uint32_t lut_lane = lut_s + (uint32_t)lane * 4;
    const uint32_t slane = slab_s + (uint32_t)(hr * 16 + qq);

    for (int it = 0; it < niter; it++) {
        int g2 = g, sb2 = sb + 1;
        if (sb2 == nsb) { sb2 = 0; g2 = g + 1; }
        const bool last_of_task = sb2 == 0 || it + 1 == niter;
        if (it + 2 < niter) { int gg, ss; unit_at(u0 + it + 2, gg, ss); load_block(gg, ss, nx2); }
        __nv_bfloat162 sc[2][2];
#pragma unroll
        for (int t = 0; t < 2; t++)
#pragma unroll
            for (int h = 0; h < 2; h++) {
                uint32_t e8;
                asm volatile("ld.shared.u8 %0, [%1];" : "=r"(e8) : "r"(slane + (uint32_t)((g * MS_TASK_ROWS + 16 * t + 8 * h) * 16 + sb * 4)));
                const uint32_t sbits = (e8 << 7) | (e8 << 23);       // bf16x2 of 2^(e-127)
                sc[t][h] = *reinterpret_cast<const __nv_bfloat162*>(&sbits);
            }
#pragma unroll
        for (int s = 0; s < 8; s++) {
            uint32_t a[2][4];
#pragma unroll
            for (int t = 0; t < 2; t++)
#pragma unroll
                for (int h = 0; h < 2; h++) {
                    // bytes 2s and 2s+1 of the lane's 16: k pairs (0,1) and (2,3) of step s.  One byte extraction (PRMT) and
                    // one multiply-add per table address.
                    const uint32_t wv = cur.w[t][h].v[s >> 1];
                    const uint32_t p01 = ms_lds(__byte_perm(wv, 0u, (s & 1) ? 0x4442u : 0x4440u) * 128u + lut_lane);
                    const uint32_t p23 = ms_lds(__byte_perm(wv, 0u, (s & 1) ? 0x4443u : 0x4441u) * 128u + lut_lane);
                    __nv_bfloat162 v01 = __hmul2(*reinterpret_cast<const __nv_bfloat162*>(&p01), sc[t][h]);
                    __nv_bfloat162 v23 = __hmul2(*reinterpret_cast<const __nv_bfloat162*>(&p23), sc[t][h]);
                    a[t][h] = *reinterpret_cast<uint32_t*>(&v01);         // a0 (row hr) / a1 (row hr + 8)
                    a[t][2 + h] = *reinterpret_cast<uint32_t*>(&v23);     // a2 / a3: the second k half of the step
                }
            uint32_t b[4];
            ms_ldsm_x4(b, xlane + (uint32_t)((sb * 8 + s) * 32));
#pragma unroll
            for (int t = 0; t < 2; t++) {
                ms_mma(acc[t][0], a[t], b[0], b[1]);
                ms_mma(acc[t][1], a[t], b[2], b[3]);
            }
        }
        if (last_of_task) {
            const int row0 = cta_row0 + g * MS_TASK_ROWS;
#pragma unroll
            for (int t = 0; t < 2; t++) {
                const int ra = row0 + 16 * t + hr, rb = ra + 8;
#pragma unroll
                for (int nt = 0; nt < 2; nt++) {
                    const int tok = nt * 8 + qq * 2;
                    if (tok < M) {
                        if (ra < N) atomicAdd(p.ws + (size_t)(m0 + tok) * N + ra, acc[t][nt][0]);
                        if (rb < N) atomicAdd(p.ws + (size_t)(m0 + tok) * N + rb, acc[t][nt][2]);
                    }
                    if (tok + 1 < M) {
                        if (ra < N) atomicAdd(p.ws + (size_t)(m0 + tok + 1) * N + ra, acc[t][nt][1]);
                        if (rb < N) atomicAdd(p.ws + (size_t)(m0 + tok + 1) * N + rb, acc[t][nt][3]);
                    }
                    acc[t][nt][0] = acc[t][nt][1] = acc[t][nt][2] = acc[t][nt][3] = 0.f;
                }
            }
        }
        cur = nx1; nx1 = nx2;
        g = g2; sb = sb2;
    }
}

// token tiles that exist: {count, (expert, first row) ...}, experts in order (one CTA, thread per expert)
__global__ void moe_small_tiles_kernel(const int* __restrict__ offsets, int groups, int* __restrict__ list) {
    __shared__ int cnt[256];
    const int g = threadIdx.x;
    const int rows = g < groups ? offsets[g + 1] - offsets[g] : 0;
    const int mine = (rows + MS_TN - 1) / MS_TN;
    cnt[g] = mine;
    __syncthreads();
    int before = 0;
    for (int i = 0; i < g; i++) before += cnt[i];
    if (g < groups) for (int i = 0; i < mine; i++) { list[1 + 2 * (before + i)] = g; list[2 + 2 * (before + i)] = offsets[g] + i * MS_TN; }
    if (g == 255) list[0] = before + mine;
}

// out[t, :] = sum_j gates[t,j] * bf16(sums[slot_of[t*k+j], :]): the down product is rounded to bf16 as the tensor-core path
// stores it, then combined in f32 in choice order
template <typename TO>
__global__ void moe_small_combine_kernel(const float* __restrict__ sums, const int32_t* __restrict__ slot_of, const float* __restrict__ gates,
                                         int k, int H, TO* __restrict__ out) {
    const int t = blockIdx.x;
    __shared__ float g_s[8];
    __shared__ int slot_s[8];
    if (threadIdx.x < k) { g_s[threadIdx.x] = gates[(size_t)t * k + threadIdx.x]; slot_s[threadIdx.x] = slot_of[(size_t)t * k + threadIdx.x]; }
    __syncthreads();
    for (int h = 2 * threadIdx.x; h < H; h += 2 * blockDim.x) {
        float2 v[8];
#pragma unroll
        for (int j = 0; j < 8; j++) if (j < k) v[j] = *reinterpret_cast<const float2*>(sums + (size_t)slot_s[j] * H + h);
        float a0 = 0.f, a1 = 0.f;
#pragma unroll
        for (int j = 0; j < 8; j++)
            if (j < k) {
                a0 = fmaf(g_s[j], __bfloat162float(__float2bfloat16_rn(v[j].x)), a0);
                a1 = fmaf(g_s[j], __bfloat162float(__float2bfloat16_rn(v[j].y)), a1);
            }
        out[(size_t)t * H + h] = from_f32<TO>(a0);
        out[(size_t)t * H + h + 1] = from_f32<TO>(a1);
    }
}

static int ms_launch(blum_ctx* ctx, const uint8_t* q, const uint8_t* s, int E, int N, int K, const __nv_bfloat16* x, const float* gu,
                     const int* offsets, const int* tiles, int tile_bound, float* ws) {
    MoeSmallParams p;
    p.q = q; p.s = s; p.x = x; p.gu = gu; p.tiles = tiles; p.offsets = offsets; p.ws = ws; p.N = N; p.K = K;
    const int nchunks = (K + MS_KC - 1) / MS_KC, total_tasks = (N + MS_TASK_ROWS - 1) / MS_TASK_ROWS;
    // tasks per CTA: the grid (sized by the tile bound) should be few waves of two CTAs per SM, each long enough to pay
    // for its table, x image and scale slab (about four units of a warp's time)
    int tpc = 2;
    double best = 1e30;
    for (int c = 2; c <= 64; c *= 2) {
        const int cc = c < total_tasks ? c : total_tasks;
        if (ms_smem_bytes(cc * MS_TASK_ROWS) > 100 * 1024) break;
        const int64_t ctas = (int64_t)nchunks * ((total_tasks + cc - 1) / cc) * tile_bound;
        const double units_per_warp = ceil((double)cc * (MS_KC / 128) / MS_WARPS);
        const double cost = ceil((double)ctas / (2.0 * ctx->sm_count)) * (units_per_warp + 4.0);
        if (cost < best) { best = cost; tpc = cc; }
        if (cc == total_tasks) break;
    }
    p.rows_per_cta = tpc * MS_TASK_ROWS;
    const int smem = ms_smem_bytes(p.rows_per_cta);
    BLUM_CUDA(ctx, cudaFuncSetAttribute(moe_small_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 100 * 1024));
    const dim3 grid(nchunks, (N + p.rows_per_cta - 1) / p.rows_per_cta, tile_bound);
    moe_small_kernel<<<grid, MS_THREADS, smem, ctx->stream>>>(p);
    BLUM_LAUNCH_CHECK(ctx);
    return BLUM_OK;
}

extern "C" {

int64_t blum_moe_experts_small_ws_bytes(int E, int64_t n_rows, int64_t inter, int64_t hidden) {
    return (int64_t)(1 + 2 * (E + n_rows / MS_TN + 1)) * 4 + 256 + n_rows * (2 * inter + hidden) * 4 + 256;
}

/* The expert half of the layer for small row counts, from the rows sorted by expert to the combined output:
 * out[t,:] = sum_j gates[t,j] * bf16(Wdown_e(bf16((Wup_e xp[r]) * swish(Wgate_e xp[r])))), r = slot_of[t*k+j], e its expert.
 * w_gate_up is the stacked weight of blum_mxfp4_weight_stack_gate_up; offsets / slot_of come from blum_moe_permute. */
int blum_moe_experts_small(blum_ctx* ctx, const blum_mxfp4_weight* w_gate_up, const blum_mxfp4_weight* w_down, const void* xp_bf16,
                           const int32_t* offsets, int64_t n_rows, const int32_t* slot_of, const float* gates, int64_t T, int k,
                           void* out, blum_dtype out_dtype) {
    if (!ctx) return BLUM_ERR_INVALID;
    BLUM_REQUIRE(ctx, w_gate_up && w_down && xp_bf16 && offsets && slot_of && gates && out, "moe_experts_small: null argument");
    const int E = w_gate_up->E;
    const int64_t I = w_gate_up->N / 2, H = w_down->N;
    BLUM_REQUIRE(ctx, w_down->E == E && E <= 256 && w_gate_up->N % 32 == 0 && w_gate_up->K == H && w_down->K == I,
                 "moe_experts_small: gate/up [E,2I,H] and down [E,H,I] do not fit together");
    BLUM_REQUIRE(ctx, H % 32 == 0 && I % 32 == 0 && n_rows == T * k && n_rows < (1 << 24) && k > 0 && k <= 8,
                 "moe_experts_small: need H, I multiples of 32, k <= 8 and T * k rows");
    BLUM_REQUIRE(ctx, out_dtype == BLUM_F32 || out_dtype == BLUM_BF16, "moe_experts_small: output must be f32 or bf16");
    if (n_rows == 0) return BLUM_OK;
    const int tile_bound = (int)std::min<int64_t>(E + n_rows / MS_TN, n_rows);
    int rc = blum_gemm_ws_reserve(ctx, (size_t)blum_moe_experts_small_ws_bytes(E, n_rows, I, H));
    if (rc) return rc;
    // workspace: [tile list][f32 gate/up sums][f32 down sums]; both sum areas are cleared by one memset
    char* base = (char*)ctx->gemm_ws;
    int* tiles = (int*)base;
    const size_t list_bytes = (((size_t)(1 + 2 * (E + n_rows / MS_TN + 1)) * 4) + 255) & ~(size_t)255;
    float* ws1 = (float*)(base + list_bytes);
    float* ws2 = ws1 + (size_t)n_rows * 2 * I;
    moe_small_tiles_kernel<<<1, 256, 0, ctx->stream>>>(offsets, E, tiles);
    BLUM_LAUNCH_CHECK(ctx);
    BLUM_CUDA(ctx, cudaMemsetAsync(ws1, 0, (size_t)n_rows * (2 * I + H) * 4, ctx->stream));
    rc = ms_launch(ctx, w_gate_up->q, w_gate_up->s, E, (int)(2 * I), (int)H, (const __nv_bfloat16*)xp_bf16, nullptr, offsets, tiles, tile_bound, ws1);
    if (rc) return rc;
    rc = ms_launch(ctx, w_down->q, w_down->s, E, (int)H, (int)I, nullptr, ws1, offsets, tiles, tile_bound, ws2);
    if (rc) return rc;
    if (out_dtype == BLUM_F32) moe_small_combine_kernel<float><<<(unsigned)T, 256, 0, ctx->stream>>>(ws2, slot_of, gates, k, (int)H, (float*)out);
    else moe_small_combine_kernel<__nv_bfloat16><<<(unsigned)T, 256, 0, ctx->stream>>>(ws2, slot_of, gates, k, (int)H, (__nv_bfloat16*)out);
    BLUM_LAUNCH_CHECK(ctx);
    return BLUM_OK;
}

}  // extern "C"
