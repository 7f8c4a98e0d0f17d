// Tensor-core GEMM (Q8_0, MXFP4 or bf16 weights; dense or grouped by expert) for M >= 3 rows of x: y[M,N] = x[M,K] * W^T on tcgen05 with TMEM accumulators.
//
// The reference has no Q8_0 GEMM on CUDA: QuantizedMatmul launches one matvec per row of x and re-streams W each
// time (crates/luminal_cuda/src/quantized.rs:156-164 in luminal); its Metal backend has a 64x32x32 simdgroup GEMM that
// dequantises to half in threadgroup memory (crates/luminal_metal/src/quantized.rs:36-199).  This is the B200 form:
//
//   * "swap-AB": the 128 weight rows of a CTA tile are the MMA M dimension (TMEM lanes), the TN tokens are the
//     MMA N dimension (TMEM columns).  Small batches (16..256 tokens) then waste no tensor throughput and every
//     weight is dequantised exactly once per token tile.
//   * warp 0: TMA producer - per k-stage (64 k) one box of int8 weights [128 x 64] (linear) and one box of bf16
//     activations [TN x 64] (128-byte swizzle) land in shared memory and complete an mbarrier.
//   * warps 2-17: dequantisers - int8 * f16 block scale -> bf16, written in the canonical K-major 128-byte-swizzled
//     UMMA layout, then fence.proxy.async + arrive.
//   * warp 1: one elected thread issues 4 tcgen05.mma (K=16 each) per stage, accumulating f32 in TMEM;
//     tcgen05.commit frees the stage for the producer and finally signals the epilogue.
//   * epilogue (warps 2-17): tcgen05.ld 32 lanes x 32 columns, convert, store y[m][n] (32 consecutive n per store).
//   * split-K over CTAs (f32 atomics into a zeroed workspace) when there are too few tiles to fill the SMs.
//   What bounds it at small token tiles is the conversion itself: ~4.4 issued instructions per weight and CTA pass
//   (prmt / fma.f32x2 / cvt per four weights plus per-chunk overhead), ~700 cycles per 64-wide k-step whatever the tile.
//   Measured and dropped: a deep ring of raw int8 boxes (16 x 8 KB) beside a three-deep ring of converted tiles - slower
//   (44 against 30 us on 4096 x 14336 at M = 64): the number of k-steps between conversion and MMA matters, not the bytes
//   in flight; pulling later weight boxes into L2 with cp.async.bulk.prefetch.tensor - no change.  An earlier variant with
//   separate rings and dequantiser groups ran 8-13 % faster at M >= 512 but ended in "unspecified launch failure" about
//   once in a few hundred launches; reading it found a missing tcgen05.fence::after_thread_sync after a barrier wait, an
//   activation tile the MMA thread never waited for itself, and a raw slot handed back to TMA without a proxy fence.
//   It is not in the tree.
// Every mbarrier wait is bounded: on expiry the CTA records an error word, stops issuing work and still frees its
// TMEM.  No TMA load here uses cluster multicast.
// Rounding: w = bf16(q*d) (8-bit significand), x bf16, f32 accumulation: ~1e-3 relative on y.  (Both MMA operands
// must have the same element type: an f16 weight operand against bf16 activations is rejected by the hardware as an
// illegal instruction.)
// Algorithmic bytes: N*K*34/32 + M*K*2 + M*N*sizeof(y); flops 2*M*N*K.
#include "common.cuh"
#include <cuda.h>
#include <stdlib.h>

#define GT_BN 128          // weight rows per CTA tile (MMA M)
#define GT_BK 64           // k per stage (one 128-byte swizzle row of bf16)
#define GT_CONV_WARPS 16    // four per scheduler: with two, the conversion chain left the issue slots two-thirds idle
#define GT_THREADS (64 + 32 * GT_CONV_WARPS)   // warp 0 TMA, warp 1 MMA, the rest dequantise, then run the epilogue
#define GT_SPIN_LIMIT (1u << 22)

struct GemmTcParams {
    const void* scales;        // f16 [rows][K/32] (Q8_0) or e8m0 bytes [rows][K/32] (MXFP4); null for bf16 weights
    void* y;                   // [M][N] output, or f32 workspace when splits > 1
    const int* group_offsets;  // grouped mode: device [groups+1] row offsets into x / y; null for a dense product
    const int* tile_list;      // grouped mode, optional: device [1 + 2 * max] = {count, (group, first row) ...}: blockIdx.y indexes
                               // the token tiles that exist instead of (group, tile) pairs that mostly do not
    int N, K, M;
    int ksteps_per_split;      // 64-wide k stages per split
    int ksteps_total;
    int atomic_out;            // 1: atomicAdd f32 into y (split-K)
    int swiglu;                // 1: weight rows alternate 16 gate / 16 up rows of the same 16 features; the epilogue pairs
                               // them and stores silu(gate) * up into y [M][N/2] (no split-K in this mode)
    int* err;
};

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
// Bounded wait: returns false (and raises the CTA's abort flag) if the phase does not complete in time.
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, volatile int* abort_flag) {
    for (uint32_t spin = 0; spin < GT_SPIN_LIMIT; spin++) {
        uint32_t ok;
        asm volatile("{\n\t.reg .pred q;\n\tmbarrier.try_wait.parity.shared::cta.b64 q, [%1], %2;\n\tselp.u32 %0, 1, 0, q;\n\t}"
                     : "=r"(ok) : "r"(smem_u32(bar)), "r"(parity) : "memory");
        if (ok) return true;
        if (*abort_flag) return false;
    }
    *abort_flag = 1;
    return false;
}
// Drain wait of the abort path: no early exit on the abort flag, bounded by the global timer (nanoseconds).
__device__ __forceinline__ bool mbar_wait_until(uint64_t* bar, uint32_t parity, uint64_t deadline_ns) {
    for (;;) {
        uint32_t ok;
        asm volatile("{\n\t.reg .pred q;\n\tmbarrier.try_wait.parity.shared::cta.b64 q, [%1], %2;\n\tselp.u32 %0, 1, 0, q;\n\t}"
                     : "=r"(ok) : "r"(smem_u32(bar)), "r"(parity) : "memory");
        if (ok) return true;
        uint64_t now;
        asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(now));
        if (now > deadline_ns) return false;
    }
}
__device__ __forceinline__ void tma_load_2d(void* dst, const CUtensorMap* map, int x, int y, uint64_t* bar) {
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
                 ::"r"(smem_u32(dst)), "l"(map), "r"(smem_u32(bar)), "r"(x), "r"(y) : "memory");
}
// the same box towards L2 only
__device__ __forceinline__ void tma_prefetch_2d(const CUtensorMap* map, int x, int y) {
    asm volatile("cp.async.bulk.prefetch.tensor.2d.L2.global [%0, {%1, %2}];" ::"l"(map), "r"(x), "r"(y) : "memory");
}
// K-major, 128-byte swizzle, 8-row groups 1024 bytes apart (the canonical layout TMA SWIZZLE_128B produces)
__device__ __forceinline__ uint64_t umma_desc_sw128(uint32_t smem_addr) {
    uint64_t desc = (uint64_t)((smem_addr & 0x3FFFFu) >> 4);
    desc |= (uint64_t)1 << 16;                 // leading byte offset (unused for swizzled K-major), 16-byte units
    desc |= (uint64_t)(1024 >> 4) << 32;       // stride byte offset between 8-row groups
    desc |= (uint64_t)1 << 46;                 // descriptor version (sm_100)
    desc |= (uint64_t)2 << 61;                 // SWIZZLE_128B
    return desc;
}
__device__ __forceinline__ void umma_bf16(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
    asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
                 "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
                 ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void umma_commit(uint64_t* bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t* r) {
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x32.b32 "
                 "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]),
                   "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]),
                   "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]),
                   "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
                 : "r"(taddr) : "memory");
}

// Weight formats the dequantising stage understands.
enum { WF_Q8_0 = 0, WF_MXFP4 = 1, WF_BF16 = 2 };

// KH: 64-wide k halves per pipeline stage.  One stage is one hand-over (barrier wait, MMA issue, commit) whatever it holds, and
// at small token tiles that fixed cost, not the tensor work, sets the pace: two halves per stage halve the hand-overs.
// CPS: CTAs meant to share an SM (the ring gets 1/CPS of the shared memory)
// NA: token tiles (accumulators) per CTA.  Every dequantised weight tile is multiplied against NA token tiles of TN rows, each
// with its own TMEM columns: the conversion work per flop, which is what bounds the kernel at large M, divides by NA.
template <int TN, int WF, int KH = 1, int CPS = 1, int NA = 1> struct GtCfg {
    static constexpr int A_BYTES = GT_BN * GT_BK * 2;       // 16384, bf16 weights in UMMA layout
    static constexpr int X_TILE_BYTES = TN * GT_BK * 2;     // bf16 activations of one token tile
    static constexpr int X_BYTES = NA * X_TILE_BYTES;
    // raw weight staging per stage: int8 [128][64], packed e2m1 nibbles [128][32], or none (bf16 lands in A directly)
    static constexpr int Q_BYTES = WF == WF_Q8_0 ? GT_BN * GT_BK : WF == WF_MXFP4 ? GT_BN * GT_BK / 2 : 0;
    static constexpr int HALF_BYTES = A_BYTES + X_BYTES + Q_BYTES;
    static constexpr int STAGE_BYTES = KH * HALF_BYTES;
    static constexpr int RING_BYTES = (NA > 1 ? 218 : 200) * 1024 / CPS;   // two token tiles: three stages of 72 KB just fit
    static constexpr int STAGES = RING_BYTES / STAGE_BYTES > 8 ? 8 : RING_BYTES / STAGE_BYTES;
    static constexpr int SMEM = STAGES * STAGE_BYTES + 1024;   // + alignment slack
    static constexpr int TMEM_COLS = NA * TN <= 32 ? 32 : NA * TN <= 64 ? 64 : NA * TN <= 128 ? 128 : NA * TN <= 256 ? 256 : 512;
    static constexpr int TX_BYTES = KH * ((WF == WF_BF16 ? A_BYTES : Q_BYTES) + X_BYTES);
};

// e2m1 code (sign, 2-bit exponent, 1-bit mantissa) -> value; codes 0..7 are {0, .5, 1, 1.5, 2, 3, 4, 6}
__device__ __forceinline__ float e2m1_value(int code) {
    const int m = code & 7;
    const float mag = m == 0 ? 0.f : m == 1 ? 0.5f : (float)(2 + (m & 1)) * 0.25f * (float)(1 << (m >> 1));
    return (code & 8) ? -mag : mag;
}

template <int TN, typename TY, int WF, int KH, int CPS, int NA>
__global__ void __launch_bounds__(GT_THREADS, CPS)
tc_gemm_kernel(const __grid_constant__ CUtensorMap wmap, const __grid_constant__ CUtensorMap xmap, const GemmTcParams p) {
    using C = GtCfg<TN, WF, KH, CPS, NA>;
    constexpr int TT = NA * TN;                                  // tokens of a CTA: NA tiles of TN consecutive rows
    static_assert(C::TMEM_COLS <= 512 && (C::TMEM_COLS & (C::TMEM_COLS - 1)) == 0, "tensor memory columns: a power of two up to 512");
    static_assert(C::STAGES >= 2 && CPS * C::TMEM_COLS <= 512, "ring or tensor memory does not fit this many CTAs per SM");
    static_assert(KH == 1 || WF == WF_Q8_0, "two halves per stage are built for Q8_0 weights only");
    extern __shared__ unsigned char smem_raw[];
    unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    __shared__ __align__(8) uint64_t full[8], a_ready[8], empty[8], acc_full, drained;
    __shared__ uint32_t tmem_base_s;
    __shared__ int abort_flag;
    __shared__ uint32_t fp4_lut[WF == WF_MXFP4 ? 256 : 1];   // byte (two nibbles) -> two bf16 values

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int n0 = blockIdx.x * GT_BN;
    // dense: blockIdx.y = token tile, blockIdx.z = k split.  grouped: blockIdx.z = group (expert); its rows of x are
    // [group_offsets[g], group_offsets[g+1]) and its weights are rows [g*N, (g+1)*N) of the stacked weight tensor.
    int m0, m_end, wrow0, ks0, nk;
    if (p.group_offsets) {
        int g = blockIdx.z;
        if (p.tile_list) {
            if ((int)blockIdx.y >= p.tile_list[0]) return;     // whole CTA: nothing allocated yet
            g = p.tile_list[1 + 2 * blockIdx.y];
            m0 = p.tile_list[2 + 2 * blockIdx.y];
        } else {
            m0 = p.group_offsets[g] + blockIdx.y * TT;
        }
        m_end = p.group_offsets[g + 1];
        if (m0 >= m_end) return;                               // whole CTA: nothing allocated yet
        wrow0 = g * p.N;
        ks0 = 0; nk = p.ksteps_total;
    } else {
        m0 = blockIdx.y * TT; m_end = p.M; wrow0 = 0;
        ks0 = blockIdx.z * p.ksteps_per_split;
        nk = min(p.ksteps_total, ks0 + p.ksteps_per_split) - ks0;
    }
    const int KB = p.K >> 5;
    auto a_s = [&](int s, int h = 0) { return smem + (size_t)s * C::STAGE_BYTES + (size_t)h * C::HALF_BYTES; };
    auto x_s = [&](int s, int h = 0) { return smem + (size_t)s * C::STAGE_BYTES + (size_t)h * C::HALF_BYTES + C::A_BYTES; };
    auto q_s = [&](int s, int h = 0) { return smem + (size_t)s * C::STAGE_BYTES + (size_t)h * C::HALF_BYTES + C::A_BYTES + C::X_BYTES; };

    if (threadIdx.x == 0) {
        for (int s = 0; s < C::STAGES; s++) { mbar_init(&full[s], 1); mbar_init(&a_ready[s], GT_CONV_WARPS); mbar_init(&empty[s], 1); }
        mbar_init(&acc_full, 1);
        mbar_init(&drained, 1);
        abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    if (WF == WF_MXFP4 && threadIdx.x >= 64) {
        const int b = threadIdx.x - 64;      // the first 256 dequantiser threads fill the 256-entry table
        if (b < 256) {
            __nv_bfloat162 v = __floats2bfloat162_rn(e2m1_value(b & 15), e2m1_value(b >> 4));
            fp4_lut[b] = *reinterpret_cast<uint32_t*>(&v);
        }
    }
    if (warp == 1) {   // TMEM allocation is a warp-wide operation
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&tmem_base_s)), "r"((uint32_t)C::TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem = tmem_base_s;
    volatile int* abortp = &abort_flag;
    int tma_issued = 0;        // thread 0 only: k-steps whose two copies were started

    if (warp == 0) {
        // ---------------- TMA producer
        if (lane == 0) {
            asm volatile("prefetch.tensormap [%0];" ::"l"(&wmap) : "memory");
            asm volatile("prefetch.tensormap [%0];" ::"l"(&xmap) : "memory");
            for (int it = 0; it < nk; it++) {
                const int s = it % C::STAGES;
                if (NA > 1 && it + 3 < nk) {
                    // Two token tiles leave room for two stages only, so a stage's copy is requested just one MMA ahead and its
                    // latency would be in the loop: the weight box of three steps on is pulled into L2 now (x is shared by
                    // all CTAs of a token tile and is there already).
                    const int kp = (ks0 + it + 3) * KH * GT_BK;
                    tma_prefetch_2d(&wmap, WF == WF_MXFP4 ? kp / 2 : kp, wrow0 + n0);
                }
                if (it >= C::STAGES && !mbar_wait(&empty[s], ((it / C::STAGES) - 1) & 1, abortp)) break;
                mbar_expect_tx(&full[s], C::TX_BYTES);
#pragma unroll
                for (int h = 0; h < KH; h++) {
                    const int k = ((ks0 + it) * KH + h) * GT_BK;
                    if (WF == WF_Q8_0) tma_load_2d(q_s(s, h), &wmap, k, wrow0 + n0, &full[s]);
                    else if (WF == WF_MXFP4) tma_load_2d(q_s(s, h), &wmap, k / 2, wrow0 + n0, &full[s]);     // two weights per byte
                    else tma_load_2d(a_s(s, h), &wmap, k, wrow0 + n0, &full[s]);                              // bf16, 128-byte swizzle
#pragma unroll
                    for (int a = 0; a < NA; a++)        // rows past the end of x arrive as zeros
                        tma_load_2d(x_s(s, h) + a * C::X_TILE_BYTES, &xmap, k, m0 + a * TN, &full[s]);
                }
                tma_issued = it + 1;
            }
        }
    } else if (warp == 1) {
        // ---------------- MMA issuer
        if (lane == 0) {
            const uint32_t idesc = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(TN >> 3) << 17) | ((uint32_t)(GT_BN >> 4) << 24);
            bool ok = true;
            for (int it = 0; it < nk && ok; it++) {
                const int s = it % C::STAGES;
                ok = mbar_wait(&a_ready[s], (it / C::STAGES) & 1, abortp);
                if (!ok) break;
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
#pragma unroll
                for (int h = 0; h < KH; h++) {
                    const uint64_t adesc = umma_desc_sw128(smem_u32(a_s(s, h)));
#pragma unroll
                    for (int a = 0; a < NA; a++) {
                        const uint64_t bdesc = umma_desc_sw128(smem_u32(x_s(s, h) + a * C::X_TILE_BYTES));
#pragma unroll
                        for (int kk = 0; kk < GT_BK / 16; kk++)   // 16 bf16 = 32 bytes = 2 descriptor units along K
                            umma_bf16(tmem + (uint32_t)(a * TN), adesc + 2 * kk, bdesc + 2 * kk, idesc, (it > 0 || h > 0 || kk > 0) ? 1u : 0u);
                    }
                }
                umma_commit(&empty[s]);
            }
            if (ok) umma_commit(&acc_full);
        }
    } else {
        // ---------------- dequantisers, then epilogue
        const int t = threadIdx.x - 64;                         // 0 .. GT_CONV_WARPS*32
        bool ok = true;
        // Block scales come straight from global memory (L2); they are requested two k-steps before use so that
        // their latency is not paid once per stage after the weights have already landed.
        constexpr int CPT = 512 / (GT_CONV_WARPS * 32);         // Q8_0: 16-byte chunks per thread per stage
        auto q8_scale = [&](int it, int h, int i) -> float {
            const int c = t + GT_CONV_WARPS * 32 * i, r = c >> 2, kq = c & 3;
            const int nrow = n0 + r, kb = ((ks0 + it) * KH + h) * 2 + (kq >> 1);
            return (it < nk && nrow < p.N && kb < KB) ? __half2float(__ldg(reinterpret_cast<const __half*>(p.scales) + (size_t)(wrow0 + nrow) * KB + kb)) : 0.f;
        };
        constexpr int FP4_TPR = GT_CONV_WARPS * 32 / GT_BN;      // MXFP4: threads per weight row per stage (32 packed bytes)
        constexpr int FP4_WORDS = 8 / FP4_TPR;                   // 32-bit words (8 weights each) per thread
        auto fp4_scale = [&](int it) -> uint32_t {
            const int nrow = n0 + t / FP4_TPR, kb = (ks0 + it) * 2 + (t % FP4_TPR) / (FP4_TPR / 2);
            return (it < nk && nrow < p.N && kb < KB) ? __ldg(reinterpret_cast<const uint8_t*>(p.scales) + (size_t)(wrow0 + nrow) * KB + kb) : 0u;
        };
        float sc[KH][CPT], sc1[KH][CPT], sc2[KH][CPT];
        uint32_t e8 = 0, e8_1 = 0, e8_2 = 0;
        if (WF == WF_Q8_0) {
#pragma unroll
            for (int h = 0; h < KH; h++)
#pragma unroll
                for (int i = 0; i < CPT; i++) { sc[h][i] = q8_scale(0, h, i); sc1[h][i] = q8_scale(1, h, i); }
        } else if (WF == WF_MXFP4) {
            e8 = fp4_scale(0); e8_1 = fp4_scale(1);
        }
        for (int it = 0; it < nk && ok; it++) {
            const int s = it % C::STAGES;
            if (WF == WF_Q8_0) {
#pragma unroll
                for (int h = 0; h < KH; h++)
#pragma unroll
                    for (int i = 0; i < CPT; i++) sc2[h][i] = q8_scale(it + 2, h, i);
                ok = mbar_wait(&full[s], (it / C::STAGES) & 1, abortp);
                if (!ok) break;
#pragma unroll
                for (int h = 0; h < KH; h++) {
                    const unsigned char* qs = q_s(s, h);
                    unsigned char* as = a_s(s, h);
#pragma unroll
                    for (int i = 0; i < CPT; i++) {
                        const int c = t + GT_CONV_WARPS * 32 * i, r = c >> 2, kq = c & 3;
                        const int4 v = *reinterpret_cast<const int4*>(qs + c * 16);
                        const int w[4] = {v.x, v.y, v.z, v.w};
                        uint32_t o[8];
                        const Q8Scale qs2 = q8_scale_consts(sc[h][i]);
#pragma unroll
                        for (int j = 0; j < 4; j++) q8_dequant4((uint32_t)w[j], qs2, o[2 * j], o[2 * j + 1]);
                        unsigned char* rowp = as + (r >> 3) * 1024 + (r & 7) * 128;
                        const int sw = r & 7;
                        *reinterpret_cast<uint4*>(rowp + (((2 * kq) ^ sw) << 4)) = make_uint4(o[0], o[1], o[2], o[3]);
                        *reinterpret_cast<uint4*>(rowp + (((2 * kq + 1) ^ sw) << 4)) = make_uint4(o[4], o[5], o[6], o[7]);
                    }
                }
#pragma unroll
                for (int h = 0; h < KH; h++)
#pragma unroll
                    for (int i = 0; i < CPT; i++) { sc[h][i] = sc1[h][i]; sc1[h][i] = sc2[h][i]; }
            } else if (WF == WF_MXFP4) {
                // FP4_TPR threads share a row's 32 packed bytes; a 16-byte half of them is one scale block
                const int r = t / FP4_TPR, part = t % FP4_TPR, hf = part / (FP4_TPR / 2), w0 = (part % (FP4_TPR / 2)) * FP4_WORDS;
                e8_2 = fp4_scale(it + 2);
                const uint32_t sbits = (e8 << 7) | (e8 << 23);      // bf16x2 of 2^(e-127): e2m1 * 2^e is exact in bf16
                const __nv_bfloat162 s2 = *reinterpret_cast<const __nv_bfloat162*>(&sbits);
                ok = mbar_wait(&full[s], (it / C::STAGES) & 1, abortp);
                if (!ok) break;
                uint32_t w[FP4_WORDS];
#pragma unroll
                for (int j = 0; j < FP4_WORDS; j++) w[j] = *reinterpret_cast<const uint32_t*>(q_s(s) + r * 32 + hf * 16 + (w0 + j) * 4);
                unsigned char* rowp = a_s(s) + (r >> 3) * 1024 + (r & 7) * 128;
                const int sw = r & 7;
#pragma unroll
                for (int jj = 0; jj < FP4_WORDS; jj++) {          // word j holds weights 8j .. 8j+7 of the block
                    const int j = w0 + jj;
                    uint32_t o[4];
#pragma unroll
                    for (int b = 0; b < 4; b++) {
                        const uint32_t pair = fp4_lut[(w[jj] >> (8 * b)) & 0xffu];
                        __nv_bfloat162 pv = __hmul2(*reinterpret_cast<const __nv_bfloat162*>(&pair), s2);
                        o[b] = *reinterpret_cast<uint32_t*>(&pv);
                    }
                    *reinterpret_cast<uint4*>(rowp + (((hf * 4 + j) ^ sw) << 4)) = make_uint4(o[0], o[1], o[2], o[3]);
                }
                e8 = e8_1; e8_1 = e8_2;
            } else {
                ok = mbar_wait(&full[s], (it / C::STAGES) & 1, abortp);   // bf16 weights are already in place
                if (!ok) break;
            }
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");   // generic-proxy writes -> visible to the tensor core
            __syncwarp();
            if (lane == 0) mbar_arrive(&a_ready[s]);
        }
        if (ok) ok = mbar_wait(&acc_full, 0, abortp);
        if (ok) {
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const int quarter = warp & 3;                       // TMEM lanes 32*quarter .. +31 belong to this warp
            const int n = n0 + quarter * 32 + lane;
            constexpr int WPQ = GT_CONV_WARPS / 4;                  // warps per TMEM lane quarter: they split the columns
            constexpr int COLS_PER = (TT / WPQ < 32) ? 32 : TT / WPQ;
            const int cbeg = ((warp - 2) >> 2) * COLS_PER;
#pragma unroll 1
            for (int c0 = cbeg; c0 < cbeg + COLS_PER && c0 < TT; c0 += 32) {
                uint32_t r[32];
                tmem_ld32(tmem + ((uint32_t)(quarter * 32) << 16) + (uint32_t)c0, r);
                asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
                if (p.swiglu) {
                    // lanes 0-15 hold the gate rows of 16 features, lanes 16-31 the up rows of the same features
                    // (m, and with it every branch around the shuffle, is the same for the whole warp)
                    const int f = ((n0 + quarter * 32) >> 1) + lane, F = p.N >> 1;
#pragma unroll
                    for (int j = 0; j < 32; j++) {
                        const int m = m0 + c0 + j;
                        if (m < m_end) {
                            const float g = __uint_as_float(r[j]);
                            const float u = __shfl_down_sync(0xffffffffu, g, 16);
                            if (lane < 16 && f < F) reinterpret_cast<TY*>(p.y)[(size_t)m * F + f] = from_f32<TY>(u * (g * (1.f / (1.f + expf(-g)))));
                        }
                    }
                } else if (n < p.N) {
#pragma unroll
                    for (int j = 0; j < 32; j++) {
                        const int m = m0 + c0 + j;
                        if (m < m_end) {
                            const float v = __uint_as_float(r[j]);
                            if (p.atomic_out) atomicAdd(reinterpret_cast<float*>(p.y) + (size_t)m * p.N + n, v);
                            else reinterpret_cast<TY*>(p.y)[(size_t)m * p.N + n] = from_f32<TY>(v);
                        }
                    }
                }
            }
        }
    }
    // Every loop above is bounded, so all threads arrive here; from this point nothing new is issued.
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (abort_flag) {
        // A wait ran out.  Shared memory and TMEM may only be released once everything this CTA started has landed:
        // a late complete_tx or tcgen05.commit arrival would otherwise hit the next CTA on this SM.  So the thread that
        // started the copies waits for the full[] phase of each of its last STAGES issues (earlier ones were waited for
        // through empty[]), and the MMA thread commits once more to a barrier of its own, which completes when every MMA
        // it issued (and with it every earlier commit) has.  Both waits are bounded by the global timer.
        uint64_t t0;
        asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t0));
        const uint64_t deadline = t0 + 500000000ull;             // half a second
        bool clean = true;
        if (threadIdx.x == 0) {
            for (int j = max(0, tma_issued - C::STAGES); j < tma_issued; j++)
                clean &= mbar_wait_until(&full[j % C::STAGES], (j / C::STAGES) & 1, deadline);
            atomicOr(p.err, clean ? 0x1000 : 0x1000 | 0x4000);   // 0x4000: gave up waiting for copies in flight
        } else if (threadIdx.x == 32) {
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            umma_commit(&drained);
            clean = mbar_wait_until(&drained, 0, deadline);
            if (!clean) atomicOr(p.err, 0x8000);                 // 0x8000: gave up waiting for tensor-core work in flight
        }
        asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
        __syncthreads();
    }
    if (warp == 1) {
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"((uint32_t)C::TMEM_COLS) : "memory");
    }
}

// ------------------------------------------------------------------ host side
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_tiled_fn() {
    static EncodeTiledFn fn = nullptr;
    if (!fn) {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess && q == cudaDriverEntryPointSuccess)
            fn = (EncodeTiledFn)p;
    }
    return fn;
}

static int make_map_2d(blum_ctx* ctx, CUtensorMap* map, CUtensorMapDataType dt, int esize, const void* base, uint64_t inner,
                       uint64_t outer, uint32_t box_inner, uint32_t box_outer, CUtensorMapSwizzle sw,
                       CUtensorMapL2promotion promo = CU_TENSOR_MAP_L2_PROMOTION_L2_128B) {
    EncodeTiledFn fn = encode_tiled_fn();
    if (!fn) return blum_fail(ctx, BLUM_ERR_CUDA, "cuTensorMapEncodeTiled is not available from this driver");
    const cuuint64_t dims[2] = {inner, outer};
    const cuuint64_t strides[1] = {inner * (uint64_t)esize};
    const cuuint32_t box[2] = {box_inner, box_outer};
    const cuuint32_t estr[2] = {1, 1};
    const CUresult r = fn(map, dt, 2, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, sw,
                          promo, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return blum_fail(ctx, BLUM_ERR_CUDA, "cuTensorMapEncodeTiled failed (%d)", (int)r);
    return BLUM_OK;
}

int blum_tensor_map_2d(blum_ctx* ctx, void* map, int is_bf16, const void* base, uint64_t inner, uint64_t outer, uint32_t box_inner,
                       uint32_t box_outer) {
    return make_map_2d(ctx, reinterpret_cast<CUtensorMap*>(map), is_bf16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2,
                       base, inner, outer, box_inner, box_outer, CU_TENSOR_MAP_SWIZZLE_128B);
}

// token tiles of a grouped product that exist: {count, (group, first row) ...}, groups in order (one CTA, thread per group)
__global__ void group_tiles_kernel(const int* __restrict__ offsets, int groups, int tn, int* __restrict__ list) {
    __shared__ int cnt[256];
    const int g = threadIdx.x;
    const int rows = g < groups ? offsets[g + 1] - offsets[g] : 0;
    const int mine = (rows + tn - 1) / tn;
    cnt[g] = mine;
    __syncthreads();
    int before = 0;
    for (int i = 0; i < g; i++) before += cnt[i];
    if (g < groups) for (int i = 0; i < mine; i++) { list[1 + 2 * (before + i)] = g; list[2 + 2 * (before + i)] = offsets[g] + i * tn; }
    if (g == 255) list[0] = before + mine;
}

__global__ void f32_to_out_kernel(const float* __restrict__ src, void* __restrict__ dst, int64_t n, int dtype) {
    for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x) {
        if (dtype == BLUM_BF16) reinterpret_cast<__nv_bfloat16*>(dst)[i] = __float2bfloat16_rn(src[i]);
        else reinterpret_cast<__half*>(dst)[i] = __float2half_rn(src[i]);
    }
}

template <int TN, typename TY, int WF, int KH = 1, int CPS = 1, int NA = 1>
static int launch_tc(blum_ctx* ctx, const CUtensorMap& wmap, const CUtensorMap& xmap, const GemmTcParams& p, dim3 grid) {
    auto kern = tc_gemm_kernel<TN, TY, WF, KH, CPS, NA>;
    BLUM_CUDA(ctx, cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, GtCfg<TN, WF, KH, CPS, NA>::SMEM));
    kern<<<grid, GT_THREADS, GtCfg<TN, WF, KH, CPS, NA>::SMEM, ctx->stream>>>(wmap, xmap, p);
    BLUM_LAUNCH_CHECK(ctx);
    return BLUM_OK;
}

// Grouped MXFP4 products with token tiles of up to 64 rows run two CTAs per SM (half the ring each): with a few rows per
// expert the k-step chain of one CTA leaves the SM idle most of the time (MoE layer at 64 tokens 421 -> 364 us, at 256
// tokens 791 -> 652 us).  The dense Q8_0 product keeps one CTA with two 64-wide halves per stage (28 us against 38 us
// for the pair on 4096 x 14336 at 64 rows).
template <int WF>
static int launch_tc_pair(blum_ctx* ctx, int TN, bool f32_store, const CUtensorMap& wmap, const CUtensorMap& xmap, const GemmTcParams& p, dim3 grid) {
#define TC2(tn) (f32_store ? launch_tc<tn, float, WF, 1, 2>(ctx, wmap, xmap, p, grid) : launch_tc<tn, __nv_bfloat16, WF, 1, 2>(ctx, wmap, xmap, p, grid))
    return TN == 32 ? TC2(32) : TC2(64);
#undef TC2
}

template <int WF>
static int launch_tc_tn(blum_ctx* ctx, int TN, bool f32_store, const CUtensorMap& wmap, const CUtensorMap& xmap, const GemmTcParams& p, dim3 grid) {
#define TC(tn) (f32_store ? launch_tc<tn, float, WF>(ctx, wmap, xmap, p, grid) : launch_tc<tn, __nv_bfloat16, WF>(ctx, wmap, xmap, p, grid))
    return TN == 32 ? TC(32) : TN == 64 ? TC(64) : TN == 128 ? TC(128) : TC(256);
#undef TC
}

// y[M,N] (or, grouped, y[rows of group g, N]) = x * W^T with W in format `wf`:
//   WF_Q8_0 : wdata int8 [w_rows][K], scales f16 [w_rows][K/32]
//   WF_MXFP4: wdata packed e2m1 [w_rows][K/2] (element 2i in the low nibble of byte i), scales e8m0 [w_rows][K/32]
//   WF_BF16 : wdata bf16 [w_rows][K]
// groups == 0: dense, w_rows == N.  groups > 0: w_rows == groups*N, group_offsets is a device array [groups+1] of row
// offsets into x / y (rows sorted by group).
int blum_tc_gemm(blum_ctx* ctx, int wf, const void* wdata, const void* scales, int64_t w_rows, int N, int K, const void* x,
                 int64_t M, void* y, int ydt, const int* group_offsets, int groups, int rows_per_group_hint, int swiglu) {
    BLUM_REQUIRE(ctx, wdata && x && y, "tc gemm: null argument");
    BLUM_REQUIRE(ctx, !swiglu || (groups > 0 && N % 32 == 0), "tc gemm: the SwiGLU epilogue is built for grouped products with N %% 32 == 0");
    BLUM_REQUIRE(ctx, K % 64 == 0 && N > 0 && M > 0 && M < (1ll << 31), "tc gemm: need K %% 64 == 0 (K=%d), N>0, M>0", K);
    BLUM_REQUIRE(ctx, ydt == BLUM_BF16 || ydt == BLUM_F32, "tc gemm: output must be bf16 or f32");
    BLUM_REQUIRE(ctx, ((uintptr_t)x % 16) == 0 && ((uintptr_t)wdata % 16) == 0, "tc gemm: operands must be 16-byte aligned");
    BLUM_REQUIRE(ctx, encode_tiled_fn() != nullptr, "tc gemm: tensor maps are not available from this driver");
    const int64_t mt = groups > 0 ? (rows_per_group_hint > 0 ? rows_per_group_hint : M) : M;
    int TN = mt <= 32 ? 32 : mt <= 64 ? 64 : mt <= 128 ? 128 : 256;
    // grouped products are bound by the conversion of the weight tiles, which a wider token tile spreads over more rows:
    // skewed expert loads put most rows into a few experts (MoE layer at 1024 tokens: 986 us with 128-row tiles, 911 us with 256)
    if (groups > 0 && TN == 128) TN = 256;
    const int n_tiles = (N + GT_BN - 1) / GT_BN;
    // Dense products with more than one wave of 256-row tiles: a CTA can hold TWO token tiles (one dequantised weight tile
    // feeds both, so the conversion work per flop halves): 2 x 192 rows with three pipeline stages, or 2 x 256 rows with
    // two.  Which one pays depends on how the tiles fill whole waves of the grid; time per k-step of a CTA, measured:
    // 0.73 us for 256 rows, 0.79 us for 2 x 192, 1.23 us for 2 x 256.
    int NA = 1;
    if (groups == 0 && wf != WF_MXFP4 && TN == 256 && (int64_t)n_tiles * ((M + 255) / 256) >= ctx->sm_count) {
        const int tt[3] = {256, 384, 512};
        const double step_us[3] = {0.73, 0.79, 1.23};
        double best = 1e30;
        int pick = 0;
        for (int o = 0; o < 3; o++) {
            const int64_t ctas = (int64_t)n_tiles * ((M + tt[o] - 1) / tt[o]);
            const double cost = (double)((ctas + ctx->sm_count - 1) / ctx->sm_count) * step_us[o];
            if (cost < best) { best = cost; pick = o; }
        }
        if (pick == 1) { TN = 192; NA = 2; }
        else if (pick == 2) NA = 2;
    }
    const bool two_acc = NA == 2;
    const int TT = NA * TN;
    const int m_tiles = (int)((M + TT - 1) / TT);
    // small token tiles of the dense Q8_0 product take two 64-wide halves per stage (half as many hand-overs)
    const bool pair = wf == WF_MXFP4 && groups > 0 && TN <= 64;
    const int KH = (!pair && wf == WF_Q8_0 && groups == 0 && TN <= 64 && K % (2 * GT_BK) == 0) ? 2 : 1;
    const int ksteps = K / (GT_BK * KH);
    int splits = 1;
    if (groups == 0) {
        // split K until the grid covers the SMs, keeping at least 8 stages per split
        while (n_tiles * m_tiles * splits * 2 <= ctx->sm_count && ksteps / (splits * 2) >= 8) splits *= 2;
    }
    const int per_split = (ksteps + splits - 1) / splits;
    splits = (ksteps + per_split - 1) / per_split;

    CUtensorMap wmap, xmap;
    int rc;
    if (wf == WF_Q8_0) rc = make_map_2d(ctx, &wmap, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, wdata, (uint64_t)K, (uint64_t)w_rows, GT_BK, GT_BN, CU_TENSOR_MAP_SWIZZLE_NONE);
    else if (wf == WF_MXFP4) rc = make_map_2d(ctx, &wmap, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, wdata, (uint64_t)K / 2, (uint64_t)w_rows, GT_BK / 2, GT_BN, CU_TENSOR_MAP_SWIZZLE_NONE);
    else rc = make_map_2d(ctx, &wmap, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, wdata, (uint64_t)K, (uint64_t)w_rows, GT_BK, GT_BN, CU_TENSOR_MAP_SWIZZLE_128B);
    if (rc) return rc;
    rc = make_map_2d(ctx, &xmap, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, x, (uint64_t)K, (uint64_t)M, GT_BK, (uint32_t)TN, CU_TENSOR_MAP_SWIZZLE_128B);
    if (rc) return rc;

    GemmTcParams p;
    p.scales = scales; p.N = N; p.K = K; p.M = (int)M;
    p.ksteps_per_split = per_split; p.ksteps_total = ksteps;
    p.err = ctx->dev_error;
    p.atomic_out = splits > 1;
    p.swiglu = swiglu;
    p.group_offsets = groups > 0 ? group_offsets : nullptr;
    p.y = y;
    float* ws = nullptr;
    if (splits > 1) {
        if (ydt == BLUM_F32) ws = (float*)y;
        else {
            const size_t need = (size_t)M * N * sizeof(float);
            const int wrc = blum_gemm_ws_reserve(ctx, need);
            if (wrc) return wrc;
            ws = (float*)ctx->gemm_ws;
        }
        BLUM_CUDA(ctx, cudaMemsetAsync(ws, 0, (size_t)M * N * sizeof(float), ctx->stream));
        p.y = ws;
    }
    dim3 grid(n_tiles, m_tiles, groups > 0 ? groups : splits);
    p.tile_list = nullptr;
    if (groups > 0 && groups <= 256) {
        // every group has at most rows / TN + 1 token tiles: when that bound is well below groups x (tiles of all rows), the
        // tiles that exist are listed on the device and the grid is sized by the bound
        const int64_t bound = groups + M / TN;
        if (bound * 2 < (int64_t)m_tiles * groups) {
            const int wrc = blum_gemm_ws_reserve(ctx, (size_t)(1 + 2 * bound) * sizeof(int));
            if (wrc) return wrc;
            group_tiles_kernel<<<1, 256, 0, ctx->stream>>>(group_offsets, groups, TN, (int*)ctx->gemm_ws);
            BLUM_LAUNCH_CHECK(ctx);
            p.tile_list = (const int*)ctx->gemm_ws;
            grid = dim3(n_tiles, (unsigned)bound, 1);
        }
    }
    const bool f32_store = (ydt == BLUM_F32) || splits > 1;
    if (KH == 2) {
        rc = TN == 32 ? (f32_store ? launch_tc<32, float, WF_Q8_0, 2>(ctx, wmap, xmap, p, grid) : launch_tc<32, __nv_bfloat16, WF_Q8_0, 2>(ctx, wmap, xmap, p, grid))
                      : (f32_store ? launch_tc<64, float, WF_Q8_0, 2>(ctx, wmap, xmap, p, grid) : launch_tc<64, __nv_bfloat16, WF_Q8_0, 2>(ctx, wmap, xmap, p, grid));
    } else if (two_acc) {
#define TC_NA2(tn, W) (f32_store ? launch_tc<tn, float, W, 1, 1, 2>(ctx, wmap, xmap, p, grid) : launch_tc<tn, __nv_bfloat16, W, 1, 1, 2>(ctx, wmap, xmap, p, grid))
        rc = wf == WF_Q8_0 ? (TN == 192 ? TC_NA2(192, WF_Q8_0) : TC_NA2(256, WF_Q8_0)) : (TN == 192 ? TC_NA2(192, WF_BF16) : TC_NA2(256, WF_BF16));
#undef TC_NA2
    } else if (pair)
        rc = launch_tc_pair<WF_MXFP4>(ctx, TN, f32_store, wmap, xmap, p, grid);
    else
    rc = wf == WF_Q8_0 ? launch_tc_tn<WF_Q8_0>(ctx, TN, f32_store, wmap, xmap, p, grid)
       : wf == WF_MXFP4 ? launch_tc_tn<WF_MXFP4>(ctx, TN, f32_store, wmap, xmap, p, grid)
                        : launch_tc_tn<WF_BF16>(ctx, TN, f32_store, wmap, xmap, p, grid);
    if (rc) return rc;
    if (splits > 1 && ydt != BLUM_F32) {
        f32_to_out_kernel<<<ctx->sm_count * 4, 256, 0, ctx->stream>>>(ws, y, (int64_t)M * N, ydt);
        BLUM_LAUNCH_CHECK(ctx);
    }
    return BLUM_OK;
}

// Grows the split-K workspace ahead of time (model objects call this at creation so that captured steps never allocate).
// A workspace that was ever handed to a kernel is never freed while the context lives: captured CUDA graphs (a model's
// decode step, anything recorded between blum_graph_begin/end) keep its address.  An outgrown buffer moves to the context's
// retired list and is released by blum_ctx_destroy.  Growth is refused while the stream is capturing, because cudaMalloc
// would invalidate the capture.
int blum_gemm_ws_reserve(blum_ctx* ctx, size_t bytes) {
    if (ctx->gemm_ws_bytes >= bytes) return BLUM_OK;
    cudaStreamCaptureStatus st = cudaStreamCaptureStatusNone;
    if (cudaStreamIsCapturing(ctx->stream, &st) == cudaSuccess && st != cudaStreamCaptureStatusNone)
        return blum_fail(ctx, BLUM_ERR_STATE, "matmul workspace of %zu bytes requested during stream capture (have %zu): run the "
                         "largest shape once, or create the model, before capturing", bytes, ctx->gemm_ws_bytes);
    void* fresh = nullptr;
    BLUM_CUDA(ctx, cudaMalloc(&fresh, bytes));
    if (ctx->gemm_ws) ctx->retired.push_back(ctx->gemm_ws);
    ctx->gemm_ws = fresh;
    ctx->gemm_ws_bytes = bytes;
    return BLUM_OK;
}

int blum_gemm_tc_supported(const blum_ctx* ctx, const blum_q8_weight* w, int xdt, int ydt, int64_t M) {
    (void)ctx;
    if (!w || xdt != BLUM_BF16) return 0;              // activations must be bf16 (the MMA's B operand comes straight from x)
    if (ydt != BLUM_BF16 && ydt != BLUM_F32) return 0;
    if (w->K % 64 != 0 || M < 1 || M >= (1ll << 31)) return 0;
    return encode_tiled_fn() != nullptr;
}

int blum_gemm_tc_dispatch(blum_ctx* ctx, const blum_q8_weight* w, const void* x, int xdt, void* y, int ydt, int64_t M) {
    BLUM_REQUIRE(ctx, w && x && y, "q8 gemm: null argument");
    BLUM_REQUIRE(ctx, blum_gemm_tc_supported(ctx, w, xdt, ydt, M), "q8 gemm: unsupported configuration (bf16 x, bf16/f32 y, K %% 64 == 0)");
    return blum_tc_gemm(ctx, WF_Q8_0, w->q, w->d, w->N, (int)w->N, (int)w->K, x, M, y, ydt, nullptr, 0, 0);
}

extern "C" {
/* y[M,N] = x[M,K] * W^T with dense bf16 weights W [N,K] on the tensor cores (router and attention projections of the
 * MoE configuration, which are not quantised). */
int blum_bf16_matmul(blum_ctx* ctx, const void* w_bf16, int64_t N, int64_t K, const void* x_bf16, void* y, blum_dtype y_dtype,
                     int64_t M) {
    if (!ctx) return BLUM_ERR_INVALID;
    if (M == 0) return BLUM_OK;
    BLUM_REQUIRE(ctx, w_bf16 && x_bf16 && y, "bf16 matmul: null argument");
    // up to eight rows: the streaming kernel without tensor-memory hand-overs (bf16_small.cu): 5120 x 2880 at one row 12.8 us
    // against 15 us here; from sixteen rows on the two are level and this kernel's wider token tiles win
    if (M <= 8 && ((uintptr_t)w_bf16 % 16) == 0 && ((uintptr_t)x_bf16 % 4) == 0 && blum_bf16_small_supported(N, K, y_dtype, M))
        return blum_bf16_small_dispatch(ctx, w_bf16, N, K, x_bf16, y, y_dtype, M);
    return blum_tc_gemm(ctx, WF_BF16, w_bf16, nullptr, N, (int)N, (int)K, x_bf16, M, y, y_dtype, nullptr, 0, 0);
}
}
