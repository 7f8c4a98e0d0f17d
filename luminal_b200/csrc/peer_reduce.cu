// Tensor-parallel exchange without a library collective: the sum over ranks of a row-parallel projection, the residual
// add and the RMSNorm that follows it, as ONE kernel that reads every rank's partial product through peer-mapped memory
// (NVLink / NVSwitch, plain loads).
//
// luminal has no distributed code (device 0 is hard-coded: crates/luminal_cuda/src/quantized.rs:247); the unsharded
// computation this replaces is the o_proj / down_proj matmul followed by the residual add of
// examples/llama/src/model.rs:180,186 and the RMSNorm of crates/luminal_nn/src/norm.rs:62-65.
//
// Layout.  Every rank owns one exchange area (cudaMalloc, exported with a CUDA IPC handle and mapped by every peer):
//     slot 0, slot 1   partial products [rows][dim] of the activation type, written by this rank's own projection kernel
//     flags            u32 [max_rows][8]: flags[row][r] = number of exchanges rank r's CTA `row` has entered
//     epochs           u32 [max_rows]:    number of exchanges this rank's CTA `row` has entered
// Protocol (one CTA per row, one-shot "pull"): the CTA counts its call (epoch e), stores e into flags[row][me] of every
// peer with release semantics at system scope, waits until its own flags[row][r] >= e for every peer r (acquire, bounded
// by the global timer: on expiry error bit 0x10000 is raised and the kernel carries on, so the context stays usable), then
// loads the row from every rank in rank order, sums in f32, rounds to the activation type (what an all-reduce would have
// returned), adds the residual row and optionally normalises - the same arithmetic as rmsnorm_kernel with a residual.
// Every rank adds in the same order, so all ranks hold bit-identical results.
// Slot reuse: consecutive exchanges must alternate slots (checked on the host).  A rank enters exchange n+1 only after its
// kernel n has finished reading; a peer leaves exchange n+1 only after seeing that, and only then can its next projection
// overwrite the slot exchange n used.  The kernel is launched without programmatic dependent launch for the same reason.
// No TMA or bulk copy touches peer memory here, and no library kernel is handed a peer pointer.
#include "common.cuh"

#define PR_MAX_RANKS 8
#define PR_THREADS 1024
#define PR_VPT 1          // 16-byte pieces of a row a thread has in flight from every rank at once (registers: 4 per rank and piece)
#define PR_TIMEOUT_NS 1000000000ull     // one second

struct blum_peer {
    int rank = 0, size = 1, max_rows = 0, last_slot = -1;
    int64_t slot_bytes = 0;
    char* local = nullptr;
    char* base[PR_MAX_RANKS] = {};       // base[rank] == local; the others are IPC mappings
    blum_comm* comm = nullptr;
};

struct PeerReduceParams {
    const char* part[PR_MAX_RANKS];      // this exchange's slot on every rank
    uint32_t* flags[PR_MAX_RANKS];       // every rank's flag array
    uint32_t* epochs;                    // local
    const void* x;                       // residual rows (may alias x_out)
    const float* w;                      // norm weight or null
    void* xn;                            // normalised rows or null
    void* x_out;                         // x + sum
    float eps;
    int rank, size;
    int64_t dim;
    int* err;
};

__device__ __forceinline__ uint32_t pr_ld_acquire_sys(const uint32_t* p) {
    uint32_t v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ void pr_st_release_sys(uint32_t* p, uint32_t v) {
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
// peer rows are read with system-scope loads: nothing cached from the slot's previous use may be served
__device__ __forceinline__ int4 pr_ld_sys_v4(const void* p) {
    int4 v;
    asm volatile("ld.relaxed.sys.global.v4.s32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p) : "memory");
    return v;
}

template <typename T>
__global__ void __launch_bounds__(PR_THREADS) peer_reduce_kernel(const PeerReduceParams p) {
    constexpr int N = 16 / (int)sizeof(T);
    __shared__ uint32_t s_epoch;
    __shared__ float red[PR_THREADS / 32];
    __shared__ float rs_sh;
    const int row = blockIdx.x, tid = threadIdx.x;
    if (tid == 0) s_epoch = p.epochs[row] + 1u;
    __syncthreads();
    const uint32_t epoch = s_epoch;
    if (tid < p.size && tid != p.rank) {
        __threadfence_system();
        pr_st_release_sys(p.flags[tid] + (size_t)row * PR_MAX_RANKS + p.rank, epoch);
        const uint32_t* mine = p.flags[p.rank] + (size_t)row * PR_MAX_RANKS + tid;
        const unsigned long long t0 = blum_globaltimer();
        uint32_t spin = 0;
        while ((int32_t)(pr_ld_acquire_sys(mine) - epoch) < 0) {
            if ((++spin & 63u) == 0u && blum_globaltimer() - t0 > PR_TIMEOUT_NS) { atomicOr(p.err, 0x10000); break; }
        }
    }
    __syncthreads();
    if (tid == 0) p.epochs[row] = epoch;

    const size_t row_off = (size_t)row * (size_t)p.dim * sizeof(T);
    const T* xr = reinterpret_cast<const T*>(p.x) + (size_t)row * p.dim;
    T* xo = reinterpret_cast<T*>(p.x_out) + (size_t)row * p.dim;
    float ss = 0.f;
    // every piece of the row costs one NVLink round trip per rank: all of a thread's loads are issued before any is used
    for (int64_t kb = 0; kb < p.dim; kb += (int64_t)PR_THREADS * N * PR_VPT) {
        int4 raw[PR_VPT][PR_MAX_RANKS];
#pragma unroll
        for (int i = 0; i < PR_VPT; i++) {
            const int64_t k = kb + ((int64_t)i * PR_THREADS + tid) * N;
#pragma unroll
            for (int r = 0; r < PR_MAX_RANKS; r++)
                if (r < p.size && k < p.dim) raw[i][r] = pr_ld_sys_v4(p.part[r] + row_off + (size_t)k * sizeof(T));
        }
#pragma unroll
        for (int i = 0; i < PR_VPT; i++) {
            const int64_t k = kb + ((int64_t)i * PR_THREADS + tid) * N;
            if (k >= p.dim) continue;
            float acc[N];
#pragma unroll
            for (int j = 0; j < N; j++) acc[j] = 0.f;
#pragma unroll
            for (int r = 0; r < PR_MAX_RANKS; r++)
                if (r < p.size) {
                    const T* e = reinterpret_cast<const T*>(&raw[i][r]);
#pragma unroll
                    for (int j = 0; j < N; j++) acc[j] += to_f32<T>(e[j]);
                }
            const int4 xraw = *reinterpret_cast<const int4*>(xr + k);
            const T* xe = reinterpret_cast<const T*>(&xraw);
            int4 oraw;
            T* oe = reinterpret_cast<T*>(&oraw);
#pragma unroll
            for (int j = 0; j < N; j++) {
                const float sum_r = to_f32<T>(from_f32<T>(acc[j]));              // the all-reduce result in the activation type
                oe[j] = from_f32<T>(to_f32<T>(xe[j]) + sum_r);
                const float v = to_f32<T>(oe[j]);
                ss += v * v;
            }
            *reinterpret_cast<int4*>(xo + k) = oraw;
        }
    }
    if (!p.xn) return;
    ss = warp_sum(ss);
    if ((tid & 31) == 0) red[tid >> 5] = ss;
    __syncthreads();
    if (tid == 0) {
        float s = 0.f;
        for (int w = 0; w < PR_THREADS / 32; w++) s += red[w];
        rs_sh = rsqrtf(s / (float)p.dim + p.eps);
    }
    __syncthreads();
    const float rs = rs_sh;
    T* yn = reinterpret_cast<T*>(p.xn) + (size_t)row * p.dim;
    for (int64_t k = (int64_t)tid * N; k < p.dim; k += (int64_t)PR_THREADS * N) {
        const int4 raw = *reinterpret_cast<const int4*>(xo + k);             // this thread's own stores
        const T* e = reinterpret_cast<const T*>(&raw);
        int4 oraw;
        T* oe = reinterpret_cast<T*>(&oraw);
#pragma unroll
        for (int j = 0; j < N; j++) oe[j] = from_f32<T>(to_f32<T>(e[j]) * rs * (p.w ? p.w[k + j] : 1.f));
        *reinterpret_cast<int4*>(yn + k) = oraw;
    }
}

static size_t pr_align(size_t v) { return (v + 255) & ~(size_t)255; }
static size_t pr_flags_off(const blum_peer* p) { return 2 * (size_t)p->slot_bytes; }
static size_t pr_epochs_off(const blum_peer* p) { return pr_flags_off(p) + pr_align((size_t)p->max_rows * PR_MAX_RANKS * 4); }
static size_t pr_total(const blum_peer* p) { return pr_epochs_off(p) + pr_align((size_t)p->max_rows * 4); }

static void pr_release(blum_peer* p) {
    for (int r = 0; r < p->size; r++)
        if (r != p->rank && p->base[r]) cudaIpcCloseMemHandle(p->base[r]);
    if (p->local) cudaFree(p->local);
    delete p;
}

extern "C" {

int blum_peer_create(blum_ctx* ctx, blum_comm* comm, int64_t row_bytes, int max_rows, int timeout_ms, blum_peer** out) {
    if (!ctx) return BLUM_ERR_INVALID;
    BLUM_REQUIRE(ctx, comm && out && row_bytes > 0 && row_bytes % 16 == 0 && max_rows > 0, "peer_create: bad argument");
    *out = nullptr;
    const int size = blum_comm_size(comm), rank = blum_comm_rank(comm);
    BLUM_REQUIRE(ctx, size >= 2 && size <= PR_MAX_RANKS, "peer_create: %d ranks (2..%d are supported)", size, PR_MAX_RANKS);
    BLUM_CUDA(ctx, cudaSetDevice(ctx->device));
    blum_peer* p = new blum_peer();
    p->rank = rank; p->size = size; p->max_rows = max_rows; p->comm = comm;
    p->slot_bytes = (int64_t)pr_align((size_t)row_bytes * (size_t)max_rows);
    unsigned char* stage = nullptr;            // [size][64] handles, then [size] status bytes
    const size_t stage_bytes = (size_t)size * (sizeof(cudaIpcMemHandle_t) + 1);
    int rc = BLUM_OK;
    cudaIpcMemHandle_t mine;
    std::vector<unsigned char> host(stage_bytes);
    auto fail = [&](int code, const char* what, cudaError_t e) {
        rc = blum_fail(ctx, code, "peer_create: %s%s%s", what, e == cudaSuccess ? "" : ": ", e == cudaSuccess ? "" : cudaGetErrorString(e));
    };
    cudaError_t e = cudaMalloc((void**)&p->local, pr_total(p));
    if (e == cudaSuccess) e = cudaMalloc((void**)&stage, stage_bytes);
    if (e != cudaSuccess) { fail(BLUM_ERR_OOM, "allocation failed", e); if (stage) cudaFree(stage); pr_release(p); return rc; }
    p->base[rank] = p->local;
    e = cudaMemsetAsync(p->local, 0, pr_total(p), ctx->stream);
    if (e == cudaSuccess) e = cudaIpcGetMemHandle(&mine, p->local);
    if (e == cudaSuccess) e = cudaMemcpyAsync(stage + (size_t)rank * sizeof mine, &mine, sizeof mine, cudaMemcpyHostToDevice, ctx->stream);
    if (e != cudaSuccess) fail(BLUM_ERR_CUDA, "exporting the exchange area failed", e);
    // every rank reaches both all-gathers whatever happened locally, so no rank is left waiting for one that gave up
    unsigned char status = rc == BLUM_OK ? 1 : 0;
    int rc2 = blum_allgather(ctx, comm, stage + (size_t)rank * sizeof mine, stage, (int64_t)sizeof mine, timeout_ms);
    if (rc2 == BLUM_OK && cudaMemcpy(host.data(), stage, (size_t)size * sizeof mine, cudaMemcpyDeviceToHost) != cudaSuccess) rc2 = BLUM_ERR_CUDA;
    if (rc2 != BLUM_OK) { cudaFree(stage); pr_release(p); return rc != BLUM_OK ? rc : rc2; }
    if (status)
        for (int r = 0; r < size && status; r++) {
            if (r == rank) continue;
            cudaIpcMemHandle_t h;
            memcpy(&h, host.data() + (size_t)r * sizeof h, sizeof h);
            void* ptr = nullptr;
            e = cudaIpcOpenMemHandle(&ptr, h, cudaIpcMemLazyEnablePeerAccess);
            if (e != cudaSuccess) { cudaGetLastError(); fail(BLUM_ERR_COMM, "mapping a peer's exchange area failed (one process per GPU with peer access is needed)", e); status = 0; }
            else p->base[r] = (char*)ptr;
        }
    unsigned char* st = stage + (size_t)size * sizeof mine;
    if (cudaMemcpyAsync(st + rank, &status, 1, cudaMemcpyHostToDevice, ctx->stream) != cudaSuccess) status = 0;
    rc2 = blum_allgather(ctx, comm, st + rank, st, 1, timeout_ms);
    if (rc2 == BLUM_OK && cudaMemcpy(host.data(), st, (size_t)size, cudaMemcpyDeviceToHost) != cudaSuccess) rc2 = BLUM_ERR_CUDA;
    cudaFree(stage);
    bool all = rc2 == BLUM_OK && status;
    for (int r = 0; r < size && all; r++) all = host[(size_t)r] == 1;
    if (!all) {
        pr_release(p);
        if (rc != BLUM_OK) return rc;
        if (rc2 != BLUM_OK) return rc2;
        return blum_fail(ctx, BLUM_ERR_COMM, "peer_create: another rank could not map the exchange areas");
    }
    *out = p;
    return BLUM_OK;
}

int blum_peer_destroy(blum_ctx* ctx, blum_peer* p) {
    if (!ctx) return BLUM_ERR_INVALID;
    if (!p) return BLUM_OK;
    cudaStreamSynchronize(ctx->stream);
    // no peer may still be reading this rank's area: meet once more (best effort; an aborted communicator just fails fast)
    unsigned char* d = nullptr;
    if (cudaMalloc((void**)&d, (size_t)p->size) == cudaSuccess) {
        if (blum_allgather(ctx, p->comm, d + p->rank, d, 1, 10000) != BLUM_OK) ctx->err.clear();
        cudaStreamSynchronize(ctx->stream);
        cudaFree(d);
    }
    pr_release(p);
    return BLUM_OK;
}

void* blum_peer_slot(blum_peer* p, int slot) {
    if (!p || slot < 0 || slot > 1) return nullptr;
    return p->local + (size_t)slot * (size_t)p->slot_bytes;
}
int blum_peer_max_rows(const blum_peer* p) { return p ? p->max_rows : 0; }

int blum_allreduce_fused(blum_ctx* ctx, blum_peer* p, int slot, const void* x, const float* norm_w, float eps, void* xn_out,
                         void* x_out, blum_dtype dt, int rows, int64_t dim) {
    if (!ctx) return BLUM_ERR_INVALID;
    BLUM_REQUIRE(ctx, p && x && x_out && rows >= 0 && dim > 0 && (slot == 0 || slot == 1), "allreduce_fused: bad argument");
    const int es = dt == BLUM_F32 ? 4 : 2;
    BLUM_REQUIRE(ctx, (dim * es) % 16 == 0, "allreduce_fused: rows must be multiples of 16 bytes");
    BLUM_REQUIRE(ctx, rows <= p->max_rows && (int64_t)rows * dim * es <= p->slot_bytes, "allreduce_fused: %d rows of %lld exceed the exchange area",
                 rows, (long long)dim);
    if (rows == 0) return BLUM_OK;
    if (slot == p->last_slot) return blum_fail(ctx, BLUM_ERR_STATE, "allreduce_fused: consecutive exchanges must alternate slots (slot %d twice)", slot);
    p->last_slot = slot;
    PeerReduceParams q{};
    for (int r = 0; r < p->size; r++) {
        q.part[r] = p->base[r] + (size_t)slot * (size_t)p->slot_bytes;
        q.flags[r] = reinterpret_cast<uint32_t*>(p->base[r] + pr_flags_off(p));
    }
    q.epochs = reinterpret_cast<uint32_t*>(p->local + pr_epochs_off(p));
    q.x = x; q.w = norm_w; q.xn = xn_out; q.x_out = x_out; q.eps = eps;
    q.rank = p->rank; q.size = p->size; q.dim = dim; q.err = ctx->dev_error;
    BLUM_DISPATCH_DTYPE(dt, T, (peer_reduce_kernel<T><<<(unsigned)rows, PR_THREADS, 0, ctx->stream>>>(q)));
    BLUM_LAUNCH_CHECK(ctx);
    return BLUM_OK;
}

}  // extern "C"
