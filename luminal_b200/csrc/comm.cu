// Multi-GPU communication for the tensor-parallel and expert-parallel configurations: NCCL over NVLink / NVSwitch.
//
// luminal has no distributed code at all (device 0 is hard-coded in every compiler: crates/luminal_cuda/src/quantized.rs:247);
// these entry points are additions.  One process per GPU: rank 0 makes a unique id (blum_comm_unique_id), every rank
// receives it out of band (file, store, MPI, ...) and calls blum_comm_init_rank.  All collectives are enqueued on the
// context's stream, so they order with the kernels around them and can be captured in CUDA graphs.
// Failure handling: every NCCL call's status is returned as BLUM_ERR_COMM with NCCL's message; nothing aborts the process.
// Every blocking step takes a timeout: the init (a rank that never joins) and, on request, every collective (a peer that
// never arrives): a host watchdog aborts the communicator and the call returns BLUM_ERR_COMM.
#include "common.cuh"
#include <dlfcn.h>
#include <nccl.h>
#include <string.h>
#include <time.h>

// NCCL is opened lazily with dlopen instead of being a link-time dependency: a process that also hosts PyTorch then
// shares whichever libnccl.so.2 is already loaded instead of pulling a second, different version in.  The table is also
// the seam the failure-path self-test fills with stubs (blum_comm_selftest): no GPU and no second rank are needed to
// show what a failed init, a failed collective or a peer that never arrives turns into.
struct NcclApi {
    ncclResult_t (*GetUniqueId)(ncclUniqueId*);
    ncclResult_t (*CommInitRank)(ncclComm_t*, int, ncclUniqueId, int);
    ncclResult_t (*CommInitRankConfig)(ncclComm_t*, int, ncclUniqueId, int, ncclConfig_t*);   // optional (NCCL >= 2.14)
    ncclResult_t (*CommGetAsyncError)(ncclComm_t, ncclResult_t*);                            // optional
    ncclResult_t (*CommAbort)(ncclComm_t);                                                   // optional
    ncclResult_t (*CommDestroy)(ncclComm_t);
    ncclResult_t (*AllReduce)(const void*, void*, size_t, ncclDataType_t, ncclRedOp_t, ncclComm_t, cudaStream_t);
    ncclResult_t (*AllGather)(const void*, void*, size_t, ncclDataType_t, ncclComm_t, cudaStream_t);
    ncclResult_t (*Send)(const void*, size_t, ncclDataType_t, int, ncclComm_t, cudaStream_t);
    ncclResult_t (*Recv)(void*, size_t, ncclDataType_t, int, ncclComm_t, cudaStream_t);
    ncclResult_t (*GroupStart)();
    ncclResult_t (*GroupEnd)();
    const char* (*GetErrorString)(ncclResult_t);
    bool ok = false;
};
// "has everything enqueued on the stream so far finished?" - CUDA events in production, a stub in the self-test
struct EventApi {
    int (*record)(cudaStream_t, void** ev);   // 0 ok
    int (*query)(void* ev);                   // 0 finished, 1 not yet, -1 error
    void (*destroy)(void* ev);
};
static int ev_record(cudaStream_t s, void** ev) {
    cudaEvent_t e;
    if (cudaEventCreateWithFlags(&e, cudaEventDisableTiming) != cudaSuccess) return -1;
    if (cudaEventRecord(e, s) != cudaSuccess) { cudaEventDestroy(e); return -1; }
    *ev = (void*)e;
    return 0;
}
static int ev_query(void* ev) {
    const cudaError_t e = cudaEventQuery((cudaEvent_t)ev);
    return e == cudaSuccess ? 0 : e == cudaErrorNotReady ? 1 : -1;
}
static void ev_destroy(void* ev) { cudaEventDestroy((cudaEvent_t)ev); }
static EventApi g_events = {ev_record, ev_query, ev_destroy};

static NcclApi g_stub_api;            // filled by the self-test
static bool g_use_stubs = false;

static NcclApi* nccl_api() {
    if (g_use_stubs) return &g_stub_api;
    static NcclApi api;
    static bool tried = false;
    if (!tried) {
        tried = true;
        void* h = dlopen("libnccl.so.2", RTLD_NOW | RTLD_LOCAL);
        if (!h) h = dlopen("libnccl.so", RTLD_NOW | RTLD_LOCAL);
        if (h) {
#define SYM(field, name) *(void**)(&api.field) = dlsym(h, name)
            SYM(GetUniqueId, "ncclGetUniqueId"); SYM(CommInitRank, "ncclCommInitRank"); SYM(CommDestroy, "ncclCommDestroy");
            SYM(CommInitRankConfig, "ncclCommInitRankConfig"); SYM(CommGetAsyncError, "ncclCommGetAsyncError"); SYM(CommAbort, "ncclCommAbort");
            SYM(AllReduce, "ncclAllReduce"); SYM(AllGather, "ncclAllGather"); SYM(Send, "ncclSend"); SYM(Recv, "ncclRecv");
            SYM(GroupStart, "ncclGroupStart"); SYM(GroupEnd, "ncclGroupEnd"); SYM(GetErrorString, "ncclGetErrorString");
#undef SYM
            api.ok = api.GetUniqueId && api.CommInitRank && api.CommDestroy && api.AllReduce && api.AllGather && api.Send &&
                     api.Recv && api.GroupStart && api.GroupEnd && api.GetErrorString;
        }
    }
    return api.ok ? &api : nullptr;
}
#define NCCL_API_OR_FAIL(ctx) NcclApi* nccl = nccl_api(); \
    if (!nccl) return blum_fail((ctx), BLUM_ERR_COMM, "libnccl.so.2 could not be loaded")

struct blum_comm {
    ncclComm_t comm = nullptr;
    int rank = 0, size = 1;
    bool aborted = false;            // a watchdog gave up on this communicator: every later call fails at once
    bool nonblocking = false;        // initialised with blocking = 0: calls may answer ncclInProgress and are then polled
};

#define BLUM_NCCL(ctx, call)                                                                                   \
    do {                                                                                                       \
        ncclResult_t r__ = (call);                                                                             \
        if (r__ != ncclSuccess)                                                                                \
            return blum_fail((ctx), BLUM_ERR_COMM, "%s failed: %s (%s:%d)", #call, nccl->GetErrorString(r__),    \
                             __FILE__, __LINE__);                                                              \
    } while (0)
#define COMM_USABLE(ctx, c, what)                                                                              \
    do {                                                                                                       \
        if ((c)->aborted || !(c)->comm)                                                                        \
            return blum_fail((ctx), BLUM_ERR_COMM, "%s: the communicator was aborted after an earlier timeout or error", what); \
    } while (0)

// A communicator that was initialised without blocking answers ncclInProgress from any call that has not finished its
// host-side work; the call's real status is then read from ncclCommGetAsyncError.  Bounded: a stuck call aborts the
// communicator like the watchdog does.
#define COMM_SETTLE_MS 60000.0
static double now_ms();
static void nap();
static void comm_abort(NcclApi* nccl, blum_comm* c);
static ncclResult_t comm_settle(NcclApi* nccl, blum_comm* c, ncclResult_t r) {
    if (r != ncclInProgress || !c->nonblocking || !nccl->CommGetAsyncError) return r;
    const double t0 = now_ms();
    for (;;) {
        ncclResult_t st = ncclSuccess;
        if (nccl->CommGetAsyncError(c->comm, &st) != ncclSuccess) return ncclInternalError;
        if (st != ncclInProgress) return st;
        const double waited = now_ms() - t0;
        if (waited > COMM_SETTLE_MS) { comm_abort(nccl, c); return ncclInternalError; }
        if (waited > 2.0) nap();          // the usual case settles within microseconds: poll, do not sleep
    }
}
#define BLUM_NCCL_ON(ctx, c, call)                                                                             \
    do {                                                                                                       \
        ncclResult_t r__ = comm_settle(nccl, (c), (call));                                                     \
        if (r__ != ncclSuccess)                                                                                \
            return blum_fail((ctx), BLUM_ERR_COMM, "%s failed: %s (%s:%d)", #call, nccl->GetErrorString(r__),    \
                             __FILE__, __LINE__);                                                              \
    } while (0)

static ncclDataType_t nccl_dtype(int dt) { return dt == BLUM_F32 ? ncclFloat32 : dt == BLUM_F16 ? ncclFloat16 : ncclBfloat16; }

ncclComm_t blum_comm_handle(blum_comm* c) { return c ? c->comm : nullptr; }

static double now_ms() {
    timespec ts;
    clock_gettime(CLOCK_MONOTONIC, &ts);
    return ts.tv_sec * 1e3 + ts.tv_nsec * 1e-6;
}
static void nap() { timespec ts = {0, 200000}; nanosleep(&ts, nullptr); }      // 0.2 ms between polls

static void comm_abort(NcclApi* nccl, blum_comm* c) {
    if (c->comm) { if (nccl->CommAbort) nccl->CommAbort(c->comm); else nccl->CommDestroy(c->comm); }
    c->comm = nullptr;
    c->aborted = true;
}

// Host watchdog of a collective that was just enqueued: with timeout_ms > 0 the call returns only when everything on the
// stream has finished, NCCL has reported an asynchronous error, or the time is up - a peer that never arrives.  In the last
// two cases the communicator is aborted (which ends the stuck kernel, so the stream and the context stay usable) and the
// call reports BLUM_ERR_COMM.  timeout_ms = 0 leaves the collective asynchronous (it may then be captured in a CUDA graph).
static int comm_watch(blum_ctx* ctx, NcclApi* nccl, blum_comm* c, int timeout_ms, const char* what) {
    if (timeout_ms <= 0) return BLUM_OK;
    void* ev = nullptr;
    if (g_events.record(ctx->stream, &ev) != 0) return blum_fail(ctx, BLUM_ERR_CUDA, "%s: could not record the completion event", what);
    const double t0 = now_ms();
    for (;;) {
        const int q = g_events.query(ev);
        if (q == 0) { g_events.destroy(ev); return BLUM_OK; }
        if (q < 0) { g_events.destroy(ev); comm_abort(nccl, c); return blum_fail(ctx, BLUM_ERR_CUDA, "%s: the stream reported an error", what); }
        if (nccl->CommGetAsyncError) {
            ncclResult_t r = ncclSuccess;
            if (nccl->CommGetAsyncError(c->comm, &r) == ncclSuccess && r != ncclSuccess && r != ncclInProgress) {
                g_events.destroy(ev);
                comm_abort(nccl, c);
                return blum_fail(ctx, BLUM_ERR_COMM, "%s: NCCL reported an asynchronous error: %s; communicator aborted", what, nccl->GetErrorString(r));
            }
        }
        if (now_ms() - t0 > (double)timeout_ms) {
            comm_abort(nccl, c);           // ends the kernel that waits for the missing peer; the event then completes
            g_events.destroy(ev);
            return blum_fail(ctx, BLUM_ERR_COMM, "%s did not complete within %d ms (a peer never arrived?); communicator aborted", what, timeout_ms);
        }
        nap();
    }
}

extern "C" {

int blum_comm_unique_id(void* out_128_bytes) {
    if (!out_128_bytes) return BLUM_ERR_INVALID;
    NcclApi* nccl = nccl_api();
    if (!nccl) return BLUM_ERR_COMM;
    ncclUniqueId id;
    if (nccl->GetUniqueId(&id) != ncclSuccess) return BLUM_ERR_COMM;
    static_assert(sizeof(ncclUniqueId) == 128, "ncclUniqueId size");
    memcpy(out_128_bytes, &id, 128);
    return BLUM_OK;
}

int blum_comm_init_rank(blum_ctx* ctx, int nranks, int rank, const void* id_128_bytes, int timeout_ms, blum_comm** out) {
    if (!ctx) return BLUM_ERR_INVALID;
    BLUM_REQUIRE(ctx, out && id_128_bytes && nranks >= 1 && rank >= 0 && rank < nranks, "comm_init_rank: bad argument");
    *out = nullptr;
    NCCL_API_OR_FAIL(ctx);
    if (!g_use_stubs) BLUM_CUDA(ctx, cudaSetDevice(ctx->device));
    ncclUniqueId id;
    memcpy(&id, id_128_bytes, 128);
    blum_comm* c = new blum_comm();
    c->rank = rank; c->size = nranks;
    ncclResult_t r;
    if (timeout_ms > 0 && nccl->CommInitRankConfig && nccl->CommGetAsyncError) {
        // non-blocking init: a rank that never joins must not hold this one for ever
        ncclConfig_t cfg = NCCL_CONFIG_INITIALIZER;
        cfg.blocking = 0;
        c->nonblocking = true;
        r = nccl->CommInitRankConfig(&c->comm, nranks, id, rank, &cfg);
        const double t0 = now_ms();
        while (r == ncclInProgress || (r == ncclSuccess && c->comm)) {
            ncclResult_t st = ncclSuccess;
            if (nccl->CommGetAsyncError(c->comm, &st) != ncclSuccess) { r = ncclInternalError; break; }
            if (st == ncclSuccess) { r = ncclSuccess; break; }
            if (st != ncclInProgress) { r = st; break; }
            if (now_ms() - t0 > (double)timeout_ms) {
                comm_abort(nccl, c);
                delete c;
                return blum_fail(ctx, BLUM_ERR_COMM, "ncclCommInitRank(rank %d of %d) did not complete within %d ms (a rank never joined?)", rank,
                                 nranks, timeout_ms);
            }
            nap();
        }
    } else {
        r = nccl->CommInitRank(&c->comm, nranks, id, rank);
    }
    if (r != ncclSuccess) {
        if (c->comm) comm_abort(nccl, c);
        delete c;
        return blum_fail(ctx, BLUM_ERR_COMM, "ncclCommInitRank(rank %d of %d) failed: %s", rank, nranks, nccl->GetErrorString(r));
    }
    *out = c;
    return BLUM_OK;
}

int blum_comm_destroy(blum_ctx* ctx, blum_comm* c) {
    if (!ctx) return BLUM_ERR_INVALID;
    if (!c) return BLUM_OK;
    if (!g_use_stubs) cudaStreamSynchronize(ctx->stream);
    if (c->comm && nccl_api()) nccl_api()->CommDestroy(c->comm);
    delete c;
    return BLUM_OK;
}

int blum_comm_rank(const blum_comm* c) { return c ? c->rank : -1; }
int blum_comm_size(const blum_comm* c) { return c ? c->size : -1; }

/* In-place sum over ranks: the exchange after the row-parallel o_proj and down_proj of a tensor-parallel decoder. */
int blum_allreduce_sum(blum_ctx* ctx, blum_comm* c, void* buf, int64_t count, blum_dtype dtype, int timeout_ms) {
    if (!ctx) return BLUM_ERR_INVALID;
    BLUM_REQUIRE(ctx, c && buf && count >= 0, "allreduce: bad argument");
    if (count == 0 || c->size == 1) return BLUM_OK;
    NCCL_API_OR_FAIL(ctx);
    COMM_USABLE(ctx, c, "allreduce");
    BLUM_NCCL_ON(ctx, c, nccl->AllReduce(buf, buf, (size_t)count, nccl_dtype(dtype), ncclSum, c->comm, ctx->stream));
    return comm_watch(ctx, nccl, c, timeout_ms, "allreduce");
}

/* recv [size * count_per_rank] <- every rank's send [count_per_rank] */
int blum_allgather(blum_ctx* ctx, blum_comm* c, const void* send, void* recv, int64_t bytes_per_rank, int timeout_ms) {
    if (!ctx) return BLUM_ERR_INVALID;
    BLUM_REQUIRE(ctx, c && send && recv && bytes_per_rank >= 0, "allgather: bad argument");
    if (bytes_per_rank == 0) return BLUM_OK;
    NCCL_API_OR_FAIL(ctx);
    COMM_USABLE(ctx, c, "allgather");
    BLUM_NCCL_ON(ctx, c, nccl->AllGather(send, recv, (size_t)bytes_per_rank, ncclInt8, c->comm, ctx->stream));
    return comm_watch(ctx, nccl, c, timeout_ms, "allgather");
}

/* Variable all-to-all in bytes (expert-parallel dispatch / combine): rank r receives recv_bytes[p] bytes from peer p at
 * recv_offsets[p] and sends send_bytes[p] bytes from send_offsets[p]; the four arrays are host int64 [size]. */
int blum_alltoallv(blum_ctx* ctx, blum_comm* c, const void* send, const int64_t* send_bytes, const int64_t* send_offsets,
                   void* recv, const int64_t* recv_bytes, const int64_t* recv_offsets, int timeout_ms) {
    if (!ctx) return BLUM_ERR_INVALID;
    BLUM_REQUIRE(ctx, c && send_bytes && send_offsets && recv_bytes && recv_offsets, "alltoallv: bad argument");
    NCCL_API_OR_FAIL(ctx);
    COMM_USABLE(ctx, c, "alltoallv");
    BLUM_NCCL(ctx, nccl->GroupStart());
    for (int p = 0; p < c->size; p++) {
        if (send_bytes[p] > 0) {
            ncclResult_t r = nccl->Send((const char*)send + send_offsets[p], (size_t)send_bytes[p], ncclInt8, p, c->comm, ctx->stream);
            if (r != ncclSuccess && r != ncclInProgress) { nccl->GroupEnd(); return blum_fail(ctx, BLUM_ERR_COMM, "ncclSend to %d failed: %s", p, nccl->GetErrorString(r)); }
        }
        if (recv_bytes[p] > 0) {
            ncclResult_t r = nccl->Recv((char*)recv + recv_offsets[p], (size_t)recv_bytes[p], ncclInt8, p, c->comm, ctx->stream);
            if (r != ncclSuccess && r != ncclInProgress) { nccl->GroupEnd(); return blum_fail(ctx, BLUM_ERR_COMM, "ncclRecv from %d failed: %s", p, nccl->GetErrorString(r)); }
        }
    }
    BLUM_NCCL_ON(ctx, c, nccl->GroupEnd());
    return comm_watch(ctx, nccl, c, timeout_ms, "alltoallv");
}

}  // extern "C"

// ------------------------------------------------------------------ failure paths without a GPU or a second rank
// The NCCL table and the completion query are replaced by host stubs and one scenario is played through the very entry
// points above, on a context that owns no CUDA resources:
//   1 ncclCommInitRank fails           2 a collective returns an error     3 a peer never arrives at a collective
//   4 a rank never joins the init      5 everything works
namespace {
int g_scenario = 0, g_abort_calls = 0, g_ready_after_abort = 0;
ncclResult_t st_unique(ncclUniqueId* id) { memset(id, 7, sizeof *id); return ncclSuccess; }
ncclResult_t st_init(ncclComm_t* c, int, ncclUniqueId, int) {
    if (g_scenario == 1) return ncclSystemError;
    *c = (ncclComm_t)0x1;
    return ncclSuccess;
}
ncclResult_t st_init_cfg(ncclComm_t* c, int n, ncclUniqueId id, int r, ncclConfig_t*) {
    if (g_scenario == 4) { *c = (ncclComm_t)0x1; return ncclInProgress; }
    return st_init(c, n, id, r);
}
ncclResult_t st_async(ncclComm_t, ncclResult_t* r) { *r = (g_scenario == 4) ? ncclInProgress : ncclSuccess; return ncclSuccess; }
ncclResult_t st_abort(ncclComm_t) { g_abort_calls++; g_ready_after_abort = 1; return ncclSuccess; }
ncclResult_t st_destroy(ncclComm_t) { return ncclSuccess; }
ncclResult_t st_allreduce(const void*, void*, size_t, ncclDataType_t, ncclRedOp_t, ncclComm_t, cudaStream_t) {
    return g_scenario == 2 ? ncclInternalError : ncclSuccess;
}
ncclResult_t st_allgather(const void*, void*, size_t, ncclDataType_t, ncclComm_t, cudaStream_t) { return ncclSuccess; }
ncclResult_t st_send(const void*, size_t, ncclDataType_t, int, ncclComm_t, cudaStream_t) { return ncclSuccess; }
ncclResult_t st_recv(void*, size_t, ncclDataType_t, int, ncclComm_t, cudaStream_t) { return ncclSuccess; }
ncclResult_t st_group() { return ncclSuccess; }
const char* st_errstr(ncclResult_t r) { return r == ncclSystemError ? "stub: system error" : r == ncclInternalError ? "stub: internal error" : "stub"; }
int st_ev_record(cudaStream_t, void** ev) { *ev = (void*)0x2; return 0; }
int st_ev_query(void*) { return (g_scenario == 3 && !g_ready_after_abort) ? 1 : 0; }     // scenario 3: the collective never finishes
void st_ev_destroy(void*) {}
}  // namespace

extern "C" int blum_comm_selftest(int scenario, int timeout_ms, char* message_out, int message_cap) {
    if (scenario < 1 || scenario > 5 || timeout_ms <= 0) return BLUM_ERR_INVALID;
    g_scenario = scenario; g_abort_calls = 0; g_ready_after_abort = 0;
    g_stub_api = NcclApi{};
    g_stub_api.GetUniqueId = st_unique; g_stub_api.CommInitRank = st_init; g_stub_api.CommInitRankConfig = st_init_cfg;
    g_stub_api.CommGetAsyncError = st_async; g_stub_api.CommAbort = st_abort; g_stub_api.CommDestroy = st_destroy;
    g_stub_api.AllReduce = st_allreduce; g_stub_api.AllGather = st_allgather; g_stub_api.Send = st_send; g_stub_api.Recv = st_recv;
    g_stub_api.GroupStart = st_group; g_stub_api.GroupEnd = st_group; g_stub_api.GetErrorString = st_errstr; g_stub_api.ok = true;
    const EventApi saved = g_events;
    g_events = EventApi{st_ev_record, st_ev_query, st_ev_destroy};
    g_use_stubs = true;
    blum_ctx fake;                       // owns no CUDA resources; only its error string is used
    fake.device = -1;
    unsigned char id[128];
    int rc = blum_comm_unique_id(id);
    blum_comm* comm = nullptr;
    if (!rc) rc = blum_comm_init_rank(&fake, 2, 0, id, timeout_ms, &comm);
    float buf[4] = {1, 2, 3, 4};
    if (!rc) rc = blum_allreduce_sum(&fake, comm, buf, 4, BLUM_F32, timeout_ms);
    if (scenario == 3 && rc == BLUM_ERR_COMM && comm) {
        // the communicator has been aborted exactly once, and says so on the next call instead of touching NCCL again
        std::string first = fake.err;
        const int rc2 = blum_allgather(&fake, comm, buf, buf, 4, timeout_ms);
        if (rc2 != BLUM_ERR_COMM || g_abort_calls != 1 || fake.err.find("aborted") == std::string::npos) rc = BLUM_ERR_STATE;
        fake.err = first;
    }
    if (scenario == 5 && !rc) {
        int64_t sb[2] = {4, 4}, so[2] = {0, 4}, rb[2] = {4, 4}, ro[2] = {0, 4};
        rc = blum_alltoallv(&fake, comm, buf, sb, so, buf, rb, ro, timeout_ms);
        if (!rc) rc = blum_allgather(&fake, comm, buf, buf, 4, timeout_ms);
    }
    if (comm) blum_comm_destroy(&fake, comm);
    if (message_out && message_cap > 0) { strncpy(message_out, fake.err.c_str(), (size_t)message_cap - 1); message_out[message_cap - 1] = 0; }
    g_use_stubs = false;
    g_events = saved;
    return rc;
}
