// Data-parallel exchange of the gradient arena: NCCL over NVLink / NVSwitch, driven from inside the engine.
//
// The reference has no multi-GPU path at all; this is the sharded-batch extension of its training step (one process
// per GPU, identical weights, gradient buckets summed over the ranks while the rest of backward still runs).
//
//   * NCCL is opened with dlopen at seera_dp_init, so a single-GPU user never loads it.
//   * The gradient arena is allocated with ncclMemAlloc and registered with the communicator (symmetric window where
//     the library offers it, plain registration otherwise): the all-reduce then works on the user buffer itself, with
//     few CTAs and no staging copy, and NVSwitch can reduce in the fabric.
//   * Collectives run on the engine's own high-priority communication stream.  seera_dp_reduce_range() makes that
//     stream wait for what the compute stream has enqueued so far and enqueues an in-place sum of a range of the arena;
//     seera_dp_join() makes the compute stream wait for every range enqueued so far.  Both are event edges only, so the
//     whole step, collectives included, can be recorded into ONE CUDA graph (the communication stream joins the capture
//     through the first edge and leaves it through the join).
//   * Errors: NCCL's asynchronous error state is polled by seera_dp_poll(); seera_dp_wait_host() waits for the last
//     collective with a deadline on the HOST (event query + poll), so a peer that stopped answering turns into a status
//     code, never into a wait inside a kernel of this library.
#include <dlfcn.h>
#include <nccl.h>

#include <chrono>
#include <cstdio>
#include <cstring>
#include <thread>
#include <unordered_map>
#include <vector>

#include "common.cuh"

namespace seera {
namespace {

struct NcclApi {
    void *lib = nullptr;
    decltype(&ncclGetUniqueId) GetUniqueId = nullptr;
    decltype(&ncclCommInitRankConfig) CommInitRankConfig = nullptr;
    decltype(&ncclCommDestroy) CommDestroy = nullptr;
    decltype(&ncclCommAbort) CommAbort = nullptr;
    decltype(&ncclAllReduce) AllReduce = nullptr;
    decltype(&ncclBroadcast) Broadcast = nullptr;
    decltype(&ncclCommGetAsyncError) CommGetAsyncError = nullptr;
    decltype(&ncclGetErrorString) GetErrorString = nullptr;
    decltype(&ncclGetVersion) GetVersion = nullptr;
    decltype(&ncclMemAlloc) MemAlloc = nullptr;
    decltype(&ncclMemFree) MemFree = nullptr;
    decltype(&ncclCommRegister) CommRegister = nullptr;
    decltype(&ncclCommDeregister) CommDeregister = nullptr;
    decltype(&ncclCommWindowRegister) CommWindowRegister = nullptr;        // may be absent in older libraries
    decltype(&ncclCommWindowDeregister) CommWindowDeregister = nullptr;
};

struct Registration { void *handle = nullptr; ncclWindow_t win = nullptr; size_t bytes = 0; };

struct Dp {
    NcclApi api;
    ncclComm_t comm = nullptr;
    int rank = 0, world = 1, version = 0;
    cudaStream_t comm_stream = nullptr;
    cudaEvent_t fork_ev = nullptr, done_ev = nullptr;
    bool pending = false;                     // a range was enqueued since the last join
    cudaStream_t main_stream = nullptr;       // the compute stream while launches are diverted (seera_dp_side_begin)
    bool side = false;
    std::unordered_map<void *, Registration> regs;
    std::vector<void *> reg_order;            // blocks in the order they were registered: window (de)registration is collective
                                              // over the ranks, so every rank must walk its blocks in the same order
};
Dp &dp() { static Dp d; return d; }

int nccl_fail(ncclResult_t r, const char *what) {
    Dp &d = dp();
    return fail(SEERA_E_CUDA, "%s: NCCL error %d (%s)", what, (int)r, d.api.GetErrorString ? d.api.GetErrorString(r) : "?");
}
#define SEERA_NCCL(call, what)                                   \
    do {                                                         \
        ncclResult_t _r = (call);                                \
        if (_r != ncclSuccess) return nccl_fail(_r, what);       \
    } while (0)

int load_api(NcclApi &a) {
    if (a.lib) return SEERA_OK;
    const char *names[] = {getenv("SEERA_NCCL_LIBRARY"), "libnccl.so.2", "libnccl.so"};
    for (const char *n : names) {
        if (!n || !*n) continue;
        a.lib = dlopen(n, RTLD_NOW | RTLD_LOCAL);
        if (a.lib) break;
    }
    if (!a.lib) return fail(SEERA_E_CUDA, "seera_dp: cannot load libnccl.so.2 (%s)", dlerror());
#define SYM(field, name, required)                                                                           \
    a.field = reinterpret_cast<decltype(a.field)>(dlsym(a.lib, name));                                       \
    if (required && !a.field) { dlclose(a.lib); a.lib = nullptr; return fail(SEERA_E_CUDA, "seera_dp: libnccl lacks %s", name); }
    SYM(GetUniqueId, "ncclGetUniqueId", true)
    SYM(CommInitRankConfig, "ncclCommInitRankConfig", true)
    SYM(CommDestroy, "ncclCommDestroy", true)
    SYM(CommAbort, "ncclCommAbort", true)
    SYM(AllReduce, "ncclAllReduce", true)
    SYM(Broadcast, "ncclBroadcast", true)
    SYM(CommGetAsyncError, "ncclCommGetAsyncError", true)
    SYM(GetErrorString, "ncclGetErrorString", true)
    SYM(GetVersion, "ncclGetVersion", true)
    SYM(MemAlloc, "ncclMemAlloc", true)
    SYM(MemFree, "ncclMemFree", true)
    SYM(CommRegister, "ncclCommRegister", true)
    SYM(CommDeregister, "ncclCommDeregister", true)
    SYM(CommWindowRegister, "ncclCommWindowRegister", false)
    SYM(CommWindowDeregister, "ncclCommWindowDeregister", false)
#undef SYM
    return SEERA_OK;
}

int need_comm(const char *what) {
    if (!dp().comm) return fail(SEERA_E_ARG, "%s: seera_dp_init has not been called", what);
    return SEERA_OK;
}

}  // namespace
}  // namespace seera

using namespace seera;

extern "C" {

int seera_dp_unique_id_bytes(void) { return (int)sizeof(ncclUniqueId); }

int seera_dp_unique_id(void *out, int size) {
    SEERA_ENSURE();
    if (!out || size < (int)sizeof(ncclUniqueId)) return fail(SEERA_E_ARG, "dp_unique_id: needs a buffer of %d bytes", (int)sizeof(ncclUniqueId));
    Dp &d = dp();
    if (int s = load_api(d.api)) return s;
    ncclUniqueId id;
    SEERA_NCCL(d.api.GetUniqueId(&id), "ncclGetUniqueId");
    memcpy(out, &id, sizeof(id));
    return SEERA_OK;
}

int seera_dp_init(int rank, int world, const void *unique_id, int size) {
    SEERA_ENSURE();
    Dp &d = dp();
    if (d.comm) return fail(SEERA_E_ARG, "dp_init: already initialised (rank %d of %d)", d.rank, d.world);
    if (world < 1 || rank < 0 || rank >= world || !unique_id || size < (int)sizeof(ncclUniqueId))
        return fail(SEERA_E_ARG, "dp_init: bad argument (rank %d, world %d)", rank, world);
    if (rt().capturing) return fail(SEERA_E_ARG, "dp_init: not allowed while a graph is being captured");
    if (int s = load_api(d.api)) return s;
    d.api.GetVersion(&d.version);
    ncclUniqueId id;
    memcpy(&id, unique_id, sizeof(id));
    ncclConfig_t cfg = NCCL_CONFIG_INITIALIZER;
    cfg.blocking = 1;
    SEERA_NCCL(d.api.CommInitRankConfig(&d.comm, world, id, rank, &cfg), "ncclCommInitRankConfig");
    d.rank = rank; d.world = world;
    int lo = 0, hi = 0;
    cudaDeviceGetStreamPriorityRange(&lo, &hi);             // hi = numerically lowest = highest priority
    if (int s = check_cuda(cudaStreamCreateWithPriority(&d.comm_stream, cudaStreamNonBlocking, hi), "cudaStreamCreateWithPriority")) return s;
    if (int s = check_cuda(cudaEventCreateWithFlags(&d.fork_ev, cudaEventDisableTiming), "cudaEventCreate")) return s;
    if (int s = check_cuda(cudaEventCreateWithFlags(&d.done_ev, cudaEventDisableTiming), "cudaEventCreate")) return s;
    return SEERA_OK;
}

int seera_dp_rank(void) { return dp().rank; }
int seera_dp_world(void) { return dp().world; }
int seera_dp_nccl_version(void) { return dp().version; }

/* Device memory the collectives can use in place: ncclMemAlloc + registration with the communicator. */
void *seera_dp_alloc(size_t bytes) {
    if (ensure_init() || need_comm("dp_alloc")) return nullptr;
    Dp &d = dp();
    void *p = nullptr;
    if (bytes == 0) bytes = 4;
    ncclResult_t r = d.api.MemAlloc(&p, bytes);
    if (r != ncclSuccess || !p) { nccl_fail(r, "ncclMemAlloc"); return nullptr; }
    Registration reg;
    reg.bytes = bytes;
    bool done = false;
    if (d.api.CommWindowRegister && getenv("SEERA_DP_NO_WINDOW") == nullptr) {
        ncclWindow_t w = nullptr;
        if (d.api.CommWindowRegister(d.comm, p, bytes, &w, NCCL_WIN_COLL_SYMMETRIC) == ncclSuccess && w) { reg.win = w; done = true; }
    }
    if (!done) {
        void *h = nullptr;
        if (d.api.CommRegister(d.comm, p, bytes, &h) == ncclSuccess) reg.handle = h;       // failure only loses the zero-copy path
    }
    cudaMemsetAsync(p, 0, bytes, rt().stream);
    d.regs[p] = reg;
    d.reg_order.push_back(p);
    return p;
}

int seera_dp_free(void *p) {
    if (!p) return SEERA_OK;
    Dp &d = dp();
    auto it = d.regs.find(p);
    if (it == d.regs.end()) return fail(SEERA_E_ARG, "dp_free: not a seera_dp_alloc block");
    cudaStreamSynchronize(rt().stream);
    if (d.comm_stream) cudaStreamSynchronize(d.comm_stream);
    if (d.comm) {
        if (it->second.win && d.api.CommWindowDeregister) d.api.CommWindowDeregister(d.comm, it->second.win);
        if (it->second.handle) d.api.CommDeregister(d.comm, it->second.handle);
    }
    d.api.MemFree(p);
    d.regs.erase(it);
    for (size_t i = 0; i < d.reg_order.size(); i++)
        if (d.reg_order[i] == p) { d.reg_order.erase(d.reg_order.begin() + (long)i); break; }
    return SEERA_OK;
}

static int red_op(int op, ncclRedOp_t *out) {
    switch (op) {
        case 0: *out = ncclSum; return SEERA_OK;
        case 1: *out = ncclMax; return SEERA_OK;
        case 2: *out = ncclMin; return SEERA_OK;
        default: return fail(SEERA_E_ARG, "dp: reduction %d (0 sum, 1 max, 2 min)", op);
    }
}

/* In-place reduction of n floats over the ranks, enqueued on the COMPUTE stream (ordered with the kernels around it). */
int seera_dp_allreduce(float *buf, long long n, int op) {
    SEERA_ENSURE();
    if (int s = need_comm("dp_allreduce")) return s;
    if (!buf || n < 0) return fail(SEERA_E_ARG, "dp_allreduce: bad argument");
    if (n == 0) return SEERA_OK;
    ncclRedOp_t o;
    if (int s = red_op(op, &o)) return s;
    Dp &d = dp();
    SEERA_NCCL(d.api.AllReduce(buf, buf, (size_t)n, ncclFloat, o, d.comm, rt().stream), "ncclAllReduce");
    graph_note_collective();
    count_launch();
    return SEERA_OK;
}

int seera_dp_broadcast(float *buf, long long n, int root) {
    SEERA_ENSURE();
    if (int s = need_comm("dp_broadcast")) return s;
    if (!buf || n < 0 || root < 0 || root >= dp().world) return fail(SEERA_E_ARG, "dp_broadcast: bad argument");
    if (n == 0) return SEERA_OK;
    Dp &d = dp();
    SEERA_NCCL(d.api.Broadcast(buf, buf, (size_t)n, ncclFloat, root, d.comm, rt().stream), "ncclBroadcast");
    graph_note_collective();
    count_launch();
    return SEERA_OK;
}

/* Sum of floats [begin, end) of `arena` over the ranks on the communication stream, after everything the compute stream
 * holds so far; returns at once. */
int seera_dp_reduce_range(float *arena, long long begin, long long end) {
    SEERA_ENSURE();
    if (int s = need_comm("dp_reduce_range")) return s;
    if (!arena || begin < 0 || end < begin) return fail(SEERA_E_ARG, "dp_reduce_range: bad range");
    if (end == begin) return SEERA_OK;
    Dp &d = dp();
    if (int s = check_cuda(cudaEventRecord(d.fork_ev, rt().stream), "cudaEventRecord")) return s;
    if (int s = check_cuda(cudaStreamWaitEvent(d.comm_stream, d.fork_ev, 0), "cudaStreamWaitEvent")) return s;
    SEERA_NCCL(d.api.AllReduce(arena + begin, arena + begin, (size_t)(end - begin), ncclFloat, ncclSum, d.comm, d.comm_stream), "ncclAllReduce");
    graph_note_collective();
    count_launch();
    d.pending = true;
    return SEERA_OK;
}

/* Between seera_dp_side_begin() and seera_dp_side_end() every launch of this library goes to the communication stream, behind
 * the collectives already enqueued there and behind what the compute stream held at the call: the optimizer's update of a
 * bucket follows that bucket's sum without waiting for the rest of backward, and seera_dp_join() covers it like the sums.
 * Only for entries that take no scratch memory from the pool (the optimizer steps): the pool recycles blocks in the order
 * of ONE stream. */
int seera_dp_side_begin(void) {
    SEERA_ENSURE();
    if (int s = need_comm("dp_side_begin")) return s;
    Dp &d = dp();
    if (d.side) return fail(SEERA_E_ARG, "dp_side_begin: already diverted");
    if (int s = check_cuda(cudaEventRecord(d.fork_ev, rt().stream), "cudaEventRecord")) return s;
    if (int s = check_cuda(cudaStreamWaitEvent(d.comm_stream, d.fork_ev, 0), "cudaStreamWaitEvent")) return s;
    d.main_stream = rt().stream;
    rt().stream = d.comm_stream;
    d.side = true;
    d.pending = true;
    return SEERA_OK;
}
int seera_dp_side_end(void) {
    Dp &d = dp();
    if (!d.side) return SEERA_OK;
    rt().stream = d.main_stream;
    d.side = false;
    return SEERA_OK;
}

/* The compute stream waits for every range enqueued since the last join. */
int seera_dp_join(void) {
    SEERA_ENSURE();
    Dp &d = dp();
    if (d.side) seera_dp_side_end();
    if (!d.comm || !d.pending) return SEERA_OK;
    if (int s = check_cuda(cudaEventRecord(d.done_ev, d.comm_stream), "cudaEventRecord")) return s;
    if (int s = check_cuda(cudaStreamWaitEvent(rt().stream, d.done_ev, 0), "cudaStreamWaitEvent")) return s;
    d.pending = false;
    return SEERA_OK;
}

/* NCCL's asynchronous error state: SEERA_OK, or SEERA_E_CUDA with the message recorded. */
int seera_dp_poll(void) {
    Dp &d = dp();
    if (!d.comm) return SEERA_OK;
    ncclResult_t st = ncclSuccess;
    ncclResult_t r = d.api.CommGetAsyncError(d.comm, &st);
    if (r != ncclSuccess) return nccl_fail(r, "ncclCommGetAsyncError");
    if (st != ncclSuccess && st != ncclInProgress) return nccl_fail(st, "asynchronous NCCL error");
    return SEERA_OK;
}

/* Host-side wait for everything enqueued on both streams, with a deadline.  On expiry (a peer has stopped taking part)
 * or on an asynchronous NCCL error the communicator is aborted, so that the process can go on without it, and an error
 * status is returned.  Not allowed during a capture. */
int seera_dp_wait_host(int timeout_ms) {
    SEERA_ENSURE();
    if (rt().capturing) return fail(SEERA_E_ARG, "dp_wait_host: not allowed while a graph is being captured");
    Dp &d = dp();
    if (!d.comm) return check_cuda(cudaStreamSynchronize(rt().stream), "cudaStreamSynchronize");
    cudaEvent_t ev[2];
    cudaStream_t st[2] = {rt().stream, d.comm_stream};
    for (int i = 0; i < 2; i++) {
        if (int s = check_cuda(cudaEventCreateWithFlags(&ev[i], cudaEventDisableTiming), "cudaEventCreate")) return s;
        cudaEventRecord(ev[i], st[i]);
    }
    auto t0 = std::chrono::steady_clock::now();
    int status = SEERA_OK;
    for (;;) {
        cudaError_t a = cudaEventQuery(ev[0]), b = cudaEventQuery(ev[1]);
        if (a == cudaSuccess && b == cudaSuccess) break;
        if ((a != cudaSuccess && a != cudaErrorNotReady) || (b != cudaSuccess && b != cudaErrorNotReady)) {
            status = check_cuda(a != cudaSuccess && a != cudaErrorNotReady ? a : b, "dp_wait_host");
            break;
        }
        if ((status = seera_dp_poll()) != SEERA_OK) break;
        auto ms = std::chrono::duration_cast<std::chrono::milliseconds>(std::chrono::steady_clock::now() - t0).count();
        if (timeout_ms >= 0 && ms > timeout_ms) {
            status = fail(SEERA_E_CUDA, "dp_wait_host: a collective did not finish within %d ms (a peer left or stalled); communicator aborted", timeout_ms);
            break;
        }
        std::this_thread::sleep_for(std::chrono::microseconds(200));
    }
    cudaEventDestroy(ev[0]); cudaEventDestroy(ev[1]);
    if (status != SEERA_OK && d.comm) {
        d.api.CommAbort(d.comm);           // unblocks the kernels of the unfinished collective on this rank
        d.comm = nullptr;
        d.pending = false;
        d.regs.clear();                    // the registrations went with the communicator; the memory stays allocated
        d.reg_order.clear();
    }
    return status;
}

/* Drops the communicator without talking to the peers (ncclCommAbort): the way out when one of them is known to be gone.
 * Blocks seera_dp_alloc handed out stay allocated until the process ends. */
int seera_dp_abort(void) {
    Dp &d = dp();
    seera_dp_side_end();
    if (!d.comm) return SEERA_OK;
    d.api.CommAbort(d.comm);
    d.comm = nullptr;
    d.pending = false;
    d.regs.clear();
    d.reg_order.clear();
    d.world = 1; d.rank = 0;
    return SEERA_OK;
}

int seera_dp_finalize(void) {
    Dp &d = dp();
    seera_dp_side_end();
    if (!d.comm) return SEERA_OK;
    cudaStreamSynchronize(rt().stream);
    cudaStreamSynchronize(d.comm_stream);
    graphs_with_collectives_release();         // recordings that hold this communicator's launches go first
    for (void *p : d.reg_order) {              // registration order, the same on every rank (not the map's hash order)
        auto it = d.regs.find(p);
        if (it == d.regs.end()) continue;
        if (it->second.win && d.api.CommWindowDeregister) d.api.CommWindowDeregister(d.comm, it->second.win);
        if (it->second.handle) d.api.CommDeregister(d.comm, it->second.handle);
        d.api.MemFree(p);
    }
    d.regs.clear();
    d.reg_order.clear();
    d.api.CommDestroy(d.comm);
    d.comm = nullptr;
    if (d.comm_stream) { cudaStreamDestroy(d.comm_stream); d.comm_stream = nullptr; }
    if (d.fork_ev) { cudaEventDestroy(d.fork_ev); d.fork_ev = nullptr; }
    if (d.done_ev) { cudaEventDestroy(d.done_ev); d.done_ev = nullptr; }
    d.world = 1; d.rank = 0; d.pending = false;
    return SEERA_OK;
}

}  // extern "C"
