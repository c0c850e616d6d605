// Runtime: device/stream selection, status, the pooled stream-ordered allocator and the
// host<->device transfers behind the memory entries of the boundary
// (reference: engine_cuda/src/cuda_bindings.cpp:23-170, which calls cudaMalloc / cudaFree /
// cudaMemcpy directly on every call).
//
// Allocator: freed blocks are kept in per-size free lists and handed out again for the same
// rounded size.  All work runs on one stream, so a block returned by cuda_free may be reused
// by the next allocation without waiting: every kernel that still reads it was enqueued earlier.
#include "common.cuh"
#include <cstdarg>
#include <cstdlib>
#include <cstring>
#include <string>
#include <map>
#include <unordered_map>
#include <vector>

namespace seera {

// Configuration by environment, read once when the library is first used:
//   SEERA_PRECISION   0..5   initial precision mode of the contractions (default 3: bf16x6 on the tensor cores - fp32-class
//                            products over fp32's whole exponent range, so that a caller who never heard of
//                            seera_set_precision still runs on tcgen05 kernels and still matches the fp32 reference)
//   SEERA_PAIR_TILES  0|1    the "pair_tiles" option (TMA-fed GEMMs as clusters of two CTAs on 256-row tiles)
//   SEERA_SM_RESERVE  n      SMs the persistent kernels leave free (the "sm_reserve" option)
//   SEERA_TC_WAIT_MS  n      budget of the bounded waits inside the tensor-core kernels, in milliseconds (default 2000)
static Runtime make_runtime() {
    Runtime r;
    r.precision = 3;
    if (const char *e = getenv("SEERA_PRECISION")) {
        int m = atoi(e);
        if (m >= 0 && m <= 5 && e[0] >= '0' && e[0] <= '5') r.precision = m;
    }
    if (const char *e = getenv("SEERA_PAIR_TILES")) r.pair_tiles = atoi(e) != 0;
    if (const char *e = getenv("SEERA_TC_WAIT_MS")) {
        long long ms = atoll(e);
        if (ms > 0) r.tc_wait_clocks = (unsigned long long)ms * 2000000ull;      // ~2e6 clocks per millisecond
    }
    return r;
}
Runtime &rt() { static Runtime r = make_runtime(); return r; }

int fail(int code, const char *fmt, ...) {
    Runtime &r = rt();
    va_list ap; va_start(ap, fmt);
    vsnprintf(r.err, sizeof(r.err), fmt, ap);
    va_end(ap);
    r.status = code;
    return code;
}

int check_cuda(cudaError_t e, const char *what) {
    if (e == cudaSuccess) return SEERA_OK;
    return fail(SEERA_E_CUDA, "%s: %s", what, cudaGetErrorString(e));
}

int ensure_init() {
    if (rt().device >= 0) return SEERA_OK;
    return seera_init(0);
}

namespace {
struct GraphRec {
    cudaGraph_t graph = nullptr;
    cudaGraphExec_t exec = nullptr;
    std::vector<std::pair<void *, size_t>> blocks;      // every block handed out while the graph was captured
    uint64_t kernels = 0;                               // kernel launches recorded in the graph
    uint64_t launches_at_begin = 0;
    bool collectives = false;                           // the recording holds launches of the data-parallel communicator
};
static std::vector<GraphRec *> &live_graphs() { static std::vector<GraphRec *> v; return v; }
struct Pool {
    std::map<size_t, std::vector<void *>> free_lists;   // rounded size -> cached blocks
    std::unordered_map<void *, size_t> live;            // every block handed out -> rounded size
    size_t reserved = 0;
    // stream capture: blocks used inside a captured step stay reserved for the graph that replays it
    bool capturing = false;
    std::map<size_t, std::vector<void *>> cap_free;     // freed during capture: reusable only inside the capture
    std::unordered_map<void *, GraphRec *> owner;       // block -> graph whose replay writes it
    GraphRec *cur = nullptr;
};
Pool &pool() { static Pool p; return p; }

size_t round_size(size_t n) {
    if (n == 0) n = 1;
    if (n <= (1u << 20)) return (n + 511) & ~size_t(511);                 // 512 B granules up to 1 MiB
    return (n + (size_t(2) << 20) - 1) & ~((size_t(2) << 20) - 1);        // 2 MiB granules above
}
}  // namespace

// Per-launch profile (seera_profile_enable): launches bracketed by profile_begin / profile_end[_bytes] are timed with
// events on the engine's stream and booked under a tag.  Contractions book FLOPs and a kind (0 forward, 1 data gradient,
// 2 weight gradient, from the entry name's "(dX)" / "(dW)" suffix); bandwidth-bound passes book their algorithmic bytes
// (kind 3).  Nothing is recorded while a graph is being captured.
struct ProfRec { cudaEvent_t a, b; double work; int kind; const char *tag; };
struct ProfAgg { int kind = 0; uint64_t n = 0; double ms = 0, work = 0; };
struct Prof { bool on = false; std::vector<ProfRec> recs; cudaEvent_t pending = nullptr; std::map<std::string, ProfAgg> table; };
static Prof &prof() { static Prof p; return p; }

void profile_begin() {
    Prof &p = prof();
    if (!p.on || rt().capturing) return;
    cudaEventCreate(&p.pending);
    cudaEventRecord(p.pending, rt().stream);
}
static int profile_kind(const char *name) {
    if (!name) return 0;
    size_t n = strlen(name);
    if (n >= 4 && name[n - 1] == ')' && name[n - 4] == '(' && name[n - 3] == 'd') {
        char c = name[n - 2];
        return (c == 'X' || c == 'A') ? 1 : ((c == 'W' || c == 'B') ? 2 : 0);
    }
    return strcmp(name, "conv2d_act_bwd") == 0 ? 2 : 0;       // the short-patch layer backward forms only the weight gradient
}
static void profile_close(double work, int kind, const char *tag) {
    Prof &p = prof();
    if (!p.on || !p.pending) return;
    ProfRec r{p.pending, nullptr, work, kind, tag ? tag : "?"};
    cudaEventCreate(&r.b);
    cudaEventRecord(r.b, rt().stream);
    p.recs.push_back(r);
    p.pending = nullptr;
}
void profile_end(double flops, const char *name) { profile_close(flops, profile_kind(name), name); }
void profile_end_bytes(double bytes, const char *tag) { profile_close(bytes, 3, tag); }

// Resolves the recorded events into the per-tag table (waits for them).
static void profile_collect() {
    Prof &p = prof();
    for (auto &r : p.recs) {
        float e = 0.f;
        cudaEventSynchronize(r.b);
        cudaEventElapsedTime(&e, r.a, r.b);
        ProfAgg &g = p.table[std::string(r.tag)];
        g.kind = r.kind; g.n++; g.ms += e; g.work += r.work;
        cudaEventDestroy(r.a); cudaEventDestroy(r.b);
    }
    p.recs.clear();
}

void *scratch_alloc(size_t bytes) { return seera_cuda_malloc(bytes); }
void scratch_free(void *p) { seera_cuda_free(p); }

}  // namespace seera

namespace seera {
// dp.cu: a collective is being recorded into the open capture
void graph_note_collective() {
    Pool &p = pool();
    if (p.capturing && p.cur) p.cur->collectives = true;
}
// dp.cu, before the communicator goes away: the library that runs the collectives keeps per-recording state alive as long as a
// recording that holds its launches exists, and tearing the communicator down waits for that state.  The executable graphs are
// destroyed here; their handles stay valid for seera_graph_destroy, and seera_graph_launch on them reports an error.
void graphs_with_collectives_release() {
    if (rt().stream) cudaStreamSynchronize(rt().stream);
    for (GraphRec *g : live_graphs()) {
        if (!g->collectives) continue;
        if (g->exec) { cudaGraphExecDestroy(g->exec); g->exec = nullptr; }
        if (g->graph) { cudaGraphDestroy(g->graph); g->graph = nullptr; }
    }
}
}  // namespace seera

using namespace seera;

extern "C" {

int seera_init(int device) {
    Runtime &r = rt();
    if (r.device == device && r.stream) return SEERA_OK;
    // one device per process: the stream, the memory pool, the tensor-core status word and the profiler events all belong to
    // the device of the first call
    if (r.device >= 0 && r.device != device)
        return fail(SEERA_E_ARG, "seera_init: this process already runs on device %d (one device per process; asked for %d)", r.device, device);
    int n = 0;
    cudaError_t e = cudaGetDeviceCount(&n);
    if (e != cudaSuccess || n == 0)
        return fail(SEERA_E_CUDA, "seera_init: no CUDA device (%s)", cudaGetErrorString(e));
    if (device < 0 || device >= n) return fail(SEERA_E_ARG, "seera_init: device %d of %d", device, n);
    if (int s = check_cuda(cudaSetDevice(device), "cudaSetDevice")) return s;
    cudaDeviceProp p;
    if (int s = check_cuda(cudaGetDeviceProperties(&p, device), "cudaGetDeviceProperties")) return s;
    r.sm_count = r.sm_physical = p.multiProcessorCount;
    if (!r.own_stream)
        if (int s = check_cuda(cudaStreamCreateWithFlags(&r.own_stream, cudaStreamNonBlocking), "cudaStreamCreate")) return s;
    r.stream = r.own_stream;
    r.device = device;
    if (const char *e = getenv("SEERA_SM_RESERVE")) {
        int n = atoi(e);
        if (n > 0 && n < r.sm_physical) r.sm_count = r.sm_physical - n;
    }
    return SEERA_OK;
}

int seera_synchronize(void) {
    SEERA_ENSURE();
    if (rt().capturing) return fail(SEERA_E_ARG, "synchronize: not allowed while a graph is being captured");
    return check_cuda(cudaStreamSynchronize(rt().stream), "cudaStreamSynchronize");
}

int seera_set_stream(void *s) {
    SEERA_ENSURE();
    rt().stream = s ? reinterpret_cast<cudaStream_t>(s) : rt().own_stream;
    return SEERA_OK;
}
void *seera_get_stream(void) { return ensure_init() ? nullptr : (void *)rt().stream; }
const char *seera_last_error(void) { return rt().err; }
int seera_last_status(void) { return rt().status; }
void seera_clear_status(void) { rt().status = 0; rt().err[0] = 0; }
uint64_t seera_launch_count(void) { return rt().launches; }
int seera_device_sm_count(void) { return ensure_init() ? 0 : rt().sm_count; }
void *seera_event_create(void) {
    if (ensure_init()) return nullptr;
    cudaEvent_t e;
    if (cudaEventCreate(&e) != cudaSuccess) { cudaGetLastError(); return nullptr; }
    return (void *)e;
}
int seera_event_record(void *ev) {
    SEERA_ENSURE();
    if (!ev) return fail(SEERA_E_ARG, "event_record: null");
    return check_cuda(cudaEventRecord((cudaEvent_t)ev, rt().stream), "cudaEventRecord");
}
float seera_event_elapsed_ms(void *a, void *b) {
    if (!a || !b) return -1.f;
    if (cudaEventSynchronize((cudaEvent_t)b) != cudaSuccess) { check_cuda(cudaGetLastError(), "cudaEventSynchronize"); return -1.f; }
    float ms = -1.f;
    if (cudaEventElapsedTime(&ms, (cudaEvent_t)a, (cudaEvent_t)b) != cudaSuccess) { cudaGetLastError(); return -1.f; }
    return ms;
}
int seera_event_destroy(void *ev) { return ev ? check_cuda(cudaEventDestroy((cudaEvent_t)ev), "cudaEventDestroy") : SEERA_OK; }

int seera_profile_enable(int on) {
    auto &p = seera::prof();
    if (on && !p.on) { seera::profile_collect(); p.table.clear(); }      // a new session starts from an empty table
    p.on = on != 0;
    return SEERA_OK;
}
int seera_profile_read_kinds(uint64_t *launches3, double *ms3, double *flops3) {
    SEERA_ENSURE();
    seera::profile_collect();
    uint64_t n[3] = {0, 0, 0};
    double t[3] = {0, 0, 0}, f[3] = {0, 0, 0};
    for (auto &kv : seera::prof().table) {
        const auto &g = kv.second;
        if (g.kind > 2) continue;
        n[g.kind] += g.n; t[g.kind] += g.ms; f[g.kind] += g.work;
    }
    for (int k = 0; k < 3; k++) {
        if (launches3) launches3[k] = n[k];
        if (ms3) ms3[k] = t[k];
        if (flops3) flops3[k] = f[k];
    }
    return SEERA_OK;
}
int seera_profile_read(uint64_t *launches, double *ms, double *flops) {
    uint64_t n[3];
    double t[3], f[3];
    if (int s = seera_profile_read_kinds(n, t, f)) return s;
    if (launches) *launches = n[0] + n[1] + n[2];
    if (ms) *ms = t[0] + t[1] + t[2];
    if (flops) *flops = f[0] + f[1] + f[2];
    seera::prof().table.clear();
    return SEERA_OK;
}
int seera_profile_report(char *buf, size_t size) {
    SEERA_ENSURE();
    if (!buf || size < 2) return fail(SEERA_E_ARG, "profile_report: no buffer");
    seera::profile_collect();
    size_t off = 0;
    buf[0] = 0;
    for (auto &kv : seera::prof().table) {
        const auto &g = kv.second;
        int w = snprintf(buf + off, size - off, "%s\t%d\t%llu\t%.6f\t%.6e\n", kv.first.c_str(), g.kind, (unsigned long long)g.n, g.ms, g.work);
        if (w < 0 || (size_t)w >= size - off) { buf[off] = 0; return fail(SEERA_E_LIMIT, "profile_report: buffer of %zu bytes is too small", size); }
        off += (size_t)w;
    }
    return SEERA_OK;
}

int seera_set_precision(int mode) {
    if (mode < 0 || mode > 5) return fail(SEERA_E_ARG, "seera_set_precision: mode %d", mode);
    rt().precision = mode;
    return SEERA_OK;
}
int seera_get_precision(void) { return rt().precision; }

void *seera_cuda_malloc(size_t n_bytes) {
    if (ensure_init()) return nullptr;
    Pool &p = pool();
    size_t sz = round_size(n_bytes);
    if (p.capturing) {
        auto ic = p.cap_free.find(sz);
        if (ic != p.cap_free.end() && !ic->second.empty()) {
            void *b = ic->second.back();
            ic->second.pop_back();
            p.live[b] = sz;
            return b;
        }
    }
    auto it = p.free_lists.find(sz);
    if (it != p.free_lists.end() && !it->second.empty()) {
        void *b = it->second.back();
        it->second.pop_back();
        p.live[b] = sz;
        if (p.capturing) { p.owner[b] = p.cur; p.cur->blocks.push_back({b, sz}); }
        return b;
    }
    void *b = nullptr;
    cudaError_t e = cudaMalloc(&b, sz);
    if (e != cudaSuccess) {            // give cached blocks back to the driver and retry once
        cudaGetLastError();
        seera_pool_trim();
        e = cudaMalloc(&b, sz);
    }
    if (e != cudaSuccess) {
        cudaGetLastError();
        fail(SEERA_E_OOM, "cuda_malloc(%zu): %s", n_bytes, cudaGetErrorString(e));
        return nullptr;
    }
    p.reserved += sz;
    p.live[b] = sz;
    if (p.capturing) { p.owner[b] = p.cur; p.cur->blocks.push_back({b, sz}); }
    return b;
}
void *seera_cuda_malloc_f32(int n) { return n < 0 ? nullptr : seera_cuda_malloc((size_t)n * 4); }
void *seera_cuda_malloc_i32(int n) { return n < 0 ? nullptr : seera_cuda_malloc((size_t)n * 4); }
void *seera_cuda_malloc_i16(int n) { return n < 0 ? nullptr : seera_cuda_malloc((size_t)n * 2); }

int seera_cuda_free(void *ptr) {
    if (!ptr) return SEERA_OK;
    Pool &p = pool();
    auto it = p.live.find(ptr);
    if (it == p.live.end()) return fail(SEERA_E_ARG, "cuda_free(%p): not a live block of this pool", ptr);
    auto ow = p.owner.find(ptr);
    if (ow != p.owner.end()) {
        // a block a captured graph writes on every replay: reusable inside that capture, otherwise kept aside
        if (p.capturing && ow->second == p.cur) p.cap_free[it->second].push_back(ptr);
    } else {
        p.free_lists[it->second].push_back(ptr);
    }
    p.live.erase(it);
    return SEERA_OK;
}

int seera_pool_trim(void) {
    Pool &p = pool();
    if (rt().stream) cudaStreamSynchronize(rt().stream);
    for (auto &kv : p.free_lists) {
        for (void *b : kv.second) { cudaFree(b); p.reserved -= kv.first; }
        kv.second.clear();
    }
    return SEERA_OK;
}
size_t seera_pool_bytes_reserved(void) { return pool().reserved; }

int seera_graph_begin(void) {
    SEERA_ENSURE();
    Pool &p = pool();
    if (p.capturing) return fail(SEERA_E_ARG, "graph_begin: a capture is already open");
    if (int s = check_cuda(cudaStreamBeginCapture(rt().stream, cudaStreamCaptureModeRelaxed), "cudaStreamBeginCapture")) return s;
    p.cur = new GraphRec();
    p.cur->launches_at_begin = rt().launches;
    p.cap_free.clear();
    p.capturing = true;
    rt().capturing = true;
    return SEERA_OK;
}

void *seera_graph_end(void) {
    Pool &p = pool();
    if (!p.capturing) { fail(SEERA_E_ARG, "graph_end: no capture is open"); return nullptr; }
    p.capturing = false;
    rt().capturing = false;
    p.cap_free.clear();
    GraphRec *g = p.cur;
    p.cur = nullptr;
    g->kernels = rt().launches - g->launches_at_begin;
    rt().launches = g->launches_at_begin;               // recorded, not executed
    cudaError_t e = cudaStreamEndCapture(rt().stream, &g->graph);
    if (e == cudaSuccess) e = cudaGraphInstantiate(&g->exec, g->graph, 0);
    if (e != cudaSuccess) {
        check_cuda(e, "graph_end");
        cudaGetLastError();
        seera_graph_destroy(g);
        return nullptr;
    }
    live_graphs().push_back(g);
    return g;
}

int seera_graph_launch(void *graph) {
    SEERA_ENSURE();
    GraphRec *g = static_cast<GraphRec *>(graph);
    if (!g || !g->exec) return fail(SEERA_E_ARG, "graph_launch: not a captured graph (or one whose communicator has been finalized)");
    rt().launches += g->kernels;
    return check_cuda(cudaGraphLaunch(g->exec, rt().stream), "cudaGraphLaunch");
}

int seera_graph_destroy(void *graph) {
    GraphRec *g = static_cast<GraphRec *>(graph);
    if (!g) return SEERA_OK;
    Pool &p = pool();
    if (rt().stream) cudaStreamSynchronize(rt().stream);
    if (g->exec) cudaGraphExecDestroy(g->exec);
    if (g->graph) cudaGraphDestroy(g->graph);
    for (auto &b : g->blocks) {
        p.owner.erase(b.first);
        if (!p.live.count(b.first)) p.free_lists[b.second].push_back(b.first);   // idle: back to the general pool
    }
    auto &lg = live_graphs();
    for (size_t i = 0; i < lg.size(); i++)
        if (lg[i] == g) { lg.erase(lg.begin() + (long)i); break; }
    delete g;
    return SEERA_OK;
}
int seera_is_capturing(void) { return pool().capturing ? 1 : 0; }

void *seera_host_alloc_pinned(size_t n) {
    if (ensure_init()) return nullptr;
    void *p = nullptr;
    if (cudaMallocHost(&p, n ? n : 1) != cudaSuccess) { cudaGetLastError(); fail(SEERA_E_OOM, "cudaMallocHost(%zu)", n); return nullptr; }
    return p;
}
int seera_host_free_pinned(void *p) { return p ? check_cuda(cudaFreeHost(p), "cudaFreeHost") : SEERA_OK; }

int seera_cuda_memcopy_devicetodevice(void *dst, const void *src, int num_elem) {
    SEERA_ENSURE();
    if (num_elem < 0 || !dst || !src) return fail(SEERA_E_ARG, "memcopy_devicetodevice: bad argument");
    return check_cuda(cudaMemcpyAsync(dst, src, (size_t)num_elem * sizeof(float), cudaMemcpyDeviceToDevice, rt().stream),
                      "cudaMemcpyAsync d2d");
}
int seera_cuda_memset(void *ptr, int value, size_t n_bytes) {
    SEERA_ENSURE();
    if (!ptr) return fail(SEERA_E_ARG, "cuda_memset: null");
    return check_cuda(cudaMemsetAsync(ptr, value, n_bytes, rt().stream), "cudaMemsetAsync");
}

void *seera_to_device(const void *host, size_t n_bytes) {
    void *d = seera_cuda_malloc(n_bytes);
    if (!d) return nullptr;
    if (n_bytes && seera_upload(d, host, n_bytes)) { seera_cuda_free(d); return nullptr; }
    return d;
}
int seera_upload(void *dev, const void *host, size_t n_bytes) {
    SEERA_ENSURE();
    if (!dev || !host) return fail(SEERA_E_ARG, "upload: null");
    // From pageable memory the runtime stages the copy before returning, so the caller may reuse
    // `host` at once; from pinned memory the copy is asynchronous and ordered on the stream.
    return check_cuda(cudaMemcpyAsync(dev, host, n_bytes, cudaMemcpyHostToDevice, rt().stream), "cudaMemcpyAsync h2d");
}
// ---- measurement aid: hold the stream for a while so that the launches that follow queue up behind it ---------
// Events recorded around a kernel in an eagerly launched sequence otherwise also time the host's gaps between launches.
__global__ void stream_delay_kernel(long long clocks) {
    const long long t0 = clock64();
    while (clock64() - t0 < clocks) {}          // bounded by `clocks` (at most 0.1 s worth, see below)
}
int seera_stream_delay(int microseconds) {
    SEERA_ENSURE();
    if (microseconds < 0 || microseconds > 100000) return fail(SEERA_E_ARG, "stream_delay: 0..100000 microseconds");
    if (rt().capturing) return fail(SEERA_E_ARG, "stream_delay: not allowed while a graph is being captured");
    int khz = 0;
    if (cudaDeviceGetAttribute(&khz, cudaDevAttrClockRate, rt().device) != cudaSuccess || khz <= 0) { cudaGetLastError(); khz = 1500000; }
    stream_delay_kernel<<<1, 1, 0, rt().stream>>>((long long)microseconds * khz / 1000);
    SEERA_LAUNCH_CHECK("stream_delay");
    return SEERA_OK;
}

// ---- copy stream: host<->device transfers that overlap the compute stream -----------------------------------
// One extra non-blocking stream per process.  Ordering against the compute stream is explicit: each fence records an
// event at the current tail of one stream and makes the other wait for it, so "everything queued so far" is the unit.
static cudaStream_t copy_stream(int *status) {
    static cudaStream_t cs[64] = {nullptr};
    const int dev = rt().device & 63;
    if (!cs[dev]) {
        cudaError_t e = cudaStreamCreateWithFlags(&cs[dev], cudaStreamNonBlocking);
        if (e != cudaSuccess) { *status = check_cuda(e, "cudaStreamCreate(copy)"); return nullptr; }
    }
    return cs[dev];
}
static int fence(cudaStream_t from, cudaStream_t to, const char *what) {
    cudaEvent_t ev;
    if (int s = check_cuda(cudaEventCreateWithFlags(&ev, cudaEventDisableTiming), what)) return s;
    cudaError_t e = cudaEventRecord(ev, from);
    if (e == cudaSuccess) e = cudaStreamWaitEvent(to, ev, 0);
    cudaEventDestroy(ev);              // released once the recorded work has completed
    return check_cuda(e, what);
}
static int copy_guard(const char *what) {
    if (rt().capturing) return fail(SEERA_E_ARG, "%s: not allowed while a graph is being captured", what);
    return SEERA_OK;
}
int seera_copy_upload(void *dev, const void *pinned_host, size_t n_bytes) {
    SEERA_ENSURE();
    if (!dev || !pinned_host) return fail(SEERA_E_ARG, "copy_upload: null");
    if (int s = copy_guard("copy_upload")) return s;
    int st = SEERA_OK; cudaStream_t cs = copy_stream(&st); if (!cs) return st;
    return check_cuda(cudaMemcpyAsync(dev, pinned_host, n_bytes, cudaMemcpyHostToDevice, cs), "cudaMemcpyAsync h2d (copy stream)");
}
int seera_copy_download(void *pinned_host, const void *dev, size_t n_bytes) {
    SEERA_ENSURE();
    if (!dev || !pinned_host) return fail(SEERA_E_ARG, "copy_download: null");
    if (int s = copy_guard("copy_download")) return s;
    int st = SEERA_OK; cudaStream_t cs = copy_stream(&st); if (!cs) return st;
    return check_cuda(cudaMemcpyAsync(pinned_host, dev, n_bytes, cudaMemcpyDeviceToHost, cs), "cudaMemcpyAsync d2h (copy stream)");
}
int seera_copy_wait_compute(void) {
    SEERA_ENSURE();
    if (int s = copy_guard("copy_wait_compute")) return s;
    int st = SEERA_OK; cudaStream_t cs = copy_stream(&st); if (!cs) return st;
    return fence(rt().stream, cs, "copy_wait_compute");
}
int seera_compute_wait_copy(void) {
    SEERA_ENSURE();
    if (int s = copy_guard("compute_wait_copy")) return s;
    int st = SEERA_OK; cudaStream_t cs = copy_stream(&st); if (!cs) return st;
    return fence(cs, rt().stream, "compute_wait_copy");
}
int seera_copy_synchronize(void) {
    SEERA_ENSURE();
    if (int s = copy_guard("copy_synchronize")) return s;
    int st = SEERA_OK; cudaStream_t cs = copy_stream(&st); if (!cs) return st;
    return check_cuda(cudaStreamSynchronize(cs), "cudaStreamSynchronize(copy)");
}

int seera_to_host(void *host, const void *dev, size_t n_bytes) {
    SEERA_ENSURE();
    if (!dev || !host) return fail(SEERA_E_ARG, "to_host: null");
    if (rt().capturing) return fail(SEERA_E_ARG, "to_host: not allowed while a graph is being captured");
    if (int s = check_cuda(cudaMemcpyAsync(host, dev, n_bytes, cudaMemcpyDeviceToHost, rt().stream), "cudaMemcpyAsync d2h")) return s;
    return check_cuda(cudaStreamSynchronize(rt().stream), "cudaStreamSynchronize");
}

}  // extern "C"
