// Device contexts, caching allocator, copies, timers.
// Replaces gpu_init / gpu_create_tensor / gpu_delete_tensor / gpu_copy_*
// (EDDL src/hardware/gpu/gpu_tensor.cu:133-233, gpu_core.cu:49-78): one context per
// device holding one compute stream, a size-bucketed free-list allocator (the
// reference does a cudaMalloc/cudaFree per tensor and its Net frees and re-creates
// every tensor on a batch-size change), a growable scratch arena and pinned words
// for scalar read-back.
#include <cstdarg>
#include <cstdio>
#include <cstring>
#include <map>
#include <mutex>
#include <unordered_map>
#include <vector>
#include "common.cuh"
#include "conv_common.cuh"

namespace eb {

struct DevCtx {
    int dev = -1;
    bool ready = false;
    cudaStream_t stream = nullptr;
    std::mutex mu;
    std::multimap<size_t, void *> free_blocks;          // rounded size -> block
    std::unordered_map<void *, size_t> live;            // block -> rounded size
    size_t bytes_in_use = 0, bytes_cached = 0;
    void *scratch_ptr = nullptr; size_t scratch_bytes = 0;
    float *h_scalars = nullptr, *d_scalars = nullptr;
    cudaEvent_t ev_start[16] = {}, ev_stop[16] = {};
    unsigned long long launches = 0;
    ncclComm *comm = nullptr; int nranks = 1, rank = 0;
    // profiling: one (start, stop) event pair per profiled call, summed at read time
    bool prof_on = false;
    struct ProfRec { int kind; double work; cudaEvent_t a, b; };
    std::vector<ProfRec> prof_recs;
    std::vector<cudaEvent_t> prof_pool;
    // deferred zero fills: start address -> bytes (disjoint ranges)
    bool lz_on = false;
    std::map<uintptr_t, size_t> lz;
    PendCopy pend;
    // write observers: start address -> (bytes, version)
    struct Watch { size_t bytes; unsigned long long version; };
    std::map<uintptr_t, Watch> watch;
    unsigned long long watch_clock = 0;
    LossCache loss;
    // staged host->device copies: a ring of (pinned host buffer, device buffer) pairs fed by a copy stream
    struct Stage { void *host = nullptr, *dev = nullptr; size_t cap = 0; cudaEvent_t landed = nullptr, consumed = nullptr; bool used = false; };
    static constexpr int kStages = 4;
    Stage stages[kStages];
    int stage_next = 0;
    cudaStream_t copy_stream = nullptr;
    cudaEvent_t ev_peer = nullptr, ev_peer_done = nullptr;
    cudaEvent_t ev_handoff = nullptr;        // created with the context: orders a caller's stream after the compute stream
    // averaging in flight on the communication stream: start address -> (bytes, event of its bucket)
    struct AvgRange { size_t bytes; cudaEvent_t done; };
    std::map<uintptr_t, AvgRange> avg_pending;
    cudaStream_t comm_stream = nullptr;
    std::vector<cudaEvent_t> avg_events;     // one per bucket, reused call after call
    cudaEvent_t ev_comm_start = nullptr;
    void *avg_bucket = nullptr; size_t avg_bucket_bytes = 0;     // packed small tensors + segment table of the asynchronous averaging
};

static DevCtx g_ctx[EDDLB200_MAX_DEVICES];
static bool g_lz_default = false;      // deferred zero fills: contexts created later start with this setting
static std::mutex g_init_mu;
static thread_local char g_err[512] = "";

int set_error(int code, const char *fmt, ...) {
    va_list ap; va_start(ap, fmt);
    vsnprintf(g_err, sizeof(g_err), fmt, ap);
    va_end(ap);
    return code;
}

int cuda_status(cudaError_t e, const char *what) {
    if (e == cudaSuccess) return 0;
    set_error((int)e, "[CUDA ERROR]: %s (%d) raised in %s", cudaGetErrorString(e), (int)e, what);
    return (int)e;
}

static int init_locked(int dev) {
    DevCtx &c = g_ctx[dev];
    if (c.ready) return 0;
    int n = 0;
    cudaError_t e = cudaGetDeviceCount(&n);
    if (e != cudaSuccess) return cuda_status(e, "cudaGetDeviceCount");
    if (dev >= n) return set_error(EDDLB200_ENOINIT, "device %d requested but only %d visible", dev, n);
    if ((e = cudaSetDevice(dev)) != cudaSuccess) return cuda_status(e, "cudaSetDevice");
    if ((e = cudaStreamCreateWithFlags(&c.stream, cudaStreamNonBlocking)) != cudaSuccess) return cuda_status(e, "cudaStreamCreate");
    if ((e = cudaMallocHost((void **)&c.h_scalars, 64 * sizeof(float))) != cudaSuccess) return cuda_status(e, "cudaMallocHost");
    if ((e = cudaMalloc((void **)&c.d_scalars, 64 * sizeof(float))) != cudaSuccess) return cuda_status(e, "cudaMalloc");
    for (int i = 0; i < 16; i++) { cudaEventCreate(&c.ev_start[i]); cudaEventCreate(&c.ev_stop[i]); }
    if ((e = cudaEventCreateWithFlags(&c.ev_handoff, cudaEventDisableTiming)) != cudaSuccess) return cuda_status(e, "cudaEventCreate");
    c.dev = dev;
    c.lz_on = g_lz_default;
    c.ready = true;
    return 0;
}

DevCtx *ctx(int dev) {
    if (dev < 0 || dev >= EDDLB200_MAX_DEVICES) { set_error(EDDLB200_ENOINIT, "device ordinal %d out of range", dev); return nullptr; }
    DevCtx &c = g_ctx[dev];
    if (!c.ready) {
        std::lock_guard<std::mutex> lk(g_init_mu);
        if (init_locked(dev) != 0) return nullptr;
    }
    if (cudaSetDevice(dev) != cudaSuccess) { set_error(EDDLB200_ENOINIT, "cudaSetDevice(%d) failed", dev); return nullptr; }
    return &c;
}

DevCtx *ctx_peek(int dev) { return (dev >= 0 && dev < EDDLB200_MAX_DEVICES && g_ctx[dev].ready) ? &g_ctx[dev] : nullptr; }
cudaStream_t stream_of(DevCtx *c) { return c->stream; }
cudaEvent_t handoff_event(DevCtx *c) { return c->ev_handoff; }
float *host_scalars(DevCtx *c) { return c->h_scalars; }
float *dev_scalars(DevCtx *c) { return c->d_scalars; }
ncclComm *comm_of(DevCtx *c) { return c->comm; }
int comm_nranks(DevCtx *c) { return c->nranks; }
void count_launch(DevCtx *c, unsigned n) { c->launches += n; }

bool prof_enabled(DevCtx *c) { return c->prof_on; }
static cudaEvent_t prof_event(DevCtx *c) {
    if (!c->prof_pool.empty()) { cudaEvent_t e = c->prof_pool.back(); c->prof_pool.pop_back(); return e; }
    cudaEvent_t e; cudaEventCreate(&e); return e;
}
int prof_begin(DevCtx *c, int kind, double work) {
    DevCtx::ProfRec r{kind, work, prof_event(c), prof_event(c)};
    cudaEventRecord(r.a, c->stream);
    c->prof_recs.push_back(r);
    return (int)c->prof_recs.size() - 1;
}
void prof_end(DevCtx *c, int record) {
    if (record >= 0 && record < (int)c->prof_recs.size()) cudaEventRecord(c->prof_recs[record].b, c->stream);
}

void set_comm(DevCtx *c, ncclComm *comm, int nranks, int rank) { c->comm = comm; c->nranks = nranks; c->rank = rank; }
int comm_rank(DevCtx *c) { return c->rank; }

void *scratch(DevCtx *c, size_t bytes) {
    if (bytes <= c->scratch_bytes) return c->scratch_ptr;
    // Work already enqueued may still read the old arena: drain before replacing it.
    cudaStreamSynchronize(c->stream);
    if (c->scratch_ptr) cudaFree(c->scratch_ptr);
    size_t want = bytes < (size_t(8) << 20) ? (size_t(8) << 20) : bytes + bytes / 2;
    c->scratch_ptr = nullptr; c->scratch_bytes = 0;
    if (cudaMalloc(&c->scratch_ptr, want) != cudaSuccess) { set_error(cudaErrorMemoryAllocation, "scratch arena of %zu bytes", want); return nullptr; }
    c->scratch_bytes = want;
    return c->scratch_ptr;
}

// ---- write observers ----------------------------------------------------------------------------------
LossCache &loss_cache(DevCtx *c) { return c->loss; }

// ---- averaging in flight ------------------------------------------------------------------------------
bool avg_any(DevCtx *c) { return !c->avg_pending.empty(); }
int avg_settle(DevCtx *c, cudaStream_t st, const void *p, size_t bytes) {
    if (c->avg_pending.empty() || !bytes) return 0;
    const uintptr_t lo = (uintptr_t)p, hi = lo + bytes;
    auto it = c->avg_pending.upper_bound(lo);
    if (it != c->avg_pending.begin()) { auto prev = std::prev(it); if (prev->first + prev->second.bytes > lo) it = prev; }
    while (it != c->avg_pending.end() && it->first < hi) {
        cudaError_t e = cudaStreamWaitEvent(st, it->second.done, 0);
        if (e != cudaSuccess) return cuda_status(e, "averaging(wait for bucket)");
        it = c->avg_pending.erase(it);
    }
    return 0;
}
// used by the collectives (comm.cu)
cudaStream_t comm_stream_of(DevCtx *c) {
    if (!c->comm_stream && cudaStreamCreateWithFlags(&c->comm_stream, cudaStreamNonBlocking) != cudaSuccess) c->comm_stream = nullptr;
    return c->comm_stream;
}
cudaEvent_t avg_event(DevCtx *c, size_t index) {
    while (c->avg_events.size() <= index) {
        cudaEvent_t e = nullptr;
        if (cudaEventCreateWithFlags(&e, cudaEventDisableTiming) != cudaSuccess) return nullptr;
        c->avg_events.push_back(e);
    }
    return c->avg_events[index];
}
cudaEvent_t comm_start_event(DevCtx *c) {
    if (!c->ev_comm_start && cudaEventCreateWithFlags(&c->ev_comm_start, cudaEventDisableTiming) != cudaSuccess) c->ev_comm_start = nullptr;
    return c->ev_comm_start;
}
void avg_register(DevCtx *c, const void *p, size_t bytes, cudaEvent_t done) { c->avg_pending[(uintptr_t)p] = DevCtx::AvgRange{bytes, done}; }
// persistent buffer of the asynchronous averaging (the shared scratch arena may be re-carved by compute kernels meanwhile)
void *avg_buffer(DevCtx *c, size_t bytes) {
    if (bytes <= c->avg_bucket_bytes) return c->avg_bucket;
    if (c->comm_stream) cudaStreamSynchronize(c->comm_stream);
    if (c->avg_bucket) cudaFree(c->avg_bucket);
    c->avg_bucket = nullptr; c->avg_bucket_bytes = 0;
    if (cudaMalloc(&c->avg_bucket, bytes + bytes / 4) != cudaSuccess) { cudaGetLastError(); return nullptr; }
    c->avg_bucket_bytes = bytes + bytes / 4;
    return c->avg_bucket;
}
bool watch_any(DevCtx *c) { return !c->watch.empty(); }
template <typename V>
static void watch_visit(DevCtx *c, const void *p, size_t bytes, V visit) {
    if (c->watch.empty() || !bytes) return;
    const uintptr_t lo = (uintptr_t)p, hi = lo + bytes;
    // registered ranges are kept disjoint (watch_add), so at most one range starting below lo can reach into [lo, hi)
    auto it = c->watch.lower_bound(lo);
    if (it != c->watch.begin()) { auto prev = std::prev(it); if (prev->first + prev->second.bytes > lo) visit(prev); }
    for (; it != c->watch.end() && it->first < hi; ++it) visit(it);
}
unsigned long long watch_add(DevCtx *c, const void *p, size_t bytes) {
    auto it = c->watch.find((uintptr_t)p);
    if (it != c->watch.end() && it->second.bytes >= bytes) return it->second.version;
    // a new range, or one that grew: drop whatever it overlaps (those observers then read version 0 = stale, which is safe)
    std::vector<uintptr_t> gone;
    watch_visit(c, p, bytes, [&](std::map<uintptr_t, DevCtx::Watch>::iterator w) { gone.push_back(w->first); });
    for (uintptr_t k : gone) c->watch.erase(k);
    const unsigned long long v = ++c->watch_clock;
    c->watch[(uintptr_t)p] = DevCtx::Watch{bytes, v};
    return v;
}
unsigned long long watch_version(DevCtx *c, const void *p) {
    auto it = c->watch.find((uintptr_t)p);
    return it == c->watch.end() ? 0ull : it->second.version;
}
void note_write(DevCtx *c, const void *p, size_t bytes) {
    watch_visit(c, p, bytes, [&](std::map<uintptr_t, DevCtx::Watch>::iterator it) { it->second.version = ++c->watch_clock; });
}
void watch_forget(DevCtx *c, const void *p, size_t bytes) {
    if (c->watch.empty() || !bytes) return;
    std::vector<uintptr_t> gone;
    watch_visit(c, p, bytes, [&](std::map<uintptr_t, DevCtx::Watch>::iterator it) { gone.push_back(it->first); });
    for (uintptr_t k : gone) c->watch.erase(k);
}

// ---- deferred zero fills ------------------------------------------------------------------------------
constexpr size_t kLazyZeroMinBytes = size_t(256) << 10;      // smaller fills are cheaper to run (batched) than to track

// totals over the process, printed at exit when EDDL_B200_LZ_STATS is set
static struct LzStats { unsigned long long deferred = 0, taken = 0, dropped = 0, written = 0; double written_bytes = 0, deferred_bytes = 0;
    ~LzStats() { if (getenv("EDDL_B200_LZ_STATS")) fprintf(stderr, "[lazy_zero] deferred %llu (%.1f MB) taken %llu dropped %llu written %llu (%.1f MB)\n", deferred, deferred_bytes / 1e6, taken, dropped, written, written_bytes / 1e6); } } g_lzs;
bool lz_any(DevCtx *c) { return !c->lz.empty(); }
bool pend_copy_active(DevCtx *c) { return c->pend.active; }
PendCopy &pend_copy(DevCtx *c) { return c->pend; }

// Visit every deferred range that overlaps [p, p + bytes): `covered` tells whether the range lies inside it.
// The visitor may not touch the map; visited ranges are erased afterwards.
template <typename V>
static int lz_visit(DevCtx *c, const void *p, size_t bytes, V visit) {
    const uintptr_t lo = (uintptr_t)p, hi = lo + bytes;
    auto it = c->lz.upper_bound(lo);
    if (it != c->lz.begin()) { auto prev = std::prev(it); if (prev->first + prev->second > lo) it = prev; }
    int status = 0;
    while (it != c->lz.end() && it->first < hi) {
        const bool covered = it->first >= lo && it->first + it->second <= hi;
        if (!status) status = visit(it->first, it->second, covered);
        it = c->lz.erase(it);
    }
    return status;
}

int lz_read(DevCtx *c, cudaStream_t st, const void *p, size_t bytes) {
    if (c->lz.empty() || !bytes) return 0;
    return lz_visit(c, p, bytes, [&](uintptr_t a, size_t n, bool) { g_lzs.written++; g_lzs.written_bytes += n; return launch_zero_fill(c, st, (float *)a, n / sizeof(float)); });
}
int lz_write(DevCtx *c, cudaStream_t st, const void *p, size_t bytes) {
    if (c->lz.empty() || !bytes) return 0;
    return lz_visit(c, p, bytes, [&](uintptr_t a, size_t n, bool covered) { if (covered) g_lzs.dropped++; else { g_lzs.written++; g_lzs.written_bytes += n; } return covered ? 0 : launch_zero_fill(c, st, (float *)a, n / sizeof(float)); });
}
bool lz_take(DevCtx *c, cudaStream_t st, const void *p, size_t bytes, int *status) {
    *status = 0;
    if (!c->watch.empty()) note_write(c, p, bytes);       // the caller is about to accumulate into [p, p + bytes)
    if (c->lz.empty() || !bytes) return false;
    auto it = c->lz.find((uintptr_t)p);
    if (it != c->lz.end() && it->second == bytes) { c->lz.erase(it); g_lzs.taken++; return true; }
    *status = lz_read(c, st, p, bytes);
    return false;
}
bool lz_defer(DevCtx *c, cudaStream_t st, void *p, size_t bytes) {
    if (!c->lz_on || bytes < kLazyZeroMinBytes || (bytes % sizeof(float))) return false;
    if (!c->watch.empty()) note_write(c, p, bytes);       // a recorded fill is a write all the same
    // older deferred fills inside the new range are superseded; ones that stick out are written now
    if (lz_write(c, st, p, bytes) != 0) return false;
    c->lz[(uintptr_t)p] = bytes;
    g_lzs.deferred++; g_lzs.deferred_bytes += bytes;
    return true;
}
void lz_forget(DevCtx *c, const void *p, size_t bytes) {
    if (c->lz.empty()) return;
    lz_visit(c, p, bytes, [](uintptr_t, size_t, bool) { return 0; });
}
int lz_set_all(int on) {
    g_lz_default = on != 0;
    int status = 0;
    for (int d = 0; d < EDDLB200_MAX_DEVICES; d++) {
        DevCtx *c = &g_ctx[d];
        if (!c->ready) continue;
        c->lz_on = g_lz_default;
        if (!on && !c->lz.empty()) {
            if (cudaSetDevice(d) != cudaSuccess) { status = set_error(EDDLB200_ENOINIT, "cudaSetDevice(%d) failed", d); continue; }
            for (auto &kv : c->lz) if (!status) status = launch_zero_fill(c, c->stream, (float *)kv.first, kv.second / sizeof(float));
            c->lz.clear();
        }
    }
    return status;
}

static size_t round_size(size_t b) {
    if (b < 512) return 512;
    if (b < (size_t(1) << 20)) return (b + 511) & ~size_t(511);
    return (b + (size_t(1) << 20) - 1) & ~((size_t(1) << 20) - 1);
}

}  // namespace eb

using namespace eb;

extern "C" {

const char *eddlb200_last_error(void) { return g_err; }
int eddlb200_version(void) { return 100; }

int eddlb200_device_count(int *n) {
    if (!n) return set_error(EDDLB200_EINVAL, "device_count: null");
    cudaError_t e = cudaGetDeviceCount(n);
    if (e != cudaSuccess) { *n = 0; return cuda_status(e, "cudaGetDeviceCount"); }
    return 0;
}

int eddlb200_init(int dev) { return ctx(dev) ? 0 : EDDLB200_ENOINIT; }

int eddlb200_alloc(int dev, size_t bytes, void **out) {
    EB_CTX(dev);
    if (!out) return set_error(EDDLB200_EINVAL, "alloc: null out");
    size_t r = round_size(bytes);
    std::lock_guard<std::mutex> lk(cx->mu);
    auto it = cx->free_blocks.lower_bound(r);
    // Reuse a cached block when it wastes at most 25% (exact match for small ones).
    if (it != cx->free_blocks.end() && it->first <= r + r / 4) {
        *out = it->second; size_t sz = it->first;
        cx->free_blocks.erase(it);
        cx->live[*out] = sz; cx->bytes_cached -= sz; cx->bytes_in_use += sz;
        return 0;
    }
    void *p = nullptr;
    cudaError_t e = cudaMalloc(&p, r);
    if (e != cudaSuccess) {
        // Give cached blocks back to the driver and retry once.
        cudaGetLastError();
        cudaStreamSynchronize(cx->stream);
        for (auto &kv : cx->free_blocks) cudaFree(kv.second);
        cx->free_blocks.clear(); cx->bytes_cached = 0;
        e = cudaMalloc(&p, r);
        if (e != cudaSuccess) return cuda_status(e, "gpu_create_tensor");
    }
    cx->live[p] = r; cx->bytes_in_use += r;
    *out = p;
    return 0;
}

int eddlb200_free(int dev, void *p) {
    EB_CTX(dev);
    if (!p) return 0;
    std::lock_guard<std::mutex> lk(cx->mu);
    auto it = cx->live.find(p);
    if (it == cx->live.end()) return set_error(EDDLB200_EINVAL, "free: pointer %p was not allocated by this library on device %d", p, dev);
    size_t sz = it->second;
    cx->live.erase(it);
    cx->bytes_in_use -= sz;
    EB_SETTLE(p, sz);           // a block handed out again must not still be the operand of a collective
    lz_forget(cx, p, sz);
    watch_forget(cx, p, sz);
    // All work of this library runs on one stream per device, so a block handed out
    // again is only touched by work ordered after everything that used it before.
    cx->free_blocks.emplace(sz, p); cx->bytes_cached += sz;
    return 0;
}

int eddlb200_mem_info(int dev, size_t *in_use, size_t *cached) {
    EB_CTX(dev);
    std::lock_guard<std::mutex> lk(cx->mu);
    if (in_use) *in_use = cx->bytes_in_use;
    if (cached) *cached = cx->bytes_cached;
    return 0;
}

int eddlb200_memcpy_h2d(int dev, void *dst, const void *src, size_t bytes) {
    EB_CTX(dev);
    if (bytes == 0) return 0;
    EB_WRITES(dst, bytes);
    cudaError_t e = cudaMemcpyAsync(dst, src, bytes, cudaMemcpyHostToDevice, st);
    if (e == cudaSuccess) e = cudaStreamSynchronize(st);
    return cuda_status(e, "gpu_copy_to_gpu");
}

int eddlb200_memcpy_h2d_async(int dev, void *dst, const void *src, size_t bytes) {
    EB_CTX(dev);
    if (bytes == 0) return 0;
    EB_WRITES(dst, bytes);
    return cuda_status(cudaMemcpyAsync(dst, src, bytes, cudaMemcpyHostToDevice, st), "memcpy_h2d_async");
}

int eddlb200_memcpy_h2d_staged(int dev, void *dst, const void *src, size_t bytes) {
    EB_CTX(dev);
    if (bytes == 0) return 0;
    if (!dst || !src) return set_error(EDDLB200_EINVAL, "memcpy_h2d_staged: null pointer");
    cudaError_t e = cudaSuccess;
    if (!cx->copy_stream && (e = cudaStreamCreateWithFlags(&cx->copy_stream, cudaStreamNonBlocking)) != cudaSuccess) return cuda_status(e, "memcpy_h2d_staged(stream)");
    DevCtx::Stage &sg = cx->stages[cx->stage_next];
    cx->stage_next = (cx->stage_next + 1) % DevCtx::kStages;
    if (!sg.landed) {
        if ((e = cudaEventCreateWithFlags(&sg.landed, cudaEventDisableTiming)) != cudaSuccess ||
            (e = cudaEventCreateWithFlags(&sg.consumed, cudaEventDisableTiming)) != cudaSuccess) return cuda_status(e, "memcpy_h2d_staged(event)");
    }
    // the pair is free again once the device-side copy of its previous use has run
    if (sg.used && (e = cudaEventSynchronize(sg.consumed)) != cudaSuccess) return cuda_status(e, "memcpy_h2d_staged(wait)");
    if (sg.cap < bytes) {
        if (sg.host) cudaFreeHost(sg.host);
        if (sg.dev) cudaFree(sg.dev);
        sg.host = sg.dev = nullptr; sg.cap = 0;
        const size_t want = (bytes + (size_t(1) << 20) - 1) & ~((size_t(1) << 20) - 1);
        if ((e = cudaMallocHost(&sg.host, want)) != cudaSuccess || (e = cudaMalloc(&sg.dev, want)) != cudaSuccess) {
            if (sg.host) cudaFreeHost(sg.host);
            sg.host = nullptr;
            return cuda_status(e, "memcpy_h2d_staged(buffers)");
        }
        sg.cap = want;
    }
    memcpy(sg.host, src, bytes);                 // from here on the caller's buffer is no longer needed
    if ((e = cudaMemcpyAsync(sg.dev, sg.host, bytes, cudaMemcpyHostToDevice, cx->copy_stream)) != cudaSuccess) return cuda_status(e, "memcpy_h2d_staged(h2d)");
    if ((e = cudaEventRecord(sg.landed, cx->copy_stream)) != cudaSuccess) return cuda_status(e, "memcpy_h2d_staged(record)");
    if ((e = cudaStreamWaitEvent(st, sg.landed, 0)) != cudaSuccess) return cuda_status(e, "memcpy_h2d_staged(wait event)");
    EB_WRITES(dst, bytes);
    if ((e = cudaMemcpyAsync(dst, sg.dev, bytes, cudaMemcpyDeviceToDevice, st)) != cudaSuccess) return cuda_status(e, "memcpy_h2d_staged(d2d)");
    sg.used = true;
    return cuda_status(cudaEventRecord(sg.consumed, st), "memcpy_h2d_staged(record)");
}

int eddlb200_memcpy_d2h(int dev, void *dst, const void *src, size_t bytes) {
    EB_CTX(dev);
    if (bytes == 0) return 0;
    EB_READS(src, bytes);
    cudaError_t e = cudaMemcpyAsync(dst, src, bytes, cudaMemcpyDeviceToHost, st);
    if (e == cudaSuccess) e = cudaStreamSynchronize(st);
    return cuda_status(e, "gpu_copy_from_gpu");
}

int eddlb200_memcpy_d2d(int dev, void *dst, const void *src, size_t bytes) {
    EB_CTX(dev);
    if (bytes == 0) return 0;
    EB_READS(src, bytes);
    EB_WRITES(dst, bytes);
    return cuda_status(cudaMemcpyAsync(dst, src, bytes, cudaMemcpyDeviceToDevice, st), "gpu_copy_gpu");
}

static cudaEvent_t peer_event(cudaEvent_t &slot) {
    if (!slot && cudaEventCreateWithFlags(&slot, cudaEventDisableTiming) != cudaSuccess) slot = nullptr;
    return slot;
}

// Device code outside this library is about to write (or has written) [p, p + bytes): everything the library still owes
// the range is written first (deferred zero fills, a pending copy, an average in flight), and whatever the library caches
// about its contents (packed weight images, the loss / metric pair) is invalidated.
int eddlb200_notify_write(int dev, void *p, size_t bytes) {
    EB_CTX(dev);
    if (!p || !bytes) return 0;
    EB_MODIFIES(p, bytes);
    return 0;
}

int eddlb200_memcpy_peer(int dst_dev, void *dst, int src_dev, const void *src, size_t bytes) {
    if (dst_dev == src_dev) return eddlb200_memcpy_d2d(dst_dev, dst, src, bytes);
    if (bytes == 0) return 0;
    if (!dst || !src) return set_error(EDDLB200_EINVAL, "memcpy_peer: null pointer");
    DevCtx *cd = ctx(dst_dev);
    if (!cd) return EDDLB200_ENOINIT;
    cudaEvent_t ready = peer_event(cd->ev_peer);
    if (!ready) return set_error(EDDLB200_ENOINIT, "memcpy_peer: cannot create an event on device %d", dst_dev);
    {
        // what the destination's stream has enqueued so far may still use dst: the copy waits for it
        DevCtx *cx = cd; cudaStream_t st = stream_of(cd);
        if (pend_copy_active(cx)) { if (int r = pend_copy_flush(cx, st)) return r; }
        EB_WRITES(dst, bytes);
        cudaError_t e = cudaEventRecord(ready, st);
        if (e != cudaSuccess) return cuda_status(e, "memcpy_peer(record)");
    }
    EB_CTX(src_dev);                              // makes src_dev current; the copy runs on the source device's stream
    EB_READS(src, bytes);
    cudaEvent_t done = peer_event(cx->ev_peer_done);
    if (!done) return set_error(EDDLB200_ENOINIT, "memcpy_peer: cannot create an event on device %d", src_dev);
    cudaError_t e = cudaStreamWaitEvent(st, ready, 0);
    if (e == cudaSuccess) e = cudaMemcpyPeerAsync(dst, dst_dev, src, src_dev, bytes, st);
    if (e == cudaSuccess) e = cudaEventRecord(done, st);
    if (e != cudaSuccess) return cuda_status(e, "memcpy_peer");
    // later work on the destination's stream is ordered after the copy
    return cuda_status(cudaStreamWaitEvent(stream_of(cd), done, 0), "memcpy_peer(order)");
}

int eddlb200_host_alloc(size_t bytes, void **out) {
    if (!out) return set_error(EDDLB200_EINVAL, "host_alloc: null out");
    return cuda_status(cudaMallocHost(out, bytes ? bytes : 1), "cudaMallocHost");
}
int eddlb200_host_free(void *p) { return p ? cuda_status(cudaFreeHost(p), "cudaFreeHost") : 0; }

int eddlb200_stream(int dev, void **s) {
    EB_CTX(dev);
    if (!s) return set_error(EDDLB200_EINVAL, "stream: null out");
    *s = (void *)st;
    return 0;
}

int eddlb200_sync(int dev) {
    EB_CTX(dev);
    if (int r = cuda_status(cudaStreamSynchronize(st), "eddlb200_sync")) return r;
    if (cx->comm_stream) { if (int r = cuda_status(cudaStreamSynchronize(cx->comm_stream), "eddlb200_sync(communication stream)")) return r; cx->avg_pending.clear(); }
    int flag = 0;
    if (int r = conv_tc_status(dev, st, &flag)) return cuda_status((cudaError_t)r, "eddlb200_sync");
    if (flag) return set_error(EDDLB200_ETIMEOUT, "a tensor-core convolution kernel gave up waiting on a pipeline barrier (site %d, warp %d, variant 0x%x)", flag & 0xff, (flag >> 8) & 0xff, flag >> 16);
    return 0;
}

int eddlb200_timer_start(int dev, int slot) {
    EB_CTX(dev);
    if (slot < 0 || slot >= 16) return set_error(EDDLB200_EINVAL, "timer slot %d", slot);
    return cuda_status(cudaEventRecord(cx->ev_start[slot], st), "timer_start");
}
int eddlb200_timer_stop(int dev, int slot) {
    EB_CTX(dev);
    if (slot < 0 || slot >= 16) return set_error(EDDLB200_EINVAL, "timer slot %d", slot);
    return cuda_status(cudaEventRecord(cx->ev_stop[slot], st), "timer_stop");
}
int eddlb200_timer_elapsed_ms(int dev, int slot, float *ms) {
    EB_CTX(dev);
    if (slot < 0 || slot >= 16 || !ms) return set_error(EDDLB200_EINVAL, "timer slot %d", slot);
    cudaError_t e = cudaEventSynchronize(cx->ev_stop[slot]);
    if (e == cudaSuccess) e = cudaEventElapsedTime(ms, cx->ev_start[slot], cx->ev_stop[slot]);
    return cuda_status(e, "timer_elapsed");
}

int eddlb200_profile_enable(int dev, int on) {
    EB_CTX(dev);
    cx->prof_on = on != 0;
    return 0;
}

int eddlb200_profile_read(int dev, int kind, unsigned long long *calls, double *total_ms, double *total_work) {
    EB_CTX(dev);
    if (kind < 0 || kind >= PROF_NKINDS) return set_error(EDDLB200_EINVAL, "profile_read: kind %d", kind);
    cudaError_t e = cudaStreamSynchronize(st);
    if (e != cudaSuccess) return cuda_status(e, "profile_read");
    unsigned long long n = 0; double ms = 0, work = 0;
    for (auto &r : cx->prof_recs) {
        if (r.kind != kind) continue;
        float t = 0.f;
        if (cudaEventElapsedTime(&t, r.a, r.b) == cudaSuccess) { ms += t; work += r.work; n++; }
        else cudaGetLastError();       // a record that was never closed: do not leave the error for the next launch check
    }
    if (calls) *calls = n; if (total_ms) *total_ms = ms; if (total_work) *total_work = work;
    return 0;
}

int eddlb200_profile_records(int dev, int kind, double *ms, double *work, int capacity, int *count) {
    EB_CTX(dev);
    if (kind < 0 || kind >= PROF_NKINDS || !count) return set_error(EDDLB200_EINVAL, "profile_records: bad argument");
    cudaError_t e = cudaStreamSynchronize(st);
    if (e != cudaSuccess) return cuda_status(e, "profile_records");
    int n = 0;
    for (auto &r : cx->prof_recs) {
        if (r.kind != kind) continue;
        float t = 0.f;
        if (cudaEventElapsedTime(&t, r.a, r.b) != cudaSuccess) { cudaGetLastError(); continue; }
        if (n < capacity && ms && work) { ms[n] = t; work[n] = r.work; }
        n++;
    }
    *count = n;
    return 0;
}

int eddlb200_profile_reset(int dev) {
    EB_CTX(dev);
    cudaStreamSynchronize(st);
    for (auto &r : cx->prof_recs) { cx->prof_pool.push_back(r.a); cx->prof_pool.push_back(r.b); }
    cx->prof_recs.clear();
    return 0;
}

int eddlb200_launch_count(int dev, unsigned long long *n) {
    EB_CTX_KEEP_PENDING(dev);       // a pure counter read: it does not touch device memory
    if (!n) return set_error(EDDLB200_EINVAL, "launch_count: null");
    *n = cx->launches;
    return 0;
}

}  // extern "C"
