// Shared host/device helpers of the eddl_b200 CUDA library (sm_100a only).
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>
#include <stddef.h>
#include "eddl_b200.h"

#define EDDLB200_MAX_DEVICES 64
#define EDDLB200_NUM_SMS 148          // B200: 2 dies x 74 SMs; grids are sized in multiples of this

struct ncclComm;

namespace eb {

struct DevCtx;

// Returns the initialised context of `dev` (creating it on first use) or nullptr
// with last_error set.  Makes `dev` the current device of the calling thread.
DevCtx *ctx(int dev);
// The context of `dev` if one has been created, else nullptr; creates and allocates nothing.
DevCtx *ctx_peek(int dev);
cudaStream_t stream_of(DevCtx *c);
// An event that exists for the lifetime of the context (nothing is created when it is used): record it on the compute
// stream and make another stream wait on it to order that stream after everything enqueued so far.
cudaEvent_t handoff_event(DevCtx *c);
// Stream-ordered scratch of at least `bytes` bytes, reused by every kernel that
// runs on the device's compute stream (valid until the next scratch() call).
void *scratch(DevCtx *c, size_t bytes);
// Pinned host words + device words used to return scalars (loss, accuracy).
float *host_scalars(DevCtx *c);    // 64 floats
float *dev_scalars(DevCtx *c);     // 64 floats
ncclComm *comm_of(DevCtx *c);
int comm_nranks(DevCtx *c);
void count_launch(DevCtx *c, unsigned n = 1);
int set_error(int code, const char *fmt, ...);

// Optional per-kernel-family device timing (CUDA events on the compute stream), off by
// default.  `work` is the family's algorithmic work of this call (FLOPs or bytes).
enum ProfKind { PROF_CONV_FWD = 0, PROF_CONV_BWD_DATA, PROF_CONV_BWD_WEIGHT, PROF_BN_FWD, PROF_BN_BWD,
                PROF_ELEMENTWISE, PROF_POOL, PROF_GEMM, PROF_OPTIM, PROF_COMM, PROF_NKINDS };
bool prof_enabled(DevCtx *c);
int prof_begin(DevCtx *c, int kind, double work);        // returns the index of the record it opened
void prof_end(DevCtx *c, int record);
struct ProfScope {
    DevCtx *c; bool on; int rec = -1;
    ProfScope(DevCtx *cx, int kind, double work) : c(cx), on(prof_enabled(cx)) { if (on) rec = prof_begin(c, kind, work); }
    ~ProfScope() { if (on) prof_end(c, rec); }      // scopes nest (a conv call that first writes owed zeros): each closes its own record
};
int cuda_status(cudaError_t e, const char *what);

// Deferred zero fills.  With the option "lazy_zero" on, a fill of a large buffer with 0.0f only records the range.
// The zeros are written when an entry point READS any part of the range (lz_read), dropped when one OVERWRITES the
// whole range (lz_write), or consumed by an accumulating kernel that owns the whole range and runs its
// "destination is zero" variant instead of a read-modify-write (lz_take).  Every entry point of the library declares
// each device pointer it is given through one of the three before launching.
bool lz_any(DevCtx *c);                                                  // anything deferred on this device?
bool lz_defer(DevCtx *c, cudaStream_t st, void *p, size_t bytes);        // true = recorded, caller skips its fill
int lz_read(DevCtx *c, cudaStream_t st, const void *p, size_t bytes);
int lz_write(DevCtx *c, cudaStream_t st, const void *p, size_t bytes);
bool lz_take(DevCtx *c, cudaStream_t st, const void *p, size_t bytes, int *status);
void lz_forget(DevCtx *c, const void *p, size_t bytes);                  // the memory is being released
int lz_set_all(int on);                                                  // every device; turning it off writes every deferred fill
int bn_set_tuning(int waves, int min_items);                             // BatchNorm grid sizing knobs (0 = leave unchanged)
int launch_zero_fill(DevCtx *c, cudaStream_t st, float *p, size_t n);    // defined with the elementwise kernels

// Deferred first term of an in-place sum.  LAdd::forward is "out = 0; out += a; out += b": with the fill deferred, the first
// add is the copy out = 1*a + 1*0.  It is recorded instead of run; if the very next call is the second in-place add into the
// same buffer, one kernel computes out = s2*b + t2*(s1*a + t1*0) (12 bytes per element instead of 8 + 12).  ANY other entry
// point writes the recorded copy out first, so the record never outlives the call that follows it.
// When that second add arrives, the SUM is kept on record in turn (kind 2): if the next call is the ReLU of the sum -- the
// activation that follows LAdd in a residual block -- one kernel writes both the sum and its ReLU (16 bytes per element instead
// of 12 + 8); again any other entry point first runs what is on record.  LAdd::backward adds its delta into the (zero) deltas of
// both parents: the second such copy FROM THE SAME SOURCE joins the record (kind 3) and one kernel reads the source once.
struct PendCopy {
    bool active = false; int kind = 1;                   // 1: dst = sa*src + sb*0     2: dst = s2*src2 + t2*(sa*src + sb*0)
                                                         // 3: dst = dst2 = sa*src + sb*0   (LAdd::backward: the delta into both parents)
    float *dst = nullptr, *dst2 = nullptr; const float *src = nullptr, *src2 = nullptr;
    float sa = 0.f, sb = 0.f, s2 = 0.f, t2 = 0.f; size_t n = 0;
};
bool pend_copy_active(DevCtx *c);
PendCopy &pend_copy(DevCtx *c);
int pend_copy_flush(DevCtx *c, cudaStream_t st);                         // defined with the elementwise kernels

}  // namespace eb

namespace eb {
// Write observers.  A cache whose contents are derived from device memory (packed weight tiles, the value of a loss)
// registers the source range with watch_add and remembers the version it returns; every entry point declares what it
// writes (EB_WRITES: overwrites, EB_MODIFIES: read-modify-write, lz_take: accumulates), and a declared write that overlaps
// a watched range gives it a new version, so the cache sees that its copy is stale.  Ranges vanish when their memory is
// released.
unsigned long long watch_add(DevCtx *c, const void *p, size_t bytes);     // registers (or finds) the range; returns its version
unsigned long long watch_version(DevCtx *c, const void *p);               // 0 = not watched (any more)
bool watch_any(DevCtx *c);
void note_write(DevCtx *c, const void *p, size_t bytes);
void watch_forget(DevCtx *c, const void *p, size_t bytes);
}  // namespace eb

namespace eb {
// Loss and metric of one (target, prediction) pair, kept per device.  Net::train_batch evaluates both twice per step
// (src/net/net_api.cpp:46 and :1300 -> :534-569) on unchanged tensors: the first request computes both values with one
// read-back, the others are answered from here as long as no declared write has touched either tensor.
struct LossCache {
    bool valid = false;
    const float *y_true = nullptr, *y_pred = nullptr; int rows = 0, cols = 0;
    unsigned long long v_true = 0, v_pred = 0;
    float loss = 0.f; int hits = 0;
};
LossCache &loss_cache(DevCtx *c);
}  // namespace eb

namespace eb {
// Buffers with an averaging collective in flight on the communication stream (avg_weights_distributed runs there, bucket by
// bucket, while the compute stream goes on with the next step).  Every declared access of an entry point to such a buffer
// first makes the compute stream wait for the bucket's event, so a layer's kernels start as soon as ITS parameters have
// been averaged, not when the whole collective is done.
bool avg_any(DevCtx *c);
int avg_settle(DevCtx *c, cudaStream_t st, const void *p, size_t bytes);
}  // namespace eb

#define EB_SETTLE(p, bytes)                                                             \
    do { if ((p) && eb::avg_any(cx)) { if (int r__ = eb::avg_settle(cx, st, (p), (bytes))) return r__; } } while (0)
#define EB_READS(p, bytes)                                                              \
    do {                                                                                \
        EB_SETTLE(p, bytes);                                                            \
        if ((p) && eb::lz_any(cx)) { if (int r__ = eb::lz_read(cx, st, (p), (bytes))) return r__; } \
    } while (0)
#define EB_WRITES(p, bytes)                                                             \
    do {                                                                                \
        EB_SETTLE(p, bytes);                                                            \
        if ((p) && eb::watch_any(cx)) eb::note_write(cx, (p), (bytes));                 \
        if ((p) && eb::lz_any(cx)) { if (int r__ = eb::lz_write(cx, st, (p), (bytes))) return r__; } \
    } while (0)
// an accumulated-into destination whose deferred zeros are dealt with separately (lz_take): tell the observers only
#define EB_NOTES(p, bytes)                                                              \
    do { EB_SETTLE(p, bytes); if ((p) && eb::watch_any(cx)) eb::note_write(cx, (p), (bytes)); } while (0)
// read-modify-write of a destination: zeros owed to it are written first, and observers of the range are told
#define EB_MODIFIES(p, bytes)                                                           \
    do {                                                                                \
        EB_SETTLE(p, bytes);                                                            \
        if ((p) && eb::watch_any(cx)) eb::note_write(cx, (p), (bytes));                 \
        if ((p) && eb::lz_any(cx)) { if (int r__ = eb::lz_read(cx, st, (p), (bytes))) return r__; } \
    } while (0)

// Every entry point but eddlb200_axpby and eddlb200_relu_fwd starts by writing out a deferred "first term" of an in-place sum (see pend_copy_*).
#define EB_CTX_KEEP_PENDING(dev)                      \
    eb::DevCtx *cx = eb::ctx(dev);                    \
    if (!cx) return EDDLB200_ENOINIT;                 \
    cudaStream_t st = eb::stream_of(cx);              \
    (void)st
#define EB_CTX(dev)                                   \
    EB_CTX_KEEP_PENDING(dev);                         \
    if (eb::pend_copy_active(cx)) { if (int r__ = eb::pend_copy_flush(cx, st)) return r__; }

#define EB_LAUNCH_CHECK(what)                                         \
    do {                                                              \
        eb::count_launch(cx);                                         \
        cudaError_t e__ = cudaGetLastError();                         \
        if (e__ != cudaSuccess) return eb::cuda_status(e__, what);    \
    } while (0)

#define EB_REQUIRE(cond, what)                                                   \
    do {                                                                         \
        if (!(cond)) return eb::set_error(EDDLB200_EINVAL, "%s: %s", what, #cond); \
    } while (0)

namespace eb {

__host__ __device__ inline size_t ceil_div(size_t a, size_t b) { return (a + b - 1) / b; }

// Grid for a grid-stride elementwise kernel over `work` thread-items:
// a multiple of the SM count, at most `waves` resident waves of blocks.
inline int grid_for(size_t work_items, int block, int max_blocks_per_sm = 8) {
    size_t blocks = ceil_div(work_items, (size_t)block);
    size_t cap = (size_t)EDDLB200_NUM_SMS * max_blocks_per_sm;
    if (blocks > cap) blocks = cap;
    if (blocks < 1) blocks = 1;
    return (int)blocks;
}

__host__ __device__ inline bool aligned16(const void *p) { return (((uintptr_t)p) & 15u) == 0; }

#ifdef __CUDACC__
__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}
// Block-wide sum; every thread gets the result.  `sm` holds >= 32 floats.
__device__ __forceinline__ float block_sum(float v, float *sm) {
    const int lane = threadIdx.x & 31, w = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
    v = warp_sum(v);
    __syncthreads();
    if (lane == 0) sm[w] = v;
    __syncthreads();
    float r = (lane < nw) ? sm[lane] : 0.f;
    r = warp_sum(r);
    return r;
}
__device__ __forceinline__ float4 ldg4(const float *p) { return __ldg(reinterpret_cast<const float4 *>(p)); }
// Streaming (evict-first) loads/stores for data touched once per pass.
__device__ __forceinline__ float4 ld_stream4(const float *p) { return __ldcs(reinterpret_cast<const float4 *>(p)); }
__device__ __forceinline__ void st_stream4(float *p, float4 v) { __stcs(reinterpret_cast<float4 *>(p), v); }
#endif

}  // namespace eb
