// Cross-replica averaging over NVLink / NVSwitch through NCCL, one process per GPU.
// Replaces Net::sync_weights (EDDL src/net/net_func.cpp:111-127), which copies every
// parameter of every replica to the host, adds them there, multiplies by 1.0f/N and copies
// the result back to every GPU, one tensor at a time with blocking copies.  Here the sum is
// an in-place ncclAllReduce on the device's compute stream and the 1.0f/N multiply is a
// kernel of this library (fused into the SGD step for gradient averaging).  Many small
// tensors are packed into one contiguous bucket so the collective is sized for launch
// latency, not for tensor count.
#include <nccl.h>
#include <chrono>
#include <cstring>
#include <thread>
#include <vector>
#include "common.cuh"

namespace eb {
void set_comm(DevCtx *c, ncclComm *comm, int nranks, int rank);
int comm_rank(DevCtx *c);
cudaStream_t comm_stream_of(DevCtx *c);
cudaEvent_t avg_event(DevCtx *c, size_t index);
cudaEvent_t comm_start_event(DevCtx *c);
void avg_register(DevCtx *c, const void *p, size_t bytes, cudaEvent_t done);
void *avg_buffer(DevCtx *c, size_t bytes);
}

namespace {

using namespace eb;
constexpr int kBlock = 256;

int nccl_status(ncclResult_t r, const char *what) {
    if (r == ncclSuccess) return 0;
    return set_error(EDDLB200_ENCCL, "[NCCL ERROR]: %s in %s", ncclGetErrorString(r), what);
}

__global__ void __launch_bounds__(kBlock) scale_kernel(float *a, float v, size_t n4, size_t n) {
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    for (size_t j = i; j < n4; j += stride) {
        float4 x = *reinterpret_cast<float4 *>(a + 4 * j);
        x.x = __fmul_rn(x.x, v); x.y = __fmul_rn(x.y, v); x.z = __fmul_rn(x.z, v); x.w = __fmul_rn(x.w, v);
        *reinterpret_cast<float4 *>(a + 4 * j) = x;
    }
    for (size_t j = 4 * n4 + i; j < n; j += stride) a[j] = __fmul_rn(a[j], v);
}

// g <- g * inv_n ; m = lr*g + mu*m ; p -= m     (one pass, 20 B/param + the write of g)
__global__ void __launch_bounds__(kBlock) avg_sgd_kernel(float *p, float *g, float *m, float inv_n, float lr, float mu, size_t n) {
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    for (size_t j = (size_t)blockIdx.x * blockDim.x + threadIdx.x; j < n; j += stride) {
        const float gj = __fmul_rn(g[j], inv_n);
        const float mj = __fadd_rn(__fmul_rn(lr, gj), __fmul_rn(mu, m[j]));
        g[j] = gj; m[j] = mj;
        p[j] = __fadd_rn(__fmul_rn(1.0f, p[j]), __fmul_rn(-1.0f, mj));
    }
}

struct Seg { float *ptr; unsigned long long n, bucket_off; };

// pack: bucket[off+i] = t[i]      unpack: t[i] = bucket[off+i] * scale
template <bool UNPACK>
__global__ void __launch_bounds__(kBlock) bucket_kernel(const Seg *__restrict__ segs, int nseg, float *bucket, float scale) {
    for (int s = blockIdx.y; s < nseg; s += gridDim.y) {
        const Seg sg = segs[s];
        for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < sg.n; i += (size_t)gridDim.x * blockDim.x) {
            if (UNPACK) sg.ptr[i] = __fmul_rn(bucket[sg.bucket_off + i], scale);
            else bucket[sg.bucket_off + i] = sg.ptr[i];
        }
    }
}

// bucket[off + i] = t[i] for the packed segments of a bucket (in-place ones, bucket_off == ~0, are left alone)
__global__ void __launch_bounds__(kBlock) bucket_pack_kernel(const Seg *__restrict__ segs, int nseg, float *__restrict__ bucket) {
    for (int s = blockIdx.y; s < nseg; s += gridDim.y) {
        const Seg sg = segs[s];
        if (sg.bucket_off == ~0ull) continue;
        for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < sg.n; i += (size_t)gridDim.x * blockDim.x) bucket[sg.bucket_off + i] = sg.ptr[i];
    }
}

// Segments of one bucket after its all-reduce: packed ones are copied back times `scale`, the others (reduced in place)
// are multiplied where they lie.  bucket_off == ~0 marks an in-place segment.
__global__ void __launch_bounds__(kBlock) bucket_finish_kernel(const Seg *__restrict__ segs, int nseg, const float *__restrict__ bucket, float scale) {
    for (int s = blockIdx.y; s < nseg; s += gridDim.y) {
        const Seg sg = segs[s];
        const bool packed = sg.bucket_off != ~0ull;
        for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < sg.n; i += (size_t)gridDim.x * blockDim.x)
            sg.ptr[i] = __fmul_rn(packed ? bucket[sg.bucket_off + i] : sg.ptr[i], scale);
    }
}

int launch_scale(DevCtx *cx, cudaStream_t st, float *buf, float v, size_t n) {
    const bool vec = aligned16(buf);
    const size_t n4 = vec ? n / 4 : 0;
    scale_kernel<<<grid_for(vec ? (n4 ? n4 : 1) : n, kBlock), kBlock, 0, st>>>(buf, v, n4, n);
    EB_LAUNCH_CHECK("allreduce_avg(scale)");
    return 0;
}

}  // namespace

using namespace eb;

extern "C" {

int eddlb200_comm_unique_id(void *id128) {
    if (!id128) return set_error(EDDLB200_EINVAL, "comm_unique_id: null");
    static_assert(sizeof(ncclUniqueId) == 128, "ncclUniqueId is 128 bytes");
    ncclUniqueId id;
    if (int r = nccl_status(ncclGetUniqueId(&id), "ncclGetUniqueId")) return r;
    memcpy(id128, &id, sizeof(id));
    return 0;
}

int eddlb200_comm_init_rank(int dev, int nranks, int rank, const void *id128) {
    EB_CTX(dev);
    EB_REQUIRE(id128 && nranks >= 1 && rank >= 0 && rank < nranks, "comm_init_rank");
    if (comm_of(cx)) return set_error(EDDLB200_EINVAL, "comm_init_rank: device %d already has a communicator", dev);
    ncclUniqueId id;
    memcpy(&id, id128, sizeof(id));
    ncclComm_t comm = nullptr;
    if (int r = nccl_status(ncclCommInitRank(&comm, nranks, id, rank), "ncclCommInitRank")) return r;
    set_comm(cx, comm, nranks, rank);
    return 0;
}

int eddlb200_comm_destroy(int dev) {
    EB_CTX(dev);
    ncclComm_t comm = comm_of(cx);
    if (!comm) return 0;
    cudaStreamSynchronize(st);
    if (cudaStream_t cs = comm_stream_of(cx)) cudaStreamSynchronize(cs);
    ncclResult_t r = ncclCommDestroy(comm);
    set_comm(cx, nullptr, 1, 0);
    return nccl_status(r, "ncclCommDestroy");
}

int eddlb200_comm_info(int dev, int *nranks, int *rank) {
    EB_CTX(dev);
    if (nranks) *nranks = comm_nranks(cx);
    if (rank) *rank = comm_rank(cx);
    return 0;
}

int eddlb200_allreduce_avg(int dev, float *buf, size_t n) {
    EB_CTX(dev);
    if (n == 0) return 0;
    EB_REQUIRE(buf, "allreduce_avg");
    EB_MODIFIES(buf, n * sizeof(float));
    ProfScope prof(cx, PROF_COMM, 4.0 * n);
    const int N = comm_nranks(cx);
    if (comm_of(cx)) {
        if (int r = nccl_status(ncclAllReduce(buf, buf, n, ncclFloat, ncclSum, comm_of(cx), st), "ncclAllReduce")) return r;
        count_launch(cx);
    }
    return launch_scale(cx, st, buf, 1.0f / N, n);      // acc *= (1.0f / N), as Tensor::div_ does
}

int eddlb200_allreduce_avg_multi(int dev, float *const *bufs, const size_t *sizes, int ntensors) {
    EB_CTX(dev);
    EB_REQUIRE(ntensors >= 0 && (ntensors == 0 || (bufs && sizes)), "allreduce_avg_multi");
    std::vector<Seg> segs;
    size_t total = 0, largest = 0;
    for (int i = 0; i < ntensors; i++) {
        if (!sizes[i]) continue;
        EB_REQUIRE(bufs[i], "allreduce_avg_multi");
        EB_MODIFIES(bufs[i], sizes[i] * sizeof(float));
        segs.push_back(Seg{bufs[i], (unsigned long long)sizes[i], (unsigned long long)total});
        total += (sizes[i] + 3) & ~size_t(3);
        if (sizes[i] > largest) largest = sizes[i];
    }
    if (segs.empty()) return 0;
    ProfScope prof(cx, PROF_COMM, 4.0 * total);
    const size_t seg_bytes = (segs.size() * sizeof(Seg) + 255) & ~size_t(255);
    char *ws = (char *)scratch(cx, seg_bytes + total * sizeof(float));
    if (!ws) return cudaErrorMemoryAllocation;
    float *bucket = (float *)(ws + seg_bytes);
    cudaError_t e = cudaMemcpyAsync(ws, segs.data(), segs.size() * sizeof(Seg), cudaMemcpyHostToDevice, st);
    if (e != cudaSuccess) return cuda_status(e, "allreduce_avg_multi(table)");
    int gy = (int)segs.size(); if (gy > 1024) gy = 1024;
    int gx = (int)ceil_div(largest, (size_t)kBlock * 8); if (gx < 1) gx = 1; if (gx > 64) gx = 64;
    dim3 grid(gx, gy);
    bucket_kernel<false><<<grid, kBlock, 0, st>>>((const Seg *)ws, (int)segs.size(), bucket, 1.f);
    EB_LAUNCH_CHECK("allreduce_avg_multi(pack)");
    const int N = comm_nranks(cx);
    if (comm_of(cx)) {
        if (int r = nccl_status(ncclAllReduce(bucket, bucket, total, ncclFloat, ncclSum, comm_of(cx), st), "ncclAllReduce")) return r;
        count_launch(cx);
    }
    bucket_kernel<true><<<grid, kBlock, 0, st>>>((const Seg *)ws, (int)segs.size(), bucket, 1.0f / N);
    EB_LAUNCH_CHECK("allreduce_avg_multi(unpack)");
    return 0;
}

int eddlb200_allreduce_avg_multi_async(int dev, float *const *bufs, const size_t *sizes, int ntensors, size_t bucket_bytes) {
    EB_CTX(dev);
    EB_REQUIRE(ntensors >= 0 && (ntensors == 0 || (bufs && sizes)), "allreduce_avg_multi_async");
    if (!comm_of(cx)) return eddlb200_allreduce_avg_multi(dev, bufs, sizes, ntensors);        // one rank: times 1.0f, nothing to overlap
    cudaStream_t cs = comm_stream_of(cx);
    cudaEvent_t start = comm_start_event(cx);
    if (!cs || !start) return set_error(EDDLB200_ENOINIT, "allreduce_avg_multi_async: cannot create the communication stream");
    if (bucket_bytes < (size_t(1) << 20)) bucket_bytes = size_t(32) << 20;
    constexpr size_t kInPlaceFloats = size_t(1) << 18;          // tensors of 1 MB or more are reduced where they lie
    // what has been enqueued on the compute stream so far (the optimizer step) comes first; an earlier averaging of the
    // same buffers that is still in flight is waited for by the declarations below
    struct Bucket { int first, last; size_t packed; };
    std::vector<Bucket> buckets;
    std::vector<Seg> segs((size_t)ntensors);
    size_t in_bucket = 0, packed_total = 0, limit = size_t(2) << 20;       // a small first bucket: the first layers are needed first
    for (int i = 0; i < ntensors; i++) {
        EB_REQUIRE(bufs[i] || !sizes[i], "allreduce_avg_multi_async");
        EB_MODIFIES(bufs[i], sizes[i] * sizeof(float));
        if (buckets.empty() || in_bucket >= limit) { if (!buckets.empty()) limit = bucket_bytes; buckets.push_back(Bucket{i, i, 0}); in_bucket = 0; }
        Bucket &b = buckets.back();
        b.last = i;
        const bool in_place = sizes[i] >= kInPlaceFloats;
        segs[i] = Seg{bufs[i], (unsigned long long)sizes[i], in_place ? ~0ull : (unsigned long long)packed_total};
        if (!in_place) { const size_t padded = (sizes[i] + 3) & ~size_t(3); packed_total += padded; b.packed += padded; }
        in_bucket += sizes[i] * sizeof(float);
    }
    if (buckets.empty()) return 0;
    const size_t seg_bytes = (segs.size() * sizeof(Seg) + 255) & ~size_t(255);
    char *ws = (char *)avg_buffer(cx, seg_bytes + packed_total * sizeof(float));
    if (!ws) return set_error((int)cudaErrorMemoryAllocation, "allreduce_avg_multi_async: bucket of %zu bytes", seg_bytes + packed_total * sizeof(float));
    float *bucket = (float *)(ws + seg_bytes);
    cudaError_t e = cudaEventRecord(start, st);
    if (e == cudaSuccess) e = cudaStreamWaitEvent(cs, start, 0);
    // pageable source: staged before the call returns; ordered on the communication stream behind the previous call's kernels
    if (e == cudaSuccess) e = cudaMemcpyAsync(ws, segs.data(), segs.size() * sizeof(Seg), cudaMemcpyHostToDevice, cs);
    if (e != cudaSuccess) return cuda_status(e, "allreduce_avg_multi_async(set-up)");
    const int N = comm_nranks(cx);
    ncclComm_t comm = comm_of(cx);
    for (size_t bi = 0; bi < buckets.size(); bi++) {
        const Bucket &b = buckets[bi];
        const int nseg = b.last - b.first + 1;
        const Seg *dsegs = (const Seg *)ws + b.first;
        size_t largest = 0, first_packed = ~size_t(0);
        for (int i = b.first; i <= b.last; i++) {
            if (sizes[i] > largest) largest = sizes[i];
            if (segs[i].bucket_off != ~0ull && first_packed == ~size_t(0)) first_packed = (size_t)segs[i].bucket_off;
        }
        int gy = nseg > 1024 ? 1024 : nseg;
        int gx = (int)ceil_div(largest, (size_t)kBlock * 8); if (gx < 1) gx = 1; if (gx > 64) gx = 64;
        dim3 grid(gx, gy);
        if (b.packed) {
            // the packed segments of a bucket are contiguous in the bucket buffer
            bucket_pack_kernel<<<grid, kBlock, 0, cs>>>(dsegs, nseg, bucket);
            EB_LAUNCH_CHECK("allreduce_avg_multi_async(pack)");
        }
        if (int r = nccl_status(ncclGroupStart(), "ncclGroupStart")) return r;
        ncclResult_t nr = ncclSuccess;
        if (b.packed) nr = ncclAllReduce(bucket + first_packed, bucket + first_packed, b.packed, ncclFloat, ncclSum, comm, cs);
        for (int i = b.first; i <= b.last && nr == ncclSuccess; i++)
            if (segs[i].bucket_off == ~0ull && sizes[i]) nr = ncclAllReduce(bufs[i], bufs[i], sizes[i], ncclFloat, ncclSum, comm, cs);
        const ncclResult_t ne = ncclGroupEnd();
        if (int r = nccl_status(nr != ncclSuccess ? nr : ne, "ncclAllReduce")) return r;
        count_launch(cx);
        bucket_finish_kernel<<<grid, kBlock, 0, cs>>>(dsegs, nseg, bucket, 1.0f / N);
        EB_LAUNCH_CHECK("allreduce_avg_multi_async(finish)");
        cudaEvent_t done = avg_event(cx, bi);
        if (!done) return set_error(EDDLB200_ENOINIT, "allreduce_avg_multi_async: cannot create an event");
        if ((e = cudaEventRecord(done, cs)) != cudaSuccess) return cuda_status(e, "allreduce_avg_multi_async(record)");
        for (int i = b.first; i <= b.last; i++) if (sizes[i]) avg_register(cx, bufs[i], sizes[i] * sizeof(float), done);
    }
    return 0;
}

int eddlb200_comm_check(int dev, int wait_ms) {
    EB_CTX_KEEP_PENDING(dev);
    ncclComm_t comm = comm_of(cx);
    if (!comm) return 0;
    cudaStream_t cs = comm_stream_of(cx);
    const auto t0 = std::chrono::steady_clock::now();
    for (;;) {
        ncclResult_t async = ncclSuccess;
        const ncclResult_t q = ncclCommGetAsyncError(comm, &async);
        if (q != ncclSuccess || (async != ncclSuccess && async != ncclInProgress)) {
            // the communicator is unusable from here on: abort it so that no later call waits on it
            const int r = nccl_status(q != ncclSuccess ? q : async, "ncclCommGetAsyncError");
            ncclCommAbort(comm);
            set_comm(cx, nullptr, 1, 0);
            return r;
        }
        const cudaError_t a = cudaStreamQuery(st), b = cs ? cudaStreamQuery(cs) : cudaSuccess;
        if (a != cudaErrorNotReady && b != cudaErrorNotReady) {
            if (a != cudaSuccess) return cuda_status(a, "comm_check");
            if (b != cudaSuccess) return cuda_status(b, "comm_check");
            return 0;
        }
        if (wait_ms >= 0 && std::chrono::duration_cast<std::chrono::milliseconds>(std::chrono::steady_clock::now() - t0).count() >= wait_ms)
            return set_error(EDDLB200_ETIMEOUT, "collectives on device %d still running after %d ms", dev, wait_ms);
        std::this_thread::sleep_for(std::chrono::microseconds(200));
    }
}

int eddlb200_broadcast(int dev, float *buf, size_t n, int root) {
    EB_CTX(dev);
    if (n == 0 || !comm_of(cx)) return 0;
    EB_REQUIRE(buf && root >= 0 && root < comm_nranks(cx), "broadcast");
    EB_MODIFIES(buf, n * sizeof(float));
    if (int r = nccl_status(ncclBroadcast(buf, buf, n, ncclFloat, root, comm_of(cx), st), "ncclBroadcast")) return r;
    count_launch(cx);
    return 0;
}

int eddlb200_avg_grad_sgd(int dev, float *p, float *g, float *m, float lr, float mu, size_t n) {
    EB_CTX(dev);
    if (n == 0) return 0;
    EB_REQUIRE(p && g && m, "avg_grad_sgd");
    EB_MODIFIES(p, n * sizeof(float)); EB_MODIFIES(g, n * sizeof(float)); EB_MODIFIES(m, n * sizeof(float));
    const int N = comm_nranks(cx);
    if (comm_of(cx)) {
        if (int r = nccl_status(ncclAllReduce(g, g, n, ncclFloat, ncclSum, comm_of(cx), st), "ncclAllReduce")) return r;
        count_launch(cx);
    }
    avg_sgd_kernel<<<grid_for(n, kBlock), kBlock, 0, st>>>(p, g, m, 1.0f / N, lr, mu, n);
    EB_LAUNCH_CHECK("avg_grad_sgd");
    return 0;
}

}  // extern "C"
