// Cross-replica averaging over NVLink / NVSwitch through NCCL, one process per GPU.
// Replaces Net::sync_weights (EDDL src/net/net_func.cpp:111-127), which copies every
// parameter of every replica to the host, adds them there, multiplies by 1.0f/N and copies
// the result back to every GPU, one tensor at a time with blocking copies.  Here the sum is
// an in-place ncclAllReduce on the device's compute stream and the 1.0f/N multiply is a
// kernel of this library (fused into the SGD step for gradient averaging).  Many small
// tensors are packed into one contiguous bucket so the collective is sized for launch
// latency, not for tensor count.
#include <nccl.h>
#include <cstring>
#include <vector>
#include "common.cuh"

namespace eb {
void set_comm(DevCtx *c, ncclComm *comm, int nranks, int rank);
int comm_rank(DevCtx *c);
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
