// Softmax forward/backward over one axis, categorical cross-entropy value, accuracy.
// Replaces full_softmax_nd / full_d_softmax_nd (EDDL src/hardware/gpu/nn/
// gpu_activations_kernels.cu:326-382: one THREAD per row), gpu_categorical_cross_entropy
// (nn/gpu_losses_kernels.cu:35-56: one atomicAdd per row + cudaMalloc/cudaMemcpy per call)
// and accuracy (nn/gpu_metrics_kernels.cu:20-54).  Arithmetic follows
// cpu_full_softmax_nd / cpu_d_full_softmax_nd (src/hardware/cpu/nn/cpu_activations.cpp:
// 329-436), cpu_categorical_cross_entropy (cpu_losses.cpp:29-48), cpu_accuracy
// (cpu_metrics.cpp:17-29).
//
// One WARP per softmax sample (shuffle reductions; 10 or 1000 classes both fit), scalars
// are reduced on the device into a context-owned word and read back through pinned
// memory with one stream-ordered copy.
#include "common.cuh"

namespace {

using namespace eb;
constexpr int kBlock = 256;
constexpr int kWarpsPerBlock = kBlock / 32;

// sample si of an [outer, cols, inner] view starts at (si / inner)*cols*inner + si % inner
__global__ void __launch_bounds__(kBlock) softmax_fwd_kernel(const float *__restrict__ a, float *__restrict__ b, int nsamples, int cols, int inner) {
    const int lane = threadIdx.x & 31;
    for (int si = blockIdx.x * kWarpsPerBlock + (threadIdx.x >> 5); si < nsamples; si += gridDim.x * kWarpsPerBlock) {
        const size_t base = (size_t)(si / inner) * cols * inner + (si % inner);
        float m = -3.40282e+38f;
        for (int i = lane; i < cols; i += 32) m = fmaxf(m, a[base + (size_t)i * inner]);
        m = warp_max(m);
        float part = 0.f;
        for (int i = lane; i < cols; i += 32) {
            const float v = expf(__fsub_rn(a[base + (size_t)i * inner], m));
            b[base + (size_t)i * inner] = v;
            part += v;
        }
        // denominator starts at machine epsilon (CPU_EPS_FLOAT) in the reference
        const float denom = __fadd_rn(1.19209e-07f, warp_sum(part));
        for (int i = lane; i < cols; i += 32) {
            const size_t p = base + (size_t)i * inner;
            b[p] = __fdiv_rn(b[p], denom);
        }
    }
}

// pd[i] += sum_j d[j]*(s[i]*[i==j] - s[j]*s[i]).  Evaluated as the reference does, term by
// term, but with the j-loop spread over the warp only through the dot product
// dot = sum_j d[j]*s[j]:  pd[i] += d[i]*s[i] - s[i]*dot  (same value up to summation order).
__global__ void __launch_bounds__(kBlock) softmax_bwd_kernel(const float *__restrict__ d, const float *__restrict__ s, float *__restrict__ pd,
                                                             int nsamples, int cols, int inner) {
    const int lane = threadIdx.x & 31;
    for (int si = blockIdx.x * kWarpsPerBlock + (threadIdx.x >> 5); si < nsamples; si += gridDim.x * kWarpsPerBlock) {
        const size_t base = (size_t)(si / inner) * cols * inner + (si % inner);
        float dot = 0.f;
        for (int i = lane; i < cols; i += 32) dot += d[base + (size_t)i * inner] * s[base + (size_t)i * inner];
        dot = warp_sum(dot);
        for (int i = lane; i < cols; i += 32) {
            const size_t p = base + (size_t)i * inner;
            const float si_ = s[p];
            pd[p] += si_ * (d[p] - dot);
        }
    }
}

// out[0] += sum over this block's rows of sum_c y*logf(p + 1e-7)
__global__ void __launch_bounds__(kBlock) cce_value_kernel(const float *__restrict__ y, const float *__restrict__ p, int rows, int cols, float *out) {
    __shared__ float sm[32];
    const int lane = threadIdx.x & 31;
    float acc = 0.f;
    for (int r = blockIdx.x * kWarpsPerBlock + (threadIdx.x >> 5); r < rows; r += gridDim.x * kWarpsPerBlock) {
        float part = 0.f;
        for (int i = lane; i < cols; i += 32) {
            const size_t q = (size_t)r * cols + i;
            part += y[q] * logf(__fadd_rn(p[q], 10e-8f));
        }
        part = warp_sum(part);
        if (lane == 0) acc += part;
    }
    acc = block_sum(acc, sm);
    if (threadIdx.x == 0) atomicAdd(out, acc);
}

__global__ void __launch_bounds__(kBlock) accuracy_kernel(const float *__restrict__ y, const float *__restrict__ p, int rows, int cols, int *out) {
    const int lane = threadIdx.x & 31;
    int hits = 0;
    for (int r = blockIdx.x * kWarpsPerBlock + (threadIdx.x >> 5); r < rows; r += gridDim.x * kWarpsPerBlock) {
        float by = -INFINITY, bp = -INFINITY; int iy = 0x7fffffff, ip = 0x7fffffff;
        for (int i = lane; i < cols; i += 32) {
            const float vy = y[(size_t)r * cols + i], vp = p[(size_t)r * cols + i];
            if (vy > by || iy == 0x7fffffff) { by = vy; iy = i; }
            if (vp > bp || ip == 0x7fffffff) { bp = vp; ip = i; }
        }
        // arg-max with "first maximum wins": larger value, or equal value and smaller index
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            float oy = __shfl_xor_sync(0xffffffffu, by, o); int oiy = __shfl_xor_sync(0xffffffffu, iy, o);
            if (oiy != 0x7fffffff && (iy == 0x7fffffff || oy > by || (oy == by && oiy < iy))) { by = oy; iy = oiy; }
            float op = __shfl_xor_sync(0xffffffffu, bp, o); int oip = __shfl_xor_sync(0xffffffffu, ip, o);
            if (oip != 0x7fffffff && (ip == 0x7fffffff || op > bp || (op == bp && oip < ip))) { bp = op; ip = oip; }
        }
        if (lane == 0 && iy == ip) hits++;
    }
    if (lane == 0 && hits) atomicAdd(out, hits);
}

}  // namespace

using namespace eb;

extern "C" {

int eddlb200_softmax_fwd(int dev, const float *a, float *b, int rows, int cols) {
    return eddlb200_softmax_fwd_nd(dev, a, b, rows, cols, 1);
}
int eddlb200_softmax_bwd(int dev, const float *d, const float *s, float *pd, int rows, int cols) {
    return eddlb200_softmax_bwd_nd(dev, d, s, pd, rows, cols, 1);
}

int eddlb200_softmax_fwd_nd(int dev, const float *a, float *b, int outer, int cols, int inner) {
    EB_CTX(dev);
    EB_REQUIRE(a && b && outer >= 0 && cols > 0 && inner > 0, "gpu_full_softmax");
    const long long ns = (long long)outer * inner;
    EB_REQUIRE(ns < 0x7fffffffLL, "gpu_full_softmax");
    if (!ns) return 0;
    EB_READS(a, (size_t)ns * cols * sizeof(float));
    if (b != a) EB_WRITES(b, (size_t)ns * cols * sizeof(float));
    softmax_fwd_kernel<<<grid_for((size_t)ns * 32, kBlock), kBlock, 0, st>>>(a, b, (int)ns, cols, inner);
    EB_LAUNCH_CHECK("gpu_full_softmax");
    return 0;
}

int eddlb200_softmax_bwd_nd(int dev, const float *d, const float *s, float *pd, int outer, int cols, int inner) {
    EB_CTX(dev);
    EB_REQUIRE(d && s && pd && outer >= 0 && cols > 0 && inner > 0, "gpu_d_full_softmax");
    const long long ns = (long long)outer * inner;
    EB_REQUIRE(ns < 0x7fffffffLL, "gpu_d_full_softmax");
    if (!ns) return 0;
    EB_READS(d, (size_t)ns * cols * sizeof(float)); EB_READS(s, (size_t)ns * cols * sizeof(float)); EB_MODIFIES(pd, (size_t)ns * cols * sizeof(float));
    softmax_bwd_kernel<<<grid_for((size_t)ns * 32, kBlock), kBlock, 0, st>>>(d, s, pd, (int)ns, cols, inner);
    EB_LAUNCH_CHECK("gpu_d_full_softmax");
    return 0;
}

// Both scalars of a (target, prediction) pair with ONE read-back, remembered until either tensor is written again.
static int loss_and_hits(DevCtx *cx, cudaStream_t st, const float *y_true, const float *y_pred, int rows, int cols, float *loss, int *hits) {
    LossCache &lc = loss_cache(cx);
    const size_t bytes = (size_t)rows * cols * sizeof(float);
    if (lc.valid && lc.y_true == y_true && lc.y_pred == y_pred && lc.rows == rows && lc.cols == cols &&
        lc.v_true == watch_version(cx, y_true) && lc.v_pred == watch_version(cx, y_pred)) {
        *loss = lc.loss; *hits = lc.hits;
        return 0;
    }
    lc.valid = false;
    float *dsc = dev_scalars(cx), *hsc = host_scalars(cx);
    EB_READS(y_true, bytes); EB_READS(y_pred, bytes);
    cudaError_t e = cudaMemsetAsync(dsc, 0, 2 * sizeof(float), st);
    if (e != cudaSuccess) return cuda_status(e, "gpu_categorical_cross_entropy");
    if (rows) {
        cce_value_kernel<<<((size_t)rows * cols <= (size_t(1) << 20)) ? 1 : grid_for((size_t)rows * 32, kBlock, 1), kBlock, 0, st>>>(y_true, y_pred, rows, cols, dsc);
        EB_LAUNCH_CHECK("gpu_categorical_cross_entropy");
        accuracy_kernel<<<grid_for((size_t)rows * 32, kBlock, 1), kBlock, 0, st>>>(y_true, y_pred, rows, cols, (int *)(dsc + 1));
        EB_LAUNCH_CHECK("gpu_accuracy");
    }
    e = cudaMemcpyAsync(hsc, dsc, 2 * sizeof(float), cudaMemcpyDeviceToHost, st);
    if (e == cudaSuccess) e = cudaStreamSynchronize(st);
    if (e != cudaSuccess) return cuda_status(e, "gpu_categorical_cross_entropy");
    *loss = -hsc[0]; *hits = ((const int *)hsc)[1];
    if (bytes) {
        lc.y_true = y_true; lc.y_pred = y_pred; lc.rows = rows; lc.cols = cols;
        lc.v_true = watch_add(cx, y_true, bytes); lc.v_pred = watch_add(cx, y_pred, bytes);
        lc.loss = *loss; lc.hits = *hits;
        lc.valid = lc.v_true != 0 && lc.v_pred != 0 && watch_version(cx, y_true) == lc.v_true;     // overlapping tensors evict each other
    }
    return 0;
}

int eddlb200_cce_value(int dev, const float *y_true, const float *y_pred, int rows, int cols, float *host_out) {
    EB_CTX(dev);
    EB_REQUIRE(y_true && y_pred && host_out && rows >= 0 && cols > 0, "gpu_categorical_cross_entropy");
    int hits = 0;
    return loss_and_hits(cx, st, y_true, y_pred, rows, cols, host_out, &hits);
}

int eddlb200_accuracy(int dev, const float *y_true, const float *y_pred, int rows, int cols, int *host_out) {
    EB_CTX(dev);
    EB_REQUIRE(y_true && y_pred && host_out && rows >= 0 && cols > 0, "gpu_accuracy");
    float loss = 0.f;
    return loss_and_hits(cx, st, y_true, y_pred, rows, cols, &loss, host_out);
}

}  // extern "C"
