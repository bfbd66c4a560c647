// Fused optimizer steps.
// The reference applies SGD-momentum as two Tensor::add launches per parameter tensor
// (EDDL src/optimizers/optim_sgd.cpp:68-89) and Adam as ten elementwise launches
// (src/optimizers/optim_adam.cpp:85-120).  Here each is ONE pass over the parameters
// (SGD: read g, m, p; write m, p = 20 B/param.  Adam: 28 B/param + the in-place g*g the
// reference leaves behind), and the multi-tensor form covers a whole network in a single
// launch.  Every product and sum is rounded separately, in the reference's order, so the
// result is bit-identical to its chain of elementwise calls.
#include <cmath>
#include <cstring>
#include <vector>
#include "common.cuh"

namespace {

using namespace eb;
constexpr int kBlock = 256;

__device__ __forceinline__ void sgd_one(float &p, float g, float &m, float lr, float mu) {
    // Tensor::add(lr, g, mu, m, m, 0);  Tensor::add(1.0, p, -1.0, m, p, 0);
    m = __fadd_rn(__fmul_rn(lr, g), __fmul_rn(mu, m));
    p = __fadd_rn(__fmul_rn(1.0f, p), __fmul_rn(-1.0f, m));
}

__global__ void __launch_bounds__(kBlock) sgd_kernel(float *p, const float *g, float *m, float lr, float mu, size_t n4, size_t n) {
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    for (size_t j = i; j < n4; j += stride) {
        float4 pv = *reinterpret_cast<float4 *>(p + 4 * j);
        const float4 gv = *reinterpret_cast<const float4 *>(g + 4 * j);
        float4 mv = *reinterpret_cast<float4 *>(m + 4 * j);
        sgd_one(pv.x, gv.x, mv.x, lr, mu); sgd_one(pv.y, gv.y, mv.y, lr, mu);
        sgd_one(pv.z, gv.z, mv.z, lr, mu); sgd_one(pv.w, gv.w, mv.w, lr, mu);
        *reinterpret_cast<float4 *>(m + 4 * j) = mv;
        *reinterpret_cast<float4 *>(p + 4 * j) = pv;
    }
    for (size_t j = 4 * n4 + i; j < n; j += stride) { float pv = p[j], mv = m[j]; sgd_one(pv, g[j], mv, lr, mu); m[j] = mv; p[j] = pv; }
}

struct TensorRef { float *p; const float *g; float *m; unsigned long long n; };

// One block-chunk table entry per 16K elements: (tensor, offset).
struct Chunk { unsigned tensor; unsigned offset_k; };   // offset in units of kChunk elements
constexpr unsigned kChunk = 16384;

__global__ void __launch_bounds__(kBlock) sgd_multi_kernel(const TensorRef *__restrict__ tensors, const Chunk *__restrict__ chunks, int nchunks, float lr, float mu) {
    for (int c = blockIdx.x; c < nchunks; c += gridDim.x) {
        const Chunk ch = chunks[c];
        const TensorRef t = tensors[ch.tensor];
        const size_t beg = (size_t)ch.offset_k * kChunk;
        const size_t end = beg + kChunk < t.n ? beg + kChunk : (size_t)t.n;
        const bool vec = ((((uintptr_t)t.p) | ((uintptr_t)t.g) | ((uintptr_t)t.m)) & 15u) == 0;
        if (vec) {
            const size_t end4 = beg + ((end - beg) & ~size_t(3));
            for (size_t j = beg + threadIdx.x * 4; j < end4; j += kBlock * 4) {
                float4 pv = *reinterpret_cast<float4 *>(t.p + j);
                const float4 gv = *reinterpret_cast<const float4 *>(t.g + j);
                float4 mv = *reinterpret_cast<float4 *>(t.m + j);
                sgd_one(pv.x, gv.x, mv.x, lr, mu); sgd_one(pv.y, gv.y, mv.y, lr, mu);
                sgd_one(pv.z, gv.z, mv.z, lr, mu); sgd_one(pv.w, gv.w, mv.w, lr, mu);
                *reinterpret_cast<float4 *>(t.m + j) = mv;
                *reinterpret_cast<float4 *>(t.p + j) = pv;
            }
            for (size_t j = end4 + threadIdx.x; j < end; j += kBlock) { float pv = t.p[j], mv = t.m[j]; sgd_one(pv, t.g[j], mv, lr, mu); t.m[j] = mv; t.p[j] = pv; }
        } else {
            for (size_t j = beg + threadIdx.x; j < end; j += kBlock) { float pv = t.p[j], mv = t.m[j]; sgd_one(pv, t.g[j], mv, lr, mu); t.m[j] = mv; t.p[j] = pv; }
        }
    }
}

struct AdamCoef { float lr, b1, b2, omb1, omb2, bc1, bc2, eps; };

__device__ __forceinline__ void adam_one(float &p, float &g, float &m, float &v, const AdamCoef &k) {
    // Tensor::add(beta_1, mT, 1-beta_1, gT, mT, 0)
    m = __fadd_rn(__fmul_rn(k.b1, m), __fmul_rn(k.omb1, g));
    // gT->sqr_() ; Tensor::add(beta_2, vT, 1-beta_2, gT, vT, 0)
    g = __fmul_rn(g, g);
    v = __fadd_rn(__fmul_rn(k.b2, v), __fmul_rn(k.omb2, g));
    // mCap = m * (1/(1-beta_1^t)) ; vCap = sqrt(v * (1/(1-beta_2^t)) + eps) ; mCap = mCap / vCap
    const float upd = __fdiv_rn(__fmul_rn(m, k.bc1), __fsqrt_rn(__fadd_rn(__fmul_rn(v, k.bc2), k.eps)));
    // Tensor::add(-lr, mCap, 1.0, p, p, 0)
    p = __fadd_rn(__fmul_rn(-k.lr, upd), __fmul_rn(1.0f, p));
}

struct AdamRef { float *p, *g, *m, *v; unsigned long long n; };

// Multi-tensor Adam: the same chunk table as sgd_multi_kernel, 28 bytes per parameter plus the squared gradient the
// reference leaves in the gradient tensor.
__global__ void __launch_bounds__(kBlock) adam_multi_kernel(const AdamRef *__restrict__ tensors, const Chunk *__restrict__ chunks, int nchunks, AdamCoef k) {
    for (int c = blockIdx.x; c < nchunks; c += gridDim.x) {
        const Chunk ch = chunks[c];
        const AdamRef t = tensors[ch.tensor];
        const size_t beg = (size_t)ch.offset_k * kChunk;
        const size_t end = beg + kChunk < t.n ? beg + kChunk : (size_t)t.n;
        const bool vec = ((((uintptr_t)t.p) | ((uintptr_t)t.g) | ((uintptr_t)t.m) | ((uintptr_t)t.v)) & 15u) == 0;
        size_t scalar_from = beg;
        if (vec) {
            const size_t end4 = beg + ((end - beg) & ~size_t(3));
            for (size_t j = beg + threadIdx.x * 4; j < end4; j += kBlock * 4) {
                float4 pv = *reinterpret_cast<float4 *>(t.p + j), gv = *reinterpret_cast<float4 *>(t.g + j);
                float4 mv = *reinterpret_cast<float4 *>(t.m + j), vv = *reinterpret_cast<float4 *>(t.v + j);
                adam_one(pv.x, gv.x, mv.x, vv.x, k); adam_one(pv.y, gv.y, mv.y, vv.y, k);
                adam_one(pv.z, gv.z, mv.z, vv.z, k); adam_one(pv.w, gv.w, mv.w, vv.w, k);
                *reinterpret_cast<float4 *>(t.p + j) = pv; *reinterpret_cast<float4 *>(t.g + j) = gv;
                *reinterpret_cast<float4 *>(t.m + j) = mv; *reinterpret_cast<float4 *>(t.v + j) = vv;
            }
            scalar_from = end4;
        }
        for (size_t j = scalar_from + threadIdx.x; j < end; j += kBlock) {
            float pv = t.p[j], gv = t.g[j], mv = t.m[j], vv = t.v[j];
            adam_one(pv, gv, mv, vv, k);
            t.p[j] = pv; t.g[j] = gv; t.m[j] = mv; t.v[j] = vv;
        }
    }
}

// 1 - pow(beta, t) is a double in the reference (std::pow(float, int), optim_adam.cpp:103-107), narrowed to float by
// div_(float), which then multiplies by the float reciprocal (tensor_math.cpp:1186-1188).
AdamCoef adam_coef(float lr, float beta1, float beta2, float eps, int t) {
    AdamCoef k;
    k.lr = lr; k.b1 = beta1; k.b2 = beta2; k.omb1 = 1 - beta1; k.omb2 = 1 - beta2; k.eps = eps;
    k.bc1 = 1.0f / (float)(1.0 - pow((double)beta1, (double)t));
    k.bc2 = 1.0f / (float)(1.0 - pow((double)beta2, (double)t));
    return k;
}

__global__ void __launch_bounds__(kBlock) adam_kernel(float *p, float *g, float *m, float *v, float lr, float b1, float b2, float omb1, float omb2,
                                                      float bc1, float bc2, float eps, size_t n) {
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    for (size_t j = (size_t)blockIdx.x * blockDim.x + threadIdx.x; j < n; j += stride) {
        const float gj = g[j];
        // Tensor::add(beta_1, mT, 1-beta_1, gT, mT, 0)
        const float mj = __fadd_rn(__fmul_rn(b1, m[j]), __fmul_rn(omb1, gj));
        // gT->sqr_() ; Tensor::add(beta_2, vT, 1-beta_2, gT, vT, 0)
        const float g2 = __fmul_rn(gj, gj);
        const float vj = __fadd_rn(__fmul_rn(b2, v[j]), __fmul_rn(omb2, g2));
        // mCap = m / (1 - beta_1^t) is evaluated as mult_(1/(1-beta^t)) in the reference (Tensor::div)
        const float mcap = __fmul_rn(mj, bc1);
        float vcap = __fmul_rn(vj, bc2);
        vcap = __fadd_rn(vcap, eps);          // vCap->add_(epsilon)
        vcap = __fsqrt_rn(vcap);              // vCap->sqrt_()
        const float upd = __fdiv_rn(mcap, vcap);   // Tensor::el_div(mCap, vCap, mCap, 0)
        // Tensor::add(-lr, mCap, 1.0, p, p, 0)
        p[j] = __fadd_rn(__fmul_rn(-lr, upd), __fmul_rn(1.0f, p[j]));
        m[j] = mj; v[j] = vj; g[j] = g2;
    }
}

}  // namespace

using namespace eb;

extern "C" {

int eddlb200_sgd_momentum(int dev, float *p, const float *g, float *m, float lr, float mu, size_t n) {
    EB_CTX(dev);
    if (n == 0) return 0;
    EB_REQUIRE(p && g && m, "sgd");
    EB_MODIFIES(p, n * sizeof(float)); EB_READS(g, n * sizeof(float)); EB_MODIFIES(m, n * sizeof(float));
    const bool vec = aligned16(p) && aligned16(g) && aligned16(m);
    const size_t n4 = vec ? n / 4 : 0;
    sgd_kernel<<<grid_for(vec ? (n4 ? n4 : 1) : n, kBlock), kBlock, 0, st>>>(p, g, m, lr, mu, n4, n);
    EB_LAUNCH_CHECK("sgd_momentum");
    return 0;
}

int eddlb200_sgd_momentum_multi(int dev, float *const *p, const float *const *g, float *const *m,
                                const size_t *sizes, int ntensors, float lr, float mu) {
    EB_CTX(dev);
    EB_REQUIRE(ntensors >= 0 && (ntensors == 0 || (p && g && m && sizes)), "sgd_multi");
    if (ntensors == 0) return 0;
    std::vector<TensorRef> refs; std::vector<Chunk> chunks;
    for (int i = 0; i < ntensors; i++) {
        if (sizes[i] == 0) continue;
        EB_REQUIRE(p[i] && g[i] && m[i], "sgd_multi");
        EB_MODIFIES(p[i], sizes[i] * sizeof(float)); EB_READS(g[i], sizes[i] * sizeof(float)); EB_MODIFIES(m[i], sizes[i] * sizeof(float));
        refs.push_back(TensorRef{p[i], g[i], m[i], (unsigned long long)sizes[i]});
        const size_t nch = ceil_div(sizes[i], (size_t)kChunk);
        for (size_t c = 0; c < nch; c++) chunks.push_back(Chunk{(unsigned)(refs.size() - 1), (unsigned)c});
    }
    if (chunks.empty()) return 0;
    double total = 0; for (auto &r : refs) total += (double)r.n;
    ProfScope prof(cx, PROF_OPTIM, 20.0 * total);
    const size_t bytes_t = refs.size() * sizeof(TensorRef), bytes_c = chunks.size() * sizeof(Chunk);
    const size_t off_c = (bytes_t + 255) & ~size_t(255);
    // The table lives in the stream-ordered scratch arena; the copy below is ordered
    // before the kernel on the same stream and its host source is staged by the runtime.
    char *tab = (char *)scratch(cx, off_c + bytes_c);
    if (!tab) return cudaErrorMemoryAllocation;
    std::vector<char> host(off_c + bytes_c);
    memcpy(host.data(), refs.data(), bytes_t);
    memcpy(host.data() + off_c, chunks.data(), bytes_c);
    cudaError_t e = cudaMemcpyAsync(tab, host.data(), host.size(), cudaMemcpyHostToDevice, st);
    if (e != cudaSuccess) return cuda_status(e, "sgd_multi(table)");
    // pageable source: cudaMemcpyAsync returns after staging, so `host` may go out of scope
    int blocks = (int)chunks.size();
    if (blocks > EDDLB200_NUM_SMS * 8) blocks = EDDLB200_NUM_SMS * 8;
    sgd_multi_kernel<<<blocks, kBlock, 0, st>>>((const TensorRef *)tab, (const Chunk *)(tab + off_c), (int)chunks.size(), lr, mu);
    EB_LAUNCH_CHECK("sgd_momentum_multi");
    return 0;
}

int eddlb200_adam(int dev, float *p, float *g, float *m, float *v, float lr, float beta1, float beta2, float eps, int t, size_t n) {
    EB_CTX(dev);
    if (n == 0) return 0;
    EB_REQUIRE(p && g && m && v && t >= 1, "adam");
    EB_MODIFIES(p, n * sizeof(float)); EB_MODIFIES(g, n * sizeof(float)); EB_MODIFIES(m, n * sizeof(float)); EB_MODIFIES(v, n * sizeof(float));
    const AdamCoef k = adam_coef(lr, beta1, beta2, eps, t);
    adam_kernel<<<grid_for(n, kBlock), kBlock, 0, st>>>(p, g, m, v, lr, beta1, beta2, k.omb1, k.omb2, k.bc1, k.bc2, eps, n);
    EB_LAUNCH_CHECK("adam");
    return 0;
}

int eddlb200_adam_multi(int dev, float *const *p, float *const *g, float *const *m, float *const *v,
                        const size_t *sizes, int ntensors, float lr, float beta1, float beta2, float eps, int t) {
    EB_CTX(dev);
    EB_REQUIRE(ntensors >= 0 && t >= 1 && (ntensors == 0 || (p && g && m && v && sizes)), "adam_multi");
    if (ntensors == 0) return 0;
    std::vector<AdamRef> refs; std::vector<Chunk> chunks;
    for (int i = 0; i < ntensors; i++) {
        if (sizes[i] == 0) continue;
        EB_REQUIRE(p[i] && g[i] && m[i] && v[i], "adam_multi");
        const size_t bytes = sizes[i] * sizeof(float);
        EB_MODIFIES(p[i], bytes); EB_MODIFIES(g[i], bytes); EB_MODIFIES(m[i], bytes); EB_MODIFIES(v[i], bytes);
        refs.push_back(AdamRef{p[i], g[i], m[i], v[i], (unsigned long long)sizes[i]});
        const size_t nch = ceil_div(sizes[i], (size_t)kChunk);
        for (size_t c = 0; c < nch; c++) chunks.push_back(Chunk{(unsigned)(refs.size() - 1), (unsigned)c});
    }
    if (chunks.empty()) return 0;
    double total = 0; for (auto &r : refs) total += (double)r.n;
    ProfScope prof(cx, PROF_OPTIM, 28.0 * total);
    const size_t bytes_t = refs.size() * sizeof(AdamRef), bytes_c = chunks.size() * sizeof(Chunk);
    const size_t off_c = (bytes_t + 255) & ~size_t(255);
    char *tab = (char *)scratch(cx, off_c + bytes_c);
    if (!tab) return cudaErrorMemoryAllocation;
    std::vector<char> host(off_c + bytes_c);
    memcpy(host.data(), refs.data(), bytes_t);
    memcpy(host.data() + off_c, chunks.data(), bytes_c);
    // pageable source: the runtime stages it before cudaMemcpyAsync returns, so `host` may go out of scope
    cudaError_t e = cudaMemcpyAsync(tab, host.data(), host.size(), cudaMemcpyHostToDevice, st);
    if (e != cudaSuccess) return cuda_status(e, "adam_multi(table)");
    int blocks = (int)chunks.size();
    if (blocks > EDDLB200_NUM_SMS * 8) blocks = EDDLB200_NUM_SMS * 8;
    adam_multi_kernel<<<blocks, kBlock, 0, st>>>((const AdamRef *)tab, (const Chunk *)(tab + off_c), (int)chunks.size(), adam_coef(lr, beta1, beta2, eps, t));
    EB_LAUNCH_CHECK("adam_multi");
    return 0;
}

}  // extern "C"
