// Bandwidth-bound elementwise kernels: fill, axpby, scale, sqr, sqrt, clamp, el_div,
// el_mult, ReLU forward/backward, CCE delta, padding.
// Replaces the one-thread-per-element kernels of EDDL's src/hardware/gpu/gpu_math_kernels.cu,
// gpu_core_kernels.cu and nn/gpu_activations_kernels.cu:21-41.  Each kernel is a
// grid-stride loop over float4 (16-byte, fully coalesced) with a scalar tail; the
// grid is a multiple of the 148 SMs.  Arithmetic is written with explicit
// round-to-nearest intrinsics where the reference evaluates a*b+c in two roundings,
// so that results are bit-identical to its CPU code (no FMA contraction).
#include <cstring>
#include <vector>
#include "common.cuh"

namespace {

using namespace eb;

constexpr int kBlock = 256;

template <typename F>
__global__ void __launch_bounds__(kBlock) map1_kernel(const float *a, float *b, size_t n4, size_t n, F f) {
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    for (size_t j = i; j < n4; j += stride) {
        float4 v = *reinterpret_cast<const float4 *>(a + 4 * j);
        v.x = f(v.x); v.y = f(v.y); v.z = f(v.z); v.w = f(v.w);
        *reinterpret_cast<float4 *>(b + 4 * j) = v;
    }
    for (size_t j = 4 * n4 + i; j < n; j += stride) b[j] = f(a[j]);
}

template <typename F>
__global__ void __launch_bounds__(kBlock) map1_scalar_kernel(const float *a, float *b, size_t n, F f) {
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    for (size_t j = (size_t)blockIdx.x * blockDim.x + threadIdx.x; j < n; j += stride) b[j] = f(a[j]);
}

// c = f(a, b, c)
template <typename F>
__global__ void __launch_bounds__(kBlock) map3_kernel(const float *a, const float *b, float *c, size_t n4, size_t n, F f) {
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    for (size_t j = i; j < n4; j += stride) {
        float4 x = *reinterpret_cast<const float4 *>(a + 4 * j);
        float4 y = *reinterpret_cast<const float4 *>(b + 4 * j);
        float4 z = F::reads_c ? *reinterpret_cast<const float4 *>(c + 4 * j) : make_float4(0, 0, 0, 0);
        z.x = f(x.x, y.x, z.x); z.y = f(x.y, y.y, z.y); z.z = f(x.z, y.z, z.z); z.w = f(x.w, y.w, z.w);
        *reinterpret_cast<float4 *>(c + 4 * j) = z;
    }
    for (size_t j = 4 * n4 + i; j < n; j += stride) c[j] = f(a[j], b[j], F::reads_c ? c[j] : 0.f);
}

template <typename F>
__global__ void __launch_bounds__(kBlock) map3_scalar_kernel(const float *a, const float *b, float *c, size_t n, F f) {
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    for (size_t j = (size_t)blockIdx.x * blockDim.x + threadIdx.x; j < n; j += stride) c[j] = f(a[j], b[j], F::reads_c ? c[j] : 0.f);
}

// c = f(a, b); r = max(c, 0): a recorded sum together with the ReLU that follows it.  n4 = 0 runs everything in the scalar loop.
template <typename F>
__global__ void __launch_bounds__(kBlock) map3_relu_kernel(const float *a, const float *b, float *c, float *r, size_t n4, size_t n, F f) {
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    for (size_t j = i; j < n4; j += stride) {
        const float4 x = *reinterpret_cast<const float4 *>(a + 4 * j);
        const float4 y = *reinterpret_cast<const float4 *>(b + 4 * j);
        float4 z;
        z.x = f(x.x, y.x, 0.f); z.y = f(x.y, y.y, 0.f); z.z = f(x.z, y.z, 0.f); z.w = f(x.w, y.w, 0.f);
        *reinterpret_cast<float4 *>(c + 4 * j) = z;
        z.x = z.x > 0.f ? z.x : 0.f; z.y = z.y > 0.f ? z.y : 0.f; z.z = z.z > 0.f ? z.z : 0.f; z.w = z.w > 0.f ? z.w : 0.f;
        *reinterpret_cast<float4 *>(r + 4 * j) = z;
    }
    for (size_t j = 4 * n4 + i; j < n; j += stride) { const float z = f(a[j], b[j], 0.f); c[j] = z; r[j] = z > 0.f ? z : 0.f; }
}

// b = c = f(a): one source copied into two destinations.  n4 = 0 runs everything in the scalar loop.
template <typename F>
__global__ void __launch_bounds__(kBlock) map1_twice_kernel(const float *a, float *b, float *c, size_t n4, size_t n, F f) {
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    for (size_t j = i; j < n4; j += stride) {
        float4 v = *reinterpret_cast<const float4 *>(a + 4 * j);
        v.x = f(v.x); v.y = f(v.y); v.z = f(v.z); v.w = f(v.w);
        *reinterpret_cast<float4 *>(b + 4 * j) = v;
        *reinterpret_cast<float4 *>(c + 4 * j) = v;
    }
    for (size_t j = 4 * n4 + i; j < n; j += stride) { const float v = f(a[j]); b[j] = v; c[j] = v; }
}

template <typename F>
int launch1(DevCtx *cx, cudaStream_t st, const float *a, float *b, size_t n, F f, const char *what, double bytes_per_element = 8.0) {
    if (n == 0) return 0;
    if (!a || !b) return set_error(EDDLB200_EINVAL, "%s: null pointer", what);
    if (!F::ignores_input) EB_READS(a, n * sizeof(float));
    EB_WRITES(b, n * sizeof(float));
    // profile work = the canonical byte count of the operation (a "destination is zero" variant moves fewer bytes but
    // is charged like the read-modify-write it replaces)
    ProfScope prof(cx, PROF_ELEMENTWISE, bytes_per_element * n);
    if (aligned16(a) && aligned16(b)) {
        size_t n4 = n / 4;
        map1_kernel<<<grid_for(n4 ? n4 : 1, kBlock), kBlock, 0, st>>>(a, b, n4, n, f);
    } else {
        map1_scalar_kernel<<<grid_for(n, kBlock), kBlock, 0, st>>>(a, b, n, f);
    }
    EB_LAUNCH_CHECK(what);
    return 0;
}

template <typename F>
int launch3(DevCtx *cx, cudaStream_t st, const float *a, const float *b, float *c, size_t n, F f, const char *what, double bytes_per_element = 0.0) {
    if (n == 0) return 0;
    if (!a || !b || !c) return set_error(EDDLB200_EINVAL, "%s: null pointer", what);
    EB_READS(a, n * sizeof(float));
    EB_READS(b, n * sizeof(float));
    if (F::reads_c) EB_MODIFIES(c, n * sizeof(float)); else EB_WRITES(c, n * sizeof(float));
    ProfScope prof(cx, PROF_ELEMENTWISE, (bytes_per_element > 0 ? bytes_per_element : (F::reads_c ? 16.0 : 12.0)) * n);
    if (aligned16(a) && aligned16(b) && aligned16(c)) {
        size_t n4 = n / 4;
        map3_kernel<<<grid_for(n4 ? n4 : 1, kBlock), kBlock, 0, st>>>(a, b, c, n4, n, f);
    } else {
        map3_scalar_kernel<<<grid_for(n, kBlock), kBlock, 0, st>>>(a, b, c, n, f);
    }
    EB_LAUNCH_CHECK(what);
    return 0;
}

struct FillF { static constexpr bool ignores_input = true; float v; __device__ float operator()(float) const { return v; } };
struct ScaleF { static constexpr bool ignores_input = false; float v; __device__ float operator()(float x) const { return __fmul_rn(x, v); } };
struct AddcF { static constexpr bool ignores_input = false; float v; __device__ float operator()(float x) const { return __fadd_rn(x, v); } };
struct SqrF { static constexpr bool ignores_input = false; __device__ float operator()(float x) const { return __fmul_rn(x, x); } };
struct SqrtF { static constexpr bool ignores_input = false; __device__ float operator()(float x) const { return __fsqrt_rn(x); } };
struct ClampF { static constexpr bool ignores_input = false; float lo, hi; __device__ float operator()(float x) const { return x < lo ? lo : (x > hi ? hi : x); } };
struct ReluF { static constexpr bool ignores_input = false; __device__ float operator()(float x) const { return x > 0.f ? x : 0.f; } };
// sa*x + sb*0: gpu_add(sa, A, sb, B, C = B, 0) -- the form Tensor::inc takes on the GPU -- with B known to hold zeros
struct AxpbZeroF { static constexpr bool ignores_input = false; float sa, sb; __device__ float operator()(float x) const { return __fadd_rn(__fmul_rn(sa, x), __fmul_rn(sb, 0.f)); } };
struct ZeroAxpbF { static constexpr bool ignores_input = false; float sa, sb; __device__ float operator()(float y) const { return __fadd_rn(__fmul_rn(sa, 0.f), __fmul_rn(sb, y)); } };
// b = 0 + a: what "b += a" leaves in a b known to hold zeros (the add keeps the sign of a zero result identical)
struct AddToZeroF { static constexpr bool ignores_input = false; __device__ float operator()(float x) const { return __fadd_rn(0.f, x); } };

// gpu_add: C = scA*A + scB*B (+ C).  Reference (cpu_math.cpp cpu_add): two products, one sum,
// then "+=" when incC -- four roundings, reproduced here.
template <bool INC> struct AxpbyF {
    static constexpr bool reads_c = INC;
    float sa, sb;
    __device__ float operator()(float a, float b, float c) const {
        float r = __fadd_rn(__fmul_rn(sa, a), __fmul_rn(sb, b));
        return INC ? __fadd_rn(c, r) : r;
    }
};
template <bool INC> struct DivF {
    static constexpr bool reads_c = INC;
    __device__ float operator()(float a, float b, float c) const { float r = __fdiv_rn(a, b); return INC ? __fadd_rn(c, r) : r; }
};
template <bool INC> struct MulF {
    static constexpr bool reads_c = INC;
    __device__ float operator()(float a, float b, float c) const { float r = __fmul_rn(a, b); return INC ? __fadd_rn(c, r) : r; }
};
// pd += (i > 0) ? d : 0      a = d, b = i, c = pd
struct ReluBwdF {
    static constexpr bool reads_c = true;
    __device__ float operator()(float d, float i, float pd) const { return i > 0.f ? __fadd_rn(pd, d) : pd; }
};
// the same with pd known to hold zeros: no read of pd
struct ReluBwdZeroF {
    static constexpr bool reads_c = false;
    __device__ float operator()(float d, float i, float) const { return i > 0.f ? __fadd_rn(0.f, d) : 0.f; }
};
// c = s2*y + t2*(s1*x + t1*0): the two in-place adds "c = s1*x + t1*c; c = s2*y + t2*c" into a c known to hold zeros
struct Sum2IntoZeroF {
    static constexpr bool reads_c = false;
    float s1, t1, s2, t2;
    __device__ float operator()(float x, float y, float) const {
        const float first = __fadd_rn(__fmul_rn(s1, x), __fmul_rn(t1, 0.f));
        return __fadd_rn(__fmul_rn(s2, y), __fmul_rn(t2, first));
    }
};
// c = 0 + (sa*a + sb*b): gpu_add with incC into a c known to hold zeros
struct AxpbyZeroF {
    static constexpr bool reads_c = false;
    float sa, sb;
    __device__ float operator()(float a, float b, float) const { return __fadd_rn(0.f, __fadd_rn(__fmul_rn(sa, a), __fmul_rn(sb, b))); }
};
// delta = -y * (1.0f / (p + 1e-7))   a = y_true, b = y_pred  (cpu_losses.cpp:50-57)
struct CceDeltaF {
    static constexpr bool reads_c = false;
    __device__ float operator()(float y, float p, float) const { return __fmul_rn(-y, __fdiv_rn(1.0f, __fadd_rn(p, 10e-8f))); }
};

// Copy the interior: one thread per four consecutive elements of a row of the SMALL tensor a[n*c,h,w] (one per element when
// rows are not a multiple of four long).  32-bit index arithmetic: the entry points refuse tensors of 2^31 elements or more.
template <bool BACK, int V>
__global__ void __launch_bounds__(kBlock) pad_kernel(float *a, float *b, unsigned total_v, int h, int w, int top, int left, int bh, int bw) {
    const unsigned stride = gridDim.x * blockDim.x, wv = (unsigned)w / V;
    for (unsigned i = blockIdx.x * blockDim.x + threadIdx.x; i < total_v; i += stride) {
        const unsigned t = i / wv, x = (i - t * wv) * V, plane = t / (unsigned)h, y = t - plane * h;
        float *pb = b + ((size_t)plane * bh + (y + top)) * bw + (x + left);
        if (V == 4) {
            float4 va = reinterpret_cast<const float4 *>(a)[i];
            if (BACK) {
                va.x = __fadd_rn(va.x, pb[0]); va.y = __fadd_rn(va.y, pb[1]); va.z = __fadd_rn(va.z, pb[2]); va.w = __fadd_rn(va.w, pb[3]);
                reinterpret_cast<float4 *>(a)[i] = va;
            } else { pb[0] = va.x; pb[1] = va.y; pb[2] = va.z; pb[3] = va.w; }
        } else {
            if (BACK) a[i] = __fadd_rn(a[i], pb[0]); else pb[0] = a[i];
        }
    }
}

// Many fills in one launch: segment table in the scratch arena, one block-chunk of 16K elements per table entry.
struct FillSeg { float *p; unsigned long long n; float v; unsigned pad; };
struct FillChunk { unsigned seg; unsigned offset_k; };
constexpr unsigned kFillChunk = 16384;
__global__ void __launch_bounds__(kBlock) fill_multi_kernel(const FillSeg *__restrict__ segs, const FillChunk *__restrict__ chunks, int nchunks) {
    for (int c = blockIdx.x; c < nchunks; c += gridDim.x) {
        const FillChunk ch = chunks[c];
        const FillSeg sg = segs[ch.seg];
        const size_t beg = (size_t)ch.offset_k * kFillChunk;
        const size_t end = beg + kFillChunk < sg.n ? beg + kFillChunk : (size_t)sg.n;
        if ((((uintptr_t)sg.p) & 15u) == 0) {
            const size_t end4 = beg + ((end - beg) & ~size_t(3));
            const float4 v4 = make_float4(sg.v, sg.v, sg.v, sg.v);
            for (size_t j = beg + threadIdx.x * 4; j < end4; j += kBlock * 4) *reinterpret_cast<float4 *>(sg.p + j) = v4;
            for (size_t j = end4 + threadIdx.x; j < end; j += kBlock) sg.p[j] = sg.v;
        } else {
            for (size_t j = beg + threadIdx.x; j < end; j += kBlock) sg.p[j] = sg.v;
        }
    }
}

}  // namespace

namespace eb {
// runs a recorded "dst = sa*src + sb*0" (see PendCopy)
int pend_copy_flush(DevCtx *cx, cudaStream_t st) {
    PendCopy &p = pend_copy(cx);
    if (!p.active) return 0;
    p.active = false;
    if (p.kind == 2) return launch3(cx, st, p.src, p.src2, p.dst, p.n, Sum2IntoZeroF{p.sa, p.sb, p.s2, p.t2}, "gpu_add", 12.0);
    if (p.kind == 3) {
        const size_t n = p.n;
        EB_READS(p.src, n * sizeof(float)); EB_WRITES(p.dst, n * sizeof(float)); EB_WRITES(p.dst2, n * sizeof(float));
        ProfScope prof(cx, PROF_ELEMENTWISE, 12.0 * n);             // one read, two writes (the two in-place adds it replaces move 24)
        const size_t n4 = (aligned16(p.src) && aligned16(p.dst) && aligned16(p.dst2)) ? n / 4 : 0;
        map1_twice_kernel<<<grid_for(n4 ? n4 : n, kBlock), kBlock, 0, st>>>(p.src, p.dst, p.dst2, n4, n, AxpbZeroF{p.sa, p.sb});
        EB_LAUNCH_CHECK("gpu_add (two destinations)");
        return 0;
    }
    return launch1(cx, st, p.src, p.dst, p.n, AxpbZeroF{p.sa, p.sb}, "gpu_add", 8.0);
}
// writes n zeros at p; used when a deferred zero fill has to be materialised
int launch_zero_fill(DevCtx *cx, cudaStream_t st, float *p, size_t n) {
    if (n == 0) return 0;
    ProfScope prof(cx, PROF_ELEMENTWISE, 4.0 * n);
    if (aligned16(p)) { const size_t n4 = n / 4; map1_kernel<<<grid_for(n4 ? n4 : 1, kBlock), kBlock, 0, st>>>(p, p, n4, n, FillF{0.f}); }
    else map1_scalar_kernel<<<grid_for(n, kBlock), kBlock, 0, st>>>(p, p, n, FillF{0.f});
    EB_LAUNCH_CHECK("gpu_fill_(deferred)");
    return 0;
}
}  // namespace eb

using namespace eb;

extern "C" {

int eddlb200_fill_multi(int dev, float *const *ptrs, const size_t *sizes, const float *values, int ntensors) {
    EB_CTX(dev);
    EB_REQUIRE(ntensors >= 0 && (ntensors == 0 || (ptrs && sizes && values)), "fill_multi");
    std::vector<FillSeg> segs; std::vector<FillChunk> chunks;
    double total = 0;
    for (int i = 0; i < ntensors; i++) {
        if (!sizes[i]) continue;
        EB_REQUIRE(ptrs[i], "fill_multi");
        if (values[i] == 0.f && lz_defer(cx, st, ptrs[i], sizes[i] * sizeof(float))) continue;
        EB_WRITES(ptrs[i], sizes[i] * sizeof(float));
        segs.push_back(FillSeg{ptrs[i], (unsigned long long)sizes[i], values[i], 0u});
        const size_t nch = ceil_div(sizes[i], (size_t)kFillChunk);
        for (size_t c = 0; c < nch; c++) chunks.push_back(FillChunk{(unsigned)(segs.size() - 1), (unsigned)c});
        total += (double)sizes[i];
    }
    if (chunks.empty()) return 0;
    const size_t bytes_s = segs.size() * sizeof(FillSeg), off_c = (bytes_s + 255) & ~size_t(255), bytes_c = chunks.size() * sizeof(FillChunk);
    char *tab = (char *)scratch(cx, off_c + bytes_c);
    if (!tab) return cudaErrorMemoryAllocation;
    std::vector<char> host(off_c + bytes_c);
    memcpy(host.data(), segs.data(), bytes_s);
    memcpy(host.data() + off_c, chunks.data(), bytes_c);
    cudaError_t e = cudaMemcpyAsync(tab, host.data(), host.size(), cudaMemcpyHostToDevice, st);   // pageable source: staged before return
    if (e != cudaSuccess) return cuda_status(e, "fill_multi(table)");
    ProfScope prof(cx, PROF_ELEMENTWISE, 4.0 * total);
    int blocks = (int)chunks.size();
    if (blocks > EDDLB200_NUM_SMS * 8) blocks = EDDLB200_NUM_SMS * 8;
    fill_multi_kernel<<<blocks, kBlock, 0, st>>>((const FillSeg *)tab, (const FillChunk *)(tab + off_c), (int)chunks.size());
    EB_LAUNCH_CHECK("gpu_fill_(batched)");
    return 0;
}

int eddlb200_fill(int dev, float *a, size_t n, float v) {
    EB_CTX(dev);
    if (a && n && v == 0.f && lz_defer(cx, st, a, n * sizeof(float))) return 0;
    return launch1(cx, st, a, a, n, FillF{v}, "gpu_fill_");
}
int eddlb200_scale(int dev, const float *a, float *b, float v, size_t n) { EB_CTX(dev); return launch1(cx, st, a, b, n, ScaleF{v}, "gpu_mult"); }
int eddlb200_addc(int dev, const float *a, float *b, float v, size_t n) { EB_CTX(dev); return launch1(cx, st, a, b, n, AddcF{v}, "gpu_add"); }
int eddlb200_sqr(int dev, const float *a, float *b, size_t n) { EB_CTX(dev); return launch1(cx, st, a, b, n, SqrF{}, "gpu_sqr"); }
int eddlb200_sqrt(int dev, const float *a, float *b, size_t n) { EB_CTX(dev); return launch1(cx, st, a, b, n, SqrtF{}, "gpu_sqrt"); }
int eddlb200_clamp(int dev, const float *a, float *b, float lo, float hi, size_t n) { EB_CTX(dev); return launch1(cx, st, a, b, n, ClampF{lo, hi}, "gpu_clamp"); }
int eddlb200_relu_fwd(int dev, const float *a, float *b, size_t n) {
    EB_CTX_KEEP_PENDING(dev);
    if (pend_copy_active(cx)) {
        PendCopy &p = pend_copy(cx);
        if (p.kind == 2 && a == p.dst && n == p.n && b && b != a && b != p.src && b != p.src2) {
            // the ReLU of a sum that is still on record: one pass writes the sum and its ReLU
            p.active = false;
            EB_READS(p.src, n * sizeof(float)); EB_READS(p.src2, n * sizeof(float));
            EB_WRITES(p.dst, n * sizeof(float)); EB_WRITES(b, n * sizeof(float));
            ProfScope prof(cx, PROF_ELEMENTWISE, 16.0 * n);          // two reads, two writes (the two adds and the ReLU it replaces move 28)
            const size_t n4 = (aligned16(p.src) && aligned16(p.src2) && aligned16(p.dst) && aligned16(b)) ? n / 4 : 0;
            map3_relu_kernel<<<grid_for(n4 ? n4 : n, kBlock), kBlock, 0, st>>>(p.src, p.src2, p.dst, b, n4, n, Sum2IntoZeroF{p.sa, p.sb, p.s2, p.t2});
            EB_LAUNCH_CHECK("gpu_add + gpu_relu");
            return 0;
        }
        if (int r = pend_copy_flush(cx, st)) return r;
    }
    return launch1(cx, st, a, b, n, ReluF{}, "gpu_relu");
}

int eddlb200_axpby(int dev, float sca, const float *a, float scb, const float *b, float *c, int inc_c, size_t n) {
    EB_CTX_KEEP_PENDING(dev);
    if (pend_copy_active(cx)) {
        PendCopy &p = pend_copy(cx);
        if (p.kind == 1 && !inc_c && c == b && c == p.dst && n == p.n && a != c && a && n) {
            // second in-place add into the buffer whose first term is still on record: both in one pass, which is itself
            // kept on record for one more call (the ReLU of the sum takes it over, anything else runs it first)
            p.kind = 2; p.src2 = a; p.s2 = sca; p.t2 = scb;
            return 0;
        }
        if (p.kind == 1 && !inc_c && c && c == b && c != p.dst && a == p.src && a != c && n == p.n && sca == p.sa && scb == p.sb && lz_any(cx)) {
            // the same source copied into a second zero destination (LAdd::backward, second parent): one pass for both
            int status = 0;
            if (lz_take(cx, st, c, n * sizeof(float), &status)) { p.kind = 3; p.dst2 = c; return 0; }
            if (status) return status;
        }
        if (int r = pend_copy_flush(cx, st)) return r;
    }
    if (inc_c && c && c != a && c != b && lz_any(cx)) {
        int status = 0;
        if (lz_take(cx, st, c, n * sizeof(float), &status)) return launch3(cx, st, a, b, c, n, AxpbyZeroF{sca, scb}, "gpu_add", 12.0);
        if (status) return status;
    }
    if (!inc_c && c && (c == b) != (c == a) && lz_any(cx)) {
        // in place on one operand (Tensor::inc on the GPU is gpu_add(1, A, 1, B, B, 0)): if that operand is known to hold
        // zeros it need not be read
        int status = 0;
        if (lz_take(cx, st, c, n * sizeof(float), &status)) {
            if (c == b) {
                // record instead of run: the next call is usually the second term of the same sum
                PendCopy &p = pend_copy(cx);
                p.active = true; p.kind = 1; p.dst = c; p.src = a; p.src2 = nullptr; p.sa = sca; p.sb = scb; p.n = n;
                return 0;
            }
            return launch1(cx, st, b, c, n, ZeroAxpbF{sca, scb}, "gpu_add", 8.0);
        }
        if (status) return status;
    }
    if (inc_c) return launch3(cx, st, a, b, c, n, AxpbyF<true>{sca, scb}, "gpu_add");
    return launch3(cx, st, a, b, c, n, AxpbyF<false>{sca, scb}, "gpu_add");
}
int eddlb200_inc(int dev, const float *a, float *b, size_t n) {
    // gpu_inc: B += A  ==  gpu_add(1, A, 1, B, B, 0) in the reference (tensor_math.cpp Tensor::inc)
    EB_CTX(dev);
    if (b && b != a && lz_any(cx)) {
        // b is known to hold zeros: 1*a + 1*0 = a + 0, one read instead of two
        int status = 0;
        if (lz_take(cx, st, b, n * sizeof(float), &status)) return launch1(cx, st, a, b, n, AddToZeroF{}, "gpu_inc", 8.0);
        if (status) return status;
    }
    return launch3(cx, st, a, b, b, n, AxpbyF<false>{1.f, 1.f}, "gpu_inc");
}
int eddlb200_el_div(int dev, const float *a, const float *b, float *c, int inc_c, size_t n) {
    EB_CTX(dev);
    if (inc_c) return launch3(cx, st, a, b, c, n, DivF<true>{}, "gpu_el_div");
    return launch3(cx, st, a, b, c, n, DivF<false>{}, "gpu_el_div");
}
int eddlb200_el_mult(int dev, const float *a, const float *b, float *c, int inc_c, size_t n) {
    EB_CTX(dev);
    if (inc_c) return launch3(cx, st, a, b, c, n, MulF<true>{}, "gpu_el_mult");
    return launch3(cx, st, a, b, c, n, MulF<false>{}, "gpu_el_mult");
}
int eddlb200_relu_bwd(int dev, const float *d, const float *i, float *pd, size_t n) {
    EB_CTX(dev);
    if (pd && pd != d && pd != i && lz_any(cx)) {
        int status = 0;
        if (lz_take(cx, st, pd, n * sizeof(float), &status)) return launch3(cx, st, d, i, pd, n, ReluBwdZeroF{}, "gpu_d_relu", 12.0);
        if (status) return status;
    }
    return launch3(cx, st, d, i, pd, n, ReluBwdF{}, "gpu_d_relu");
}
int eddlb200_cce_delta(int dev, const float *y_true, const float *y_pred, float *delta, size_t n) {
    EB_CTX(dev);
    return launch3(cx, st, y_true, y_pred, delta, n, CceDeltaF{}, "gpu_d_categorical_cross_entropy");
}

int eddlb200_pad(int dev, const float *a, float *b, int n, int c, int h, int w, int top, int bottom, int left, int right) {
    EB_CTX(dev);
    EB_REQUIRE(a && b && n >= 0 && c >= 0 && h >= 0 && w >= 0 && top >= 0 && bottom >= 0 && left >= 0 && right >= 0, "gpu_pad");
    size_t total = (size_t)n * c * h * w;
    if (!total) return 0;
    // the kernel writes the interior of b only: zeros owed to b have to be there first
    EB_READS(a, total * sizeof(float));
    EB_MODIFIES(b, (size_t)n * c * (h + top + bottom) * (w + left + right) * sizeof(float));
    ProfScope prof(cx, PROF_ELEMENTWISE, 8.0 * total);
    EB_REQUIRE(total < 0x7fffffffull, "gpu_pad: tensor larger than 2^31 elements");
    if (w % 4 == 0 && ((uintptr_t)a & 15) == 0)
        pad_kernel<false, 4><<<grid_for(total / 4, kBlock), kBlock, 0, st>>>(const_cast<float *>(a), b, (unsigned)(total / 4), h, w, top, left, h + top + bottom, w + left + right);
    else
        pad_kernel<false, 1><<<grid_for(total, kBlock), kBlock, 0, st>>>(const_cast<float *>(a), b, (unsigned)total, h, w, top, left, h + top + bottom, w + left + right);
    EB_LAUNCH_CHECK("gpu_pad");
    return 0;
}
int eddlb200_pad_bwd(int dev, float *a_delta, const float *b_delta, int n, int c, int h, int w, int top, int bottom, int left, int right) {
    EB_CTX(dev);
    EB_REQUIRE(a_delta && b_delta && n >= 0 && c >= 0 && h >= 0 && w >= 0 && top >= 0 && bottom >= 0 && left >= 0 && right >= 0, "gpu_pad_back");
    size_t total = (size_t)n * c * h * w;
    if (!total) return 0;
    EB_MODIFIES(a_delta, total * sizeof(float));
    EB_READS(b_delta, (size_t)n * c * (h + top + bottom) * (w + left + right) * sizeof(float));
    ProfScope prof(cx, PROF_ELEMENTWISE, 12.0 * total);
    EB_REQUIRE(total < 0x7fffffffull, "gpu_pad_back: tensor larger than 2^31 elements");
    if (w % 4 == 0 && ((uintptr_t)a_delta & 15) == 0)
        pad_kernel<true, 4><<<grid_for(total / 4, kBlock), kBlock, 0, st>>>(a_delta, const_cast<float *>(b_delta), (unsigned)(total / 4), h, w, top, left, h + top + bottom, w + left + right);
    else
        pad_kernel<true, 1><<<grid_for(total, kBlock), kBlock, 0, st>>>(a_delta, const_cast<float *>(b_delta), (unsigned)total, h, w, top, left, h + top + bottom, w + left + right);
    EB_LAUNCH_CHECK("gpu_pad_back");
    return 0;
}

}  // extern "C"
