// BatchNorm forward / backward for [b, z, rc] fp32 tensors (NCHW with rc = H*W).
// Replaces gpu_batchnorm_forward_{1,2,3} / gpu_batchnorm_backward_{1,2,3}
// (EDDL src/hardware/gpu/nn/gpu_bn_kernels.cu:92-204, host gpu_bn.cu:65-117); the
// arithmetic follows cpu_batchnorm_forward / cpu_batchnorm_backward
// (src/hardware/cpu/nn/cpu_bn.cpp:118-249) operation by operation.
//
// Two launches per direction, each a single streaming pass:
//   stats : grid (z, S)  every block reduces one slice of one channel with float4
//           loads and warp shuffles and stores a partial (sum, sumsq) pair;
//   apply : grid (z, S)  every block re-reduces its channel's S partials in double
//           (deterministic, no atomics), derives the per-channel constants and
//           streams its slice: normalise (+affine, + optional fused ReLU output) or
//           the backward formula.  Block y == 0 also writes the per-channel outputs.
// Algorithmic traffic: forward 16 B/element (x twice, opa, y), backward 24 B/element
// (+4 for the in-place `delta *= gamma` the reference performs).
#include <mutex>
#include "common.cuh"

namespace {

using namespace eb;

constexpr int kBlock = 256;
constexpr int kMaxSplit = 256;

struct Slice { unsigned begin, end; };   // element range inside one channel's b*rc items

__device__ __forceinline__ Slice slice_of(unsigned per_channel, unsigned nsplit, unsigned s) {
    // chunk is a multiple of 4 so float4 accesses never straddle slices
    unsigned chunk = ((per_channel + nsplit - 1) / nsplit + 3u) & ~3u;
    Slice r;
    r.begin = min(s * chunk, per_channel);
    r.end = min(r.begin + chunk, per_channel);
    return r;
}

// offset of item t (= i*rc + l) of channel j inside the [b, z, rc] tensor
__device__ __forceinline__ size_t item_offset(unsigned t, unsigned rc, unsigned z, unsigned j) {
    unsigned i = t / rc, l = t - i * rc;
    return ((size_t)i * z + j) * rc + l;
}

// ---- reductions -----------------------------------------------------------------
// MODE 0: (sum x, sum x*x)      MODE 1: (sum d*o, sum d)
template <int MODE, bool VEC>
__global__ void __launch_bounds__(kBlock) bn_stats_kernel(const float *__restrict__ x, const float *__restrict__ o,
                                                          float2 *__restrict__ partial, unsigned b, unsigned z, unsigned rc) {
    __shared__ float sm[32];
    const unsigned j = blockIdx.x, s = blockIdx.y, nsplit = gridDim.y;
    const Slice sl = slice_of(b * rc, nsplit, s);
    float a0 = 0.f, a1 = 0.f;
    if (VEC) {
#pragma unroll 4
        for (unsigned t = sl.begin + threadIdx.x * 4; t < sl.end; t += kBlock * 4) {
            const size_t off = item_offset(t, rc, z, j);
            const float4 v = ldg4(x + off);           // left in L2 on purpose: the apply pass walks its slice backwards
            if (MODE == 0) {
                a0 += (v.x + v.y) + (v.z + v.w);
                a1 += (v.x * v.x + v.y * v.y) + (v.z * v.z + v.w * v.w);
            } else {
                const float4 w = ldg4(o + off);
                a0 += (v.x * w.x + v.y * w.y) + (v.z * w.z + v.w * w.w);
                a1 += (v.x + v.y) + (v.z + v.w);
            }
        }
    } else {
        for (unsigned t = sl.begin + threadIdx.x; t < sl.end; t += kBlock) {
            const size_t off = item_offset(t, rc, z, j);
            const float v = x[off];
            if (MODE == 0) { a0 += v; a1 += v * v; }
            else { a0 += v * o[off]; a1 += v; }
        }
    }
    a0 = block_sum(a0, sm);
    a1 = block_sum(a1, sm);
    if (threadIdx.x == 0) partial[(size_t)j * nsplit + s] = make_float2(a0, a1);
}

__device__ __forceinline__ void reduce_partials(const float2 *partial, unsigned j, unsigned nsplit, float *sh, float &s0, float &s1) {
    // nsplit <= kMaxSplit <= blockDim.x ; combine in double, round once
    double d0 = 0.0, d1 = 0.0;
    if (threadIdx.x < 32) {
        for (unsigned s = threadIdx.x; s < nsplit; s += 32) {
            const float2 p = partial[(size_t)j * nsplit + s];
            d0 += (double)p.x; d1 += (double)p.y;
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            d0 += __shfl_xor_sync(0xffffffffu, d0, o);
            d1 += __shfl_xor_sync(0xffffffffu, d1, o);
        }
        if (threadIdx.x == 0) { sh[0] = (float)d0; sh[1] = (float)d1; }
    }
    __syncthreads();
    s0 = sh[0]; s1 = sh[1];
}

// ---- forward apply ----------------------------------------------------------------
template <bool TRAIN, bool VEC>
__global__ void __launch_bounds__(kBlock) bn_fwd_apply_kernel(const float *__restrict__ x, float *__restrict__ y, float *__restrict__ opa,
                                                              float *__restrict__ relu_out,
                                                              const float2 *__restrict__ partial,
                                                              float *global_mean, float *global_var,
                                                              const float *__restrict__ g, const float *__restrict__ beta,
                                                              float *mean_out, float *var_out,
                                                              unsigned b, unsigned z, unsigned rc, float eps, float momentum) {
    __shared__ float sh[2];
    // slices in reverse launch order: the statistics pass finished with the highest slices, so those are what the L2 holds
    const unsigned j = blockIdx.x, nsplit = gridDim.y, s = nsplit - 1 - blockIdx.y;
    float mean, sigma;
    if (TRAIN) {
        float sum, sumsq;
        reduce_partials(partial, j, nsplit, sh, sum, sumsq);
        const float N = (float)(b * rc);                               // float N = b * rc;
        mean = __fdiv_rn(sum, N);                                      // mean[j] / N
        const float var = __fsub_rn(__fdiv_rn(sumsq, N), __fmul_rn(mean, mean));
        sigma = __fsqrt_rn(__fadd_rn(var, eps));                       // sqrt(variance[j] + epsilon)
        if (s == 0 && threadIdx.x == 0) {
            if (momentum != 0.0f) {
                // momentum * global[j] is a float product; (1.0 - momentum) * stat is double
                const double keep = 1.0 - (double)momentum;
                global_mean[j] = (float)((double)__fmul_rn(momentum, global_mean[j]) + keep * (double)mean);
                global_var[j] = (float)((double)__fmul_rn(momentum, global_var[j]) + keep * (double)var);
            }
            mean_out[j] = mean;
            var_out[j] = sigma;
        }
    } else {
        mean = global_mean[j];
        sigma = __fsqrt_rn(__fadd_rn(global_var[j], eps));
        if (s == 0 && threadIdx.x == 0) var_out[j] = sigma;
    }
    const bool affine = (g != nullptr);
    const float gj = affine ? g[j] : 1.f, bj = affine ? beta[j] : 0.f;
    const Slice sl = slice_of(b * rc, nsplit, s);
    if (VEC) {
#pragma unroll 4
        // Backwards through the slice: the statistics pass read it forwards just before, so its tail is what the L2 still
        // holds; the second read of tensors up to about the L2 size then costs no HBM traffic.
        for (unsigned it = (sl.end - sl.begin + kBlock * 4 - 1) / (kBlock * 4); it-- > 0;) {
            const unsigned t = sl.begin + it * (kBlock * 4) + threadIdx.x * 4;
            if (t >= sl.end) continue;
            const size_t off = item_offset(t, rc, z, j);
            const float4 v = ld_stream4(x + off);
            float4 o, r;
            o.x = __fdiv_rn(__fsub_rn(v.x, mean), sigma); o.y = __fdiv_rn(__fsub_rn(v.y, mean), sigma);
            o.z = __fdiv_rn(__fsub_rn(v.z, mean), sigma); o.w = __fdiv_rn(__fsub_rn(v.w, mean), sigma);
            if (affine) {
                *reinterpret_cast<float4 *>(opa + off) = o;
                r.x = __fadd_rn(__fmul_rn(o.x, gj), bj); r.y = __fadd_rn(__fmul_rn(o.y, gj), bj);
                r.z = __fadd_rn(__fmul_rn(o.z, gj), bj); r.w = __fadd_rn(__fmul_rn(o.w, gj), bj);
            } else {
                r = o;
            }
            *reinterpret_cast<float4 *>(y + off) = r;
            if (relu_out) {
                r.x = r.x > 0.f ? r.x : 0.f; r.y = r.y > 0.f ? r.y : 0.f; r.z = r.z > 0.f ? r.z : 0.f; r.w = r.w > 0.f ? r.w : 0.f;
                *reinterpret_cast<float4 *>(relu_out + off) = r;
            }
        }
    } else {
        for (unsigned it = (sl.end - sl.begin + kBlock - 1) / kBlock; it-- > 0;) {
            const unsigned t = sl.begin + it * kBlock + threadIdx.x;
            if (t >= sl.end) continue;
            const size_t off = item_offset(t, rc, z, j);
            const float o = __fdiv_rn(__fsub_rn(x[off], mean), sigma);
            float r = o;
            if (affine) { opa[off] = o; r = __fadd_rn(__fmul_rn(o, gj), bj); }
            y[off] = r;
            if (relu_out) relu_out[off] = r > 0.f ? r : 0.f;
        }
    }
}

// ---- backward apply ---------------------------------------------------------------
// PD_ZERO: the parent delta is known to hold zeros, so it is written without being read (0 + x keeps the bits of the
// read-modify-write form).
template <bool VEC, bool PD_ZERO>
__global__ void __launch_bounds__(kBlock) bn_bwd_apply_kernel(float *__restrict__ delta, const float *__restrict__ opa, float *__restrict__ pdelta,
                                                              const float2 *__restrict__ partial,
                                                              float *gbn_g, float *gbn_b, const float *__restrict__ bn_g,
                                                              const float *__restrict__ variance, float *mean1, float *mean2,
                                                              unsigned b, unsigned z, unsigned rc) {
    __shared__ float sh[2];
    const unsigned j = blockIdx.x, nsplit = gridDim.y, s = nsplit - 1 - blockIdx.y;     // reverse launch order, see forward
    float s1, s2;
    reduce_partials(partial, j, nsplit, sh, s1, s2);
    const float N = (float)(b * rc);
    float m1 = __fdiv_rn(s1, N), m2 = __fdiv_rn(s2, N);
    const bool affine = (bn_g != nullptr);
    const float gj = affine ? bn_g[j] : 1.f;
    if (s == 0 && threadIdx.x == 0 && affine) {
        gbn_g[j] = __fadd_rn(gbn_g[j], m1);      // gradients of gamma/beta are MEANS in the reference
        gbn_b[j] = __fadd_rn(gbn_b[j], m2);
    }
    if (affine) { m1 = __fmul_rn(m1, gj); m2 = __fmul_rn(m2, gj); }
    if (s == 0 && threadIdx.x == 0) { mean1[j] = m1; mean2[j] = m2; }
    const float sigma = variance[j];
    const Slice sl = slice_of(b * rc, nsplit, s);
    if (VEC) {
#pragma unroll 4
        // Backwards through the slice: the statistics pass read it forwards just before, so its tail is what the L2 still
        // holds; the second read of tensors up to about the L2 size then costs no HBM traffic.
        for (unsigned it = (sl.end - sl.begin + kBlock * 4 - 1) / (kBlock * 4); it-- > 0;) {
            const unsigned t = sl.begin + it * (kBlock * 4) + threadIdx.x * 4;
            if (t >= sl.end) continue;
            const size_t off = item_offset(t, rc, z, j);
            float4 d = *reinterpret_cast<const float4 *>(delta + off);
            const float4 o = ld_stream4(opa + off);
            float4 p = PD_ZERO ? make_float4(0.f, 0.f, 0.f, 0.f) : *reinterpret_cast<const float4 *>(pdelta + off);
            if (affine) {
                d.x = __fmul_rn(d.x, gj); d.y = __fmul_rn(d.y, gj); d.z = __fmul_rn(d.z, gj); d.w = __fmul_rn(d.w, gj);
                *reinterpret_cast<float4 *>(delta + off) = d;            // delta[p] *= bn_g[j]
            }
            p.x = __fadd_rn(p.x, __fdiv_rn(__fsub_rn(d.x, __fadd_rn(__fmul_rn(o.x, m1), m2)), sigma));
            p.y = __fadd_rn(p.y, __fdiv_rn(__fsub_rn(d.y, __fadd_rn(__fmul_rn(o.y, m1), m2)), sigma));
            p.z = __fadd_rn(p.z, __fdiv_rn(__fsub_rn(d.z, __fadd_rn(__fmul_rn(o.z, m1), m2)), sigma));
            p.w = __fadd_rn(p.w, __fdiv_rn(__fsub_rn(d.w, __fadd_rn(__fmul_rn(o.w, m1), m2)), sigma));
            *reinterpret_cast<float4 *>(pdelta + off) = p;
        }
    } else {
        for (unsigned it = (sl.end - sl.begin + kBlock - 1) / kBlock; it-- > 0;) {
            const unsigned t = sl.begin + it * kBlock + threadIdx.x;
            if (t >= sl.end) continue;
            const size_t off = item_offset(t, rc, z, j);
            float d = delta[off];
            if (affine) { d = __fmul_rn(d, gj); delta[off] = d; }
            pdelta[off] = __fadd_rn(PD_ZERO ? 0.f : pdelta[off], __fdiv_rn(__fsub_rn(d, __fadd_rn(__fmul_rn(opa[off], m1), m2)), sigma));
        }
    }
}

// Slices per channel.  A launch is cut into several waves of short-lived blocks (g_bn_waves times the 8 blocks of 256 threads
// an SM holds): with barely more blocks than the GPU holds at once, the few left over for a second wave run almost alone
// at a fraction of the bandwidth while the rest of the GPU idles.
int g_bn_waves = 16, g_bn_min_items = 8192;
inline unsigned pick_split(unsigned z, unsigned per_channel) {
    unsigned want = (EDDLB200_NUM_SMS * 8 * (unsigned)g_bn_waves + z - 1) / z;
    unsigned cap = (per_channel + (unsigned)g_bn_min_items - 1) / (unsigned)g_bn_min_items;
    unsigned s = want < cap ? want : cap;
    if (s < 1) s = 1;
    if (s > kMaxSplit) s = kMaxSplit;
    return s;
}

}  // namespace

namespace eb {
// tuning knobs behind eddlb200_set_option("bn_waves" / "bn_min_items")
int bn_set_tuning(int waves, int min_items) {
    if (waves > 0) g_bn_waves = waves > 64 ? 64 : waves;
    if (min_items > 0) g_bn_min_items = min_items < 1024 ? 1024 : min_items;
    return 0;
}
}  // namespace eb

using namespace eb;

extern "C" {

int eddlb200_bn_fwd(int dev, int b, int z, int rc, const float *input, float *output, float *opa,
                    float *global_mean, float *global_variance, const float *affine_g, const float *affine_b,
                    float *mean, float *variance, int trmode, float epsilon, float momentum, float *relu_out) {
    EB_CTX(dev);
    EB_REQUIRE(b > 0 && z > 0 && rc > 0 && input && output && global_mean && global_variance && variance, "gpu_batchnorm_forward");
    EB_REQUIRE((size_t)b * rc < 0xfffffff0u, "gpu_batchnorm_forward");
    EB_REQUIRE(!affine_g || (affine_b && opa), "gpu_batchnorm_forward");
    EB_REQUIRE(!trmode || mean, "gpu_batchnorm_forward");
    {
        const size_t tb = (size_t)b * z * rc * sizeof(float), zb = (size_t)z * sizeof(float);
        EB_READS(input, tb); EB_WRITES(output, tb); EB_WRITES(opa, tb); EB_WRITES(relu_out, tb);
        EB_MODIFIES(global_mean, zb); EB_MODIFIES(global_variance, zb); EB_READS(affine_g, zb); EB_READS(affine_b, zb);
        EB_MODIFIES(mean, zb); EB_MODIFIES(variance, zb);
    }
    // algorithmic bytes per element: x once per pass (two passes when the batch statistics are computed), y, and the two
    // optional outputs -- opa (the normalised value BN backward needs) and the ReLU of y written for the layer that follows
    ProfScope prof(cx, PROF_BN_FWD, ((trmode ? 8.0 : 4.0) + 4.0 + (opa ? 4.0 : 0.0) + (relu_out ? 4.0 : 0.0)) * b * (double)z * rc);
    const unsigned per = (unsigned)b * rc, S = pick_split(z, per);
    const bool vec = (rc % 4 == 0) && aligned16(input) && aligned16(output) && (!opa || aligned16(opa)) && (!relu_out || aligned16(relu_out));
    dim3 grid(z, S);
    float2 *partial = nullptr;
    if (trmode) {
        partial = (float2 *)scratch(cx, (size_t)z * S * sizeof(float2));
        if (!partial) return cudaErrorMemoryAllocation;
        if (vec) bn_stats_kernel<0, true><<<grid, kBlock, 0, st>>>(input, nullptr, partial, b, z, rc);
        else bn_stats_kernel<0, false><<<grid, kBlock, 0, st>>>(input, nullptr, partial, b, z, rc);
        EB_LAUNCH_CHECK("gpu_batchnorm_forward(stats)");
        if (vec) bn_fwd_apply_kernel<true, true><<<grid, kBlock, 0, st>>>(input, output, opa, relu_out, partial, global_mean, global_variance, affine_g, affine_b, mean, variance, b, z, rc, epsilon, momentum);
        else bn_fwd_apply_kernel<true, false><<<grid, kBlock, 0, st>>>(input, output, opa, relu_out, partial, global_mean, global_variance, affine_g, affine_b, mean, variance, b, z, rc, epsilon, momentum);
    } else {
        if (vec) bn_fwd_apply_kernel<false, true><<<grid, kBlock, 0, st>>>(input, output, opa, relu_out, nullptr, global_mean, global_variance, affine_g, affine_b, mean, variance, b, z, rc, epsilon, momentum);
        else bn_fwd_apply_kernel<false, false><<<grid, kBlock, 0, st>>>(input, output, opa, relu_out, nullptr, global_mean, global_variance, affine_g, affine_b, mean, variance, b, z, rc, epsilon, momentum);
    }
    EB_LAUNCH_CHECK("gpu_batchnorm_forward(apply)");
    return 0;
}

int eddlb200_bn_bwd(int dev, int b, int z, int rc, float *delta, const float *opa, float *pdelta,
                    float *gbn_g, float *gbn_b, const float *bn_g, const float *variance, float *mean1, float *mean2) {
    EB_CTX(dev);
    EB_REQUIRE(b > 0 && z > 0 && rc > 0 && delta && opa && pdelta && variance && mean1 && mean2, "gpu_batchnorm_backward");
    EB_REQUIRE((size_t)b * rc < 0xfffffff0u, "gpu_batchnorm_backward");
    EB_REQUIRE(!bn_g || (gbn_g && gbn_b), "gpu_batchnorm_backward");
    bool pd_zero = false;
    {
        const size_t tb = (size_t)b * z * rc * sizeof(float), zb = (size_t)z * sizeof(float);
        EB_MODIFIES(delta, tb); EB_READS(opa, tb);
        EB_MODIFIES(gbn_g, zb); EB_MODIFIES(gbn_b, zb); EB_READS(bn_g, zb); EB_READS(variance, zb); EB_MODIFIES(mean1, zb); EB_MODIFIES(mean2, zb);
        EB_NOTES(pdelta, tb);
        if (lz_any(cx) && pdelta != delta && pdelta != opa) {
            int status = 0;
            pd_zero = lz_take(cx, st, pdelta, tb, &status);
            if (status) return status;
        }
    }
    ProfScope prof(cx, PROF_BN_BWD, 24.0 * b * (double)z * rc);     // canonical count; the pd_zero variant moves 20 B/element
    const unsigned per = (unsigned)b * rc, S = pick_split(z, per);
    const bool vec = (rc % 4 == 0) && aligned16(delta) && aligned16(opa) && aligned16(pdelta);
    dim3 grid(z, S);
    float2 *partial = (float2 *)scratch(cx, (size_t)z * S * sizeof(float2));
    if (!partial) return cudaErrorMemoryAllocation;
    if (vec) bn_stats_kernel<1, true><<<grid, kBlock, 0, st>>>(delta, opa, partial, b, z, rc);
    else bn_stats_kernel<1, false><<<grid, kBlock, 0, st>>>(delta, opa, partial, b, z, rc);
    EB_LAUNCH_CHECK("gpu_batchnorm_backward(stats)");
    if (vec && pd_zero) bn_bwd_apply_kernel<true, true><<<grid, kBlock, 0, st>>>(delta, opa, pdelta, partial, gbn_g, gbn_b, bn_g, variance, mean1, mean2, b, z, rc);
    else if (vec) bn_bwd_apply_kernel<true, false><<<grid, kBlock, 0, st>>>(delta, opa, pdelta, partial, gbn_g, gbn_b, bn_g, variance, mean1, mean2, b, z, rc);
    else if (pd_zero) bn_bwd_apply_kernel<false, true><<<grid, kBlock, 0, st>>>(delta, opa, pdelta, partial, gbn_g, gbn_b, bn_g, variance, mean1, mean2, b, z, rc);
    else bn_bwd_apply_kernel<false, false><<<grid, kBlock, 0, st>>>(delta, opa, pdelta, partial, gbn_g, gbn_b, bn_g, variance, mean1, mean2, b, z, rc);
    EB_LAUNCH_CHECK("gpu_batchnorm_backward(apply)");
    return 0;
}

}  // extern "C"

// ---------------------------------------------------------------------------------------------
// BatchNorm forward for callers that are not allowed to allocate device memory.
//
// eddlb200_bn_fwd keeps its per-channel partial sums in the library's growable scratch arena,
// which it obtains with cudaMalloc the first time (and whenever a larger one is needed), and the
// device context behind it also allocates on first use.  Some hosts cannot tolerate that: a
// process whose device memory has been handed over in full to another allocator (a cudaMalloc
// from a plug-in then fails or fragments that pool), or a latency-critical loop in which the
// implicit device synchronisation of cudaMalloc / cudaFree is not acceptable.  For them this
// entry point runs the same two kernels with the partial sums in a fixed array that is part of
// the library image: kNoAllocPairs (sum, sum-of-squares) pairs = 2 MiB of device memory, held by
// every GPU that loads the library until the process exits.
//
// * It calls no cudaMalloc / cudaFree / cudaMallocHost and does not create the library's device
//   context; the caller supplies the stream.
// * The array's name is only a host-side handle.  Its device address is looked up once per
//   device with cudaGetSymbolAddress while that device is current; this happens inside the FIRST
//   call on each device, so make that first call before any stream capture begins.
// * Shapes that need more than kNoAllocPairs partial pairs (channels x slices) are rejected with
//   EDDLB200_ELIMIT.
// * All calls on a device share the one array and it keeps whatever the last call left there.
//   Nothing has to be cleared between calls: the statistics kernel overwrites every pair the
//   apply kernel reads.  Two calls that overlap on the GPU (different streams, no ordering) race
//   on the array and give wrong statistics; order them.
namespace {

constexpr unsigned kNoAllocPairs = 262144u;               // float2 pairs = 2 MiB
static __device__ __align__(256) float2 g_noalloc_partials[kNoAllocPairs];

float2 *g_noalloc_addr[EDDLB200_MAX_DEVICES] = {};
std::mutex g_noalloc_mu;

// Device address of g_noalloc_partials on `dev` (which must be current); nullptr + error text on failure.
float2 *noalloc_scratch(int dev) {
    std::lock_guard<std::mutex> lk(g_noalloc_mu);
    if (g_noalloc_addr[dev]) return g_noalloc_addr[dev];
    void *p = nullptr;
    const cudaError_t e = cudaGetSymbolAddress(&p, g_noalloc_partials);
    if (e != cudaSuccess || !p) {
        cuda_status(e == cudaSuccess ? cudaErrorInvalidSymbol : e, "eddlb200_bn_fwd_noalloc(cudaGetSymbolAddress)");
        return nullptr;
    }
    g_noalloc_addr[dev] = (float2 *)p;
    return g_noalloc_addr[dev];
}

}  // namespace

extern "C" int eddlb200_bn_fwd_noalloc(int dev, int b, int z, int rc, const float *input, float *output, float *opa,
                                       float *global_mean, float *global_variance, const float *affine_g, const float *affine_b,
                                       float *mean, float *variance, int trmode, float epsilon, float momentum, float *relu_out,
                                       void *cuda_stream) {
    if (dev < 0 || dev >= EDDLB200_MAX_DEVICES) return set_error(EDDLB200_ENOINIT, "bn_fwd_noalloc: device ordinal %d out of range", dev);
    if (!(b > 0 && z > 0 && rc > 0 && input && output && global_mean && global_variance && variance) ||
        (affine_g && !(affine_b && opa)) || (trmode && !mean) || (size_t)b * rc >= 0xfffffff0u)
        return set_error(EDDLB200_EINVAL, "bn_fwd_noalloc: bad argument");
    const unsigned per = (unsigned)b * rc, S = pick_split(z, per);
    if (trmode && (size_t)z * S > kNoAllocPairs)          // inference reads no partial sums
        return set_error(EDDLB200_ELIMIT, "bn_fwd_noalloc: %d channels x %u slices need %zu partial pairs, the built-in scratch holds %u",
                         z, S, (size_t)z * S, kNoAllocPairs);
    cudaError_t e = cudaSetDevice(dev);
    if (e != cudaSuccess) return cuda_status(e, "bn_fwd_noalloc(cudaSetDevice)");
    float2 *partial = noalloc_scratch(dev);
    if (!partial) return EDDLB200_ENOINIT;
    const cudaStream_t caller = (cudaStream_t)cuda_stream;
    if (DevCtx *cx = ctx_peek(dev)) {
        // A device context exists.  It may owe deferred zeros or a recorded copy -- possibly to buffers this call never
        // sees -- and that work belongs on the library's compute stream, where whatever produces its operands runs.  It
        // is settled THERE; when the caller's stream is a different one, an event that exists since the context was
        // created is recorded behind it and the caller's stream waits on it, so the kernels below run after the settled
        // work and after everything the library had enqueued (nothing is created or allocated on this path).
        const cudaStream_t st = stream_of(cx);
        if (pend_copy_active(cx)) { if (int r = pend_copy_flush(cx, st)) return r; }
        const size_t tb = (size_t)b * z * rc * sizeof(float), zb = (size_t)z * sizeof(float);
        EB_READS(input, tb); EB_WRITES(output, tb); EB_WRITES(opa, tb); EB_WRITES(relu_out, tb);
        EB_MODIFIES(global_mean, zb); EB_MODIFIES(global_variance, zb); EB_READS(affine_g, zb); EB_READS(affine_b, zb);
        EB_MODIFIES(mean, zb); EB_MODIFIES(variance, zb);
        if (caller != st) {
            if ((e = cudaEventRecord(handoff_event(cx), st)) != cudaSuccess) return cuda_status(e, "bn_fwd_noalloc(record)");
            if ((e = cudaStreamWaitEvent(caller, handoff_event(cx), 0)) != cudaSuccess) return cuda_status(e, "bn_fwd_noalloc(wait)");
        }
    }
    const cudaStream_t st = caller;
    const bool vec = (rc % 4 == 0) && aligned16(input) && aligned16(output) && (!opa || aligned16(opa)) && (!relu_out || aligned16(relu_out));
    dim3 grid(z, S);
    if (trmode) {
        if (vec) bn_stats_kernel<0, true><<<grid, kBlock, 0, st>>>(input, nullptr, partial, b, z, rc);
        else bn_stats_kernel<0, false><<<grid, kBlock, 0, st>>>(input, nullptr, partial, b, z, rc);
        if ((e = cudaGetLastError()) != cudaSuccess) return cuda_status(e, "bn_fwd_noalloc(stats)");
        if (vec) bn_fwd_apply_kernel<true, true><<<grid, kBlock, 0, st>>>(input, output, opa, relu_out, partial, global_mean, global_variance, affine_g, affine_b, mean, variance, b, z, rc, epsilon, momentum);
        else bn_fwd_apply_kernel<true, false><<<grid, kBlock, 0, st>>>(input, output, opa, relu_out, partial, global_mean, global_variance, affine_g, affine_b, mean, variance, b, z, rc, epsilon, momentum);
    } else {
        if (vec) bn_fwd_apply_kernel<false, true><<<grid, kBlock, 0, st>>>(input, output, opa, relu_out, nullptr, global_mean, global_variance, affine_g, affine_b, mean, variance, b, z, rc, epsilon, momentum);
        else bn_fwd_apply_kernel<false, false><<<grid, kBlock, 0, st>>>(input, output, opa, relu_out, nullptr, global_mean, global_variance, affine_g, affine_b, mean, variance, b, z, rc, epsilon, momentum);
    }
    if ((e = cudaGetLastError()) != cudaSuccess) return cuda_status(e, "bn_fwd_noalloc(apply)");
    return 0;
}
