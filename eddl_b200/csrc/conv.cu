// Conv2D C-ABI entry points: argument checks, kernel selection, bias gradient,
// split-K combine.  See conv_tc.cu (tcgen05 tensor-core path) and conv_simt.cu
// (exact-fp32 FMA path).
#include <cstdint>
#include <cstdlib>
#include <cstring>
#include "common.cuh"
#include "conv_common.cuh"

namespace {

using namespace eb;

__global__ void __launch_bounds__(256) splitk_reduce_kernel(const float *__restrict__ part, float *__restrict__ out, size_t count, int splits) {
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < count; i += stride) {
        float s = 0.f;
        for (int z = 0; z < splits; z++) s += part[(size_t)z * count + i];
        out[i] = __fadd_rn(out[i], s);
    }
}

// gbias[k] += sum_{n,p,q} dy[n,k,p,q]   (cpu_conv2D_grad, src/hardware/cpu/nn/cpu_conv.cpp:466-478)
__global__ void __launch_bounds__(256) bias_grad_kernel(const float *__restrict__ dy, float *__restrict__ gbias, int n, int k, int pq) {
    __shared__ float sm[32];
    const int kk = blockIdx.x;
    float s = 0.f;
    const long long total = (long long)n * pq;
    for (long long t = threadIdx.x; t < total; t += blockDim.x) {
        const int img = (int)(t / pq), r = (int)(t - (long long)img * pq);
        s += dy[((size_t)img * k + kk) * pq + r];
    }
    s = block_sum(s, sm);
    if (threadIdx.x == 0) gbias[kk] = __fadd_rn(gbias[kk], s);
}

// ---- 1x1 convolutions that skip pixels (stride > 1) or whose planes are not a multiple of four pixels long ----
// Such a layer is a dense 1x1 stride-1 convolution over the pixels it actually reads.  Gathering those pixels into a dense
// [image][channel][pitch] copy (pitch = pixels rounded up to four, the tail zero) is one pass over the smaller tensor, after which
// the TMA-fed kernels apply: the strided kernels spend most of their time computing addresses, the copy moves a few tens of MB.
// dst plane: rows of `ow` elements of which the first `vw` come from the source (the rest are zero), npix elements in all
__global__ void __launch_bounds__(256) plane_gather_kernel(const float *__restrict__ src, float *__restrict__ dst, unsigned total,
                                                           int ihw, int iw, int sr, int sc, int ow, int vw, int npix, int pitch) {
    const unsigned stride = gridDim.x * blockDim.x;
    for (unsigned idx = blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += stride) {
        const unsigned plane = idx / (unsigned)pitch, p = idx - plane * pitch;
        float v = 0.f;
        if (p < (unsigned)npix) {
            const unsigned oy = p / (unsigned)ow, ox = p - oy * ow;
            if (ox < (unsigned)vw) v = src[(size_t)plane * ihw + oy * sr * iw + ox * sc];
        }
        dst[idx] = v;
    }
}

// dx (full resolution) += the dense result at the pixels the convolution read; the others are left alone
__global__ void __launch_bounds__(256) plane_scatter_add_kernel(const float *__restrict__ dense, float *__restrict__ dst, unsigned total,
                                                                int ihw, int iw, int sr, int sc, int ow, int npix, int pitch) {
    const unsigned stride = gridDim.x * blockDim.x;
    for (unsigned idx = blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += stride) {
        const unsigned plane = idx / (unsigned)pitch, p = idx - plane * pitch;
        if (p >= (unsigned)npix) continue;
        const unsigned oy = p / (unsigned)ow, ox = p - oy * ow;
        float *d = dst + (size_t)plane * ihw + oy * sr * iw + ox * sc;
        *d = __fadd_rn(*d, dense[idx]);
    }
}

// dx = the dense result at those pixels and zero everywhere else: every element of dx is written.  V = elements per thread
// (4 when rows are a multiple of four pixels long and dx is 16-byte aligned)
template <int V>
__global__ void __launch_bounds__(256) plane_scatter_store_kernel(const float *__restrict__ dense, float *__restrict__ dst, unsigned total_v,
                                                                  int ihw, int iw, int sr, int sc, int oh, int ow, int pitch) {
    const unsigned stride = gridDim.x * blockDim.x, ihw_v = ihw / V, iw_v = iw / V;
    for (unsigned idx = blockIdx.x * blockDim.x + threadIdx.x; idx < total_v; idx += stride) {
        const unsigned plane = idx / ihw_v, r = idx - plane * ihw_v, y = r / iw_v, x0 = (r - y * iw_v) * V, oy = y / (unsigned)sr;
        const bool row_hit = oy * sr == y && oy < (unsigned)oh;
        float v[V];
#pragma unroll
        for (int e = 0; e < V; e++) {
            const unsigned x = x0 + e, ox = x / (unsigned)sc;
            v[e] = (row_hit && ox * sc == x && ox < (unsigned)ow) ? dense[(size_t)plane * pitch + oy * ow + ox] : 0.f;
        }
        if (V == 4) reinterpret_cast<float4 *>(dst)[idx] = make_float4(v[0], v[1], v[2], v[3]);
        else dst[idx] = v[0];
    }
}

struct Dense1x1 { bool on; bool ragged; int pitch; ConvGeom g; };

int g_conv_dense = 1;          // eddlb200_set_option("conv_dense_1x1", 0 / 1)

// Conv2D calls served by the tensor-core kernels [0] and by the fp32 FMA kernels [1], per device: a caller can tell whether
// any layer of its net left the tensor-core path (a shape the kernel does not take, or the path forced by an option)
unsigned long long g_conv_calls[EDDLB200_MAX_DEVICES][2] = {};

// exact_out: the output tensor (forward) or dy (backward-data) is used where it lies, so its planes must already be dense
Dense1x1 dense_1x1(const ConvGeom &g, bool exact_out) {
    Dense1x1 d{false, false, 0, g};
    const int pq = g.oh * g.ow;
    if (!g_conv_dense || g.kr != 1 || g.kc != 1 || g.pt != 0 || g.pl != 0 || g.c < 32 || g.k < 32 || pq < 32) return d;
    if ((g.oh - 1) * g.sr >= g.ih || (g.ow - 1) * g.sc >= g.iw) return d;
    const bool strided = g.sr > 1 || g.sc > 1;
    d.ragged = pq % 4 != 0;
    if (!strided && !d.ragged) return d;                        // dense already
    if (d.ragged && exact_out) return d;
    d.pitch = (pq + 3) & ~3;
    if (d.pitch >= 16000 && d.ragged) return d;
    d.g.sr = d.g.sc = 1;
    d.g.ih = d.g.oh = d.ragged ? 1 : g.oh;
    d.g.iw = d.g.ow = d.ragged ? d.pitch : g.ow;
    d.on = true;
    return d;
}

// device buffers for the dense copies: slot 0 = gathered x, 1 = gathered dy, 2 = dense dx.  They only grow.
float *dense_buf(cudaStream_t st, int slot, size_t bytes) {
    static float *buf[EDDLB200_MAX_DEVICES][3] = {}; static size_t cap[EDDLB200_MAX_DEVICES][3] = {};
    int dev = 0; cudaGetDevice(&dev);
    if (cap[dev][slot] < bytes) {
        cudaStreamSynchronize(st);
        if (buf[dev][slot]) cudaFree(buf[dev][slot]);
        buf[dev][slot] = nullptr; cap[dev][slot] = 0;
        if (cudaMalloc(&buf[dev][slot], bytes) != cudaSuccess) { cudaGetLastError(); return nullptr; }
        cap[dev][slot] = bytes;
    }
    return buf[dev][slot];
}

int gather_planes(DevCtx *cx, cudaStream_t st, const float *src, float *dst, size_t planes, int ih, int iw, int sr, int sc, int oh, int ow, int pitch,
                  int valid_w = -1) {
    const unsigned total = (unsigned)(planes * pitch);
    plane_gather_kernel<<<grid_for(total, 256), 256, 0, st>>>(src, dst, total, ih * iw, iw, sr, sc, ow, valid_w < 0 ? ow : valid_w, oh * ow, pitch);
    EB_LAUNCH_CHECK("conv2D(gather)");
    return 0;
}

int check(const char *what, const ConvGeom &g) {
    if (g.n < 0 || g.c <= 0 || g.ih <= 0 || g.iw <= 0 || g.k <= 0 || g.kr <= 0 || g.kc <= 0 || g.oh <= 0 || g.ow <= 0 ||
        g.sr <= 0 || g.sc <= 0 || g.pt < 0 || g.pl < 0)
        return set_error(EDDLB200_EINVAL, "%s: bad geometry", what);
    if ((long long)g.n * g.c * g.ih * g.iw >= 0x7fffffffLL || (long long)g.n * g.k * g.oh * g.ow >= 0x7fffffffLL ||
        (long long)g.k * g.c * g.kr * g.kc >= 0x7fffffffLL)
        return set_error(EDDLB200_ELIMIT, "%s: tensor larger than 2^31 elements", what);
    return 0;
}

// EDDL_B200_CONV=simt (or eddlb200_set_option("conv_path", 1)) forces the FMA path; tests use it to
// compare the two paths.
int g_conv_path = -1;
bool tc_enabled() {
    if (g_conv_path < 0) { const char *e = getenv("EDDL_B200_CONV"); g_conv_path = (e && e[0] == 's') ? 1 : 0; }
    return g_conv_path == 0;
}

}  // namespace

namespace eb {
bool conv_tc_allowed() { return tc_enabled(); }
int splitk_reduce_accumulate(DevCtx *cx, cudaStream_t st, const float *part, float *out, size_t count, int splits) {
    splitk_reduce_kernel<<<grid_for(count, 256), 256, 0, st>>>(part, out, count, splits);
    EB_LAUNCH_CHECK("splitk_reduce");
    return 0;
}
}  // namespace eb

using namespace eb;

extern "C" {

int eddlb200_set_option(const char *name, int value) {
    if (name && !strcmp(name, "conv_path") && (value == 0 || value == 1)) { g_conv_path = value; return 0; }
    if (name && !strcmp(name, "lazy_zero") && (value == 0 || value == 1)) return lz_set_all(value);
    if (name && !strcmp(name, "conv_prefetch") && (value == 0 || value == 1)) return conv_tc_set_prefetch(value);
    if (name && !strcmp(name, "conv_tma") && value >= 0 && value <= 2) return conv_tc_set_tma(value);
    if (name && !strcmp(name, "conv_pack_cache") && (value == 0 || value == 1)) return conv_tc_set_pack_cache(value);
    if (name && !strcmp(name, "conv_tma_3x3") && (value == 0 || value == 1)) return conv_tc_set_tma_3x3(value);
    if (name && !strcmp(name, "conv_dense_1x1") && (value == 0 || value == 1)) { g_conv_dense = value; return 0; }
    if (name && !strcmp(name, "conv_tma_wgrad_3x3") && (value == 0 || value == 1)) return conv_tc_set_tma_wgrad_3x3(value);
    if (name && !strcmp(name, "conv_tma_wgrad") && value >= 0 && value <= 2) return conv_tc_set_tma_wgrad(value);
    if (name && !strcmp(name, "bn_waves") && value >= 1) return bn_set_tuning(value, 0);
    if (name && !strcmp(name, "bn_min_items") && value >= 1) return bn_set_tuning(0, value);
    return set_error(EDDLB200_EINVAL, "set_option: unknown option or value");
}

int eddlb200_conv_path_counts(int dev, unsigned long long *tensor_core_calls, unsigned long long *fma_calls) {
    if (dev < 0 || dev >= EDDLB200_MAX_DEVICES) return set_error(EDDLB200_EINVAL, "conv_path_counts: device ordinal out of range");
    if (tensor_core_calls) *tensor_core_calls = g_conv_calls[dev][0];
    if (fma_calls) *fma_calls = g_conv_calls[dev][1];
    return 0;
}

int eddlb200_conv2d_fwd(int dev, const float *x, const float *w, const float *bias, float *y,
                        int n, int c, int ih, int iw, int k, int kr, int kc, int oh, int ow,
                        int sr, int sc, int pad_top, int pad_left, int precision) {
    EB_CTX(dev);
    ConvGeom g{n, c, ih, iw, k, kr, kc, oh, ow, sr, sc, pad_top, pad_left};
    if (int r = check("gpu_conv2D", g)) return r;
    EB_REQUIRE(x && w && y && precision >= 0 && precision <= 2, "gpu_conv2D");
    if (n == 0) return 0;
    EB_READS(x, (size_t)n * c * ih * iw * sizeof(float)); EB_READS(w, (size_t)k * c * kr * kc * sizeof(float)); EB_READS(bias, (size_t)k * sizeof(float));
    EB_WRITES(y, (size_t)n * k * oh * ow * sizeof(float));
    ProfScope prof(cx, PROF_CONV_FWD, 2.0 * n * (double)k * c * kr * kc * oh * ow);
    if (tc_enabled()) {
        const Dense1x1 d = dense_1x1(g, true);
        float *xs = d.on ? dense_buf(st, 0, (size_t)n * c * d.pitch * sizeof(float)) : nullptr;
        if (xs) {
            if (int r = gather_planes(cx, st, x, xs, (size_t)n * c, ih, iw, sr, sc, oh, ow, d.pitch)) return r;
            int r = conv_tc_fwd(cx, st, d.g, xs, w, bias, y, precision);
            if (r != 1) { g_conv_calls[dev][0]++; return r; }
        }
        int r = conv_tc_fwd(cx, st, g, x, w, bias, y, precision);
        if (r != 1) { g_conv_calls[dev][0]++; return r; }
    }
    g_conv_calls[dev][1]++;
    return conv_simt_fwd(cx, st, g, x, w, bias, y);
}

int eddlb200_conv2d_bwd_data(int dev, const float *dy, const float *w, float *dx,
                             int n, int c, int ih, int iw, int k, int kr, int kc, int oh, int ow,
                             int sr, int sc, int pad_top, int pad_left, int precision) {
    EB_CTX(dev);
    ConvGeom g{n, c, ih, iw, k, kr, kc, oh, ow, sr, sc, pad_top, pad_left};
    if (int r = check("gpu_conv2D_back", g)) return r;
    EB_REQUIRE(dy && w && dx && precision >= 0 && precision <= 2, "gpu_conv2D_back");
    if (n == 0) return 0;
    EB_READS(dy, (size_t)n * k * oh * ow * sizeof(float)); EB_READS(w, (size_t)k * c * kr * kc * sizeof(float));
    const size_t dx_elems = (size_t)n * c * ih * iw;
    bool dx_zero = false;
    EB_NOTES(dx, dx_elems * sizeof(float));
    if (lz_any(cx)) { int status = 0; dx_zero = lz_take(cx, st, dx, dx_elems * sizeof(float), &status); if (status) return status; }
    ProfScope prof(cx, PROF_CONV_BWD_DATA, 2.0 * n * (double)k * c * kr * kc * oh * ow);
    if (tc_enabled()) {
        const Dense1x1 d = dense_1x1(g, true);
        float *dense = d.on ? dense_buf(st, 2, (size_t)n * c * d.pitch * sizeof(float)) : nullptr;
        if (dense) {
            int r = conv_tc_bwd_data(cx, st, d.g, dy, w, dense, precision, true);       // stores every element of the dense dx
            if (r == 0) {
                const unsigned dense_elems = (unsigned)((size_t)n * c * d.pitch);
                if (!dx_zero) plane_scatter_add_kernel<<<grid_for(dense_elems, 256), 256, 0, st>>>(dense, dx, dense_elems, ih * iw, iw, sr, sc, ow, oh * ow, d.pitch);
                else if (iw % 4 == 0 && ((uintptr_t)dx & 15) == 0)
                    plane_scatter_store_kernel<4><<<grid_for(dx_elems / 4, 256), 256, 0, st>>>(dense, dx, (unsigned)(dx_elems / 4), ih * iw, iw, sr, sc, oh, ow, d.pitch);
                else plane_scatter_store_kernel<1><<<grid_for(dx_elems, 256), 256, 0, st>>>(dense, dx, (unsigned)dx_elems, ih * iw, iw, sr, sc, oh, ow, d.pitch);
                EB_LAUNCH_CHECK("gpu_conv2D_back(scatter)");
                g_conv_calls[dev][0]++;
                return 0;
            }
            if (r != 1) return r;
        }
        int r = conv_tc_bwd_data(cx, st, g, dy, w, dx, precision, dx_zero);
        if (r != 1) { g_conv_calls[dev][0]++; return r; }
    }
    g_conv_calls[dev][1]++;
    if (dx_zero) { if (int r = launch_zero_fill(cx, st, dx, dx_elems)) return r; }     // the FMA kernel adds into dx
    return conv_simt_bwd_data(cx, st, g, dy, w, dx);
}

int eddlb200_conv2d_bwd_weight(int dev, const float *x, const float *dy, float *gw, float *gbias,
                               int n, int c, int ih, int iw, int k, int kr, int kc, int oh, int ow,
                               int sr, int sc, int pad_top, int pad_left, int precision) {
    EB_CTX(dev);
    ConvGeom g{n, c, ih, iw, k, kr, kc, oh, ow, sr, sc, pad_top, pad_left};
    if (int r = check("gpu_conv2D_grad", g)) return r;
    EB_REQUIRE(x && dy && gw && precision >= 0 && precision <= 2, "gpu_conv2D_grad");
    if (n == 0) return 0;
    EB_READS(x, (size_t)n * c * ih * iw * sizeof(float)); EB_READS(dy, (size_t)n * k * oh * ow * sizeof(float));
    EB_READS(gbias, (size_t)k * sizeof(float));
    const size_t gw_elems = (size_t)k * c * kr * kc;
    bool gw_zero = false;
    EB_NOTES(gw, gw_elems * sizeof(float)); EB_NOTES(gbias, (size_t)k * sizeof(float));
    if (lz_any(cx)) { int status = 0; gw_zero = lz_take(cx, st, gw, gw_elems * sizeof(float), &status); if (status) return status; }
    ProfScope prof(cx, PROF_CONV_BWD_WEIGHT, 2.0 * n * (double)k * c * kr * kc * oh * ow);
    if (gbias) {
        bias_grad_kernel<<<k, 256, 0, st>>>(dy, gbias, n, k, oh * ow);
        EB_LAUNCH_CHECK("gpu_conv2D_grad(bias)");
    }
    if (tc_enabled() && g_conv_dense && kr == 3 && kc == 3 && sr == 1 && sc == 1 && pad_top == 1 && pad_left == 1 && ih == oh && iw == ow &&
        (ih * iw) % 4 != 0 && ih * iw >= 32 && c >= 14 && k >= 32) {
        // A 3x3 "same" layer on a ragged plane (7x7 = 49 pixels): the TMA-fed backward-weight kernel needs planes of a multiple of
        // four pixels.  Copies of x and dy with rows padded by zero columns give it one: the zero column of dy adds nothing, the
        // zero column of x is exactly what the right-hand padding of the layer reads, and the left edge is masked by the kernel.
        int wp = iw + 1;
        while ((ih * wp) % 4 != 0) wp++;
        float *xs = dense_buf(st, 0, (size_t)n * c * ih * wp * sizeof(float));
        float *dys = dense_buf(st, 1, (size_t)n * k * ih * wp * sizeof(float));
        if (xs && dys) {
            if (int r = gather_planes(cx, st, x, xs, (size_t)n * c, ih, iw, 1, 1, ih, wp, ih * wp, iw)) return r;
            if (int r = gather_planes(cx, st, dy, dys, (size_t)n * k, oh, ow, 1, 1, oh, wp, oh * wp, ow)) return r;
            const ConvGeom gp{n, c, ih, wp, k, 3, 3, oh, wp, 1, 1, 1, 1};
            int r = conv_tc_bwd_weight(cx, st, gp, xs, dys, gw, precision, gw_zero);
            if (r != 1) { g_conv_calls[dev][0]++; return r; }
        }
    }
    if (tc_enabled()) {
        const Dense1x1 d = dense_1x1(g, false);
        float *xs = d.on ? dense_buf(st, 0, (size_t)n * c * d.pitch * sizeof(float)) : nullptr;
        float *dys = d.on && d.ragged ? dense_buf(st, 1, (size_t)n * k * d.pitch * sizeof(float)) : nullptr;
        if (xs && (dys || !d.ragged)) {
            if (int r = gather_planes(cx, st, x, xs, (size_t)n * c, ih, iw, sr, sc, oh, ow, d.pitch)) return r;
            if (dys) { if (int r = gather_planes(cx, st, dy, dys, (size_t)n * k, oh, ow, 1, 1, oh, ow, d.pitch)) return r; }
            int r = conv_tc_bwd_weight(cx, st, d.g, xs, dys ? dys : dy, gw, precision, gw_zero);
            if (r != 1) { g_conv_calls[dev][0]++; return r; }
        }
        int r = conv_tc_bwd_weight(cx, st, g, x, dy, gw, precision, gw_zero);
        if (r != 1) { g_conv_calls[dev][0]++; return r; }
    }
    g_conv_calls[dev][1]++;
    if (gw_zero) { if (int r = launch_zero_fill(cx, st, gw, gw_elems)) return r; }     // the FMA path adds into gw
    return conv_simt_bwd_weight(cx, st, g, x, dy, gw);
}

}  // extern "C"
