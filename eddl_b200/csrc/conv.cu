// Conv2D C-ABI entry points: argument checks, kernel selection, bias gradient,
// split-K combine.  See conv_tc.cu (tcgen05 tensor-core path) and conv_simt.cu
// (exact-fp32 FMA path).
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
    if (name && !strcmp(name, "conv_tma_wgrad") && value >= 0 && value <= 2) return conv_tc_set_tma_wgrad(value);
    if (name && !strcmp(name, "bn_waves") && value >= 1) return bn_set_tuning(value, 0);
    if (name && !strcmp(name, "bn_min_items") && value >= 1) return bn_set_tuning(0, value);
    return set_error(EDDLB200_EINVAL, "set_option: unknown option or value");
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
        int r = conv_tc_fwd(cx, st, g, x, w, bias, y, precision);
        if (r != 1) return r;
    }
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
        int r = conv_tc_bwd_data(cx, st, g, dy, w, dx, precision, dx_zero);
        if (r != 1) return r;
    }
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
    if (tc_enabled()) {
        int r = conv_tc_bwd_weight(cx, st, g, x, dy, gw, precision, gw_zero);
        if (r != 1) return r;
    }
    if (gw_zero) { if (int r = launch_zero_fill(cx, st, gw, gw_elems)) return r; }     // the FMA path adds into gw
    return conv_simt_bwd_weight(cx, st, g, x, dy, gw);
}

}  // extern "C"
