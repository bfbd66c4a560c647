// Conv2D forward / backward-data / backward-weight as implicit GEMM on the fp32 FMA
// pipe (no materialised im2col, no col2im atomics, no transposes).
// Replaces gpu_im2col_k + cublasSgemm + gpu_traspose_batch_depth + gpu_addbias_k /
// gpu_deltabias_k (EDDL src/hardware/gpu/nn/gpu_conv.cu:159-372, gpu_conv_kernels.cu:21-112);
// the contraction is the one spelled out by cpu_low_mem_conv3D (src/hardware/cpu/nn/
// cpu_conv.cpp:282-314) and by cpu_im2col_conv2D{,_grad,_back} (:114-280):
//   fwd        y[n,k,p,q]   =  sum_{c,r,s} x[n,c,p*sr+r-pt,q*sc+s-pl] * w[k,c,r,s] (+ bias[k])
//   bwd-data   dx[n,c,y,x]  += sum_{k,r,s} dy[n,k,p,q] * w[k,c,r,s],  p*sr+r-pt = y, q*sc+s-pl = x
//   bwd-weight gw[k,c,r,s]  += sum_{n,p,q} dy[n,k,p,q] * x[n,c,p*sr+r-pt,q*sc+s-pl]
// This file is the exact-fp32 path used for shapes the tensor-core kernel does not take
// (tiny channel counts, ragged tiles).  64x64x16 block tiles, 4x4 accumulators/thread;
// backward-weight splits the long n*p*q reduction across blockIdx.z and combines the
// partials in a fixed order (deterministic, no float atomics).
#include "common.cuh"
#include "conv_common.cuh"

namespace {

using namespace eb;

constexpr int BM = 64, BN = 64, BK = 16, TB = 256;

// ---- operand gathers ---------------------------------------------------------------
struct FwdOps {
    ConvGeom g; const float *x, *w;
    __device__ int M() const { return g.k; }
    __device__ int N() const { return g.n * g.oh * g.ow; }
    __device__ int K() const { return g.c * g.kr * g.kc; }
    static constexpr bool a_k_fastest = true, b_k_fastest = false;
    __device__ float a(int m, int kd) const { return __ldg(w + (size_t)m * K() + kd); }
    __device__ float b(int kd, int j) const {
        const int krc = g.kr * g.kc;
        const int c = kd / krc, rs = kd - c * krc, r = rs / g.kc, s = rs - r * g.kc;
        const int pq = g.oh * g.ow;
        const int n = j / pq, t = j - n * pq, p = t / g.ow, q = t - p * g.ow;
        const int y = p * g.sr + r - g.pt, xx = q * g.sc + s - g.pl;
        if (y < 0 || y >= g.ih || xx < 0 || xx >= g.iw) return 0.f;
        return __ldg(x + (((size_t)n * g.c + c) * g.ih + y) * g.iw + xx);
    }
};

struct BwdDataOps {
    ConvGeom g; const float *dy, *w;
    __device__ int M() const { return g.c; }
    __device__ int N() const { return g.n * g.ih * g.iw; }
    __device__ int K() const { return g.k * g.kr * g.kc; }
    static constexpr bool a_k_fastest = true, b_k_fastest = false;
    __device__ float a(int m, int kd) const {
        const int krc = g.kr * g.kc;
        const int k = kd / krc, rs = kd - k * krc;
        return __ldg(w + ((size_t)k * g.c + m) * krc + rs);
    }
    __device__ float b(int kd, int j) const {
        const int krc = g.kr * g.kc;
        const int k = kd / krc, rs = kd - k * krc, r = rs / g.kc, s = rs - r * g.kc;
        const int hw = g.ih * g.iw;
        const int n = j / hw, t = j - n * hw, y = t / g.iw, xx = t - y * g.iw;
        const int py = y + g.pt - r, qx = xx + g.pl - s;
        if (py < 0 || qx < 0) return 0.f;
        const int p = py / g.sr, q = qx / g.sc;
        if (p * g.sr != py || q * g.sc != qx || p >= g.oh || q >= g.ow) return 0.f;
        return __ldg(dy + (((size_t)n * g.k + k) * g.oh + p) * g.ow + q);
    }
};

struct BwdWeightOps {
    ConvGeom g; const float *dy, *x;
    __device__ int M() const { return g.k; }
    __device__ int N() const { return g.c * g.kr * g.kc; }
    __device__ int K() const { return g.n * g.oh * g.ow; }
    static constexpr bool a_k_fastest = true, b_k_fastest = true;
    __device__ float a(int m, int kd) const {
        const int pq = g.oh * g.ow;
        const int n = kd / pq, t = kd - n * pq;
        return __ldg(dy + ((size_t)n * g.k + m) * pq + t);
    }
    __device__ float b(int kd, int j) const {
        const int krc = g.kr * g.kc;
        const int c = j / krc, rs = j - c * krc, r = rs / g.kc, s = rs - r * g.kc;
        const int pq = g.oh * g.ow;
        const int n = kd / pq, t = kd - n * pq, p = t / g.ow, q = t - p * g.ow;
        const int y = p * g.sr + r - g.pt, xx = q * g.sc + s - g.pl;
        if (y < 0 || y >= g.ih || xx < 0 || xx >= g.iw) return 0.f;
        return __ldg(x + (((size_t)n * g.c + c) * g.ih + y) * g.iw + xx);
    }
};

// ---- epilogues -----------------------------------------------------------------------
struct FwdEpi {
    ConvGeom g; float *y; const float *bias;
    __device__ void operator()(int m, int j, float v) const {
        const int pq = g.oh * g.ow;
        const int n = j / pq, t = j - n * pq;
        if (bias) v = __fadd_rn(v, __ldg(bias + m));
        y[((size_t)n * g.k + m) * pq + t] = v;
    }
};
struct BwdDataEpi {
    ConvGeom g; float *dx;
    __device__ void operator()(int m, int j, float v) const {
        const int hw = g.ih * g.iw;
        const int n = j / hw, t = j - n * hw;
        float *p = dx + ((size_t)n * g.c + m) * hw + t;
        *p = __fadd_rn(*p, v);
    }
};
struct PartialEpi {   // split-K partial: part[z][m][j]
    float *part; int N; size_t MN;
    __device__ void operator()(int m, int j, float v) const { part[(size_t)blockIdx.z * MN + (size_t)m * N + j] = v; }
};

template <typename Ops, typename Epi>
__global__ void __launch_bounds__(TB) igemm_simt_kernel(Ops ops, Epi epi, int k_per_split) {
    __shared__ float As[BK][BM + 4];
    __shared__ float Bs[BK][BN + 4];
    const int M = ops.M(), N = ops.N(), K = ops.K();
    const int tx = threadIdx.x % 16, ty = threadIdx.x / 16;
    const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
    const int kbeg = blockIdx.z * k_per_split;
    const int kend = min(K, kbeg + k_per_split);
    float acc[4][4] = {};
    for (int k0 = kbeg; k0 < kend; k0 += BK) {
#pragma unroll
        for (int e = threadIdx.x; e < BM * BK; e += TB) {
            int mi, ki;
            if (Ops::a_k_fastest) { ki = e % BK; mi = e / BK; } else { mi = e % BM; ki = e / BM; }
            const int gm = m0 + mi, gk = k0 + ki;
            As[ki][mi] = (gm < M && gk < kend) ? ops.a(gm, gk) : 0.f;
        }
#pragma unroll
        for (int e = threadIdx.x; e < BN * BK; e += TB) {
            int ni, ki;
            if (Ops::b_k_fastest) { ki = e % BK; ni = e / BK; } else { ni = e % BN; ki = e / BN; }
            const int gn = n0 + ni, gk = k0 + ki;
            Bs[ki][ni] = (gn < N && gk < kend) ? ops.b(gk, gn) : 0.f;
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < BK; kk++) {
            float a[4], b[4];
#pragma unroll
            for (int i = 0; i < 4; i++) a[i] = As[kk][ty * 4 + i];
#pragma unroll
            for (int j = 0; j < 4; j++) b[j] = Bs[kk][tx * 4 + j];
#pragma unroll
            for (int i = 0; i < 4; i++)
#pragma unroll
                for (int j = 0; j < 4; j++) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 4; i++) {
        const int gm = m0 + ty * 4 + i;
        if (gm >= M) continue;
#pragma unroll
        for (int j = 0; j < 4; j++) {
            const int gn = n0 + tx * 4 + j;
            if (gn < N) epi(gm, gn, acc[i][j]);
        }
    }
}

}  // namespace

namespace eb {

int conv_simt_fwd(DevCtx *cx, cudaStream_t st, const ConvGeom &g, const float *x, const float *w, const float *bias, float *y) {
    FwdOps ops{g, x, w};
    FwdEpi epi{g, y, bias};
    const long long N = (long long)g.n * g.oh * g.ow;
    dim3 grid((unsigned)ceil_div(N, BN), (unsigned)ceil_div(g.k, BM), 1);
    igemm_simt_kernel<<<grid, TB, 0, st>>>(ops, epi, g.c * g.kr * g.kc);
    EB_LAUNCH_CHECK("gpu_conv2D");
    return 0;
}

int conv_simt_bwd_data(DevCtx *cx, cudaStream_t st, const ConvGeom &g, const float *dy, const float *w, float *dx) {
    BwdDataOps ops{g, dy, w};
    BwdDataEpi epi{g, dx};
    const long long N = (long long)g.n * g.ih * g.iw;
    dim3 grid((unsigned)ceil_div(N, BN), (unsigned)ceil_div(g.c, BM), 1);
    igemm_simt_kernel<<<grid, TB, 0, st>>>(ops, epi, g.k * g.kr * g.kc);
    EB_LAUNCH_CHECK("gpu_conv2D_back");
    return 0;
}

int conv_simt_bwd_weight(DevCtx *cx, cudaStream_t st, const ConvGeom &g, const float *x, const float *dy, float *gw) {
    BwdWeightOps ops{g, dy, x};
    const int M = g.k, N = g.c * g.kr * g.kc;
    const long long K = (long long)g.n * g.oh * g.ow;
    const int tiles = (int)(ceil_div(N, BN) * ceil_div(M, BM));
    int splits = (EDDLB200_NUM_SMS * 4 + tiles - 1) / tiles;
    const int max_splits = (int)ceil_div((size_t)K, (size_t)BK * 8);
    if (splits > max_splits) splits = max_splits;
    if (splits > 512) splits = 512;
    if (splits < 1) splits = 1;
    int k_per_split = (int)ceil_div((size_t)K, (size_t)splits);
    k_per_split = (k_per_split + BK - 1) / BK * BK;
    splits = (int)ceil_div((size_t)K, (size_t)k_per_split);
    const size_t MN = (size_t)M * N;
    float *part = (float *)scratch(cx, MN * splits * sizeof(float));
    if (!part) return cudaErrorMemoryAllocation;
    PartialEpi epi{part, N, MN};
    dim3 grid((unsigned)ceil_div(N, BN), (unsigned)ceil_div(M, BM), splits);
    igemm_simt_kernel<<<grid, TB, 0, st>>>(ops, epi, k_per_split);
    EB_LAUNCH_CHECK("gpu_conv2D_grad");
    return splitk_reduce_accumulate(cx, st, part, gw, MN, splits);
}

}  // namespace eb
