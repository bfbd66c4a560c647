// MaxPool2D / AvgPool2D forward and backward, NCHW fp32.
// Replaces maxpool2d / maxpool2d_back / avgpool2d / avgpool2d_back
// (EDDL src/hardware/gpu/nn/gpu_pool_kernels.cu:43-169,353-482); semantics follow
// cpu_mpool2D / cpu_mpool2D_back / cpu_avgpool2D / cpu_avgpool2D_back
// (src/hardware/cpu/nn/cpu_pool.cpp:74-145,226-304):
//   * window scan is rows-outer / cols-inner with a strict '>' from -3.40282e38, out of
//     bounds positions count as that lowest value, so ties keep the first position;
//   * ind_x / ind_y hold the absolute input column / row of the maximum AS FLOATS;
//   * average divides by the full window kr*kc, padded positions included.
// Forward: one thread per output element, consecutive threads on consecutive output
// columns (coalesced stores of y and both index planes).  Backward is written in
// gather form -- one thread per INPUT element that visits the (at most
// ceil(kr/sr)*ceil(kc/sc)) windows covering it in increasing output order -- so there
// are no float atomics and the sum order equals the reference's sequential order.
#include <cstdint>
#include "common.cuh"

namespace {

using namespace eb;
constexpr int kBlock = 256;

struct PoolGeom { int ih, iw, oh, ow, kr, kc, sr, sc, pt, pl; };

// IDX = unsigned when the tensors have fewer than 2^32 elements (32-bit divisions), size_t otherwise.
// KR, KC > 0: window size known at compile time (2x2, 3x3) -- the loops unroll and all of a window's loads are issued
// before the first compare, so an output costs one memory latency instead of kr*kc of them.  0, 0: any window.
template <int KR, int KC, typename IDX>
__global__ void __launch_bounds__(kBlock) maxpool_fwd_kernel(const float *__restrict__ in, float *__restrict__ out,
                                                             float *__restrict__ ind_x, float *__restrict__ ind_y,
                                                             size_t total, PoolGeom g) {
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    const int kr = KR > 0 ? KR : g.kr, kc = KC > 0 ? KC : g.kc;
    for (size_t p = (size_t)blockIdx.x * blockDim.x + threadIdx.x; p < total; p += stride) {
        const IDX pi = (IDX)p;
        const IDX t = pi / (IDX)g.ow;
        const int oj = (int)(pi - t * (IDX)g.ow);
        const IDX plane = t / (IDX)g.oh;
        const int oi = (int)(t - plane * (IDX)g.oh);
        const float *src = in + plane * (size_t)g.ih * g.iw;
        const int i0 = oi * g.sr - g.pt, j0 = oj * g.sc - g.pl;
        float m = -3.40282e+38f;
        // A window in which nothing exceeds the lowest value (all NaN / -inf) reports
        // position (0, 0); the reference leaves the previous content there.
        float bx = 0.f, by = 0.f;
        if (KR > 0) {
            float v[KR > 0 ? KR * KC : 1];
#pragma unroll
            for (int ki = 0; ki < KR; ki++)
#pragma unroll
                for (int kj = 0; kj < KC; kj++) {
                    const int y = i0 + ki, x = j0 + kj;
                    v[ki * KC + kj] = (y >= 0 && y < g.ih && x >= 0 && x < g.iw) ? __ldg(src + (y * g.iw + x)) : -3.40282e+38f;
                }
#pragma unroll
            for (int ki = 0; ki < KR; ki++)
#pragma unroll
                for (int kj = 0; kj < KC; kj++)
                    if (v[ki * KC + kj] > m) { m = v[ki * KC + kj]; bx = (float)(j0 + kj); by = (float)(i0 + ki); }
        } else {
            for (int ki = 0; ki < kr; ki++) {
                const int y = i0 + ki;
                for (int kj = 0; kj < kc; kj++) {
                    const int x = j0 + kj;
                    float v = -3.40282e+38f;
                    if (y >= 0 && y < g.ih && x >= 0 && x < g.iw) v = __ldg(src + (y * g.iw + x));
                    if (v > m) { m = v; bx = (float)x; by = (float)y; }
                }
            }
        }
        out[p] = m; ind_x[p] = bx; ind_y[p] = by;
    }
}

template <typename IDX>
__global__ void __launch_bounds__(kBlock) avgpool_fwd_kernel(const float *__restrict__ in, float *__restrict__ out, size_t total, PoolGeom g) {
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    const float ksize = (float)(g.kr * g.kc);
    for (size_t p = (size_t)blockIdx.x * blockDim.x + threadIdx.x; p < total; p += stride) {
        const IDX pi = (IDX)p;
        const IDX t = pi / (IDX)g.ow;
        const int oj = (int)(pi - t * (IDX)g.ow);
        const IDX plane = t / (IDX)g.oh;
        const int oi = (int)(t - plane * (IDX)g.oh);
        const float *src = in + plane * (size_t)g.ih * g.iw;
        const int i0 = oi * g.sr - g.pt, j0 = oj * g.sc - g.pl;
        float s = 0.f;
        for (int ki = 0; ki < g.kr; ki++) {
            const int y = i0 + ki;
            if (y < 0 || y >= g.ih) continue;
            for (int kj = 0; kj < g.kc; kj++) {
                const int x = j0 + kj;
                if (x >= 0 && x < g.iw) s = __fadd_rn(s, __ldg(src + (y * g.iw + x)));
            }
        }
        out[p] = __fdiv_rn(s, ksize);
    }
}

// Argmax coordinates as one key: the element's index inside its plane, -1 for coordinates outside the plane.
__device__ __forceinline__ int pool_key(int x, int y, int iw, int ih) {
    return ((unsigned)x < (unsigned)iw && (unsigned)y < (unsigned)ih) ? y * iw + x : -1;
}

// First / last output index whose window [o*s - pad, o*s - pad + k) contains position v.
__device__ __forceinline__ void covering(int v, int k, int s, int pad, int on, int &lo, int &hi) {
    const int a = v + pad;                 // o*s <= a  and  o*s > a - k
    hi = a / s;
    if (hi > on - 1) hi = on - 1;
    int num = a - k + 1;                   // o*s >= num
    lo = num <= 0 ? 0 : (num + s - 1) / s;
}

// IDX = unsigned when the tensor has fewer than 2^32 elements (32-bit divisions), size_t otherwise.
template <bool MAX, typename IDX>
__global__ void __launch_bounds__(kBlock) pool_bwd_kernel(const float *__restrict__ d, const float *__restrict__ ind_x,
                                                          const float *__restrict__ ind_y, float *__restrict__ id,
                                                          size_t total_in, PoolGeom g, int id_zero) {
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    const float ksize = (float)(g.kr * g.kc);
    for (size_t q = (size_t)blockIdx.x * blockDim.x + threadIdx.x; q < total_in; q += stride) {
        const IDX qi = (IDX)q;
        const int x = (int)(qi % (IDX)g.iw);
        const IDX t = qi / (IDX)g.iw;
        const int y = (int)(t % (IDX)g.ih);
        const size_t plane = t / (IDX)g.ih;
        int oi0, oi1, oj0, oj1;
        covering(y, g.kr, g.sr, g.pt, g.oh, oi0, oi1);
        covering(x, g.kc, g.sc, g.pl, g.ow, oj0, oj1);
        // id_zero: the input delta is known to hold zeros; it is written in full and never read
        float acc = id_zero ? 0.f : id[q];
        bool touched = id_zero != 0;
        const size_t obase = plane * (size_t)g.oh * g.ow;
        if (oi1 - oi0 <= 1 && oj1 - oj0 <= 1) {
            // at most 2 x 2 covering windows (kernel <= 2 * stride, the usual case): all loads go out together, with no
            // data-dependent branches between them; the adds keep the reference's window order
            float vd[4], vx[4], vy[4]; bool in[4];
#pragma unroll
            for (int w = 0; w < 4; w++) {
                const int oi = oi0 + (w >> 1), oj = oj0 + (w & 1);
                in[w] = oi <= oi1 && oj <= oj1;
                const size_t p = obase + (size_t)(in[w] ? oi : oi0) * g.ow + (in[w] ? oj : oj0);
                in[w] = in[w] && oi0 <= oi1 && oj0 <= oj1;
                if (in[w]) {
                    vd[w] = __ldg(d + p);
                    if (MAX) { vx[w] = __ldg(ind_x + p); vy[w] = __ldg(ind_y + p); }
                }
            }
#pragma unroll
            for (int w = 0; w < 4; w++) {
                if (!in[w]) continue;
                if (MAX) {
                    // int x = D->indX->ptr[p]  (float -> int conversion in the reference)
                    if ((int)vx[w] == x && (int)vy[w] == y) { acc = __fadd_rn(acc, vd[w]); touched = true; }
                } else {
                    acc = __fadd_rn(acc, __fdiv_rn(vd[w], ksize));
                    touched = true;
                }
            }
        } else
        for (int oi = oi0; oi <= oi1; oi++)
            for (int oj = oj0; oj <= oj1; oj++) {
                const size_t p = obase + (size_t)oi * g.ow + oj;
                if (MAX) {
                    // int x = D->indX->ptr[p]  (float -> int conversion in the reference)
                    if ((int)__ldg(ind_x + p) == x && (int)__ldg(ind_y + p) == y) { acc = __fadd_rn(acc, __ldg(d + p)); touched = true; }
                } else {
                    acc = __fadd_rn(acc, __fdiv_rn(__ldg(d + p), ksize));
                    touched = true;
                }
            }
        if (touched) id[q] = acc;
    }
}

// Max-pool backward, one block per (n, c) plane.  The plane's output-side tensors are staged in shared memory once, as 8
// bytes per output element: the delta and the argmax position folded into ONE integer key (row * iw + column, or -1 when
// the stored coordinates lie outside the plane and can match no element).  The covering-window ranges of every input row
// and column are tabulated once per block (they need integer divisions by the stride), so an input element costs two table
// reads plus, per covering window, one key compare and a predicated add.  Same window order and arithmetic as
// pool_bwd_kernel; used when the plane fits.
__global__ void __launch_bounds__(256) maxpool_bwd_plane_kernel(const float *__restrict__ d, const float *__restrict__ ind_x,
                                                                const float *__restrict__ ind_y, float *__restrict__ id,
                                                                unsigned planes, PoolGeom g, int id_zero) {
    extern __shared__ float sm_pool[];
    const int opl = g.oh * g.ow, ipl = g.ih * g.iw;
    float *sd = sm_pool;
    int *skey = reinterpret_cast<int *>(sm_pool + opl);
    int *rowtab = skey + opl, *coltab = rowtab + g.ih;        // (first | last << 16) covering output row / column
    for (int v = threadIdx.x; v < g.ih + g.iw; v += blockDim.x) {
        int lo, hi;
        if (v < g.ih) covering(v, g.kr, g.sr, g.pt, g.oh, lo, hi);
        else covering(v - g.ih, g.kc, g.sc, g.pl, g.ow, lo, hi);
        rowtab[v] = lo | (hi << 16);         // lo > hi: no window covers it; both grow with v
    }
    const bool vec = (opl & 3) == 0 && aligned16(d) && aligned16(ind_x) && aligned16(ind_y);
    for (unsigned plane = blockIdx.x; plane < planes; plane += gridDim.x) {
        const size_t obase = (size_t)plane * opl;
        __syncthreads();                       // the previous plane's readers are done
        if (vec) {
            // 16-byte loads, several per thread in flight: the staging is one memory latency, not one per element
#pragma unroll 4
            for (int p = threadIdx.x * 4; p < opl; p += blockDim.x * 4) {
                const float4 a = ld_stream4(d + obase + p), b = ld_stream4(ind_x + obase + p), c = ld_stream4(ind_y + obase + p);
                *reinterpret_cast<float4 *>(sd + p) = a;
                int4 k;
                // int x = D->indX->ptr[p]  (float -> int conversion in the reference)
                k.x = pool_key((int)b.x, (int)c.x, g.iw, g.ih); k.y = pool_key((int)b.y, (int)c.y, g.iw, g.ih);
                k.z = pool_key((int)b.z, (int)c.z, g.iw, g.ih); k.w = pool_key((int)b.w, (int)c.w, g.iw, g.ih);
                *reinterpret_cast<int4 *>(skey + p) = k;
            }
        } else {
            for (int p = threadIdx.x; p < opl; p += blockDim.x) {
                sd[p] = __ldg(d + obase + p);
                skey[p] = pool_key((int)__ldg(ind_x + obase + p), (int)__ldg(ind_y + obase + p), g.iw, g.ih);
            }
        }
        __syncthreads();
        float *idp = id + (size_t)plane * ipl;
        if ((g.iw & 3) == 0 && aligned16(id)) {
            // Four consecutive elements of one row per thread (16-byte accesses to the input delta).  They share the row's
            // window range, and the windows of columns first(x0) .. last(x0 + 3) are each read once: a window's key names
            // at most one of the four elements, which takes its delta.  Per element the order stays rows-outer, columns-inner.
            const int iw4 = g.iw >> 2;
            int y = threadIdx.x / iw4, xq = threadIdx.x - y * iw4;
            const int dy = blockDim.x / iw4, dxq = blockDim.x - dy * iw4;
#pragma unroll 2
            for (int q4 = threadIdx.x; q4 < (ipl >> 2); q4 += blockDim.x) {
                const int rt = rowtab[y], x0 = xq << 2, base = q4 << 2;
                const int oi0 = rt & 0xffff, oi1 = rt >> 16, oj0 = coltab[x0] & 0xffff, oj1 = coltab[x0 + 3] >> 16;
                float4 acc = id_zero ? make_float4(0.f, 0.f, 0.f, 0.f) : *reinterpret_cast<const float4 *>(idp + base);
                for (int oi = oi0; oi <= oi1; oi++)
                    for (int oj = oj0; oj <= oj1; oj++) {
                        const int p = oi * g.ow + oj, e = skey[p] - base;
                        const float v = sd[p];
                        acc.x = e == 0 ? __fadd_rn(acc.x, v) : acc.x;
                        acc.y = e == 1 ? __fadd_rn(acc.y, v) : acc.y;
                        acc.z = e == 2 ? __fadd_rn(acc.z, v) : acc.z;
                        acc.w = e == 3 ? __fadd_rn(acc.w, v) : acc.w;
                    }
                *reinterpret_cast<float4 *>(idp + base) = acc;        // untouched elements get their own value back
                xq += dxq; y += dy;
                if (xq >= iw4) { xq -= iw4; y++; }
            }
        } else if ((g.iw & 1) == 0 && (((uintptr_t)id) & 7) == 0) {
            // the same with two elements per thread (rows of an even length that is not a multiple of four, e.g. the 114 x 114
            // planes behind an explicit padding layer): 8-byte accesses to the input delta
            const int iw2 = g.iw >> 1;
            int y = threadIdx.x / iw2, xq = threadIdx.x - y * iw2;
            const int dy = blockDim.x / iw2, dxq = blockDim.x - dy * iw2;
#pragma unroll 2
            for (int q2 = threadIdx.x; q2 < (ipl >> 1); q2 += blockDim.x) {
                const int rt = rowtab[y], x0 = xq << 1, base = q2 << 1;
                const int oi0 = rt & 0xffff, oi1 = rt >> 16, oj0 = coltab[x0] & 0xffff, oj1 = coltab[x0 + 1] >> 16;
                float2 acc = id_zero ? make_float2(0.f, 0.f) : *reinterpret_cast<const float2 *>(idp + base);
                for (int oi = oi0; oi <= oi1; oi++)
                    for (int oj = oj0; oj <= oj1; oj++) {
                        const int p = oi * g.ow + oj, e = skey[p] - base;
                        const float v = sd[p];
                        acc.x = e == 0 ? __fadd_rn(acc.x, v) : acc.x;
                        acc.y = e == 1 ? __fadd_rn(acc.y, v) : acc.y;
                    }
                *reinterpret_cast<float2 *>(idp + base) = acc;
                xq += dxq; y += dy;
                if (xq >= iw2) { xq -= iw2; y++; }
            }
        } else {
            int y = threadIdx.x / g.iw, x = threadIdx.x - y * g.iw;
            const int dy = blockDim.x / g.iw, dx = blockDim.x - dy * g.iw;      // advance of (y, x) per blockDim.x elements
            for (int q = threadIdx.x; q < ipl; q += blockDim.x) {
                const int rt = rowtab[y], ct = coltab[x];
                const int oi0 = rt & 0xffff, oi1 = rt >> 16, oj0 = ct & 0xffff, oj1 = ct >> 16;
                float acc = id_zero ? 0.f : idp[q];
                for (int oi = oi0; oi <= oi1; oi++)
                    for (int oj = oj0; oj <= oj1; oj++) {
                        const int p = oi * g.ow + oj;
                        if (skey[p] == q) acc = __fadd_rn(acc, sd[p]);
                    }
                idp[q] = acc;
                x += dx; y += dy;
                if (x >= g.iw) { x -= g.iw; y++; }
            }
        }
    }
}

int check_geom(const char *what, int n, int c, int ih, int iw, int oh, int ow, int kr, int kc, int sr, int sc, int pt, int pl) {
    if (n < 0 || c < 0 || ih <= 0 || iw <= 0 || oh <= 0 || ow <= 0 || kr <= 0 || kc <= 0 || sr <= 0 || sc <= 0 || pt < 0 || pl < 0)
        return set_error(EDDLB200_EINVAL, "%s: bad geometry", what);
    return 0;
}

}  // namespace

using namespace eb;

extern "C" {

int eddlb200_maxpool2d_fwd(int dev, const float *in, float *out, float *ind_x, float *ind_y, int n, int c, int ih, int iw, int oh, int ow,
                           int kr, int kc, int sr, int sc, int pad_top, int pad_left) {
    EB_CTX(dev);
    if (int r = check_geom("gpu_mpool2D", n, c, ih, iw, oh, ow, kr, kc, sr, sc, pad_top, pad_left)) return r;
    EB_REQUIRE(in && out && ind_x && ind_y, "gpu_mpool2D");
    const size_t total = (size_t)n * c * oh * ow;
    if (!total) return 0;
    PoolGeom g{ih, iw, oh, ow, kr, kc, sr, sc, pad_top, pad_left};
    EB_READS(in, (size_t)n * c * ih * iw * sizeof(float));
    EB_WRITES(out, total * sizeof(float)); EB_WRITES(ind_x, total * sizeof(float)); EB_WRITES(ind_y, total * sizeof(float));
    ProfScope prof(cx, PROF_POOL, 4.0 * n * c * ih * iw + 12.0 * total);
    const int blocks = grid_for(total, kBlock);
    if ((size_t)n * c * ih * iw >= (size_t(1) << 32)) maxpool_fwd_kernel<0, 0, size_t><<<blocks, kBlock, 0, st>>>(in, out, ind_x, ind_y, total, g);
    else if (kr == 2 && kc == 2) maxpool_fwd_kernel<2, 2, unsigned><<<blocks, kBlock, 0, st>>>(in, out, ind_x, ind_y, total, g);
    else if (kr == 3 && kc == 3) maxpool_fwd_kernel<3, 3, unsigned><<<blocks, kBlock, 0, st>>>(in, out, ind_x, ind_y, total, g);
    else maxpool_fwd_kernel<0, 0, unsigned><<<blocks, kBlock, 0, st>>>(in, out, ind_x, ind_y, total, g);
    EB_LAUNCH_CHECK("gpu_mpool2D");
    return 0;
}

int eddlb200_maxpool2d_bwd(int dev, const float *d, const float *ind_x, const float *ind_y, float *id, int n, int c, int ih, int iw, int oh, int ow,
                           int kr, int kc, int sr, int sc, int pad_top, int pad_left) {
    EB_CTX(dev);
    if (int r = check_geom("gpu_mpool2D_back", n, c, ih, iw, oh, ow, kr, kc, sr, sc, pad_top, pad_left)) return r;
    EB_REQUIRE(d && ind_x && ind_y && id, "gpu_mpool2D_back");
    const size_t total = (size_t)n * c * ih * iw;
    if (!total) return 0;
    PoolGeom g{ih, iw, oh, ow, kr, kc, sr, sc, pad_top, pad_left};
    const size_t ob = (size_t)n * c * oh * ow * sizeof(float);
    EB_READS(d, ob); EB_READS(ind_x, ob); EB_READS(ind_y, ob);
    int id_zero = 0;
    EB_NOTES(id, total * sizeof(float));
    if (lz_any(cx) && id != d) { int status = 0; id_zero = lz_take(cx, st, id, total * sizeof(float), &status); if (status) return status; }
    ProfScope prof(cx, PROF_POOL, 12.0 * n * c * oh * ow + (id_zero ? 4.0 : 8.0) * total);     // the delta is stored, or read and written
    const size_t plane_smem = (size_t)8 * oh * ow + (size_t)4 * (ih + iw);
    if (plane_smem <= (size_t)160 * 1024 && ih * iw >= 1024 && oh < 32768 && ow < 32768 && (size_t)n * c < 0x7fffffffu) {
        static bool configured[EDDLB200_MAX_DEVICES] = {};
        if (!configured[dev]) {
            cudaError_t e = cudaFuncSetAttribute(maxpool_bwd_plane_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 160 * 1024);
            if (e != cudaSuccess) return cuda_status(e, "gpu_mpool2D_back(smem attribute)");
            configured[dev] = true;
        }
        const unsigned planes = (unsigned)(n * c);
        int per_sm = (int)((size_t)200 * 1024 / plane_smem);
        if (per_sm > 8) per_sm = 8;
        if (per_sm < 1) per_sm = 1;
        unsigned blocks = planes < (unsigned)(EDDLB200_NUM_SMS * per_sm) ? planes : (unsigned)(EDDLB200_NUM_SMS * per_sm);
        maxpool_bwd_plane_kernel<<<blocks, 256, plane_smem, st>>>(d, ind_x, ind_y, id, planes, g, id_zero);
        EB_LAUNCH_CHECK("gpu_mpool2D_back");
        return 0;
    }
    if (total < (size_t(1) << 32)) pool_bwd_kernel<true, unsigned><<<grid_for(total, kBlock), kBlock, 0, st>>>(d, ind_x, ind_y, id, total, g, id_zero);
    else pool_bwd_kernel<true, size_t><<<grid_for(total, kBlock), kBlock, 0, st>>>(d, ind_x, ind_y, id, total, g, id_zero);
    EB_LAUNCH_CHECK("gpu_mpool2D_back");
    return 0;
}

int eddlb200_avgpool2d_fwd(int dev, const float *in, float *out, int n, int c, int ih, int iw, int oh, int ow,
                           int kr, int kc, int sr, int sc, int pad_top, int pad_left) {
    EB_CTX(dev);
    if (int r = check_geom("gpu_avgpool2D", n, c, ih, iw, oh, ow, kr, kc, sr, sc, pad_top, pad_left)) return r;
    EB_REQUIRE(in && out, "gpu_avgpool2D");
    const size_t total = (size_t)n * c * oh * ow;
    if (!total) return 0;
    PoolGeom g{ih, iw, oh, ow, kr, kc, sr, sc, pad_top, pad_left};
    EB_READS(in, (size_t)n * c * ih * iw * sizeof(float));
    EB_WRITES(out, total * sizeof(float));
    ProfScope prof(cx, PROF_POOL, 4.0 * n * c * ih * iw + 4.0 * total);
    if ((size_t)n * c * ih * iw < (size_t(1) << 32)) avgpool_fwd_kernel<unsigned><<<grid_for(total, kBlock), kBlock, 0, st>>>(in, out, total, g);
    else avgpool_fwd_kernel<size_t><<<grid_for(total, kBlock), kBlock, 0, st>>>(in, out, total, g);
    EB_LAUNCH_CHECK("gpu_avgpool2D");
    return 0;
}

int eddlb200_avgpool2d_bwd(int dev, const float *d, float *id, int n, int c, int ih, int iw, int oh, int ow,
                           int kr, int kc, int sr, int sc, int pad_top, int pad_left) {
    EB_CTX(dev);
    if (int r = check_geom("gpu_avgpool2D_back", n, c, ih, iw, oh, ow, kr, kc, sr, sc, pad_top, pad_left)) return r;
    EB_REQUIRE(d && id, "gpu_avgpool2D_back");
    const size_t total = (size_t)n * c * ih * iw;
    if (!total) return 0;
    PoolGeom g{ih, iw, oh, ow, kr, kc, sr, sc, pad_top, pad_left};
    EB_READS(d, (size_t)n * c * oh * ow * sizeof(float));
    int id_zero = 0;
    EB_NOTES(id, total * sizeof(float));
    if (lz_any(cx) && id != d) { int status = 0; id_zero = lz_take(cx, st, id, total * sizeof(float), &status); if (status) return status; }
    ProfScope prof(cx, PROF_POOL, 4.0 * n * c * oh * ow + (id_zero ? 4.0 : 8.0) * total);
    if (total < (size_t(1) << 32)) pool_bwd_kernel<false, unsigned><<<grid_for(total, kBlock), kBlock, 0, st>>>(d, nullptr, nullptr, id, total, g, id_zero);
    else pool_bwd_kernel<false, size_t><<<grid_for(total, kBlock), kBlock, 0, st>>>(d, nullptr, nullptr, id, total, g, id_zero);
    EB_LAUNCH_CHECK("gpu_avgpool2D_back");
    return 0;
}

}  // extern "C"
