// Layers that EDDL's own convnet examples use beside the benchmark nets: Concat, UpSampling (nearest-neighbour repeat),
// Dropout's mask, RandomFlip and RandomCropScale.  Replaces gpu_concat (EDDL src/hardware/gpu/gpu_core.cu:384-409),
// gpu_repeat_nn / gpu_d_repeat_nn (src/hardware/gpu/nn/gpu_core_nn.cu), gpu_rand_binary (src/hardware/gpu/gpu_generator.cu),
// gpu_flip_random / gpu_crop_scale_random (src/hardware/gpu/gpu_da.cu:250-302).  Arithmetic follows cpu_concat
// (src/hardware/cpu/cpu_core.cpp:368-396), cpu_repeat_nn / cpu_d_repeat_nn (src/hardware/cpu/nn/cpu_tensor_nn.cpp:13-50),
// cpu_single_flip and cpu_single_crop_scale (src/hardware/cpu/cpu_da.cpp:315-336, 363-384).
//
// All of them are copies with index arithmetic, bound by HBM: grid-stride kernels over the LARGER tensor with consecutive
// threads on consecutive output addresses.  The random layers take their per-image decisions (flip or not, crop box) as
// explicit arguments -- the host side of the layer draws them -- so every kernel is a deterministic function that the
// parity tests can check; only the Dropout mask is drawn on the device, from a counter-based generator.
#include <vector>
#include "common.cuh"

namespace {

using namespace eb;
constexpr int kBlock = 256;

// dest[(j / src_stride) * steps + j % src_stride] = src[j]   (derivative: src[j] += dest[...])
template <bool DERIV>
__global__ void __launch_bounds__(kBlock) concat_kernel(float *__restrict__ dest, float *__restrict__ src, size_t n, unsigned src_stride, unsigned steps) {
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    for (size_t j = (size_t)blockIdx.x * blockDim.x + threadIdx.x; j < n; j += stride) {
        const size_t q = j / src_stride, k = j - q * src_stride;
        if (DERIV) src[j] = __fadd_rn(src[j], dest[q * steps + k]);
        else dest[q * steps + k] = src[j];
    }
}

// B[row_b][col_b] = A[row_b / sr][col_b / sc] over all (image, channel, row) rows at once
__global__ void __launch_bounds__(kBlock) repeat_nn_kernel(const float *__restrict__ a, float *__restrict__ b, size_t nb, int bw, int aw, int sr, int sc) {
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < nb; i += stride) {
        const size_t row_b = i / bw; const int col_b = (int)(i - row_b * bw);
        b[i] = __ldg(a + (row_b / sr) * aw + col_b / sc);
    }
}

// A[row_a][col_a] += D over its sr x sc block, added one by one in row-major order of the block (the order in which the
// reference's loop over D meets them), without atomics: one thread per element of A
__global__ void __launch_bounds__(kBlock) repeat_nn_bwd_kernel(const float *__restrict__ d, float *__restrict__ a, size_t na, int dw, int aw, int sr, int sc) {
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < na; i += stride) {
        const size_t row_a = i / aw; const int col_a = (int)(i - row_a * aw);
        float acc = a[i];
        for (int r = 0; r < sr; r++)
            for (int c = 0; c < sc; c++) acc = __fadd_rn(acc, __ldg(d + (row_a * sr + r) * dw + col_a * sc + c));
        a[i] = acc;
    }
}

// B[n,c,i,j] = apply[n] ? A[n,c,flip(i,j)] : A[n,c,i,j]
__global__ void __launch_bounds__(kBlock) flip_kernel(const float *__restrict__ a, float *__restrict__ b, size_t total, int c, int h, int w, int axis,
                                                      const unsigned char *__restrict__ apply) {
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    const size_t plane = (size_t)h * w, image = plane * c;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += stride) {
        const size_t n = i / image;
        size_t src = i;
        if (apply[n]) {
            const size_t t = i % plane; const int y = (int)(t / w), x = (int)(t - (size_t)y * w);
            src = i - t + (axis == 0 ? (size_t)(h - 1 - y) * w + x : (size_t)y * w + (w - 1 - x));
        }
        b[i] = __ldg(a + src);
    }
}

// B[n,c,i,j] = A[n,c, i*hc/BH + y0, j*wc/BW + x0] with (y0, x0, hc, wc) per image
__global__ void __launch_bounds__(kBlock) crop_scale_kernel(const float *__restrict__ a, float *__restrict__ b, size_t total, int c, int ah, int aw, int bh, int bw,
                                                            const int4 *__restrict__ box) {
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    const size_t bplane = (size_t)bh * bw, bimage = bplane * c;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += stride) {
        const size_t n = i / bimage, rest = i - n * bimage, ch = rest / bplane, t = rest - ch * bplane;
        const int bi = (int)(t / bw), bj = (int)(t - (size_t)bi * bw);
        const int4 bx = __ldg(box + n);
        const int ai = (bi * bx.z) / bh + bx.x, aj = (bj * bx.w) / bw + bx.y;
        b[i] = __ldg(a + ((n * c + ch) * ah + ai) * aw + aj);
    }
}

// Resize by nearest neighbour (Tensor::scale -> cpu_single_scale, src/hardware/cpu/cpu_da.cpp:88-138): the source index of
// output index b, with the reference's float arithmetic and its truncation to int.  mode: 0 half-pixel, 2 align-corners,
// 3 asymmetric.
struct ScaleGeom { int ah, aw, bh, bw, nh, nw, off_y, off_x, mode, wrap; float cval; };
__host__ __device__ __forceinline__ int scale_src(int b, int off, int n_new, int a_extent, int mode) {
    int a = b + off;
    if (mode == 0) { const float s = (float)n_new / a_extent; a = (int)(((float)a + 0.5f) / s - 0.5f); }
    else if (mode == 2) { const float s = (float)(n_new - 1) / (a_extent - 1); a = (int)(a / s); }
    else { const float s = (float)n_new / a_extent; a = (int)(a / s); }
    return a;
}
__global__ void __launch_bounds__(kBlock) scale_kernel(const float *__restrict__ a, float *__restrict__ b, size_t total, ScaleGeom g) {
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    const size_t bplane = (size_t)g.bh * g.bw;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += stride) {
        const size_t plane = i / bplane, t = i - plane * bplane;
        const int bi = (int)(t / g.bw), bj = (int)(t - (size_t)bi * g.bw);
        const int ai = scale_src(bi, g.off_y, g.nh, g.ah, g.mode), aj = scale_src(bj, g.off_x, g.nw, g.aw, g.mode);
        float v;
        if (ai >= 0 && ai < g.ah && aj >= 0 && aj < g.aw) v = __ldg(a + (plane * g.ah + ai) * g.aw + aj);
        else v = g.wrap == 5 ? __ldg(a + i) : g.cval;               // WrappingMode::Original reads A at B's own position
        b[i] = v;
    }
}
// A[ai][aj] += every B[bi][bj] that maps to it, added one by one in row-major order of B (cpu_single_scale_back, :140-190),
// one thread per element of A: the mapping is monotonic, so the candidates of a source row are the output rows around ai*scale.
__global__ void __launch_bounds__(kBlock) scale_bwd_kernel(float *__restrict__ a, const float *__restrict__ b, size_t total, ScaleGeom g) {
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    const size_t aplane = (size_t)g.ah * g.aw;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += stride) {
        const size_t plane = i / aplane, t = i - plane * aplane;
        const int ai = (int)(t / g.aw), aj = (int)(t - (size_t)ai * g.aw);
        const float sy = (float)g.nh / g.ah, sx = (float)g.nw / g.aw;
        int i0 = (int)floorf(ai * sy) - g.off_y - 2, i1 = (int)ceilf((ai + 1) * sy) - g.off_y + 2;
        int j0 = (int)floorf(aj * sx) - g.off_x - 2, j1 = (int)ceilf((aj + 1) * sx) - g.off_x + 2;
        if (g.mode == 2) { i0 = 0; i1 = g.bh - 1; j0 = 0; j1 = g.bw - 1; }      // align-corners: scan everything (rare, small)
        i0 = max(i0, 0); j0 = max(j0, 0); i1 = min(i1, g.bh - 1); j1 = min(j1, g.bw - 1);
        float acc = a[i];
        for (int bi = i0; bi <= i1; bi++) {
            if (scale_src(bi, g.off_y, g.nh, g.ah, g.mode) != ai) continue;
            for (int bj = j0; bj <= j1; bj++)
                if (scale_src(bj, g.off_x, g.nw, g.aw, g.mode) == aj) acc = __fadd_rn(acc, __ldg(b + (plane * g.bh + bi) * g.bw + bj));
        }
        a[i] = acc;
    }
}

// Counter-based uniform generator: the i-th value of stream (seed, offset) is a hash of its index, so the mask does not
// depend on the launch geometry and a seed reproduces it.  (Two rounds of a 64-bit mix of the splitmix kind.)
__device__ __forceinline__ float uniform01(unsigned long long seed, unsigned long long index) {
    unsigned long long z = seed + 0x9E3779B97F4A7C15ull * (index + 1);
    z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
    z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
    z ^= z >> 31;
    return (float)(z >> 40) * (1.0f / 16777216.0f);       // 24 random bits -> [0, 1)
}
__global__ void __launch_bounds__(kBlock) rand_binary_kernel(float *__restrict__ a, size_t n, float p, unsigned long long seed, unsigned long long offset) {
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) a[i] = uniform01(seed, offset + i) < p ? 1.0f : 0.0f;
}

}  // namespace

using namespace eb;

extern "C" {

int eddlb200_concat(int dev, float *a, float *const *parts, const size_t *part_sizes, const size_t *part_strides, int nparts, size_t steps, int derivative) {
    EB_CTX(dev);
    EB_REQUIRE(a && nparts >= 1 && parts && part_sizes && part_strides && steps > 0, "gpu_concat");
    size_t offset = 0, total = 0;
    for (int i = 0; i < nparts; i++) { EB_REQUIRE(parts[i] && part_strides[i] > 0 && part_sizes[i] % part_strides[i] == 0, "gpu_concat"); total += part_sizes[i]; }
    EB_REQUIRE(steps < 0xffffffffull, "gpu_concat");
    if (derivative) EB_READS(a, total * sizeof(float)); else EB_MODIFIES(a, total * sizeof(float));
    ProfScope prof(cx, PROF_ELEMENTWISE, (derivative ? 12.0 : 8.0) * (double)total);
    for (int i = 0; i < nparts; i++) {
        const size_t n = part_sizes[i];
        if (n) {
            if (derivative) { EB_MODIFIES(parts[i], n * sizeof(float)); concat_kernel<true><<<grid_for(n, kBlock), kBlock, 0, st>>>(a + offset, parts[i], n, (unsigned)part_strides[i], (unsigned)steps); }
            else { EB_READS(parts[i], n * sizeof(float)); concat_kernel<false><<<grid_for(n, kBlock), kBlock, 0, st>>>(a + offset, parts[i], n, (unsigned)part_strides[i], (unsigned)steps); }
            EB_LAUNCH_CHECK("gpu_concat");
        }
        offset += part_strides[i];
    }
    return 0;
}

int eddlb200_repeat_nn(int dev, const float *a, float *b, size_t rows_a, int cols_a, int size_r, int size_c) {
    EB_CTX(dev);
    EB_REQUIRE(a && b && cols_a > 0 && size_r > 0 && size_c > 0, "gpu_repeat_nn");
    const size_t nb = rows_a * size_r * (size_t)cols_a * size_c;
    if (!nb) return 0;
    EB_READS(a, rows_a * cols_a * sizeof(float)); EB_WRITES(b, nb * sizeof(float));
    ProfScope prof(cx, PROF_ELEMENTWISE, 4.0 * rows_a * cols_a + 4.0 * nb);
    repeat_nn_kernel<<<grid_for(nb, kBlock), kBlock, 0, st>>>(a, b, nb, cols_a * size_c, cols_a, size_r, size_c);
    EB_LAUNCH_CHECK("gpu_repeat_nn");
    return 0;
}

int eddlb200_repeat_nn_bwd(int dev, const float *d, float *a, size_t rows_a, int cols_a, int size_r, int size_c) {
    EB_CTX(dev);
    EB_REQUIRE(a && d && cols_a > 0 && size_r > 0 && size_c > 0, "gpu_d_repeat_nn");
    const size_t na = rows_a * cols_a;
    if (!na) return 0;
    EB_READS(d, na * size_r * size_c * sizeof(float)); EB_MODIFIES(a, na * sizeof(float));
    ProfScope prof(cx, PROF_ELEMENTWISE, 8.0 * na + 4.0 * na * size_r * size_c);
    repeat_nn_bwd_kernel<<<grid_for(na, kBlock), kBlock, 0, st>>>(d, a, na, cols_a * size_c, cols_a, size_r, size_c);
    EB_LAUNCH_CHECK("gpu_d_repeat_nn");
    return 0;
}

int eddlb200_flip_batch(int dev, const float *a, float *b, int n, int c, int h, int w, int axis, const unsigned char *apply_host) {
    EB_CTX(dev);
    EB_REQUIRE(a && b && a != b && n >= 0 && c > 0 && h > 0 && w > 0 && (axis == 0 || axis == 1) && (n == 0 || apply_host), "gpu_flip_random");
    const size_t total = (size_t)n * c * h * w;
    if (!total) return 0;
    EB_READS(a, total * sizeof(float)); EB_WRITES(b, total * sizeof(float));
    unsigned char *flags = (unsigned char *)scratch(cx, (size_t)n);
    if (!flags) return cudaErrorMemoryAllocation;
    cudaError_t e = cudaMemcpyAsync(flags, apply_host, (size_t)n, cudaMemcpyHostToDevice, st);      // pageable source: staged before return
    if (e != cudaSuccess) return cuda_status(e, "gpu_flip_random(flags)");
    ProfScope prof(cx, PROF_ELEMENTWISE, 8.0 * total);
    flip_kernel<<<grid_for(total, kBlock), kBlock, 0, st>>>(a, b, total, c, h, w, axis, flags);
    EB_LAUNCH_CHECK("gpu_flip_random");
    return 0;
}

int eddlb200_crop_scale_batch(int dev, const float *a, float *b, int n, int c, int ah, int aw, int bh, int bw, const int *boxes_host) {
    EB_CTX(dev);
    EB_REQUIRE(a && b && a != b && n >= 0 && c > 0 && ah > 0 && aw > 0 && bh > 0 && bw > 0 && (n == 0 || boxes_host), "gpu_crop_scale_random");
    const size_t total = (size_t)n * c * bh * bw;
    if (!total) return 0;
    // (y0, x0, y1, x1) per image; the source extent is y1 - y0 + 1 like the reference's cpu_single_crop_scale
    std::vector<int4> box((size_t)n);
    for (int i = 0; i < n; i++) {
        const int y0 = boxes_host[4 * i], x0 = boxes_host[4 * i + 1], hc = boxes_host[4 * i + 2] - y0 + 1, wc = boxes_host[4 * i + 3] - x0 + 1;
        EB_REQUIRE(y0 >= 0 && x0 >= 0 && hc >= 1 && wc >= 1 && ((long long)(bh - 1) * hc) / bh + y0 < ah && ((long long)(bw - 1) * wc) / bw + x0 < aw, "gpu_crop_scale_random(box)");
        box[i] = make_int4(y0, x0, hc, wc);
    }
    EB_READS(a, (size_t)n * c * ah * aw * sizeof(float)); EB_WRITES(b, total * sizeof(float));
    int4 *dbox = (int4 *)scratch(cx, (size_t)n * sizeof(int4));
    if (!dbox) return cudaErrorMemoryAllocation;
    cudaError_t e = cudaMemcpyAsync(dbox, box.data(), (size_t)n * sizeof(int4), cudaMemcpyHostToDevice, st);
    if (e != cudaSuccess) return cuda_status(e, "gpu_crop_scale_random(boxes)");
    ProfScope prof(cx, PROF_ELEMENTWISE, 8.0 * total);
    crop_scale_kernel<<<grid_for(total, kBlock), kBlock, 0, st>>>(a, b, total, c, ah, aw, bh, bw, dbox);
    EB_LAUNCH_CHECK("gpu_crop_scale_random");
    return 0;
}

static int scale_geom(const char *what, ScaleGeom &g, int ah, int aw, int bh, int bw, int new_h, int new_w, int wrap, float cval, int mode, bool backward) {
    if (!(ah > 0 && aw > 0 && bh > 0 && bw > 0 && new_h > 0 && new_w > 0) || !(mode == 0 || mode == 2 || mode == 3) || (mode == 2 && (ah < 2 || aw < 2)))
        return set_error(EDDLB200_EINVAL, "%s: bad shape or transformation mode", what);
    g = ScaleGeom{ah, aw, bh, bw, new_h, new_w, (int)((new_h - bh) / 2.0f), (int)((new_w - bw) / 2.0f), mode, wrap, cval};
    // the mapping is monotonic: the first and the last output index tell whether any source index leaves the tensor
    const bool inside = scale_src(0, g.off_y, new_h, ah, mode) >= 0 && scale_src(bh - 1, g.off_y, new_h, ah, mode) < ah &&
                        scale_src(0, g.off_x, new_w, aw, mode) >= 0 && scale_src(bw - 1, g.off_x, new_w, aw, mode) < aw;
    if (!inside && !(wrap == 0 || (wrap == 5 && !backward && ah == bh && aw == bw)))
        return set_error(EDDLB200_EINVAL, "%s: source indices leave the tensor and wrapping mode %d is not implemented for that", what, wrap);
    return 0;
}

int eddlb200_resize(int dev, const float *a, float *b, int n, int c, int ah, int aw, int bh, int bw, int new_h, int new_w, int wrap, float cval, int mode) {
    EB_CTX(dev);
    EB_REQUIRE(a && b && a != b && n >= 0 && c > 0, "gpu_scale");
    ScaleGeom g;
    if (int r = scale_geom("gpu_scale", g, ah, aw, bh, bw, new_h, new_w, wrap, cval, mode, false)) return r;
    const size_t total = (size_t)n * c * bh * bw;
    if (!total) return 0;
    EB_READS(a, (size_t)n * c * ah * aw * sizeof(float)); EB_WRITES(b, total * sizeof(float));
    ProfScope prof(cx, PROF_ELEMENTWISE, 8.0 * total);
    scale_kernel<<<grid_for(total, kBlock), kBlock, 0, st>>>(a, b, total, g);
    EB_LAUNCH_CHECK("gpu_scale");
    return 0;
}

int eddlb200_resize_bwd(int dev, float *a_delta, const float *b_delta, int n, int c, int ah, int aw, int bh, int bw, int new_h, int new_w, int wrap, float cval, int mode) {
    EB_CTX(dev);
    EB_REQUIRE(a_delta && b_delta && a_delta != b_delta && n >= 0 && c > 0, "gpu_scale_back");
    ScaleGeom g;
    if (int r = scale_geom("gpu_scale_back", g, ah, aw, bh, bw, new_h, new_w, wrap, cval, mode, true)) return r;
    const size_t total = (size_t)n * c * ah * aw;
    if (!total) return 0;
    EB_READS(b_delta, (size_t)n * c * bh * bw * sizeof(float)); EB_MODIFIES(a_delta, total * sizeof(float));
    ProfScope prof(cx, PROF_ELEMENTWISE, 8.0 * total + 4.0 * n * c * bh * bw);
    scale_bwd_kernel<<<grid_for(total, kBlock), kBlock, 0, st>>>(a_delta, b_delta, total, g);
    EB_LAUNCH_CHECK("gpu_scale_back");
    return 0;
}

int eddlb200_rand_binary(int dev, float *a, size_t n, float p, size_t seed, size_t offset) {
    EB_CTX(dev);
    if (!n) return 0;
    EB_REQUIRE(a, "gpu_rand_binary");
    EB_WRITES(a, n * sizeof(float));
    ProfScope prof(cx, PROF_ELEMENTWISE, 4.0 * n);
    rand_binary_kernel<<<grid_for(n, kBlock), kBlock, 0, st>>>(a, n, p, (unsigned long long)seed, (unsigned long long)offset);
    EB_LAUNCH_CHECK("gpu_rand_binary");
    return 0;
}

}  // extern "C"
