// Dense-layer algebra: C = op(A)*op(B) (+C), row bias add, column/row sums.
// Replaces gpu_mult2D (cublasSgemm, EDDL src/hardware/gpu/gpu_math.cu:457-490),
// gpu_sum2D_rowwise (gpu_math.cu:517-528) and gpu_reduce_sum2D (gpu_reduction.cu:232-244,
// one atomicAdd per element); arithmetic as cpu_mult2D / cpu_sum2D_rowwise /
// cpu_reduce_sum2D (src/hardware/cpu/cpu_math.cpp:302-325,369-380; cpu_reduction.cpp:91-112).
// The dense layers of the convnets are small (<= 64x2048x1000), so this is an fp32
// FMA kernel: 64x64 block tile, 16-deep k slices staged in shared memory, 4x4
// accumulators per thread, exact fp32 accumulation.  When the output has fewer tiles than the GPU has SMs (batch 64:
// 16 or 32 tiles) the k range is split across blockIdx.z and the partials are combined in a fixed order.
#include "common.cuh"
#include "conv_common.cuh"

namespace {

using namespace eb;

constexpr int BM = 64, BN = 64, BK = 16, TB = 256;

// Row-major storage.  A: ta ? [k,m] : [m,k]; B: tb ? [n,k] : [k,n]; C: [m,n].
__global__ void __launch_bounds__(TB) sgemm_kernel(const float *__restrict__ A, int ta, const float *__restrict__ B, int tb,
                                                   float *__restrict__ C, int inc_c, int m, int n, int k, int k_per_split,
                                                   float *__restrict__ part) {
    __shared__ float As[BK][BM + 4];
    __shared__ float Bs[BK][BN + 4];
    const int tx = threadIdx.x % 16, ty = threadIdx.x / 16;
    const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
    float acc[4][4] = {};
    const int kbeg = blockIdx.z * k_per_split;
    int kend = k;
    if (part) { kend = min(k, kbeg + k_per_split); C = part + (size_t)blockIdx.z * m * n; inc_c = 0; }
    for (int k0 = kbeg; k0 < kend; k0 += BK) {
        for (int e = threadIdx.x; e < BM * BK; e += TB) {
            // choose the traversal that is contiguous in memory
            int mi, ki;
            if (ta) { mi = e % BM; ki = e / BM; } else { ki = e % BK; mi = e / BK; }
            const int gm = m0 + mi, gk = k0 + ki;
            float v = 0.f;
            if (gm < m && gk < kend) v = ta ? A[(size_t)gk * m + gm] : A[(size_t)gm * k + gk];
            As[ki][mi] = v;
        }
        for (int e = threadIdx.x; e < BN * BK; e += TB) {
            int ni, ki;
            if (tb) { ki = e % BK; ni = e / BK; } else { ni = e % BN; ki = e / BN; }
            const int gn = n0 + ni, gk = k0 + ki;
            float v = 0.f;
            if (gn < n && gk < kend) v = tb ? B[(size_t)gn * k + gk] : B[(size_t)gk * n + gn];
            Bs[ki][ni] = v;
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
        if (gm >= m) continue;
#pragma unroll
        for (int j = 0; j < 4; j++) {
            const int gn = n0 + tx * 4 + j;
            if (gn >= n) continue;
            float *c = C + (size_t)gm * n + gn;
            *c = inc_c == 1 ? __fadd_rn(*c, acc[i][j]) : (inc_c == 2 ? __fadd_rn(0.f, acc[i][j]) : acc[i][j]);     // 2: c is known to hold zeros
        }
    }
}

// c[i] = (inc_c ? c[i] : 0) + part[0][i] + part[1][i] + ...   (fixed order)
__global__ void __launch_bounds__(256) sgemm_combine_kernel(const float *__restrict__ part, float *__restrict__ c, size_t count, int splits, int inc_c) {
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < count; i += stride) {
        float v = inc_c ? c[i] : 0.f;
        for (int z = 0; z < splits; z++) v = __fadd_rn(v, part[(size_t)z * count + i]);
        c[i] = v;
    }
}

__global__ void __launch_bounds__(256) rowbias_kernel(const float *__restrict__ a, const float *__restrict__ b, float *__restrict__ c, size_t total, int cols) {
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    for (size_t p = (size_t)blockIdx.x * blockDim.x + threadIdx.x; p < total; p += stride) c[p] = __fadd_rn(a[p], __ldg(b + (p % cols)));
}

// axis 0: one thread per column walks the rows in order (the reference's order), coalesced
// across columns.  axis 1: one warp per row.
__global__ void __launch_bounds__(256) colsum_kernel(const float *__restrict__ a, float *__restrict__ b, int rows, int cols, int inc_b) {
    const int j = blockIdx.x * blockDim.x + threadIdx.x;
    if (j >= cols) return;
    float s = inc_b ? b[j] : 0.f;
    for (int i = 0; i < rows; i++) s = __fadd_rn(s, a[(size_t)i * cols + j]);
    b[j] = s;
}
__global__ void __launch_bounds__(256) rowsum_kernel(const float *__restrict__ a, float *__restrict__ b, int rows, int cols, int inc_b) {
    const int lane = threadIdx.x & 31;
    const int r = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (r >= rows) return;
    float s = 0.f;
    for (int j = lane; j < cols; j += 32) s += a[(size_t)r * cols + j];
    s = warp_sum(s);
    if (lane == 0) b[r] = inc_b ? __fadd_rn(b[r], s) : s;
}

}  // namespace

using namespace eb;

extern "C" {

int eddlb200_mult2d(int dev, const float *a, int ta, const float *b, int tb, float *c, int inc_c, int m, int n, int k) {
    EB_CTX(dev);
    EB_REQUIRE(a && b && c && m >= 0 && n >= 0 && k >= 0, "gpu_mult2D");
    if (m == 0 || n == 0) return 0;
    EB_READS(a, (size_t)m * k * sizeof(float)); EB_READS(b, (size_t)k * n * sizeof(float));
    if (inc_c && lz_any(cx) && c != a && c != b) {
        int status = 0;
        if (lz_take(cx, st, c, (size_t)m * n * sizeof(float), &status)) inc_c = 2;
        if (status) return status;
    }
    if (inc_c == 1) EB_MODIFIES(c, (size_t)m * n * sizeof(float)); else EB_WRITES(c, (size_t)m * n * sizeof(float));
    ProfScope prof(cx, PROF_GEMM, 2.0 * m * (double)n * k);
    // Large products (ResNet-50's 2048 x 1000 classifier at batch 64) run on the tensor-core kernel (3xTF32, like the
    // convolutions).  Below 2^26 multiply-adds its extra launches (operand packing, split-K combine) cost more than they save
    // (VGG-16-BN's 512 x 512 layers at batch 128 were 2 % of a step slower there), and a library forced to the FMA path stays here.
    if (conv_tc_allowed() && k >= 32 && (double)m * n * k >= 67108864.0) {
        const int r = conv_tc_gemm(cx, st, a, ta, b, tb, c, inc_c, m, n, k, 0);
        if (r != 1) return r;
    }
    dim3 grid((n + BN - 1) / BN, (m + BM - 1) / BM);
    const int tiles = (int)(grid.x * grid.y);
    int splits = 1;
    if (tiles < EDDLB200_NUM_SMS) {
        splits = (2 * EDDLB200_NUM_SMS + tiles - 1) / tiles;
        if (splits > k / (4 * BK)) splits = k / (4 * BK);
        if (splits < 1) splits = 1;
    }
    if (splits == 1) {
        sgemm_kernel<<<grid, TB, 0, st>>>(a, ta, b, tb, c, inc_c, m, n, k, k, nullptr);
        EB_LAUNCH_CHECK("gpu_mult2D");
        return 0;
    }
    int kps = (k + splits - 1) / splits;
    kps = (kps + BK - 1) / BK * BK;
    splits = (k + kps - 1) / kps;
    const size_t count = (size_t)m * n;
    float *part = (float *)scratch(cx, count * splits * sizeof(float));
    if (!part) return cudaErrorMemoryAllocation;
    grid.z = splits;
    sgemm_kernel<<<grid, TB, 0, st>>>(a, ta, b, tb, c, inc_c, m, n, k, kps, part);
    EB_LAUNCH_CHECK("gpu_mult2D");
    sgemm_combine_kernel<<<grid_for(count, 256), 256, 0, st>>>(part, c, count, splits, inc_c == 1);
    EB_LAUNCH_CHECK("gpu_mult2D(combine)");
    return 0;
}

int eddlb200_sum2d_rowwise(int dev, const float *a, const float *b, float *c, int rows, int cols) {
    EB_CTX(dev);
    EB_REQUIRE(a && b && c && rows >= 0 && cols >= 0, "gpu_sum2D_rowwise");
    const size_t total = (size_t)rows * cols;
    if (!total) return 0;
    EB_READS(a, total * sizeof(float)); EB_READS(b, (size_t)cols * sizeof(float));
    if (c != a) EB_WRITES(c, total * sizeof(float));
    rowbias_kernel<<<grid_for(total, 256), 256, 0, st>>>(a, b, c, total, cols);
    EB_LAUNCH_CHECK("gpu_sum2D_rowwise");
    return 0;
}

int eddlb200_reduce_sum2d(int dev, const float *a, float *b, int rows, int cols, int axis, int inc_b) {
    EB_CTX(dev);
    EB_REQUIRE(a && b && rows >= 0 && cols >= 0 && (axis == 0 || axis == 1), "gpu_reduce_sum2D");
    EB_READS(a, (size_t)rows * cols * sizeof(float));
    if (inc_b) EB_MODIFIES(b, (size_t)(axis == 0 ? cols : rows) * sizeof(float)); else EB_WRITES(b, (size_t)(axis == 0 ? cols : rows) * sizeof(float));
    if (axis == 0) {
        if (!cols) return 0;
        colsum_kernel<<<(cols + 255) / 256, 256, 0, st>>>(a, b, rows, cols, inc_b);
    } else {
        if (!rows) return 0;
        rowsum_kernel<<<(rows + 7) / 8, 256, 0, st>>>(a, b, rows, cols, inc_b);
    }
    EB_LAUNCH_CHECK("gpu_reduce_sum2D");
    return 0;
}

}  // extern "C"
