// Geometry and internal entry points shared by the Conv2D kernels.
#pragma once
#include "common.cuh"

namespace eb {

struct ConvGeom {
    int n, c, ih, iw;       // input  [n, c, ih, iw]
    int k, kr, kc;          // filter [k, c, kr, kc]
    int oh, ow;             // output [n, k, oh, ow]
    int sr, sc, pt, pl;     // strides, top / left zero padding
};

// Exact-fp32 FMA implicit GEMM (conv_simt.cu).
int conv_simt_fwd(DevCtx *cx, cudaStream_t st, const ConvGeom &g, const float *x, const float *w, const float *bias, float *y);
int conv_simt_bwd_data(DevCtx *cx, cudaStream_t st, const ConvGeom &g, const float *dy, const float *w, float *dx);
int conv_simt_bwd_weight(DevCtx *cx, cudaStream_t st, const ConvGeom &g, const float *x, const float *dy, float *gw);

// Tensor-core implicit GEMM (conv_tc.cu).  Each returns 1 when the shape is outside what
// the kernel takes (the caller then uses the FMA path), 0 on success, or an error code.
int conv_tc_fwd(DevCtx *cx, cudaStream_t st, const ConvGeom &g, const float *x, const float *w, const float *bias, float *y, int precision);
// dx_zero: dx is known to hold zeros (the caller took over a deferred zero fill of it), so the result may be stored
// instead of added; routes that cannot use this write the zeros first.
int conv_tc_bwd_data(DevCtx *cx, cudaStream_t st, const ConvGeom &g, const float *dy, const float *w, float *dx, int precision, bool dx_zero);
int conv_tc_bwd_weight(DevCtx *cx, cudaStream_t st, const ConvGeom &g, const float *x, const float *dy, float *gw, int precision, bool gw_zero);

// 1 (default): the tensor-core kernel's prefetch warp pulls the activation operand of 1x1 layers into L2 ahead of the gather.
int conv_tc_set_prefetch(int on);

// Reads and clears the device's time-out flag of the tensor-core kernels (blocking).
int conv_tc_status(int dev, cudaStream_t st, int *out);

// out[i] += sum_{s<splits} part[s*count + i], s ascending.
int splitk_reduce_accumulate(DevCtx *cx, cudaStream_t st, const float *part, float *out, size_t count, int splits);

}  // namespace eb
