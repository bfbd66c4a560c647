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
int conv_tc_gemm(DevCtx *cx, cudaStream_t st, const float *a, int ta, const float *b, int tb, float *c, int inc_c, int m, int n, int k, int precision);
bool conv_tc_allowed();          // false while eddlb200_set_option("conv_path", 1) / EDDL_B200_CONV=simt forces the fp32 FMA kernels
int conv_tc_bwd_weight(DevCtx *cx, cudaStream_t st, const ConvGeom &g, const float *x, const float *dy, float *gw, int precision, bool gw_zero);

// 1 (default): the tensor-core kernel's prefetch warp pulls the activation operand of 1x1 layers into L2 ahead of the gather.
int conv_tc_set_prefetch(int on);
// 2 (default): 1x1 stride-1 forward / backward-data layers are fed and drained by TMA tensor copies, accumulating outputs by
// TMA fp32 adds; 1: only where the output is stored; 0: every layer takes the gather kernel.
int conv_tc_set_tma(int level);
// 1 (default): backward-weight of those layers has both operands copied by TMA into the operand ring; 2: in addition the landed
// values serve as the hi plane unmasked; 0: the 16-byte gather.
int conv_tc_set_tma_wgrad(int level);
int conv_tc_set_tma_wgrad_3x3(int on);
// 1 (default): forward / backward-data of 3x3 stride-1 "same" layers (planes up to 60 pixels wide) read raw slabs delivered by TMA
int conv_tc_set_tma_3x3(int on);
// 1 (default): packed weight images are kept per (weight tensor, tiling) and re-packed, all stale ones in one launch, only after
// the tensor has been written; 0: every call packs its own.
int conv_tc_set_pack_cache(int on);

// Reads and clears the device's time-out flag of the tensor-core kernels (blocking).
int conv_tc_status(int dev, cudaStream_t st, int *out);

// out[i] += sum_{s<splits} part[s*count + i], s ascending.
int splitk_reduce_accumulate(DevCtx *cx, cudaStream_t st, const float *part, float *out, size_t count, int splits);

}  // namespace eb
