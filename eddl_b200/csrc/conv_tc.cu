// placeholder, replaced below
#include "conv_common.cuh"
namespace eb {
int conv_tc_fwd(DevCtx *, cudaStream_t, const ConvGeom &, const float *, const float *, const float *, float *, int) { return 1; }
int conv_tc_bwd_data(DevCtx *, cudaStream_t, const ConvGeom &, const float *, const float *, float *, int) { return 1; }
int conv_tc_bwd_weight(DevCtx *, cudaStream_t, const ConvGeom &, const float *, const float *, float *, int) { return 1; }
}
