// C++ shim: defines the `gpu_*` free functions that EDDL v1.1's Tensor / tensorNN dispatch
// calls when built with -DcGPU (declared in include/eddl/hardware/gpu/gpu_tensor.h:35-53,
// gpu_hw.h:30-257, nn/gpu_tensor_nn.h:26-147) on top of the eddl_b200 C ABI.  Same names,
// argument meaning and error behaviour as the reference's src/hardware/gpu: failures surface
// as std::runtime_error("[CUDA ERROR]: ...") exactly like check_cuda (gpu_tensor.cu:103-112).
// Functions outside the convnet training step are not defined here; the build turns each of
// them into a stub that throws (there is no CPU fallback).
//
// Peephole fusion: LBatchNorm and LActivation("relu") are separate layers with separate
// output tensors, so the BN kernel cannot know its consumer when it is called.  The shim
// therefore keeps the apply pass of the most recent gpu_batchnorm_forward pending (per
// device) until the next backend call: if that call is gpu_relu on the BN output it launches
// one kernel that writes both tensors; any other call flushes the pending pass first.
#include <cstdlib>
#include <cstring>
#include <random>
#include <stdexcept>
#include <string>
#include <vector>

#include "eddl/hardware/gpu/gpu_tensor.h"
#include "eddl/hardware/gpu/gpu_hw.h"
#include "eddl/hardware/gpu/nn/gpu_tensor_nn.h"
#include "eddl_b200.h"

cublasHandle_t hcublas[64];              // declared by the reference header; unused here
curandGenerator_t random_generator[64];

namespace {

void ok(int status, const char *where) {
    if (status == 0) return;
    std::string text = eddlb200_last_error();
    if (status > 0) throw std::runtime_error(text.empty() ? std::string("[CUDA ERROR]: ") + where : text);
    throw std::runtime_error(std::string("[eddl_b200 ERROR ") + std::to_string(status) + "]: " + text + " (" + where + ")");
}

// ---- pending BN apply (see header comment) ---------------------------------------------
struct PendingBN {
    bool active = false;
    int b, z, rc; const float *input; float *output, *opa, *gmean, *gvar; const float *g, *bb;
    float *mean, *var; int trmode; float eps, momentum;
};
PendingBN g_pending[64];
bool fusion_enabled() {
    static int v = -1;
    if (v < 0) { const char *e = getenv("EDDL_B200_FUSE_BN_RELU"); v = (e && e[0] == '0') ? 0 : 1; }
    return v == 1;
}
void launch_bn(int dev, PendingBN &p, float *relu_out) {
    p.active = false;
    ok(eddlb200_bn_fwd(dev, p.b, p.z, p.rc, p.input, p.output, p.opa, p.gmean, p.gvar, p.g, p.bb, p.mean, p.var,
                       p.trmode, p.eps, p.momentum, relu_out), "gpu_batchnorm_forward");
}
// Pending gpu_fill_ calls (per device).  Net::do_reset / do_reset_grads zero every delta and every gradient tensor with
// one call each -- several hundred back-to-back launches per step for a ResNet-50; they are collected here and issued as
// one multi-tensor launch as soon as any other backend call arrives.
struct FillQueue { std::vector<float *> ptrs; std::vector<size_t> sizes; std::vector<float> values; };
FillQueue g_fills[64];
bool fill_batching_enabled() {
    static int v = -1;
    if (v < 0) { const char *e = getenv("EDDL_B200_BATCH_FILLS"); v = (e && e[0] == '0') ? 0 : 1; }
    return v == 1;
}
inline void flush(int dev) {
    if (dev < 0 || dev >= 64) return;
    FillQueue &q = g_fills[dev];
    if (!q.ptrs.empty()) {
        std::vector<float *> p; std::vector<size_t> s; std::vector<float> v;
        p.swap(q.ptrs); s.swap(q.sizes); v.swap(q.values);
        ok(eddlb200_fill_multi(dev, p.data(), s.data(), v.data(), (int)p.size()), "gpu_fill_");
    }
    if (g_pending[dev].active) launch_bn(dev, g_pending[dev], nullptr);
}
inline int dev_of(const Tensor *t) { flush(t->gpu_device); return t->gpu_device; }

}  // namespace

// ---- gpu_tensor.h ---------------------------------------------------------------------
void check_cuda(cudaError_t err, const char *msg) {
    if (err != cudaSuccess) {
        std::string s = "[CUDA ERROR]: " + std::string(cudaGetErrorString(err)) + " (" + std::to_string(err) + ") raised in " + std::string(msg);
        throw std::runtime_error(s);
    }
}
void check_cublas(cublasStatus_t status, const char *f) {
    if (status != CUBLAS_STATUS_SUCCESS) throw std::runtime_error(std::string("[CUBLAS ERROR]: ") + f);
}
void check_curand(curandStatus_t status, const char *f) {
    if (status != CURAND_STATUS_SUCCESS) throw std::runtime_error(std::string("[CURAND ERROR]: ") + f);
}
namespace {
// Net::do_reset zeroes every delta tensor at the start of a step, and every backward kernel then ADDS into its parent's
// delta.  With "lazy_zero" on, the library records those fills instead of running them and lets the first accumulating
// kernel store its result (EDDL_B200_LAZY_ZERO=0 runs every fill as issued).
void configure_once() {
    static bool done = false;
    if (done) return;
    done = true;
    const char *e = getenv("EDDL_B200_LAZY_ZERO");
    ok(eddlb200_set_option("lazy_zero", (e && e[0] == '0') ? 0 : 1), "gpu_init");
}
}
void gpu_set_device(int device) { configure_once(); ok(eddlb200_init(device), "gpu_set_device"); }
void gpu_init(int device) { configure_once(); ok(eddlb200_init(device), "gpu_init"); }
int gpu_devices() { int n = 0; eddlb200_device_count(&n); return n; }

float *gpu_create_tensor(int dev, int size) {
    configure_once();
    void *p = nullptr;
    ok(eddlb200_alloc(dev, (size_t)size * sizeof(float), &p), "gpu_create_tensor");
    return (float *)p;
}
void gpu_delete_tensor(int dev, float *p) { flush(dev); ok(eddlb200_free(dev, p), "gpu_delete_tensor"); }
void gpu_delete_tensor_int(int dev, int *p) { flush(dev); ok(eddlb200_free(dev, p), "gpu_delete_tensor_int"); }

// ---- copies / fills ---------------------------------------------------------------------
// Host -> device copies go through the library's pinned staging ring, so that Net::train_batch's per-step copies of inputs
// and targets (src/net/net_api.cpp:1273-1283; blocking cudaMemcpy in the reference, gpu_core.cu:49-53) neither wait for the
// previous step's kernels nor keep the GPU idle while they run.  EDDL_B200_STAGED_H2D=0 restores the blocking copy.
namespace {
bool staged_h2d() {
    static int v = -1;
    if (v < 0) { const char *e = getenv("EDDL_B200_STAGED_H2D"); v = (e && e[0] == '0') ? 0 : 1; }
    return v == 1;
}
}
void gpu_copy_to_gpu(float *nptr, Tensor *B) {
    const int dev = dev_of(B);
    if (staged_h2d()) ok(eddlb200_memcpy_h2d_staged(dev, B->ptr, nptr, B->size * sizeof(float)), "gpu_copy_to_gpu");
    else ok(eddlb200_memcpy_h2d(dev, B->ptr, nptr, B->size * sizeof(float)), "gpu_copy_to_gpu");
}
void gpu_copy_from_gpu(Tensor *A, float *nptr) { ok(eddlb200_memcpy_d2h(dev_of(A), nptr, A->ptr, A->size * sizeof(float)), "gpu_copy_from_gpu"); }
void gpu_copy_gpu(Tensor *A, Tensor *B) {
    if (A->gpu_device != B->gpu_device) {
        // two replicas of one process (CS_GPU({1,1,...})): a direct peer copy instead of the host round trip
        const int src = dev_of(A), dst = dev_of(B);
        ok(eddlb200_memcpy_peer(dst, B->ptr, src, A->ptr, A->size * sizeof(float)), "gpu_copy_gpu");
        return;
    }
    ok(eddlb200_memcpy_d2d(dev_of(A), B->ptr, A->ptr, A->size * sizeof(float)), "gpu_copy_gpu");
}
void gpu_fill_(Tensor *A, float v) {
    const int dev = A->gpu_device;
    if (fill_batching_enabled() && dev >= 0 && dev < 64 && !g_pending[dev].active) {
        FillQueue &q = g_fills[dev];
        // a tensor filled twice before the flush keeps only the last value (two queued fills would race)
        for (size_t i = 0; i < q.ptrs.size(); i++)
            if (q.ptrs[i] == A->ptr && q.sizes[i] == A->size) { q.values[i] = v; return; }
        q.ptrs.push_back(A->ptr); q.sizes.push_back(A->size); q.values.push_back(v);
        return;
    }
    ok(eddlb200_fill(dev_of(A), A->ptr, A->size, v), "gpu_fill_");
}

// Device-side initialisers (the reference uses cuRAND MRG32K3A with a fixed seed per device,
// gpu_tensor.cu:179-185): values are drawn on the host with a fixed-seed generator and copied.
namespace {
std::mt19937 &rng(int dev) { static std::mt19937 g[64]; static bool init = false; if (!init) { for (int i = 0; i < 64; i++) g[i].seed(1234); init = true; } return g[dev & 63]; }
template <typename D> void fill_random(Tensor *A, D dist) {
    std::vector<float> h(A->size);
    auto &g = rng(A->gpu_device);
    for (auto &x : h) x = dist(g);
    ok(eddlb200_memcpy_h2d(dev_of(A), A->ptr, h.data(), h.size() * sizeof(float)), "gpu_rand");
}
}
void gpu_rand_uniform(Tensor *A, float v) { std::uniform_real_distribution<float> d(0.f, 1.f); fill_random(A, [&](std::mt19937 &g) { return d(g) * v; }); }
void gpu_rand_signed_uniform(Tensor *A, float v) { std::uniform_real_distribution<float> d(-1.f, 1.f); fill_random(A, [&](std::mt19937 &g) { return d(g) * v; }); }
void gpu_rand_normal(Tensor *A, float m, float s) { std::normal_distribution<float> d(m, s); fill_random(A, [&](std::mt19937 &g) { return d(g); }); }
// Dropout's mask (LDropout::forward, src/layers/core/layer_drop.cpp:50-58) is as large as the activations: it is drawn on
// the device.  The stream position advances by the tensor size, so successive masks are independent.
void gpu_rand_binary(Tensor *A, float v) {
    static size_t position[64] = {};
    const int dev = dev_of(A);
    ok(eddlb200_rand_binary(dev, A->ptr, A->size, v, 1234, position[dev & 63]), "gpu_rand_binary");
    position[dev & 63] += A->size;
}

// ---- elementwise ------------------------------------------------------------------------
void gpu_add(Tensor *A, Tensor *B, float v) { ok(eddlb200_addc(dev_of(A), A->ptr, B->ptr, v, A->size), "gpu_add"); }
void gpu_mult(Tensor *A, Tensor *B, float v) { ok(eddlb200_scale(dev_of(A), A->ptr, B->ptr, v, A->size), "gpu_mult"); }
void gpu_sqr(Tensor *A, Tensor *B) { ok(eddlb200_sqr(dev_of(A), A->ptr, B->ptr, A->size), "gpu_sqr"); }
void gpu_sqrt(Tensor *A, Tensor *B) { ok(eddlb200_sqrt(dev_of(A), A->ptr, B->ptr, A->size), "gpu_sqrt"); }
void gpu_clamp(Tensor *A, Tensor *B, float min, float max) { ok(eddlb200_clamp(dev_of(A), A->ptr, B->ptr, min, max, A->size), "gpu_clamp"); }
void gpu_add(float scA, Tensor *A, float scB, Tensor *B, Tensor *C, int incC) {
    ok(eddlb200_axpby(dev_of(A), scA, A->ptr, scB, B->ptr, C->ptr, incC, A->size), "gpu_add");
}
void gpu_inc(Tensor *A, Tensor *B) { ok(eddlb200_inc(dev_of(A), A->ptr, B->ptr, A->size), "gpu_inc"); }
void gpu_el_div(Tensor *A, Tensor *B, Tensor *C, int incC) { ok(eddlb200_el_div(dev_of(A), A->ptr, B->ptr, C->ptr, incC, A->size), "gpu_el_div"); }
void gpu_el_mult(Tensor *A, Tensor *B, Tensor *C, int incC) { ok(eddlb200_el_mult(dev_of(A), A->ptr, B->ptr, C->ptr, incC, A->size), "gpu_el_mult"); }

// ---- dense ------------------------------------------------------------------------------
void gpu_mult2D(Tensor *A, int tA, Tensor *B, int tB, Tensor *C, int incC) {
    const int m = tA ? A->shape[1] : A->shape[0];
    const int k = tA ? A->shape[0] : A->shape[1];
    const int n = tB ? B->shape[0] : B->shape[1];
    ok(eddlb200_mult2d(dev_of(A), A->ptr, tA, B->ptr, tB, C->ptr, incC, m, n, k), "gpu_mult2D");
}
void gpu_sum2D_rowwise(Tensor *A, Tensor *B, Tensor *C) { ok(eddlb200_sum2d_rowwise(dev_of(A), A->ptr, B->ptr, C->ptr, A->shape[0], A->shape[1]), "gpu_sum2D_rowwise"); }
void gpu_reduce_sum2D(Tensor *A, Tensor *B, int axis, int incB) { ok(eddlb200_reduce_sum2d(dev_of(A), A->ptr, B->ptr, A->shape[0], A->shape[1], axis, incB), "gpu_reduce_sum2D"); }

// ---- padding (pads = top, right, bottom, left; LPad, src/layers/da/layer_pad.cpp:18-48) ----
void gpu_pad(Tensor *A, Tensor *B, vector<int> pads) {
    ok(eddlb200_pad(dev_of(A), A->ptr, B->ptr, A->shape[0], A->shape[1], A->shape[2], A->shape[3], pads[0], pads[2], pads[3], pads[1]), "gpu_pad");
}
void gpu_pad_back(Tensor *A, Tensor *B, vector<int> pads) {
    ok(eddlb200_pad_bwd(dev_of(A), A->ptr, B->ptr, A->shape[0], A->shape[1], A->shape[2], A->shape[3], pads[0], pads[2], pads[3], pads[1]), "gpu_pad_back");
}

// ---- Concat, UpSampling, random flips and crops (the host side draws the random decisions) ----------------------
void gpu_concat(Tensor *A, vector<Tensor *> t, unsigned int axis, bool derivative) {
    std::vector<float *> parts; std::vector<size_t> sizes, strides;
    for (Tensor *p : t) { parts.push_back(p->ptr); sizes.push_back(p->size); strides.push_back((size_t)p->stride[axis] * p->shape[axis]); }
    ok(eddlb200_concat(dev_of(A), A->ptr, parts.data(), sizes.data(), strides.data(), (int)parts.size(), (size_t)A->stride[axis] * A->shape[axis], derivative),
       "gpu_concat");
}
void gpu_repeat_nn(Tensor *A, Tensor *B, vector<int> size) {
    ok(eddlb200_repeat_nn(dev_of(A), A->ptr, B->ptr, A->size / A->shape[3], A->shape[3], size[0], size[1]), "gpu_repeat_nn");
}
void gpu_d_repeat_nn(Tensor *D, Tensor *A, vector<int> size) {
    ok(eddlb200_repeat_nn_bwd(dev_of(A), D->ptr, A->ptr, A->size / A->shape[3], A->shape[3], size[0], size[1]), "gpu_d_repeat_nn");
}
void gpu_scale(Tensor *A, Tensor *B, vector<int> new_shape, int wrapping_mode, float constant, int transformation_mode) {
    ok(eddlb200_resize(dev_of(A), A->ptr, B->ptr, A->shape[0], A->shape[1], A->shape[2], A->shape[3], B->shape[2], B->shape[3],
                      new_shape[0], new_shape[1], wrapping_mode, constant, transformation_mode), "gpu_scale");
}
void gpu_scale_back(Tensor *A, Tensor *B, vector<int> new_shape, int wrapping_mode, float constant, int transformation_mode) {
    ok(eddlb200_resize_bwd(dev_of(A), A->ptr, B->ptr, A->shape[0], A->shape[1], A->shape[2], A->shape[3], B->shape[2], B->shape[3],
                          new_shape[0], new_shape[1], wrapping_mode, constant, transformation_mode), "gpu_scale_back");
}
void gpu_flip_random(Tensor *A, Tensor *B, int axis) {
    std::uniform_real_distribution<float> u(0.f, 1.f);
    std::vector<unsigned char> apply(A->shape[0]);
    for (auto &a : apply) a = u(rng(A->gpu_device)) >= 0.5f;               // cpu_flip_random, src/hardware/cpu/cpu_da.cpp:584-595
    ok(eddlb200_flip_batch(dev_of(A), A->ptr, B->ptr, A->shape[0], A->shape[1], A->shape[2], A->shape[3], axis, apply.data()), "gpu_flip_random");
}
void gpu_crop_scale_random(Tensor *A, Tensor *B, vector<float> factor, int wrapping_mode, float constant) {
    (void)wrapping_mode; (void)constant;                                    // unused by the reference's arithmetic as well
    std::vector<int> boxes(4 * (size_t)A->shape[0]);
    auto &g = rng(A->gpu_device);
    for (int b = 0; b < A->shape[0]; b++) {
        // cpu_crop_scale_random, src/hardware/cpu/cpu_da.cpp:625-646
        const float scale = std::uniform_real_distribution<float>(factor[0], factor[1])(g);
        const int h = (int)(A->shape[2] * scale), w = (int)(A->shape[3] * scale);
        const int y = (int)((A->shape[2] - h) * std::uniform_real_distribution<float>(0.f, 1.f)(g));
        const int x = (int)((A->shape[3] - w) * std::uniform_real_distribution<float>(0.f, 1.f)(g));
        boxes[4 * b] = y; boxes[4 * b + 1] = x; boxes[4 * b + 2] = y + h; boxes[4 * b + 3] = x + w;
    }
    ok(eddlb200_crop_scale_batch(dev_of(A), A->ptr, B->ptr, A->shape[0], A->shape[1], A->shape[2], A->shape[3], B->shape[2], B->shape[3], boxes.data()),
       "gpu_crop_scale_random");
}

// ---- activations ------------------------------------------------------------------------
void gpu_relu(Tensor *A, Tensor *B) {
    const int dev = A->gpu_device;
    PendingBN &p = g_pending[dev & 63];
    if (p.active && p.output == A->ptr && (size_t)p.b * p.z * p.rc == A->size && B->ptr != A->ptr) {
        launch_bn(dev, p, B->ptr);          // BN apply + ReLU in one pass
        return;
    }
    ok(eddlb200_relu_fwd(dev_of(A), A->ptr, B->ptr, A->size), "gpu_relu");
}
void gpu_d_relu(Tensor *D, Tensor *I, Tensor *PD) { ok(eddlb200_relu_bwd(dev_of(D), D->ptr, I->ptr, PD->ptr, D->size), "gpu_d_relu"); }

namespace {
void softmax_view(Tensor *A, int axis, int &outer, int &cols, int &inner) {
    if (axis < 0) axis += (int)A->ndim;
    cols = A->shape[axis];
    inner = A->stride[axis];
    outer = (int)(A->size / ((size_t)cols * inner));
}
}
void gpu_full_softmax(Tensor *A, Tensor *B, int axis, bool stable) {
    if (!stable) throw std::runtime_error("[eddl_b200] gpu_full_softmax: only the stable form is implemented");
    int outer, cols, inner; softmax_view(A, axis, outer, cols, inner);
    ok(eddlb200_softmax_fwd_nd(dev_of(A), A->ptr, B->ptr, outer, cols, inner), "gpu_full_softmax");
}
void gpu_d_full_softmax(Tensor *D, Tensor *I, Tensor *PD, int axis) {
    int outer, cols, inner; softmax_view(D, axis, outer, cols, inner);
    ok(eddlb200_softmax_bwd_nd(dev_of(D), D->ptr, I->ptr, PD->ptr, outer, cols, inner), "gpu_d_full_softmax");
}

// ---- losses / metrics ---------------------------------------------------------------------
float gpu_categorical_cross_entropy(Tensor *y_true, Tensor *y_pred) {
    float v = 0.f;
    ok(eddlb200_cce_value(dev_of(y_true), y_true->ptr, y_pred->ptr, y_true->shape[0], (int)(y_true->size / y_true->shape[0]), &v), "gpu_categorical_cross_entropy");
    return v;
}
void gpu_d_categorical_cross_entropy(Tensor *y_true, Tensor *y_pred, Tensor *delta) {
    ok(eddlb200_cce_delta(dev_of(y_true), y_true->ptr, y_pred->ptr, delta->ptr, y_true->size), "gpu_d_categorical_cross_entropy");
}
void gpu_accuracy(Tensor *A, Tensor *B, int *acc) {
    ok(eddlb200_accuracy(dev_of(A), A->ptr, B->ptr, A->shape[0], (int)(A->size / A->shape[0]), acc), "gpu_accuracy");
}

// ---- convolution ----------------------------------------------------------------------------
namespace {
int conv_precision() {
    static int v = -1;
    if (v < 0) { const char *e = getenv("EDDL_B200_CONV_PRECISION"); v = (e && (e[0] == 't' || e[0] == 'T' || e[0] == '1')) ? 1 : (e && (e[0] == 'b' || e[0] == 'B' || e[0] == '2')) ? 2 : 0; }
    return v;
}
}
void gpu_conv2D(ConvolDescriptor *D) {
    ok(eddlb200_conv2d_fwd(dev_of(D->I), D->I->ptr, D->K->ptr, D->use_bias ? D->bias->ptr : nullptr, D->O->ptr,
                           D->I->shape[0], D->iz, D->ir, D->ic, D->nk, D->kr, D->kc, D->r, D->c,
                           D->sr, D->sc, D->padrt, D->padcl, conv_precision()), "gpu_conv2D");
}
void gpu_conv2D_grad(ConvolDescriptor *D) {
    ok(eddlb200_conv2d_bwd_weight(dev_of(D->I), D->I->ptr, D->D->ptr, D->gK->ptr, D->use_bias ? D->gbias->ptr : nullptr,
                                  D->I->shape[0], D->iz, D->ir, D->ic, D->nk, D->kr, D->kc, D->r, D->c,
                                  D->sr, D->sc, D->padrt, D->padcl, conv_precision()), "gpu_conv2D_grad");
}
void gpu_conv2D_back(ConvolDescriptor *D) {
    ok(eddlb200_conv2d_bwd_data(dev_of(D->I), D->D->ptr, D->K->ptr, D->ID->ptr,
                                D->I->shape[0], D->iz, D->ir, D->ic, D->nk, D->kr, D->kc, D->r, D->c,
                                D->sr, D->sc, D->padrt, D->padcl, conv_precision()), "gpu_conv2D_back");
}

// ---- pooling ------------------------------------------------------------------------------
void gpu_mpool2D(PoolDescriptor *D) {
    ok(eddlb200_maxpool2d_fwd(dev_of(D->I), D->I->ptr, D->O->ptr, D->indX->ptr, D->indY->ptr,
                              D->I->shape[0], D->iz, D->ir, D->ic, D->r, D->c, D->kr, D->kc, D->sr, D->sc, D->padrt, D->padcl), "gpu_mpool2D");
}
void gpu_mpool2D_back(PoolDescriptor *D) {
    ok(eddlb200_maxpool2d_bwd(dev_of(D->I), D->D->ptr, D->indX->ptr, D->indY->ptr, D->ID->ptr,
                              D->I->shape[0], D->iz, D->ir, D->ic, D->r, D->c, D->kr, D->kc, D->sr, D->sc, D->padrt, D->padcl), "gpu_mpool2D_back");
}
void gpu_avgpool2D(PoolDescriptor *D) {
    ok(eddlb200_avgpool2d_fwd(dev_of(D->I), D->I->ptr, D->O->ptr,
                              D->I->shape[0], D->iz, D->ir, D->ic, D->r, D->c, D->kr, D->kc, D->sr, D->sc, D->padrt, D->padcl), "gpu_avgpool2D");
}
void gpu_avgpool2D_back(PoolDescriptor *D) {
    ok(eddlb200_avgpool2d_bwd(dev_of(D->I), D->D->ptr, D->ID->ptr,
                              D->I->shape[0], D->iz, D->ir, D->ic, D->r, D->c, D->kr, D->kc, D->sr, D->sc, D->padrt, D->padcl), "gpu_avgpool2D_back");
}

// ---- batch normalisation ----------------------------------------------------------------------
void gpu_batchnorm_forward(int gpu_device, int b, int z, int rc, float *input, float *output, float *opa,
                           float *global_mean, float *global_variance, float *affine_g, float *affine_b,
                           float *mean, float *variance, bool trmode, float epsilon, float momentum) {
    flush(gpu_device);
    PendingBN &p = g_pending[gpu_device & 63];
    p.b = b; p.z = z; p.rc = rc; p.input = input; p.output = output; p.opa = opa; p.gmean = global_mean; p.gvar = global_variance;
    p.g = affine_g; p.bb = affine_b; p.mean = mean; p.var = variance; p.trmode = trmode; p.eps = epsilon; p.momentum = momentum;
    if (fusion_enabled()) { p.active = true; return; }
    launch_bn(gpu_device, p, nullptr);
}
void gpu_batchnorm_backward(int gpu_device, int b, int z, int rc, float *delta, float *opa, float *pdelta, float *gbn_g, float *gbn_b,
                            float *bn_g, float *variance, float *mean1, float *mean2) {
    flush(gpu_device);
    ok(eddlb200_bn_bwd(gpu_device, b, z, rc, delta, opa, pdelta, gbn_g, gbn_b, bn_g, variance, mean1, mean2), "gpu_batchnorm_backward");
}

// Called by the harness / distributed API before it reads device memory behind the shim's back.
extern "C" void eddlb200_shim_flush(int dev) { flush(dev); }
