// TEST INFRASTRUCTURE ONLY (parity checker and timed CPU baseline; never part of the
// product path).  A C ABI over EDDL v1.1's OWN CPU implementation, compiled in place from the
// EDDL source tree (oracle/build_ref.py): each function wraps caller buffers in the
// reference's Tensor / descriptor objects and calls the reference's cpu_* function, nothing
// else.  Cited functions live under src/hardware/cpu/ of the EDDL tree.
#include <cstring>
#include <stdexcept>
#include <string>
#include <vector>

#include "eddl/tensor/tensor.h"
#include "eddl/tensor/nn/tensor_nn.h"
#include "eddl/descriptors/descriptors.h"
#include "eddl/hardware/cpu/cpu_tensor.h"
#include "eddl/hardware/cpu/nn/cpu_tensor_nn.h"

namespace {

thread_local std::string g_err;

template <typename F> int guarded(F f) {
    try { f(); return 0; }
    catch (const std::exception &e) { g_err = e.what(); return -1; }
    catch (...) { g_err = "unknown exception"; return -1; }
}

// Tensor that borrows caller memory.
struct View {
    Tensor *t;
    View(std::vector<int> shape, const float *p) { t = new Tensor(shape, const_cast<float *>(p), DEV_CPU); t->isshared = true; }
    ~View() { delete t; }
    Tensor *operator->() { return t; }
    operator Tensor *() { return t; }
};

struct ConvCase {
    ConvolDescriptor *cd; Tensor *I;
    ConvCase(const float *x, const float *w, const float *bias, int n, int c, int ih, int iw, int k, int kr, int kc,
             int sr, int sc, int pt, int pb, int pl, int pr) {
        cd = new ConvolDescriptor(k, {kr, kc}, {sr, sc}, "custom", {pt, pb, pl, pr}, 1, {1, 1}, bias != nullptr, 0);
        I = new Tensor({n, c, ih, iw}, DEV_CPU);
        memcpy(I->ptr, x, I->size * sizeof(float));
        cd->build(I);
        memcpy(cd->K->ptr, w, cd->K->size * sizeof(float));
        if (bias) memcpy(cd->bias->ptr, bias, k * sizeof(float)); else cd->bias->fill_(0.f);
        cd->gK->fill_(0.f); cd->gbias->fill_(0.f);
    }
    ~ConvCase() { delete cd->O; delete cd->K; delete cd->bias; delete cd->gK; delete cd->gbias; delete cd; delete I; }
};

struct PoolCase {
    PoolDescriptor *pd; Tensor *I;
    PoolCase(const float *x, int n, int c, int ih, int iw, int kr, int kc, int sr, int sc, int pt, int pb, int pl, int pr) {
        pd = new PoolDescriptor({kr, kc}, {sr, sc}, std::vector<int>{pt, pb, pl, pr}, 0);
        I = new Tensor({n, c, ih, iw}, DEV_CPU);
        memcpy(I->ptr, x, I->size * sizeof(float));
        pd->build(I);
        pd->indX = new Tensor(pd->O->shape, DEV_CPU); pd->indY = new Tensor(pd->O->shape, DEV_CPU);
        pd->indX->fill_(0.f); pd->indY->fill_(0.f);
    }
    ~PoolCase() { delete pd->O; delete pd; delete I; }
};

}  // namespace

// defined in src/hardware/cpu/cpu_da.cpp, not declared in a public header
void cpu_single_flip(int b, bool apply, Tensor *A, Tensor *B, int axis);
void cpu_single_crop_scale(int b, Tensor *A, Tensor *B, vector<int> coords_from, vector<int> coords_to, int wrapping_mode, float constant);

extern "C" {

const char *ref_last_error() { return g_err.c_str(); }

// ---- Conv2D: cpu_conv2D / cpu_conv2D_grad / cpu_conv2D_back (nn/cpu_conv.cpp:316-527) ----------
int ref_conv2d_out_shape(int ih, int iw, int kr, int kc, int sr, int sc, int pt, int pb, int pl, int pr, int *oh, int *ow) {
    return guarded([&] {
        *oh = ConvolDescriptor::compute_output(std::vector<int>{pt, pb}, ih, kr, sr, 1);
        *ow = ConvolDescriptor::compute_output(std::vector<int>{pl, pr}, iw, kc, sc, 1);
    });
}

// y: [n,k,oh,ow] out.  dy (optional): runs backward too; gw [k,c,kr,kc] and gbias [k] are IN/OUT
// (accumulated into), dx [n,c,ih,iw] is IN/OUT (accumulated into).
int ref_conv2d(const float *x, const float *w, const float *bias, float *y, const float *dy, float *gw, float *gbias, float *dx,
               int n, int c, int ih, int iw, int k, int kr, int kc, int sr, int sc, int pt, int pb, int pl, int pr) {
    return guarded([&] {
        ConvCase cc(x, w, bias, n, c, ih, iw, k, kr, kc, sr, sc, pt, pb, pl, pr);
        cpu_conv2D(cc.cd);
        if (y) memcpy(y, cc.cd->O->ptr, cc.cd->O->size * sizeof(float));
        if (dy) {
            Tensor *D = new Tensor(cc.cd->O->shape, DEV_CPU);
            memcpy(D->ptr, dy, D->size * sizeof(float));
            cc.cd->D = D;
            if (gw) {
                memcpy(cc.cd->gK->ptr, gw, cc.cd->gK->size * sizeof(float));
                if (gbias) memcpy(cc.cd->gbias->ptr, gbias, k * sizeof(float));
                cpu_conv2D_grad(cc.cd);
                memcpy(gw, cc.cd->gK->ptr, cc.cd->gK->size * sizeof(float));
                if (gbias) memcpy(gbias, cc.cd->gbias->ptr, k * sizeof(float));
            }
            if (dx) {
                Tensor *ID = new Tensor({n, c, ih, iw}, DEV_CPU);
                memcpy(ID->ptr, dx, ID->size * sizeof(float));
                cc.cd->ID = ID;
                cpu_conv2D_back(cc.cd);
                memcpy(dx, ID->ptr, ID->size * sizeof(float));
                delete ID;
            }
            delete D;
        }
    });
}

// ---- pooling: cpu_mpool2D(_back), cpu_avgpool2D(_back) (nn/cpu_pool.cpp:74-145,226-304) ----------
int ref_pool2d(int is_max, const float *x, float *y, float *ind_x, float *ind_y, const float *dy, float *dx,
               int n, int c, int ih, int iw, int kr, int kc, int sr, int sc, int pt, int pb, int pl, int pr, int *oh, int *ow) {
    return guarded([&] {
        PoolCase pc(x, n, c, ih, iw, kr, kc, sr, sc, pt, pb, pl, pr);
        if (oh) *oh = pc.pd->r; if (ow) *ow = pc.pd->c;
        if (!y) return;
        if (is_max) cpu_mpool2D(pc.pd); else cpu_avgpool2D(pc.pd);
        memcpy(y, pc.pd->O->ptr, pc.pd->O->size * sizeof(float));
        if (is_max && ind_x) memcpy(ind_x, pc.pd->indX->ptr, pc.pd->O->size * sizeof(float));
        if (is_max && ind_y) memcpy(ind_y, pc.pd->indY->ptr, pc.pd->O->size * sizeof(float));
        if (dy && dx) {
            Tensor *D = new Tensor(pc.pd->O->shape, DEV_CPU); memcpy(D->ptr, dy, D->size * sizeof(float));
            Tensor *ID = new Tensor({n, c, ih, iw}, DEV_CPU); memcpy(ID->ptr, dx, ID->size * sizeof(float));
            pc.pd->D = D; pc.pd->ID = ID;
            if (is_max) cpu_mpool2D_back(pc.pd); else cpu_avgpool2D_back(pc.pd);
            memcpy(dx, ID->ptr, ID->size * sizeof(float));
            delete D; delete ID;
        }
    });
}

// ---- batch norm: cpu_batchnorm_forward / backward (nn/cpu_bn.cpp:118-249), raw-pointer API -------
int ref_bn_fwd(int b, int z, int rc, float *input, float *output, float *opa, float *global_mean, float *global_variance,
               float *affine_g, float *affine_b, float *mean, float *variance, int trmode, float epsilon, float momentum) {
    return guarded([&] { cpu_batchnorm_forward(b, z, rc, input, output, opa, global_mean, global_variance, affine_g, affine_b, mean, variance, trmode != 0, epsilon, momentum); });
}
int ref_bn_bwd(int b, int z, int rc, float *delta, float *opa, float *pdelta, float *gbn_g, float *gbn_b, float *bn_g,
               float *variance, float *mean1, float *mean2) {
    return guarded([&] { cpu_batchnorm_backward(b, z, rc, delta, opa, pdelta, gbn_g, gbn_b, bn_g, variance, mean1, mean2); });
}

// ---- activations (nn/cpu_activations.cpp:20-45,329-436) -------------------------------------------
int ref_relu(const float *a, float *b, long long n) { return guarded([&] { View A({(int)n}, a), B({(int)n}, b); cpu_relu(A, B); }); }
int ref_d_relu(const float *d, const float *i, float *pd, long long n) { return guarded([&] { View D({(int)n}, d), I({(int)n}, i), PD({(int)n}, pd); cpu_d_relu(D, I, PD); }); }
int ref_softmax(const float *a, float *b, int rows, int cols) { return guarded([&] { View A({rows, cols}, a), B({rows, cols}, b); cpu_full_softmax(A, B, 1, true); }); }
int ref_d_softmax(const float *d, const float *s, float *pd, int rows, int cols) {
    return guarded([&] { View D({rows, cols}, d), S({rows, cols}, s), PD({rows, cols}, pd); cpu_d_full_softmax(D, S, PD, 1); });
}

// ---- losses / metrics (nn/cpu_losses.cpp:29-57, nn/cpu_metrics.cpp:17-29) ---------------------------
int ref_cce(const float *y, const float *p, int rows, int cols, float *value, float *delta) {
    return guarded([&] {
        View Y({rows, cols}, y), P({rows, cols}, p);
        if (value) *value = cpu_categorical_cross_entropy(Y, P);
        if (delta) { View Dl({rows, cols}, delta); cpu_d_categorical_cross_entropy(Y, P, Dl); }
    });
}
int ref_accuracy(const float *y, const float *p, int rows, int cols, int *acc) {
    return guarded([&] { View Y({rows, cols}, y), P({rows, cols}, p); *acc = cpu_accuracy(Y, P); });
}

// ---- elementwise / dense (cpu_math.cpp:278-325,369-380; cpu_reduction.cpp:91-112; cpu_da.cpp:502-534)
int ref_axpby(float sca, const float *a, float scb, const float *b, float *c, int inc_c, long long n) {
    return guarded([&] { View A({(int)n}, a), B({(int)n}, b), C({(int)n}, c); cpu_add(sca, A, scb, B, C, inc_c); });
}
int ref_mult2d(const float *a, int ta, const float *b, int tb, float *c, int inc_c, int m, int n, int k) {
    return guarded([&] {
        View A(ta ? std::vector<int>{k, m} : std::vector<int>{m, k}, a), B(tb ? std::vector<int>{n, k} : std::vector<int>{k, n}, b), C({m, n}, c);
        cpu_mult2D(A, ta, B, tb, C, inc_c);
    });
}
int ref_sum2d_rowwise(const float *a, const float *b, float *c, int rows, int cols) {
    return guarded([&] { View A({rows, cols}, a), B({cols}, b), C({rows, cols}, c); cpu_sum2D_rowwise(A, B, C); });
}
int ref_reduce_sum2d(const float *a, float *b, int rows, int cols, int axis, int inc_b) {
    return guarded([&] { View A({rows, cols}, a), B({axis == 0 ? cols : rows}, b); cpu_reduce_sum2D(A, B, axis, inc_b); });
}
int ref_pad(const float *a, float *b, float *a_delta, const float *b_delta, int n, int c, int h, int w, int top, int right, int bottom, int left) {
    return guarded([&] {
        std::vector<int> pads{top, right, bottom, left};
        if (a && b) { View A({n, c, h, w}, a), B({n, c, h + top + bottom, w + left + right}, b); cpu_pad(A, B, pads); }
        if (a_delta && b_delta) { View A({n, c, h, w}, a_delta), B({n, c, h + top + bottom, w + left + right}, b_delta); cpu_pad_back(A, B, pads); }
    });
}

// ---- optimizer steps: the reference's own chains of Tensor operations ------------------------------
// SGD::applygrads body (src/optimizers/optim_sgd.cpp:78-79)
int ref_sgd_step(float *p, const float *g, float *m, float lr, float mu, long long n) {
    return guarded([&] {
        View P({(int)n}, p), G({(int)n}, g), M({(int)n}, m);
        Tensor::add(lr, G, mu, M, M, 0);
        Tensor::add(1.0, P, -1.0, M, P, 0);
    });
}
// Adam::applygrads body (src/optimizers/optim_adam.cpp:96-110); t is the step count AFTER t++
int ref_adam_step(float *p, float *g, float *m, float *v, float lr, float beta_1, float beta_2, float epsilon, int t, long long n) {
    return guarded([&] {
        View P({(int)n}, p), G({(int)n}, g), M({(int)n}, m), V({(int)n}, v);
        Tensor *mCap = new Tensor({(int)n}), *vCap = new Tensor({(int)n});
        Tensor::add(beta_1, M, (1 - beta_1), G, M, 0);
        G->sqr_();
        Tensor::add(beta_2, V, (1 - beta_2), G, V, 0);
        Tensor::copy(M, mCap);
        mCap->div_(1 - pow(beta_1, t));
        Tensor::copy(V, vCap);
        vCap->div_(1 - pow(beta_2, t));
        vCap->add_(epsilon);
        vCap->sqrt_();
        Tensor::el_div(mCap, vCap, mCap, 0);
        Tensor::add(-lr, mCap, 1.0, P, P, 0);
        delete mCap; delete vCap;
    });
}
// Net::sync_weights arithmetic (src/net/net_func.cpp:111-127) over `nrep` replica buffers of n floats
// laid out back to back in `reps`; the average is written to out.
int ref_sync_weights(const float *reps, int nrep, float *out, long long n) {
    return guarded([&] {
        View acc({(int)n}, out);
        acc->fill_(0.0);
        for (int r = 0; r < nrep; r++) { View w({(int)n}, reps + (size_t)r * n); Tensor::inc(w, acc); }
        acc->div_(nrep);
    });
}

// Concat of two tensors along axis 1 and its backward (cpu_concat, src/hardware/cpu/cpu_core.cpp:368-396); UpSampling
// (cpu_repeat_nn / cpu_d_repeat_nn, nn/cpu_tensor_nn.cpp:13-50); one image's flip and crop-scale (cpu_da.cpp:315-336, 363-384).
int ref_concat2(float *a, float *p0, float *p1, int n, int c0, int c1, int h, int w, int derivative) {
    return guarded([&] { View A({n, c0 + c1, h, w}, a), P0({n, c0, h, w}, p0), P1({n, c1, h, w}, p1); cpu_concat(A, {P0.t, P1.t}, 1, derivative != 0); });
}
int ref_repeat_nn(const float *a, float *b, float *a_delta, const float *b_delta, int n, int c, int h, int w, int sr, int sc) {
    return guarded([&] {
        View A({n, c, h, w}, a), B({n, c, h * sr, w * sc}, b);
        cpu_repeat_nn(A, B, {sr, sc});
        if (a_delta) { View AD({n, c, h, w}, a_delta), BD({n, c, h * sr, w * sc}, b_delta); cpu_d_repeat_nn(BD, AD, {sr, sc}); }
    });
}
// Tensor::scale / scale_back (cpu_scale, cpu_scale_back: src/hardware/cpu/cpu_da.cpp:407-459)
int ref_scale(const float *a, float *b, float *a_delta, const float *b_delta, int n, int c, int ah, int aw, int bh, int bw, int nh, int nw,
              int wrap, float cval, int mode) {
    return guarded([&] {
        View A({n, c, ah, aw}, a), B({n, c, bh, bw}, b);
        cpu_scale(A, B, {nh, nw}, wrap, cval, mode);
        if (a_delta) { View AD({n, c, ah, aw}, a_delta), BD({n, c, bh, bw}, b_delta); cpu_scale_back(AD, BD, {nh, nw}, wrap, cval, mode); }
    });
}
int ref_flip_batch(const float *a, float *b, int n, int c, int h, int w, int axis, const unsigned char *apply) {
    return guarded([&] { View A({n, c, h, w}, a), B({n, c, h, w}, b); for (int i = 0; i < n; i++) cpu_single_flip(i, apply[i] != 0, A, B, axis); });
}
int ref_crop_scale_batch(const float *a, float *b, int n, int c, int ah, int aw, int bh, int bw, const int *boxes) {
    return guarded([&] {
        View A({n, c, ah, aw}, a), B({n, c, bh, bw}, b);
        for (int i = 0; i < n; i++) cpu_single_crop_scale(i, A, B, {boxes[4 * i], boxes[4 * i + 1]}, {boxes[4 * i + 2], boxes[4 * i + 3]}, 0, 0.f);
    });
}

}  // extern "C"

// OpenMP team size used by the reference's cpu_* loops (omp_set_num_threads).  Parity runs use 1: the
// reference's BatchNorm reductions accumulate per-channel sums from a parallel loop without atomics
// (src/hardware/cpu/nn/cpu_bn.cpp:130-141, 193-205), so their results are only reproducible single-threaded.
#include <omp.h>
extern "C" int ref_set_omp_threads(int n) { omp_set_num_threads(n > 0 ? n : omp_get_num_procs()); return 0; }
