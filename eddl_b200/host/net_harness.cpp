// Net harness: builds the benchmark convnets through EDDL's own public API (eddl::Input,
// Conv, BatchNormalization, ReLu, MaxPool, Pad, Add, Dense, Softmax, build, train_batch ...)
// and exposes them to Python / C callers through a small C ABI.  The same file is compiled
// twice: against EDDL's host sources built WITHOUT -DcGPU (CS_CPU: the reference's own CPU
// implementation, used as the parity checker and the timed CPU baseline) and WITH -DcGPU on top
// of the eddl_b200 backend (CS_GPU).  Weights, inputs and labels are injected by the caller,
// because EDDL's initialisers ignore their seed (src/initializers/initializer_glorot_uniform.cpp:
// 29-32; src/random.cpp:25-26).
//
// Architectures (templates: examples/nn/1_mnist/7_mnist_conv.cpp, examples/nn/2_cifar10/
// 4_cifar_vgg16_bn.cpp, examples/nn/2_cifar10/7_cifar_resnet50_da_bn.cpp):
//   "cnn"      3 x [Conv3x3 same (16,32,64) -> ReLU -> MaxPool2x2] -> Dense 10 -> Softmax, input 1x28x28
//   "vgg16bn"  13 x [Conv3x3 same, no bias -> BN -> ReLU], 5 MaxPool2x2, Dense512-ReLU-Dense10-Softmax, 3x32x32
//   "resnet50" bottleneck [3,4,6,3], stride on the 3x3, explicit Pad layers wherever "same" padding
//              would be asymmetric (LConv / LMaxPool reject it: src/layers/conv/layer_conv2D.cpp:56-61)
#include <chrono>
#include <cstring>
#include <map>
#include <stdexcept>
#include <string>
#include <vector>

#include "eddl/apis/eddl.h"
#ifdef cGPU
#include "eddl_b200/distributed.h"
#include "eddl_b200.h"
extern "C" void eddlb200_shim_flush(int dev);
#endif

using namespace eddl;

namespace {

struct Handle {
    model net = nullptr;
    int in_c = 0, in_h = 0, in_w = 0, classes = 0;
    bool gpu = false;
    int dev = 0;
    std::vector<Tensor *> flat;      // every parameter tensor of the master net, in layer order
    Tensor *x = nullptr, *y = nullptr; int xy_batch = 0;
};

thread_local std::string g_err;
std::map<int, Handle *> g_handles;
int g_next = 1;

layer conv_bn_relu(layer l, int f, std::vector<int> k, std::vector<int> s, const std::string &pad, bool relu = true) {
    l = BatchNormalization(Conv(l, f, k, s, pad, false));
    return relu ? ReLu(l) : l;
}

layer bottleneck(layer l, int filters, bool half, bool expand) {
    layer in = l;
    l = conv_bn_relu(l, filters, {1, 1}, {1, 1}, "same");
    if (half) l = conv_bn_relu(Pad(l, {1, 1, 1, 1}), filters, {3, 3}, {2, 2}, "valid");
    else l = conv_bn_relu(l, filters, {3, 3}, {1, 1}, "same");
    l = conv_bn_relu(l, 4 * filters, {1, 1}, {1, 1}, "same", false);
    if (half) return ReLu(Add({conv_bn_relu(in, 4 * filters, {1, 1}, {2, 2}, "valid", false), l}));
    if (expand) return ReLu(Add({conv_bn_relu(in, 4 * filters, {1, 1}, {1, 1}, "same", false), l}));
    return ReLu(Add({in, l}));
}

model make_net(const std::string &cfg, Handle *h, int hw, int classes) {
    layer in, l;
    if (cfg == "cnn") {
        h->in_c = 1; h->in_h = h->in_w = hw > 0 ? hw : 28; h->classes = classes > 0 ? classes : 10;
        in = Input({h->in_c, h->in_h, h->in_w}); l = in;
        for (int f : {16, 32, 64}) l = MaxPool(ReLu(Conv(l, f, {3, 3}, {1, 1}, "same")), {2, 2}, {2, 2});
        l = Reshape(l, {-1});
        return Model({in}, {Softmax(Dense(l, h->classes))});
    }
    if (cfg == "vgg16bn") {
        h->in_c = 3; h->in_h = h->in_w = hw > 0 ? hw : 32; h->classes = classes > 0 ? classes : 10;
        in = Input({h->in_c, h->in_h, h->in_w}); l = in;
        const int plan[] = {64, 64, -1, 128, 128, -1, 256, 256, 256, -1, 512, 512, 512, -1, 512, 512, 512, -1};
        for (int f : plan) l = f < 0 ? MaxPool(l, {2, 2}, {2, 2}) : conv_bn_relu(l, f, {3, 3}, {1, 1}, "same");
        l = Reshape(l, {-1});
        l = ReLu(Dense(l, 512));
        return Model({in}, {Softmax(Dense(l, h->classes))});
    }
    if (cfg == "resnet50") {
        h->in_c = 3; h->in_h = h->in_w = hw > 0 ? hw : 224; h->classes = classes > 0 ? classes : 1000;
        if (h->in_h % 32) throw std::runtime_error("resnet50 input size must be a multiple of 32");
        in = Input({h->in_c, h->in_h, h->in_w}); l = in;
        l = conv_bn_relu(Pad(l, {3, 3, 3, 3}), 64, {7, 7}, {2, 2}, "valid");
        l = MaxPool(Pad(l, {1, 1, 1, 1}), {3, 3}, {2, 2}, "valid");
        for (int i = 0; i < 3; i++) l = bottleneck(l, 64, false, i == 0);
        for (int i = 0; i < 4; i++) l = bottleneck(l, 128, i == 0, false);
        for (int i = 0; i < 6; i++) l = bottleneck(l, 256, i == 0, false);
        for (int i = 0; i < 3; i++) l = bottleneck(l, 512, i == 0, false);
        const int last = h->in_h / 32;
        l = AveragePool(l, {last, last}, {1, 1}, "none");
        l = Reshape(l, {-1});
        return Model({in}, {Softmax(Dense(l, h->classes))});
    }
    if (cfg == "cifar_da") {
        // the layers EDDL's CIFAR-10 examples add around their conv stacks (examples/nn/2_cifar10/*_da*.cpp): random
        // crop-scale and flip on the input, Concat, UpSampling, GlobalMaxPool, Dropout
        h->in_c = 3; h->in_h = h->in_w = hw > 0 ? hw : 32; h->classes = classes > 0 ? classes : 10;
        in = Input({h->in_c, h->in_h, h->in_w});
        l = RandomHorizontalFlip(RandomCropScale(in, {0.8f, 1.0f}));
        l = MaxPool(conv_bn_relu(l, 32, {3, 3}, {1, 1}, "same"), {2, 2}, {2, 2});
        layer a = conv_bn_relu(l, 16, {1, 1}, {1, 1}, "same"), b = conv_bn_relu(l, 48, {3, 3}, {1, 1}, "same");
        l = Concat({a, b});
        l = MaxPool(UpSampling(l, {2, 2}), {2, 2}, {2, 2});
        l = conv_bn_relu(l, 64, {3, 3}, {1, 1}, "same");
        l = Reshape(GlobalMaxPool(l), {-1});
        l = Dropout(l, 0.25f);
        return Model({in}, {Softmax(Dense(l, h->classes))});
    }
    throw std::runtime_error("unknown net config '" + cfg + "'");
}

Handle *get(int id) {
    auto it = g_handles.find(id);
    if (it == g_handles.end()) throw std::runtime_error("bad net handle");
    return it->second;
}

void ensure_xy(Handle *h, int batch) {
    if (h->x && h->xy_batch == batch) return;
    delete h->x; delete h->y;
    h->x = new Tensor({batch, h->in_c, h->in_h, h->in_w});
    h->y = new Tensor({batch, h->classes});
    h->xy_batch = batch;
}

template <typename F> int guarded(F f) {
    try { f(); return 0; }
    catch (const std::exception &e) { g_err = e.what(); return -1; }
    catch (...) { g_err = "unknown exception"; return -1; }
}

}  // namespace

extern "C" {

const char *ebh_last_error() { return g_err.c_str(); }

// device < 0: CS_CPU(threads) ; device >= 0: CS_GPU with that single device (needs the -DcGPU build).
// optimizer: "sgd" / "adam" (the reference's classes) or "sgd_fused" / "adam_fused" (eddl_b200::SGDFused / AdamFused, GPU build only).
// loss: "categorical_cross_entropy" | "softmax_cross_entropy".
int ebh_create(const char *config, int hw, int classes, int device, int threads, const char *optimizer,
               float lr, float mu, const char *loss, int *out_handle) {
    return guarded([&] {
        Handle *h = new Handle();
        h->net = make_net(config, h, hw, classes);
        Optimizer *opt = nullptr;
        const std::string o = optimizer ? optimizer : "sgd";
        if (o == "sgd") opt = sgd(lr, mu);
        else if (o == "adam") opt = adam(lr);
#ifdef cGPU
        else if (o == "sgd_fused") opt = new eddl_b200::SGDFused(lr, mu);
        else if (o == "sgd_fused_gradavg") { auto *s = new eddl_b200::SGDFused(lr, mu); s->average_gradients = true; opt = s; }
        else if (o == "adam_fused") opt = new eddl_b200::AdamFused(lr, 0.9f, 0.999f, 0.000001f);      // eddl::adam's defaults
#endif
        else throw std::runtime_error("unknown optimizer '" + o + "'");
        CompServ *cs = nullptr;
        if (device >= 0) {
#ifdef cGPU
            std::vector<int> mask(device + 1, 0); mask[device] = 1;
            cs = CS_GPU(mask, 1, "full_mem");
            h->gpu = true; h->dev = device;
#else
            throw std::runtime_error("this build of the harness has no GPU backend");
#endif
        } else {
            cs = CS_CPU(threads);
        }
        build(h->net, opt, {loss ? loss : "categorical_cross_entropy"}, {"categorical_accuracy"}, cs, true);
        for (Layer *l : h->net->layers) for (Tensor *t : l->params) h->flat.push_back(t);
        *out_handle = g_next; g_handles[g_next++] = h;
    });
}

int ebh_destroy(int id) {
    return guarded([&] { Handle *h = get(id); g_handles.erase(id); delete h->x; delete h->y; delete h->net; delete h; });
}

int ebh_num_params(int id, int *ntensors, long long *nfloats) {
    return guarded([&] {
        Handle *h = get(id); long long n = 0;
        for (Tensor *t : h->flat) n += (long long)t->size;
        *ntensors = (int)h->flat.size(); *nfloats = n;
    });
}

// shape4 receives up to 4 extents (unused ones 0); name (>= 64 bytes) the owning layer's name
int ebh_param_info(int id, int index, int *ndim, int *shape4, char *name) {
    return guarded([&] {
        Handle *h = get(id); int q = 0;
        for (Layer *l : h->net->layers) for (Tensor *t : l->params) {
            if (q++ != index) continue;
            *ndim = (int)t->ndim;
            for (int d = 0; d < 4; d++) shape4[d] = d < (int)t->ndim ? t->shape[d] : 0;
            strncpy(name, l->name.c_str(), 63); name[63] = 0;
            return;
        }
        throw std::runtime_error("param index out of range");
    });
}

int ebh_set_params(int id, const float *flat) {
    return guarded([&] {
        Handle *h = get(id);
        std::vector<vtensor> all; std::vector<Tensor *> owned; const float *p = flat;
        for (Layer *l : h->net->layers) {
            vtensor lp;
            for (Tensor *t : l->params) {
                Tensor *n = new Tensor(t->getShape());
                memcpy(n->ptr, p, t->size * sizeof(float)); p += t->size;
                lp.push_back(n); owned.push_back(n);
            }
            all.push_back(lp);
        }
        set_parameters(h->net, all);
        for (Tensor *t : owned) delete t;
    });
}

int ebh_get_params(int id, float *flat) {
    return guarded([&] {
        Handle *h = get(id);
        std::vector<vtensor> all = get_parameters(h->net, false);   // collects device copies into the master net
        float *p = flat;
        for (auto &lp : all) for (Tensor *t : lp) { memcpy(p, t->ptr, t->size * sizeof(float)); p += t->size; }
    });
}

// One eddl::train_batch on host buffers x [batch, c, h, w], y one-hot [batch, classes].
// loss = mean per-sample loss of this batch as eddl::get_losses reports it, acc likewise.
int ebh_train_batch(int id, const float *x, const float *y, int batch, float *loss, float *acc) {
    return guarded([&] {
        Handle *h = get(id);
        ensure_xy(h, batch);
        memcpy(h->x->ptr, x, h->x->size * sizeof(float));
        memcpy(h->y->ptr, y, h->y->size * sizeof(float));
        reset_loss(h->net);
        train_batch(h->net, {h->x}, {h->y});
        if (loss) *loss = get_losses(h->net)[0];
        if (acc) *acc = get_metrics(h->net)[0];
    });
}

// Same as ebh_train_batch but the caller's buffers ARE the tensors EDDL reads (no staging copy):
// x/y must stay valid during the call.
int ebh_train_batch_nocopy(int id, float *x, float *y, int batch, float *loss, float *acc) {
    return guarded([&] {
        Handle *h = get(id);
        Tensor tx({batch, h->in_c, h->in_h, h->in_w}, x, DEV_CPU), ty({batch, h->classes}, y, DEV_CPU);
        tx.isshared = true; ty.isshared = true;     // EDDL must not free the caller's memory
        reset_loss(h->net);
        train_batch(h->net, {&tx}, {&ty});
        if (loss) *loss = get_losses(h->net)[0];
        if (acc) *acc = get_metrics(h->net)[0];
    });
}

// One training step through the fine-grained API instead of train_batch (src/net/net_api.cpp:266-298, 384-433, 762-783):
// zeroGrads, forward, backward(target), update.  Reports the same loss / metric figures as ebh_train_batch.
int ebh_train_fine(int id, const float *x, const float *y, int batch, float *loss, float *acc) {
    return guarded([&] {
        Handle *h = get(id);
        ensure_xy(h, batch);
        memcpy(h->x->ptr, x, h->x->size * sizeof(float));
        memcpy(h->y->ptr, y, h->y->size * sizeof(float));
        reset_loss(h->net);
        set_mode(h->net, TRMODE);
        zeroGrads(h->net);
        forward(h->net, std::vector<Tensor *>{h->x});
        backward(h->net, std::vector<Tensor *>{h->y});
        update(h->net);
        if (loss) *loss = get_losses(h->net)[0];
        if (acc) *acc = get_metrics(h->net)[0];
    });
}

// Net::save / Net::load (src/net/net.cpp:411-449), "bin" format.
int ebh_save(int id, const char *path) { return guarded([&] { save(get(id)->net, path, "bin"); }); }
int ebh_load(int id, const char *path) { return guarded([&] { load(get(id)->net, path, "bin"); }); }

// `steps` training steps on the batch already resident in the replica (set by the last
// ebh_train_batch): the body of train_batch_t (src/net/net_api.cpp:39-53) without the
// host->device copy of inputs.  Returns the last step's summed loss.
int ebh_train_resident(int id, int steps, float *loss_sum) {
    return guarded([&] {
        Handle *h = get(id);
        Net *rep = h->net->snets[0];
        for (int s = 0; s < steps; s++) {
            rep->do_reset(); rep->do_reset_grads(); rep->do_forward(); rep->do_compute_loss();
            rep->do_delta(); rep->do_backward(); rep->do_applygrads();
#ifdef cGPU
            if (eddl_b200::get_world_size_distributed() > 1) eddl_b200::avg_weights_distributed(h->net, 1, 1);
#endif
        }
        if (loss_sum) *loss_sum = rep->fiterr[0];
    });
}

// One step of the body of train_batch_t on the resident batch WITHOUT the cross-rank averaging that
// ebh_train_resident applies: afterwards the replicas of different ranks differ (used to check the averaging).
int ebh_local_step(int id) {
    return guarded([&] {
        Net *rep = get(id)->net->snets[0];
        rep->do_reset(); rep->do_reset_grads(); rep->do_forward(); rep->do_compute_loss();
        rep->do_delta(); rep->do_backward(); rep->do_applygrads();
    });
}

// Forward only (inference mode off: training-mode batch statistics), copies the net output to out.
int ebh_forward(int id, const float *x, int batch, float *out) {
    return guarded([&] {
        Handle *h = get(id);
        ensure_xy(h, batch);
        memcpy(h->x->ptr, x, h->x->size * sizeof(float));
        set_mode(h->net, TRMODE);
        forward(h->net, std::vector<Tensor *>{h->x});
        Tensor *o = getOutput(getOut(h->net)[0]);
        memcpy(out, o->ptr, o->size * sizeof(float));
        delete o;
    });
}

// Copies the output tensor / delta / first gradient of layer `layer_index` of the replica to host.
// what: 0 output, 1 delta, 2 gradient[0], 3 gradient[1]
int ebh_layer_tensor(int id, int layer_index, int what, float *out, long long capacity, long long *size) {
    return guarded([&] {
        Handle *h = get(id);
        Net *rep = h->net->snets[0];
        if (layer_index < 0 || layer_index >= (int)rep->layers.size()) throw std::runtime_error("layer index out of range");
        Layer *l = rep->layers[layer_index];
        Tensor *t = what == 0 ? l->output : what == 1 ? l->delta : (what - 2 < (int)l->gradients.size() ? l->gradients[what - 2] : nullptr);
        if (!t) throw std::runtime_error("tensor not available");
        *size = (long long)t->size;
        if (!out) return;
        if ((long long)t->size > capacity) throw std::runtime_error("buffer too small");
        Tensor host(t->getShape(), out, DEV_CPU); host.isshared = true;
        Tensor::copy(t, &host);
    });
}

int ebh_num_layers(int id, int *n) { return guarded([&] { *n = (int)get(id)->net->layers.size(); }); }
int ebh_layer_name(int id, int layer_index, char *name) {
    return guarded([&] { Handle *h = get(id); strncpy(name, h->net->layers.at(layer_index)->name.c_str(), 63); name[63] = 0; });
}

#ifdef cGPU
int ebh_init_distributed(int rank, int nranks, int device, const void *id128) {
    return guarded([&] { eddl_b200::init_distributed(rank, nranks, device, id128); });
}
int ebh_end_distributed() { return guarded([&] { eddl_b200::end_distributed(); }); }
int ebh_broadcast_params(int id) { return guarded([&] { eddl_b200::broadcast_params_distributed(get(id)->net); }); }
int ebh_avg_weights(int id, int curr_batch, int batches_per_avg) {
    return guarded([&] { eddl_b200::avg_weights_distributed(get(id)->net, curr_batch, batches_per_avg); });
}
int ebh_check_distributed(int wait_ms) { return guarded([&] { eddl_b200::check_distributed(wait_ms); }); }
int ebh_sync(int id) { return guarded([&] { Handle *h = get(id); eddlb200_shim_flush(h->dev); if (eddlb200_sync(h->dev)) throw std::runtime_error(eddlb200_last_error()); }); }
#endif

}  // extern "C"
