// init_distributed / broadcast_params_distributed / avg_weights_distributed and the fused SGD
// optimizer: host-side glue between EDDL's Net / Optimizer classes and the eddl_b200 C ABI.
#include <cstdlib>
#include <cstring>
#include <stdexcept>
#include <string>
#include <vector>
#include "eddl_b200/distributed.h"
#include "eddl_b200.h"

extern "C" void eddlb200_shim_flush(int dev);

namespace eddl_b200 {

namespace {
int g_rank = 0, g_nranks = 1, g_dev = -1;

void ok(int status, const char *where) {
    if (status != 0) throw std::runtime_error(std::string("[eddl_b200] ") + where + ": " + eddlb200_last_error());
}
int env_int(const char *name, int dflt) { const char *e = getenv(name); return e ? atoi(e) : dflt; }

// Device pointers and sizes of every parameter tensor of the replica that lives in this process.
void collect_params(Net *net, std::vector<float *> &ptrs, std::vector<size_t> &sizes, int &dev) {
    if (net->snets.empty()) throw std::runtime_error("[eddl_b200] the net is not built");
    Net *rep = net->snets[0];
    dev = -1;
    for (Layer *l : rep->layers)
        for (Tensor *t : l->params) {
            if (!t->isGPU()) throw std::runtime_error("[eddl_b200] distributed averaging needs a CS_GPU net");
            if (dev < 0) dev = t->gpu_device;
            ptrs.push_back(t->ptr); sizes.push_back(t->size);
        }
}
}  // namespace

int init_distributed(int rank, int nranks, int device, const void *id128) {
    ok(eddlb200_init(device), "init_distributed");
    if (nranks > 1) ok(eddlb200_comm_init_rank(device, nranks, rank, id128), "init_distributed");
    g_rank = rank; g_nranks = nranks; g_dev = device;
    return rank;
}

int init_distributed() {
    const int rank = env_int("RANK", 0), nranks = env_int("WORLD_SIZE", 1), dev = env_int("LOCAL_RANK", 0);
    unsigned char id[128] = {};
    if (nranks > 1) {
        const char *hex = getenv("EDDLB200_NCCL_ID");
        if (!hex || strlen(hex) != 256) throw std::runtime_error("[eddl_b200] init_distributed: EDDLB200_NCCL_ID must hold 256 hex characters");
        for (int i = 0; i < 128; i++) { unsigned v = 0; if (sscanf(hex + 2 * i, "%2x", &v) != 1) throw std::runtime_error("[eddl_b200] bad EDDLB200_NCCL_ID"); id[i] = (unsigned char)v; }
    }
    return init_distributed(rank, nranks, dev, id);
}

void end_distributed() { if (g_dev >= 0) eddlb200_comm_destroy(g_dev); g_nranks = 1; g_rank = 0; }
int get_rank_distributed() { return g_rank; }
int get_world_size_distributed() { return g_nranks; }

void broadcast_params_distributed(Net *net) {
    std::vector<float *> ptrs; std::vector<size_t> sizes; int dev;
    collect_params(net, ptrs, sizes, dev);
    eddlb200_shim_flush(dev);
    for (size_t i = 0; i < ptrs.size(); i++) ok(eddlb200_broadcast(dev, ptrs[i], sizes[i], 0), "broadcast_params_distributed");
}

void avg_weights_distributed(Net *net, int curr_batch, int batches_per_avg) {
    if (batches_per_avg <= 0 || curr_batch % batches_per_avg != 0) return;
    std::vector<float *> ptrs; std::vector<size_t> sizes; int dev;
    collect_params(net, ptrs, sizes, dev);
    eddlb200_shim_flush(dev);
    // layers come in forward order, so the buckets do too: the collective runs on its own stream and the next step's
    // forward pass waits bucket by bucket (EDDL_B200_AVG_ASYNC=0: one bucket on the compute stream)
    static const bool async = !(getenv("EDDL_B200_AVG_ASYNC") && getenv("EDDL_B200_AVG_ASYNC")[0] == '0');
    if (async) ok(eddlb200_allreduce_avg_multi_async(dev, ptrs.data(), sizes.data(), (int)ptrs.size(), 0), "avg_weights_distributed");
    else ok(eddlb200_allreduce_avg_multi(dev, ptrs.data(), sizes.data(), (int)ptrs.size()), "avg_weights_distributed");
}

void check_distributed(int wait_ms) {
    if (g_dev >= 0 && g_nranks > 1) ok(eddlb200_comm_check(g_dev, wait_ms), "check_distributed");
}

SGDFused::SGDFused(float lr, float momentum, float weight_decay, bool nesterov) : SGD(lr, momentum, weight_decay, nesterov) {}

Optimizer *SGDFused::clone() { SGDFused *n = new SGDFused(lr, mu, weight_decay, nesterov); n->clip_val = clip_val; n->average_gradients = average_gradients; return n; }
Optimizer *SGDFused::share() {
    SGDFused *n = new SGDFused(lr, mu, weight_decay, nesterov);
    n->orig = this; n->isshared = true; n->clip_val = clip_val; n->average_gradients = average_gradients;
    return n;
}

void SGDFused::applygrads(int batch) {
    if (isshared) { orig->applygrads(batch); return; }
    bool on_gpu = !layers.empty();
    for (Layer *l : layers) for (Tensor *t : l->params) if (!t->isGPU()) on_gpu = false;
    bool accumulates = false;
    for (Layer *l : layers) if (!l->acc_gradients.empty()) accumulates = true;
    if (!on_gpu || accumulates) { SGD::applygrads(batch); return; }
    clip();
    std::vector<float *> p, m; std::vector<const float *> g; std::vector<size_t> sizes;
    int dev = -1, q = 0;
    for (size_t i = 0; i < layers.size(); i++) {
        const int ntr = layers[i]->get_trainable_params_count();
        if (layers[i]->trainable)
            for (int j = 0; j < ntr; j++) {
                Tensor *pt = layers[i]->params[j];
                if (dev < 0) dev = pt->gpu_device;
                p.push_back(pt->ptr); g.push_back(layers[i]->gradients[j]->ptr); m.push_back(mT[q + j]->ptr); sizes.push_back(pt->size);
            }
        q += ntr;
    }
    if (p.empty()) return;
    eddlb200_shim_flush(dev);
    if (average_gradients && g_nranks > 1) {
        // gradient averaging: every rank applies the same averaged gradient, so parameters and momentum stay identical on
        // all ranks without averaging the weights afterwards
        std::vector<float *> gm(g.size());
        for (size_t i = 0; i < g.size(); i++) gm[i] = const_cast<float *>(g[i]);
        ok(eddlb200_allreduce_avg_multi(dev, gm.data(), sizes.data(), (int)gm.size()), "SGDFused::applygrads(average gradients)");
    }
    ok(eddlb200_sgd_momentum_multi(dev, p.data(), g.data(), m.data(), sizes.data(), (int)p.size(), lr, mu), "SGDFused::applygrads");
}

AdamFused::AdamFused(float lr, float beta_1, float beta_2, float epsilon, float weight_decay, bool amsgrad)
    : Adam(lr, beta_1, beta_2, epsilon, weight_decay, amsgrad) {}

Optimizer *AdamFused::clone() { AdamFused *n = new AdamFused(lr, beta_1, beta_2, epsilon, weight_decay, amsgrad); n->clip_val = clip_val; return n; }
Optimizer *AdamFused::share() {
    AdamFused *n = new AdamFused(lr, beta_1, beta_2, epsilon, weight_decay, amsgrad);
    n->orig = this; n->isshared = true; n->clip_val = clip_val;
    return n;
}

void AdamFused::applygrads(int batch) {
    if (isshared) { orig->applygrads(batch); return; }
    bool on_gpu = !layers.empty();
    for (Layer *l : layers) for (Tensor *t : l->params) if (!t->isGPU()) on_gpu = false;
    bool accumulates = false;
    for (Layer *l : layers) if (!l->acc_gradients.empty()) accumulates = true;
    if (!on_gpu || accumulates) { Adam::applygrads(batch); return; }
    clip();
    t++;
    std::vector<float *> p, g, m, v; std::vector<size_t> sizes;
    int dev = -1, q = 0;
    for (size_t i = 0; i < layers.size(); i++) {
        const int ntr = layers[i]->get_trainable_params_count();
        if (layers[i]->trainable)
            for (int j = 0; j < ntr; j++) {
                Tensor *pt = layers[i]->params[j];
                if (dev < 0) dev = pt->gpu_device;
                p.push_back(pt->ptr); g.push_back(layers[i]->gradients[j]->ptr); m.push_back(mT[q + j]->ptr); v.push_back(vT[q + j]->ptr);
                sizes.push_back(pt->size);
            }
        q += ntr;
    }
    if (p.empty()) return;
    eddlb200_shim_flush(dev);
    ok(eddlb200_adam_multi(dev, p.data(), g.data(), m.data(), v.data(), sizes.data(), (int)p.size(), lr, beta_1, beta_2, epsilon, t),
       "AdamFused::applygrads");
}

}  // namespace eddl_b200
