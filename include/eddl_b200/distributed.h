// Distributed data-parallel entry points and fused optimizer for EDDL nets running on the
// eddl_b200 backend.  EDDL v1.1 has no init_distributed / broadcast_params_distributed /
// avg_weights_distributed: its only multi-GPU mechanism is Net::sync_weights
// (src/net/net_func.cpp:111-127, called from src/net/net_api.cpp:1295-1297 and :779-781),
// which averages parameters through host memory inside ONE process.  These functions give
// the same arithmetic (sum over replicas in fp32, times 1.0f/N, every replica receives the
// result; all `params`, BatchNorm running statistics included) for ONE PROCESS PER GPU, over
// NCCL on NVLink.
#pragma once
#include "eddl/net/net.h"
#include "eddl/optimizers/optim.h"

namespace eddl_b200 {

// Joins the job described by the environment: RANK, WORLD_SIZE, LOCAL_RANK (as set by
// torchrun / mpirun wrappers) and EDDLB200_NCCL_ID, 256 hex characters holding the NCCL
// unique id made by rank 0 (eddlb200_comm_unique_id).  Returns this process's rank.
// The GPU used is LOCAL_RANK.  Throws std::runtime_error on failure.
int init_distributed();
// Same with explicit arguments (id128 = the 128-byte NCCL unique id).
int init_distributed(int rank, int nranks, int device, const void *id128);
void end_distributed();
int get_rank_distributed();
int get_world_size_distributed();

// Rank 0's parameters overwrite every other rank's (call once after build).
void broadcast_params_distributed(Net *net);
// Average all parameters across ranks when curr_batch % batches_per_avg == 0
// (the trigger of Net::train_batch: tr_batches % lsb == 0).
void avg_weights_distributed(Net *net, int curr_batch, int batches_per_avg);

// Health check of the communicator and of the averaging collectives in flight: throws std::runtime_error when NCCL reports
// an asynchronous error (the communicator is then aborted) or when they are still running after wait_ms milliseconds
// (< 0: no limit).  A host-side poll; nothing waits on the GPU.
void check_distributed(int wait_ms);

// Averaged parameters live in the replica on the GPU; the coordinator copy (net->layers[*]->params on the host) is not
// refreshed by avg_weights_distributed or broadcast_params_distributed.  Read parameters through eddl::get_parameters (or
// Net::save), which collect the device copies first.

// SGD with momentum whose applygrads is ONE multi-tensor kernel launch instead of two
// elementwise launches per parameter tensor (src/optimizers/optim_sgd.cpp:68-89); results are
// bit-identical to SGD::applygrads.  Use it as eddl::build(net, new eddl_b200::SGDFused(lr, mu), ...).
class SGDFused : public SGD {
public:
    // true: the gradients are averaged across ranks (all-reduce, times 1.0f/N) before the step, so that every rank applies
    // the same update and neither parameters nor momentum need averaging afterwards; do not combine it with
    // avg_weights_distributed.  For SGD with momentum this equals weight averaging up to rounding (the update is linear).
    bool average_gradients = false;
    explicit SGDFused(float lr = 0.01f, float momentum = 0.0f, float weight_decay = 0.0f, bool nesterov = false);
    Optimizer *clone() override;
    Optimizer *share() override;
    void applygrads(int batch) override;
};

// Adam whose applygrads is ONE multi-tensor kernel launch instead of ten elementwise launches per parameter tensor
// (src/optimizers/optim_adam.cpp:85-120).  Parameters, both moment tensors and the squared gradient the reference leaves
// in the gradient tensor are bit-identical to Adam::applygrads; its two scratch tensors (mCap, vCap) are not written.
class AdamFused : public Adam {
public:
    explicit AdamFused(float lr = 0.01f, float beta_1 = 0.9f, float beta_2 = 0.999f, float epsilon = 1e-8f, float weight_decay = 0.0f,
                       bool amsgrad = false);
    Optimizer *clone() override;
    Optimizer *share() override;
    void applygrads(int batch) override;
};

}  // namespace eddl_b200
