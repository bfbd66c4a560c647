"""GPU whole-step parity: EDDL nets built through EDDL's own API run on CS_GPU behind this backend (the drop-in library) and
are compared with the reference's CS_CPU path on the same injected weights and synthetic data.  Requirement: per-step loss
within 1e-4 relative of the reference."""
import os

import numpy as np
import pytest

from eddl_b200 import harness

pytestmark = pytest.mark.gpu
F = np.float32


@pytest.fixture(scope="module")
def gpu_lib(lib):
    return harness.load()


def synth(cfg_shape, classes, batch, seed, dist="normal"):
    rng = np.random.default_rng(seed)
    x = rng.random((batch, *cfg_shape), dtype=F) if dist == "uniform" else rng.standard_normal((batch, *cfg_shape)).astype(F)
    lab = rng.integers(0, classes, batch)
    return x, np.eye(classes, dtype=F)[lab]


def test_small_cnn_trajectory_matches_reference_fixture(gpu_lib, refout):
    """60-step config: 3x[Conv3x3-ReLU-MaxPool] + Dense10, batch 100, SGD lr 0.01 mu 0.9; the first 10 steps are pinned by
    the committed trajectory of the reference's CS_CPU run."""
    net = harness.NetHarness(gpu_lib, "cnn", device=0, optimizer="sgd", lr=0.01, mu=0.9)
    assert net.nfloats == 29066
    net.set_params(harness.init_weights(net.param_info(), seed=1234))
    drng = np.random.default_rng(1234)
    x = drng.random((100, 1, 28, 28), dtype=F); lab = drng.integers(0, 10, 100); y = np.eye(10, dtype=F)[lab]
    np.testing.assert_array_equal(lab.astype(np.int32), refout["cnn_labels"])
    losses = [net.train_batch(x, y)[0]]
    p1 = net.get_params()
    # one update: every parameter within 1e-5 of the largest parameter magnitude
    assert np.max(np.abs(p1 - refout["cnn_params_step1"])) <= 1e-5 * np.max(np.abs(refout["cnn_params_step1"]))
    losses += [net.train_batch(x, y)[0] for _ in range(9)]
    np.testing.assert_allclose(losses, refout["cnn_losses"], rtol=1e-4)
    p = net.get_params()
    # ten momentum updates through ReLU / max-pool switches amplify fp32 summation-order differences of the
    # gradient reductions; the loss (the stated requirement) stays within 1e-4, parameters within 1e-3
    err = np.max(np.abs(p - refout["cnn_params_after"])) / np.max(np.abs(refout["cnn_params_after"]))
    assert err <= 1e-3
    # the remaining 50 steps keep decreasing the loss on the fixed batch
    more = [net.train_batch(x, y)[0] for _ in range(50)]
    assert more[-1] < losses[0]
    net.close()


@pytest.mark.parametrize("opt", ["sgd", "sgd_fused"])
@pytest.mark.parametrize("cfg,hw,classes,batch,steps,mode", [("vgg16bn", 32, 10, 16, 3, "he"), ("resnet50", 64, 100, 8, 3, "he"), ("resnet50", 224, 1000, 2, 2, "he")])
def test_bn_nets_match_live_reference(gpu_lib, ref, cfg, hw, classes, batch, steps, mode, opt):
    if ref is None:
        pytest.skip("oracle/_ref not built")
    os.environ["OMP_NUM_THREADS"] = "1"
    # A small learning rate keeps each update a small perturbation: with lr 0.01 the first update of these randomly
    # initialised nets changes the loss by 50-90%, and a handful of ReLU / max-pool decisions that flip on 1e-7
    # differences of the forward pass (different fp32 summation orders) then move the next loss by several 1e-4.
    cpu = harness.NetHarness(ref.lib(), cfg, device=-1, hw=hw, classes=classes, threads=1, optimizer="sgd", lr=1e-3, mu=0.9)
    gpu = harness.NetHarness(gpu_lib, cfg, device=0, hw=hw, classes=classes, optimizer=opt, lr=1e-3, mu=0.9)
    # layer names carry process-wide counters; shapes and order must agree
    assert cpu.nfloats == gpu.nfloats and [s for _, s in cpu.param_info()] == [s for _, s in gpu.param_info()]
    w0 = harness.init_weights(cpu.param_info(), seed=99, mode="he_normal")
    cpu.set_params(w0); gpu.set_params(w0)
    np.testing.assert_array_equal(gpu.get_params(), w0)
    x, y = synth((3, hw, hw), classes, batch, seed=5)
    for s in range(steps):
        lc, ac = cpu.train_batch(x, y)
        lg, ag = gpu.train_batch(x, y)
        assert abs(lg - lc) <= 1e-4 * abs(lc), (s, lg, lc)
    pc, pg = cpu.get_params(), gpu.get_params()
    # parameters (BatchNorm running statistics included) after `steps` updates, in the L2 sense
    assert np.linalg.norm(pc.astype(np.float64) - pg) <= 1e-4 * np.linalg.norm(pc.astype(np.float64))
    cpu.close(); gpu.close()


def test_resident_step_equals_train_batch(gpu_lib):
    """The device-resident step loop used for the HBM-resident throughput figure performs the same update as train_batch."""
    a = harness.NetHarness(gpu_lib, "cnn", device=0, optimizer="sgd", lr=0.01, mu=0.9)
    b = harness.NetHarness(gpu_lib, "cnn", device=0, optimizer="sgd", lr=0.01, mu=0.9)
    w0 = harness.init_weights(a.param_info(), seed=7); a.set_params(w0); b.set_params(w0)
    x, y = synth((1, 28, 28), 10, 100, seed=3, dist="uniform")
    for _ in range(3):
        a.train_batch(x, y)
    b.train_batch(x, y); b.train_resident(2)
    np.testing.assert_array_equal(a.get_params(), b.get_params())
    a.close(); b.close()
