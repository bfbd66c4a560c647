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


def _trajectory(lib_, cfg, hw, classes, device, opt, w0, x, y, steps, threads=-1):
    net = harness.NetHarness(lib_, cfg, device=device, hw=hw, classes=classes, threads=threads, optimizer=opt, lr=1e-3, mu=0.9)
    net.set_params(w0)
    losses = [net.train_batch(x, y)[0] for _ in range(steps)]
    p = net.get_params()
    net.close()
    return np.array(losses, np.float64), p


@pytest.mark.parametrize("opt", ["sgd", "sgd_fused"])
@pytest.mark.parametrize("cfg,hw,classes,batch,steps", [("vgg16bn", 32, 10, 16, 3), ("resnet50", 64, 100, 8, 3), ("resnet50", 224, 1000, 2, 1)])
def test_bn_nets_match_live_reference(gpu_lib, ref, cfg, hw, classes, batch, steps, opt):
    """First step (pure forward + loss): within 1e-4 relative of the reference's CS_CPU path, the stated requirement.
    Later steps: these randomly initialised BatchNorm nets are chaotic -- the reference itself moves its step-2 loss by
    0.4-1.6% when its weights are perturbed by 1e-7 relative, because a few ReLU / max-pool decisions flip -- so the bound
    for steps >= 2 is calibrated on the reference: the GPU trajectory must stay within 3x the spread the reference shows
    under 1e-6 relative weight perturbations (or within 1e-4, whichever is larger)."""
    if ref is None:
        pytest.skip("oracle/_ref not built")
    ref.set_threads(1)          # the reference's BatchNorm sums race under OpenMP; one thread makes them reproducible
    probe = harness.NetHarness(ref.lib(), cfg, device=-1, hw=hw, classes=classes, threads=1)
    info = probe.param_info(); probe.close()
    w0 = harness.init_weights(info, seed=99, mode="he_normal")
    x, y = synth((3, hw, hw), classes, batch, seed=5)
    base, pc = _trajectory(ref.lib(), cfg, hw, classes, -1, "sgd", w0, x, y, steps, threads=1)
    spread = np.zeros(steps)
    for t in ((1, 2) if steps > 1 else ()):
        wp = (w0 * (1 + 1e-6 * np.random.default_rng(t).standard_normal(w0.size))).astype(F)
        pert, _ = _trajectory(ref.lib(), cfg, hw, classes, -1, "sgd", wp, x, y, steps, threads=1)
        spread = np.maximum(spread, np.abs(pert - base))
    got, pg = _trajectory(gpu_lib, cfg, hw, classes, 0, opt, w0, x, y, steps)
    assert abs(got[0] - base[0]) <= 1e-4 * abs(base[0]), (got[0], base[0])
    for s in range(1, steps):
        assert abs(got[s] - base[s]) <= max(1e-4 * abs(base[s]), 3 * spread[s]), (s, got[s], base[s], spread[s])
    assert np.all(np.isfinite(pg)) and pg.shape == pc.shape


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


@pytest.mark.parametrize("cfg,hw,classes,batch", [("resnet50", 224, 1000, 64), ("vgg16bn", 32, 10, 128)])
def test_first_step_loss_at_benchmark_batch(gpu_lib, ref, cfg, hw, classes, batch):
    """The two benchmark nets at the batch size their throughput is quoted on: the loss of the first step (forward pass
    of the injected weights on the full batch) is within 1e-4 relative of the reference's CS_CPU path.  The reference
    runs on all host threads here; its BatchNorm sums then differ run to run by ~1e-7, far inside the bound."""
    if ref is None:
        pytest.skip("oracle/_ref not built")
    ref.set_threads(os.cpu_count() or 1)
    cpu = harness.NetHarness(ref.lib(), cfg, device=-1, hw=hw, classes=classes, threads=os.cpu_count() or 1)
    w0 = harness.init_weights(cpu.param_info(), seed=77, mode="he_normal")
    x, y = synth((3, hw, hw), classes, batch, seed=6)
    cpu.set_params(w0)
    want = cpu.train_batch(x, y)[0]
    cpu.close()
    ref.set_threads(1)
    net = harness.NetHarness(gpu_lib, cfg, device=0, hw=hw, classes=classes, optimizer="sgd_fused", lr=1e-3, mu=0.9)
    net.set_params(w0)
    got = net.train_batch(x, y)[0]
    net.close()
    print(cfg, "batch", batch, "first-step loss", got, "reference", want)
    assert abs(got - want) <= 1e-4 * abs(want), (got, want)


@pytest.mark.parametrize("opt,loss", [("adam", "categorical_cross_entropy"), ("adam_fused", "categorical_cross_entropy"),
                                      ("sgd", "softmax_cross_entropy"), ("adam_fused", "softmax_cross_entropy")])
def test_small_cnn_with_adam_and_softmax_cross_entropy(gpu_lib, ref, opt, loss):
    """Adam (the reference's ten-launch chain and the fused multi-tensor class) and the softmax_cross_entropy loss (whose
    softmax layer backpropagates delta unchanged) through a Net: five steps of the small CNN against the reference's CS_CPU
    run of the same configuration.  Loss within 1e-4 relative at every step, parameters within 1e-3 of the largest."""
    if ref is None:
        pytest.skip("oracle/_ref not built")
    ref.set_threads(1)
    x, y = synth((1, 28, 28), 10, 100, seed=8, dist="uniform")
    probe = harness.NetHarness(ref.lib(), "cnn", device=-1, threads=1)
    w0 = harness.init_weights(probe.param_info(), seed=21); probe.close()

    def run(lib_, device, optimizer):
        net = harness.NetHarness(lib_, "cnn", device=device, threads=1, optimizer=optimizer, lr=0.002, mu=0.9, loss=loss)
        net.set_params(w0)
        losses = [net.train_batch(x, y)[0] for _ in range(5)]
        p = net.get_params(); net.close()
        return np.array(losses), p
    want, pw = run(ref.lib(), -1, "adam" if opt.startswith("adam") else "sgd")
    got, pg = run(gpu_lib, 0, opt)
    np.testing.assert_allclose(got, want, rtol=1e-4)
    assert np.max(np.abs(pg - pw)) <= 1e-3 * np.max(np.abs(pw))


def test_fused_adam_is_bit_identical_to_the_reference_chain(gpu_lib):
    """On the GPU the one-launch AdamFused leaves the same parameters as Adam::applygrads' ten elementwise launches."""
    x, y = synth((1, 28, 28), 10, 100, seed=9, dist="uniform")
    out = []
    for opt in ("adam", "adam_fused"):
        net = harness.NetHarness(gpu_lib, "cnn", device=0, optimizer=opt, lr=0.002)
        net.set_params(harness.init_weights(net.param_info(), seed=22))
        losses = [net.train_batch(x, y)[0] for _ in range(4)]
        out.append((losses, net.get_params())); net.close()
    assert out[0][0] == out[1][0]
    np.testing.assert_array_equal(out[0][1], out[1][1])


def test_forward_backward_update_equals_train_batch(gpu_lib):
    """zeroGrads / forward / backward(target) / update on CS_GPU perform the step train_batch performs: same losses, same
    metric, bit-identical parameters (a BatchNorm net, so running statistics are covered too)."""
    x, y = synth((3, 32, 32), 10, 16, seed=10)
    res = []
    for fine in (False, True):
        net = harness.NetHarness(gpu_lib, "vgg16bn", device=0, hw=32, classes=10, optimizer="sgd", lr=1e-3, mu=0.9)
        net.set_params(harness.init_weights(net.param_info(), seed=23, mode="he_normal"))
        steps = [(net.train_fine(x, y) if fine else net.train_batch(x, y)) for _ in range(3)]
        res.append((steps, net.get_params())); net.close()
    assert res[0][0] == res[1][0], (res[0][0], res[1][0])
    np.testing.assert_array_equal(res[0][1], res[1][1])


def test_save_and_load_round_trip_on_the_gpu(gpu_lib, tmp_path):
    """Net::save collects the replica's parameters through the backend and Net::load sends them back: a trained net saved
    and loaded into a freshly built one gives identical parameters and an identical next step."""
    x, y = synth((1, 28, 28), 10, 100, seed=11, dist="uniform")
    a = harness.NetHarness(gpu_lib, "cnn", device=0, optimizer="sgd", lr=0.01, mu=0.9)
    a.set_params(harness.init_weights(a.param_info(), seed=24))
    for _ in range(2):
        a.train_batch(x, y)
    path = str(tmp_path / "cnn.bin")
    a.save(path)
    pa = a.get_params()
    b = harness.NetHarness(gpu_lib, "cnn", device=0, optimizer="sgd", lr=0.01, mu=0.9)
    b.load(path)
    np.testing.assert_array_equal(b.get_params(), pa)
    # the optimizer state is not part of the file, so compare a forward pass rather than a momentum step
    np.testing.assert_array_equal(a.forward(x, 10), b.forward(x, 10))
    a.close(); b.close()
