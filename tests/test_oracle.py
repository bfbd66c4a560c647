"""CPU tests: the numpy restatement (oracle/eddl_oracle.py) against the reference's golden vectors, against
committed outputs of the reference's own CPU code, and -- where oracle/_ref is built -- against that code run live."""
import numpy as np
import pytest

from oracle import eddl_oracle as orc

ATOL_KAT = 1e-3   # Tensor::equivalent(atol=1e-3, rtol=0) in the reference's tests


def _conv_case(c):
    x = np.array(c["x"], np.float32).reshape(c["x_shape"])
    k = c["filters"]; kr, kc = c["kernel"]
    w = np.ones((k, x.shape[1], kr, kc), np.float32) if c["w"] is None else np.array(c["w"], np.float32).reshape(k, x.shape[1], kr, kc)
    b = np.zeros(k, np.float32) if c["bias"] is None else np.array(c["bias"], np.float32)
    return x, w, b


def test_conv_output_size_table(kats):
    t = kats["conv_output_sizes"]; i = 0
    for p in t["padding"]:
        for isz in t["input_sizes"]:
            for s in t["strides"]:
                for k in t["kernels"]:
                    assert orc.compute_output(p, isz, k, s) == t["output_sizes"][i]; i += 1
    assert i == len(t["output_sizes"])


def test_conv_golden_vectors(kats):
    assert len(kats["conv2d"]) == 7
    for c in kats["conv2d"]:
        x, w, b = _conv_case(c)
        y = orc.conv2d_fwd(x, w, b, tuple(c["stride"]), c["padding"])
        np.testing.assert_allclose(y.ravel(), c["fwd"], atol=ATOL_KAT, rtol=0, err_msg=c["name"])
        dx = orc.conv2d_bwd_data(np.ones_like(y), w, x.shape, None, tuple(c["stride"]), c["padding"])
        np.testing.assert_allclose(dx.ravel(), c["bwd"], atol=ATOL_KAT, rtol=0, err_msg=c["name"])


def test_pool_golden_vectors(kats):
    assert len(kats["maxpool2d"]) == 6 and len(kats["avgpool2d"]) == 6
    for c in kats["maxpool2d"]:
        x = np.array(c["x"], np.float32).reshape(c["x_shape"])
        y, ix, iy = orc.maxpool2d_fwd(x, c["kernel"], c["stride"], c["padding"])
        np.testing.assert_allclose(y.ravel(), c["fwd"], atol=ATOL_KAT, rtol=0, err_msg=c["name"])
        dx = orc.maxpool2d_bwd(np.ones_like(y), ix, iy, x.shape)
        np.testing.assert_allclose(dx.ravel(), c["bwd"], atol=ATOL_KAT, rtol=0, err_msg=c["name"])
    for c in kats["avgpool2d"]:
        x = np.array(c["x"], np.float32).reshape(c["x_shape"])
        y = orc.avgpool2d_fwd(x, c["kernel"], c["stride"], c["padding"])
        np.testing.assert_allclose(y.ravel(), c["fwd"], atol=ATOL_KAT, rtol=0, err_msg=c["name"])
        dx = orc.avgpool2d_bwd(np.ones_like(y), x.shape, c["kernel"], c["stride"], c["padding"])
        np.testing.assert_allclose(dx.ravel(), c["bwd"], atol=ATOL_KAT, rtol=0, err_msg=c["name"])


def test_cce_and_softmax_golden(kats):
    c = kats["cce"]
    y = np.array(c["y_true"], np.float32).reshape(c["shape"]); p = np.array(c["y_pred"], np.float32).reshape(c["shape"])
    assert abs(orc.cce_value(y, p) / y.shape[0] - c["value_per_sample"]) < 1e-3
    np.testing.assert_allclose(orc.cce_delta(y, p).ravel(), c["delta_times_batch"], atol=1e-3)
    s = kats["softmax"]
    x = np.array(s["x"], np.float32).reshape(s["shape"])
    out = orc.softmax(x)
    np.testing.assert_allclose(out.ravel(), s["y"], atol=1e-3)
    pd = orc.d_softmax(np.array(s["delta"], np.float32).reshape(s["shape"]), out, np.zeros_like(out))
    np.testing.assert_allclose(pd.ravel(), s["parent_delta"], atol=1e-3)


CONV_TAGS = ["conv_a", "conv_b", "conv_c", "conv_d"]


@pytest.mark.parametrize("tag", CONV_TAGS)
def test_conv_against_reference_outputs(refout, tag):
    r = refout; st, pt, pb, pl, pr, ub = [int(v) for v in r[tag + "_meta"]]
    x, w, dy = r[tag + "_x"], r[tag + "_w"], r[tag + "_dy"]
    b = r[tag + "_b"] if ub else None
    y = orc.conv2d_fwd(x, w, b, (st, st), (pt, pb, pl, pr))
    np.testing.assert_allclose(y, r[tag + "_y"], rtol=1e-5, atol=1e-5)
    gw, gb = orc.conv2d_bwd_weight(x, dy, r[tag + "_gw0"], r[tag + "_gb0"] if ub else None, (st, st), (pt, pb, pl, pr), w.shape[2:])
    np.testing.assert_allclose(gw, r[tag + "_gw"], rtol=1e-5, atol=2e-5)
    if ub:
        np.testing.assert_allclose(gb, r[tag + "_gb"], rtol=1e-5, atol=2e-5)
    dx = orc.conv2d_bwd_data(dy, w, x.shape, r[tag + "_dx0"], (st, st), (pt, pb, pl, pr))
    np.testing.assert_allclose(dx, r[tag + "_dx"], rtol=1e-5, atol=2e-5)


@pytest.mark.parametrize("tag,affine,mom", [("bn_a", True, 0.99), ("bn_b", False, 0.9), ("bn_c", True, 0.0)])
def test_bn_against_reference_outputs(refout, tag, affine, mom):
    r = refout
    g = r[tag + "_g"] if affine else None; b = r[tag + "_b"] if affine else None
    f = orc.bn_fwd(r[tag + "_x"], r[tag + "_gm"], r[tag + "_gv"], g, b, True, 1e-3, mom)
    np.testing.assert_allclose(f["y"], r[tag + "_y"], rtol=2e-5, atol=2e-5)
    np.testing.assert_allclose(f["mean"], r[tag + "_mean"], rtol=1e-5, atol=1e-6)
    np.testing.assert_allclose(f["var"], r[tag + "_var"], rtol=1e-5, atol=1e-6)
    np.testing.assert_allclose(f["gmean"], r[tag + "_gm1"], rtol=1e-6, atol=1e-7)
    np.testing.assert_allclose(f["gvar"], r[tag + "_gv1"], rtol=1e-5, atol=1e-7)
    fe = orc.bn_fwd(r[tag + "_x"], r[tag + "_gm1"], r[tag + "_gv1"], g, b, False, 1e-3, mom)
    np.testing.assert_allclose(fe["y"], r[tag + "_yeval"], rtol=1e-5, atol=1e-5)
    opa = r[tag + "_opa"] if affine else r[tag + "_y"]
    bw = orc.bn_bwd(r[tag + "_d"], opa, r[tag + "_pd0"], r[tag + "_gg0"], r[tag + "_gb0"], g, r[tag + "_var"])
    np.testing.assert_allclose(bw["pdelta"], r[tag + "_pd"], rtol=2e-5, atol=2e-5)
    np.testing.assert_allclose(bw["delta"], r[tag + "_dout"], rtol=1e-6, atol=1e-7)
    if affine:
        np.testing.assert_allclose(bw["gg"], r[tag + "_gg"], rtol=1e-5, atol=1e-6)
        np.testing.assert_allclose(bw["gb"], r[tag + "_gb"], rtol=1e-5, atol=1e-6)


def test_dense_optim_sync_against_reference_outputs(refout):
    r = refout
    a, b, c0 = r["mm_a"], r["mm_b"], r["mm_c0"]
    np.testing.assert_allclose(orc.mult2d(a, 0, b, 0), r["mm_nn"], rtol=1e-5, atol=1e-5)
    np.testing.assert_allclose(orc.mult2d(a, 0, b, 0, c0, 1), r["mm_nn_inc"], rtol=1e-5, atol=1e-5)
    np.testing.assert_allclose(orc.mult2d(a.T.copy(), 1, b, 0), r["mm_tn"], rtol=1e-5, atol=1e-5)
    np.testing.assert_allclose(orc.mult2d(a, 0, b.T.copy(), 1), r["mm_nt"], rtol=1e-5, atol=1e-5)
    np.testing.assert_array_equal(orc.reduce_sum2d(a, 0), r["rs_axis0"])
    np.testing.assert_allclose(orc.reduce_sum2d(a, 1), r["rs_axis1"], rtol=1e-6, atol=1e-6)
    np.testing.assert_array_equal(orc.sum2d_rowwise(a, a[0]), r["rowbias"])
    p1, m1 = orc.sgd_step(r["opt_p"], r["opt_g"], r["opt_m"], 0.1, 0.9)
    np.testing.assert_array_equal(p1, r["sgd_p"]); np.testing.assert_array_equal(m1, r["sgd_m"])
    ap, ag, am, av = orc.adam_step(r["opt_p"], r["opt_g"], r["opt_m"], r["opt_v"], 0.01, 0.9, 0.999, 1e-6, 3)
    np.testing.assert_array_equal(am, r["adam_m"]); np.testing.assert_array_equal(av, r["adam_v"]); np.testing.assert_array_equal(ag, r["adam_g"])
    np.testing.assert_allclose(ap, r["adam_p"], rtol=0, atol=1e-7)
    np.testing.assert_array_equal(orc.sync_weights(r["sync_reps"]), r["sync_avg"])


# ---- the reference's own CPU code, run live (only where oracle/_ref has been built) -------------------------------
def test_reference_build_reproduces_its_golden_vectors(ref, kats):
    if ref is None:
        pytest.skip("oracle/_ref not built")
    for c in kats["conv2d"]:
        x, w, b = _conv_case(c)
        oh, ow, pads = orc.resolve(c["padding"], x.shape[2], x.shape[3], *c["kernel"], *c["stride"])
        y, _, _, dx = ref.conv2d(x, w, b, dy=np.ones((1, c["filters"], oh, ow), np.float32), stride=tuple(c["stride"]), pads=pads)
        np.testing.assert_allclose(y.ravel(), c["fwd"], atol=ATOL_KAT, rtol=0, err_msg=c["name"])
        np.testing.assert_allclose(dx.ravel(), c["bwd"], atol=ATOL_KAT, rtol=0, err_msg=c["name"])
    for kind, is_max in (("maxpool2d", 1), ("avgpool2d", 0)):
        for c in kats[kind]:
            x = np.array(c["x"], np.float32).reshape(c["x_shape"])
            oh, ow, pads = orc.resolve(c["padding"], x.shape[2], x.shape[3], *c["kernel"], *c["stride"])
            y, ix, iy, dx = ref.pool2d(is_max, x, c["kernel"], c["stride"], pads, dy=np.ones((1, x.shape[1], oh, ow), np.float32))
            np.testing.assert_allclose(y.ravel(), c["fwd"], atol=ATOL_KAT, rtol=0, err_msg=c["name"])
            np.testing.assert_allclose(dx.ravel(), c["bwd"], atol=ATOL_KAT, rtol=0, err_msg=c["name"])


def test_restatement_matches_live_reference_on_random_cases(ref):
    if ref is None:
        pytest.skip("oracle/_ref not built")
    rng = np.random.default_rng(7)
    for (n, c, h, w, k, kr, st, pads) in [(2, 5, 10, 9, 4, 3, 1, (1, 1, 1, 1)), (1, 3, 12, 12, 8, 3, 2, (1, 1, 1, 1)), (3, 16, 5, 5, 16, 1, 1, (0, 0, 0, 0))]:
        x = rng.standard_normal((n, c, h, w)).astype(np.float32); wt = rng.standard_normal((k, c, kr, kr)).astype(np.float32)
        y0 = orc.conv2d_fwd(x, wt, None, (st, st), pads); dy = rng.standard_normal(y0.shape).astype(np.float32)
        y, gw, _, dx = ref.conv2d(x, wt, None, dy, stride=(st, st), pads=pads)
        np.testing.assert_allclose(y0, y, rtol=1e-5, atol=1e-5)
        np.testing.assert_allclose(orc.conv2d_bwd_weight(x, dy, None, None, (st, st), pads, (kr, kr))[0], gw, rtol=1e-5, atol=3e-5)
        np.testing.assert_allclose(orc.conv2d_bwd_data(dy, wt, x.shape, None, (st, st), pads), dx, rtol=1e-5, atol=3e-5)
    for kernel, stride, pads in [((2, 2), (2, 2), (0, 0, 0, 0)), ((3, 3), (2, 2), (1, 1, 1, 1)), ((3, 3), (1, 1), (1, 1, 1, 1))]:
        x = rng.standard_normal((2, 3, 9, 10)).astype(np.float32)
        y0, ix0, iy0 = orc.maxpool2d_fwd(x, kernel, stride, pads); dy = rng.standard_normal(y0.shape).astype(np.float32)
        y, ix, iy, dx = ref.pool2d(1, x, kernel, stride, pads, dy)
        np.testing.assert_array_equal(y0, y); np.testing.assert_array_equal(ix0, ix); np.testing.assert_array_equal(iy0, iy)
        np.testing.assert_allclose(orc.maxpool2d_bwd(dy, ix0, iy0, x.shape), dx, rtol=1e-6, atol=1e-6)
        ya, _, _, dxa = ref.pool2d(0, x, kernel, stride, pads, dy)
        np.testing.assert_allclose(orc.avgpool2d_fwd(x, kernel, stride, pads), ya, rtol=1e-6, atol=1e-6)
        np.testing.assert_allclose(orc.avgpool2d_bwd(dy, x.shape, kernel, stride, pads), dxa, rtol=1e-6, atol=1e-6)
    a = rng.standard_normal((33, 17)).astype(np.float32)
    np.testing.assert_array_equal(orc.relu(a), ref.relu(a))
    np.testing.assert_allclose(orc.softmax(a), ref.softmax(a), rtol=1e-6, atol=1e-7)
    y = np.eye(17, dtype=np.float32)[rng.integers(0, 17, 33)]; p = ref.softmax(a)
    v, d = ref.cce(y, p)
    assert abs(orc.cce_value(y, p) - v) <= 1e-5 * abs(v)
    np.testing.assert_array_equal(orc.cce_delta(y, p), d)
    assert orc.accuracy(y, p) == ref.accuracy(y, p)
    np.testing.assert_array_equal(orc.pad(a.reshape(1, 3, 11, 17), (1, 2, 3, 4)), ref.pad(a.reshape(1, 3, 11, 17), (1, 2, 3, 4)))


def test_reference_outputs_fixture_is_current(ref, refout):
    """The committed ref_outputs.npz equals what the reference build produces now (spot check)."""
    if ref is None:
        pytest.skip("oracle/_ref not built")
    r = refout
    p1, m1 = ref.sgd_step(r["opt_p"], r["opt_g"], r["opt_m"], 0.1, 0.9)
    np.testing.assert_array_equal(p1, r["sgd_p"])
    np.testing.assert_array_equal(ref.sync_weights(r["sync_reps"]), r["sync_avg"])
    st, pt, pb, pl, pr, ub = [int(v) for v in r["conv_b_meta"]]
    y, _, _, _ = ref.conv2d(r["conv_b_x"], r["conv_b_w"], None, stride=(st, st), pads=(pt, pb, pl, pr))
    np.testing.assert_allclose(y, r["conv_b_y"], rtol=1e-6, atol=1e-6)


def test_sampled_conv_evaluation_agrees_with_the_full_restatement():
    """conv2d_samples (used on tensors too large for the host) follows the same index arithmetic as the full functions."""
    rng = np.random.default_rng(0)
    for (n, c, h, w, k, kr, kc, st, pads) in [(2, 3, 9, 8, 5, 3, 3, 1, (1, 1, 1, 1)), (3, 4, 11, 11, 6, 3, 3, 2, (1, 1, 1, 1)),
                                                (2, 3, 14, 14, 4, 7, 7, 2, (3, 3, 3, 3)), (2, 5, 7, 9, 3, 2, 3, 1, (0, 1, 1, 1))]:
        x = rng.standard_normal((n, c, h, w)).astype(np.float32); wt = rng.standard_normal((k, c, kr, kc)).astype(np.float32)
        y = orc.conv2d_fwd(x, wt, None, (st, st), pads); dy = rng.standard_normal(y.shape).astype(np.float32)
        gw, _ = orc.conv2d_bwd_weight(x, dy, None, None, (st, st), pads, (kr, kc))
        dx = orc.conv2d_bwd_data(dy, wt, x.shape, None, (st, st), pads)
        s = orc.conv2d_samples(x, wt, dy, (st, st), pads, 100, seed=1)
        for key, full in (("y", y), ("gw", gw), ("dx", dx)):
            idx, v = s[key]
            np.testing.assert_allclose(full.ravel()[idx], v, rtol=0, atol=2e-6 * max(1.0, float(np.max(np.abs(full)))))
