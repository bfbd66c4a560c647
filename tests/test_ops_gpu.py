"""GPU parity tests: every C-ABI entry point against the CPU restatement (oracle/eddl_oracle.py), the committed outputs
of the reference's own CPU code, its golden vectors, and -- where oracle/_ref travels with the repo -- that code run live.
Integer/index results must be bit-exact; elementwise fp32 chains must be bit-exact; reductions and contractions
carry the tolerance written at each assert."""
import ctypes

import numpy as np
import pytest

from oracle import eddl_oracle as orc

pytestmark = pytest.mark.gpu
F = np.float32


def dev(lib, a):
    return lib.to_device(np.asarray(a, F))


def rnd(rng, *shape):
    return rng.standard_normal(shape).astype(F)


# ---------------------------------------------------------------------------------------- elementwise
@pytest.mark.parametrize("n", [0, 1, 3, 4, 1023, 4096, 1 << 20, (1 << 20) + 5])
def test_elementwise_bit_exact(lib, n):
    rng = np.random.default_rng(n)
    a, b, c = rnd(rng, n), rnd(rng, n), rnd(rng, n)
    da, db, dc = dev(lib, a), dev(lib, b), dev(lib, c)
    lib.call("axpby", 0, 0.3, da, -1.7, db, dc, 0, n)
    np.testing.assert_array_equal(dc.numpy(), orc.axpby(0.3, a, -1.7, b))
    dc = dev(lib, c); lib.call("axpby", 0, 0.3, da, -1.7, db, dc, 1, n)
    np.testing.assert_array_equal(dc.numpy(), orc.axpby(0.3, a, -1.7, b, c, 1))
    out = lib.empty((n,))
    lib.call("scale", 0, da, out, 0.37, n); np.testing.assert_array_equal(out.numpy(), (a * F(0.37)).astype(F))
    lib.call("addc", 0, da, out, 0.5, n); np.testing.assert_array_equal(out.numpy(), (a + F(0.5)).astype(F))
    lib.call("sqr", 0, da, out, n); np.testing.assert_array_equal(out.numpy(), (a * a).astype(F))
    lib.call("sqrt", 0, dev(lib, np.abs(a)), out, n); np.testing.assert_array_equal(out.numpy(), np.sqrt(np.abs(a)).astype(F))
    lib.call("clamp", 0, da, out, -0.5, 0.25, n); np.testing.assert_array_equal(out.numpy(), np.clip(a, F(-0.5), F(0.25)))
    lib.call("relu_fwd", 0, da, out, n); np.testing.assert_array_equal(out.numpy(), orc.relu(a))
    dc = dev(lib, c); lib.call("relu_bwd", 0, da, db, dc, n); np.testing.assert_array_equal(dc.numpy(), orc.d_relu(a, b, c))
    dc = dev(lib, c); lib.call("inc", 0, da, dc, n); np.testing.assert_array_equal(dc.numpy(), (c + a).astype(F))
    bb = np.where(np.abs(b) < 0.1, F(0.5), b)
    lib.call("el_div", 0, da, dev(lib, bb), out, 0, n); np.testing.assert_array_equal(out.numpy(), (a / bb).astype(F))
    lib.call("el_mult", 0, da, db, out, 0, n); np.testing.assert_array_equal(out.numpy(), (a * b).astype(F))
    lib.call("fill", 0, out, n, 2.5); np.testing.assert_array_equal(out.numpy(), np.full(n, 2.5, F))


def test_elementwise_unaligned_views(lib):
    """Pointers that are only 4-byte aligned take the scalar path and give the same result."""
    rng = np.random.default_rng(1)
    n = 1001
    a, b = rnd(rng, n + 1), rnd(rng, n + 1)
    da, db, dc = dev(lib, a), dev(lib, b), lib.zeros((n + 1,))
    off = lambda d: ctypes.c_void_p(d.ptr.value + 4)
    lib.call("axpby", 0, 2.0, off(da), 3.0, off(db), off(dc), 0, n)
    np.testing.assert_array_equal(dc.numpy()[1:], orc.axpby(2.0, a[1:], 3.0, b[1:]))
    assert dc.numpy()[0] == 0


def test_pad_and_pad_back(lib, ref):
    rng = np.random.default_rng(2)
    a = rnd(rng, 2, 3, 5, 7); pads = (1, 2, 3, 4)   # top, right, bottom, left
    db = lib.zeros((2, 3, 5 + 4, 7 + 6))
    lib.call("pad", 0, dev(lib, a), db, 2, 3, 5, 7, pads[0], pads[2], pads[3], pads[1])
    np.testing.assert_array_equal(db.numpy(), orc.pad(a, pads))
    bd = rnd(rng, 2, 3, 9, 13); ad = dev(lib, a)
    lib.call("pad_bwd", 0, ad, dev(lib, bd), 2, 3, 5, 7, pads[0], pads[2], pads[3], pads[1])
    np.testing.assert_array_equal(ad.numpy(), orc.pad_back(a, bd, pads))
    if ref is not None:
        np.testing.assert_array_equal(db.numpy(), ref.pad(a, pads))
        np.testing.assert_array_equal(ad.numpy(), ref.pad_back(a, bd, pads))


# ---------------------------------------------------------------------------------------- softmax / loss / metric
@pytest.mark.parametrize("rows,cols", [(2, 3), (100, 10), (128, 10), (64, 1000), (7, 33), (0, 10)])
def test_softmax_cce_accuracy(lib, ref, rows, cols):
    rng = np.random.default_rng(rows * 1000 + cols)
    a = (rnd(rng, rows, cols) * 3).astype(F)
    out = lib.empty((rows, cols))
    lib.call("softmax_fwd", 0, dev(lib, a), out, rows, cols)
    s = out.numpy()
    np.testing.assert_allclose(s, orc.softmax(a), rtol=2e-6, atol=1e-8)      # exp + a cols-long sum
    if rows == 0:
        return
    y = np.eye(cols, dtype=F)[rng.integers(0, cols, rows)]
    d = rnd(rng, rows, cols); pd0 = rnd(rng, rows, cols)
    dpd = dev(lib, pd0)
    lib.call("softmax_bwd", 0, dev(lib, d), out, dpd, rows, cols)
    np.testing.assert_allclose(dpd.numpy(), orc.d_softmax(d, s, pd0), rtol=1e-5, atol=2e-6)
    v = ctypes.c_float()
    lib.call("cce_value", 0, dev(lib, y), out, rows, cols, ctypes.byref(v))
    assert abs(v.value - orc.cce_value(y, s)) <= 2e-6 * abs(orc.cce_value(y, s)) + 1e-6
    dd = lib.empty((rows, cols))
    lib.call("cce_delta", 0, dev(lib, y), out, dd, rows * cols)
    np.testing.assert_array_equal(dd.numpy(), orc.cce_delta(y, s))
    acc = ctypes.c_int()
    lib.call("accuracy", 0, dev(lib, y), out, rows, cols, ctypes.byref(acc))
    assert acc.value == orc.accuracy(y, s)
    ties = np.zeros((rows, cols), F)                       # all-equal rows: first maximum wins on both sides
    lib.call("accuracy", 0, dev(lib, ties), dev(lib, ties), rows, cols, ctypes.byref(acc))
    assert acc.value == rows
    if ref is not None:
        np.testing.assert_allclose(s, ref.softmax(a), rtol=2e-6, atol=1e-8)
        rv, rd = ref.cce(y, s)
        assert abs(v.value - rv) <= 2e-6 * abs(rv) + 1e-6
        assert acc.value == rows and ref.accuracy(y, s) == orc.accuracy(y, s)


def test_softmax_middle_axis(lib):
    rng = np.random.default_rng(5)
    a = rnd(rng, 3, 6, 4)
    out = lib.empty(a.shape)
    lib.call("softmax_fwd_nd", 0, dev(lib, a), out, 3, 6, 4)
    want = np.moveaxis(orc.softmax(np.moveaxis(a, 1, -1)), -1, 1)
    np.testing.assert_allclose(out.numpy(), want, rtol=2e-6, atol=1e-8)


def test_softmax_and_cce_golden(lib, kats):
    s = kats["softmax"]; x = np.array(s["x"], F).reshape(s["shape"])
    out = lib.empty(x.shape); lib.call("softmax_fwd", 0, dev(lib, x), out, *s["shape"])
    np.testing.assert_allclose(out.numpy().ravel(), s["y"], atol=1e-3)
    pd = lib.zeros(x.shape); lib.call("softmax_bwd", 0, dev(lib, np.array(s["delta"], F)), out, pd, *s["shape"])
    np.testing.assert_allclose(pd.numpy().ravel(), s["parent_delta"], atol=1e-3)
    c = kats["cce"]; v = ctypes.c_float()
    lib.call("cce_value", 0, dev(lib, np.array(c["y_true"], F)), dev(lib, np.array(c["y_pred"], F)), 2, 3, ctypes.byref(v))
    assert abs(v.value / 2 - c["value_per_sample"]) < 1e-3


# ---------------------------------------------------------------------------------------- pooling
POOL_CASES = [((2, 2), (2, 2), (0, 0, 0, 0), (2, 3, 28, 28)), ((2, 2), (2, 2), (0, 0, 0, 0), (2, 3, 7, 7)),
              ((3, 3), (2, 2), (0, 0, 0, 0), (2, 4, 18, 18)), ((3, 3), (2, 2), (1, 1, 1, 1), (1, 2, 9, 11)),
              ((3, 3), (1, 1), (1, 1, 1, 1), (2, 2, 6, 5)), ((7, 7), (1, 1), (0, 0, 0, 0), (3, 16, 7, 7)),
              ((2, 2), (2, 2), (0, 1, 0, 1), (1, 1, 5, 5)),
              # planes of >= 1024 elements: max-pool backward stages each plane's output side in shared memory
              ((3, 3), (2, 2), (1, 1, 1, 1), (3, 5, 40, 36)), ((2, 2), (2, 2), (0, 0, 0, 0), (2, 300, 32, 32)),
              ((3, 3), (1, 1), (1, 1, 1, 1), (1, 3, 33, 34)),
              # four-elements-per-thread path (width a multiple of 4): nine covering windows per element; windows with gaps
              ((3, 3), (1, 1), (1, 1, 1, 1), (2, 2, 36, 40)), ((2, 2), (3, 3), (0, 0, 0, 0), (1, 2, 36, 36)),
              ((5, 5), (2, 2), (2, 2, 2, 2), (1, 2, 32, 48)),
              # two-elements-per-thread path (even width, not a multiple of 4): the 114 x 114 planes behind ResNet's padding layer
              ((3, 3), (2, 2), (0, 0, 0, 0), (2, 3, 114, 114)), ((3, 3), (1, 1), (1, 1, 1, 1), (1, 2, 33, 34)), ((2, 2), (2, 2), (0, 0, 0, 0), (1, 3, 38, 42))]


@pytest.mark.parametrize("kernel,stride,pads,shape", POOL_CASES)
def test_pooling(lib, ref, kernel, stride, pads, shape):
    rng = np.random.default_rng(sum(shape))
    x = rnd(rng, *shape); x[0, 0, :2, :2] = 1.5          # a tie inside the first window
    n, c, ih, iw = shape
    y0, ix0, iy0 = orc.maxpool2d_fwd(x, kernel, stride, pads)
    oh, ow = y0.shape[2:]
    geo = (n, c, ih, iw, oh, ow, kernel[0], kernel[1], stride[0], stride[1], pads[0], pads[2])
    y, ix, iy = lib.empty(y0.shape), lib.empty(y0.shape), lib.empty(y0.shape)
    lib.call("maxpool2d_fwd", 0, dev(lib, x), y, ix, iy, *geo)
    np.testing.assert_array_equal(y.numpy(), y0)
    np.testing.assert_array_equal(ix.numpy(), ix0)       # indices bit-exact
    np.testing.assert_array_equal(iy.numpy(), iy0)
    dy = rnd(rng, *y0.shape); dx0 = rnd(rng, *shape)
    dx = dev(lib, dx0)
    lib.call("maxpool2d_bwd", 0, dev(lib, dy), ix, iy, dx, *geo)
    np.testing.assert_array_equal(dx.numpy(), orc.maxpool2d_bwd(dy, ix0, iy0, shape, dx0))
    ya = lib.empty(y0.shape)
    lib.call("avgpool2d_fwd", 0, dev(lib, x), ya, *geo)
    np.testing.assert_array_equal(ya.numpy(), orc.avgpool2d_fwd(x, kernel, stride, pads))
    dxa = dev(lib, dx0)
    lib.call("avgpool2d_bwd", 0, dev(lib, dy), dxa, *geo)
    np.testing.assert_array_equal(dxa.numpy(), orc.avgpool2d_bwd(dy, shape, kernel, stride, pads, dx0))
    if ref is not None:
        ry, rix, riy, rdx = ref.pool2d(1, x, kernel, stride, pads, dy, dx0)
        np.testing.assert_array_equal(y.numpy(), ry); np.testing.assert_array_equal(ix.numpy(), rix)
        np.testing.assert_array_equal(iy.numpy(), riy); np.testing.assert_array_equal(dx.numpy(), rdx)
        ry, _, _, rdx = ref.pool2d(0, x, kernel, stride, pads, dy, dx0)
        np.testing.assert_array_equal(ya.numpy(), ry); np.testing.assert_array_equal(dxa.numpy(), rdx)


def test_pooling_golden_vectors(lib, kats):
    for kind in ("maxpool2d", "avgpool2d"):
        for c in kats[kind]:
            x = np.array(c["x"], F).reshape(c["x_shape"]); n, ch, ih, iw = x.shape
            oh, ow, pads = orc.resolve(c["padding"], ih, iw, *c["kernel"], *c["stride"])
            geo = (n, ch, ih, iw, oh, ow, *c["kernel"], *c["stride"], pads[0], pads[2])
            y, dx = lib.empty((n, ch, oh, ow)), lib.zeros(x.shape)
            ones = dev(lib, np.ones((n, ch, oh, ow), F))
            if kind == "maxpool2d":
                ix, iy = lib.empty((n, ch, oh, ow)), lib.empty((n, ch, oh, ow))
                lib.call("maxpool2d_fwd", 0, dev(lib, x), y, ix, iy, *geo)
                lib.call("maxpool2d_bwd", 0, ones, ix, iy, dx, *geo)
            else:
                lib.call("avgpool2d_fwd", 0, dev(lib, x), y, *geo)
                lib.call("avgpool2d_bwd", 0, ones, dx, *geo)
            np.testing.assert_allclose(y.numpy().ravel(), c["fwd"], atol=1e-3, rtol=0, err_msg=c["name"])
            np.testing.assert_allclose(dx.numpy().ravel(), c["bwd"], atol=1e-3, rtol=0, err_msg=c["name"])


# ---------------------------------------------------------------------------------------- batch norm
BN_SHAPES = [(4, 6, 5, 4), (8, 3, 7, 7), (16, 10), (128, 64, 32, 32), (64, 256, 14, 14), (32, 2048, 7, 7), (3, 5, 3, 3), (64, 7, 1, 1)]


def _bn_run(lib, x, gm, gv, g, b, trmode, eps, mom, relu=False):
    z = x.shape[1]; bsz = x.shape[0]; rc = int(np.prod(x.shape[2:])) if x.ndim > 2 else 1
    dy, dopa = lib.zeros(x.shape), lib.zeros(x.shape)
    dgm, dgv, dm, dv = dev(lib, gm), dev(lib, gv), lib.zeros((z,)), lib.zeros((z,))
    drelu = lib.zeros(x.shape) if relu else None
    lib.call("bn_fwd", 0, bsz, z, rc, dev(lib, x), dy, dopa, dgm, dgv, None if g is None else dev(lib, g), None if b is None else dev(lib, b),
             dm, dv, int(trmode), eps, mom, drelu)
    return dict(y=dy.numpy(), opa=dopa.numpy(), gmean=dgm.numpy(), gvar=dgv.numpy(), mean=dm.numpy(), var=dv.numpy(),
                relu=None if drelu is None else drelu.numpy())


@pytest.mark.parametrize("shape", BN_SHAPES)
@pytest.mark.parametrize("affine", [True, False])
def test_batchnorm_forward_backward(lib, ref, shape, affine):
    rng = np.random.default_rng(sum(shape) + affine)
    x = (rnd(rng, *shape) * 2 + 0.5).astype(F); z = shape[1]
    g = rnd(rng, z) if affine else None; b = rnd(rng, z) if affine else None
    gm, gv = rnd(rng, z), (rng.random(z) + 0.5).astype(F)
    got = _bn_run(lib, x, gm, gv, g, b, True, 1e-3, 0.99, relu=True)
    want = orc.bn_fwd(x, gm, gv, g, b, True, 1e-3, 0.99)
    # per-channel sums over up to 131072 items: fp32 tree sum vs float64, tolerance 1e-5 relative to the spread
    np.testing.assert_allclose(got["mean"], want["mean"], rtol=1e-5, atol=2e-6)
    np.testing.assert_allclose(got["var"], want["var"], rtol=2e-5, atol=2e-6)
    np.testing.assert_allclose(got["gmean"], want["gmean"], rtol=1e-5, atol=1e-6)
    np.testing.assert_allclose(got["gvar"], want["gvar"], rtol=1e-5, atol=1e-6)
    np.testing.assert_allclose(got["y"], want["y"], rtol=1e-4, atol=5e-5)
    np.testing.assert_array_equal(got["relu"], np.maximum(got["y"], 0))           # fused ReLU output == relu(BN output)
    if affine:
        np.testing.assert_allclose(got["opa"], want["opa"], rtol=1e-4, atol=5e-5)
    # given identical statistics the per-element arithmetic is bit-exact: redo the normalisation from the GPU's own stats
    opa = ((x.reshape(shape[0], z, -1) - got["mean"][None, :, None]) / got["var"][None, :, None]).astype(F)
    yy = opa if not affine else (opa * g[None, :, None] + b[None, :, None]).astype(F)
    np.testing.assert_array_equal(got["y"].reshape(shape[0], z, -1), yy)
    # eval mode
    ge = _bn_run(lib, x, got["gmean"], got["gvar"], g, b, False, 1e-3, 0.99)
    we = orc.bn_fwd(x, got["gmean"], got["gvar"], g, b, False, 1e-3, 0.99)
    np.testing.assert_array_equal(ge["y"], we["y"]); np.testing.assert_array_equal(ge["var"], we["var"])
    # backward
    d, pd0, gg0, gb0 = rnd(rng, *shape), rnd(rng, *shape), rnd(rng, z), rnd(rng, z)
    opa_in = got["opa"] if affine else got["y"]
    bsz = shape[0]; rc = int(np.prod(shape[2:])) if len(shape) > 2 else 1
    dd, dpd, dgg, dgb, m1, m2 = dev(lib, d), dev(lib, pd0), dev(lib, gg0), dev(lib, gb0), lib.zeros((z,)), lib.zeros((z,))
    lib.call("bn_bwd", 0, bsz, z, rc, dd, dev(lib, opa_in), dpd, dgg if affine else None, dgb if affine else None,
             dev(lib, g) if affine else None, dev(lib, got["var"]), m1, m2)
    wb = orc.bn_bwd(d, opa_in, pd0, gg0, gb0, g, got["var"])
    np.testing.assert_allclose(m1.numpy(), wb["m1"], rtol=2e-5, atol=2e-6)
    np.testing.assert_allclose(m2.numpy(), wb["m2"], rtol=2e-5, atol=2e-6)
    np.testing.assert_allclose(dpd.numpy(), wb["pdelta"], rtol=1e-4, atol=5e-5)
    np.testing.assert_array_equal(dd.numpy(), wb["delta"])                         # delta *= gamma in place, bit-exact
    if affine:
        np.testing.assert_allclose(dgg.numpy(), wb["gg"], rtol=2e-5, atol=2e-6)
        np.testing.assert_allclose(dgb.numpy(), wb["gb"], rtol=2e-5, atol=2e-6)
    if ref is not None and x.size <= 1 << 20:
        rf = ref.bn_fwd(x, gm, gv, g, b, True, 1e-3, 0.99)
        np.testing.assert_allclose(got["y"], rf["y"], rtol=1e-4, atol=1e-4)
        np.testing.assert_allclose(got["var"], rf["var"], rtol=1e-4, atol=1e-5)
        np.testing.assert_allclose(got["gmean"], rf["gmean"], rtol=1e-4, atol=1e-5)


@pytest.mark.parametrize("tag,affine,mom", [("bn_a", True, 0.99), ("bn_b", False, 0.9), ("bn_c", True, 0.0)])
def test_batchnorm_against_reference_fixture(lib, refout, tag, affine, mom):
    r = refout
    g = r[tag + "_g"] if affine else None; b = r[tag + "_b"] if affine else None
    got = _bn_run(lib, r[tag + "_x"], r[tag + "_gm"], r[tag + "_gv"], g, b, True, 1e-3, mom)
    np.testing.assert_allclose(got["y"], r[tag + "_y"], rtol=2e-5, atol=2e-5)
    np.testing.assert_allclose(got["var"], r[tag + "_var"], rtol=1e-5, atol=1e-6)
    np.testing.assert_allclose(got["gmean"], r[tag + "_gm1"], rtol=1e-6, atol=1e-7)   # momentum 0 leaves running stats untouched
    np.testing.assert_allclose(got["gvar"], r[tag + "_gv1"], rtol=1e-5, atol=1e-7)


# ---------------------------------------------------------------------------------------- dense algebra
@pytest.mark.parametrize("m,n,k", [(7, 5, 13), (100, 10, 576), (128, 512, 512), (64, 1000, 2048), (1, 1, 1), (65, 129, 17),
                                   (192, 320, 1100)])       # the last two large ones run on the tensor-core kernel (one with a ragged k)
def test_mult2d_and_reductions(lib, ref, m, n, k):
    rng = np.random.default_rng(m * n + k)
    a, b, c0 = rnd(rng, m, k), rnd(rng, k, n), rnd(rng, m, n)
    tol = dict(rtol=2e-5, atol=2e-5 * np.sqrt(k))     # k-long fp32 dot products, order differs from the reference GEMM
    for ta, tb in ((0, 0), (1, 0), (0, 1), (1, 1)):
        A = a.T.copy() if ta else a; B = b.T.copy() if tb else b
        for inc in (0, 1):
            dc = dev(lib, c0)
            lib.call("mult2d", 0, dev(lib, A), ta, dev(lib, B), tb, dc, inc, m, n, k)
            np.testing.assert_allclose(dc.numpy(), orc.mult2d(A, ta, B, tb, c0, inc), **tol)
    out = lib.empty((m, k)); lib.call("sum2d_rowwise", 0, dev(lib, a), dev(lib, a[0]), out, m, k)
    np.testing.assert_array_equal(out.numpy(), orc.sum2d_rowwise(a, a[0]))
    for inc in (0, 1):
        b0 = rnd(rng, k); db = dev(lib, b0)
        lib.call("reduce_sum2d", 0, dev(lib, a), db, m, k, 0, inc)
        np.testing.assert_array_equal(db.numpy(), orc.reduce_sum2d(a, 0, b0, inc))      # same sequential order: bit-exact
        b1 = rnd(rng, m); db = dev(lib, b1)
        lib.call("reduce_sum2d", 0, dev(lib, a), db, m, k, 1, inc)
        np.testing.assert_allclose(db.numpy(), orc.reduce_sum2d(a, 1, b1, inc), rtol=1e-5, atol=1e-5)
    if ref is not None:
        dc = lib.empty((m, n)); lib.call("mult2d", 0, dev(lib, a), 0, dev(lib, b), 0, dc, 0, m, n, k)
        np.testing.assert_allclose(dc.numpy(), ref.mult2d(a, 0, b, 0), **tol)


# ---------------------------------------------------------------------------------------- optimizers
@pytest.mark.parametrize("n", [1, 1000, 4097, 1 << 20])
def test_sgd_and_adam_bit_exact(lib, ref, n):
    rng = np.random.default_rng(n)
    p, g, m, v = rnd(rng, n), rnd(rng, n), (rnd(rng, n) * 0.1).astype(F), (rng.random(n) * 0.01).astype(F)
    dp, dm = dev(lib, p), dev(lib, m)
    lib.call("sgd_momentum", 0, dp, dev(lib, g), dm, 0.1, 0.9, n)
    wp, wm = orc.sgd_step(p, g, m, 0.1, 0.9)
    np.testing.assert_array_equal(dp.numpy(), wp); np.testing.assert_array_equal(dm.numpy(), wm)
    dp, dg, dm, dv = dev(lib, p), dev(lib, g), dev(lib, m), dev(lib, v)
    lib.call("adam", 0, dp, dg, dm, dv, 0.01, 0.9, 0.999, 1e-6, 3, n)
    ap, ag, am, av = orc.adam_step(p, g, m, v, 0.01, 0.9, 0.999, 1e-6, 3)
    np.testing.assert_array_equal(dm.numpy(), am); np.testing.assert_array_equal(dv.numpy(), av); np.testing.assert_array_equal(dg.numpy(), ag)
    np.testing.assert_array_equal(dp.numpy(), ap)
    if ref is not None:
        rp, rm = ref.sgd_step(p, g, m, 0.1, 0.9)
        np.testing.assert_array_equal(wp, rp); np.testing.assert_array_equal(wm, rm)
        rp, rg, rm, rv = ref.adam_step(p, g, m, v, 0.01, 0.9, 0.999, 1e-6, 3)
        np.testing.assert_array_equal(dp.numpy(), rp); np.testing.assert_array_equal(dv.numpy(), rv)


def test_sgd_multi_tensor_equals_per_tensor(lib):
    rng = np.random.default_rng(3)
    sizes = [1, 3, 64, 1000, 16384, 16385, 70001, 0, 5]
    ps, gs, ms = [rnd(rng, s) for s in sizes], [rnd(rng, s) for s in sizes], [rnd(rng, s) for s in sizes]
    dps, dgs, dms = [dev(lib, a) for a in ps], [dev(lib, a) for a in gs], [dev(lib, a) for a in ms]
    arr = lambda ds: (ctypes.c_void_p * len(ds))(*[d.ptr.value for d in ds])
    csz = (ctypes.c_size_t * len(sizes))(*sizes)
    before = lib.launches()
    lib.call("sgd_momentum_multi", 0, arr(dps), arr(dgs), arr(dms), csz, len(sizes), 0.05, 0.9)
    assert lib.launches() - before == 1                       # one launch for the whole parameter set
    for p, g, m, dp, dm in zip(ps, gs, ms, dps, dms):
        wp, wm = orc.sgd_step(p, g, m, 0.05, 0.9)
        np.testing.assert_array_equal(dp.numpy(), wp); np.testing.assert_array_equal(dm.numpy(), wm)


def test_single_rank_averaging_is_identity_and_fused_update(lib):
    """Without a communicator N = 1: averaging multiplies by 1.0f and the fused gradient-average + SGD step equals SGD."""
    rng = np.random.default_rng(4)
    n = 5000
    w = rnd(rng, n); dw = dev(lib, w)
    lib.call("allreduce_avg", 0, dw, n); np.testing.assert_array_equal(dw.numpy(), w)
    bufs = [rnd(rng, s) for s in (7, 1024, 33)]; dbufs = [dev(lib, b) for b in bufs]
    lib.call("allreduce_avg_multi", 0, (ctypes.c_void_p * 3)(*[d.ptr.value for d in dbufs]), (ctypes.c_size_t * 3)(7, 1024, 33), 3)
    for b, d in zip(bufs, dbufs):
        np.testing.assert_array_equal(d.numpy(), b)
    p, g, m = rnd(rng, n), rnd(rng, n), rnd(rng, n)
    dp, dg, dm = dev(lib, p), dev(lib, g), dev(lib, m)
    lib.call("avg_grad_sgd", 0, dp, dg, dm, 0.1, 0.9, n)
    wp, wm = orc.sgd_step(p, g, m, 0.1, 0.9)
    np.testing.assert_array_equal(dp.numpy(), wp); np.testing.assert_array_equal(dm.numpy(), wm)


def test_allocator_reuse_and_errors(lib):
    import ctypes as ct
    used0, cached0 = ct.c_size_t(), ct.c_size_t()
    a = lib.empty((123457,)); del a                          # freed blocks go to the cache ...
    lib.call("mem_info", 0, ct.byref(used0), ct.byref(cached0))
    b = lib.empty((123457,))                                 # ... and are handed out again instead of a new cudaMalloc
    used1, cached1 = ct.c_size_t(), ct.c_size_t()
    lib.call("mem_info", 0, ct.byref(used1), ct.byref(cached1))
    assert cached1.value < cached0.value and used1.value > used0.value
    from eddl_b200 import capi
    with pytest.raises(capi.Error):
        lib.call("free", 0, ctypes.c_void_p(12345))
    with pytest.raises(capi.Error):
        lib.call("conv2d_fwd", 0, b, b, None, b, 1, 0, 4, 4, 1, 3, 3, 2, 2, 1, 1, 0, 0, 0)   # c = 0 is rejected


def test_fill_multi_and_profile_records(lib):
    """Batched fills (one launch for many tensors, different values, ragged and unaligned sizes) and the per-call profile."""
    rng = np.random.default_rng(9)
    sizes = [1, 5, 4096, 16384, 16385, 100003, 0, 7]
    vals = [0.0, 1.5, -2.0, 0.0, 3.25, 0.0, 9.0, -0.5]
    bufs = [dev(lib, rnd(rng, s)) for s in sizes]
    before = lib.launches()
    lib.call("fill_multi", 0, (ctypes.c_void_p * len(bufs))(*[b.ptr.value for b in bufs]), (ctypes.c_size_t * len(sizes))(*sizes),
             (ctypes.c_float * len(vals))(*vals), len(sizes))
    assert lib.launches() - before == 1
    for b, s, v in zip(bufs, sizes, vals):
        np.testing.assert_array_equal(b.numpy(), np.full(s, v, F))
    lib.call("profile_reset", 0); lib.call("profile_enable", 0, 1)
    a = dev(lib, rnd(rng, 64, 32)); b = dev(lib, rnd(rng, 32, 16)); c = lib.empty((64, 16))
    for _ in range(3):
        lib.call("mult2d", 0, a, 0, b, 0, c, 0, 64, 16, 32)
    lib.call("profile_enable", 0, 0)
    n, ms, wk = ctypes.c_int(), (ctypes.c_double * 8)(), (ctypes.c_double * 8)()
    lib.call("profile_records", 0, 7, ms, wk, 8, ctypes.byref(n))
    assert n.value == 3 and all(wk[i] == 2.0 * 64 * 16 * 32 for i in range(3)) and all(ms[i] > 0 for i in range(3))
    calls, tot, work = ctypes.c_ulonglong(), ctypes.c_double(), ctypes.c_double()
    lib.call("profile_read", 0, 7, ctypes.byref(calls), ctypes.byref(tot), ctypes.byref(work))
    assert calls.value == 3 and abs(tot.value - sum(ms[i] for i in range(3))) < 1e-9
    lib.call("profile_reset", 0)


def test_adam_multi_tensor_equals_per_tensor(lib):
    """One launch over ragged, unaligned and empty tensors; every tensor bit-identical to the restated ten-call chain of
    Adam::applygrads (parameters, both moments, and the squared gradient left in the gradient tensor)."""
    rng = np.random.default_rng(31)
    sizes = [1, 3, 64, 1000, 16384, 16385, 70001, 0, 5]
    ps, gs, ms = [rnd(rng, s) for s in sizes], [rnd(rng, s) for s in sizes], [rnd(rng, s) for s in sizes]
    vs = [np.abs(rnd(rng, s)) for s in sizes]
    dps, dgs, dms, dvs = ([dev(lib, a) for a in group] for group in (ps, gs, ms, vs))
    arr = lambda ds: (ctypes.c_void_p * len(ds))(*[d.ptr.value for d in ds])
    csz = (ctypes.c_size_t * len(sizes))(*sizes)
    before = lib.launches()
    lib.call("adam_multi", 0, arr(dps), arr(dgs), arr(dms), arr(dvs), csz, len(sizes), 0.01, 0.9, 0.999, 1e-6, 4)
    assert lib.launches() - before == 1
    for p, g, m, v, dp, dg, dm, dv in zip(ps, gs, ms, vs, dps, dgs, dms, dvs):
        ap, ag, am, av = orc.adam_step(p, g, m, v, 0.01, 0.9, 0.999, 1e-6, 4)
        np.testing.assert_array_equal(dp.numpy(), ap); np.testing.assert_array_equal(dg.numpy(), ag)
        np.testing.assert_array_equal(dm.numpy(), am); np.testing.assert_array_equal(dv.numpy(), av)


def test_loss_and_metric_are_read_back_once_per_pair(lib):
    """The first request for the loss (or the metric) of a (target, prediction) pair computes both; repeats are answered
    without a launch until either tensor is written through the library, and then give the new values."""
    rng = np.random.default_rng(32)
    rows, cols = 64, 1000
    p = rng.random((rows, cols)).astype(F); p /= p.sum(axis=1, keepdims=True)
    lab = rng.integers(0, cols, rows); y = np.eye(cols, dtype=F)[lab]
    dy, dp = dev(lib, y), dev(lib, p)
    loss, hits = ctypes.c_float(), ctypes.c_int()
    lib.call("cce_value", 0, dy, dp, rows, cols, ctypes.byref(loss))
    first = loss.value
    assert abs(first - orc.cce_value(y, p)) <= 2e-6 * abs(first)
    before = lib.launches()
    lib.call("accuracy", 0, dy, dp, rows, cols, ctypes.byref(hits))
    lib.call("cce_value", 0, dy, dp, rows, cols, ctypes.byref(loss))
    lib.call("accuracy", 0, dy, dp, rows, cols, ctypes.byref(hits))
    assert lib.launches() == before and loss.value == first and hits.value == orc.accuracy(y, p)
    # a write to the prediction (here: through a copy) invalidates what was remembered
    p2 = np.roll(p, 1, axis=1).copy()
    lib.call("memcpy_h2d", 0, dp, p2.ctypes.data_as(ctypes.c_void_p), p2.nbytes)
    lib.call("cce_value", 0, dy, dp, rows, cols, ctypes.byref(loss))
    lib.call("accuracy", 0, dy, dp, rows, cols, ctypes.byref(hits))
    assert lib.launches() > before
    assert abs(loss.value - orc.cce_value(y, p2)) <= 2e-6 * abs(loss.value) and hits.value == orc.accuracy(y, p2)
    # so does an in-place kernel on the target
    lib.call("scale", 0, dy, dy, 2.0, rows * cols)
    lib.call("cce_value", 0, dy, dp, rows, cols, ctypes.byref(loss))
    assert abs(loss.value - orc.cce_value(2 * y, p2)) <= 2e-6 * abs(loss.value)


def test_staged_host_to_device_copy_and_peer_copy(lib):
    """Copies through the pinned staging ring deliver the bytes (more copies in a row than the ring has pairs, growing and
    shrinking sizes, the source overwritten right after the call); a peer copy with both ends on one device is a plain copy."""
    rng = np.random.default_rng(33)
    keep = []
    for n in (5, 300000, 17, 1 << 20, 3, 2500001, 64, 99999, 1):
        src = rnd(rng, n); want = src.copy()
        d = lib.empty((n,))
        lib.call("memcpy_h2d_staged", 0, d, src.ctypes.data_as(ctypes.c_void_p), src.nbytes)
        src[...] = -1.0                                     # the caller's buffer is free as soon as the call returns
        keep.append((d, want))
    for d, want in keep:
        np.testing.assert_array_equal(d.numpy(), want)
    a = dev(lib, rnd(rng, 4097)); b = lib.zeros((4097,))
    lib.call("memcpy_peer", 0, b, 0, a, 4097 * 4)
    np.testing.assert_array_equal(b.numpy(), a.numpy())
