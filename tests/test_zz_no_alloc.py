"""GPU test of eddlb200_bn_fwd_noalloc, the BatchNorm forward for callers that may not allocate device memory (its
partial sums live in a fixed array inside the library instead of the cudaMalloc'ed scratch arena).  Kept in a file that
pytest collects last, so a run that stops at the first failure has already run every other test.  It calls the entry
point through the C ABI twice in a row, with different shapes, and checks every output against eddlb200_bn_fwd."""
import ctypes

import numpy as np
import pytest

pytestmark = pytest.mark.gpu
F = np.float32


def _run(lib, which, x, gm, gv, g, b, stream):
    bsz, z = x.shape[:2]; rc = int(np.prod(x.shape[2:]))
    y, opa, relu = lib.zeros(x.shape), lib.zeros(x.shape), lib.zeros(x.shape)
    dgm, dgv, mean, var = lib.to_device(gm), lib.to_device(gv), lib.zeros((z,)), lib.zeros((z,))
    args = [0, bsz, z, rc, lib.to_device(x), y, opa, dgm, dgv, lib.to_device(g), lib.to_device(b), mean, var, 1, 1e-3, 0.99, relu]
    if which == "noalloc":
        lib.call("bn_fwd_noalloc", *args, stream)
    else:
        lib.call("bn_fwd", *args)
    lib.sync(0)
    return [t.numpy() for t in (y, opa, relu, dgm, dgv, mean, var)]


def test_bn_fwd_noalloc_matches_bn_fwd_on_two_calls_in_a_row(lib):
    stream = ctypes.c_void_p()
    lib.call("stream", 0, ctypes.byref(stream))
    rng = np.random.default_rng(2024)
    # the second shape uses fewer partial pairs than the first: stale pairs of the first call stay in the shared
    # array and must not leak into the second result
    for shape in ((32, 256, 28, 28), (8, 24, 7, 5)):
        z = shape[1]
        x = (rng.standard_normal(shape) * 1.5 + 0.25).astype(F)
        gm, gv = rng.standard_normal(z).astype(F), (rng.random(z) + 0.5).astype(F)
        g, b = rng.standard_normal(z).astype(F), rng.standard_normal(z).astype(F)
        want = _run(lib, "bn_fwd", x, gm, gv, g, b, stream)
        got = _run(lib, "noalloc", x, gm, gv, g, b, stream)
        for a, w, name in zip(got, want, ("y", "opa", "relu", "running mean", "running var", "mean", "sigma")):
            np.testing.assert_allclose(a, w, rtol=1e-6, atol=1e-6, err_msg="%s %s" % (name, shape))


def test_bn_fwd_noalloc_rejects_shapes_beyond_its_scratch(lib):
    from eddl_b200 import capi
    z = 300000                      # 300000 channels x 1 slice > 262144 pairs
    buf = lib.zeros((z,))
    with pytest.raises(capi.Error) as e:
        lib.call("bn_fwd_noalloc", 0, 1, z, 1, buf, buf, buf, buf, buf, buf, buf, buf, buf, 1, 1e-3, 0.99, None, None)
    assert "-5" in str(e.value) and "scratch" in str(e.value)
