"""GPU parity tests of Conv2D forward / backward-data / backward-weight through the C ABI.
Tolerance: max |got - want| <= 1e-5 * max |want| for the fp32-equivalent mode (precision 0; the requirement is rel 1e-5 of
the reference's fp32 path) and 1e-3 for plain TF32 (precision 1).  `want` is the float64-accumulated restatement, the
committed outputs of the reference's CPU code, its golden vectors, and that code run live where oracle/_ref is present."""
import ctypes

import numpy as np
import pytest

from oracle import eddl_oracle as orc

pytestmark = pytest.mark.gpu
F = np.float32


def relerr(got, want):
    return float(np.max(np.abs(got.astype(np.float64) - want.astype(np.float64))) / max(float(np.max(np.abs(want))), 1e-30))


def run_conv(lib, x, w, b, dy, gw0, gb0, dx0, stride, pads, precision=0):
    n, c, ih, iw = x.shape; k, _, kr, kc = w.shape
    oh, ow, pads = orc.resolve(pads, ih, iw, kr, kc, *stride)
    geo = (n, c, ih, iw, k, kr, kc, oh, ow, stride[0], stride[1], pads[0], pads[2], precision)
    dx_, dw_ = lib.to_device(x), lib.to_device(w)
    y = lib.empty((n, k, oh, ow))
    lib.call("conv2d_fwd", 0, dx_, dw_, None if b is None else lib.to_device(b), y, *geo)
    out = dict(y=y.numpy())
    if dy is not None:
        ddy = lib.to_device(dy)
        gw = lib.to_device(gw0 if gw0 is not None else np.zeros_like(w))
        gb = None if b is None else lib.to_device(gb0 if gb0 is not None else np.zeros(k, F))
        lib.call("conv2d_bwd_weight", 0, dx_, ddy, gw, gb, *geo)
        dxx = lib.to_device(dx0 if dx0 is not None else np.zeros_like(x))
        lib.call("conv2d_bwd_data", 0, ddy, dw_, dxx, *geo)
        out.update(gw=gw.numpy(), gb=None if gb is None else gb.numpy(), dx=dxx.numpy())
    return out


SHAPES = [  # n, c, h, w, k, kr, kc, stride, pads(t,b,l,r), bias
    (2, 3, 9, 8, 5, 3, 3, 1, (1, 1, 1, 1), True),
    (3, 4, 11, 11, 6, 3, 3, 2, (1, 1, 1, 1), False),
    (2, 8, 6, 6, 7, 1, 1, 1, (0, 0, 0, 0), False),
    (2, 3, 14, 14, 4, 7, 7, 2, (3, 3, 3, 3), False),
    (4, 1, 28, 28, 16, 3, 3, 1, (1, 1, 1, 1), True),       # small-CNN first layer
    (2, 64, 8, 8, 64, 3, 3, 1, (1, 1, 1, 1), False),
    (2, 128, 7, 7, 256, 1, 1, 1, (0, 0, 0, 0), False),
    (2, 64, 16, 16, 128, 1, 1, 2, (0, 0, 0, 0), False),    # 1x1 stride-2 downsample
    (1, 32, 10, 10, 32, 3, 3, 2, (0, 0, 0, 0), False),     # "valid" stride 2 after an explicit Pad layer
    (2, 5, 7, 9, 3, 2, 3, 1, (0, 1, 1, 1), True),          # ragged: rectangular kernel, asymmetric pads
    (1, 256, 14, 14, 256, 3, 3, 1, (1, 1, 1, 1), False),
    (2, 512, 7, 7, 512, 3, 3, 1, (1, 1, 1, 1), False),
]


@pytest.mark.parametrize("shape", SHAPES)
def test_conv_all_three_passes(lib, ref, shape):
    n, c, h, w, k, kr, kc, st, pads, use_bias = shape
    rng = np.random.default_rng(abs(hash(shape)) % (1 << 31))
    x = rng.standard_normal((n, c, h, w)).astype(F); wt = rng.standard_normal((k, c, kr, kc)).astype(F)
    b = rng.standard_normal(k).astype(F) if use_bias else None
    y0 = orc.conv2d_fwd(x, wt, b, (st, st), pads)
    dy = rng.standard_normal(y0.shape).astype(F)
    gw0 = rng.standard_normal(wt.shape).astype(F); dx0 = rng.standard_normal(x.shape).astype(F)
    gb0 = rng.standard_normal(k).astype(F) if use_bias else None
    got = run_conv(lib, x, wt, b, dy, gw0, gb0, dx0, (st, st), pads)
    assert relerr(got["y"], y0) <= 1e-5
    gw, gb = orc.conv2d_bwd_weight(x, dy, gw0, gb0, (st, st), pads, (kr, kc))
    assert relerr(got["gw"], gw) <= 1e-5                    # accumulates into the incoming gradient
    if use_bias:
        assert relerr(got["gb"], gb) <= 1e-5
    assert relerr(got["dx"], orc.conv2d_bwd_data(dy, wt, x.shape, dx0, (st, st), pads)) <= 1e-5
    if ref is not None and x.size * k * kr * kc < 5e8:
        ry, rgw, rgb, rdx = ref.conv2d(x, wt, b, dy, gw0, gb0, dx0, stride=(st, st), pads=pads)
        assert relerr(got["y"], ry) <= 1e-5 and relerr(got["gw"], rgw) <= 1e-5 and relerr(got["dx"], rdx) <= 1e-5


def test_conv_golden_vectors(lib, kats):
    for c in kats["conv2d"]:
        x = np.array(c["x"], F).reshape(c["x_shape"]); k = c["filters"]; kr, kc = c["kernel"]
        w = np.ones((k, x.shape[1], kr, kc), F) if c["w"] is None else np.array(c["w"], F).reshape(k, x.shape[1], kr, kc)
        b = np.zeros(k, F) if c["bias"] is None else np.array(c["bias"], F)
        oh, ow, _ = orc.resolve(c["padding"], x.shape[2], x.shape[3], kr, kc, *c["stride"])
        got = run_conv(lib, x, w, b, np.ones((1, k, oh, ow), F), None, None, None, tuple(c["stride"]), c["padding"])
        np.testing.assert_allclose(got["y"].ravel(), c["fwd"], atol=1e-3, rtol=0, err_msg=c["name"])
        np.testing.assert_allclose(got["dx"].ravel(), c["bwd"], atol=1e-3, rtol=0, err_msg=c["name"])


@pytest.mark.parametrize("tag", ["conv_a", "conv_b", "conv_c", "conv_d"])
def test_conv_against_reference_fixture(lib, refout, tag):
    r = refout; st, pt, pb, pl, pr, ub = [int(v) for v in r[tag + "_meta"]]
    got = run_conv(lib, r[tag + "_x"], r[tag + "_w"], r[tag + "_b"] if ub else None, r[tag + "_dy"], r[tag + "_gw0"],
                   r[tag + "_gb0"] if ub else None, r[tag + "_dx0"], (st, st), (pt, pb, pl, pr))
    assert relerr(got["y"], r[tag + "_y"]) <= 1e-5
    assert relerr(got["gw"], r[tag + "_gw"]) <= 1e-5
    assert relerr(got["dx"], r[tag + "_dx"]) <= 1e-5
    if ub:
        assert relerr(got["gb"], r[tag + "_gb"]) <= 1e-5


def test_conv_linearity_at_benchmark_size(lib):
    """Size-independent property at a full microbenchmark shape (N=64, C=1024 -> K=256, 14x14, 1x1): conv(x1 + x2) ==
    conv(x1) + conv(x2), and <dy, conv(x)> == <conv^T(dy), x> ties the three passes together (adjoint identity)."""
    rng = np.random.default_rng(11)
    n, c, h, k = 64, 1024, 14, 256
    x1 = rng.standard_normal((n, c, h, h)).astype(F); x2 = rng.standard_normal((n, c, h, h)).astype(F)
    w = (rng.standard_normal((k, c, 1, 1)) / 32).astype(F)
    dy = rng.standard_normal((n, k, h, h)).astype(F)
    a = run_conv(lib, x1, w, None, dy, None, None, None, (1, 1), (0, 0, 0, 0))
    b = run_conv(lib, x2, w, None, None, None, None, None, (1, 1), (0, 0, 0, 0))
    s = run_conv(lib, (x1 + x2).astype(F), w, None, None, None, None, None, (1, 1), (0, 0, 0, 0))
    assert relerr(s["y"], a["y"] + b["y"]) <= 2e-5
    lhs = float(np.sum(dy.astype(np.float64) * a["y"].astype(np.float64)))
    assert abs(lhs - float(np.sum(a["dx"].astype(np.float64) * x1.astype(np.float64)))) <= 1e-5 * abs(lhs)
    assert abs(lhs - float(np.sum(a["gw"].astype(np.float64) * w.astype(np.float64)))) <= 1e-5 * abs(lhs)


@pytest.mark.parametrize("shape", [(4, 64, 14, 14, 96, 3, 3, 1, (1, 1, 1, 1)), (2, 48, 9, 9, 40, 1, 1, 1, (0, 0, 0, 0)), (2, 16, 20, 20, 24, 3, 3, 2, (1, 1, 1, 1)),
                                   # 1x1 stride 1 with p*q a multiple of 4: backward-weight gathers both operands with 16-byte loads
                                   (4, 48, 8, 8, 40, 1, 1, 1, (0, 0, 0, 0)), (8, 200, 28, 28, 136, 1, 1, 1, (0, 0, 0, 0))])
def test_tensor_core_path_against_fma_path_and_tf32_mode(lib, shape):
    """The tcgen05 kernel (3xTF32) and the fp32 FMA kernel agree to 1e-5, and so does precision 2 (bf16 cross terms of the
    split, coarser but inside the same bound); plain TF32 (precision 1) stays within 1e-3."""
    n, c, h, w, k, kr, kc, st, pads = shape
    rng = np.random.default_rng(17)
    x = rng.standard_normal((n, c, h, w)).astype(F); wt = rng.standard_normal((k, c, kr, kc)).astype(F)
    oh, ow, _ = orc.resolve(pads, h, w, kr, kc, st, st)
    dy = rng.standard_normal((n, k, oh, ow)).astype(F)
    try:
        lib.call("set_option", b"conv_path", 1)
        a = run_conv(lib, x, wt, None, dy, None, None, None, (st, st), pads)
    finally:
        lib.call("set_option", b"conv_path", 0)
    b = run_conv(lib, x, wt, None, dy, None, None, None, (st, st), pads)
    t = run_conv(lib, x, wt, None, dy, None, None, None, (st, st), pads, precision=1)
    h = run_conv(lib, x, wt, None, dy, None, None, None, (st, st), pads, precision=2)
    for key in ("y", "gw", "dx"):
        print(key, "3xTF32 %.2e  bf16-cross %.2e  TF32 %.2e" % (relerr(b[key], a[key]), relerr(h[key], a[key]), relerr(t[key], a[key])))
        assert relerr(b[key], a[key]) <= 1e-5, key
        assert relerr(h[key], a[key]) <= 1e-5, key
        assert relerr(t[key], a[key]) <= 1e-3, key
    with pytest.raises(Exception):
        run_conv(lib, x, wt, None, dy, None, None, None, (st, st), pads, precision=3)
    lib.call("sync", 0)     # also reports a pipeline time-out of the tensor-core kernel, if any


def test_conv_empty_batch_and_long_reduction(lib):
    """n = 0 is a no-op; a K = 9216 reduction (1024 channels x 3x3) stays within 1e-5 -- the tensor core's truncating
    accumulation would drift to ~7e-5 there with a single accumulator."""
    e = lib.empty((1,))
    lib.call("conv2d_fwd", 0, e, e, None, e, 0, 4, 8, 8, 4, 3, 3, 8, 8, 1, 1, 1, 1, 0)
    rng = np.random.default_rng(23)
    x = rng.standard_normal((2, 1024, 6, 6)).astype(F); w = rng.standard_normal((32, 1024, 3, 3)).astype(F)
    got = run_conv(lib, x, w, None, None, None, None, None, (1, 1), (1, 1, 1, 1))
    assert relerr(got["y"], orc.conv2d_fwd(x, w, None, (1, 1), (1, 1, 1, 1))) <= 1e-5


BENCH_SHAPES = [  # the four microbenchmark shapes at their full batch: n, c, h, w, k, kr, kc, stride, pads
    (64, 256, 56, 56, 256, 3, 3, 1, (1, 1, 1, 1)),
    (64, 1024, 14, 14, 256, 1, 1, 1, (0, 0, 0, 0)),
    (64, 3, 224, 224, 64, 7, 7, 2, (3, 3, 3, 3)),
    (32, 512, 7, 7, 512, 3, 3, 1, (1, 1, 1, 1)),
]


@pytest.mark.parametrize("shape", BENCH_SHAPES)
def test_benchmark_shapes_at_full_batch(lib, shape):
    """The shapes whose TFLOP/s are quoted, at the quoted size (they take split-K and persistent-tile routes the small
    stand-ins do not): the tensor-core result of all three passes is compared on the FULL tensors with the exact-fp32 FMA
    kernel (itself checked against the oracle above), and on 1000 sampled elements per tensor with a float64 evaluation
    of the reference's index arithmetic.  Bound: 1e-5 of the largest magnitude."""
    n, c, h, w, k, kr, kc, st, pads = shape
    rng = np.random.default_rng(41)
    x = rng.standard_normal((n, c, h, w), dtype=F); wt = rng.standard_normal((k, c, kr, kc), dtype=F)
    oh, ow, _ = orc.resolve(pads, h, w, kr, kc, st, st)
    dy = rng.standard_normal((n, k, oh, ow), dtype=F)
    try:
        lib.call("set_option", b"conv_path", 1)
        a = run_conv(lib, x, wt, None, dy, None, None, None, (st, st), pads)
    finally:
        lib.call("set_option", b"conv_path", 0)
    b = run_conv(lib, x, wt, None, dy, None, None, None, (st, st), pads)
    lib.call("sync", 0)
    samples = orc.conv2d_samples(x, wt, dy, (st, st), pads, 1000, seed=43)
    for key in ("y", "gw", "dx"):
        scale = float(np.max(np.abs(a[key])))
        full = float(np.max(np.abs(b[key].astype(np.float64) - a[key].astype(np.float64)))) / scale
        idx, want = samples[key]
        sampled = float(np.max(np.abs(b[key].ravel()[idx].astype(np.float64) - want))) / scale
        print(key, "vs FMA path %.2e   vs float64 samples %.2e" % (full, sampled))
        assert full <= 1e-5, (key, full)
        assert sampled <= 1e-5, (key, sampled)


TMA_SHAPES = [  # 1x1 stride-1 layers fed and drained by TMA tensor copies: n, c, h, w, k
    (2, 64, 8, 8, 96),          # 64 pixels: two whole chunks per image
    (3, 40, 6, 6, 72),          # 36 pixels: a ragged second chunk; channel counts that are not multiples of 32
    (5, 96, 14, 14, 160),       # 196 pixels: seven chunks, the last with 4 pixels; rows of a tile from two images
    (4, 256, 28, 28, 64),       # 784 pixels, 8 K-blocks
    (2, 1024, 14, 14, 256),     # 32 K-blocks: rotating accumulators, one accumulator set
]


@pytest.mark.parametrize("shape", TMA_SHAPES)
def test_tma_fed_1x1_layers_match_the_gather_kernel_bit_for_bit(lib, shape):
    """Forward (with and without bias) and backward-data (into zeros and into a non-zero delta, i.e. TMA store and TMA
    add) of 1x1 stride-1 layers: the TMA-fed kernel issues the same MMAs in the same order as the gather kernel, so the
    results are identical bits wherever the gather kernel does not split the reduction; both are within 1e-5 of the oracle."""
    n, c, h, w, k = shape
    rng = np.random.default_rng(51)
    x = rng.standard_normal((n, c, h, w)).astype(F); wt = rng.standard_normal((k, c, 1, 1)).astype(F)
    b = rng.standard_normal(k).astype(F)
    dy = rng.standard_normal((n, k, h, w)).astype(F); dx0 = rng.standard_normal(x.shape).astype(F)
    out = {}
    for level in (0, 2):
        try:
            lib.call("set_option", b"conv_tma", level)
            r1 = run_conv(lib, x, wt, b, dy, None, None, dx0, (1, 1), (0, 0, 0, 0))
            r2 = run_conv(lib, x, wt, None, dy, None, None, None, (1, 1), (0, 0, 0, 0))
        finally:
            lib.call("set_option", b"conv_tma", 2)
        out[level] = (r1["y"], r1["dx"], r2["y"], r2["dx"])
    lib.call("sync", 0)
    for a, bb, name in zip(out[0], out[2], ("y+bias", "dx accumulated", "y", "dx into zeros")):
        if c < 256:
            np.testing.assert_array_equal(a, bb, err_msg=name)
        else:
            # reductions of 8 K-blocks or more on a grid this small make the gather kernel split K (another summation order)
            assert relerr(a, bb) <= 2e-6, name
    assert relerr(out[2][0], orc.conv2d_fwd(x, wt, b, (1, 1), (0, 0, 0, 0))) <= 1e-5
    assert relerr(out[2][1], orc.conv2d_bwd_data(dy, wt, x.shape, dx0, (1, 1), (0, 0, 0, 0))) <= 1e-5


@pytest.mark.parametrize("shape", TMA_SHAPES + [(16, 64, 56, 56, 256)])
def test_tma_fed_backward_weight_of_1x1_layers(lib, shape):
    """Backward-weight of 1x1 stride-1 layers with both operands copied by TMA into the operand ring (reduction over
    32-pixel chunks of one image, zero-filled past the end of the image): within 1e-5 of the oracle and of the 16-byte
    gather kernel, accumulating into a non-zero gradient.  Level 2 leaves the landed fp32 values as the hi plane; the tensor
    core reads only their upper 19 bits, so the result is the same bits as with the explicit mask."""
    n, c, h, w, k = shape
    rng = np.random.default_rng(61)
    x = rng.standard_normal((n, c, h, w)).astype(F); wt = rng.standard_normal((k, c, 1, 1)).astype(F)
    dy = rng.standard_normal((n, k, h, w)).astype(F); gw0 = rng.standard_normal(wt.shape).astype(F)
    want, _ = orc.conv2d_bwd_weight(x, dy, gw0, None, (1, 1), (0, 0, 0, 0), (1, 1))
    got = {}
    for level in (0, 1, 2):
        try:
            lib.call("set_option", b"conv_tma_wgrad", level)
            got[level] = run_conv(lib, x, wt, None, dy, gw0, None, None, (1, 1), (0, 0, 0, 0))["gw"]
        finally:
            lib.call("set_option", b"conv_tma_wgrad", 2)
    lib.call("sync", 0)
    for level in (0, 1, 2):
        assert relerr(got[level], want) <= 1e-5, level
    print("masked vs unmasked hi plane: max |difference| =", float(np.max(np.abs(got[1] - got[2]))))
    np.testing.assert_array_equal(got[1], got[2])


def test_packed_weight_images_follow_every_write_to_the_weights(lib):
    """The packed (split, swizzled) weight images are kept between calls and re-made only after the weight tensor has been
    written: every way of writing it through the library -- a copy, an in-place kernel, an optimizer step, releasing the
    buffer and getting the same address back with other contents -- must be seen, for the forward and the backward-data
    tiling alike; with the cache off the results are the same bits."""
    rng = np.random.default_rng(71)
    n, c, h, k = 4, 64, 12, 96
    geo3 = (n, c, h, h, k, 3, 3, h, h, 1, 1, 1, 1, 0)
    x = rng.standard_normal((n, c, h, h)).astype(F); dy = rng.standard_normal((n, k, h, h)).astype(F)
    dx_, ddy = lib.to_device(x), lib.to_device(dy)
    y, dxo = lib.empty((n, k, h, h)), lib.empty((n, c, h, h))

    def both(dw):
        lib.call("conv2d_fwd", 0, dx_, dw, None, y, *geo3)
        lib.call("fill", 0, dxo, dxo.size, 0.0)
        lib.call("conv2d_bwd_data", 0, ddy, dw, dxo, *geo3)
        return y.numpy(), dxo.numpy()

    def check(dw, w):
        gy, gdx = both(dw)
        assert relerr(gy, orc.conv2d_fwd(x, w, None, (1, 1), (1, 1, 1, 1))) <= 1e-5
        assert relerr(gdx, orc.conv2d_bwd_data(dy, w, x.shape, None, (1, 1), (1, 1, 1, 1))) <= 1e-5
        return gy, gdx

    w = rng.standard_normal((k, c, 3, 3)).astype(F)
    dw = lib.to_device(w)
    first = check(dw, w)
    before = lib.launches()
    again = both(dw)                                                 # nothing written: no packing launch this time
    steady = lib.launches() - before
    np.testing.assert_array_equal(first[0], again[0]); np.testing.assert_array_equal(first[1], again[1])
    w2 = rng.standard_normal(w.shape).astype(F)
    lib.call("memcpy_h2d", 0, dw, w2.ctypes.data_as(ctypes.c_void_p), w2.nbytes)          # a copy
    before = lib.launches()
    both(dw)
    assert lib.launches() - before == steady + 1                    # ONE launch re-packs both tilings
    check(dw, w2)
    lib.call("scale", 0, dw, dw, -0.5, w.size)                                            # an in-place kernel
    check(dw, (w2 * F(-0.5)).astype(F))
    g_, m_ = lib.to_device(rng.standard_normal(w.size).astype(F)), lib.zeros((w.size,))
    lib.call("sgd_momentum", 0, dw, g_, m_, 0.1, 0.0, w.size)                               # an optimizer step
    w3 = dw.numpy()
    check(dw, w3)
    try:
        lib.call("set_option", b"conv_pack_cache", 0)
        off = both(dw)
    finally:
        lib.call("set_option", b"conv_pack_cache", 1)
    on = both(dw)
    np.testing.assert_array_equal(off[0], on[0]); np.testing.assert_array_equal(off[1], on[1])
    addr = dw.ptr.value
    del dw                                                                                # released ...
    w4 = rng.standard_normal(w.shape).astype(F)
    dw4 = lib.to_device(w4)                                                               # ... and (usually) handed out again
    print("same address reused:", dw4.ptr.value == addr)
    check(dw4, w4)
    # a write the library does not see (another CUDA runtime instance copying into the tensor) has to be announced
    import os
    rt_path = next((p for p in ("/usr/local/cuda/lib64/libcudart.so", "/usr/local/cuda/lib64/libcudart.so.12") if os.path.exists(p)), None)
    if rt_path:
        rt = ctypes.CDLL(rt_path)
        rt.cudaMemcpy.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_size_t, ctypes.c_int]
        w5 = rng.standard_normal(w.shape).astype(F)
        lib.call("notify_write", 0, dw4, w5.nbytes)
        lib.call("sync", 0)
        assert rt.cudaMemcpy(dw4.ptr.value, w5.ctypes.data_as(ctypes.c_void_p), w5.nbytes, 1) == 0
        check(dw4, w5)


SLAB_SHAPES = [  # 3x3 stride-1 "same" layers fed from raw slabs by TMA: n, c, h, w, k
    (2, 64, 8, 8, 96),          # 64 pixels: one ragged tile per image
    (3, 40, 12, 12, 72),        # 144 pixels: a second tile with 16 valid rows; channel counts that are not multiples of 32
    (2, 64, 56, 56, 64),        # the widest plane a slab holds comfortably; 25 tiles per image
    (4, 128, 28, 28, 128),
    (3, 256, 14, 14, 256),      # 72 K-blocks: rotating accumulators
    (2, 32, 16, 60, 32),        # a 60-pixel-wide plane: the largest halo
]


@pytest.mark.parametrize("shape", SLAB_SHAPES)
def test_slab_fed_3x3_layers(lib, shape):
    """Forward (with bias) and backward-data (into zeros and into a non-zero delta) of 3x3 stride-1 pad-1 layers: the slab-fed
    kernel orders its reduction (channel group, tap, channel) instead of (channel, tap), so results agree with the gather
    kernel to rounding, not to the bit; both are within 1e-5 of the oracle."""
    n, c, h, w, k = shape
    rng = np.random.default_rng(81)
    x = rng.standard_normal((n, c, h, w)).astype(F); wt = rng.standard_normal((k, c, 3, 3)).astype(F)
    b = rng.standard_normal(k).astype(F)
    dy = rng.standard_normal((n, k, h, w)).astype(F); dx0 = rng.standard_normal(x.shape).astype(F)
    out = {}
    for level in (0, 1):
        try:
            lib.call("set_option", b"conv_tma_3x3", level)
            r1 = run_conv(lib, x, wt, b, dy, None, None, dx0, (1, 1), (1, 1, 1, 1))
            r2 = run_conv(lib, x, wt, None, dy, None, None, None, (1, 1), (1, 1, 1, 1))
        finally:
            lib.call("set_option", b"conv_tma_3x3", 1)
        out[level] = (r1["y"], r1["dx"], r2["y"], r2["dx"])
    lib.call("sync", 0)
    want = (orc.conv2d_fwd(x, wt, b, (1, 1), (1, 1, 1, 1)), orc.conv2d_bwd_data(dy, wt, x.shape, dx0, (1, 1), (1, 1, 1, 1)),
            orc.conv2d_fwd(x, wt, None, (1, 1), (1, 1, 1, 1)), orc.conv2d_bwd_data(dy, wt, x.shape, None, (1, 1), (1, 1, 1, 1)))
    for a, bb, wv, name in zip(out[0], out[1], want, ("y+bias", "dx accumulated", "y", "dx into zeros")):
        assert relerr(bb, wv) <= 1e-5, name
        assert relerr(a, bb) <= 3e-6, name


DENSE_SHAPES = [  # 1x1 layers that skip pixels or have ragged planes, run as dense 1x1 layers over gathered copies: n, c, h, w, k, stride
    (3, 64, 16, 16, 96, (2, 2)),     # the ResNet shortcut form: a quarter of the pixels
    (2, 256, 28, 28, 128, (2, 2)),
    (4, 96, 14, 14, 64, (2, 2)),     # 7x7 output: ragged planes, backward-weight only
    (5, 64, 7, 7, 160, (1, 1)),      # stride 1, 49-pixel planes: backward-weight over copies padded to 52 pixels
    (2, 40, 15, 18, 48, (3, 2)),     # different strides per axis, rows and columns the last window does not reach
    (1, 32, 9, 9, 32, (1, 1)),       # 81 pixels, a batch of one: the padded reduction is not a multiple of 32
]


@pytest.mark.parametrize("shape", DENSE_SHAPES)
def test_strided_and_ragged_1x1_layers_as_dense_layers(lib, shape):
    """All three passes with and without the rewrite, into zeros and into non-zero gradients; both within 1e-5 of the oracle
    and within rounding of each other (the reduction over channels or pixels is tiled differently)."""
    n, c, h, w, k, stride = shape
    rng = np.random.default_rng(91)
    x = rng.standard_normal((n, c, h, w)).astype(F); wt = rng.standard_normal((k, c, 1, 1)).astype(F)
    b = rng.standard_normal(k).astype(F)
    oh, ow, _ = orc.resolve((0, 0, 0, 0), h, w, 1, 1, *stride)
    dy = rng.standard_normal((n, k, oh, ow)).astype(F)
    gw0 = rng.standard_normal(wt.shape).astype(F); gb0 = rng.standard_normal(k).astype(F); dx0 = rng.standard_normal(x.shape).astype(F)
    out = {}
    for level in (0, 1):
        try:
            lib.call("set_option", b"conv_dense_1x1", level)
            r1 = run_conv(lib, x, wt, b, dy, gw0, gb0, dx0, stride, (0, 0, 0, 0))
            r2 = run_conv(lib, x, wt, None, dy, None, None, None, stride, (0, 0, 0, 0))
        finally:
            lib.call("set_option", b"conv_dense_1x1", 1)
        out[level] = (r1["y"], r1["gw"], r1["dx"], r2["y"], r2["gw"], r2["dx"])
    lib.call("sync", 0)
    pads = (0, 0, 0, 0)
    want = (orc.conv2d_fwd(x, wt, b, stride, pads), orc.conv2d_bwd_weight(x, dy, gw0, None, stride, pads, (1, 1))[0],
            orc.conv2d_bwd_data(dy, wt, x.shape, dx0, stride, pads), orc.conv2d_fwd(x, wt, None, stride, pads),
            orc.conv2d_bwd_weight(x, dy, None, None, stride, pads, (1, 1))[0], orc.conv2d_bwd_data(dy, wt, x.shape, None, stride, pads))
    for a, bb, wv, name in zip(out[0], out[1], want, ("y+bias", "gw accumulated", "dx accumulated", "y", "gw into zeros", "dx into zeros")):
        assert relerr(bb, wv) <= 1e-5, name
        assert relerr(a, bb) <= 3e-6, name


def test_conv_path_counts_tell_fallbacks_from_tensor_core_calls(lib):
    """A call that ends on the fp32 FMA kernels is counted as such, so a training run can check that none of its layers did."""
    def counts():
        a, b = ctypes.c_ulonglong(0), ctypes.c_ulonglong(0)
        lib.call("conv_path_counts", 0, ctypes.byref(a), ctypes.byref(b))
        return a.value, b.value
    rng = np.random.default_rng(5)
    x = rng.standard_normal((2, 8, 10, 10)).astype(F); w = rng.standard_normal((16, 8, 3, 3)).astype(F); dy = rng.standard_normal((2, 16, 10, 10)).astype(F)
    t0, f0 = counts()
    run_conv(lib, x, w, None, dy, None, None, None, (1, 1), (1, 1, 1, 1))
    t1, f1 = counts()
    assert (t1 - t0, f1 - f0) == (3, 0)
    try:
        lib.call("set_option", b"conv_path", 1)
        run_conv(lib, x, w, None, dy, None, None, None, (1, 1), (1, 1, 1, 1))
    finally:
        lib.call("set_option", b"conv_path", 0)
    t2, f2 = counts()
    assert (t2 - t1, f2 - f1) == (0, 3)


WSLAB_SHAPES = SLAB_SHAPES + [(2, 20, 6, 6, 32), (5, 14, 10, 10, 40), (2, 15, 8, 12, 33),
                              # ragged planes (not a multiple of four pixels): run over copies whose rows are padded with zero columns
                              (3, 64, 7, 7, 48), (2, 33, 9, 9, 40), (4, 16, 5, 11, 32),
                              (2, 16, 8, 57, 32)]          # the widest row a backward-weight slab holds


@pytest.mark.parametrize("shape", WSLAB_SHAPES)
def test_slab_fed_backward_weight_of_3x3_layers(lib, shape):
    """Backward-weight of 3x3 stride-1 pad-1 layers with the x operand built from TMA-delivered slabs (tiles of 14 channels x 9
    taps, K-blocks of 32 pixels of one image): into zeros and into a non-zero gradient, with the bias gradient, against the
    oracle within 1e-5 and against the gather kernel to rounding (the reduction is cut into other K-blocks: an image's last
    chunk is padded instead of running on into the next image)."""
    n, c, h, w, k = shape
    rng = np.random.default_rng(83)
    x = rng.standard_normal((n, c, h, w)).astype(F); wt = rng.standard_normal((k, c, 3, 3)).astype(F)
    b = rng.standard_normal(k).astype(F)
    dy = rng.standard_normal((n, k, h, w)).astype(F)
    gw0 = rng.standard_normal(wt.shape).astype(F); gb0 = rng.standard_normal(k).astype(F)
    out = {}
    for level in (0, 1):
        try:
            lib.call("set_option", b"conv_tma_wgrad_3x3", level)
            r1 = run_conv(lib, x, wt, b, dy, gw0, gb0, None, (1, 1), (1, 1, 1, 1))
            r2 = run_conv(lib, x, wt, None, dy, None, None, None, (1, 1), (1, 1, 1, 1))
        finally:
            lib.call("set_option", b"conv_tma_wgrad_3x3", 1)
        out[level] = (r1["gw"], r1["gb"], r2["gw"])
    lib.call("sync", 0)
    g1, gb1 = orc.conv2d_bwd_weight(x, dy, gw0, gb0, (1, 1), (1, 1, 1, 1), (3, 3))
    g2, _ = orc.conv2d_bwd_weight(x, dy, None, None, (1, 1), (1, 1, 1, 1), (3, 3))
    for a, bb, wv, name in zip(out[0], out[1], (g1, gb1, g2), ("gw accumulated", "bias gradient", "gw into zeros")):
        assert relerr(bb, wv) <= 1e-5, name
        assert relerr(a, bb) <= 3e-6, name
