"""GPU parity of the layers EDDL's own convnet examples use beside the benchmark nets: Concat, UpSampling, Dropout's mask,
RandomFlip, RandomCropScale, GlobalMaxPool -- through the C ABI against the oracle.  Copies and fp32 adds in the reference's
order: every comparison is bit-exact.  The random layers take their decisions as arguments, so they are deterministic here;
the Dropout mask (drawn on the device) is checked for its statistics and its reproducibility."""
import ctypes

import numpy as np
import pytest

from oracle import eddl_oracle as orc

pytestmark = pytest.mark.gpu
F = np.float32


def dev(lib, a):
    return lib.to_device(np.ascontiguousarray(a, F))


def ptr_array(ds):
    return (ctypes.c_void_p * len(ds))(*[d.ptr.value for d in ds])


@pytest.mark.parametrize("axis,shapes", [(1, [(3, 4, 6, 7), (3, 5, 6, 7)]), (1, [(2, 64, 14, 14), (2, 32, 14, 14), (2, 1, 14, 14)]),
                                         (2, [(2, 3, 4, 5), (2, 3, 1, 5)]), (3, [(2, 3, 4, 5), (2, 3, 4, 2)])])
def test_concat_forward_and_backward(lib, axis, shapes):
    rng = np.random.default_rng(1)
    parts = [rng.standard_normal(s).astype(F) for s in shapes]
    want = orc.concat(parts, axis)
    dparts = [dev(lib, p) for p in parts]
    a = lib.empty(want.shape)
    sizes = (ctypes.c_size_t * len(parts))(*[p.size for p in parts])
    strides = (ctypes.c_size_t * len(parts))(*[int(np.prod(p.shape[axis:])) for p in parts])
    steps = int(np.prod(want.shape[axis:]))
    lib.call("concat", 0, a, ptr_array(dparts), sizes, strides, len(parts), steps, 0)
    np.testing.assert_array_equal(a.numpy(), want)
    delta = rng.standard_normal(want.shape).astype(F)
    lib.call("concat", 0, dev(lib, delta), ptr_array(dparts), sizes, strides, len(parts), steps, 1)      # parts += their slices
    for d, w in zip(dparts, orc.concat_back(delta, parts, axis)):
        np.testing.assert_array_equal(d.numpy(), w)


@pytest.mark.parametrize("shape,size", [((2, 3, 4, 5), (2, 3)), ((4, 16, 7, 7), (2, 2)), ((1, 1, 3, 3), (1, 4))])
def test_upsampling_forward_and_backward(lib, shape, size):
    rng = np.random.default_rng(2)
    a = rng.standard_normal(shape).astype(F)
    rows = shape[0] * shape[1] * shape[2]
    b = lib.empty((shape[0], shape[1], shape[2] * size[0], shape[3] * size[1]))
    lib.call("repeat_nn", 0, dev(lib, a), b, rows, shape[3], size[0], size[1])
    np.testing.assert_array_equal(b.numpy(), orc.repeat_nn(a, size))
    d = rng.standard_normal(b.shape).astype(F); a0 = rng.standard_normal(shape).astype(F)
    da = dev(lib, a0)
    lib.call("repeat_nn_bwd", 0, dev(lib, d), da, rows, shape[3], size[0], size[1])
    np.testing.assert_array_equal(da.numpy(), orc.d_repeat_nn(d, a0, size))


@pytest.mark.parametrize("case", [(4, 5, 8, 15, 8, 15, 2, 3), (7, 7, 10, 13, 10, 13, 0, 3), (10, 10, 10, 10, 6, 6, 0, 3), (5, 6, 11, 9, 11, 9, 0, 0),
                                  (28, 28, 56, 56, 56, 56, 2, 3)])
def test_resize_forward_and_backward(lib, case):
    """eddl::UpSampling2D builds a resize layer (Tensor::scale / scale_back): whole-factor and ragged zooms, a centred
    zoom-out with constant fill, half-pixel mode."""
    ah, aw, bh, bw, nh, nw, wrap, mode = case
    rng = np.random.default_rng(6)
    n, c = 3, 5
    x = rng.standard_normal((n, c, ah, aw)).astype(F)
    b = lib.empty((n, c, bh, bw))
    lib.call("resize", 0, dev(lib, x), b, n, c, ah, aw, bh, bw, nh, nw, wrap, 1.5, mode)
    np.testing.assert_array_equal(b.numpy(), orc.scale(x, (bh, bw), (nh, nw), mode, wrap, 1.5))
    ad0 = rng.standard_normal(x.shape).astype(F); bd = rng.standard_normal((n, c, bh, bw)).astype(F)
    ad = dev(lib, ad0)
    lib.call("resize_bwd", 0, ad, dev(lib, bd), n, c, ah, aw, bh, bw, nh, nw, wrap, 1.5, mode)
    np.testing.assert_array_equal(ad.numpy(), orc.scale_back(ad0, bd, (nh, nw), mode))


def test_flip_and_crop_scale_with_given_decisions(lib):
    rng = np.random.default_rng(3)
    n, c, h, w = 6, 3, 32, 32
    x = rng.standard_normal((n, c, h, w)).astype(F)
    apply = np.array([1, 0, 1, 1, 0, 0], np.uint8)
    for axis in (0, 1):
        b = lib.empty(x.shape)
        lib.call("flip_batch", 0, dev(lib, x), b, n, c, h, w, axis, apply.ctypes.data_as(ctypes.c_void_p))
        np.testing.assert_array_equal(b.numpy(), orc.flip_batch(x, apply, axis))
    # boxes drawn the way cpu_crop_scale_random draws them: scale in [0.8, 1.0], (y0, x0, y0 + h', x0 + w')
    boxes = []
    for i in range(n):
        s = rng.uniform(0.8, 1.0); hh, ww = int(h * s), int(w * s)
        y0, x0 = int((h - hh) * rng.random()), int((w - ww) * rng.random())
        boxes.append((y0, x0, y0 + hh, x0 + ww))
    boxes = np.array(boxes, np.int32)
    if np.any(boxes[:, 2] >= h) or np.any(boxes[:, 3] >= w):
        boxes[:, 2] = np.minimum(boxes[:, 2], h - 1); boxes[:, 3] = np.minimum(boxes[:, 3], w - 1)
    b = lib.empty(x.shape)
    lib.call("crop_scale_batch", 0, dev(lib, x), b, n, c, h, w, h, w, boxes.ctypes.data_as(ctypes.c_void_p))
    np.testing.assert_array_equal(b.numpy(), orc.crop_scale_batch(x, boxes, (h, w)))
    from eddl_b200 import capi
    bad = boxes.copy(); bad[0, 2] = h + 5                      # a box that reaches past the image is refused, not read
    with pytest.raises(capi.Error):
        lib.call("crop_scale_batch", 0, dev(lib, x), b, n, c, h, w, h, w, bad.ctypes.data_as(ctypes.c_void_p))


def test_dropout_mask_statistics_and_reproducibility(lib):
    n = 1 << 20
    a, b, c = lib.empty((n,)), lib.empty((n,)), lib.empty((n,))
    lib.call("rand_binary", 0, a, n, 0.7, 1234, 0)
    lib.call("rand_binary", 0, b, n, 0.7, 1234, 0)
    lib.call("rand_binary", 0, c, n, 0.7, 1234, n)             # the next stretch of the same stream
    ma, mb, mc = a.numpy(), b.numpy(), c.numpy()
    assert set(np.unique(ma)) <= {0.0, 1.0}
    np.testing.assert_array_equal(ma, mb)
    assert abs(ma.mean() - 0.7) < 5e-3 and abs(mc.mean() - 0.7) < 5e-3      # 5 sigma is 2.2e-3
    assert 0.45 < np.mean(ma == mc) < 0.7                      # independent stretches agree with probability 0.58
    # no structure between neighbours
    assert abs(np.corrcoef(ma[:-1], ma[1:])[0, 1]) < 5e-3


def test_global_max_pool_is_a_max_pool_over_the_whole_plane(lib):
    rng = np.random.default_rng(4)
    n, c, h, w = 4, 32, 7, 7
    x = rng.standard_normal((n, c, h, w)).astype(F)
    want = orc.maxpool2d_fwd(x, (h, w), (1, 1), (0, 0, 0, 0))
    y, ix, iy = lib.empty((n, c, 1, 1)), lib.empty((n, c, 1, 1)), lib.empty((n, c, 1, 1))
    geo = (n, c, h, w, 1, 1, h, w, 1, 1, 0, 0)
    lib.call("maxpool2d_fwd", 0, dev(lib, x), y, ix, iy, *geo)
    np.testing.assert_array_equal(y.numpy(), want[0])
    np.testing.assert_array_equal(ix.numpy(), want[1]); np.testing.assert_array_equal(iy.numpy(), want[2])
    d = rng.standard_normal((n, c, 1, 1)).astype(F); dx0 = rng.standard_normal(x.shape).astype(F)
    dx = dev(lib, dx0)
    lib.call("maxpool2d_bwd", 0, dev(lib, d), ix, iy, dx, *geo)
    np.testing.assert_array_equal(dx.numpy(), orc.maxpool2d_bwd(d, want[1], want[2], x.shape, dx0))


def test_net_with_augmentation_concat_upsampling_dropout_trains_on_the_gpu(lib):
    """A net built through EDDL's API from the layers above (RandomCropScale, RandomHorizontalFlip, Concat, UpSampling,
    GlobalMaxPool, Dropout) trains on CS_GPU: none of them falls through to a missing-backend stub.  Its random layers draw
    from generators the reference does not share, so the check is that training works (finite, decreasing loss on a fixed
    batch), and that evaluation mode -- where all of them are deterministic -- reproduces itself."""
    from eddl_b200 import harness
    G = harness.load()
    rng = np.random.default_rng(5)
    x = rng.standard_normal((32, 3, 32, 32)).astype(F); y = np.eye(10, dtype=F)[rng.integers(0, 10, 32)]
    net = harness.NetHarness(G, "cifar_da", device=0, optimizer="sgd_fused", lr=0.01, mu=0.9)
    net.set_params(harness.init_weights(net.param_info(), seed=3, mode="he_normal"))
    losses = [net.train_batch(x, y)[0] for _ in range(30)]
    assert np.all(np.isfinite(losses)) and np.mean(losses[-5:]) < np.mean(losses[:5])
    net.close()
