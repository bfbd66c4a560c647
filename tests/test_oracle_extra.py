"""CPU: the numpy restatement of Concat, UpSampling, flip and crop-scale agrees bit for bit with the reference's own CPU code
(oracle/_ref) -- the reference's unit tests hold no vectors for these through the layer path, so the restatement is pinned
to the reference's execution."""
import ctypes

import numpy as np
import pytest

from oracle import eddl_oracle as orc

F = np.float32


def _p(a):
    return a.ctypes.data_as(ctypes.c_void_p)


def test_extra_layer_restatements_match_the_reference(ref):
    if ref is None:
        pytest.skip("oracle/_ref not built")
    L = ref.lib()
    if not hasattr(L, "ref_concat2"):
        pytest.skip("oracle/_ref predates these wrappers")
    rng = np.random.default_rng(0)
    n, c0, c1, h, w = 3, 4, 5, 6, 7
    p0 = rng.standard_normal((n, c0, h, w)).astype(F); p1 = rng.standard_normal((n, c1, h, w)).astype(F)
    a = np.zeros((n, c0 + c1, h, w), F)
    assert L.ref_concat2(_p(a), _p(p0), _p(p1), n, c0, c1, h, w, 0) == 0
    np.testing.assert_array_equal(a, orc.concat([p0, p1], 1))
    d = rng.standard_normal(a.shape).astype(F); q0, q1 = p0.copy(), p1.copy()
    assert L.ref_concat2(_p(d), _p(q0), _p(q1), n, c0, c1, h, w, 1) == 0
    w0, w1 = orc.concat_back(d, [p0, p1], 1)
    np.testing.assert_array_equal(q0, w0); np.testing.assert_array_equal(q1, w1)

    x = rng.standard_normal((2, 3, 4, 5)).astype(F); b = np.zeros((2, 3, 8, 15), F)
    ad = rng.standard_normal(x.shape).astype(F); ad0 = ad.copy(); bd = rng.standard_normal(b.shape).astype(F)
    assert L.ref_repeat_nn(_p(x), _p(b), _p(ad), _p(bd), 2, 3, 4, 5, 2, 3) == 0
    np.testing.assert_array_equal(b, orc.repeat_nn(x, (2, 3)))
    np.testing.assert_array_equal(ad, orc.d_repeat_nn(bd, ad0, (2, 3)))

    # resize: whole-factor upsampling (eddl::UpSampling2D), a ragged zoom, a zoom-out with constant fill, half-pixel mode
    for (ah, aw, bh, bw, nh, nw, wrap, mode) in ((4, 5, 8, 15, 8, 15, 2, 3), (7, 7, 10, 13, 10, 13, 0, 3), (10, 10, 10, 10, 6, 6, 0, 3),
                                                 (5, 6, 11, 9, 11, 9, 0, 0)):
        x = rng.standard_normal((2, 3, ah, aw)).astype(F); b = np.zeros((2, 3, bh, bw), F)
        ad = rng.standard_normal(x.shape).astype(F); ad0 = ad.copy(); bd = rng.standard_normal(b.shape).astype(F)
        assert L.ref_scale(_p(x), _p(b), _p(ad), _p(bd), 2, 3, ah, aw, bh, bw, nh, nw, wrap, ctypes.c_float(1.5), mode) == 0
        np.testing.assert_array_equal(b, orc.scale(x, (bh, bw), (nh, nw), mode, wrap, 1.5))
        np.testing.assert_array_equal(ad, orc.scale_back(ad0, bd, (nh, nw), mode))

    x = rng.standard_normal((4, 2, 6, 7)).astype(F); ap = np.array([1, 0, 1, 1], np.uint8)
    for axis in (0, 1):
        b = np.zeros_like(x)
        assert L.ref_flip_batch(_p(x), _p(b), 4, 2, 6, 7, axis, _p(ap)) == 0
        np.testing.assert_array_equal(b, orc.flip_batch(x, ap, axis))
    boxes = np.array([[0, 0, 5, 6], [1, 2, 4, 5], [2, 1, 5, 4], [0, 3, 3, 6]], np.int32); b = np.zeros((4, 2, 6, 7), F)
    assert L.ref_crop_scale_batch(_p(x), _p(b), 4, 2, 6, 7, 6, 7, _p(boxes)) == 0
    np.testing.assert_array_equal(b, orc.crop_scale_batch(x, boxes, (6, 7)))
