"""Deferred zero fills ("lazy_zero" option of the C ABI): a large fill with 0.0f is only recorded, and the first entry
point that touches the buffer either writes the zeros (reads), drops them (full overwrite) or runs its "destination is
zero" variant (accumulating kernels).  Every result must be bit-identical to the one obtained with immediate fills."""
import ctypes

import numpy as np
import pytest

from oracle import eddl_oracle as orc

pytestmark = pytest.mark.gpu
F = np.float32
N = 1 << 18          # 1 MB of fp32: above the 256 KB deferral threshold


def dev(lib, a):
    return lib.to_device(np.asarray(a, F))


@pytest.fixture()
def lazy(lib):
    lib.call("set_option", b"lazy_zero", 1)
    yield lib
    lib.call("set_option", b"lazy_zero", 0)


def garbage(lib, shape, rng):
    return dev(lib, rng.standard_normal(shape).astype(F) * 100)


def test_deferred_fill_launches_nothing_until_read(lazy):
    lib = lazy
    rng = np.random.default_rng(0)
    d = garbage(lib, (N,), rng)
    before = lib.launches()
    lib.call("fill", 0, d, N, 0.0)
    assert lib.launches() == before                          # recorded, not run
    np.testing.assert_array_equal(d.numpy(), np.zeros(N, F))   # the read writes the zeros first
    assert lib.launches() == before + 1
    small = garbage(lib, (1000,), rng)                        # below the threshold: runs at once
    lib.call("fill", 0, small, 1000, 0.0)
    assert lib.launches() == before + 2
    np.testing.assert_array_equal(small.numpy(), np.zeros(1000, F))
    lib.call("fill", 0, d, N, 1.5)                            # non-zero values are never deferred
    np.testing.assert_array_equal(d.numpy(), np.full(N, 1.5, F))


def test_overwrite_drops_and_partial_access_materialises(lazy):
    lib = lazy
    rng = np.random.default_rng(1)
    d = garbage(lib, (N,), rng)
    lib.call("fill", 0, d, N, 0.0)
    x = rng.standard_normal(N).astype(F)
    before = lib.launches()
    lib.call("memcpy_h2d", 0, d.ptr, x.ctypes.data_as(ctypes.c_void_p), x.nbytes)     # full overwrite: the fill is dropped
    assert lib.launches() == before
    np.testing.assert_array_equal(d.numpy(), x)
    # a kernel that writes only part of a deferred range must find the zeros in the rest
    d2 = garbage(lib, (N,), rng)
    lib.call("fill", 0, d2, N, 0.0)
    a = dev(lib, x[:1000])
    lib.call("scale", 0, a, ctypes.c_void_p(d2.ptr.value + 4 * 500), 2.0, 1000)
    want = np.zeros(N, F); want[500:1500] = x[:1000] * F(2.0)
    np.testing.assert_array_equal(d2.numpy(), want)
    # freeing a buffer forgets its deferred fill; a new tensor at the same address starts clean
    d3 = garbage(lib, (N,), rng)
    lib.call("fill", 0, d3, N, 0.0)
    addr = d3.ptr.value
    del d3
    d4 = dev(lib, x)
    if d4.ptr.value == addr:
        np.testing.assert_array_equal(d4.numpy(), x)
    # switching the option off writes whatever is still deferred
    d5 = garbage(lib, (N,), rng)
    lib.call("fill", 0, d5, N, 0.0)
    lib.call("set_option", b"lazy_zero", 0)
    before = lib.launches()
    np.testing.assert_array_equal(d5.numpy(), np.zeros(N, F))
    assert lib.launches() == before


def test_accumulating_kernels_take_over_the_fill(lazy):
    """relu_bwd, inc, axpby(inc), bn_bwd, max-pool backward and conv backward-data into a deferred-zero destination give
    the bits of the read-modify-write into real zeros, and launch no fill."""
    lib = lazy
    rng = np.random.default_rng(2)
    a, b = rng.standard_normal(N).astype(F), rng.standard_normal(N).astype(F)
    a[::7] = -0.0; a[3::11] = 0.0
    da, db = dev(lib, a), dev(lib, b)
    zero = np.zeros(N, F)

    def fresh():
        d = garbage(lib, (N,), rng)
        lib.call("fill", 0, d, N, 0.0)
        return d

    d = fresh(); before = lib.launches()
    lib.call("relu_bwd", 0, da, db, d, N)
    assert lib.launches() == before + 1
    got = d.numpy(); want = orc.d_relu(a, b, zero)
    np.testing.assert_array_equal(got, want); np.testing.assert_array_equal(np.signbit(got), np.signbit(want))

    d = fresh(); before = lib.launches()
    lib.call("inc", 0, da, d, N)
    assert lib.launches() == before + 1
    got = d.numpy(); want = (zero + a).astype(F)
    np.testing.assert_array_equal(got, want); np.testing.assert_array_equal(np.signbit(got), np.signbit(want))

    d = fresh(); before = lib.launches()
    lib.call("axpby", 0, 0.3, da, -1.7, db, d, 1, N)
    assert lib.launches() == before + 1
    np.testing.assert_array_equal(d.numpy(), orc.axpby(0.3, a, -1.7, b, zero, 1))

    # the second accumulation into the same buffer is an ordinary read-modify-write
    lib.call("inc", 0, da, d, N)
    np.testing.assert_array_equal(d.numpy(), (orc.axpby(0.3, a, -1.7, b, zero, 1) + a).astype(F))

    # LAdd::forward on the GPU: out = 0; out = 1*a + 1*out; out = 1*b + 1*out.  The first add is only recorded, the second
    # runs both in one launch
    d = fresh(); before = lib.launches()
    lib.call("axpby", 0, 1.0, da, 1.0, d, d, 0, N)
    assert lib.launches() == before
    lib.call("axpby", 0, 0.5, db, 2.0, d, d, 0, N)
    assert lib.launches() == before                          # the sum stays on record for one more call ...
    first = orc.axpby(1.0, a, 1.0, zero)
    got = d.numpy(); want = orc.axpby(0.5, b, 2.0, first)    # ... and the read runs both adds in one launch
    assert lib.launches() == before + 1
    np.testing.assert_array_equal(got, want); np.testing.assert_array_equal(np.signbit(got), np.signbit(want))
    # the activation that follows LAdd: the ReLU of a sum still on record writes the sum and its ReLU in ONE launch
    for n_el in (N, N - 3):                                  # 16-byte path and the scalar tail
        d = fresh(); r = garbage(lib, (N,), rng); before = lib.launches()
        lib.call("axpby", 0, 1.0, da, 1.0, d, d, 0, N)
        lib.call("axpby", 0, 1.0, db, 1.0, d, d, 0, N)
        if n_el == N:
            lib.call("relu_fwd", 0, d, r, N)
            assert lib.launches() == before + 1
            want = orc.axpby(1.0, b, 1.0, first)
            np.testing.assert_array_equal(d.numpy(), want)
            np.testing.assert_array_equal(r.numpy(), np.where(want > 0, want, F(0.0)).astype(F))
        else:
            # a ReLU of another length is not the layer that follows: the sum is written first, then the ReLU runs alone
            lib.call("relu_fwd", 0, d, r, n_el)
            assert lib.launches() == before + 2
            want = orc.axpby(1.0, b, 1.0, first)
            np.testing.assert_array_equal(d.numpy(), want)
            np.testing.assert_array_equal(r.numpy()[:n_el], np.where(want > 0, want, F(0.0)).astype(F)[:n_el])
    # LAdd::backward: the same delta is added into the (zero) deltas of both parents -- one launch for both copies
    d = fresh(); d2 = fresh(); before = lib.launches()
    lib.call("axpby", 0, 1.0, da, 1.0, d, d, 0, N)
    lib.call("axpby", 0, 1.0, da, 1.0, d2, d2, 0, N)
    assert lib.launches() == before
    got = d.numpy()
    assert lib.launches() == before + 1
    np.testing.assert_array_equal(got, first); np.testing.assert_array_equal(np.signbit(got), np.signbit(first))
    got = d2.numpy()
    np.testing.assert_array_equal(got, first); np.testing.assert_array_equal(np.signbit(got), np.signbit(first))
    # ... but not when the second copy has another source: two launches
    d = fresh(); d2 = fresh(); before = lib.launches()
    lib.call("axpby", 0, 1.0, da, 1.0, d, d, 0, N)
    lib.call("axpby", 0, 1.0, db, 1.0, d2, d2, 0, N)
    np.testing.assert_array_equal(d.numpy(), first)
    np.testing.assert_array_equal(d2.numpy(), orc.axpby(1.0, b, 1.0, zero))
    assert lib.launches() == before + 2
    # a recorded first term is written out by whatever else comes next: a read of the destination ...
    d = fresh()
    lib.call("axpby", 0, 1.0, da, 1.0, d, d, 0, N)
    np.testing.assert_array_equal(d.numpy(), first)
    # ... or an operation that is about to change the source
    d = fresh(); src = dev(lib, a)
    lib.call("axpby", 0, 1.0, src, 1.0, d, d, 0, N)
    lib.call("scale", 0, src, src, 3.0, N)
    np.testing.assert_array_equal(d.numpy(), first)
    np.testing.assert_array_equal(src.numpy(), (a * F(3.0)).astype(F))


@pytest.mark.parametrize("stride,c", [(1, 32), (2, 32), (1, 3)])
def test_conv_bn_pool_backward_into_deferred_zero(lazy, stride, c):
    """Same results with and without the option for the three big accumulating kernels (stride 2 and the 3-channel case take
    the routes that write the owed zeros first)."""
    lib = lazy
    rng = np.random.default_rng(3 + stride + c)
    n, h, k = 16, 32, 64
    oh = (h + 2 - 3) // stride + 1
    x = rng.standard_normal((n, c, h, h)).astype(F); w = rng.standard_normal((k, c, 3, 3)).astype(F)
    dy = rng.standard_normal((n, k, oh, oh)).astype(F)
    geo = (n, c, h, h, k, 3, 3, oh, oh, stride, stride, 1, 1, 0)
    opa_h = rng.standard_normal(x.shape).astype(F)
    z, rc = c, h * h
    ph = (h - 2) // 2 + 1
    pgeo = (n, c, h, h, ph, ph, 2, 2, 2, 2, 0, 0)
    outs = []
    for lazy_on in (1, 0):
        lib.call("set_option", b"lazy_zero", lazy_on)
        dx = garbage(lib, x.shape, rng); lib.call("fill", 0, dx, dx.size, 0.0)
        lib.call("conv2d_bwd_data", 0, dev(lib, dy), dev(lib, w), dx, *geo)
        # BatchNorm backward into a zeroed parent delta
        delta, opa, pd = dev(lib, x), dev(lib, opa_h), garbage(lib, x.shape, rng)
        lib.call("fill", 0, pd, pd.size, 0.0)
        gg, gb = lib.zeros((z,)), lib.zeros((z,)); g = dev(lib, np.ones(z, F) * 1.5); var = dev(lib, np.ones(z, F) * 0.7)
        m1, m2 = lib.empty((z,)), lib.empty((z,))
        lib.call("bn_bwd", 0, n, z, rc, delta, opa, pd, gg, gb, g, var, m1, m2)
        # max-pool backward into a zeroed input delta (the pooled values double as the incoming delta)
        pin = dev(lib, x); pout, ix, iy = lib.empty((n, c, ph, ph)), lib.empty((n, c, ph, ph)), lib.empty((n, c, ph, ph))
        lib.call("maxpool2d_fwd", 0, pin, pout, ix, iy, *pgeo)
        pid = garbage(lib, x.shape, rng); lib.call("fill", 0, pid, pid.size, 0.0)
        lib.call("maxpool2d_bwd", 0, pout, ix, iy, pid, *pgeo)
        outs.append((dx.numpy(), pd.numpy(), pid.numpy()))
    for got, want in zip(outs[0], outs[1]):
        np.testing.assert_array_equal(got, want)
    lib.sync()
