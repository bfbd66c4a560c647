"""TEST INFRASTRUCTURE ONLY: Python binding of ``oracle/_ref/libeddl_ref_cpu.so``.

That library is EDDL v1.1's own CPU implementation compiled in place (``oracle/build_ref.py``)
plus the thin C wrappers of ``oracle/ref_capi.cpp``.  Tests use it as the parity checker and
``bench.py`` times it as the CPU baseline; nothing in the product path may import this module.
"""
import ctypes
import os

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
LIBPATH = os.path.join(HERE, "_ref", "libeddl_ref_cpu.so")

_lib = None


def available():
    return os.path.exists(LIBPATH)


def lib():
    global _lib
    if _lib is None:
        _lib = ctypes.CDLL(LIBPATH)
        _lib.ref_last_error.restype = ctypes.c_char_p
        _lib.ebh_last_error.restype = ctypes.c_char_p
    return _lib


def _p(a):
    return None if a is None else a.ctypes.data_as(ctypes.c_void_p)


def _f(a):
    return np.ascontiguousarray(a, dtype=np.float32)


def _ck(st):
    if st != 0:
        raise RuntimeError("reference: " + lib().ref_last_error().decode())


def conv_out_shape(ih, iw, kr, kc, sr, sc, pads):
    oh, ow = ctypes.c_int(), ctypes.c_int()
    _ck(lib().ref_conv2d_out_shape(ih, iw, kr, kc, sr, sc, *pads, ctypes.byref(oh), ctypes.byref(ow)))
    return oh.value, ow.value


def conv2d(x, w, bias=None, dy=None, gw0=None, gbias0=None, dx0=None, stride=(1, 1), pads=(0, 0, 0, 0)):
    """Returns (y, gw, gbias, dx); backward outputs are None unless dy is given.  gw0/gbias0/dx0 are the
    values accumulated into (default zeros).  pads = (top, bottom, left, right)."""
    x, w = _f(x), _f(w)
    n, c, ih, iw = x.shape; k, _, kr, kc = w.shape
    oh, ow = conv_out_shape(ih, iw, kr, kc, stride[0], stride[1], pads)
    y = np.empty((n, k, oh, ow), np.float32)
    gw = gb = dx = None
    if dy is not None:
        dy = _f(dy)
        gw = np.zeros_like(w) if gw0 is None else _f(gw0).copy()
        gb = None if bias is None else (np.zeros(k, np.float32) if gbias0 is None else _f(gbias0).copy())
        dx = np.zeros_like(x) if dx0 is None else _f(dx0).copy()
    b = None if bias is None else _f(bias)
    _ck(lib().ref_conv2d(_p(x), _p(w), _p(b), _p(y), _p(dy), _p(gw), _p(gb), _p(dx), n, c, ih, iw, k, kr, kc,
                         stride[0], stride[1], *pads))
    return y, gw, gb, dx


def pool2d(is_max, x, kernel, stride, pads, dy=None, dx0=None):
    x = _f(x); n, c, ih, iw = x.shape
    oh, ow = ctypes.c_int(), ctypes.c_int()
    args = (n, c, ih, iw, kernel[0], kernel[1], stride[0], stride[1], *pads)
    _ck(lib().ref_pool2d(int(is_max), _p(x), None, None, None, None, None, *args, ctypes.byref(oh), ctypes.byref(ow)))
    y = np.empty((n, c, oh.value, ow.value), np.float32)
    ix, iy = np.zeros_like(y), np.zeros_like(y)
    dx = None
    if dy is not None:
        dy = _f(dy); dx = np.zeros_like(x) if dx0 is None else _f(dx0).copy()
    _ck(lib().ref_pool2d(int(is_max), _p(x), _p(y), _p(ix), _p(iy), _p(dy), _p(dx), *args, None, None))
    return y, ix, iy, dx


def bn_fwd(x, gmean, gvar, g, b, trmode, eps, momentum):
    """x [b,z,rc...]; returns dict(y, opa, gmean, gvar, mean, var)."""
    x = _f(x); bsz, z = x.shape[0], x.shape[1]; rc = int(np.prod(x.shape[2:])) if x.ndim > 2 else 1
    y, opa = np.zeros_like(x), np.zeros_like(x)
    gm, gv = _f(gmean).copy(), _f(gvar).copy()
    mean, var = np.zeros(z, np.float32), np.zeros(z, np.float32)
    gg = None if g is None else _f(g); bb = None if b is None else _f(b)
    _ck(lib().ref_bn_fwd(bsz, z, rc, _p(x), _p(y), _p(opa), _p(gm), _p(gv), _p(gg), _p(bb), _p(mean), _p(var), int(trmode),
                         ctypes.c_float(eps), ctypes.c_float(momentum)))
    return dict(y=y, opa=opa, gmean=gm, gvar=gv, mean=mean, var=var)


def bn_bwd(delta, opa, pdelta0, gg0, gb0, g, var):
    delta = _f(delta).copy(); opa = _f(opa); bsz, z = delta.shape[0], delta.shape[1]
    rc = int(np.prod(delta.shape[2:])) if delta.ndim > 2 else 1
    pd = _f(pdelta0).copy()
    gg = None if g is None else _f(gg0).copy(); gb = None if g is None else _f(gb0).copy()
    gw = None if g is None else _f(g)
    m1, m2 = np.zeros(z, np.float32), np.zeros(z, np.float32)
    _ck(lib().ref_bn_bwd(bsz, z, rc, _p(delta), _p(opa), _p(pd), _p(gg), _p(gb), _p(gw), _p(_f(var)), _p(m1), _p(m2)))
    return dict(delta=delta, pdelta=pd, gg=gg, gb=gb, m1=m1, m2=m2)


def relu(a):
    a = _f(a); b = np.empty_like(a); _ck(lib().ref_relu(_p(a), _p(b), ctypes.c_longlong(a.size))); return b


def d_relu(d, i, pd0):
    pd = _f(pd0).copy(); _ck(lib().ref_d_relu(_p(_f(d)), _p(_f(i)), _p(pd), ctypes.c_longlong(pd.size))); return pd


def softmax(a):
    a = _f(a); b = np.empty_like(a); _ck(lib().ref_softmax(_p(a), _p(b), a.shape[0], a.shape[1])); return b


def d_softmax(d, s, pd0):
    pd = _f(pd0).copy(); _ck(lib().ref_d_softmax(_p(_f(d)), _p(_f(s)), _p(pd), pd.shape[0], pd.shape[1])); return pd


def cce(y, p):
    y, p = _f(y), _f(p); v = ctypes.c_float(); delta = np.empty_like(y)
    _ck(lib().ref_cce(_p(y), _p(p), y.shape[0], y.shape[1], ctypes.byref(v), _p(delta)))
    return v.value, delta


def accuracy(y, p):
    y, p = _f(y), _f(p); a = ctypes.c_int()
    _ck(lib().ref_accuracy(_p(y), _p(p), y.shape[0], y.shape[1], ctypes.byref(a))); return a.value


def axpby(sca, a, scb, b, c0=None, inc=0):
    a, b = _f(a), _f(b); c = np.zeros_like(a) if c0 is None else _f(c0).copy()
    _ck(lib().ref_axpby(ctypes.c_float(sca), _p(a), ctypes.c_float(scb), _p(b), _p(c), inc, ctypes.c_longlong(a.size))); return c


def mult2d(a, ta, b, tb, c0=None, inc=0):
    a, b = _f(a), _f(b)
    m = a.shape[1] if ta else a.shape[0]; k = a.shape[0] if ta else a.shape[1]; n = b.shape[0] if tb else b.shape[1]
    c = np.zeros((m, n), np.float32) if c0 is None else _f(c0).copy()
    _ck(lib().ref_mult2d(_p(a), ta, _p(b), tb, _p(c), inc, m, n, k)); return c


def sum2d_rowwise(a, b):
    a, b = _f(a), _f(b); c = np.empty_like(a); _ck(lib().ref_sum2d_rowwise(_p(a), _p(b), _p(c), a.shape[0], a.shape[1])); return c


def reduce_sum2d(a, axis, b0=None, inc=0):
    a = _f(a); b = np.zeros(a.shape[1] if axis == 0 else a.shape[0], np.float32) if b0 is None else _f(b0).copy()
    _ck(lib().ref_reduce_sum2d(_p(a), _p(b), a.shape[0], a.shape[1], axis, inc)); return b


def pad(a, pads):
    """pads = (top, right, bottom, left) as LPad."""
    a = _f(a); n, c, h, w = a.shape; t, r, bo, l = pads
    b = np.zeros((n, c, h + t + bo, w + l + r), np.float32)
    _ck(lib().ref_pad(_p(a), _p(b), None, None, n, c, h, w, t, r, bo, l)); return b


def pad_back(a_delta0, b_delta, pads):
    ad = _f(a_delta0).copy(); n, c, h, w = ad.shape; t, r, bo, l = pads
    _ck(lib().ref_pad(None, None, _p(ad), _p(_f(b_delta)), n, c, h, w, t, r, bo, l)); return ad


def sgd_step(p, g, m, lr, mu):
    p, m = _f(p).copy(), _f(m).copy()
    _ck(lib().ref_sgd_step(_p(p), _p(_f(g)), _p(m), ctypes.c_float(lr), ctypes.c_float(mu), ctypes.c_longlong(p.size))); return p, m


def adam_step(p, g, m, v, lr, b1, b2, eps, t):
    p, g, m, v = _f(p).copy(), _f(g).copy(), _f(m).copy(), _f(v).copy()
    _ck(lib().ref_adam_step(_p(p), _p(g), _p(m), _p(v), ctypes.c_float(lr), ctypes.c_float(b1), ctypes.c_float(b2),
                            ctypes.c_float(eps), t, ctypes.c_longlong(p.size)))
    return p, g, m, v


def sync_weights(reps):
    reps = _f(reps); out = np.empty(reps.shape[1], np.float32)
    _ck(lib().ref_sync_weights(_p(reps), reps.shape[0], _p(out), ctypes.c_longlong(reps.shape[1]))); return out


def set_threads(n):
    """OpenMP threads for the reference's CPU loops (0 = all cores).  Use 1 for reproducible BatchNorm sums."""
    lib().ref_set_omp_threads(int(n))
