"""GPU tests of eddlb200_bn_fwd_noalloc, the BatchNorm forward for callers that may not allocate device memory (its
partial sums live in a fixed array inside the library instead of the cudaMalloc'ed scratch arena).  Kept in a file that
pytest collects last, so a run that stops at the first failure has already run every other test.  The entry point is
called through the C ABI twice in a row, with different shapes, and every output is compared bit for bit with
eddlb200_bn_fwd (same kernels, same slicing) and, within the BatchNorm tolerance of the other tests, with the oracle."""
import ctypes
import os
import subprocess
import sys
import textwrap

import numpy as np
import pytest

from oracle import eddl_oracle as orc

pytestmark = pytest.mark.gpu
F = np.float32
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _run(lib, which, x, gm, gv, g, b, stream, trmode=1, relu=True):
    bsz, z = x.shape[:2]; rc = int(np.prod(x.shape[2:]))
    y, opa = lib.zeros(x.shape), lib.zeros(x.shape)
    r = lib.zeros(x.shape) if relu else None
    dgm, dgv, mean, var = lib.to_device(gm), lib.to_device(gv), lib.zeros((z,)), lib.zeros((z,))
    args = [0, bsz, z, rc, lib.to_device(x), y, opa if g is not None else None, dgm, dgv,
            None if g is None else lib.to_device(g), None if g is None else lib.to_device(b), mean, var, trmode, 1e-3, 0.99, r]
    lib.sync(0)
    if which == "noalloc":
        used0, cached0, used1, cached1 = (ctypes.c_size_t() for _ in range(4))
        lib.call("mem_info", 0, ctypes.byref(used0), ctypes.byref(cached0))
        free0 = _free_bytes()
        lib.call("bn_fwd_noalloc", *args, stream)
        lib.call("mem_info", 0, ctypes.byref(used1), ctypes.byref(cached1))
        # nothing was taken from the library's allocator nor from the device
        assert (used1.value, cached1.value) == (used0.value, cached0.value)
        assert _free_bytes() == free0
    else:
        lib.call("bn_fwd", *args)
    lib.sync(0)
    if stream is not None and stream.value:
        _cudart().cudaStreamSynchronize(stream)
    outs = [y, opa, dgm, dgv, mean, var] + ([r] if relu else [])
    return [t.numpy() for t in outs]


_rt = None


def _cudart():
    global _rt
    if _rt is None:
        import glob
        cands = sorted(glob.glob(os.path.join(os.environ.get("CUDA_HOME", "/usr/local/cuda"), "lib64", "libcudart.so*")))
        _rt = ctypes.CDLL(cands[-1])
        _rt.cudaStreamSynchronize.argtypes = [ctypes.c_void_p]
        _rt.cudaStreamCreate.argtypes = [ctypes.POINTER(ctypes.c_void_p)]
        _rt.cudaMemGetInfo.argtypes = [ctypes.POINTER(ctypes.c_size_t), ctypes.POINTER(ctypes.c_size_t)]
    return _rt


def _free_bytes():
    free, total = ctypes.c_size_t(), ctypes.c_size_t()
    assert _cudart().cudaMemGetInfo(ctypes.byref(free), ctypes.byref(total)) == 0
    return free.value


NAMES = ("y", "opa", "running mean", "running var", "mean", "sigma", "relu")


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
        for a, w, name in zip(got, want, NAMES):
            np.testing.assert_array_equal(a, w, err_msg="%s %s" % (name, shape))
        o = orc.bn_fwd(x, gm, gv, g, b, True, 1e-3, 0.99)
        np.testing.assert_allclose(got[0], o["y"], rtol=1e-4, atol=5e-5)
        np.testing.assert_allclose(got[4], o["mean"], rtol=1e-5, atol=1e-6)


def test_bn_fwd_noalloc_inference_and_non_affine_variants(lib):
    stream = ctypes.c_void_p()
    lib.call("stream", 0, ctypes.byref(stream))
    rng = np.random.default_rng(7)
    shape = (16, 40, 9, 9); z = shape[1]
    x = rng.standard_normal(shape).astype(F)
    gm, gv = rng.standard_normal(z).astype(F), (rng.random(z) + 0.5).astype(F)
    g, b = rng.standard_normal(z).astype(F), rng.standard_normal(z).astype(F)
    for trmode, affine in ((0, True), (1, False), (0, False)):
        gg, bb = (g, b) if affine else (None, None)
        want = _run(lib, "bn_fwd", x, gm, gv, gg, bb, stream, trmode=trmode, relu=affine)
        got = _run(lib, "noalloc", x, gm, gv, gg, bb, stream, trmode=trmode, relu=affine)
        for a, w, name in zip(got, want, NAMES):
            if name == "opa" and not affine:
                continue                       # not written without an affine transform
            np.testing.assert_array_equal(a, w, err_msg="%s trmode=%d affine=%s" % (name, trmode, affine))
    # inference needs no partial sums, so a channel count beyond the scratch is accepted there
    zbig = 300000
    xb = rng.standard_normal((1, zbig, 1, 1)).astype(F)
    ones = np.ones(zbig, F)
    got = _run(lib, "noalloc", xb, np.zeros(zbig, F), ones, None, None, stream, trmode=0, relu=False)
    want = _run(lib, "bn_fwd", xb, np.zeros(zbig, F), ones, None, None, stream, trmode=0, relu=False)
    np.testing.assert_array_equal(got[0], want[0])


def test_bn_fwd_noalloc_on_another_stream_with_library_work_outstanding(lib):
    """The caller's stream is not the library's, and the library still owes a deferred zero fill (to a buffer this call reads)
    and a recorded first term of an in-place sum (to a buffer this call never sees): both are settled on the library's
    stream, the caller's stream is ordered behind it, and the results match the plain entry point."""
    other = ctypes.c_void_p()
    assert _cudart().cudaStreamCreate(ctypes.byref(other)) == 0
    rng = np.random.default_rng(11)
    shape = (16, 64, 32, 32); z = shape[1]; n = int(np.prod(shape))
    g, b = rng.standard_normal(z).astype(F), rng.standard_normal(z).astype(F)
    gm, gv = np.zeros(z, F), np.ones(z, F)
    src = rng.standard_normal(shape).astype(F)
    try:
        lib.call("set_option", b"lazy_zero", 1)
        # every buffer first: any other entry point would settle the outstanding work before the call under test
        dx = lib.to_device(rng.standard_normal(shape).astype(F))
        dsrc, dsum = lib.to_device(src), lib.to_device(rng.standard_normal(shape).astype(F))
        y, opa = lib.empty(shape), lib.empty(shape)
        dgm, dgv, mean, var = lib.to_device(gm), lib.to_device(gv), lib.zeros((z,)), lib.zeros((z,))
        dg, db = lib.to_device(g), lib.to_device(b)
        lib.call("fill", 0, dx, n, 0.0)                           # recorded, not run: the input of the BatchNorm below is "zeros"
        lib.call("fill", 0, dsum, n, 0.0)
        lib.call("axpby", 0, 1.0, dsrc, 1.0, dsum, dsum, 0, n)    # recorded first term: dsum = 1*src + 1*0
        lib.call("bn_fwd_noalloc", 0, shape[0], z, shape[2] * shape[3], dx, y, opa, dgm, dgv, dg, db,
                 mean, var, 1, 1e-3, 0.99, None, other)
        assert _cudart().cudaStreamSynchronize(other) == 0
        lib.sync(0)
        # BatchNorm of an all-zero input: y = beta in every position; the unrelated recorded copy was written out
        np.testing.assert_array_equal(y.numpy(), np.broadcast_to(b[None, :, None, None], shape))
        np.testing.assert_array_equal(mean.numpy(), np.zeros(z, F))
        np.testing.assert_array_equal(dsum.numpy(), src)
    finally:
        lib.call("set_option", b"lazy_zero", 0)


def test_bn_fwd_noalloc_first_call_in_a_fresh_process_creates_no_context():
    """A process whose FIRST use of the library is this entry point: it must work without the library's device context
    (no eddlb200_init, no allocation through the library), on memory and a stream the caller made itself, and agree with
    the oracle."""
    code = textwrap.dedent('''
        import ctypes, glob, os, sys
        import numpy as np
        sys.path.insert(0, %r)
        from eddl_b200 import capi
        from oracle import eddl_oracle as orc
        rt = ctypes.CDLL(sorted(glob.glob(os.path.join(os.environ.get("CUDA_HOME", "/usr/local/cuda"), "lib64", "libcudart.so*")))[-1])
        rt.cudaMalloc.argtypes = [ctypes.POINTER(ctypes.c_void_p), ctypes.c_size_t]
        rt.cudaMemcpy.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_size_t, ctypes.c_int]
        rt.cudaStreamCreate.argtypes = [ctypes.POINTER(ctypes.c_void_p)]
        rt.cudaStreamSynchronize.argtypes = [ctypes.c_void_p]
        L = capi.lib()
        F = np.float32
        rng = np.random.default_rng(5)
        shape = (8, 48, 14, 14); z = shape[1]
        x = rng.standard_normal(shape).astype(F); g = rng.standard_normal(z).astype(F); b = rng.standard_normal(z).astype(F)
        def dev(a):
            p = ctypes.c_void_p(); assert rt.cudaMalloc(ctypes.byref(p), a.nbytes) == 0
            assert rt.cudaMemcpy(p, a.ctypes.data_as(ctypes.c_void_p), a.nbytes, 1) == 0
            return p
        def host(p, like):
            out = np.empty_like(like); assert rt.cudaMemcpy(out.ctypes.data_as(ctypes.c_void_p), p, out.nbytes, 2) == 0
            return out
        zeros = np.zeros(z, F)
        dx, dy, dopa = dev(x), dev(np.zeros_like(x)), dev(np.zeros_like(x))
        dgm, dgv, dg, db, dm, dv = dev(zeros), dev(zeros), dev(g), dev(b), dev(zeros), dev(zeros)
        st = ctypes.c_void_p(); assert rt.cudaStreamCreate(ctypes.byref(st)) == 0
        L.call("bn_fwd_noalloc", 0, shape[0], z, shape[2] * shape[3], dx, dy, dopa, dgm, dgv, dg, db, dm, dv, 1, 1e-3, 0.99, None, st)
        assert rt.cudaStreamSynchronize(st) == 0
        want = orc.bn_fwd(x, zeros, zeros, g, b, True, 1e-3, 0.99)
        np.testing.assert_allclose(host(dy, x), want["y"], rtol=1e-4, atol=5e-5)
        np.testing.assert_allclose(host(dm, zeros), want["mean"], rtol=1e-5, atol=1e-6)
        # still no context: the library's allocator has handed out nothing (mem_info would create one, so ask last)
        used, cached = ctypes.c_size_t(), ctypes.c_size_t()
        L.call("mem_info", 0, ctypes.byref(used), ctypes.byref(cached))
        assert used.value == 0 and cached.value == 0
        print("fresh-process ok")
    ''') % ROOT
    r = subprocess.run([sys.executable, "-c", code], capture_output=True, text=True, timeout=600)
    assert r.returncode == 0 and "fresh-process ok" in r.stdout, r.stdout[-2000:] + r.stderr[-4000:]


def test_bn_fwd_noalloc_rejects_shapes_beyond_its_scratch(lib):
    from eddl_b200 import capi
    z = 300000                      # 300000 channels x 1 slice > 262144 pairs
    buf = lib.zeros((z,))
    with pytest.raises(capi.Error) as e:
        lib.call("bn_fwd_noalloc", 0, 1, z, 1, buf, buf, buf, buf, buf, buf, buf, buf, buf, 1, 1e-3, 0.99, None, None)
    assert "-5" in str(e.value) and "scratch" in str(e.value)
