"""TEST INFRASTRUCTURE ONLY: numpy restatement of EDDL v1.1's CPU arithmetic for the convnet
training step.  Only tests, the smoke check and the CPU-baseline leg of the benchmark may
import it; the product path never does.

Every function restates one reference function (path inside the EDDL source tree : lines) in
fp32, operation by operation where the order of roundings is observable.  Pinning: the
restatement is checked (tests/test_oracle.py) against (a) the golden vectors of the
reference's own unit tests (tests/golden/reference_kats.json, extracted by
tests/golden/make_golden.py), and (b) outputs of the reference's own CPU code compiled here
(oracle/_ref, or the committed tests/golden/ref_outputs.npz made from it).  Where the
reference delegates a contraction to Eigen 3.4.0 (conv GEMMs, dense), the summation order is a
property of that third-party library and is not pinned by any reference test beyond atol 1e-3;
contractions here accumulate in float64 and round once, and tests compare with tolerances.
"""
import math

import numpy as np

F = np.float32
EPS_SOFTMAX = F(1.19209e-07)      # CPU_EPS_FLOAT, include/eddl/tensor/tensor.h:57
LOWEST = F(-3.40282e+38)          # CPU_LOWEST_FLOAT, include/eddl/tensor/tensor.h:58
EPS_CCE = F(10e-8)                # cpu_losses.cpp:31


# ---- output size / padding arithmetic: src/descriptors/descriptor_conv2D.cpp:295-360 ----------
def compute_output(padding, input_size, kernel_size, stride, dilation=1):
    if isinstance(padding, str):
        if padding in ("same", "zeros"):
            return int(math.ceil(F(input_size) / F(stride)))
        if padding in ("valid", "none"):
            return int(math.ceil((F(input_size) - (F(kernel_size) - F(1.0)) * F(dilation)) / F(stride)))
        raise ValueError("Incorrect padding type")
    p0, p1 = padding
    return int((F(input_size) - (F(kernel_size) - F(1.0)) * F(dilation) + F(p0) + F(p1) - F(1.0)) / F(stride) + F(1.0))


def compute_padding(output_size, input_size, kernel_size, stride, padding="same", dilation=1):
    if padding in ("same", "zeros"):
        pad = (output_size - 1) * stride + kernel_size - input_size + (dilation - 1) * (kernel_size - 1)
        pad = max(pad, 0)
        return [pad // 2, pad - pad // 2]
    if padding in ("valid", "none"):
        return [0, 0]
    raise ValueError("Incorrect padding type")


def resolve(padding, ih, iw, kr, kc, sr, sc):
    """(oh, ow, (top, bottom, left, right)) as ConvolDescriptor::build / PoolDescriptor::build
    (descriptor_conv2D.cpp:104-139, descriptor_pool2D.cpp:66-87)."""
    if isinstance(padding, str):
        oh, ow = compute_output(padding, ih, kr, sr), compute_output(padding, iw, kc, sc)
        pr_, pc_ = compute_padding(oh, ih, kr, sr, padding), compute_padding(ow, iw, kc, sc, padding)
        return oh, ow, (pr_[0], pr_[1], pc_[0], pc_[1])
    pt, pb, pl, pr = padding
    return compute_output([pt, pb], ih, kr, sr), compute_output([pl, pr], iw, kc, sc), (pt, pb, pl, pr)


# ---- Conv2D: cpu_conv2D / cpu_conv2D_grad / cpu_conv2D_back, src/hardware/cpu/nn/cpu_conv.cpp:114-280,316-527
def _im2col(x, kr, kc, sr, sc, pads, oh, ow):
    n, c, ih, iw = x.shape
    pt, pb, pl, pr = pads
    need_h, need_w = (oh - 1) * sr + kr, (ow - 1) * sc + kc
    xp = np.zeros((n, c, max(need_h, ih + pt), max(need_w, iw + pl)), x.dtype)
    xp[:, :, pt:pt + ih, pl:pl + iw] = x
    s0, s1, s2, s3 = xp.strides
    return np.lib.stride_tricks.as_strided(xp, (n, c, kr, kc, oh, ow), (s0, s1, s2, s3, s2 * sr, s3 * sc), writeable=False)


def conv2d_fwd(x, w, bias=None, stride=(1, 1), padding=(0, 0, 0, 0)):
    """O[n,k,p,q] = sum_{c,r,s} I[n,c,p*sr+r-pt,q*sc+s-pl] K[k,c,r,s] (+ bias[k])  (cpu_conv.cpp:114-226,316-346)"""
    x = np.asarray(x, F); w = np.asarray(w, F)
    k, c, kr, kc = w.shape
    oh, ow, pads = resolve(padding, x.shape[2], x.shape[3], kr, kc, *stride)
    cols = _im2col(x.astype(np.float64), kr, kc, stride[0], stride[1], pads, oh, ow)
    y = np.einsum("ncrspq,kcrs->nkpq", cols, w.astype(np.float64), optimize=True).astype(F)
    if bias is not None:
        y = y + np.asarray(bias, F)[None, :, None, None]
    return y


def conv2d_bwd_weight(x, dy, gw0=None, gbias0=None, stride=(1, 1), padding=(0, 0, 0, 0), kernel=None):
    """gK[k,c,r,s] += sum_{n,p,q} D[n,k,p,q] I[...] ; gbias[k] += sum D   (cpu_conv.cpp:228-251,459-481)"""
    x = np.asarray(x, F); dy = np.asarray(dy, F)
    kr, kc = kernel
    oh, ow, pads = resolve(padding, x.shape[2], x.shape[3], kr, kc, *stride)
    cols = _im2col(x.astype(np.float64), kr, kc, stride[0], stride[1], pads, oh, ow)
    g = np.einsum("ncrspq,nkpq->kcrs", cols, dy.astype(np.float64), optimize=True).astype(F)
    gb = dy.astype(np.float64).sum(axis=(0, 2, 3)).astype(F)
    if gw0 is not None:
        g = np.asarray(gw0, F) + g
    if gbias0 is not None:
        gb = np.asarray(gbias0, F) + gb
    return g, gb


def conv2d_bwd_data(dy, w, x_shape, dx0=None, stride=(1, 1), padding=(0, 0, 0, 0)):
    """ID[n,c,y,x] += sum_{k,r,s} D[n,k,p,q] K[k,c,r,s] at y=p*sr+r-pt, x=q*sc+s-pl  (cpu_conv.cpp:253-280,518-527;
    col2im via add_pixel, :47-58)"""
    dy = np.asarray(dy, F); w = np.asarray(w, F)
    n, c, ih, iw = x_shape
    k, _, kr, kc = w.shape
    oh, ow, pads = resolve(padding, ih, iw, kr, kc, *stride)
    pt, pb, pl, pr = pads
    H, W = max((oh - 1) * stride[0] + kr, ih + pt), max((ow - 1) * stride[1] + kc, iw + pl)
    acc = np.zeros((n, c, H, W), np.float64)
    contrib = np.einsum("nkpq,kcrs->ncrspq", dy.astype(np.float64), w.astype(np.float64), optimize=True)
    for r in range(kr):
        for s in range(kc):
            acc[:, :, r:r + oh * stride[0]:stride[0], s:s + ow * stride[1]:stride[1]] += contrib[:, :, r, s]
    dx = acc[:, :, pt:pt + ih, pl:pl + iw].astype(F)
    return dx if dx0 is None else np.asarray(dx0, F) + dx


def conv2d_samples(x, w, dy, stride, padding, count, seed):
    """float64 values of `count` randomly chosen elements of each of the three conv results, for tensors too large to
    evaluate whole on the host: returns {"y": (flat indices, values), "gw": ..., "dx": ...} with the same index
    arithmetic as conv2d_fwd / conv2d_bwd_weight / conv2d_bwd_data above (cpu_conv.cpp:114-280)."""
    x = np.asarray(x, F); w = np.asarray(w, F); dy = np.asarray(dy, F)
    n, c, ih, iw = x.shape
    k, _, kr, kc = w.shape
    sr, sc = stride
    oh, ow, pads = resolve(padding, ih, iw, kr, kc, sr, sc)
    pt, pl = pads[0], pads[2]
    rng = np.random.default_rng(seed)
    x64 = None

    def patch(img, p, q):          # [c, kr, kc] window of image `img` under output pixel (p, q), zero padded
        out = np.zeros((c, kr, kc), np.float64)
        y0, x0 = p * sr - pt, q * sc - pl
        ya, yb, xa, xb = max(y0, 0), min(y0 + kr, ih), max(x0, 0), min(x0 + kc, iw)
        if ya < yb and xa < xb:
            out[:, ya - y0:yb - y0, xa - x0:xb - x0] = x[img, :, ya:yb, xa:xb]
        return out

    res = {}
    idx = rng.integers(0, n * k * oh * ow, count)
    vals = np.empty(count, np.float64)
    for i, f in enumerate(idx):
        img, kk, p, q = np.unravel_index(f, (n, k, oh, ow))
        vals[i] = np.sum(patch(img, p, q) * w[kk].astype(np.float64))
    res["y"] = (idx, vals)
    idx = rng.integers(0, k * c * kr * kc, count)
    vals = np.empty(count, np.float64)
    for i, f in enumerate(idx):
        kk, cc, r, s = np.unravel_index(f, (k, c, kr, kc))
        # x[n, cc, p*sr + r - pt, q*sc + s - pl] over all (n, p, q) with the tap inside the image
        p_lo = max(0, -(-(pt - r) // sr)); p_hi = min(oh, (ih - 1 + pt - r) // sr + 1)
        q_lo = max(0, -(-(pl - s) // sc)); q_hi = min(ow, (iw - 1 + pl - s) // sc + 1)
        if p_lo >= p_hi or q_lo >= q_hi:
            vals[i] = 0.0
            continue
        xs = x[:, cc, p_lo * sr + r - pt:(p_hi - 1) * sr + r - pt + 1:sr, q_lo * sc + s - pl:(q_hi - 1) * sc + s - pl + 1:sc]
        vals[i] = np.sum(xs.astype(np.float64) * dy[:, kk, p_lo:p_hi, q_lo:q_hi].astype(np.float64))
    res["gw"] = (idx, vals)
    idx = rng.integers(0, n * c * ih * iw, count)
    vals = np.empty(count, np.float64)
    for i, f in enumerate(idx):
        img, cc, yy, xx = np.unravel_index(f, (n, c, ih, iw))
        acc = 0.0
        for r in range(kr):
            pn = yy + pt - r
            if pn % sr or not 0 <= pn // sr < oh:
                continue
            for s in range(kc):
                qn = xx + pl - s
                if qn % sc or not 0 <= qn // sc < ow:
                    continue
                acc += float(np.dot(dy[img, :, pn // sr, qn // sc].astype(np.float64), w[:, cc, r, s].astype(np.float64)))
        vals[i] = acc
    res["dx"] = (idx, vals)
    return res


# ---- pooling: src/hardware/cpu/nn/cpu_pool.cpp:74-145 (max), 226-304 (avg) ---------------------------
def _windows(ih, iw, kr, kc, sr, sc, pads):
    pt, pb, pl, pr = pads
    rows = list(range(-pt, ih + pb - kr + 1, sr))
    cols = list(range(-pl, iw + pr - kc + 1, sc))
    return rows, cols


def maxpool2d_fwd(x, kernel, stride, padding):
    """Row-major window scan, strict '>' from CPU_LOWEST_FLOAT, out-of-bounds = lowest (get_pixel, :20-31);
    indX/indY = absolute input column/row stored as floats (:93-97)."""
    x = np.asarray(x, F); n, c, ih, iw = x.shape
    kr, kc = kernel; sr, sc = stride
    oh, ow, pads = resolve(padding, ih, iw, kr, kc, sr, sc)
    rows, cols = _windows(ih, iw, kr, kc, sr, sc, pads)
    assert len(rows) == oh and len(cols) == ow, "window count differs from compute_output"
    y = np.full((n, c, oh, ow), LOWEST, F); ix = np.zeros((n, c, oh, ow), F); iy = np.zeros((n, c, oh, ow), F)
    for a, i in enumerate(rows):
        for b, j in enumerate(cols):
            m = np.full((n, c), LOWEST, F); bx = np.zeros((n, c), F); by = np.zeros((n, c), F)
            for ki in range(kr):
                for kj in range(kc):
                    py, px = i + ki, j + kj
                    if 0 <= py < ih and 0 <= px < iw:
                        v = x[:, :, py, px]
                        better = v > m
                        m = np.where(better, v, m); bx = np.where(better, F(px), bx); by = np.where(better, F(py), by)
            y[:, :, a, b] = m; ix[:, :, a, b] = bx; iy[:, :, a, b] = by
    return y, ix, iy


def maxpool2d_bwd(dy, ix, iy, x_shape, dx0=None):
    """ID[n,c,indY,indX] += D, outputs visited in row-major order (cpu_pool.cpp:122-145)."""
    dy = np.asarray(dy, F)
    n, c, ih, iw = x_shape
    dx = np.zeros(x_shape, F) if dx0 is None else np.asarray(dx0, F).copy()
    oh, ow = dy.shape[2:]
    nn, cc = np.meshgrid(np.arange(n), np.arange(c), indexing="ij")
    for a in range(oh):
        for b in range(ow):
            xs = ix[:, :, a, b].astype(np.int64); ys = iy[:, :, a, b].astype(np.int64)
            ok = (xs >= 0) & (ys >= 0) & (xs < iw) & (ys < ih)
            np.add.at(dx, (nn[ok], cc[ok], ys[ok], xs[ok]), dy[:, :, a, b][ok])
    return dx


def avgpool2d_fwd(x, kernel, stride, padding):
    """Sum of in-bounds values divided by the FULL window size kr*kc (cpu_pool.cpp:226-266)."""
    x = np.asarray(x, F); n, c, ih, iw = x.shape
    kr, kc = kernel; sr, sc = stride
    oh, ow, pads = resolve(padding, ih, iw, kr, kc, sr, sc)
    rows, cols = _windows(ih, iw, kr, kc, sr, sc, pads)
    y = np.zeros((n, c, oh, ow), F)
    for a, i in enumerate(rows):
        for b, j in enumerate(cols):
            s = np.zeros((n, c), F)
            for ki in range(kr):
                for kj in range(kc):
                    py, px = i + ki, j + kj
                    if 0 <= py < ih and 0 <= px < iw:
                        s = s + x[:, :, py, px]
            y[:, :, a, b] = s / F(kr * kc)
    return y


def avgpool2d_bwd(dy, x_shape, kernel, stride, padding, dx0=None):
    """ID += D/(kr*kc) at every in-bounds window position (cpu_pool.cpp:268-304)."""
    dy = np.asarray(dy, F); n, c, ih, iw = x_shape
    kr, kc = kernel; sr, sc = stride
    oh, ow, pads = resolve(padding, ih, iw, kr, kc, sr, sc)
    rows, cols = _windows(ih, iw, kr, kc, sr, sc, pads)
    dx = np.zeros(x_shape, F) if dx0 is None else np.asarray(dx0, F).copy()
    for a, i in enumerate(rows):
        for b, j in enumerate(cols):
            v = dy[:, :, a, b] / F(kr * kc)
            for ki in range(kr):
                for kj in range(kc):
                    py, px = i + ki, j + kj
                    if 0 <= py < ih and 0 <= px < iw:
                        dx[:, :, py, px] = dx[:, :, py, px] + v
    return dx


# ---- BatchNorm: src/hardware/cpu/nn/cpu_bn.cpp:118-249 ---------------------------------------------------
def bn_fwd(x, global_mean, global_var, g, b, trmode, eps, momentum):
    """Training: mean = sum/N, var = sumsq/N - mean^2 (one pass, biased); running stats
    g = momentum*g + (1.0-momentum)*batch (the second product in double) unless momentum == 0;
    `var` then holds sqrt(var+eps); opa = (x-mean)/var; y = opa*g + b.  The reference sums
    sequentially in fp32; sums here are float64 rounded once (closer to the exact value)."""
    x = np.asarray(x, F); bsz, z = x.shape[:2]
    xr = x.reshape(bsz, z, -1); N = F(bsz * xr.shape[2])
    gm, gv = np.asarray(global_mean, F).copy(), np.asarray(global_var, F).copy()
    if trmode:
        s = xr.astype(np.float64).sum(axis=(0, 2)).astype(F)
        sq = (xr.astype(np.float64) ** 2).sum(axis=(0, 2)).astype(F)
        mean = s / N
        var = sq / N - mean * mean
        if momentum != 0.0:
            keep = 1.0 - float(F(momentum))
            gm = ((F(momentum) * gm).astype(np.float64) + keep * mean.astype(np.float64)).astype(F)
            gv = ((F(momentum) * gv).astype(np.float64) + keep * var.astype(np.float64)).astype(F)
        sigma = np.sqrt(var + F(eps)).astype(F)
        mean_out = mean
    else:
        mean = gm; mean_out = None
        sigma = np.sqrt(gv + F(eps)).astype(F)
    opa = ((xr - mean[None, :, None]) / sigma[None, :, None]).astype(F)
    y = opa if g is None else (opa * np.asarray(g, F)[None, :, None] + np.asarray(b, F)[None, :, None]).astype(F)
    return dict(y=y.reshape(x.shape), opa=opa.reshape(x.shape), gmean=gm, gvar=gv, mean=mean_out, var=sigma)


def bn_bwd(delta, opa, pdelta0, gg0, gb0, g, sigma):
    """m1 = sum(delta*opa)/N, m2 = sum(delta)/N; gg += m1, gb += m2 (MEANS); delta *= g in place;
    m1, m2 *= g; pdelta += (delta - (opa*m1 + m2)) / sigma."""
    delta = np.asarray(delta, F); opa = np.asarray(opa, F); bsz, z = delta.shape[:2]
    dr, orr = delta.reshape(bsz, z, -1), opa.reshape(bsz, z, -1); N = F(bsz * dr.shape[2])
    m1 = ((dr.astype(np.float64) * orr.astype(np.float64)).sum(axis=(0, 2)).astype(F)) / N
    m2 = (dr.astype(np.float64).sum(axis=(0, 2)).astype(F)) / N
    gg = gb = None
    if g is not None:
        g = np.asarray(g, F)
        gg = np.asarray(gg0, F) + m1; gb = np.asarray(gb0, F) + m2
        dr = (dr * g[None, :, None]).astype(F)
        m1 = m1 * g; m2 = m2 * g
    sig = np.asarray(sigma, F)
    t = (orr * m1[None, :, None]).astype(F) + m2[None, :, None]
    pd = np.asarray(pdelta0, F).reshape(bsz, z, -1) + ((dr - t) / sig[None, :, None]).astype(F)
    return dict(delta=dr.reshape(delta.shape), pdelta=pd.reshape(delta.shape).astype(F), gg=gg, gb=gb, m1=m1, m2=m2)


# ---- activations: src/hardware/cpu/nn/cpu_activations.cpp:20-45, 329-436 ---------------------------------------
def relu(a):
    a = np.asarray(a, F); return np.where(a > 0, a, F(0)).astype(F)


def d_relu(d, i, pd0):
    return (np.asarray(pd0, F) + np.where(np.asarray(i, F) > 0, np.asarray(d, F), F(0))).astype(F)


def softmax(a):
    """Stable softmax over the last axis, denominator initialised to CPU_EPS_FLOAT (:352-364)."""
    a = np.asarray(a, F)
    e = np.exp((a - a.max(axis=-1, keepdims=True)).astype(F)).astype(F)
    den = (EPS_SOFTMAX + e.astype(np.float64).sum(axis=-1, keepdims=True)).astype(F)
    return (e / den).astype(F)


def d_softmax(d, s, pd0):
    """PD[i] += sum_j D[j]*(S[i]*[i==j] - S[j]*S[i])  (:410-436)"""
    d = np.asarray(d, np.float64); s = np.asarray(s, np.float64)
    dot = (d * s).sum(axis=-1, keepdims=True)
    return (np.asarray(pd0, F) + (s * (d - dot)).astype(F)).astype(F)


# ---- losses / metrics: cpu_losses.cpp:29-57, cpu_metrics.cpp:17-29 ------------------------------------------------
def cce_value(y, p):
    """-sum_batch sum_c y*logf(p + 1e-7): a SUM, not a mean."""
    y = np.asarray(y, F); p = np.asarray(p, F)
    return F(-(y.astype(np.float64) * np.log((p + EPS_CCE).astype(F)).astype(np.float64)).sum())


def cce_delta(y, p):
    return (-np.asarray(y, F) * (F(1.0) / (np.asarray(p, F) + EPS_CCE))).astype(F)


def accuracy(y, p):
    return int((np.argmax(np.asarray(y), axis=1) == np.argmax(np.asarray(p), axis=1)).sum())


# ---- elementwise / dense: cpu_math.cpp:278-325, 369-380; cpu_reduction.cpp:91-112; cpu_da.cpp:502-534 ---------------
def axpby(sca, a, scb, b, c0=None, inc=0):
    r = (F(sca) * np.asarray(a, F) + F(scb) * np.asarray(b, F)).astype(F)
    return (np.asarray(c0, F) + r).astype(F) if inc else r


def mult2d(a, ta, b, tb, c0=None, inc=0):
    A = np.asarray(a, np.float64); B = np.asarray(b, np.float64)
    r = ((A.T if ta else A) @ (B.T if tb else B)).astype(F)
    return (np.asarray(c0, F) + r).astype(F) if inc else r


def sum2d_rowwise(a, b):
    return (np.asarray(a, F) + np.asarray(b, F)[None, :]).astype(F)


def reduce_sum2d(a, axis, b0=None, inc=0):
    """Sequential fp32 accumulation in row order (the order is observable in fp32)."""
    a = np.asarray(a, F)
    acc = (np.asarray(b0, F).copy() if inc else np.zeros(a.shape[1] if axis == 0 else a.shape[0], F))
    if axis == 0:
        for i in range(a.shape[0]):
            acc = (acc + a[i]).astype(F)
    else:
        acc = (acc + a.astype(np.float64).sum(axis=1).astype(F)).astype(F)
    return acc


def pad(a, pads):
    """pads = (top, right, bottom, left); the output is pre-filled (zeros) by the layer."""
    a = np.asarray(a, F); t, r, bo, l = pads
    return np.pad(a, ((0, 0), (0, 0), (t, bo), (l, r)))


def pad_back(a_delta0, b_delta, pads):
    t, r, bo, l = pads; h, w = a_delta0.shape[2:]
    return (np.asarray(a_delta0, F) + np.asarray(b_delta, F)[:, :, t:t + h, l:l + w]).astype(F)


# ---- optimizers: src/optimizers/optim_sgd.cpp:68-89, optim_adam.cpp:85-120 -----------------------------------------
def sgd_step(p, g, m, lr, mu):
    """m = lr*g + mu*m ; p = 1.0*p + (-1.0)*m   (weight_decay and nesterov are never read)."""
    m = (F(lr) * np.asarray(g, F) + F(mu) * np.asarray(m, F)).astype(F)
    return (np.asarray(p, F) - m).astype(F), m


def adam_step(p, g, m, v, lr, b1, b2, eps, t):
    """t is the step count after the increment.  g is squared in place; eps sits inside the sqrt;
    div_(x) multiplies by the float reciprocal (src/tensor/tensor_math.cpp:1186-1188)."""
    b1f, b2f = F(b1), F(b2)
    m = (b1f * np.asarray(m, F) + (F(1) - b1f) * np.asarray(g, F)).astype(F)
    g2 = (np.asarray(g, F) * np.asarray(g, F)).astype(F)
    v = (b2f * np.asarray(v, F) + (F(1) - b2f) * g2).astype(F)
    d1 = F(1.0 - float(b1f) ** t); d2 = F(1.0 - float(b2f) ** t)
    mcap = (m * (F(1.0) / d1)).astype(F)
    vcap = np.sqrt(((v * (F(1.0) / d2)).astype(F) + F(eps)).astype(F)).astype(F)
    p = (F(-lr) * (mcap / vcap).astype(F) + np.asarray(p, F)).astype(F)
    return p, g2, m, v


# ---- Net::sync_weights: src/net/net_func.cpp:111-127 ------------------------------------------------------------------
def sync_weights(reps):
    """acc = 0; acc += w_i in replica order (fp32); acc *= 1.0f/N."""
    reps = np.asarray(reps, F)
    acc = np.zeros(reps.shape[1:], F)
    for r in reps:
        acc = (acc + r).astype(F)
    return (acc * (F(1.0) / F(reps.shape[0]))).astype(F)


# ---- Concat / UpSampling / flips and crops: cpu_core.cpp:368-396, nn/cpu_tensor_nn.cpp:13-50, cpu_da.cpp:315-336, 363-384 -----
def concat(parts, axis):
    return np.concatenate([np.asarray(p, F) for p in parts], axis=axis)


def concat_back(a_delta, parts0, axis):
    """part_i += its slice of a_delta (cpu_concat with derivative = true)."""
    out, pos = [], 0
    for p in parts0:
        n = p.shape[axis]
        sl = [slice(None)] * a_delta.ndim; sl[axis] = slice(pos, pos + n)
        out.append(np.asarray(p, F) + np.asarray(a_delta, F)[tuple(sl)]); pos += n
    return out


def repeat_nn(a, size):
    return np.repeat(np.repeat(np.asarray(a, F), size[0], axis=2), size[1], axis=3)


def d_repeat_nn(d, a0, size):
    """A[row, col] += every value of its block of D, one by one in row-major order of the block (fp32 adds)."""
    a = np.asarray(a0, F).copy(); d = np.asarray(d, F)
    for r in range(size[0]):
        for c in range(size[1]):
            a = (a + d[:, :, r::size[0], c::size[1]]).astype(F)
    return a


def _scale_src(b, off, n_new, a_extent, mode):
    """Source index of output index b: cpu_single_scale's float arithmetic, truncated to int (cpu_da.cpp:95-116)."""
    a = (np.asarray(b, np.int64) + off).astype(F)
    if mode == 0:
        s = F(n_new) / F(a_extent); v = (a + F(0.5)) / s - F(0.5)
    elif mode == 2:
        s = F(n_new - 1) / F(a_extent - 1); v = a / s
    else:
        s = F(n_new) / F(a_extent); v = a / s
    return np.trunc(v.astype(F)).astype(np.int64)


def scale(a, out_hw, new_shape, mode=3, wrap=0, cval=0.0):
    """Nearest-neighbour resize (cpu_scale -> cpu_single_scale, cpu_da.cpp:88-138, 407-437)."""
    a = np.asarray(a, F); bh, bw = out_hw
    off_y, off_x = int((new_shape[0] - bh) / 2.0), int((new_shape[1] - bw) / 2.0)
    ai = _scale_src(np.arange(bh), off_y, new_shape[0], a.shape[2], mode); aj = _scale_src(np.arange(bw), off_x, new_shape[1], a.shape[3], mode)
    oki = (ai >= 0) & (ai < a.shape[2]); okj = (aj >= 0) & (aj < a.shape[3])
    b = a[:, :, np.clip(ai, 0, a.shape[2] - 1)][:, :, :, np.clip(aj, 0, a.shape[3] - 1)].copy()
    outside = ~(oki[:, None] & okj[None, :])
    if outside.any():
        if wrap == 5:
            b[:, :, outside] = a[:, :, outside]
        else:
            b[:, :, outside] = F(cval)
    return b


def scale_back(a_delta0, b_delta, new_shape, mode=3):
    """A[ai][aj] += B[bi][bj] for every output element, visited in row-major order (cpu_single_scale_back, cpu_da.cpp:140-190)."""
    a = np.asarray(a_delta0, F).copy(); b = np.asarray(b_delta, F); bh, bw = b.shape[2:]
    off_y, off_x = int((new_shape[0] - bh) / 2.0), int((new_shape[1] - bw) / 2.0)
    ai = _scale_src(np.arange(bh), off_y, new_shape[0], a.shape[2], mode); aj = _scale_src(np.arange(bw), off_x, new_shape[1], a.shape[3], mode)
    for i in range(bh):
        for j in range(bw):
            if 0 <= ai[i] < a.shape[2] and 0 <= aj[j] < a.shape[3]:
                a[:, :, ai[i], aj[j]] = (a[:, :, ai[i], aj[j]] + b[:, :, i, j]).astype(F)
    return a


def flip_batch(a, apply, axis):
    a = np.asarray(a, F); b = a.copy()
    for i, ap in enumerate(apply):
        if ap:
            b[i] = a[i, :, ::-1, :] if axis == 0 else a[i, :, :, ::-1]
    return b


def crop_scale_batch(a, boxes, out_hw):
    """B[n,c,i,j] = A[n,c, i*(y1-y0+1)//BH + y0, j*(x1-x0+1)//BW + x0]  (integer arithmetic of cpu_single_crop_scale)."""
    a = np.asarray(a, F); bh, bw = out_hw
    b = np.empty(a.shape[:2] + (bh, bw), F)
    for n, (y0, x0, y1, x1) in enumerate(boxes):
        ai = (np.arange(bh) * (y1 - y0 + 1)) // bh + y0
        aj = (np.arange(bw) * (x1 - x0 + 1)) // bw + x0
        b[n] = a[n][:, ai][:, :, aj]
    return b
