"""Kernel microbenchmarks through the C ABI (CUDA-event timed, L2 flushed between timed launches).

    python -m eddl_b200.microbench conv [--precision 0|1|2] [--batch-scale 1.0] [--iters 5]
    python -m eddl_b200.microbench hbm
    python -m eddl_b200.microbench allreduce          (under torchrun for N > 1)
    python -m eddl_b200.microbench step [--net resnet50] [--batch 64] [--steps 1]

conv      forward / backward-data / backward-weight at the four Conv2D microbenchmark shapes (--set resnet: ResNet-50's layers)
          (N=64 C=K=256 56x56 3x3; N=64 C=1024 K=256 14x14 1x1; N=64 C=3 K=64 224x224 7x7 s2 p3; N=32 C=K=512 7x7 3x3),
          TFLOP/s = 2*N*K*C*kr*kc*P*Q / time.
hbm       BatchNorm forward/backward, ReLU forward/backward, max-pool, axpby, fused SGD at ResNet-50 sizes,
          GB/s = algorithmic bytes / time.
allreduce parameter averaging over NCCL for 1 KB ... 1 GB buffers: algbw = S/t, busbw = algbw * 2(N-1)/N.
step      builds the net through the drop-in library, runs one train_batch on host buffers and then --steps steps
          with the batch resident in HBM, and exits: the short program to put under a profiler's launch list.
Each line of output is one JSON object.
"""
import argparse
import ctypes
import json
import os
import sys

import numpy as np

CONV_SHAPES = [  # n, c, h, w, k, kr, kc, stride, pad
    (64, 256, 56, 56, 256, 3, 3, 1, 1),
    (64, 1024, 14, 14, 256, 1, 1, 1, 0),
    (64, 3, 224, 224, 64, 7, 7, 2, 3),
    (32, 512, 7, 7, 512, 3, 3, 1, 1),
]


RESNET_SHAPES = [  # the distinct Conv2D layers of ResNet-50 at batch 64 (bottleneck blocks; stage entry layers have stride 2)
    (64, 64, 56, 56, 64, 1, 1, 1, 0), (64, 64, 56, 56, 64, 3, 3, 1, 1), (64, 64, 56, 56, 256, 1, 1, 1, 0), (64, 256, 56, 56, 64, 1, 1, 1, 0),
    (64, 256, 56, 56, 128, 1, 1, 1, 0), (64, 128, 56, 56, 128, 3, 3, 2, 1), (64, 128, 28, 28, 512, 1, 1, 1, 0), (64, 512, 28, 28, 128, 1, 1, 1, 0),
    (64, 128, 28, 28, 128, 3, 3, 1, 1), (64, 256, 56, 56, 512, 1, 1, 2, 0),
    (64, 512, 28, 28, 256, 1, 1, 1, 0), (64, 256, 28, 28, 256, 3, 3, 2, 1), (64, 256, 14, 14, 1024, 1, 1, 1, 0), (64, 1024, 14, 14, 256, 1, 1, 1, 0),
    (64, 256, 14, 14, 256, 3, 3, 1, 1), (64, 512, 28, 28, 1024, 1, 1, 2, 0),
    (64, 1024, 14, 14, 512, 1, 1, 1, 0), (64, 512, 14, 14, 512, 3, 3, 2, 1), (64, 512, 7, 7, 2048, 1, 1, 1, 0), (64, 2048, 7, 7, 512, 1, 1, 1, 0),
    (64, 512, 7, 7, 512, 3, 3, 1, 1), (64, 1024, 14, 14, 2048, 1, 1, 2, 0),
]


def _timed(L, dev, fn, iters, flush):
    ms_all = []
    for _ in range(iters):
        if flush is not None:
            L.call("fill", dev, flush, flush.size, 0.0)      # 256 MB write: evicts the 126 MB L2
        L.call("timer_start", dev, 2)
        fn()
        L.call("timer_stop", dev, 2)
        ms = ctypes.c_float()
        L.call("timer_elapsed_ms", dev, 2, ctypes.byref(ms))
        ms_all.append(ms.value)
    return float(np.median(ms_all)), float(min(ms_all))


def conv_bench(L, dev, shapes, precision=0, iters=5, only=None, batch_scale=1.0):
    """Yields one record per (shape, pass): CUDA-event time with a flushed L2, TFLOP/s from the real FLOP count."""
    flush = L.empty((64 << 20,), dev)
    rng = np.random.default_rng(0)
    for (n, c, h, w, k, kr, kc, st, pad) in shapes:
        n = max(1, int(round(n * batch_scale)))
        oh = (h + 2 * pad - kr) // st + 1; ow = (w + 2 * pad - kc) // st + 1
        x = L.to_device(rng.standard_normal((n, c, h, w), dtype=np.float32), dev)
        wt = L.to_device(rng.standard_normal((k, c, kr, kc), dtype=np.float32), dev)
        dy = L.to_device(rng.standard_normal((n, k, oh, ow), dtype=np.float32), dev)
        y, gw, dx = L.empty((n, k, oh, ow), dev), L.zeros((k, c, kr, kc), dev), L.zeros((n, c, h, w), dev)
        geo = (n, c, h, w, k, kr, kc, oh, ow, st, st, pad, pad, precision)
        flops = 2.0 * n * k * c * kr * kc * oh * ow
        nbytes = 4.0 * (n * c * h * w + k * c * kr * kc + n * k * oh * ow)     # each tensor once
        passes = {"fwd": lambda: L.call("conv2d_fwd", dev, x, wt, None, y, *geo),
                  "bwd_data": lambda: L.call("conv2d_bwd_data", dev, dy, wt, dx, *geo),
                  "bwd_weight": lambda: L.call("conv2d_bwd_weight", dev, x, dy, gw, None, *geo)}
        for name, fn in passes.items():
            if only and name != only:
                continue
            fn(); fn(); fn(); L.sync(dev)
            med, best = _timed(L, dev, fn, iters, flush)
            yield {"bench": "conv", "pass": name, "shape": {"n": n, "c": c, "h": h, "w": w, "k": k, "kr": kr, "kc": kc, "stride": st, "pad": pad},
                   "precision": {0: "3xTF32", 1: "TF32", 2: "TF32+bf16 cross terms"}[precision], "gflop": flops / 1e9, "ms": med, "ms_best": best,
                   "tflops": flops / (med * 1e-3) / 1e12, "GB/s_each_tensor_once": nbytes / (med * 1e-3) / 1e9}
        L.sync(dev)


def run_conv(args):
    from . import capi
    L = capi.lib(); dev = 0
    L.call("init", dev)
    for o in args.opt:
        k_, v_ = o.split("=")
        L.call("set_option", k_.encode(), int(v_))
    table = RESNET_SHAPES if args.set == "resnet" else CONV_SHAPES
    shapes = table if args.shape < 0 else [table[args.shape]]
    for rec in conv_bench(L, dev, shapes, args.precision, args.iters, args.only, args.batch_scale):
        print(json.dumps(rec), flush=True)


def run_hbm(args):
    from . import capi
    L = capi.lib(); dev = 0
    L.call("init", dev)
    flush = L.empty((64 << 20,), dev)
    rng = np.random.default_rng(0)
    peak = 6541.5
    p = os.path.join(capi.ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        peak = json.load(open(p))["hbm_gbs"]

    for o in args.opt:
        k, v = o.split("=")
        L.call("set_option", k.encode(), int(v))
    only = args.only.split(",") if args.only else None

    def report(name, shape, nbytes, fn):
        if only and not any(name.startswith(o) for o in only):
            return
        fn(); fn(); fn(); L.sync(dev)
        med, best = _timed(L, dev, fn, args.iters, flush)
        gbs = nbytes / (med * 1e-3) / 1e9
        print(json.dumps({"bench": "hbm", "kernel": name, "shape": shape, "bytes": nbytes, "ms": med, "GB/s": gbs, "frac_of_measured_hbm": gbs / peak}), flush=True)

    for (b, z, hw) in [(64, 64, 112), (64, 256, 56), (64, 512, 28), (64, 1024, 14), (64, 2048, 7)]:
        rc = hw * hw; E = b * z * rc
        x = L.to_device(rng.standard_normal((b, z, hw, hw), dtype=np.float32), dev)
        y, opa, d, pd, r = L.empty(x.shape, dev), L.empty(x.shape, dev), L.to_device(rng.standard_normal(x.shape, dtype=np.float32), dev), L.zeros(x.shape, dev), L.empty(x.shape, dev)
        g, bt, gm, gv, mean, var = (L.to_device(np.ones(z, np.float32), dev), L.zeros((z,), dev), L.zeros((z,), dev), L.zeros((z,), dev), L.zeros((z,), dev), L.zeros((z,), dev))
        gg, gb, m1, m2 = L.zeros((z,), dev), L.zeros((z,), dev), L.zeros((z,), dev), L.zeros((z,), dev)
        shape = [b, z, hw, hw]
        report("bn_fwd", shape, 16 * E, lambda: L.call("bn_fwd", dev, b, z, rc, x, y, opa, gm, gv, g, bt, mean, var, 1, 1e-3, 0.99, None))
        report("bn_relu_fwd_fused", shape, 20 * E, lambda: L.call("bn_fwd", dev, b, z, rc, x, y, opa, gm, gv, g, bt, mean, var, 1, 1e-3, 0.99, r))
        report("bn_bwd", shape, 24 * E, lambda: L.call("bn_bwd", dev, b, z, rc, d, opa, pd, gg, gb, g, var, m1, m2))
        report("relu_fwd", shape, 8 * E, lambda: L.call("relu_fwd", dev, x, y, E))
        report("relu_bwd", shape, 16 * E, lambda: L.call("relu_bwd", dev, d, x, pd, E))
        report("axpby_inc", shape, 16 * E, lambda: L.call("axpby", dev, 1.0, x, 1.0, d, pd, 1, E))
        report("fill", shape, 4 * E, lambda: L.call("fill", dev, pd, E, 0.0))
    # max-pool 3x3 s2 p1 on 64x64x112x112 (ResNet stem) and 2x2 s2 on 128x64x32x32 (VGG)
    for (n, c, ih, k, s, pad) in [(64, 64, 112, 3, 2, 1), (128, 64, 32, 2, 2, 0)]:
        oh = (ih + 2 * pad - k) // s + 1
        x = L.to_device(rng.standard_normal((n, c, ih, ih), dtype=np.float32), dev)
        y, ix, iy = L.empty((n, c, oh, oh), dev), L.empty((n, c, oh, oh), dev), L.empty((n, c, oh, oh), dev)
        d, dx = L.to_device(rng.standard_normal((n, c, oh, oh), dtype=np.float32), dev), L.zeros((n, c, ih, ih), dev)
        geo = (n, c, ih, ih, oh, oh, k, k, s, s, pad, pad)
        Ein, Eout = n * c * ih * ih, n * c * oh * oh
        report("maxpool_fwd", [n, c, ih, ih, k, s], 4 * Ein + 12 * Eout, lambda: L.call("maxpool2d_fwd", dev, x, y, ix, iy, *geo))
        report("maxpool_bwd", [n, c, ih, ih, k, s], 12 * Eout + 8 * Ein, lambda: L.call("maxpool2d_bwd", dev, d, ix, iy, dx, *geo))
    # fused SGD over a ResNet-50 sized parameter set (25.6 M floats in one tensor)
    nparam = 25636712
    p_, g_, m_ = L.zeros((nparam,), dev), L.zeros((nparam,), dev), L.zeros((nparam,), dev)
    report("sgd_momentum", [nparam], 20 * nparam, lambda: L.call("sgd_momentum", dev, p_, g_, m_, 0.1, 0.9, nparam))


def allreduce_bench(L, ebd, local, rank, world, max_floats=1 << 28):
    """Parameter averaging over the communicator already set up on `local`: for 1 KB ... 4*max_floats bytes (powers of 4) a
    correctness record (against the fp32 rank-order sum times 1.0f/N, the arithmetic of Net::sync_weights) and a timing
    record per mode.  Every rank must run it; records are meaningful on rank 0."""
    size = 256
    while size <= max_floats:
        rng = np.random.default_rng(1234 + rank)
        host = rng.standard_normal(size, dtype=np.float32)
        buf = L.to_device(host, local)
        p_, m_ = L.zeros((size,), local), L.zeros((size,), local)
        if size <= (1 << 24):
            # every rank can regenerate every rank's buffer
            reps = [np.random.default_rng(1234 + r).standard_normal(size, dtype=np.float32) for r in range(world)]
            want = ebd.average_replicas_host(reps)
            chk = L.to_device(host, local)
            L.call("allreduce_avg", local, chk, size)
            got = chk.numpy()
            err = float(np.max(np.abs(got - want)) / max(float(np.max(np.abs(want))), 1e-30))
            pc, gc, mc = L.to_device(reps[0] * 0 + 1.0, local), L.to_device(host, local), L.zeros((size,), local)
            L.call("avg_grad_sgd", local, pc, gc, mc, 0.1, 0.9, size)
            m_want = (np.float32(0.1) * want).astype(np.float32)
            err2 = float(np.max(np.abs(pc.numpy() - (np.float32(1.0) - m_want))))
            worst = ebd.max_over_ranks(max(err, err2))
            yield {"bench": "allreduce_check", "ranks": world, "floats": size, "max_rel_err_weight_avg": err,
                   "max_abs_err_fused_sgd": err2, "worst_over_ranks": worst, "ok": bool(worst <= 1e-6)}
        for mode, fn in (("weight_avg", lambda: L.call("allreduce_avg", local, buf, size)),
                         ("grad_avg_sgd", lambda: L.call("avg_grad_sgd", local, p_, buf, m_, 0.1, 0.9, size))):
            for _ in range(3):
                fn()
            L.sync(local); ebd.barrier()
            iters = 20 if size <= (1 << 22) else 5
            L.call("timer_start", local, 3)
            for _ in range(iters):
                fn()
            L.call("timer_stop", local, 3)
            ms = ctypes.c_float(); L.call("timer_elapsed_ms", local, 3, ctypes.byref(ms))
            t = ebd.max_over_ranks(ms.value / iters) * 1e-3
            alg = size * 4 / t / 1e9
            yield {"bench": "allreduce", "mode": mode, "ranks": world, "bytes": size * 4, "us": t * 1e6, "algbw_GB/s": alg,
                   "busbw_GB/s": alg * 2 * (world - 1) / world if world > 1 else 0.0,
                   "frac_of_900_GB/s": (alg * 2 * (world - 1) / world / 900.0) if world > 1 else 0.0}
        size *= 4


def run_allreduce(args):
    import torch  # noqa: F401  first: the process-wide libnccl.so.2 must be the one torch was built against
    from . import capi, dist as ebd
    rank, world, local = ebd.rendezvous("gloo")
    L = capi.lib()
    L.call("init", local)
    if world > 1:
        def make_id():
            buf = ctypes.create_string_buffer(128); L.call("comm_unique_id", buf); return buf.raw
        uid = ebd.share_unique_id(make_id)
        L.call("comm_init_rank", local, world, rank, uid)
    for rec in allreduce_bench(L, ebd, local, rank, world):
        if rank == 0:
            print(json.dumps(rec), flush=True)
    if world > 1:
        L.call("comm_destroy", local)


def run_step(args):
    import time
    from . import capi, harness
    L = capi.lib(); L.call("init", 0)
    G = harness.load()
    hw, classes = (224, 1000) if args.net != "cnn" else (28, 10)
    net = harness.NetHarness(G, args.net, device=0, hw=hw, classes=classes, optimizer="sgd_fused", lr=0.1, mu=0.9)
    net.set_params(harness.init_weights(net.param_info(), seed=1234, mode="he_normal"))
    rng = np.random.default_rng(0)
    shape = (args.batch, 3, hw, hw) if args.net != "cnn" else (args.batch, 1, hw, hw)
    x = rng.standard_normal(shape, dtype=np.float32)
    y = np.eye(classes, dtype=np.float32)[rng.integers(0, classes, args.batch)]
    net.train_batch(x, y); net.sync()
    before = L.launches()
    t0 = time.perf_counter()
    loss = net.train_resident(args.steps); net.sync()
    dt = time.perf_counter() - t0
    print(json.dumps({"bench": "step", "net": args.net, "batch": args.batch, "steps": args.steps, "loss_sum": loss,
                      "ms_per_step_wall": 1e3 * dt / max(args.steps, 1), "launches_per_step": (L.launches() - before) / max(args.steps, 1)}), flush=True)
    net.close()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("what", choices=["conv", "hbm", "allreduce", "step"])
    ap.add_argument("--precision", type=int, default=0)
    ap.add_argument("--set", choices=["micro", "resnet"], default="micro", help="conv shape list: the four microbenchmark shapes or ResNet-50's layers")
    ap.add_argument("--batch-scale", type=float, default=1.0)
    ap.add_argument("--iters", type=int, default=5)
    ap.add_argument("--net", default="resnet50", help="step: cnn | vgg16bn | resnet50")
    ap.add_argument("--batch", type=int, default=64)
    ap.add_argument("--steps", type=int, default=1)
    ap.add_argument("--only", default=None, help="hbm: comma-separated kernel-name prefixes (bn, relu, maxpool, ...)")
    ap.add_argument("--opt", action="append", default=[], help="name=value for eddlb200_set_option (repeatable)")
    ap.add_argument("--shape", type=int, default=-1, help="index into the conv shape list (default: all)")
    args = ap.parse_args()
    {"conv": run_conv, "hbm": run_hbm, "allreduce": run_allreduce, "step": run_step}[args.what](args)


if __name__ == "__main__":
    main()
