#!/usr/bin/env python
"""ResNet-50 fp32 training throughput (img/s) of EDDL nets on the eddl_b200 backend.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl b200|reference]

N = 1: one process.  N > 1: launched by torchrun, one process per GPU (RANK / LOCAL_RANK / WORLD_SIZE),
weak scaling (64 images per GPU), parameters averaged across ranks after every step over NCCL.

A "step" is one eddl::train_batch-equivalent pass (zero deltas/grads, forward, loss+metric, backward, SGD-momentum
update, weight averaging) of ResNet-50 [3,4,6,3] on a 64x3x224x224 ~N(0,1) batch with uniform labels over 1000 classes,
He-normal weights injected from a seeded generator, SGD lr 0.1 momentum 0.9.
  value  whole-job img/s with the batch resident in HBM (the body of EDDL's train_batch_t on the replica).
  e2e    the same through eddl::train_batch on HOST buffers: the host->device copy of inputs and targets and the
         device->host read of loss and metric happen every step inside the timed region.
  roofline  Conv2D family (forward + backward-data + backward-weight), timed live with CUDA events around every conv
         call of the timed region; achieved = algorithmic FLOPs (2*N*K*C*kr*kc*P*Q per pass) / summed duration.
  cpu_baseline  the reference's own CS_CPU path (oracle/_ref: EDDL's sources compiled in place, Eigen replaced by a
         stand-in GEMM) on a bounded sample of the same workload.
The activations of one step (about 11 GB at batch 64) exceed the 126 MB L2 many times over, so no explicit L2 flush is
needed between timed iterations.
"""
import argparse
import ctypes
import json
import os
import subprocess
import sys
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

WORKLOAD = ("ResNet-50 [3,4,6,3] fp32 training step, batch 64 per GPU, input 3x224x224 ~N(0,1), 1000 classes, "
            "He-normal init (seeded, injected), SGD lr 0.1 momentum 0.9 (weight_decay is never read by EDDL's SGD), "
            "weights averaged across GPUs every step")
METRIC = "resnet50_train_img_per_s"


def measured_peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        d = json.load(open(p))
        return d, "measured"
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}, "fallback"


class ClockSampler:
    FIELDS = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.proc, self.index = None, index

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "--query-gpu=" + self.FIELDS, "--format=csv,noheader,nounits", "-lms", "200",
                                          "-i", str(self.index)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.proc = None

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            out, _ = self.proc.communicate(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill(); out, _ = self.proc.communicate()
        sm, smax, reasons = [], [], set()
        for line in out.splitlines():
            f = [x.strip() for x in line.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1])); smax.append(float(f[2]))
            except ValueError:
                continue
            for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), f[5:9]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": float(np.median(sm)) if sm else None, "sm_max_mhz": max(smax) if smax else None,
                "reasons": sorted(reasons), "samples": len(sm)}


def synth_batch(batch, hw, classes, seed):
    rng = np.random.default_rng(seed)
    x = rng.standard_normal((batch, 3, hw, hw), dtype=np.float32)
    y = np.zeros((batch, classes), np.float32)
    y[np.arange(batch), rng.integers(0, classes, batch)] = 1.0
    return x, y


def cpu_reference_run(steps, warmup, hw, classes, batch):
    """Times the reference's own CS_CPU path (all host threads) on `batch` images per step."""
    from oracle import ref
    from eddl_b200 import harness
    if not ref.available():
        return None
    cores = os.cpu_count() or 1
    ref.set_threads(cores)
    net = harness.NetHarness(ref.lib(), "resnet50", device=-1, hw=hw, classes=classes, threads=cores, optimizer="sgd", lr=0.1, mu=0.9)
    net.set_params(harness.init_weights(net.param_info(), seed=1234, mode="he_normal"))
    x, y = synth_batch(batch, hw, classes, seed=1)
    for _ in range(warmup):
        net.train_batch(x, y)
    t0 = time.perf_counter()
    for _ in range(steps):
        net.train_batch(x, y)
    dt = time.perf_counter() - t0
    net.close()
    return {"value": batch * steps / dt, "unit": "img/s", "cores": cores, "kind": "reference",
            "sample": "%d steps of batch %d (of the 64-image step) through eddl::train_batch on CS_CPU(%d); EDDL sources compiled "
                      "in place, Eigen 3.4.0 replaced by a stand-in blocked OpenMP SGEMM" % (steps, batch, cores),
            "ms_per_step": 1e3 * dt / steps}


def run_reference_arm(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    batch = 4
    r = cpu_reference_run(args.steps, args.warmup, args.hw, args.classes, batch)
    if r is None:
        print(json.dumps({"impl": "reference", "unavailable": "oracle/_ref (the reference's CPU build) is not present"}))
        return
    line = {"impl": "reference", "metric": METRIC, "value": r["value"], "unit": "img/s", "n_gpus": args.gpus, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": r["ms_per_step"], "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "f32", "data": "synthetic", "config": {"workload": WORKLOAD, "reference_sample_batch": batch},
            "cpu_baseline": {k: r[k] for k in ("value", "unit", "cores", "kind", "sample")},
            "e2e": {"value": r["value"], "unit": "img/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}, "gpu_launches": 0}
    print(json.dumps(line), flush=True)


def run_b200_arm(args):
    # EDDL's host side of train_batch (Tensor::select gathering the batch, the host->device copy of it) runs under OpenMP:
    # give every rank an equal share of the host cores and keep its workers spinning between the short parallel regions.
    # Set before anything loads an OpenMP runtime; an explicit setting in the environment wins.
    os.environ.setdefault("OMP_NUM_THREADS", str(max(1, (os.cpu_count() or 1) // max(1, int(os.environ.get("WORLD_SIZE", "1"))))))
    os.environ.setdefault("OMP_WAIT_POLICY", "active")
    if args.gpus > 1:
        import torch  # noqa: F401  (first, so that the process-wide libnccl.so.2 is the one torch was built against)
    from eddl_b200 import capi, harness, dist as ebd
    rank, world, local = ebd.rendezvous("gloo")
    if world != args.gpus:
        raise SystemExit("--gpus %d but WORLD_SIZE=%d (launch N>1 with torchrun)" % (args.gpus, world))
    L = capi.lib()
    if L.device_count() <= local:
        raise SystemExit("no CUDA device %d: the B200 backend has no CPU fallback" % local)
    G = harness.load()
    L.call("init", local)
    if world > 1:
        def make_id():
            buf = ctypes.create_string_buffer(128)
            L.call("comm_unique_id", buf)
            return buf.raw
        uid = ebd.share_unique_id(make_id)
        if G.ebh_init_distributed(rank, world, local, uid) != 0:
            raise SystemExit(G.ebh_last_error().decode())
    batch = args.batch
    net = harness.NetHarness(G, "resnet50", device=local, hw=args.hw, classes=args.classes, optimizer=args.optimizer, lr=0.1, mu=0.9)
    net.set_params(harness.init_weights(net.param_info(), seed=1234, mode="he_normal"))
    if world > 1:
        net.broadcast_params()
    # this rank's shard of the global batch, in pinned host memory
    start, end = ebd.shard_rows(batch * world, world, rank)
    xg, yg = synth_batch(end - start, args.hw, args.classes, seed=1000 + rank)
    px, py = ctypes.c_void_p(), ctypes.c_void_p()
    L.call("host_alloc", xg.nbytes, ctypes.byref(px)); L.call("host_alloc", yg.nbytes, ctypes.byref(py))
    x = np.frombuffer((ctypes.c_char * xg.nbytes).from_address(px.value), dtype=np.float32).reshape(xg.shape); x[...] = xg
    y = np.frombuffer((ctypes.c_char * yg.nbytes).from_address(py.value), dtype=np.float32).reshape(yg.shape); y[...] = yg

    def e2e_step(i):
        loss, _ = net.train_batch(x, y, nocopy=True)
        if world > 1:
            net.avg_weights(i + 1, 1)
        return loss

    sampler = ClockSampler(local); sampler.start()      # samples SM clocks / throttle reasons across both timed regions
    for i in range(args.warmup):
        loss0 = e2e_step(i)
    net.sync(); ebd.barrier()

    # ---- e2e: host buffers in, loss/metric out, every step --------------------------------------------------
    L.call("timer_start", local, 0)
    t0 = time.perf_counter()
    for i in range(args.steps):
        loss_e2e = e2e_step(i)
    L.call("timer_stop", local, 0)
    net.sync()
    wall_e2e = time.perf_counter() - t0
    ms = ctypes.c_float(); L.call("timer_elapsed_ms", local, 0, ctypes.byref(ms))
    e2e_s = ebd.max_over_ranks(max(ms.value / 1e3, wall_e2e))
    ebd.barrier()

    # ---- value: batch resident in HBM -------------------------------------------------------------------------
    net.train_resident(1)
    net.sync(); ebd.barrier()
    L.call("profile_reset", local); L.call("profile_enable", local, 1)
    launches0 = L.launches(local)
    L.call("timer_start", local, 1)
    t0 = time.perf_counter()
    loss_res = net.train_resident(args.steps)
    L.call("timer_stop", local, 1)
    net.sync()
    wall_res = time.perf_counter() - t0
    L.call("timer_elapsed_ms", local, 1, ctypes.byref(ms))
    launches = L.launches(local) - launches0
    L.call("profile_enable", local, 0)
    clocks = sampler.stop()
    res_s = ebd.max_over_ranks(max(ms.value / 1e3, wall_res))

    prof = {}
    names = ["conv_fwd", "conv_bwd_data", "conv_bwd_weight", "bn_fwd", "bn_bwd", "elementwise", "pool", "dense", "optimizer", "collectives"]
    for kind, nm in enumerate(names):
        c, t, w = ctypes.c_ulonglong(), ctypes.c_double(), ctypes.c_double()
        L.call("profile_read", local, kind, ctypes.byref(c), ctypes.byref(t), ctypes.byref(w))
        prof[nm] = (c.value, t.value, w.value)
    L.call("profile_reset", local)

    if rank != 0:
        net.close()
        return
    peaks, peak_src = measured_peaks()
    conv_calls = sum(prof[k][0] for k in names[:3]); conv_ms = sum(prof[k][1] for k in names[:3]); conv_fl = sum(prof[k][2] for k in names[:3])
    # fp32-equivalent tensor-core peak: TF32 MMA runs at half the bf16 rate and a 3xTF32 product costs three MMAs
    tc_peak = peaks["bf16_tflops_sustained"] / 2.0 / 3.0
    achieved = conv_fl / (conv_ms * 1e-3) / 1e12 if conv_ms > 0 else 0.0
    roofline = {"bound": "tensor", "kernel": "Conv2D implicit GEMM (forward + backward-data + backward-weight)",
                "achieved": achieved, "peak": tc_peak, "unit": "TFLOP/s", "frac": achieved / tc_peak if tc_peak else None,
                "peak_source": "%s bf16_tflops_sustained / 2 (TF32 rate) / 3 (3xTF32 split)" % peak_src,
                "launches": conv_calls, "avg_launch_ms": conv_ms / conv_calls if conv_calls else None,
                "flops_per_step": conv_fl / args.steps,
                # dram__bytes_read.sum + dram__bytes_write.sum of one captured launch (profiles/conv_fwd_n64_c256_56x56_k3_igemm_tc.md)
                "traffic": 599.1e6,
                "traffic_of": "one forward launch of the N=64 C=K=256 56x56 3x3 layer under ncu; its algorithmic bytes "
                              "(input + weights + output once) are 413.4e6",
                "share_of_step": conv_ms / (ms.value if ms.value else 1.0)}
    hbm = {}
    for nm in ("bn_fwd", "bn_bwd", "elementwise", "pool", "optimizer"):
        c, t, w = prof[nm]
        if t > 0:
            hbm[nm] = {"GB/s": w / (t * 1e-3) / 1e9, "frac_of_%s_hbm" % peak_src: w / (t * 1e-3) / 1e9 / peaks["hbm_gbs"], "calls": c,
                       "share_of_step": t / (ms.value if ms.value else 1.0)}
    cpu = None
    if world == 1 and not args.no_cpu_baseline:
        cpu = cpu_reference_run(2, 1, args.hw, args.classes, 4)
    imgs = batch * world * args.steps
    line = {"metric": METRIC, "value": imgs / res_s, "unit": "img/s", "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": 1e3 * res_s / args.steps, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32",
            "data": "synthetic",
            "config": {"workload": WORKLOAD, "global_batch": batch * world, "optimizer": args.optimizer,
                       "l2": "per-step working set (about 11 GB of activations) far exceeds the 126 MB L2; no explicit flush",
                       "conv_precision": "fp32-equivalent (mode 0)", "host_threads_per_rank": int(os.environ.get("OMP_NUM_THREADS", "0"))},
            "clocks": clocks,
            "e2e": {"value": imgs / e2e_s, "unit": "img/s", "h2d_bytes_per_step": int(x.nbytes + y.nbytes), "d2h_bytes_per_step": 16,
                    "ms_per_step": 1e3 * e2e_s / args.steps},
            "gpu_launches": int(launches), "roofline": roofline, "hbm_kernels": hbm,
            "breakdown_ms_per_step": {k: round(v[1] / args.steps, 3) for k, v in prof.items()},
            "loss": {"after_warmup": loss0 if args.warmup else None, "e2e_last": loss_e2e, "resident_last_sum": loss_res}}
    if cpu is not None:
        line["cpu_baseline"] = {k: cpu[k] for k in ("value", "unit", "cores", "kind", "sample")}
    print(json.dumps(line), flush=True)
    net.close()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--batch", type=int, default=64)
    ap.add_argument("--hw", type=int, default=224)
    ap.add_argument("--classes", type=int, default=1000)
    ap.add_argument("--optimizer", default="sgd_fused", choices=["sgd", "sgd_fused"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    args = ap.parse_args()
    # EDDL's host code prints progress text on stdout; keep stdout for the one JSON line
    sys.stdout.flush()
    real_stdout = os.dup(1)
    os.dup2(2, 1)
    sys.stdout = os.fdopen(real_stdout, "w")
    if args.impl == "reference":
        run_reference_arm(args)
    else:
        run_b200_arm(args)


if __name__ == "__main__":
    main()
