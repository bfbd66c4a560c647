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
         device->host read of loss and metric (one 8-byte copy) happen every step inside the timed region.
  roofline  Conv2D family (forward + backward-data + backward-weight), timed live with CUDA events around every conv
         call of a second pass over the same resident steps; achieved = algorithmic FLOPs (2*N*K*C*kr*kc*P*Q per pass) /
         summed duration.
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


def profiled_traffic():
    """dram__bytes_read.sum + dram__bytes_write.sum of the captured launch of the dominant kernel, read from the committed
    ncu summary (a capture cannot run inside a timed benchmark)."""
    import re
    name = "conv_fwd_n64_c256_56x56_k3_igemm_tc.md"
    try:
        text = open(os.path.join(ROOT, "profiles", name)).read()
        m = re.search(r"traffic\s+([0-9.]+)\s*MB per launch", text)
        a = re.search(r"algorithmic bytes[^|]*\|\s*([0-9.]+)\s*MB", text)
        if m:
            return float(m.group(1)) * 1e6, ("profiles/%s: one forward launch of the N=64 C=K=256 56x56 3x3 layer under ncu%s"
                                             % (name, "; its algorithmic bytes (input + weights + output once) are %se6" % a.group(1) if a else ""))
    except OSError:
        pass
    return None, "no committed capture found"


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
            "dtype": "f32", "data": "synthetic", "config": {"workload": WORKLOAD, "reference_sample_batch": batch,
                       "note": "img/s measured on steps of %d images and quoted per image: the 64-image step is this rate extrapolated linearly" % batch},
            "cpu_baseline": {k: r[k] for k in ("value", "unit", "cores", "kind", "sample")},
            "e2e": {"value": r["value"], "unit": "img/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}, "gpu_launches": 0}
    print(json.dumps(line), flush=True)


def averaging_check(net, ebd, rank, world):
    """One local step WITHOUT averaging makes the replicas differ (every rank trains on its own shard); then one
    avg_weights_distributed.  On a strided sample of about a million parameters: the result against the arithmetic of
    Net::sync_weights (fp32 sum in rank order, times 1.0f/N), and whether every rank ends with the same bits."""
    import zlib
    import torch
    import torch.distributed as dist
    net.local_step(); net.sync()
    before = net.get_params()
    stride = max(1, before.size // (1 << 20))
    mine = torch.from_numpy(np.ascontiguousarray(before[::stride]))
    parts = [torch.empty_like(mine) for _ in range(world)]
    dist.all_gather(parts, mine)
    want = ebd.average_replicas_host([p.numpy() for p in parts])
    net.avg_weights(1, 1); net.sync()
    after = net.get_params()
    got = after[::stride]
    err = float(np.max(np.abs(got.astype(np.float64) - want.astype(np.float64))) / max(float(np.max(np.abs(want))), 1e-30))
    crc = torch.tensor([zlib.crc32(after.tobytes())], dtype=torch.int64)
    crcs = [torch.empty_like(crc) for _ in range(world)]
    dist.all_gather(crcs, crc)
    spread = float(np.max(np.abs(parts[0].numpy().astype(np.float64) - parts[-1].numpy().astype(np.float64))))
    return {"max_rel_err": ebd.max_over_ranks(err), "tolerance": 1e-6, "sampled_parameters": int(got.size), "of": int(after.size),
            "all_ranks_bit_identical": bool(len({int(c.item()) for c in crcs}) == 1),
            "replicas_differed_before_by": spread,
            "against": "fp32 sum in rank order times 1.0f/N (Net::sync_weights, src/net/net_func.cpp:111-127)"}


def extras(args, L, G, ebd, rank, world, local):
    """The other benchmark configurations, after the headline measurement: the four Conv2D microbenchmark shapes
    (TFLOP/s against the fp32-equivalent tensor peak), VGG-16-BN at batch 128 per GPU, and at N > 1 the averaging sweep
    (bus bandwidth against 900 GB/s).  Rank 0 reports; collective parts run on every rank."""
    from eddl_b200 import harness, microbench
    peaks, peak_src = measured_peaks()
    out = {}
    if rank == 0:
        tc_peak = peaks["bf16_tflops_sustained"] / 6.0
        rows = []
        for rec in microbench.conv_bench(L, local, microbench.CONV_SHAPES, 0, 3):
            s = rec["shape"]
            rows.append({"shape": "N=%d C=%d K=%d %dx%d %dx%d s%d p%d" % (s["n"], s["c"], s["k"], s["h"], s["w"], s["kr"], s["kc"], s["stride"], s["pad"]),
                         "pass": rec["pass"], "ms": round(rec["ms"], 4), "tflops": round(rec["tflops"], 1), "frac": round(rec["tflops"] / tc_peak, 3)})
        out["conv_microbench"] = {"precision": "3xTF32", "peak_tflops": tc_peak, "l2": "flushed by a 256 MB fill before every timed launch",
                                  "rows": rows}
    ebd.barrier()
    # VGG-16-BN, 3x32x32, batch 128 per GPU, SGD momentum 0.9, averaged every step
    vb = 128
    net = harness.NetHarness(G, "vgg16bn", device=local, hw=32, classes=10, optimizer="sgd_fused", lr=0.01, mu=0.9)
    net.set_params(harness.init_weights(net.param_info(), seed=1234, mode="he_normal"))
    if world > 1:
        net.broadcast_params()
    x, y = synth_batch(vb, 32, 10, seed=2000 + rank)
    for i in range(3):
        net.train_batch(x, y)
        if world > 1:
            net.avg_weights(i + 1, 1)
    net.sync(); ebd.barrier()
    steps = 20
    t0 = time.perf_counter()
    for i in range(steps):
        net.train_batch(x, y)
        if world > 1:
            net.avg_weights(i + 1, 1)
    net.sync()
    e2e_s = ebd.max_over_ranks(time.perf_counter() - t0)
    ebd.barrier()
    L.call("timer_start", local, 4)
    net.train_resident(steps)
    L.call("timer_stop", local, 4)
    net.sync()
    ms = ctypes.c_float(); L.call("timer_elapsed_ms", local, 4, ctypes.byref(ms))
    res_s = ebd.max_over_ranks(ms.value / 1e3)
    net.close()
    out["vgg16bn"] = {"workload": "VGG-16-BN 3x32x32, batch 128 per GPU, 10 classes, SGD momentum 0.9, averaged every step",
                      "value_img_per_s": vb * world * steps / res_s, "e2e_img_per_s": vb * world * steps / e2e_s, "steps": steps,
                      "ms_per_step": 1e3 * res_s / steps}
    if world > 1:
        rows, worst = [], 0.0
        for rec in microbench.allreduce_bench(L, ebd, local, rank, world):
            if rec["bench"] == "allreduce":
                rows.append({"mode": rec["mode"], "bytes": rec["bytes"], "us": round(rec["us"], 1), "busbw_GB/s": round(rec["busbw_GB/s"], 1),
                             "frac_of_900": round(rec["frac_of_900_GB/s"], 3)})
            else:
                worst = max(worst, rec["worst_over_ranks"])
        out["averaging_sweep"] = {"ranks": world, "worst_error_up_to_64MB": worst, "tolerance": 1e-6, "rows": rows}
    return out


def run_b200_arm(args):
    # EDDL's host side of train_batch (Tensor::select gathering the batch, the host->device copy of it) runs under OpenMP:
    # give every rank an equal share of the host cores and keep its workers spinning between the short parallel regions.
    # Set before anything loads an OpenMP runtime.
    # torchrun exports OMP_NUM_THREADS=1 as a default of its own, not as the user's choice, so it is overridden; an
    # explicit EDDL_B200_HOST_THREADS wins.
    world_env = max(1, int(os.environ.get("WORLD_SIZE", "1")))
    # With several ranks on one host two cores per rank stay free for the NCCL proxy and the Python threads, and the OpenMP
    # workers sleep between EDDL's short parallel regions instead of spinning: spinning workers starved those threads
    # (two ranks, VGG-16-BN's 4 ms step: 13 300 img/s end to end with spinning workers, 64 300 with sleeping ones; ResNet-50's
    # 27 ms step loses 3 % end to end to the wake-ups).  One rank has the host to itself and keeps its workers spinning.
    share = (os.cpu_count() or 1) // world_env
    host_threads = int(os.environ.get("EDDL_B200_HOST_THREADS", "0")) or max(1, share - 2 if world_env > 1 else share)
    os.environ["OMP_NUM_THREADS"] = str(host_threads)
    os.environ.setdefault("OMP_WAIT_POLICY", "passive" if world_env > 1 else "active")
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
        ebd.check_same_layout([int(np.prod(s)) for _, s in net.param_info()])      # a host-side check: nothing is enqueued if ranks disagree
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
    launches0 = L.launches(local)
    L.call("timer_start", local, 1)
    t0 = time.perf_counter()
    loss_res = net.train_resident(args.steps)
    L.call("timer_stop", local, 1)
    net.sync()
    wall_res = time.perf_counter() - t0
    L.call("timer_elapsed_ms", local, 1, ctypes.byref(ms))
    launches = L.launches(local) - launches0
    tc_calls, fma_calls = ctypes.c_ulonglong(0), ctypes.c_ulonglong(0)
    L.call("conv_path_counts", local, ctypes.byref(tc_calls), ctypes.byref(fma_calls))
    conv_paths = {"tensor_core": int(tc_calls.value), "fp32_fma_fallback": int(fma_calls.value), "since": "process start"}
    res_s = ebd.max_over_ranks(max(ms.value / 1e3, wall_res))
    ebd.barrier()
    # ---- the same steps once more with a CUDA-event pair around every backend call: per-family durations for the roofline
    # and the breakdown (kept out of the region `value` is taken from: the event pairs themselves cost a little)
    L.call("profile_reset", local); L.call("profile_enable", local, 1)
    L.call("timer_start", local, 1)
    net.train_resident(args.steps)
    L.call("timer_stop", local, 1)
    net.sync()
    L.call("timer_elapsed_ms", local, 1, ctypes.byref(ms))
    L.call("profile_enable", local, 0)
    clocks = sampler.stop()

    prof = {}
    names = ["conv_fwd", "conv_bwd_data", "conv_bwd_weight", "bn_fwd", "bn_bwd", "elementwise", "pool", "dense", "optimizer", "collectives"]
    for kind, nm in enumerate(names):
        c, t, w = ctypes.c_ulonglong(), ctypes.c_double(), ctypes.c_double()
        L.call("profile_read", local, kind, ctypes.byref(c), ctypes.byref(t), ctypes.byref(w))
        prof[nm] = (c.value, t.value, w.value)
    L.call("profile_reset", local)

    # ---- outside the timed regions: averaging check (N > 1) and the other benchmark configurations ---------------
    avg_check = averaging_check(net, ebd, rank, world) if world > 1 else None
    net.close()
    extra = None if args.no_extras else extras(args, L, G, ebd, rank, world, local)
    if rank != 0:
        return
    peaks, peak_src = measured_peaks()
    traffic, traffic_from = profiled_traffic()
    conv_calls = sum(prof[k][0] for k in names[:3]); conv_ms = sum(prof[k][1] for k in names[:3]); conv_fl = sum(prof[k][2] for k in names[:3])
    # fp32-equivalent tensor-core peak: TF32 MMA runs at half the bf16 rate and a 3xTF32 product costs three MMAs
    tc_peak = peaks["bf16_tflops_sustained"] / 2.0 / 3.0
    achieved = conv_fl / (conv_ms * 1e-3) / 1e12 if conv_ms > 0 else 0.0
    roofline = {"bound": "tensor", "kernel": "Conv2D implicit GEMM (forward + backward-data + backward-weight)",
                "achieved": achieved, "peak": tc_peak, "unit": "TFLOP/s", "frac": achieved / tc_peak if tc_peak else None,
                "peak_source": "%s bf16_tflops_sustained / 2 (TF32 rate) / 3 (3xTF32 split)" % peak_src,
                "launches": conv_calls, "avg_launch_ms": conv_ms / conv_calls if conv_calls else None,
                "flops_per_step": conv_fl / args.steps,
                "traffic": traffic, "traffic_from": traffic_from,
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
                       "conv_precision": "fp32-equivalent (mode 0)", "host_threads_per_rank": host_threads},
            "clocks": clocks,
            "e2e": {"value": imgs / e2e_s, "unit": "img/s", "h2d_bytes_per_step": int(x.nbytes + y.nbytes), "d2h_bytes_per_step": 8,
                    "ms_per_step": 1e3 * e2e_s / args.steps},
            "gpu_launches": int(launches), "conv_calls": conv_paths, "roofline": roofline, "hbm_kernels": hbm,
            "breakdown_ms_per_step": {k: round(v[1] / args.steps, 3) for k, v in prof.items()},
            "profiled_ms_per_step": round(ms.value / args.steps, 3),
            "loss": {"after_warmup": loss0 if args.warmup else None, "e2e_last": loss_e2e, "resident_last_sum": loss_res}}
    if cpu is not None:
        line["cpu_baseline"] = {k: cpu[k] for k in ("value", "unit", "cores", "kind", "sample")}
    if avg_check is not None:
        line["avg_check"] = avg_check
    if extra:
        line["extra"] = extra
    print(json.dumps(line), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--batch", type=int, default=64)
    ap.add_argument("--hw", type=int, default=224)
    ap.add_argument("--classes", type=int, default=1000)
    ap.add_argument("--optimizer", default="sgd_fused", choices=["sgd", "sgd_fused", "adam", "adam_fused"])
    ap.add_argument("--no-extras", action="store_true", help="skip the other configurations (conv shapes, VGG-16-BN, averaging sweep)")
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
